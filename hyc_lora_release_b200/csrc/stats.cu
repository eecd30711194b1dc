// Calibration-time statistics: per-channel min/max scale (and zero point), channel L2
// norms and the top-k channel selection.  These run only during the first few training
// iterations; they are written for exactness first (bit-identical to the CPU statement).
#include "hyc_common.cuh"

namespace hyc {

constexpr int kStatCols = 64;     // columns per block (8 vectors of 8)
constexpr int kStatRowLanes = 32; // row lanes per block

__device__ __forceinline__ float bf16_round(float v) { return bf16bits_to_f32(f32_to_bf16bits_rn(v)); }

// One block owns 64 columns and walks all M rows.
__global__ void __launch_bounds__(256)
colstats_kernel(const __nv_bfloat16* __restrict__ x0, int M, int N, int64_t ldx, int q_bit,
                const int64_t* __restrict__ oidx, int k,
                __nv_bfloat16* __restrict__ scale_out, int8_t* __restrict__ zp_out) {
  const int cv = threadIdx.x & 7, rl = threadIdx.x >> 3;
  const int c = blockIdx.x * kStatCols + cv * 8;
  __shared__ float s_mx[kStatRowLanes][kStatCols + 1];
  __shared__ float s_mn[kStatRowLanes][kStatCols + 1];
  float mx[8], mn[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) { mx[e] = -INFINITY; mn[e] = INFINITY; }
  if (c < N) {
    for (int m = rl; m < M; m += kStatRowLanes) {
      uint4 v = *reinterpret_cast<const uint4*>(x0 + (int64_t)m * ldx + c);
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        float f = (e & 1) ? bf16hi_to_f32(w[e >> 1]) : bf16lo_to_f32(w[e >> 1]);
        mx[e] = fmaxf(mx[e], f);
        mn[e] = fminf(mn[e], f);
      }
    }
  }
#pragma unroll
  for (int e = 0; e < 8; ++e) { s_mx[rl][cv * 8 + e] = mx[e]; s_mn[rl][cv * 8 + e] = mn[e]; }
  __syncthreads();
  if (threadIdx.x < kStatCols) {
    const int col = blockIdx.x * kStatCols + threadIdx.x;
    if (col < N) {
      float a = -INFINITY, b = INFINITY;
      for (int r = 0; r < kStatRowLanes; ++r) { a = fmaxf(a, s_mx[r][threadIdx.x]); b = fminf(b, s_mn[r][threadIdx.x]); }
      bool is_out = false;
      for (int j = 0; j < k; ++j) is_out |= (oidx[j] == col);
      if (is_out) { a = 0.f; b = 0.f; }
      const float levels = (float)((1 << q_bit) - 1);
      // every step of the reference is a bf16 tensor op: (max - min) -> bf16, / levels -> bf16
      float d = bf16_round(a - b);
      float sc = bf16_round(__fdiv_rn(d, levels));
      if (zp_out) {
        // zero point from the unguarded scale: -round_half_even(bf16(min / scale)) - 2^(q-1), as int8
        float zq = bf16_round(__fdiv_rn(b, sc));
        float zz = bf16_round(-rintf(zq) - (float)(1 << (q_bit - 1)));
        // the reference casts the bf16 value to int8, which wraps when a column's minimum is positive
        zz = fminf(fmaxf(zz, -2.0e9f), 2.0e9f);
        zp_out[col] = (int8_t)(int)zz;
      }
      if (oidx != nullptr && sc == 0.f) sc = bf16_round(0.f + 1e-3f);
      scale_out[col] = __ushort_as_bfloat16(f32_to_bf16bits_rn(sc));
    }
  }
}

// Sum of squares in fp64 (exact for bf16 inputs), sqrt in fp64, then fp32, then bf16.
__global__ void __launch_bounds__(256)
channel_norm_kernel(const __nv_bfloat16* __restrict__ x0, int M, int N, int64_t ldx,
                    __nv_bfloat16* __restrict__ norm_out) {
  const int cv = threadIdx.x & 7, rl = threadIdx.x >> 3;
  const int c = blockIdx.x * kStatCols + cv * 8;
  __shared__ double s_acc[kStatRowLanes][kStatCols + 1];
  double acc[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) acc[e] = 0.0;
  if (c < N) {
    for (int m = rl; m < M; m += kStatRowLanes) {
      uint4 v = *reinterpret_cast<const uint4*>(x0 + (int64_t)m * ldx + c);
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        float f = (e & 1) ? bf16hi_to_f32(w[e >> 1]) : bf16lo_to_f32(w[e >> 1]);
        acc[e] += (double)f * (double)f;
      }
    }
  }
#pragma unroll
  for (int e = 0; e < 8; ++e) s_acc[rl][cv * 8 + e] = acc[e];
  __syncthreads();
  if (threadIdx.x < kStatCols) {
    const int col = blockIdx.x * kStatCols + threadIdx.x;
    if (col < N) {
      double a = 0.0;
      for (int r = 0; r < kStatRowLanes; ++r) a += s_acc[r][threadIdx.x];
      norm_out[col] = __ushort_as_bfloat16(f32_to_bf16bits_rn((float)sqrt(a)));
    }
  }
}

// Single-block bitonic sort of (norm bits << 16 | (0xffff - column)) in descending order:
// larger norm first, equal norms by ascending column.  Norms are non-negative, so the bf16
// bit pattern orders like the value.
__global__ void __launch_bounds__(1024)
channel_topk_kernel(const __nv_bfloat16* __restrict__ norm, int N, int n_pow2, int k,
                    int64_t* __restrict__ idx_out) {
  extern __shared__ uint32_t s_key[];
  for (int i = threadIdx.x; i < n_pow2; i += blockDim.x) {
    uint32_t key = 0u;
    if (i < N) key = ((uint32_t)__bfloat16_as_ushort(norm[i]) << 16) | (uint32_t)(0xffff - i);
    s_key[i] = key;
  }
  __syncthreads();
  for (int size = 2; size <= n_pow2; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      for (int i = threadIdx.x; i < n_pow2 / 2; i += blockDim.x) {
        int lo = 2 * i - (i & (stride - 1));
        int hi = lo + stride;
        bool desc = ((lo & size) == 0);
        uint32_t a = s_key[lo], b = s_key[hi];
        if ((a < b) == desc) { s_key[lo] = b; s_key[hi] = a; }
      }
      __syncthreads();
    }
  }
  for (int i = threadIdx.x; i < k; i += blockDim.x) idx_out[i] = (int64_t)(0xffff - (s_key[i] & 0xffffu));
}

}  // namespace hyc

using namespace hyc;

extern "C" HYC_API int hyc_colstats_scale(const void* x0, int M, int N, int64_t ldx, int q_bit,
                                  const int64_t* outlier_idx, int k,
                                  void* scale_out, int8_t* zp_out, void* stream) {
  if (!x0 || !scale_out) return HYC_ERR_NULL;
  if (q_bit != 2 && q_bit != 4 && q_bit != 8) return HYC_ERR_QBIT;
  if (M <= 0 || N <= 0 || N % 8 != 0 || ldx < N || k < 0) return HYC_ERR_SHAPE;
  if (!aligned(x0, 16) || ldx % 8 != 0) return HYC_ERR_ALIGN;
  // a non-null (possibly empty) index list selects the channel-base variant with its zero guard
  colstats_kernel<<<(N + kStatCols - 1) / kStatCols, 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)x0, M, N, ldx, q_bit, outlier_idx, outlier_idx ? k : 0,
      (__nv_bfloat16*)scale_out, zp_out);
  HYC_CHECK_LAUNCH();
  return HYC_OK;
}

extern "C" HYC_API int hyc_channel_norm_topk(const void* x0, int M, int N, int64_t ldx, int k,
                                     void* norm_out, int64_t* idx_out, void* stream) {
  if (!x0 || !norm_out || (k > 0 && !idx_out)) return HYC_ERR_NULL;
  if (M <= 0 || N <= 0 || N % 8 != 0 || ldx < N || k < 0 || k > N || N > 32768) return HYC_ERR_SHAPE;
  if (!aligned(x0, 16) || ldx % 8 != 0) return HYC_ERR_ALIGN;
  cudaStream_t st = (cudaStream_t)stream;
  channel_norm_kernel<<<(N + kStatCols - 1) / kStatCols, 256, 0, st>>>(
      (const __nv_bfloat16*)x0, M, N, ldx, (__nv_bfloat16*)norm_out);
  HYC_CHECK_LAUNCH();
  if (k > 0) {
    int n_pow2 = 2;
    while (n_pow2 < N) n_pow2 <<= 1;
    size_t smem = (size_t)n_pow2 * sizeof(uint32_t);
    static bool attr_set[64] = {false};      // per device
    const int slot = current_device_slot();
    if (smem > 48 * 1024 && (slot < 0 || !attr_set[slot])) {
      if (cudaFuncSetAttribute(channel_topk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 128 * 1024) != cudaSuccess) {
        hyc_set_last_cuda_error((int)cudaGetLastError());
        return HYC_ERR_LAUNCH;
      }
      if (slot >= 0) attr_set[slot] = true;
    }
    channel_topk_kernel<<<1, 1024, smem, st>>>((const __nv_bfloat16*)norm_out, N, n_pow2, k, idx_out);
    HYC_CHECK_LAUNCH();
  }
  return HYC_OK;
}

// RMSNorm forward/backward and softmax backward: the producers and consumers of the
// compressed tensors.  Plain streaming kernels, one row per block (norm) or per warp
// (softmax), the row held in registers between the reduction and the second pass.
#include "hyc_common.cuh"

namespace hyc {

constexpr int kNormThreads = 256;
constexpr int kNormMaxVec = 8;     // 8 x (256 threads x 8 elements) = 16384 columns

__device__ __forceinline__ float block_sum(float v) {
  __shared__ float s_p[kNormThreads / 32];
  __shared__ float s_tot;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if ((threadIdx.x & 31) == 0) s_p[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < kNormThreads / 32; ++i) t += s_p[i];
    s_tot = t;
  }
  __syncthreads();
  float r = s_tot;
  __syncthreads();
  return r;
}

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  f[0] = bf16lo_to_f32(v.x); f[1] = bf16hi_to_f32(v.x); f[2] = bf16lo_to_f32(v.y); f[3] = bf16hi_to_f32(v.y);
  f[4] = bf16lo_to_f32(v.z); f[5] = bf16hi_to_f32(v.z); f[6] = bf16lo_to_f32(v.w); f[7] = bf16hi_to_f32(v.w);
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  return make_uint4(pack_bf16x2_rn(f[0], f[1]), pack_bf16x2_rn(f[2], f[3]), pack_bf16x2_rn(f[4], f[5]), pack_bf16x2_rn(f[6], f[7]));
}

__global__ void __launch_bounds__(kNormThreads)
rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w, float eps,
                   __nv_bfloat16* __restrict__ y, float* __restrict__ rstd, int64_t rows, int N) {
  const int nvec = N / 8;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    uint4 xv[kNormMaxVec];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < kNormMaxVec; ++i) {
      const int v = threadIdx.x + i * kNormThreads;
      if (v < nvec) {
        xv[i] = ld_stream_v4(x + row * N + 8 * v);
        float f[8]; unpack8(xv[i], f);
#pragma unroll
        for (int e = 0; e < 8; ++e) ss = fmaf(f[e], f[e], ss);
      }
    }
    const float var = block_sum(ss) / (float)N;
    const float rs = 1.f / sqrtf(var + eps);
    if (threadIdx.x == 0) rstd[row] = rs;
#pragma unroll
    for (int i = 0; i < kNormMaxVec; ++i) {
      const int v = threadIdx.x + i * kNormThreads;
      if (v < nvec) {
        float f[8], wf[8];
        unpack8(xv[i], f);
        unpack8(*reinterpret_cast<const uint4*>(w + 8 * v), wf);
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] = (f[e] * rs) * wf[e];
        st_stream_v4(y + row * N + 8 * v, pack8(f));
      }
    }
  }
}

__global__ void __launch_bounds__(kNormThreads)
rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                   const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd,
                   __nv_bfloat16* __restrict__ dx, int64_t rows, int N) {
  const int nvec = N / 8;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const float rs = rstd[row];
    uint4 xv[kNormMaxVec], gv[kNormMaxVec];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < kNormMaxVec; ++i) {
      const int v = threadIdx.x + i * kNormThreads;
      if (v < nvec) {
        xv[i] = ld_stream_v4(x + row * N + 8 * v);
        gv[i] = ld_stream_v4(dy + row * N + 8 * v);
        float xf[8], gf[8], wf[8];
        unpack8(xv[i], xf); unpack8(gv[i], gf);
        unpack8(*reinterpret_cast<const uint4*>(w + 8 * v), wf);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float wdy = wf[e] * gf[e];
          s1 = fmaf(xf[e] * rs, wdy, s1);
          s2 += wdy;
        }
      }
    }
    const float c1 = block_sum(s1) / (float)N;
    const float c2 = block_sum(s2) / (float)N;
#pragma unroll
    for (int i = 0; i < kNormMaxVec; ++i) {
      const int v = threadIdx.x + i * kNormThreads;
      if (v < nvec) {
        float xf[8], gf[8], wf[8];
        unpack8(xv[i], xf); unpack8(gv[i], gf);
        unpack8(*reinterpret_cast<const uint4*>(w + 8 * v), wf);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float wdy = wf[e] * gf[e];
          xf[e] = (wdy - ((xf[e] * rs) * c1 + c2)) * rs;
        }
        st_stream_v4(dx + row * N + 8 * v, pack8(xf));
      }
    }
  }
}

constexpr int kSmMaxVec = 16;   // 16 x (32 lanes x 8 elements) = 4096 columns
__global__ void __launch_bounds__(256)
softmax_bwd_kernel(const __nv_bfloat16* __restrict__ y, const __nv_bfloat16* __restrict__ g,
                   __nv_bfloat16* __restrict__ o, int64_t rows, int S) {
  const int lane = threadIdx.x & 31;
  const int nvec = S / 8;
  for (int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5); row < rows; row += (int64_t)gridDim.x * 8) {
    uint4 yv[kSmMaxVec], gv[kSmMaxVec];
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < kSmMaxVec; ++i) {
      const int v = lane + 32 * i;
      if (v < nvec) {
        yv[i] = ld_stream_v4(y + row * S + 8 * v);
        gv[i] = ld_stream_v4(g + row * S + 8 * v);
        float yf[8], gf[8];
        unpack8(yv[i], yf); unpack8(gv[i], gf);
#pragma unroll
        for (int e = 0; e < 8; ++e) acc += bf16bits_to_f32(f32_to_bf16bits_rn(yf[e] * gf[e]));   // y*g is a bf16 product
      }
    }
#pragma unroll
    for (int of = 16; of > 0; of >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, of);
#pragma unroll
    for (int i = 0; i < kSmMaxVec; ++i) {
      const int v = lane + 32 * i;
      if (v < nvec) {
        float yf[8], gf[8];
        unpack8(yv[i], yf); unpack8(gv[i], gf);
#pragma unroll
        for (int e = 0; e < 8; ++e) gf[e] = (gf[e] - acc) * yf[e];
        st_stream_v4(o + row * S + 8 * v, pack8(gf));
      }
    }
  }
}

}  // namespace hyc

using namespace hyc;

extern "C" HYC_API int hyc_rmsnorm_fwd(const void* x, const void* w, float eps, void* y, float* rstd,
                               int64_t rows, int N, void* stream) {
  if (!x || !w || !y || !rstd) return HYC_ERR_NULL;
  if (rows < 0 || N <= 0 || N % 8 != 0 || N > kNormThreads * 8 * kNormMaxVec) return HYC_ERR_SHAPE;
  if (!aligned(x, 16) || !aligned(w, 16) || !aligned(y, 16)) return HYC_ERR_ALIGN;
  if (rows == 0) return HYC_OK;
  int64_t grid = rows < (int64_t)kNumSMs * 8 ? rows : (int64_t)kNumSMs * 8;
  rmsnorm_fwd_kernel<<<(int)grid, kNormThreads, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, eps, (__nv_bfloat16*)y, rstd, rows, N);
  HYC_CHECK_LAUNCH();
  return HYC_OK;
}

extern "C" HYC_API int hyc_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, void* dx,
                               int64_t rows, int N, void* stream) {
  if (!dy || !x || !w || !rstd || !dx) return HYC_ERR_NULL;
  if (rows < 0 || N <= 0 || N % 8 != 0 || N > kNormThreads * 8 * kNormMaxVec) return HYC_ERR_SHAPE;
  if (!aligned(x, 16) || !aligned(w, 16) || !aligned(dy, 16) || !aligned(dx, 16)) return HYC_ERR_ALIGN;
  if (rows == 0) return HYC_OK;
  int64_t grid = rows < (int64_t)kNumSMs * 8 ? rows : (int64_t)kNumSMs * 8;
  rmsnorm_bwd_kernel<<<(int)grid, kNormThreads, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, rstd, (__nv_bfloat16*)dx, rows, N);
  HYC_CHECK_LAUNCH();
  return HYC_OK;
}

extern "C" HYC_API int hyc_softmax_bwd(const void* y, const void* g, void* o, int64_t rows, int S, void* stream) {
  if (!y || !g || !o) return HYC_ERR_NULL;
  if (rows < 0 || S <= 0 || S % 8 != 0 || S > 32 * 8 * kSmMaxVec) return HYC_ERR_SHAPE;
  if (!aligned(y, 16) || !aligned(g, 16) || !aligned(o, 16)) return HYC_ERR_ALIGN;
  if (rows == 0) return HYC_OK;
  int64_t grid = (rows + 7) / 8;
  if (grid > (int64_t)kNumSMs * 8) grid = (int64_t)kNumSMs * 8;
  softmax_bwd_kernel<<<(int)grid, 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)y, (const __nv_bfloat16*)g, (__nv_bfloat16*)o, rows, S);
  HYC_CHECK_LAUNCH();
  return HYC_OK;
}

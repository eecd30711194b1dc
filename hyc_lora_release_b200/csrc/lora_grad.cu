// LoRA-A gradient with the de-quantizer inside the contraction.
//
//   out[r, h] = sum_t gm[t, r] * x_hat[t, h],     x_hat = dequant(q, scale)
//
// The saved activation exists only as packed codes.  Each block owns 128 hidden columns and a
// chunk of tokens; per step it unpacks a 32-token x 128-column tile of codes into a bf16 tile in
// shared memory (one 32-column block of the packed layout per thread), and contracts it with the
// matching 32 x R tile of gm on the tensor cores (m16n8k16, fp32 accumulate; both operands are
// read from shared memory with transposing ldmatrix).  x_hat never goes to HBM: the kernel reads
// T*H*q/8 bytes of codes where the two-step version reads and writes 2*T*H bytes twice.
// Token chunks leave fp32 partials in a workspace; a second tiny kernel sums them in a fixed order.
#include "hyc_common.cuh"

namespace hyc {

constexpr int kGaCols = 128;      // hidden columns per block
constexpr int kGaStep = 32;       // tokens per step
constexpr int kGaChunk = 256;     // tokens per block
constexpr int kGaMaxR = 64;

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem_ptr) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(smem_ptr);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// de-quantize one 32-column block of one row into 32 bf16 (16 packed words), reference rounding
template <int QBIT>
__device__ __forceinline__ void dequant_block32(const uint8_t* __restrict__ src, const uint32_t (&s2)[16], uint32_t (&out)[16]) {
  constexpr int EPP = 8 / QBIT, SLAB = 32 / EPP;
  constexpr uint32_t MASK = (1u << QBIT) - 1u, BM = MASK * 0x01010101u;
  uint32_t w[8];
  if (QBIT == 8) {
    const uint4 a = *reinterpret_cast<const uint4*>(src), b = *reinterpret_cast<const uint4*>(src + 16);
    w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w; w[4] = b.x; w[5] = b.y; w[6] = b.z; w[7] = b.w;
#pragma unroll
    for (int j = 0; j < 16; ++j) {     // columns 2j, 2j+1 = bytes 2j, 2j+1
      const float f0 = (byte_to_magic_float(w[j >> 1], (2 * j) & 3) - 8388736.f) * bf16lo_to_f32(s2[j]);
      const float f1 = (byte_to_magic_float(w[j >> 1], ((2 * j) & 3) + 1) - 8388736.f) * bf16hi_to_f32(s2[j]);
      out[j] = pack_bf16x2_rn(f0, f1);
    }
  } else {
    if (QBIT == 4) {
      const uint4 a = *reinterpret_cast<const uint4*>(src);
      w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w;
    } else {
      const uint2 a = *reinterpret_cast<const uint2*>(src);
      w[0] = a.x; w[1] = a.y;
    }
    constexpr uint32_t C1 = 0x4300u | (uint32_t)(1 << (QBIT - 1));
    const uint32_t c1 = C1 | (C1 << 16);
#pragma unroll
    for (int i = 0; i < EPP; ++i) {          // slab i: columns [i*SLAB, (i+1)*SLAB) = field i of bytes 0..SLAB-1
#pragma unroll
      for (int jj = 0; jj < SLAB / 2; ++jj) {
        const int byte0 = 2 * jj;            // bytes byte0, byte0+1 of the block
        const uint32_t f = (w[byte0 >> 2] >> (QBIT * i)) & BM;
        const uint32_t pr = __byte_perm(f, 0x43434343u, (byte0 & 2) ? 0x4342u : 0x4140u);
        __nv_bfloat162 t = __hsub2(*reinterpret_cast<const __nv_bfloat162*>(&pr), *reinterpret_cast<const __nv_bfloat162*>(&c1));
        const int j = (i * SLAB + byte0) >> 1;   // output pair index (columns 2j, 2j+1)
        t = __hmul2(t, *reinterpret_cast<const __nv_bfloat162*>(&s2[j]));
        out[j] = *reinterpret_cast<const uint32_t*>(&t);
      }
    }
  }
}

template <int QBIT, int RT>   // RT = number of 16-row tiles of the LoRA dimension (R2 = 16 * RT)
__global__ void __launch_bounds__(128)
lora_grad_a_kernel(const uint8_t* __restrict__ q, const __nv_bfloat16* __restrict__ scale,
                   const __nv_bfloat16* __restrict__ gm, int64_t ldg, int T, int H, float* __restrict__ ws) {
  constexpr int R2 = 16 * RT;
  __shared__ __align__(16) __nv_bfloat16 xs[kGaStep][kGaCols + 8];
  __shared__ __align__(16) __nv_bfloat16 gs[kGaStep][R2 + 8];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int h0 = blockIdx.x * kGaCols;
  const int t_begin = blockIdx.y * kGaChunk;
  const int t_end = min(T, t_begin + kGaChunk);
  const int64_t qld = (int64_t)H * QBIT / 8;

  // this thread de-quantizes block `blk` (32 columns) of row `lrow` of every step
  const int lrow = tid >> 2, blk = tid & 3;
  uint32_t s2[16];
  {
    const uint4* sp = reinterpret_cast<const uint4*>(scale + h0 + 32 * blk);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const uint4 v = sp[i]; s2[4 * i] = v.x; s2[4 * i + 1] = v.y; s2[4 * i + 2] = v.z; s2[4 * i + 3] = v.w; }
  }
  float acc[RT][4][4];
#pragma unroll
  for (int m = 0; m < RT; ++m)
#pragma unroll
    for (int n = 0; n < 4; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[m][n][e] = 0.f;

  for (int t0 = t_begin; t0 < t_end; t0 += kGaStep) {
    const int row = t0 + lrow;
    uint32_t xv[16];
    if (row < t_end) {
      dequant_block32<QBIT>(q + row * qld + (int64_t)(h0 + 32 * blk) * QBIT / 8, s2, xv);
    } else {
#pragma unroll
      for (int j = 0; j < 16; ++j) xv[j] = 0u;
    }
    uint4* xdst = reinterpret_cast<uint4*>(&xs[lrow][32 * blk]);
#pragma unroll
    for (int i = 0; i < 4; ++i) xdst[i] = make_uint4(xv[4 * i], xv[4 * i + 1], xv[4 * i + 2], xv[4 * i + 3]);
    // gm tile: 32 rows x R2 columns, 16-byte pieces
    for (int i = tid; i < kGaStep * (R2 / 8); i += 128) {
      const int r = i / (R2 / 8), c = i % (R2 / 8);
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (t0 + r < t_end) v = *reinterpret_cast<const uint4*>(gm + (int64_t)(t0 + r) * ldg + 8 * c);
      *reinterpret_cast<uint4*>(&gs[r][8 * c]) = v;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < kGaStep / 16; ++kk) {
      const int k0 = 16 * kk;
      uint32_t a[RT][4];
#pragma unroll
      for (int m = 0; m < RT; ++m)
        ldmatrix_x4_trans(a[m], &gs[k0 + (lane & 7) + ((lane >> 4) & 1) * 8][16 * m + ((lane >> 3) & 1) * 8]);
#pragma unroll
      for (int np = 0; np < 2; ++np) {     // two 8-column tiles per ldmatrix
        uint32_t b[4];
        ldmatrix_x4_trans(b, &xs[k0 + (lane & 7) + ((lane >> 3) & 1) * 8][32 * warp + 16 * np + ((lane >> 4) & 1) * 8]);
#pragma unroll
        for (int m = 0; m < RT; ++m) {
          mma16816(acc[m][2 * np], a[m], b[0], b[1]);
          mma16816(acc[m][2 * np + 1], a[m], b[2], b[3]);
        }
      }
    }
    __syncthreads();
  }
  // fp32 partials: ws[split][r][h]
  float* wbase = ws + (int64_t)blockIdx.y * R2 * H;
  const int g = lane >> 2, tq = lane & 3;
#pragma unroll
  for (int m = 0; m < RT; ++m)
#pragma unroll
    for (int n = 0; n < 4; ++n) {
      const int h = h0 + 32 * warp + 8 * n + 2 * tq;
      *reinterpret_cast<float2*>(wbase + (int64_t)(16 * m + g) * H + h) = make_float2(acc[m][n][0], acc[m][n][1]);
      *reinterpret_cast<float2*>(wbase + (int64_t)(16 * m + g + 8) * H + h) = make_float2(acc[m][n][2], acc[m][n][3]);
    }
}

__global__ void __launch_bounds__(256)
lora_grad_a_reduce_kernel(const float* __restrict__ ws, int splits, int64_t n, __nv_bfloat16* __restrict__ out) {
  for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < n; i += (int64_t)gridDim.x * 256) {
    float s = 0.f;
    for (int k = 0; k < splits; ++k) s += ws[(int64_t)k * n + i];
    out[i] = __ushort_as_bfloat16(f32_to_bf16bits_rn(s));
  }
}

}  // namespace hyc

using namespace hyc;

extern "C" HYC_API size_t hyc_lora_grad_a_workspace_bytes(int T, int H, int R2) {
  if (T <= 0 || H <= 0 || R2 <= 0) return 0;
  return (size_t)((T + kGaChunk - 1) / kGaChunk) * (size_t)R2 * (size_t)H * sizeof(float);
}

extern "C" HYC_API int hyc_lora_grad_a_dequant(const void* q, const void* scale, const void* gm, int64_t ldg, int R2,
                                               int T, int H, int q_bit, void* out, void* workspace, size_t workspace_bytes,
                                               void* stream) {
  if (!q || !scale || !gm || !out || !workspace) return HYC_ERR_NULL;
  if (q_bit != 2 && q_bit != 4 && q_bit != 8) return HYC_ERR_QBIT;
  if (T <= 0 || H <= 0 || H % kGaCols != 0 || R2 <= 0 || R2 % 16 != 0 || R2 > kGaMaxR || ldg < R2) return HYC_ERR_SHAPE;
  if (!aligned(q, 16) || !aligned(scale, 16) || !aligned(gm, 16) || ldg % 8 != 0 || !aligned(workspace, 16)) return HYC_ERR_ALIGN;
  if (workspace_bytes < hyc_lora_grad_a_workspace_bytes(T, H, R2)) return HYC_ERR_WORKSPACE;
  cudaStream_t st = (cudaStream_t)stream;
  const int splits = (T + kGaChunk - 1) / kGaChunk;
  dim3 grid(H / kGaCols, splits);
#define GA(QB, RT) lora_grad_a_kernel<QB, RT><<<grid, 128, 0, st>>>((const uint8_t*)q, (const __nv_bfloat16*)scale, \
      (const __nv_bfloat16*)gm, ldg, T, H, (float*)workspace)
#define GAQ(QB) do { switch (R2 / 16) { case 1: GA(QB, 1); break; case 2: GA(QB, 2); break; case 3: GA(QB, 3); break; default: GA(QB, 4); } } while (0)
  if (q_bit == 2) GAQ(2); else if (q_bit == 4) GAQ(4); else GAQ(8);
#undef GAQ
#undef GA
  HYC_CHECK_LAUNCH();
  const int64_t n = (int64_t)R2 * H;
  int64_t rb = (n + 255) / 256;
  if (rb > num_sms() * 8) rb = num_sms() * 8;
  lora_grad_a_reduce_kernel<<<(int)rb, 256, 0, st>>>((const float*)workspace, splits, n, (__nv_bfloat16*)out);
  HYC_CHECK_LAUNCH();
  return HYC_OK;
}

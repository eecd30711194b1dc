// Stand-alone fused LoRA + SiLU + Hadamard kernels with the quantizer (forward) and the
// de-quantizer (backward) of the saved gate/up activations folded in.  These are the
// drop-ins for the two element-wise launch wrappers of the reference; the rank-16 LoRA
// term is one m16n8k16 tensor-core instruction per 16x8 output tile, everything else is
// streaming.  A warp owns one 32-column block (the unit of the packed byte layout) and
// walks down the rows in tiles of 16; eight warps of a block sit side by side so that a
// row tile touches 512 contiguous bytes per row.
#include "hyc_common.cuh"

namespace hyc {

__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(0.f), "f"(0.f), "f"(0.f), "f"(0.f));
}

__device__ __forceinline__ float bfr(float v) { return bf16bits_to_f32(f32_to_bf16bits_rn(v)); }
__device__ __forceinline__ float sigmoid_f32(float y) { return 1.f / (1.f + __expf(-y)); }

struct SiluTerms { float y1, sig, y1s, y2, o; };
// rounding points of the reference kernels: every named value is a bf16
__device__ __forceinline__ SiluTerms silu_terms(float x1, float l1, float x2, float l2) {
  SiluTerms r;
  r.y1 = bfr(x1 + bfr(l1));
  r.sig = bfr(sigmoid_f32(r.y1));
  r.y1s = bfr(r.y1 * r.sig);
  r.y2 = bfr(x2 + bfr(l2));
  r.o = bfr(r.y1s * r.y2);
  return r;
}

template <int QBIT>
struct FGeo {
  static constexpr int EPP = 8 / QBIT;
  static constexpr int NT_PER_SLAB = 4 / EPP;   // 8-column tiles per slab
};

template <int QBIT, bool BACKWARD>
__global__ void __launch_bounds__(256)
fused_silu_kernel(const __nv_bfloat16* __restrict__ xa1, const __nv_bfloat16* __restrict__ bt1,
                  const __nv_bfloat16* __restrict__ xa2, const __nv_bfloat16* __restrict__ bt2,
                  const __nv_bfloat16* __restrict__ s1v, const __nv_bfloat16* __restrict__ s2v,
                  const __nv_bfloat16* __restrict__ x1, const __nv_bfloat16* __restrict__ x2,   // forward inputs
                  uint8_t* __restrict__ q1, uint8_t* __restrict__ q2,                           // fwd: out, bwd: in
                  const __nv_bfloat16* __restrict__ go,                                         // backward input
                  __nv_bfloat16* __restrict__ o, __nv_bfloat16* __restrict__ gg, __nv_bfloat16* __restrict__ gu,
                  int64_t rows, int N) {
  using G = FGeo<QBIT>;
  constexpr int EPP = G::EPP, NPS = G::NT_PER_SLAB;
  constexpr uint32_t CM = (1u << QBIT) - 1u;
  constexpr float HALF = (float)(1 << (QBIT - 1));
  const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int cb = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (cb * 32 >= N) return;
  const int cbase = 32 * cb;
  const int64_t qld = (int64_t)N / EPP;

  uint32_t b1f[4][2], b2f[4][2];
  float s1[4][2], s2[4][2], r1[4][2], r2[4][2];
#pragma unroll
  for (int nt = 0; nt < 4; ++nt) {
    const int n = cbase + 8 * nt + g;
    b1f[nt][0] = *reinterpret_cast<const uint32_t*>(bt1 + (int64_t)n * 16 + 2 * t);
    b1f[nt][1] = *reinterpret_cast<const uint32_t*>(bt1 + (int64_t)n * 16 + 2 * t + 8);
    b2f[nt][0] = *reinterpret_cast<const uint32_t*>(bt2 + (int64_t)n * 16 + 2 * t);
    b2f[nt][1] = *reinterpret_cast<const uint32_t*>(bt2 + (int64_t)n * 16 + 2 * t + 8);
    const uint32_t sa = *reinterpret_cast<const uint32_t*>(s1v + cbase + 8 * nt + 2 * t);
    const uint32_t sb = *reinterpret_cast<const uint32_t*>(s2v + cbase + 8 * nt + 2 * t);
    s1[nt][0] = bf16lo_to_f32(sa); s1[nt][1] = bf16hi_to_f32(sa);
    s2[nt][0] = bf16lo_to_f32(sb); s2[nt][1] = bf16hi_to_f32(sb);
    if (!BACKWARD) {
      r1[nt][0] = fastq_scale<QBIT>(__frcp_rn(s1[nt][0])); r1[nt][1] = fastq_scale<QBIT>(__frcp_rn(s1[nt][1]));
      r2[nt][0] = fastq_scale<QBIT>(__frcp_rn(s2[nt][0])); r2[nt][1] = fastq_scale<QBIT>(__frcp_rn(s2[nt][1]));
    }
  }

  const int64_t n_tiles = (rows + 15) / 16;
  for (int64_t rt = blockIdx.y; rt < n_tiles; rt += gridDim.y) {
    const int64_t ra = rt * 16 + g, rb = ra + 8;
    const bool va = ra < rows, vb = rb < rows;
    uint32_t a1[4] = {0u, 0u, 0u, 0u}, a2[4] = {0u, 0u, 0u, 0u};
    if (va) {
      a1[0] = *reinterpret_cast<const uint32_t*>(xa1 + ra * 16 + 2 * t);
      a1[2] = *reinterpret_cast<const uint32_t*>(xa1 + ra * 16 + 2 * t + 8);
      a2[0] = *reinterpret_cast<const uint32_t*>(xa2 + ra * 16 + 2 * t);
      a2[2] = *reinterpret_cast<const uint32_t*>(xa2 + ra * 16 + 2 * t + 8);
    }
    if (vb) {
      a1[1] = *reinterpret_cast<const uint32_t*>(xa1 + rb * 16 + 2 * t);
      a1[3] = *reinterpret_cast<const uint32_t*>(xa1 + rb * 16 + 2 * t + 8);
      a2[1] = *reinterpret_cast<const uint32_t*>(xa2 + rb * 16 + 2 * t);
      a2[3] = *reinterpret_cast<const uint32_t*>(xa2 + rb * 16 + 2 * t + 8);
    }
    // main-branch values of the two rows of this thread: [row half][nt][2]
    float m1[2][4][2], m2[2][4][2], gof[2][4][2];
    if (!BACKWARD) {
      uint32_t w1[2][4], w2[2][4];
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        const int c = cbase + 8 * nt + 2 * t;
        w1[0][nt] = va ? ld_stream_u32(x1 + ra * N + c) : 0u;
        w1[1][nt] = vb ? ld_stream_u32(x1 + rb * N + c) : 0u;
        w2[0][nt] = va ? ld_stream_u32(x2 + ra * N + c) : 0u;
        w2[1][nt] = vb ? ld_stream_u32(x2 + rb * N + c) : 0u;
      }
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
          m1[h][nt][0] = bf16lo_to_f32(w1[h][nt]); m1[h][nt][1] = bf16hi_to_f32(w1[h][nt]);
          m2[h][nt][0] = bf16lo_to_f32(w2[h][nt]); m2[h][nt][1] = bf16hi_to_f32(w2[h][nt]);
        }
      // quantize the main branches and store the packed bytes (two adjacent bytes per slab tile)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int64_t row = h ? rb : ra;
        if (!(h ? vb : va)) continue;
#pragma unroll
        for (int jj = 0; jj < NPS; ++jj) {
          uint32_t p1 = 0u, p2 = 0u;
#pragma unroll
          for (int i = 0; i < EPP; ++i) {
            const int nt = i * NPS + jj;
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              uint32_t c1 = fastq_code_bits<QBIT>(m1[h][nt][e], r1[nt][e]) & CM;
              uint32_t c2 = fastq_code_bits<QBIT>(m2[h][nt][e], r2[nt][e]) & CM;
              p1 |= c1 << (QBIT * i + 8 * e);
              p2 |= c2 << (QBIT * i + 8 * e);
            }
          }
          const int64_t qo = row * qld + (int64_t)cb * (32 / EPP) + 8 * jj + 2 * t;
          *reinterpret_cast<uint16_t*>(q1 + qo) = (uint16_t)p1;
          *reinterpret_cast<uint16_t*>(q2 + qo) = (uint16_t)p2;
        }
      }
    } else {
      // de-quantize the saved main branches: bf16( bf16(code - half) * s )
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int64_t row = h ? rb : ra;
        const bool v = h ? vb : va;
#pragma unroll
        for (int jj = 0; jj < NPS; ++jj) {
          const int64_t qo = row * qld + (int64_t)cb * (32 / EPP) + 8 * jj + 2 * t;
          const uint32_t p1 = v ? (uint32_t)*reinterpret_cast<const uint16_t*>(q1 + qo) : 0u;
          const uint32_t p2 = v ? (uint32_t)*reinterpret_cast<const uint16_t*>(q2 + qo) : 0u;
#pragma unroll
          for (int i = 0; i < EPP; ++i) {
            const int nt = i * NPS + jj;
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const float c1 = (float)((p1 >> (QBIT * i + 8 * e)) & CM) - HALF;
              const float c2 = (float)((p2 >> (QBIT * i + 8 * e)) & CM) - HALF;
              m1[h][nt][e] = bfr(c1 * s1[nt][e]);
              m2[h][nt][e] = bfr(c2 * s2[nt][e]);
            }
          }
        }
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
          const int c = cbase + 8 * nt + 2 * t;
          const uint32_t w = v ? ld_stream_u32(go + row * N + c) : 0u;
          gof[h][nt][0] = bf16lo_to_f32(w); gof[h][nt][1] = bf16hi_to_f32(w);
        }
      }
    }
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      float l1[4], l2[4];
      mma_bf16_16816(l1, a1, b1f[nt][0], b1f[nt][1]);
      mma_bf16_16816(l2, a2, b2f[nt][0], b2f[nt][1]);
      const int c = cbase + 8 * nt + 2 * t;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int64_t row = h ? rb : ra;
        if (!(h ? vb : va)) continue;
        SiluTerms e0 = silu_terms(m1[h][nt][0], l1[2 * h], m2[h][nt][0], l2[2 * h]);
        SiluTerms e1 = silu_terms(m1[h][nt][1], l1[2 * h + 1], m2[h][nt][1], l2[2 * h + 1]);
        st_stream_u32(o + row * N + c, pack_bf16x2_rn(e0.o, e1.o));
        if (BACKWARD) {
          float gg0, gg1, gu0, gu1;
          {
            const float gv = gof[h][nt][0];
            const float gh1 = bfr(gv * e0.y2);
            gu0 = bfr(gv * e0.y1s);
            const float inner = bfr(1.f + bfr(e0.y1 * bfr(1.f - e0.sig)));
            gg0 = bfr(gh1 * bfr(e0.sig * inner));
          }
          {
            const float gv = gof[h][nt][1];
            const float gh1 = bfr(gv * e1.y2);
            gu1 = bfr(gv * e1.y1s);
            const float inner = bfr(1.f + bfr(e1.y1 * bfr(1.f - e1.sig)));
            gg1 = bfr(gh1 * bfr(e1.sig * inner));
          }
          st_stream_u32(gg + row * N + c, pack_bf16x2_rn(gg0, gg1));
          st_stream_u32(gu + row * N + c, pack_bf16x2_rn(gu0, gu1));
        }
      }
    }
  }
}

static inline dim3 fused_grid(int64_t rows, int N) {
  const int cgroups = (N / 32 + 7) / 8;
  const int64_t tiles = (rows + 15) / 16;
  int64_t slots = ((int64_t)kNumSMs * 6 + cgroups - 1) / cgroups;
  if (slots > tiles) slots = tiles;
  if (slots < 1) slots = 1;
  if (slots > 65535) slots = 65535;
  return dim3((unsigned)cgroups, (unsigned)slots, 1);
}

}  // namespace hyc

using namespace hyc;

static int check_fused(int64_t rows, int N, int R, int q_bit) {
  if (q_bit != 2 && q_bit != 4 && q_bit != 8) return HYC_ERR_QBIT;
  if (rows < 0 || N <= 0 || N % 32 != 0) return HYC_ERR_SHAPE;
  if (R != 16) return HYC_ERR_UNSUPPORTED;
  return HYC_OK;
}

extern "C" HYC_API int hyc_fused_lora_silu_hadamard_fwd(const void* xa1, const void* bt1, const void* x1, const void* s1,
                                                const void* xa2, const void* bt2, const void* x2, const void* s2,
                                                void* q1, void* q2, void* o,
                                                int64_t rows, int N, int R, int q_bit, void* stream) {
  if (!xa1 || !bt1 || !x1 || !s1 || !xa2 || !bt2 || !x2 || !s2 || !q1 || !q2 || !o) return HYC_ERR_NULL;
  int rc = check_fused(rows, N, R, q_bit);
  if (rc) return rc;
  const void* ps[] = {xa1, bt1, x1, s1, xa2, bt2, x2, s2, q1, q2, o};
  for (const void* p : ps) if (!aligned(p, 4)) return HYC_ERR_ALIGN;
  if (rows == 0) return HYC_OK;
  dim3 grid = fused_grid(rows, N);
#define FW(QB) fused_silu_kernel<QB, false><<<grid, 256, 0, (cudaStream_t)stream>>>(                         \
      (const __nv_bfloat16*)xa1, (const __nv_bfloat16*)bt1, (const __nv_bfloat16*)xa2, (const __nv_bfloat16*)bt2, \
      (const __nv_bfloat16*)s1, (const __nv_bfloat16*)s2, (const __nv_bfloat16*)x1, (const __nv_bfloat16*)x2,     \
      (uint8_t*)q1, (uint8_t*)q2, nullptr, (__nv_bfloat16*)o, nullptr, nullptr, rows, N)
  if (q_bit == 2) FW(2); else if (q_bit == 4) FW(4); else FW(8);
#undef FW
  HYC_CHECK_LAUNCH();
  return HYC_OK;
}

extern "C" HYC_API int hyc_fused_lora_silu_hadamard_bwd(const void* xa1, const void* bt1, const void* q1, const void* s1,
                                                const void* xa2, const void* bt2, const void* q2, const void* s2,
                                                const void* grad_o, void* o, void* grad_gate, void* grad_up,
                                                int64_t rows, int N, int R, int q_bit, void* stream) {
  if (!xa1 || !bt1 || !q1 || !s1 || !xa2 || !bt2 || !q2 || !s2 || !grad_o || !o || !grad_gate || !grad_up) return HYC_ERR_NULL;
  int rc = check_fused(rows, N, R, q_bit);
  if (rc) return rc;
  const void* ps[] = {xa1, bt1, q1, s1, xa2, bt2, q2, s2, grad_o, o, grad_gate, grad_up};
  for (const void* p : ps) if (!aligned(p, 4)) return HYC_ERR_ALIGN;
  if (rows == 0) return HYC_OK;
  dim3 grid = fused_grid(rows, N);
#define BW(QB) fused_silu_kernel<QB, true><<<grid, 256, 0, (cudaStream_t)stream>>>(                          \
      (const __nv_bfloat16*)xa1, (const __nv_bfloat16*)bt1, (const __nv_bfloat16*)xa2, (const __nv_bfloat16*)bt2, \
      (const __nv_bfloat16*)s1, (const __nv_bfloat16*)s2, nullptr, nullptr,                                       \
      (uint8_t*)q1, (uint8_t*)q2, (const __nv_bfloat16*)grad_o, (__nv_bfloat16*)o, (__nv_bfloat16*)grad_gate,     \
      (__nv_bfloat16*)grad_up, rows, N)
  if (q_bit == 2) BW(2); else if (q_bit == 4) BW(4); else BW(8);
#undef BW
  HYC_CHECK_LAUNCH();
  return HYC_OK;
}

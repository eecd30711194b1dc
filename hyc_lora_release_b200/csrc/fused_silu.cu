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
__device__ __forceinline__ float sigmoid_f32(float y) { return __fdividef(1.f, 1.f + __expf(-y)); }

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

// ---------------------------------------------------------------- wide variant (16-byte aligned tensors)
// Same arithmetic, memory-friendly layout.  A warp owns 64 consecutive columns and walks down the rows in
// tiles of 16.  The rank-16 LoRA terms of a tile come from 16 tensor-core instructions; their fragments
// (two rows x two columns per thread) are rounded to bf16 pairs and turned, through a padded shared-memory
// tile, into the layout everything else uses: a lane holds EIGHT consecutive columns of one row, eight lanes
// cover the 128 contiguous bytes of a row, a warp instruction covers four rows.  Every global access is then
// a 128-bit one, and the element-wise chain runs on packed bf16 pairs: for bf16 operands a packed add or
// multiply (non-contracting form) is exactly the reference's "fp32 operation, round to bf16" step.
typedef __nv_bfloat162 bf2;
__device__ __forceinline__ bf2 as_bf2(uint32_t v) { return *reinterpret_cast<bf2*>(&v); }
__device__ __forceinline__ uint32_t as_u32(bf2 v) { return *reinterpret_cast<uint32_t*>(&v); }
__device__ __forceinline__ uint32_t add2(uint32_t a, uint32_t b) { return as_u32(__hadd2_rn(as_bf2(a), as_bf2(b))); }
__device__ __forceinline__ uint32_t sub2(uint32_t a, uint32_t b) { return as_u32(__hsub2_rn(as_bf2(a), as_bf2(b))); }
__device__ __forceinline__ uint32_t mul2(uint32_t a, uint32_t b) { return as_u32(__hmul2_rn(as_bf2(a), as_bf2(b))); }
constexpr uint32_t kOne2 = 0x3f803f80u;   // (1.0, 1.0)
__device__ __forceinline__ uint32_t sigmoid2(uint32_t y) {
  return pack_bf16x2_rn(sigmoid_f32(bf16lo_to_f32(y)), sigmoid_f32(bf16hi_to_f32(y)));
}

constexpr int kWideLd = 36;      // words per row of the shared LoRA tile: 64 bf16 + padding, conflict-free both ways

#ifndef HYC_FUSED_UNROLL
#define HYC_FUSED_UNROLL 4
#endif
constexpr int kFusedUnroll = HYC_FUSED_UNROLL;   // row passes unrolled together (loads in flight vs registers)
#ifndef HYC_FUSED_MINB
#define HYC_FUSED_MINB 3
#endif
template <int QBIT, bool BACKWARD>
__global__ void __launch_bounds__(256, HYC_FUSED_MINB)
fused_silu_wide_kernel(const __nv_bfloat16* __restrict__ xa1, const __nv_bfloat16* __restrict__ bt1,
                       const __nv_bfloat16* __restrict__ xa2, const __nv_bfloat16* __restrict__ bt2,
                       const __nv_bfloat16* __restrict__ s1v, const __nv_bfloat16* __restrict__ s2v,
                       const __nv_bfloat16* __restrict__ x1, const __nv_bfloat16* __restrict__ x2,   // forward inputs
                       uint8_t* __restrict__ q1, uint8_t* __restrict__ q2,                           // fwd: out, bwd: in
                       const __nv_bfloat16* __restrict__ go,                                         // backward input
                       __nv_bfloat16* __restrict__ o, __nv_bfloat16* __restrict__ gg, __nv_bfloat16* __restrict__ gu,
                       int64_t rows, int N) {
  constexpr int EPP = 8 / QBIT;
  constexpr uint32_t CM = (1u << QBIT) - 1u, BM = CM * 0x01010101u;
  __shared__ __align__(16) uint32_t s_l[8][2][16 * kWideLd];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int cw = blockIdx.x * 8 + warp;          // 64-column group of this warp
  const int c0 = 64 * cw;
  if (c0 >= N) return;
  const int64_t qld = (int64_t)N / EPP;
  uint32_t* sl1 = s_l[warp][0];
  uint32_t* sl2 = s_l[warp][1];

  // element-wise layout: this lane's eight columns
  const int cl = lane & 7, rsub = lane >> 3;     // column octet of the group, row within a group of four
  const int col = c0 + 8 * cl;
  const bool col_ok = col < N;
  const int blk = col >> 5, cg = (col >> 3) & 3; // 32-column block and octet inside it
  uint32_t s1p[4] = {0u, 0u, 0u, 0u}, s2p[4] = {0u, 0u, 0u, 0u};    // scales as packed pairs
  float r1[8], r2[8];                                                 // quantizer constants (forward)
  if (col_ok) {
    const uint4 a = *reinterpret_cast<const uint4*>(s1v + col), b = *reinterpret_cast<const uint4*>(s2v + col);
    s1p[0] = a.x; s1p[1] = a.y; s1p[2] = a.z; s1p[3] = a.w;
    s2p[0] = b.x; s2p[1] = b.y; s2p[2] = b.z; s2p[3] = b.w;
  }
  if (!BACKWARD) {
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float sa = (e & 1) ? bf16hi_to_f32(s1p[e >> 1]) : bf16lo_to_f32(s1p[e >> 1]);
      const float sb = (e & 1) ? bf16hi_to_f32(s2p[e >> 1]) : bf16lo_to_f32(s2p[e >> 1]);
      r1[e] = fastq_scale<QBIT>(__frcp_rn(sa));
      r2[e] = fastq_scale<QBIT>(__frcp_rn(sb));
    }
  }

  const int64_t n_tiles = (rows + 15) / 16;
  for (int64_t rt = blockIdx.y; rt < n_tiles; rt += gridDim.y) {
    // ---- the tile's global loads go out first (four rows per lane), their latency hides behind the LoRA part
    uint4 pa[4], pb[4];     // forward: x1, x2;  backward: (codes of gate, codes of up), grad_out
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int64_t row = rt * 16 + 4 * i + rsub;
      pa[i] = make_uint4(0u, 0u, 0u, 0u); pb[i] = pa[i];
      if (row < rows && col_ok) {
        if (!BACKWARD) {
          pa[i] = ld_stream_v4(x1 + row * N + col);
          pb[i] = ld_stream_v4(x2 + row * N + col);
        } else {
          uint2 a, b;
          if (QBIT == 8) {
            a = ld_stream_v2(q1 + row * qld + col); b = ld_stream_v2(q2 + row * qld + col);
          } else if (QBIT == 4) {
            a = ld_stream_v2(q1 + row * qld + 16 * blk + 8 * (cg & 1)); b = ld_stream_v2(q2 + row * qld + 16 * blk + 8 * (cg & 1));
          } else {
            a = ld_stream_v2(q1 + row * qld + 8 * blk); b = ld_stream_v2(q2 + row * qld + 8 * blk);
          }
          pa[i] = make_uint4(a.x, a.y, b.x, b.y);
          pb[i] = ld_stream_v4(go + row * N + col);
        }
      }
    }
    // ---- LoRA terms of the 16 x 64 tile -> shared memory as bf16 pairs
    {
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
#pragma unroll 2
      for (int nt = 0; nt < 8; ++nt) {
        // B fragments of eight columns (a few KB per warp in total: they stay in L1 across the row tiles)
        const int n = c0 + 8 * nt + g;
        uint32_t b1a = 0u, b1b = 0u, b2a = 0u, b2b = 0u;
        if (n < N) {
          b1a = *reinterpret_cast<const uint32_t*>(bt1 + (int64_t)n * 16 + 2 * t);
          b1b = *reinterpret_cast<const uint32_t*>(bt1 + (int64_t)n * 16 + 2 * t + 8);
          b2a = *reinterpret_cast<const uint32_t*>(bt2 + (int64_t)n * 16 + 2 * t);
          b2b = *reinterpret_cast<const uint32_t*>(bt2 + (int64_t)n * 16 + 2 * t + 8);
        }
        float l1[4], l2[4];
        mma_bf16_16816(l1, a1, b1a, b1b);
        mma_bf16_16816(l2, a2, b2a, b2b);
        // fragment: (row g, columns 8nt + 2t, +1) and (row g + 8, same columns)
        sl1[g * kWideLd + 4 * nt + t] = pack_bf16x2_rn(l1[0], l1[1]);
        sl1[(g + 8) * kWideLd + 4 * nt + t] = pack_bf16x2_rn(l1[2], l1[3]);
        sl2[g * kWideLd + 4 * nt + t] = pack_bf16x2_rn(l2[0], l2[1]);
        sl2[(g + 8) * kWideLd + 4 * nt + t] = pack_bf16x2_rn(l2[2], l2[3]);
      }
    }
    __syncwarp();
    // ---- element-wise part, four rows per pass
#pragma unroll kFusedUnroll
    for (int i = 0; i < 4; ++i) {
      const int lr = 4 * i + rsub;
      const int64_t row = rt * 16 + lr;
      const bool ok = row < rows && col_ok;
      const uint4 l1q = *reinterpret_cast<const uint4*>(sl1 + lr * kWideLd + 4 * cl);
      const uint4 l2q = *reinterpret_cast<const uint4*>(sl2 + lr * kWideLd + 4 * cl);
      const uint32_t l1w[4] = {l1q.x, l1q.y, l1q.z, l1q.w}, l2w[4] = {l2q.x, l2q.y, l2q.z, l2q.w};
      uint32_t x1w[4] = {0u, 0u, 0u, 0u}, x2w[4] = {0u, 0u, 0u, 0u}, gw[4] = {0u, 0u, 0u, 0u};
      if (!BACKWARD) {
        x1w[0] = pa[i].x; x1w[1] = pa[i].y; x1w[2] = pa[i].z; x1w[3] = pa[i].w;
        x2w[0] = pb[i].x; x2w[1] = pb[i].y; x2w[2] = pb[i].z; x2w[3] = pb[i].w;
        // codes of the lane's eight columns, one per byte
        uint32_t k1[2], k2[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint32_t c1[4], c2[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int idx = 4 * h + e;
            const float f1 = (idx & 1) ? bf16hi_to_f32(x1w[idx >> 1]) : bf16lo_to_f32(x1w[idx >> 1]);
            const float f2 = (idx & 1) ? bf16hi_to_f32(x2w[idx >> 1]) : bf16lo_to_f32(x2w[idx >> 1]);
            c1[e] = fastq_code_bits<QBIT>(f1, r1[idx]);
            c2[e] = fastq_code_bits<QBIT>(f2, r2[idx]);
          }
          k1[h] = gather_low_bytes(c1[0], c1[1], c1[2], c1[3]);     // the low byte of a code word is the code
          k2[h] = gather_low_bytes(c2[0], c2[1], c2[2], c2[3]);
        }
        // reference byte layout of a 32-column block: byte j holds columns j, j + 32/EPP, ... at rising bit
        // positions; the block's four lanes (octets 0..3) combine their fields with two butterfly exchanges
        if (QBIT == 8) {
          if (ok) st_stream_v2(q1 + row * qld + col, make_uint2(k1[0], k1[1]));
          if (ok) st_stream_v2(q2 + row * qld + col, make_uint2(k2[0], k2[1]));
        } else if (QBIT == 4) {
          // octets 0, 1: low nibbles of bytes 0..7, 8..15; octets 2, 3: high nibbles of the same bytes
          const int sh = 4 * (cg >> 1);
          uint32_t p1[2] = {k1[0] << sh, k1[1] << sh}, p2[2] = {k2[0] << sh, k2[1] << sh};
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            p1[h] |= __shfl_xor_sync(0xffffffffu, p1[h], 2);
            p2[h] |= __shfl_xor_sync(0xffffffffu, p2[h], 2);
          }
          // both lanes of a pair now hold the same 8 bytes; the lower one writes them
          if (ok && cg < 2) {
            st_stream_v2(q1 + row * qld + 16 * blk + 8 * cg, make_uint2(p1[0], p1[1]));
            st_stream_v2(q2 + row * qld + 16 * blk + 8 * cg, make_uint2(p2[0], p2[1]));
          }
        } else {
          // octet cg supplies bit field cg of bytes 0..7
          const int sh = 2 * cg;
          uint32_t p1[2] = {k1[0] << sh, k1[1] << sh}, p2[2] = {k2[0] << sh, k2[1] << sh};
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            p1[h] |= __shfl_xor_sync(0xffffffffu, p1[h], 1); p1[h] |= __shfl_xor_sync(0xffffffffu, p1[h], 2);
            p2[h] |= __shfl_xor_sync(0xffffffffu, p2[h], 1); p2[h] |= __shfl_xor_sync(0xffffffffu, p2[h], 2);
          }
          if (ok && cg == 0) {
            st_stream_v2(q1 + row * qld + 8 * blk, make_uint2(p1[0], p1[1]));
            st_stream_v2(q2 + row * qld + 8 * blk, make_uint2(p2[0], p2[1]));
          }
        }
      } else {
        // packed codes of the lane's octet -> one code per byte -> bf16 pairs (code - half) * scale
        uint32_t k1[2], k2[2];
        {
          const int sh = QBIT == 8 ? 0 : (QBIT == 4 ? 4 * (cg >> 1) : 2 * cg);
          k1[0] = (pa[i].x >> sh) & BM; k1[1] = (pa[i].y >> sh) & BM;
          k2[0] = (pa[i].z >> sh) & BM; k2[1] = (pa[i].w >> sh) & BM;
          gw[0] = pb[i].x; gw[1] = pb[i].y; gw[2] = pb[i].z; gw[3] = pb[i].w;
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint32_t w1 = k1[j >> 1], w2 = k2[j >> 1];
          if (QBIT == 8) {
            const float a0 = (byte_to_magic_float(w1, (2 * j) & 3) - 8388736.f) * bf16lo_to_f32(s1p[j]);
            const float a1 = (byte_to_magic_float(w1, ((2 * j) & 3) + 1) - 8388736.f) * bf16hi_to_f32(s1p[j]);
            const float b0 = (byte_to_magic_float(w2, (2 * j) & 3) - 8388736.f) * bf16lo_to_f32(s2p[j]);
            const float b1 = (byte_to_magic_float(w2, ((2 * j) & 3) + 1) - 8388736.f) * bf16hi_to_f32(s2p[j]);
            x1w[j] = pack_bf16x2_rn(a0, a1);
            x2w[j] = pack_bf16x2_rn(b0, b1);
          } else {
            constexpr uint32_t C1 = 0x4300u | (uint32_t)(1 << (QBIT - 1));
            const uint32_t sel = (j & 1) ? 0x4342u : 0x4140u;
            x1w[j] = mul2(sub2(__byte_perm(w1, 0x43434343u, sel), C1 | (C1 << 16)), s1p[j]);
            x2w[j] = mul2(sub2(__byte_perm(w2, 0x43434343u, sel), C1 | (C1 << 16)), s2p[j]);
          }
        }
      }
      // ---- the chain on four packed pairs
      uint32_t ov[4], ggv[4], guv[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint32_t y1 = add2(x1w[j], l1w[j]), sig = sigmoid2(y1), y1s = mul2(y1, sig), y2 = add2(x2w[j], l2w[j]);
        ov[j] = mul2(y1s, y2);
        if (BACKWARD) {
          guv[j] = mul2(gw[j], y1s);
          const uint32_t inner = add2(kOne2, mul2(y1, sub2(kOne2, sig)));
          ggv[j] = mul2(mul2(gw[j], y2), mul2(sig, inner));
        }
      }
      if (ok) {
        st_stream_v4(o + row * N + col, make_uint4(ov[0], ov[1], ov[2], ov[3]));
        if (BACKWARD) {
          st_stream_v4(gg + row * N + col, make_uint4(ggv[0], ggv[1], ggv[2], ggv[3]));
          st_stream_v4(gu + row * N + col, make_uint4(guv[0], guv[1], guv[2], guv[3]));
        }
      }
    }
    __syncwarp();    // the LoRA tile is rewritten in the next round
  }
}

// ---------------------------------------------------------------- de-quantize + LoRA re-add
// y = bf16( dequant(q, s) + bf16(xa * bt^T) ): the backward-side reconstruction of a LoRA projection whose
// main branch was saved as codes (the q/k/v projections: `decompression_dequantization` followed by
// `+ x_lora_a @ w_lora_b`, fused_llama_layer_intra_inter_full_fuse.py:416-452).  Same layout as the wide
// kernel above with one branch.
template <int QBIT>
__global__ void __launch_bounds__(256, HYC_FUSED_MINB)
dequant_lora_add_kernel(const __nv_bfloat16* __restrict__ xa, const __nv_bfloat16* __restrict__ bt,
                        const __nv_bfloat16* __restrict__ sv, const uint8_t* __restrict__ q,
                        __nv_bfloat16* __restrict__ y, int64_t rows, int N) {
  constexpr int EPP = 8 / QBIT;
  constexpr uint32_t CM = (1u << QBIT) - 1u, BM = CM * 0x01010101u;
  __shared__ __align__(16) uint32_t s_l[8][16 * kWideLd];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int c0 = 64 * (blockIdx.x * 8 + warp);
  if (c0 >= N) return;
  const int64_t qld = (int64_t)N / EPP;
  uint32_t* sl = s_l[warp];
  const int cl = lane & 7, rsub = lane >> 3;
  const int col = c0 + 8 * cl;
  const bool col_ok = col < N;
  const int blk = col >> 5, cg = (col >> 3) & 3;
  uint32_t sp[4] = {0u, 0u, 0u, 0u};
  if (col_ok) {
    const uint4 a = *reinterpret_cast<const uint4*>(sv + col);
    sp[0] = a.x; sp[1] = a.y; sp[2] = a.z; sp[3] = a.w;
  }
  const int64_t n_tiles = (rows + 15) / 16;
  for (int64_t rt = blockIdx.y; rt < n_tiles; rt += gridDim.y) {
    uint2 pq[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int64_t row = rt * 16 + 4 * i + rsub;
      pq[i] = make_uint2(0u, 0u);
      if (row < rows && col_ok) {
        if (QBIT == 8) pq[i] = ld_stream_v2(q + row * qld + col);
        else if (QBIT == 4) pq[i] = ld_stream_v2(q + row * qld + 16 * blk + 8 * (cg & 1));
        else pq[i] = ld_stream_v2(q + row * qld + 8 * blk);
      }
    }
    {
      const int64_t ra = rt * 16 + g, rb = ra + 8;
      uint32_t a[4] = {0u, 0u, 0u, 0u};
      if (ra < rows) {
        a[0] = *reinterpret_cast<const uint32_t*>(xa + ra * 16 + 2 * t);
        a[2] = *reinterpret_cast<const uint32_t*>(xa + ra * 16 + 2 * t + 8);
      }
      if (rb < rows) {
        a[1] = *reinterpret_cast<const uint32_t*>(xa + rb * 16 + 2 * t);
        a[3] = *reinterpret_cast<const uint32_t*>(xa + rb * 16 + 2 * t + 8);
      }
#pragma unroll 2
      for (int nt = 0; nt < 8; ++nt) {
        const int n = c0 + 8 * nt + g;
        uint32_t ba = 0u, bb = 0u;
        if (n < N) {
          ba = *reinterpret_cast<const uint32_t*>(bt + (int64_t)n * 16 + 2 * t);
          bb = *reinterpret_cast<const uint32_t*>(bt + (int64_t)n * 16 + 2 * t + 8);
        }
        float l[4];
        mma_bf16_16816(l, a, ba, bb);
        sl[g * kWideLd + 4 * nt + t] = pack_bf16x2_rn(l[0], l[1]);
        sl[(g + 8) * kWideLd + 4 * nt + t] = pack_bf16x2_rn(l[2], l[3]);
      }
    }
    __syncwarp();
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int lr = 4 * i + rsub;
      const int64_t row = rt * 16 + lr;
      const uint4 lq = *reinterpret_cast<const uint4*>(sl + lr * kWideLd + 4 * cl);
      const uint32_t lw[4] = {lq.x, lq.y, lq.z, lq.w};
      const int sh = QBIT == 8 ? 0 : (QBIT == 4 ? 4 * (cg >> 1) : 2 * cg);
      const uint32_t k[2] = {(pq[i].x >> sh) & BM, (pq[i].y >> sh) & BM};
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint32_t w = k[j >> 1];
        uint32_t x;
        if (QBIT == 8) {
          const float a0 = (byte_to_magic_float(w, (2 * j) & 3) - 8388736.f) * bf16lo_to_f32(sp[j]);
          const float a1 = (byte_to_magic_float(w, ((2 * j) & 3) + 1) - 8388736.f) * bf16hi_to_f32(sp[j]);
          x = pack_bf16x2_rn(a0, a1);
        } else {
          constexpr uint32_t C1 = 0x4300u | (uint32_t)(1 << (QBIT - 1));
          x = mul2(sub2(__byte_perm(w, 0x43434343u, (j & 1) ? 0x4342u : 0x4140u), C1 | (C1 << 16)), sp[j]);
        }
        o[j] = add2(x, lw[j]);
      }
      if (row < rows && col_ok) st_stream_v4(y + row * N + col, make_uint4(o[0], o[1], o[2], o[3]));
    }
    __syncwarp();
  }
}

// one resident wave: every block walks down the rows with a fixed stride, so a second, partial wave would
// only add a tail
template <typename K>
static inline dim3 fused_wide_grid(K kern, int64_t rows, int N) {
  const int cgroups = ((N + 63) / 64 + 7) / 8;
  const int64_t tiles = (rows + 15) / 16;
  int per_sm = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, 256, 0) != cudaSuccess || per_sm < 1) per_sm = 2;
  int64_t slots = ((int64_t)num_sms() * per_sm) / cgroups;
  if (slots > tiles) slots = tiles;
  if (slots < 1) slots = 1;
  if (slots > 65535) slots = 65535;
  return dim3((unsigned)cgroups, (unsigned)slots, 1);
}

static inline dim3 fused_grid(int64_t rows, int N) {
  const int cgroups = (N / 32 + 7) / 8;
  const int64_t tiles = (rows + 15) / 16;
  int64_t slots = ((int64_t)num_sms() * 6 + cgroups - 1) / cgroups;
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
  bool wide = true;
  for (const void* p : ps) wide = wide && aligned(p, 16);
  dim3 grid = fused_grid(rows, N);
#define FWW(QB) fused_silu_wide_kernel<QB, false><<<fused_wide_grid(fused_silu_wide_kernel<QB, false>, rows, N), 256, 0, (cudaStream_t)stream>>>(                    \
      (const __nv_bfloat16*)xa1, (const __nv_bfloat16*)bt1, (const __nv_bfloat16*)xa2, (const __nv_bfloat16*)bt2, \
      (const __nv_bfloat16*)s1, (const __nv_bfloat16*)s2, (const __nv_bfloat16*)x1, (const __nv_bfloat16*)x2,     \
      (uint8_t*)q1, (uint8_t*)q2, nullptr, (__nv_bfloat16*)o, nullptr, nullptr, rows, N)
  if (wide) {
    if (q_bit == 2) FWW(2); else if (q_bit == 4) FWW(4); else FWW(8);
    HYC_CHECK_LAUNCH();
    return HYC_OK;
  }
#undef FWW
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
  bool wide = true;
  for (const void* p : ps) wide = wide && aligned(p, 16);
  dim3 grid = fused_grid(rows, N);
#define BWW(QB) fused_silu_wide_kernel<QB, true><<<fused_wide_grid(fused_silu_wide_kernel<QB, true>, rows, N), 256, 0, (cudaStream_t)stream>>>(                     \
      (const __nv_bfloat16*)xa1, (const __nv_bfloat16*)bt1, (const __nv_bfloat16*)xa2, (const __nv_bfloat16*)bt2, \
      (const __nv_bfloat16*)s1, (const __nv_bfloat16*)s2, nullptr, nullptr,                                       \
      (uint8_t*)q1, (uint8_t*)q2, (const __nv_bfloat16*)grad_o, (__nv_bfloat16*)o, (__nv_bfloat16*)grad_gate,     \
      (__nv_bfloat16*)grad_up, rows, N)
  if (wide) {
    if (q_bit == 2) BWW(2); else if (q_bit == 4) BWW(4); else BWW(8);
    HYC_CHECK_LAUNCH();
    return HYC_OK;
  }
#undef BWW
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

extern "C" HYC_API int hyc_dequant_lora_add(const void* q, const void* scale, const void* xa, const void* bt,
                                            void* y, int64_t rows, int N, int R, int q_bit, void* stream) {
  if (!q || !scale || !xa || !bt || !y) return HYC_ERR_NULL;
  int rc = check_fused(rows, N, R, q_bit);
  if (rc) return rc;
  if (!aligned(q, 8) || !aligned(scale, 16) || !aligned(xa, 4) || !aligned(bt, 4) || !aligned(y, 16)) return HYC_ERR_ALIGN;
  if (rows == 0) return HYC_OK;
#define DL(QB) dequant_lora_add_kernel<QB><<<fused_wide_grid(dequant_lora_add_kernel<QB>, rows, N), 256, 0, (cudaStream_t)stream>>>( \
      (const __nv_bfloat16*)xa, (const __nv_bfloat16*)bt, (const __nv_bfloat16*)scale, (const uint8_t*)q, (__nv_bfloat16*)y, rows, N)
  if (q_bit == 2) DL(2); else if (q_bit == 4) DL(4); else DL(8);
#undef DL
  HYC_CHECK_LAUNCH();
  return HYC_OK;
}

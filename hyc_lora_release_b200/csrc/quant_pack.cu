// Per-channel quantize-and-pack and unpack-dequantize (HBM-bound streaming kernels).
//
// Thread t of a row produces packed bytes [8t, 8t+8) of that row.  With epp = 8/QBIT codes
// per byte and the reference's interleaved layout, those bytes draw on epp slabs of eight
// consecutive columns each, slab i starting at column 32*b + i*(32/epp) + 8*u where
// (b, u) = (t / tpb, t % tpb), tpb = 4/epp.  So every thread issues epp 128-bit loads and
// one 64-bit store (quantize) or one 64-bit load and epp 128-bit stores (dequantize), all
// sector-aligned.  A thread keeps its columns for all the rows it visits, so the
// per-column scale, reciprocal and zero point live in registers.
#include "hyc_common.cuh"

namespace hyc {

#ifndef HYC_ROW_UNROLL
#define HYC_ROW_UNROLL 2
#endif
#ifndef HYC_Q_MINBLOCKS
#define HYC_Q_MINBLOCKS 4
#endif
constexpr int kThreads = 256;          // upper bound; the launch picks the width that wastes fewest lanes
constexpr int kRowUnroll = HYC_ROW_UNROLL;
#ifndef HYC_DEQ_MINBLOCKS
#define HYC_DEQ_MINBLOCKS 3     // resident blocks per SM the de-quantizer is compiled for (register cap 80)
#endif
#ifndef HYC_DEQ_UNROLL
#define HYC_DEQ_UNROLL 4
#endif
constexpr int kDeqUnroll = HYC_DEQ_UNROLL;          // the de-quantizer loads only 8 bytes per row: keep more rows in flight

template <int QBIT>
struct Geo {
  static constexpr int EPP = 8 / QBIT;           // codes per byte
  static constexpr int SLAB = 32 / EPP;          // columns between the codes of one byte
  static constexpr int TPB = SLAB / 8;           // threads per 32-column block
  static constexpr int COLS_PER_THREAD = 8 * EPP;
  __device__ static __forceinline__ int slab_col(int ct, int i) {
    return 32 * (ct / TPB) + i * SLAB + 8 * (ct % TPB);
  }
};

constexpr int kMaxOwn = 2;        // outlier columns a lane serves from registers
constexpr int kWarpList = 32 * kMaxOwn;   // outlier columns of a warp's span that are dealt out to its lanes

// Outlier columns.  The block builds a map "column of my span -> position j in the outlier list" in
// shared memory.  The outlier columns inside a warp's span (512 columns for 4-bit codes) are then DEALT
// OUT to the lanes of that warp, one or two each, whoever owns the column: however the columns cluster,
// no lane has more than two scalar copies per row, and it issues them right next to its streaming
// loads, so their latency is hidden.  (Letting the owner of a column copy it makes the one thread that
// owns several outliers the slowest of the kernel, and every block waits for the slowest warp.)
// Columns beyond the first two per lane of a warp's span (outlier ratios above 12 % for 4-bit codes) stay
// with their owner, which looks them up in the map again for every row: slow, rare, correct.
struct LaneOutliers {
  int n;                 // entries served by this lane (0..kMaxOwn)
  int col[kMaxOwn];      // absolute column
  int j[kMaxOwn];        // position in the outlier list
  uint32_t extra;        // columns owned by this thread that were not dealt out: bit (8 * slab + element)
  bool warp_has;         // the warp's span holds at least one outlier column (warp-uniform)
};

__device__ __forceinline__ int warp_excl_scan_i(int v, int lane, int& total) {
  int incl = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int t = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += t;
  }
  total = __shfl_sync(0xffffffffu, incl, 31);
  return incl - v;
}

// Deal the outlier columns of the warp's span out to its lanes.  `n_own` = outlier columns among this
// thread's own columns (0 for a thread beyond the last column), listed by for_each_own(f) as
// f(slab, element, absolute column, j).  Every thread of the block must call this.
template <typename ForEachOwn>
__device__ __forceinline__ LaneOutliers deal_outliers(uint32_t* s_list, int col0, bool active, int n_own, ForEachOwn for_each_own) {
  const int lane = threadIdx.x & 31;
  // threads beyond the last column are the trailing lanes of the last warp; they serve nothing
  const int n_act = __popc(__ballot_sync(0xffffffffu, active));
  uint32_t* wl = s_list + (threadIdx.x >> 5) * kWarpList;
  LaneOutliers lo;
  lo.n = 0; lo.extra = 0u;
#pragma unroll
  for (int t = 0; t < kMaxOwn; ++t) { lo.col[t] = 0; lo.j[t] = 0; }
  int total;
  int rank = warp_excl_scan_i(n_own, lane, total);
  lo.warp_has = total > 0;
  if (total == 0) return lo;
  const int cap = kMaxOwn * n_act;
  if (n_own > 0) {
    for_each_own([&](int slab, int e, int col, int j) {
      if (rank < cap) wl[rank] = (uint32_t)(col - col0) | ((uint32_t)j << 16);
      else lo.extra |= 1u << (8 * slab + e);
      ++rank;
    });
  }
  __syncwarp();
  const int n_list = total < cap ? total : cap;
#pragma unroll
  for (int t = 0; t < kMaxOwn; ++t) {
    const int i = lane + n_act * t;
    if (active && i < n_list) {
      const uint32_t w = wl[i];
      lo.col[t] = col0 + (int)(w & 0xffffu);
      lo.j[t] = (int)(w >> 16);
      lo.n = t + 1;
    }
  }
  return lo;
}

__device__ __forceinline__ void build_outlier_map(int16_t* s_map, int span_cols, int col0,
                                                  const int64_t* __restrict__ oidx, int k) {
  for (int i = threadIdx.x; i < span_cols / 2; i += blockDim.x) reinterpret_cast<uint32_t*>(s_map)[i] = 0xffffffffu;
  __syncthreads();
  for (int j = threadIdx.x; j < k; j += blockDim.x) {
    const int64_t c = oidx[j] - col0;
    if (c >= 0 && c < span_cols) s_map[c] = (int16_t)j;
  }
  __syncthreads();
}

// grid: (col_tiles, row_slots).  Row groups of kRowUnroll rows are dealt round-robin to slots.
template <int QBIT, bool HAS_ZP>
__global__ void __launch_bounds__(kThreads, (QBIT == 2 || (QBIT == 4 && HAS_ZP)) ? 2 : HYC_Q_MINBLOCKS)
quant_pack_kernel(const __nv_bfloat16* __restrict__ x, int64_t rows, int N, int64_t ldx,
                  const __nv_bfloat16* __restrict__ scale, const int8_t* __restrict__ zp,
                  const int64_t* __restrict__ oidx, int k,
                  uint8_t* __restrict__ q, __nv_bfloat16* __restrict__ oout) {
  using G = Geo<QBIT>;
  constexpr int EPP = G::EPP;
  const int ct = blockIdx.x * blockDim.x + threadIdx.x;
  const int n_ct = N / G::COLS_PER_THREAD;
  const bool active = ct < n_ct;
  const int64_t qld = (int64_t)N / EPP;

  extern __shared__ __align__(16) uint8_t s_dyn[];
  int16_t* s_map = reinterpret_cast<int16_t*>(s_dyn);
  const int span_cols = blockDim.x * G::COLS_PER_THREAD;
  const int col0 = blockIdx.x * span_cols;
  if (k > 0) build_outlier_map(s_map, span_cols, col0, oidx, k);

  // without a zero point only one constant per column is needed (see fastq_code_bits); the
  // zero-point variant keeps the exact quotient (scale, reciprocal, zero point per column)
  float s[HAS_ZP ? EPP : 1][8], rc[EPP][8], z[HAS_ZP ? EPP : 1][8];
  int n_own = 0;
  if (active) {
#pragma unroll
    for (int i = 0; i < EPP; ++i) {
      const int c = G::slab_col(ct, i);
      uint4 sv = *reinterpret_cast<const uint4*>(scale + c);
      const uint32_t sw[4] = {sv.x, sv.y, sv.z, sv.w};
      uint4 mv = make_uint4(0xffffffffu, 0xffffffffu, 0xffffffffu, 0xffffffffu);
      if (k > 0) mv = *reinterpret_cast<const uint4*>(s_map + (c - col0));
      const uint32_t mw[4] = {mv.x, mv.y, mv.z, mv.w};
      uint2 zv = make_uint2(0u, 0u);
      if (HAS_ZP) zv = *reinterpret_cast<const uint2*>(zp + c);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        float sf = (e & 1) ? bf16hi_to_f32(sw[e >> 1]) : bf16lo_to_f32(sw[e >> 1]);
        if (HAS_ZP) s[i][e] = sf;
        float r = HAS_ZP ? __frcp_rn(sf) : fastq_scale<QBIT>(__frcp_rn(sf));
        const int jv = (int)(int16_t)((mw[e >> 1] >> (16 * (e & 1))) & 0xffffu);
        if (jv >= 0) {
          r = 0.f;     // the column encodes as zero, as if it had been cleared beforehand
          ++n_own;
        }
        rc[i][e] = r;
        if (HAS_ZP) {
          int zb = (int)(int8_t)(((e < 4 ? zv.x : zv.y) >> (8 * (e & 3))) & 0xffu);
          z[i][e] = (float)zb;
        }
      }
    }
  }
  LaneOutliers lo;
  lo.n = 0; lo.extra = 0u; lo.warp_has = false;
  if (k > 0) {
    lo = deal_outliers(reinterpret_cast<uint32_t*>(s_dyn + 2 * span_cols), col0, active, n_own, [&](auto f) {
      for (int i = 0; i < EPP; ++i)
        for (int e = 0; e < 8; ++e) {
          const int col = G::slab_col(ct, i) + e;
          const int jv = s_map[col - col0];
          if (jv >= 0) f(i, e, col, jv);
        }
    });
  }

  const int64_t n_groups = (rows + kRowUnroll - 1) / kRowUnroll;
  for (int64_t g = blockIdx.y; g < n_groups; g += gridDim.y) {
    const int64_t r0 = g * kRowUnroll;
    if (active) {
      uint4 v[kRowUnroll][EPP];
#pragma unroll
      for (int r = 0; r < kRowUnroll; ++r) {
        const bool ok = (r0 + r) < rows;
#pragma unroll
        for (int i = 0; i < EPP; ++i) {
          v[r][i] = make_uint4(0u, 0u, 0u, 0u);
          if (ok) v[r][i] = ld_stream_v4(x + (r0 + r) * ldx + G::slab_col(ct, i));
        }
      }
      // the lane's share of the outlier columns: full-precision values fetched alongside the vector loads
      // (same cache lines, so the latency is shared)
      __nv_bfloat16 ov[kRowUnroll][kMaxOwn];
      if (lo.n > 0) {
#pragma unroll
        for (int r = 0; r < kRowUnroll; ++r)
#pragma unroll
          for (int t = 0; t < kMaxOwn; ++t)
            if (t < lo.n && (r0 + r) < rows) ov[r][t] = x[(r0 + r) * ldx + lo.col[t]];
      }
#pragma unroll
      for (int r = 0; r < kRowUnroll; ++r) {
        if ((r0 + r) >= rows) break;
        uint2 packed;
        if (HAS_ZP) {
          uint32_t w[EPP][2];
#pragma unroll
          for (int i = 0; i < EPP; ++i) {
            const uint32_t xw[4] = {v[r][i].x, v[r][i].y, v[r][i].z, v[r][i].w};
            int c[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              float xf = (e & 1) ? bf16hi_to_f32(xw[e >> 1]) : bf16lo_to_f32(xw[e >> 1]);
              c[e] = quant_code_signed_zp<QBIT>(xf, s[i][e], rc[i][e], z[i][e]);
            }
            w[i][0] = pack4_s8(c[0], c[1], c[2], c[3]);
            w[i][1] = pack4_s8(c[4], c[5], c[6], c[7]);
          }
          packed = interleave_slabs<QBIT>(w);
        } else {
          packed = make_uint2(0u, 0u);
#pragma unroll
          for (int i = 0; i < EPP; ++i) {
            const uint32_t xw[4] = {v[r][i].x, v[r][i].y, v[r][i].z, v[r][i].w};
            uint32_t b[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              float xf = (e & 1) ? bf16hi_to_f32(xw[e >> 1]) : bf16lo_to_f32(xw[e >> 1]);
              b[e] = fastq_code_bits<QBIT>(xf, rc[i][e]);
            }
            // codes are already offset-binary and below 2^QBIT: slab i goes to bit QBIT*i of each byte
            packed.x |= gather_low_bytes(b[0], b[1], b[2], b[3]) << (QBIT * i);
            packed.y |= gather_low_bytes(b[4], b[5], b[6], b[7]) << (QBIT * i);
          }
        }
        st_stream_v2(q + (r0 + r) * qld + 8 * (int64_t)ct, packed);
        if (lo.n > 0) {
#pragma unroll
          for (int t = 0; t < kMaxOwn; ++t)
            if (t < lo.n) oout[(r0 + r) * k + lo.j[t]] = ov[r][t];
          // columns that were not dealt out (more than two per lane in the warp's span; every lane of
          // such a warp serves dealt entries, so the owner gets here)
          for (uint32_t bits = lo.extra; bits; bits &= bits - 1u) {
            const int b = __ffs(bits) - 1;
            const int col = G::slab_col(ct, b >> 3) + (b & 7);
            oout[(r0 + r) * k + s_map[col - col0]] = x[(r0 + r) * ldx + col];
          }
        }
      }
    }
  }
}

// With a zero point, an outlier column must still encode as "zero": rc == 0 makes the
// quotient 0, and the zero point of that column is then added like for any other column,
// which is what the reference does (it zeroes x, then runs the same kernel).

template <int QBIT, bool HAS_ZP>
__global__ void __launch_bounds__(kThreads, HAS_ZP ? 2 : (QBIT == 8 ? HYC_DEQ_MINBLOCKS + 1 : HYC_DEQ_MINBLOCKS))
unpack_dequant_kernel(const uint8_t* __restrict__ q, int64_t rows, int N,
                      const __nv_bfloat16* __restrict__ scale, const int8_t* __restrict__ zp,
                      const int64_t* __restrict__ oidx, int k, const __nv_bfloat16* __restrict__ oin,
                      __nv_bfloat16* __restrict__ xo, int64_t ldx) {
  using G = Geo<QBIT>;
  constexpr int EPP = G::EPP;
  constexpr uint32_t MASK = (1u << QBIT) - 1u;
  const int ct = blockIdx.x * blockDim.x + threadIdx.x;
  const int n_ct = N / G::COLS_PER_THREAD;
  const bool active = ct < n_ct;
  const int64_t qld = (int64_t)N / EPP;
  const int span_cols = blockDim.x * G::COLS_PER_THREAD;
  const int col0 = blockIdx.x * span_cols;

  extern __shared__ __align__(16) uint8_t s_dyn[];
  int16_t* s_map = reinterpret_cast<int16_t*>(s_dyn);
  if (k > 0) build_outlier_map(s_map, span_cols, col0, oidx, k);

  // x_hat = bf16( bf16(code - half [- z]) * s ).  (code - half - z) is an integer of magnitude
  // <= 255, exact in bf16; the product of two bf16 values rounded once to bf16 is the reference's
  // bf16 multiply.
  //   q = 2, 4 : packed bf16x2 arithmetic on two columns at a time.  0x4300 | code is the bf16
  //              128 + code; one byte-permute builds the pair, one packed subtract removes
  //              128 + half (+ z), one packed multiply applies the scale pair as loaded.
  //   q = 8    : codes reach 255, so the integer goes through fp32: 0x4B000000 | code is 2^23 + code.
  constexpr bool PACKED = QBIT < 8;
  uint32_t s2[EPP][4], off2[(PACKED && HAS_ZP) ? EPP : 1][4];
  float s[PACKED ? 1 : EPP][8], off[PACKED ? 1 : EPP][8];
  int n_own = 0;
  if (active) {
#pragma unroll
    for (int i = 0; i < EPP; ++i) {
      const int c = G::slab_col(ct, i);
      uint4 sv = *reinterpret_cast<const uint4*>(scale + c);
      const uint32_t sw[4] = {sv.x, sv.y, sv.z, sv.w};
      uint2 zv = make_uint2(0u, 0u);
      if (HAS_ZP) zv = *reinterpret_cast<const uint2*>(zp + c);
      uint4 mv = make_uint4(0xffffffffu, 0xffffffffu, 0xffffffffu, 0xffffffffu);
      if (k > 0) mv = *reinterpret_cast<const uint4*>(s_map + (c - col0));
      const uint32_t mw[4] = {mv.x, mv.y, mv.z, mv.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) s2[i][j] = sw[j];
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        int zb = HAS_ZP ? (int)(int8_t)(((e < 4 ? zv.x : zv.y) >> (8 * (e & 3))) & 0xffu) : 0;
        if (PACKED) {
          if (HAS_ZP) {
            const uint32_t ob = f32_to_bf16bits_rn((float)zb);   // |z| <= 128: exact in bf16
            if (e & 1) off2[i][e >> 1] |= ob << 16; else off2[i][e >> 1] = ob;
          }
        } else {
          s[i][e] = (e & 1) ? bf16hi_to_f32(sw[e >> 1]) : bf16lo_to_f32(sw[e >> 1]);
          off[i][e] = 8388608.f + (float)((1 << (QBIT - 1)) + zb);
        }
        const int jv = (int)(int16_t)((mw[e >> 1] >> (16 * (e & 1))) & 0xffffu);
        if (jv >= 0) ++n_own;
      }
    }
  }
  LaneOutliers lo;
  lo.n = 0; lo.extra = 0u; lo.warp_has = false;
  if (k > 0) {
    lo = deal_outliers(reinterpret_cast<uint32_t*>(s_dyn + 2 * span_cols), col0, active, n_own, [&](auto f) {
      for (int i = 0; i < EPP; ++i)
        for (int e = 0; e < 8; ++e) {
          const int col = G::slab_col(ct, i) + e;
          const int jv = s_map[col - col0];
          if (jv >= 0) f(i, e, col, jv);
        }
    });
  }

  const int64_t n_groups = (rows + kDeqUnroll - 1) / kDeqUnroll;
  // 2- and 8-bit codes: the codes of the block's next row group are in flight while the current one is expanded
  // and stored (measured: +3 % and +6 %; the 4-bit instantiation loses 18 % with it and loads in place)
  constexpr bool PIPE = QBIT != 4;
  uint2 pnext[PIPE ? kDeqUnroll : 1];
  if constexpr (PIPE) {
#pragma unroll
    for (int r = 0; r < kDeqUnroll; ++r) {
      const int64_t row = (int64_t)blockIdx.y * kDeqUnroll + r;
      pnext[r] = make_uint2(0u, 0u);
      if (active && row < rows) pnext[r] = ld_stream_v2(q + row * qld + 8 * (int64_t)ct);
    }
  }
  for (int64_t g = blockIdx.y; g < n_groups; g += gridDim.y) {
    const int64_t r0 = g * kDeqUnroll;
    // the lane's share of the saved outlier values, fetched ahead of the de-quantization
    __nv_bfloat16 ov[kDeqUnroll][kMaxOwn];
    if (lo.n > 0) {
#pragma unroll
      for (int r = 0; r < kDeqUnroll; ++r)
#pragma unroll
        for (int t = 0; t < kMaxOwn; ++t)
          if (t < lo.n && (r0 + r) < rows) ov[r][t] = oin[(r0 + r) * k + lo.j[t]];
    }
    uint2 p[kDeqUnroll];
    if constexpr (PIPE) {
      const int64_t n0 = (g + gridDim.y) * kDeqUnroll;
#pragma unroll
      for (int r = 0; r < kDeqUnroll; ++r) {
        p[r] = pnext[r];
        if (active && (n0 + r) < rows) pnext[r] = ld_stream_v2(q + (n0 + r) * qld + 8 * (int64_t)ct);
      }
    } else {
      if (active) {
#pragma unroll
        for (int r = 0; r < kDeqUnroll; ++r) {
          p[r] = make_uint2(0u, 0u);
          if ((r0 + r) < rows) p[r] = ld_stream_v2(q + (r0 + r) * qld + 8 * (int64_t)ct);
        }
      }
    }
#pragma unroll
    for (int r = 0; r < kDeqUnroll; ++r) {
      if ((r0 + r) >= rows) break;
      if (active) {
        uint4 prev = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
        for (int i = 0; i < EPP; ++i) {
          // the codes of slab i, one per byte, then each byte straight into the float 2^23 + code
          constexpr uint32_t BM = MASK * 0x01010101u;
          const uint32_t f0 = (p[r].x >> (QBIT * i)) & BM, f1 = (p[r].y >> (QBIT * i)) & BM;
          uint4 o;
          if (PACKED) {
            constexpr uint32_t C1 = 0x4300u + (uint32_t)((1 << (QBIT - 1)) << 0);   // bf16 bits of 128 + half (half < 128)
            uint32_t ow[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              // bytes 2j, 2j+1 of the slab -> the bf16 pair (128 + code, 128 + code)
              const uint32_t pr = __byte_perm(j < 2 ? f0 : f1, 0x43434343u, 0x4040u | (uint32_t)((2 * j) & 3) | ((uint32_t)(((2 * j) & 3) + 1) << 8));
              const uint32_t sub = C1 | (C1 << 16);
              __nv_bfloat162 v = __hsub2(*reinterpret_cast<const __nv_bfloat162*>(&pr),
                                         *reinterpret_cast<const __nv_bfloat162*>(&sub));
              // code - half in [-8, 7] minus z in [-128, 127]: still an exact bf16 integer
              if (HAS_ZP) v = __hsub2(v, *reinterpret_cast<const __nv_bfloat162*>(&off2[i][j]));
              const __nv_bfloat162 m = __hmul2(v, *reinterpret_cast<const __nv_bfloat162*>(&s2[i][j]));
              ow[j] = *reinterpret_cast<const uint32_t*>(&m);
            }
            o = make_uint4(ow[0], ow[1], ow[2], ow[3]);
          } else {
            float f[8];
#pragma unroll
            for (int e = 0; e < 8; ++e)
              f[e] = (byte_to_magic_float(e < 4 ? f0 : f1, e & 3) - off[i][e]) * s[i][e];
            o.x = pack_bf16x2_rn(f[0], f[1]);
            o.y = pack_bf16x2_rn(f[2], f[3]);
            o.z = pack_bf16x2_rn(f[4], f[5]);
            o.w = pack_bf16x2_rn(f[6], f[7]);
          }
          if (EPP == 4) {
            // 2-bit codes: a thread owns the whole 32-column block, so two slabs make one 32-byte store
            if (i & 1) {
              const uint32_t w8[8] = {prev.x, prev.y, prev.z, prev.w, o.x, o.y, o.z, o.w};
              st_stream_v8(xo + (r0 + r) * ldx + G::slab_col(ct, i - 1), w8);
            } else {
              prev = o;
            }
          } else {
            st_stream_v4(xo + (r0 + r) * ldx + G::slab_col(ct, i), o);
          }
        }
      }
    }
    // the saved values go back on top of the warp's own stores to those columns (another lane's, as a
    // rule): the barrier orders the two.  lo.warp_has is warp-uniform.
    if (lo.warp_has) {
      __syncwarp();
      if (lo.n > 0) {
#pragma unroll
        for (int r = 0; r < kDeqUnroll; ++r) {
          if ((r0 + r) >= rows) break;
#pragma unroll
          for (int t = 0; t < kMaxOwn; ++t)
            if (t < lo.n) xo[(r0 + r) * ldx + lo.col[t]] = ov[r][t];
          // columns that were not dealt out stay with their owner
          for (uint32_t bits = lo.extra; bits; bits &= bits - 1u) {
            const int b = __ffs(bits) - 1;
            const int col = G::slab_col(ct, b >> 3) + (b & 7);
            xo[(r0 + r) * ldx + col] = oin[(r0 + r) * k + s_map[col - col0]];
          }
        }
      }
    }
  }
}

// One resident wave: blocks_per_sm * 148 blocks in total, split over the column tiles, so that the
// per-block set-up (reciprocals, outlier map) is paid once per SM slot and not once per wave.
// block width in {256, 224, ..., 128} that leaves the fewest idle lanes in the last column tile
static inline int pick_threads(int n_ct) {
  int best = 256, best_waste = 1 << 30;
  for (int t = 256; t >= 128; t -= 32) {
    const int tiles = (n_ct + t - 1) / t;
    const int waste = tiles * t - n_ct;
    if (waste < best_waste) { best_waste = waste; best = t; }
  }
  return best;
}

template <typename Kernel>
static inline dim3 stream_grid(Kernel kern, int threads, size_t smem, int64_t rows, int n_ct, int unroll) {
  const int col_tiles = (n_ct + threads - 1) / threads;
  const int64_t groups = (rows + unroll - 1) / unroll;
  int per_sm = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, threads, smem) != cudaSuccess || per_sm < 1) per_sm = 2;
  int64_t slots = ((int64_t)num_sms() * per_sm) / col_tiles;
  if (slots > groups) slots = groups;
  if (slots < 1) slots = 1;
  if (slots > 65535) slots = 65535;
  return dim3((unsigned)col_tiles, (unsigned)slots, 1);
}

}  // namespace hyc

using namespace hyc;

static int check_common(const void* a, const void* b, int64_t rows, int N, int64_t ldx, int q_bit) {
  if (!a || !b) return HYC_ERR_NULL;
  if (q_bit != 2 && q_bit != 4 && q_bit != 8) return HYC_ERR_QBIT;
  if (rows < 0 || N <= 0 || N % 32 != 0 || ldx < N) return HYC_ERR_SHAPE;
  if (ldx % 8 != 0) return HYC_ERR_ALIGN;
  return HYC_OK;
}

extern "C" HYC_API int hyc_quant_pack(const void* x, int64_t rows, int N, int64_t ldx,
                              const void* scale, const int8_t* zp,
                              const int64_t* outlier_idx, int k,
                              void* q_out, void* outlier_out, int q_bit, void* stream) {
  int rc = check_common(x, q_out, rows, N, ldx, q_bit);
  if (rc) return rc;
  if (!scale) return HYC_ERR_NULL;
  if (k < 0 || k > N || k > 32767) return HYC_ERR_SHAPE;
  if (k > 0 && (!outlier_idx || !outlier_out)) return HYC_ERR_NULL;
  if (!aligned(x, 16) || !aligned(scale, 16) || !aligned(q_out, 8) || (zp && !aligned(zp, 8))) return HYC_ERR_ALIGN;
  if (rows == 0) return HYC_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const int cpt = 8 * (8 / q_bit);
  const int threads = pick_threads(N / cpt);
  size_t smem = k > 0 ? (size_t)threads * cpt * 2 + (size_t)(threads / 32) * kWarpList * 4 : 0;   // int16 column map + per-warp lists
#define LAUNCH_Q(QB, ZP)                                                                          \
  quant_pack_kernel<QB, ZP><<<stream_grid(quant_pack_kernel<QB, ZP>, threads, smem, rows, N / cpt, kRowUnroll), threads, smem, st>>>( \
      (const __nv_bfloat16*)x, rows, N, ldx, (const __nv_bfloat16*)scale, zp, outlier_idx, k,      \
      (uint8_t*)q_out, (__nv_bfloat16*)outlier_out)
  if (zp) {
    if (q_bit == 2) LAUNCH_Q(2, true); else if (q_bit == 4) LAUNCH_Q(4, true); else LAUNCH_Q(8, true);
  } else {
    if (q_bit == 2) LAUNCH_Q(2, false); else if (q_bit == 4) LAUNCH_Q(4, false); else LAUNCH_Q(8, false);
  }
#undef LAUNCH_Q
  HYC_CHECK_LAUNCH();
  return HYC_OK;
}

extern "C" HYC_API int hyc_unpack_dequant(const void* q, int64_t rows, int N,
                                  const void* scale, const int8_t* zp,
                                  const int64_t* outlier_idx, int k, const void* outlier,
                                  void* x_out, int64_t ldx, int q_bit, void* stream) {
  int rc = check_common(q, x_out, rows, N, ldx, q_bit);
  if (rc) return rc;
  if (!scale) return HYC_ERR_NULL;
  if (k < 0 || k > N || k > 32767) return HYC_ERR_SHAPE;
  if (k > 0 && (!outlier_idx || !outlier)) return HYC_ERR_NULL;
  if (!aligned(x_out, q_bit == 2 ? 32 : 16) || !aligned(scale, 16) || !aligned(q, 8) || (zp && !aligned(zp, 8))) return HYC_ERR_ALIGN;
  if (q_bit == 2 && ldx % 16 != 0) return HYC_ERR_ALIGN;
  if (rows == 0) return HYC_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const int cpt = 8 * (8 / q_bit);
  const int threads = pick_threads(N / cpt);
  size_t smem = k > 0 ? (size_t)threads * cpt * 2 + (size_t)(threads / 32) * kWarpList * 4 : 0;
#define LAUNCH_D(QB, ZP)                                                                          \
  unpack_dequant_kernel<QB, ZP><<<stream_grid(unpack_dequant_kernel<QB, ZP>, threads, smem, rows, N / cpt, kDeqUnroll), threads, smem, st>>>(                                        \
      (const uint8_t*)q, rows, N, (const __nv_bfloat16*)scale, zp, outlier_idx, k,                 \
      (const __nv_bfloat16*)outlier, (__nv_bfloat16*)x_out, ldx)
  if (zp) {
    if (q_bit == 2) LAUNCH_D(2, true); else if (q_bit == 4) LAUNCH_D(4, true); else LAUNCH_D(8, true);
  } else {
    if (q_bit == 2) LAUNCH_D(2, false); else if (q_bit == 4) LAUNCH_D(4, false); else LAUNCH_D(8, false);
  }
#undef LAUNCH_D
  HYC_CHECK_LAUNCH();
  return HYC_OK;
}

// Per-row top-k attention-map path, lane-per-group layout.
//
// A row of S = 64 * LPR columns (LPR = 1, 2, ..., 32 lanes per row) is spread over LPR adjacent lanes,
// every lane owning ONE quantization group: 64 consecutive columns = 128 contiguous bytes = 32 packed
// bf16 pairs.  A warp therefore works on 32 / LPR rows at a time, and everything that costs one warp
// instruction per row in a warp-per-row layout (reductions, scans, group parameters) is shared by
// those rows; group min/max needs no shuffle at all.
//
// Selection of the k largest magnitudes of a row is an exact radix select on BIT PLANES:
//   1. the lane's 64 magnitude patterns (15 bits) are bit-transposed in registers into 15 planes of
//      64 bits (plane b, bit c = bit b of the magnitude of the lane's column c): one byte-permute stage
//      and three shift/mask stages over 32 registers;
//   2. from the top plane down, one round per bit: ones = popc(plane & active) summed over the row's
//      lanes (one redux); if (count above + ones) >= k the bit of the threshold is 1 and the active set
//      shrinks to those elements, otherwise they are certainly selected ("greater" set) and leave the
//      active set.  Fifteen rounds of about a dozen instructions, whatever the data.
//   3. what is still active equals the threshold; those ties are taken in ascending column order.
// The selected elements are picked out of a shared-memory copy of the rows (which also zeroes them),
// staged as (column << 16 | value) words and written as one contiguous run per warp: the lists of
// adjacent rows are adjacent in memory.
#include "topk_lane.cuh"

#ifndef HYC_TK_MINB
#define HYC_TK_MINB 4      // resident blocks per SM the kernels are compiled for (register cap 64)
#endif

namespace hyc {

template <int LPR>
__device__ __forceinline__ int seg_add(unsigned segmask, int v) {
  if (LPR == 1) return v;
  return (int)__reduce_add_sync(segmask, (unsigned)v);
}
template <int LPR>
__device__ __forceinline__ int seg_excl_scan(int v, int lr) {
  int incl = v;
#pragma unroll
  for (int o = 1; o < LPR; o <<= 1) {
    const int t = __shfl_up_sync(kFull, incl, o, LPR);
    if (lr >= o) incl += t;
  }
  return incl - v;
}

// w with only its n lowest set bits kept (n < popc(w))
__device__ __forceinline__ uint32_t keep_lowest_bits(uint32_t w, int n) {
  uint32_t r = w;
  for (int i = 0; i < n; ++i) r &= r - 1u;
  return w ^ r;
}

// address (in 32-bit words) of 16-byte chunk c of a lane's 128-byte slot: chunks are rotated by the
// lane number so that 128-bit accesses of eight adjacent lanes fall on distinct banks
__device__ __forceinline__ int park_chunk(int c, int lane) { return ((c ^ (lane & 7)) << 2); }

// min / max over the 64 values of a lane
__device__ __forceinline__ void lane_minmax(const uint32_t (&xw)[32], float& mn, float& mx) {
  __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&xw[0]), hi = lo;
#pragma unroll
  for (int j = 1; j < 32; ++j) {
    const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(&xw[j]);
    lo = __hmin2(lo, v);
    hi = __hmax2(hi, v);
  }
  mn = fminf(__bfloat162float(lo.x), __bfloat162float(lo.y));
  mx = fmaxf(__bfloat162float(hi.x), __bfloat162float(hi.y));
}

// Quantize the lane's 64 values and store them in the reference byte layout (two 32-column blocks).
// 4- and 8-bit codes leave as 256-bit stores: the packed rows must be 32-byte aligned.
template <int QBIT>
__device__ __forceinline__ void lane_quant_store(const uint32_t (&xw)[32], const GroupParams& p,
                                                 uint8_t* __restrict__ qgroup) {
  uint32_t w[16];   // w[i] = codes of columns 4i..4i+3, one per byte
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const uint32_t b0 = group_code_bits<QBIT>(bf16lo_to_f32(xw[2 * i]), p);
    const uint32_t b1 = group_code_bits<QBIT>(bf16hi_to_f32(xw[2 * i]), p);
    const uint32_t b2 = group_code_bits<QBIT>(bf16lo_to_f32(xw[2 * i + 1]), p);
    const uint32_t b3 = group_code_bits<QBIT>(bf16hi_to_f32(xw[2 * i + 1]), p);
    w[i] = gather_low_bytes(b0, b1, b2, b3);
  }
  if (QBIT == 8) {
#pragma unroll
    for (int i = 0; i < 2; ++i) st_stream_v8(qgroup + 32 * i, *reinterpret_cast<const uint32_t(*)[8]>(&w[8 * i]));
  } else if (QBIT == 4) {
    // block h: byte j = code[j] | code[16 + j] << 4
    uint32_t o[8];
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
      for (int i = 0; i < 4; ++i) o[4 * h + i] = w[8 * h + i] | (w[8 * h + 4 + i] << 4);
    st_stream_v8(qgroup, o);
  } else {
    // block h: byte j = code[j] | code[8 + j] << 2 | code[16 + j] << 4 | code[24 + j] << 6
    uint32_t o[4];
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
      for (int i = 0; i < 2; ++i)
        o[2 * h + i] = w[8 * h + i] | (w[8 * h + 2 + i] << 2) | (w[8 * h + 4 + i] << 4) | (w[8 * h + 6 + i] << 6);
    st_stream_v4(qgroup, make_uint4(o[0], o[1], o[2], o[3]));
  }
}

// ---------------------------------------------------------------- compress
template <int QBIT, int LPR>
__global__ void __launch_bounds__(256, HYC_TK_MINB)
topk_lane_compress_kernel(const __nv_bfloat16* __restrict__ a, int64_t rows, int k,
                          __nv_bfloat16* __restrict__ val_out, uint16_t* __restrict__ col_out,
                          uint8_t* __restrict__ q, __nv_bfloat16* __restrict__ scale, int8_t* __restrict__ zp) {
  constexpr int RPW = 32 / LPR;          // rows per warp
  constexpr int S = 64 * LPR;
  constexpr int64_t QLD = (int64_t)S * QBIT / 8;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int lr = lane & (LPR - 1), rw = lane / LPR;
  const unsigned segmask = (LPR == 32) ? kFull : (((1u << LPR) - 1u) << (lane & ~(LPR - 1)));
  __shared__ __align__(16) uint32_t s_x[8][32 * 32];          // the warp's rows, 128 bytes per lane
  __shared__ uint32_t s_out[8][kLaneStageEntries];            // staged (column << 16 | value) words
  uint32_t* sx = s_x[warp] + lane * 32;
  uint32_t* so = s_out[warp];
  const int64_t items = (rows + RPW - 1) / RPW;
  for (int64_t item = (int64_t)blockIdx.x * 8 + warp; item < items; item += (int64_t)gridDim.x * 8) {
    const int64_t row0 = item * RPW, row = row0 + rw;
    const bool valid = row < rows;
    // The warp's rows are one contiguous run of 4 KB.  It is fetched as four fully coalesced 1 KB loads
    // (lane t takes the 32-byte piece 32 i + t), parked in shared memory at its owner's slot, and every
    // lane then reads its own group back.
    const int64_t left = rows - row0;
    const int n_pieces = (int)(left < RPW ? left : RPW) * (S / 16);      // valid 32-byte pieces of the run
    {
      const __nv_bfloat16* run = a + row0 * S;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int p = 32 * i + lane;
        uint32_t t[8];
        if (p < n_pieces) {
          ld_stream_v8(run + 16 * p, t);
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) t[j] = 0u;
        }
        const int owner = p >> 2, c0 = 2 * (p & 3);
        uint32_t* dst = s_x[warp] + owner * 32;
        *reinterpret_cast<uint4*>(dst + park_chunk(c0, owner)) = make_uint4(t[0], t[1], t[2], t[3]);
        *reinterpret_cast<uint4*>(dst + park_chunk(c0 + 1, owner)) = make_uint4(t[4], t[5], t[6], t[7]);
      }
    }
    __syncwarp();
    uint32_t xw[32];
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      const uint4 t = *reinterpret_cast<const uint4*>(sx + park_chunk(c, lane));
      xw[4 * c] = t.x; xw[4 * c + 1] = t.y; xw[4 * c + 2] = t.z; xw[4 * c + 3] = t.w;
    }

    if (k > 0) {
      // ---- magnitudes, paired (column c, column c + 16) so that the transposed planes come out in
      // column order: m[16 h + c] = (|x[32 h + c]|, |x[32 h + 16 + c]|), c = 0..15
      uint32_t m[32];
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const uint32_t lo = xw[16 * h + i], hi = xw[16 * h + 8 + i];
          m[16 * h + 2 * i] = __byte_perm(lo, hi, 0x5410) & 0x7fff7fffu;
          m[16 * h + 2 * i + 1] = __byte_perm(lo, hi, 0x7632) & 0x7fff7fffu;
        }
      // ---- bit transpose.  Register index j = (h, c3 c2 c1 c0), bit position = (c4, b3 b2 b1 b0); every
      // stage swaps one index bit with one position bit, after the last one register 16 h + b holds
      // plane b of columns 32 h .. 32 h + 31 with column c at bit c.
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if ((j & 8) == 0) {
          const uint32_t x = m[j], y = m[j + 8];
          m[j] = __byte_perm(x, y, 0x6240);
          m[j + 8] = __byte_perm(x, y, 0x7351);
        }
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if ((j & 4) == 0) {
          const uint32_t x = m[j], y = m[j + 4];
          m[j] = (x & 0x0f0f0f0fu) | ((y << 4) & 0xf0f0f0f0u);
          m[j + 4] = ((x >> 4) & 0x0f0f0f0fu) | (y & 0xf0f0f0f0u);
        }
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if ((j & 2) == 0) {
          const uint32_t x = m[j], y = m[j + 2];
          m[j] = (x & 0x33333333u) | ((y << 2) & 0xccccccccu);
          m[j + 2] = ((x >> 2) & 0x33333333u) | (y & 0xccccccccu);
        }
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if ((j & 1) == 0) {
          const uint32_t x = m[j], y = m[j + 1];
          m[j] = (x & 0x55555555u) | ((y << 1) & 0xaaaaaaaau);
          m[j + 1] = ((x >> 1) & 0x55555555u) | (y & 0xaaaaaaaau);
        }
      // ---- radix select, most significant plane first
      // (branch-free: the rows of a warp take different sides)
      uint32_t A0 = kFull, A1 = kFull, G0 = 0u, G1 = 0u;
      int rem = k;                       // k - (number of magnitudes known to be above the threshold)
#pragma unroll
      for (int b = 14; b >= 0; --b) {
        const uint32_t x0 = m[b] & A0, x1 = m[16 + b] & A1;
        const int tot = seg_add<LPR>(segmask, __popc(x0) + __popc(x1));
        const uint32_t drop = (tot >= rem) ? 0u : kFull;   // all ones: the threshold has a 0 here, the ones are above it
        G0 |= x0 & drop; G1 |= x1 & drop;
        A0 &= m[b] ^ drop; A1 &= m[16 + b] ^ drop;
        rem -= tot & (int)drop;
      }
      // ---- ties at the threshold: the first `rem` of them in column order
      {
        const int nt = __popc(A0) + __popc(A1);
        const int pre = seg_excl_scan<LPR>(nt, lr);
        const int take = min(max(rem - pre, 0), nt);
        if (take < nt) {
          const int n0 = __popc(A0);
          if (take >= n0) { A1 = keep_lowest_bits(A1, take - n0); }
          else { A0 = keep_lowest_bits(A0, take); A1 = 0u; }
        }
      }
      uint32_t sel0 = G0 | A0, sel1 = G1 | A1;
      if (!valid) { sel0 = 0u; sel1 = 0u; }
      // ---- pick the selected elements (ascending columns) out of the parked copy and zero them there
      // (highest bit first, so the slots are filled from the lane's last one down)
      const int nsel = __popc(sel0) + __popc(sel1);
      uint32_t* slot = so + rw * k + seg_excl_scan<LPR>(nsel, lr) + nsel;
      uint16_t* sx16 = reinterpret_cast<uint16_t*>(sx);
      const uint32_t sw8 = (uint32_t)(lane & 7) << 3;          // chunk rotation, in halfword units
#pragma unroll
      for (int h = 1; h >= 0; --h) {
        uint32_t bits = h ? sel1 : sel0;
        const uint32_t colh = (64u * (uint32_t)lr + 32u * h) << 16;
        while (bits) {
          const uint32_t e = 31u - (uint32_t)__clz(bits);
          bits ^= 1u << e;
          uint16_t* at = sx16 + ((e + 32u * h) ^ sw8);
          const uint32_t v = *at;
          *at = 0;
          *--slot = (colh + (e << 16)) | v;
        }
      }
      __syncwarp();
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const uint4 t = *reinterpret_cast<const uint4*>(sx + park_chunk(c, lane));
        xw[4 * c] = t.x; xw[4 * c + 1] = t.y; xw[4 * c + 2] = t.z; xw[4 * c + 3] = t.w;
      }
      // the lists of the warp's rows are one contiguous run
      const int n_ent = (int)(left < RPW ? left : RPW) * k;
      __nv_bfloat16* vrun = val_out + row0 * k;
      uint16_t* crun = col_out + row0 * k;
      for (int j = lane; j < n_ent; j += 32) {
        const uint32_t w = so[j];
        vrun[j] = __ushort_as_bfloat16((uint16_t)(w & 0xffffu));
        crun[j] = (uint16_t)(w >> 16);
      }
      __syncwarp();
    }

    float mn, mx;
    lane_minmax(xw, mn, mx);
    const GroupParams p = group_params<QBIT>(mn, mx);
    if (valid) {
      lane_quant_store<QBIT>(xw, p, q + row * QLD + (64 * QBIT / 8) * lr);
      scale[row * LPR + lr] = __ushort_as_bfloat16(f32_to_bf16bits_rn(p.s));
      zp[row * LPR + lr] = (int8_t)(int)p.z;
    }
  }
}

// ---------------------------------------------------------------- restore
// x_hat = bf16((code - half - z) * s) for the lane's 64 columns (see load_dequant16 in group_topk.cu
// for why the packed bf16 path is exact).
template <int QBIT>
__device__ __forceinline__ void lane_load_dequant(const uint8_t* __restrict__ qgroup, float s, float z, uint32_t (&out)[32]) {
  if (QBIT == 8) {
    const float off = 8388608.f + 128.f + z;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      uint32_t b[8];
      ld_stream_v8(qgroup + 32 * i, b);
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const float f0 = (byte_to_magic_float(b[j >> 1], (2 * j) & 3) - off) * s;
        const float f1 = (byte_to_magic_float(b[j >> 1], ((2 * j) & 3) + 1) - off) * s;
        out[16 * i + j] = pack_bf16x2_rn(f0, f1);
      }
    }
  } else {
    constexpr uint32_t BM = ((1u << QBIT) - 1u) * 0x01010101u;
    constexpr uint32_t C1 = 0x4300u | (uint32_t)(1 << (QBIT - 1));      // bf16 bits of 128 + half
    const uint32_t c1 = C1 | (C1 << 16);
    const uint32_t zb = f32_to_bf16bits_rn(z), z2 = zb | (zb << 16);
    const uint32_t sb = f32_to_bf16bits_rn(s), s2 = sb | (sb << 16);
    uint32_t w[16];    // codes of columns 4i..4i+3, one per byte
    if (QBIT == 4) {
      uint32_t v[8];
      ld_stream_v8(qgroup, v);
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          w[8 * h + i] = v[4 * h + i] & BM;
          w[8 * h + 4 + i] = (v[4 * h + i] >> 4) & BM;
        }
    } else {
      const uint4 v0 = ld_stream_v4(qgroup);
      const uint32_t v[4] = {v0.x, v0.y, v0.z, v0.w};
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int f = 0; f < 4; ++f)
#pragma unroll
          for (int i = 0; i < 2; ++i) w[8 * h + 2 * f + i] = (v[2 * h + i] >> (2 * f)) & BM;
    }
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      const uint32_t pr = __byte_perm(w[j >> 1], 0x43434343u, (j & 1) ? 0x4342u : 0x4140u);
      __nv_bfloat162 t = __hsub2(*reinterpret_cast<const __nv_bfloat162*>(&pr), *reinterpret_cast<const __nv_bfloat162*>(&c1));
      t = __hsub2(t, *reinterpret_cast<const __nv_bfloat162*>(&z2));
      t = __hmul2(t, *reinterpret_cast<const __nv_bfloat162*>(&s2));
      out[j] = *reinterpret_cast<const uint32_t*>(&t);
    }
  }
}

template <int QBIT, int LPR>
__global__ void __launch_bounds__(256, HYC_TK_MINB)
topk_lane_restore_kernel(const __nv_bfloat16* __restrict__ val, const uint16_t* __restrict__ colv, int k, float inv_k,
                         const uint8_t* __restrict__ q, const __nv_bfloat16* __restrict__ scale,
                         const int8_t* __restrict__ zp, int64_t rows, __nv_bfloat16* __restrict__ ao) {
  constexpr int RPW = 32 / LPR;
  constexpr int S = 64 * LPR;
  constexpr int64_t QLD = (int64_t)S * QBIT / 8;
  constexpr int PRE = 4;                 // list entries per lane fetched before the de-quantization
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int lr = lane & (LPR - 1), rw = lane / LPR;
  __shared__ __align__(16) uint32_t s_x[8][32 * 32];          // the warp's rows, 128 bytes per lane
  uint32_t* sx = s_x[warp] + lane * 32;
  uint16_t* sw16 = reinterpret_cast<uint16_t*>(s_x[warp]);
  const int64_t items = (rows + RPW - 1) / RPW;
  for (int64_t item = (int64_t)blockIdx.x * 8 + warp; item < items; item += (int64_t)gridDim.x * 8) {
    const int64_t row0 = item * RPW, row = row0 + rw;
    const bool valid = row < rows;
    const int64_t left = rows - row0;
    const int n_rows = (int)(left < RPW ? left : RPW);
    const int n_ent = n_rows * k;
    const __nv_bfloat16* vrun = val + row0 * k;
    const uint16_t* crun = colv + row0 * k;
    uint16_t pc[PRE], pv[PRE];
#pragma unroll
    for (int i = 0; i < PRE; ++i) {
      const int j = lane + 32 * i;
      pc[i] = 0; pv[i] = 0;
      if (j < n_ent) { pc[i] = crun[j]; pv[i] = __bfloat16_as_ushort(vrun[j]); }
    }
    // de-quantize the lane's group into its shared-memory slot
    {
      uint32_t o[32];
      if (valid) {
        const float s = __bfloat162float(scale[row * LPR + lr]);
        const float z = (float)zp[row * LPR + lr];
        lane_load_dequant<QBIT>(q + row * QLD + (64 * QBIT / 8) * lr, s, z, o);
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) o[j] = 0u;
      }
#pragma unroll
      for (int c = 0; c < 8; ++c)
        *reinterpret_cast<uint4*>(sx + park_chunk(c, lane)) = make_uint4(o[4 * c], o[4 * c + 1], o[4 * c + 2], o[4 * c + 3]);
    }
    __syncwarp();
    // the outlier lists overwrite their entries there.  Entry j of the run belongs to row j / k of the warp:
    // (j + 0.5) / k is never within 1/(2k) of an integer, so the fp32 product truncates to the exact quotient.
    // Column c of that row lives in lane (row * LPR + c / 64), halfword (c % 64) rotated like the chunks.
#pragma unroll
    for (int i = 0; i < PRE; ++i) {
      const int j = lane + 32 * i;
      if (j < n_ent) {
        const int r = (int)(((float)j + 0.5f) * inv_k);
        const int owner = r * LPR + (pc[i] >> 6);
        sw16[owner * 64 + ((pc[i] & 63) ^ ((owner & 7) << 3))] = pv[i];
      }
    }
    for (int j = lane + 32 * PRE; j < n_ent; j += 32) {
      const int r = (int)(((float)j + 0.5f) * inv_k);
      const int c = crun[j];
      const int owner = r * LPR + (c >> 6);
      sw16[owner * 64 + ((c & 63) ^ ((owner & 7) << 3))] = __bfloat16_as_ushort(vrun[j]);
    }
    __syncwarp();
    // the warp's rows leave as four fully coalesced 1 KB stores (lane t writes the 32-byte piece 32 i + t)
    {
      const int n_pieces = n_rows * (S / 16);
      __nv_bfloat16* run = ao + row0 * S;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int p = 32 * i + lane;
        const int owner = p >> 2, c0 = 2 * (p & 3);
        const uint32_t* src = s_x[warp] + owner * 32;
        const uint4 t0 = *reinterpret_cast<const uint4*>(src + park_chunk(c0, owner));
        const uint4 t1 = *reinterpret_cast<const uint4*>(src + park_chunk(c0 + 1, owner));
        const uint32_t t[8] = {t0.x, t0.y, t0.z, t0.w, t1.x, t1.y, t1.z, t1.w};
        if (p < n_pieces) st_stream_v8(run + 16 * p, t);
      }
    }
    __syncwarp();
  }
}

// ---------------------------------------------------------------- launchers
template <typename K>
static int lane_grid(K kern, int64_t rows, int rows_per_warp) {
  int per_sm = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, 256, 0) != cudaSuccess || per_sm < 1) per_sm = 1;
  const int64_t items = (rows + rows_per_warp - 1) / rows_per_warp;
  int64_t blocks = (items + 7) / 8;
  const int64_t cap = (int64_t)kNumSMs * per_sm;
  if (blocks > cap) blocks = cap;
  return (int)(blocks < 1 ? 1 : blocks);
}

template <int QBIT, int LPR>
static void launch_compress(const void* a, int64_t rows, int k, void* val, uint16_t* col, void* q, void* scale,
                            int8_t* zp, cudaStream_t st) {
  auto kern = topk_lane_compress_kernel<QBIT, LPR>;
  kern<<<lane_grid(kern, rows, 32 / LPR), 256, 0, st>>>((const __nv_bfloat16*)a, rows, k, (__nv_bfloat16*)val, col,
                                                       (uint8_t*)q, (__nv_bfloat16*)scale, zp);
}
template <int QBIT, int LPR>
static void launch_restore(const void* val, const uint16_t* col, int k, const void* q, const void* scale,
                           const int8_t* zp, int64_t rows, void* ao, cudaStream_t st) {
  auto kern = topk_lane_restore_kernel<QBIT, LPR>;
  kern<<<lane_grid(kern, rows, 32 / LPR), 256, 0, st>>>((const __nv_bfloat16*)val, col, k, k > 0 ? 1.0f / (float)k : 0.f,
                                                       (const uint8_t*)q, (const __nv_bfloat16*)scale, zp, rows,
                                                       (__nv_bfloat16*)ao);
}

#define HYC_LANE_DISPATCH(FN, ...)                                            \
  switch (S / 64) {                                                           \
    case 1: FN<QB, 1>(__VA_ARGS__); break;                                    \
    case 2: FN<QB, 2>(__VA_ARGS__); break;                                    \
    case 4: FN<QB, 4>(__VA_ARGS__); break;                                    \
    case 8: FN<QB, 8>(__VA_ARGS__); break;                                    \
    case 16: FN<QB, 16>(__VA_ARGS__); break;                                  \
    case 32: FN<QB, 32>(__VA_ARGS__); break;                                  \
    default: return HYC_ERR_SHAPE;                                            \
  }

template <int QB>
static int compress_q(const void* a, int64_t rows, int S, int k, void* val, uint16_t* col, void* q, void* scale,
                      int8_t* zp, cudaStream_t st) {
  HYC_LANE_DISPATCH(launch_compress, a, rows, k, val, col, q, scale, zp, st);
  return HYC_OK;
}
template <int QB>
static int restore_q(const void* val, const uint16_t* col, int k, const void* q, const void* scale, const int8_t* zp,
                     int64_t rows, int S, void* ao, cudaStream_t st) {
  HYC_LANE_DISPATCH(launch_restore, val, col, k, q, scale, zp, rows, ao, st);
  return HYC_OK;
}

int topk_lane_compress(const void* a, int64_t rows, int S, int k, void* val_out, uint16_t* col_out,
                       void* q_out, void* scale_out, int8_t* zp_out, int q_bit, cudaStream_t st) {
  if (!topk_lane_ok(S, k)) return HYC_ERR_SHAPE;
  if (q_bit == 2) return compress_q<2>(a, rows, S, k, val_out, col_out, q_out, scale_out, zp_out, st);
  if (q_bit == 4) return compress_q<4>(a, rows, S, k, val_out, col_out, q_out, scale_out, zp_out, st);
  return compress_q<8>(a, rows, S, k, val_out, col_out, q_out, scale_out, zp_out, st);
}
int topk_lane_restore(const void* val, const uint16_t* col, int k, const void* q, const void* scale,
                      const int8_t* zp, int64_t rows, int S, void* a_out, int q_bit, cudaStream_t st) {
  if (!topk_lane_ok(S, k)) return HYC_ERR_SHAPE;
  if (q_bit == 2) return restore_q<2>(val, col, k, q, scale, zp, rows, S, a_out, st);
  if (q_bit == 4) return restore_q<4>(val, col, k, q, scale, zp, rows, S, a_out, st);
  return restore_q<8>(val, col, k, q, scale, zp, rows, S, a_out, st);
}

}  // namespace hyc

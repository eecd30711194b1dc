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
#include "lane_group.cuh"

namespace hyc {

// sum over the LPR lanes of a row.  A whole warp uses the hardware reduction; for a part of a warp
// __reduce_add_sync with a partial mask is expanded into some twenty instructions, log2(LPR) butterfly
// steps are far cheaper (measured: 4.4 M of the kernel's 31 M warp instructions, 8 us of 47)
template <int LPR>
__device__ __forceinline__ int seg_add(int v) {
  if (LPR == 32) return (int)__reduce_add_sync(kFull, (unsigned)v);
#pragma unroll
  for (int o = 1; o < LPR; o <<= 1) v += __shfl_xor_sync(kFull, v, o);
  return v;
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

// What the SOFTMAX form of the compress kernel needs besides the map itself: the raw scores are read from `a`, turned
// into probabilities (scale, additive mask, softmax with the rounding points of softmax_fwd_kernel in
// norm_softmax.cu), written to `dense` for the P.V product, and saved in the same pass.
struct SoftmaxPrologue {
  float scale;
  const __nv_bfloat16* mask;     // additive mask or NULL; row m of (batch b, head h) at mask + b * mb + h * mh + m * S
  int64_t mb, mh;
  int heads, M;                  // rows = batch * heads * M, M a multiple of the rows a warp takes
  __nv_bfloat16* dense;          // [rows, S] probabilities (may be the scores buffer itself)
};

// ---------------------------------------------------------------- compress
template <int QBIT, int LPR, bool SOFTMAX>
__global__ void __launch_bounds__(256, HYC_LANE_MINB)
topk_lane_compress_kernel(const __nv_bfloat16* __restrict__ a, int64_t rows, int k,
                          __nv_bfloat16* __restrict__ val_out, uint16_t* __restrict__ col_out,
                          uint8_t* __restrict__ q, __nv_bfloat16* __restrict__ scale, int8_t* __restrict__ zp,
                          SoftmaxPrologue sp) {
  constexpr int RPW = 32 / LPR;          // rows per warp
  constexpr int S = 64 * LPR;
  constexpr int64_t QLD = (int64_t)S * QBIT / 8;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int lr = lane & (LPR - 1), rw = lane / LPR;
  __shared__ __align__(16) uint32_t s_x[8][32 * 32];          // the warp's rows, 128 bytes per lane
  __shared__ uint32_t s_out[8][kLaneStageEntries];            // staged (column << 16 | value) words
  uint32_t* sx = s_x[warp] + lane * 32;
  uint32_t* so = s_out[warp];
  const int64_t items = (rows + RPW - 1) / RPW;
  for (int64_t item = (int64_t)blockIdx.x * nwarps + warp; item < items; item += (int64_t)gridDim.x * nwarps) {
    const int64_t row0 = item * RPW, row = row0 + rw;
    const bool valid = row < rows;
    // the warp's rows are one contiguous run of 4 KB: fetch it, park it, read the lane's own group back
    const int64_t left = rows - row0;
    const int n_rows = (int)(left < RPW ? left : RPW);
    lane_run_to_shared(a + row0 * S, n_rows * (S / 16), s_x[warp], lane);
    __syncwarp();
    uint32_t xw[32];
    lane_slot_load(sx, lane, xw);

    if (SOFTMAX) {
      // ---- scores -> probabilities.  u = bf16(bf16(s * scale) + mask) replaces the raw scores in xw; the row maximum,
      // the exponentials and their sum are fp32; p = bf16(e / sum).  The exponentials are evaluated twice (once for
      // the sum, once for the result) instead of keeping 64 fp32 values per lane alive.
      constexpr float kLog2e = 1.4426950408889634f;
      __syncwarp();
      if (sp.mask != nullptr) {
        const int64_t bh = row0 / sp.M;
        const int m0 = (int)(row0 - bh * sp.M);
        lane_run_to_shared(sp.mask + (bh / sp.heads) * sp.mb + (bh % sp.heads) * sp.mh + (int64_t)m0 * S, n_rows * (S / 16),
                           s_x[warp], lane);
        __syncwarp();
      }
      __nv_bfloat162 hmx = __float2bfloat162_rn(-INFINITY);
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        uint4 mk = make_uint4(0u, 0u, 0u, 0u);
        if (sp.mask != nullptr) mk = *reinterpret_cast<const uint4*>(sx + park_chunk(c, lane));
        const uint32_t mw[4] = {mk.x, mk.y, mk.z, mk.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint32_t t = pack_bf16x2_rn(bf16lo_to_f32(xw[4 * c + j]) * sp.scale, bf16hi_to_f32(xw[4 * c + j]) * sp.scale);
          if (sp.mask != nullptr)
            t = pack_bf16x2_rn(bf16lo_to_f32(t) + bf16lo_to_f32(mw[j]), bf16hi_to_f32(t) + bf16hi_to_f32(mw[j]));
          xw[4 * c + j] = t;
          hmx = __hmax2(hmx, *reinterpret_cast<const __nv_bfloat162*>(&t));
        }
      }
      float mx = fmaxf(__bfloat162float(hmx.x), __bfloat162float(hmx.y));
#pragma unroll
      for (int o = 1; o < LPR; o <<= 1) mx = fmaxf(mx, __shfl_xor_sync(kFull, mx, o));
      const float mxl = mx * kLog2e;
      float sum = 0.f;
#pragma unroll
      for (int j = 0; j < 32; ++j)
        sum += exp2f(fmaf(bf16lo_to_f32(xw[j]), kLog2e, -mxl)) + exp2f(fmaf(bf16hi_to_f32(xw[j]), kLog2e, -mxl));
#pragma unroll
      for (int o = 1; o < LPR; o <<= 1) sum += __shfl_xor_sync(kFull, sum, o);
      const float inv = 1.0f / sum;
#pragma unroll
      for (int j = 0; j < 32; ++j)
        xw[j] = pack_bf16x2_rn(exp2f(fmaf(bf16lo_to_f32(xw[j]), kLog2e, -mxl)) * inv,
                               exp2f(fmaf(bf16hi_to_f32(xw[j]), kLog2e, -mxl)) * inv);
      // the probabilities go to the parked copy (the emission below picks its entries there) and out as the dense map
      __syncwarp();
      lane_slot_store(sx, lane, xw);
      __syncwarp();
      lane_shared_to_run(s_x[warp], sp.dense + row0 * S, n_rows * (S / 16), lane);
      __syncwarp();
    }

    if (k > 0) {
      // ---- values paired (column c, column c + 16) so that the transposed planes come out in column
      // order: m[16 h + c] = (x[32 h + c], x[32 h + 16 + c]), c = 0..15.  Plane 15 (the signs) is never
      // read, so planes 14..0 are the magnitude patterns.
      uint32_t m[32];
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const uint32_t lo = xw[16 * h + i], hi = xw[16 * h + 8 + i];
          m[16 * h + 2 * i] = __byte_perm(lo, hi, 0x5410);
          m[16 * h + 2 * i + 1] = __byte_perm(lo, hi, 0x7632);
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
        const int tot = seg_add<LPR>(__popc(x0) + __popc(x1));
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
        // two elements per trip: the busiest lane of the warp sets the number of trips (the large entries of a
        // causal row sit in few groups), and each trip is a load -> store chain
        while (bits) {
          const uint32_t e0 = 31u - (uint32_t)__clz(bits);
          bits ^= 1u << e0;
          const bool two = bits != 0u;
          const uint32_t e1 = two ? 31u - (uint32_t)__clz(bits) : e0;
          bits &= ~(1u << e1);
          uint16_t* at0 = sx16 + ((e0 + 32u * h) ^ sw8);
          uint16_t* at1 = sx16 + ((e1 + 32u * h) ^ sw8);
          const uint32_t v0 = *at0, v1 = *at1;
          *at0 = 0;
          *at1 = 0;                      // the same halfword again when there was only one
          slot[-1] = (colh + (e0 << 16)) | v0;
          if (two) slot[-2] = (colh + (e1 << 16)) | v1;
          slot -= two ? 2 : 1;
        }
      }
      __syncwarp();
      lane_slot_load(sx, lane, xw);
      // the lists of the warp's rows are one contiguous run
      const int n_ent = n_rows * k;
      __nv_bfloat16* vrun = val_out + row0 * k;
      uint16_t* crun = col_out + row0 * k;
      for (int j = lane; j < n_ent; j += 32) {
        const uint32_t w = so[j];
        vrun[j] = __ushort_as_bfloat16((uint16_t)(w & 0xffffu));
        crun[j] = (uint16_t)(w >> 16);
      }
    }

    float mn, mx;
    lane_minmax(xw, mn, mx);
    const GroupParams p = group_params<QBIT>(mn, mx);
    if (valid) {
      lane_quant_store<QBIT>(xw, p, q + row * QLD + (64 * QBIT / 8) * lr);
      scale[row * LPR + lr] = __ushort_as_bfloat16(f32_to_bf16bits_rn(p.s));
      zp[row * LPR + lr] = (int8_t)(int)p.z;
    }
    __syncwarp();   // the slots and the staging area are rewritten by other lanes in the next round
  }
}

// ---------------------------------------------------------------- restore
// SMBWD: instead of the restored map y itself, write the softmax backward of it for the upstream gradient
// `grad`:  out = (g - sum_row(bf16(y * g))) * y  (operators/softmax_kernels.py:7-38: the product is a bf16
// operation, the row sum and the rest fp32).  The restored map never goes to HBM.
template <int QBIT, int LPR, bool SMBWD>
__global__ void __launch_bounds__(256, SMBWD ? 3 : HYC_LANE_MINB)      // SMBWD: two tiles per warp, 3 blocks fill the SM
topk_lane_restore_kernel(const __nv_bfloat16* __restrict__ val, const uint16_t* __restrict__ colv, int k, float inv_k,
                         const uint8_t* __restrict__ q, const __nv_bfloat16* __restrict__ scale,
                         const int8_t* __restrict__ zp, int64_t rows, const __nv_bfloat16* __restrict__ grad,
                         float oscale, __nv_bfloat16* __restrict__ ao) {
  constexpr int RPW = 32 / LPR;
  constexpr int S = 64 * LPR;
  constexpr int64_t QLD = (int64_t)S * QBIT / 8;
  constexpr int PRE = 4;                 // list entries per lane fetched before the de-quantization
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int lr = lane & (LPR - 1), rw = lane / LPR;
  // dynamic shared memory: per warp its rows (128 bytes per lane) and, SMBWD, a second tile for the gradient rows
  extern __shared__ __align__(16) uint32_t s_dyn[];
  uint32_t* s_xw = s_dyn + warp * 1024;
  uint32_t* s_gw = s_dyn + (nwarps + warp) * 1024;
  uint32_t* sx = s_xw + lane * 32;
  uint16_t* sw16 = reinterpret_cast<uint16_t*>(s_xw);
  const int64_t items = (rows + RPW - 1) / RPW;
  for (int64_t item = (int64_t)blockIdx.x * nwarps + warp; item < items; item += (int64_t)gridDim.x * nwarps) {
    const int64_t row0 = item * RPW, row = row0 + rw;
    const bool valid = row < rows;
    const int64_t left = rows - row0;
    const int n_rows = (int)(left < RPW ? left : RPW);
    const int n_ent = n_rows * k;
    // the gradient rows start their way into shared memory now and arrive while the map is being rebuilt
    if (SMBWD) lane_run_to_shared_async(grad + row0 * S, n_rows * (S / 16), s_gw, lane);
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
      lane_slot_store(sx, lane, o);
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
    if (SMBWD) {
      uint32_t yv[32], gv[32];
      lane_slot_load(sx, lane, yv);                       // the lane's own group of the restored row
      lane_async_wait();
      __syncwarp();
      lane_slot_load(s_gw + lane * 32, lane, gv);
      float acc = 0.f;
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const __nv_bfloat162 p = __hmul2_rn(*reinterpret_cast<const __nv_bfloat162*>(&yv[j]),
                                            *reinterpret_cast<const __nv_bfloat162*>(&gv[j]));
        acc += __bfloat162float(p.x) + __bfloat162float(p.y);
      }
#pragma unroll
      for (int o = 1; o < LPR; o <<= 1) acc += __shfl_xor_sync(kFull, acc, o);     // stays inside the row's lanes
#pragma unroll
      for (int j = 0; j < 32; ++j)
        gv[j] = pack_bf16x2_rn((bf16lo_to_f32(gv[j]) - acc) * bf16lo_to_f32(yv[j]),
                               (bf16hi_to_f32(gv[j]) - acc) * bf16hi_to_f32(yv[j]));
      if (oscale != 1.f) {        // a second bf16 operation on the result (the layer's `grad_s / sqrt(d)`)
#pragma unroll
        for (int j = 0; j < 32; ++j) gv[j] = pack_bf16x2_rn(bf16lo_to_f32(gv[j]) * oscale, bf16hi_to_f32(gv[j]) * oscale);
      }
      __syncwarp();
      lane_slot_store(sx, lane, gv);
      __syncwarp();
    }
    // the warp's rows leave as four fully coalesced 1 KB stores
    lane_shared_to_run(s_xw, ao + row0 * S, n_rows * (S / 16), lane);
    __syncwarp();
  }
}

// ---------------------------------------------------------------- softmax backward on dense maps
// out = (g - sum_row(bf16(y * g))) * y for rows of 64 * LPR columns, same layout and staging as above
template <int LPR>
__global__ void __launch_bounds__(256, 3)
softmax_bwd_lane_kernel(const __nv_bfloat16* __restrict__ y, const __nv_bfloat16* __restrict__ g, int64_t rows,
                        float oscale, __nv_bfloat16* __restrict__ out) {
  constexpr int RPW = 32 / LPR;
  constexpr int S = 64 * LPR;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  // dynamic shared memory: two 4 KB tiles per warp, so that both operands are on their way at once (cp.async)
  extern __shared__ __align__(16) uint32_t s_dyn[];
  uint32_t* s_yw = s_dyn + warp * 1024;
  uint32_t* s_gw = s_dyn + (nwarps + warp) * 1024;
  uint32_t* sx = s_yw + lane * 32;
  const int64_t items = (rows + RPW - 1) / RPW;
  for (int64_t item = (int64_t)blockIdx.x * nwarps + warp; item < items; item += (int64_t)gridDim.x * nwarps) {
    const int64_t row0 = item * RPW, left = rows - row0;
    const int n_pieces = (int)(left < RPW ? left : RPW) * (S / 16);
    uint32_t yv[32], gv[32];
    lane_run_to_shared_async(y + row0 * S, n_pieces, s_yw, lane);
    lane_run_to_shared_async(g + row0 * S, n_pieces, s_gw, lane);
    lane_async_wait();
    __syncwarp();
    lane_slot_load(sx, lane, yv);
    lane_slot_load(s_gw + lane * 32, lane, gv);
    float acc = 0.f;
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      const __nv_bfloat162 p = __hmul2_rn(*reinterpret_cast<const __nv_bfloat162*>(&yv[j]),
                                          *reinterpret_cast<const __nv_bfloat162*>(&gv[j]));
      acc += __bfloat162float(p.x) + __bfloat162float(p.y);
    }
#pragma unroll
    for (int o = 1; o < LPR; o <<= 1) acc += __shfl_xor_sync(kFull, acc, o);
#pragma unroll
    for (int j = 0; j < 32; ++j)
      gv[j] = pack_bf16x2_rn((bf16lo_to_f32(gv[j]) - acc) * bf16lo_to_f32(yv[j]),
                             (bf16hi_to_f32(gv[j]) - acc) * bf16hi_to_f32(yv[j]));
    if (oscale != 1.f) {
#pragma unroll
      for (int j = 0; j < 32; ++j) gv[j] = pack_bf16x2_rn(bf16lo_to_f32(gv[j]) * oscale, bf16hi_to_f32(gv[j]) * oscale);
    }
    __syncwarp();
    lane_slot_store(sx, lane, gv);
    __syncwarp();
    lane_shared_to_run(s_yw, out + row0 * S, n_pieces, lane);
    __syncwarp();
  }
}

template <int LPR>
static void launch_softmax_bwd(const void* y, const void* g, int64_t rows, float oscale, void* out, cudaStream_t st) {
  auto kern = softmax_bwd_lane_kernel<LPR>;
  static bool attr[64] = {false};      // up to 64 KB of dynamic shared memory per block: set per device
  const int slot = current_device_slot();
  if (slot < 0 || !attr[slot]) {
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 8 * 8192);
    if (slot >= 0) attr[slot] = true;
  }
  int grid, threads;
  lane_launch_shape(kern, rows, 32 / LPR, grid, threads, 8192);
  kern<<<grid, threads, (threads / 32) * 8192, st>>>((const __nv_bfloat16*)y, (const __nv_bfloat16*)g, rows, oscale,
                                                     (__nv_bfloat16*)out);
}

// rows of 64 * 2^n <= 2048 columns, 32-byte aligned tensors; false = not covered (nothing launched)
bool softmax_bwd_lane(const void* y, const void* g, int64_t rows, int S, float oscale, void* out, cudaStream_t st) {
  if (S < 64 || S > 2048 || (S & (S - 1)) != 0 || !aligned(y, 32) || !aligned(g, 32) || !aligned(out, 32)) return false;
  switch (S / 64) {
    case 1: launch_softmax_bwd<1>(y, g, rows, oscale, out, st); break;
    case 2: launch_softmax_bwd<2>(y, g, rows, oscale, out, st); break;
    case 4: launch_softmax_bwd<4>(y, g, rows, oscale, out, st); break;
    case 8: launch_softmax_bwd<8>(y, g, rows, oscale, out, st); break;
    case 16: launch_softmax_bwd<16>(y, g, rows, oscale, out, st); break;
    default: launch_softmax_bwd<32>(y, g, rows, oscale, out, st); break;
  }
  return true;
}

// ---------------------------------------------------------------- launchers
template <int QBIT, int LPR>
static void launch_compress(const void* a, int64_t rows, int k, void* val, uint16_t* col, void* q, void* scale,
                            int8_t* zp, const SoftmaxPrologue* sp, cudaStream_t st) {
  int grid, threads;
  if (sp == nullptr) {
    auto kern = topk_lane_compress_kernel<QBIT, LPR, false>;
    lane_launch_shape(kern, rows, 32 / LPR, grid, threads);
    kern<<<grid, threads, 0, st>>>((const __nv_bfloat16*)a, rows, k, (__nv_bfloat16*)val, col,
                                   (uint8_t*)q, (__nv_bfloat16*)scale, zp, SoftmaxPrologue{});
  } else {
    auto kern = topk_lane_compress_kernel<QBIT, LPR, true>;
    lane_launch_shape(kern, rows, 32 / LPR, grid, threads);
    kern<<<grid, threads, 0, st>>>((const __nv_bfloat16*)a, rows, k, (__nv_bfloat16*)val, col,
                                   (uint8_t*)q, (__nv_bfloat16*)scale, zp, *sp);
  }
}
template <int QBIT, int LPR>
static void launch_restore(const void* val, const uint16_t* col, int k, const void* q, const void* scale,
                           const int8_t* zp, int64_t rows, const void* grad, float oscale, void* ao, cudaStream_t st) {
  int grid, threads;
  if (grad == nullptr) {
    auto kern = topk_lane_restore_kernel<QBIT, LPR, false>;
    lane_launch_shape(kern, rows, 32 / LPR, grid, threads, 4096);
    kern<<<grid, threads, (threads / 32) * 4096, st>>>((const __nv_bfloat16*)val, col, k, k > 0 ? 1.0f / (float)k : 0.f,
                                   (const uint8_t*)q, (const __nv_bfloat16*)scale, zp, rows, nullptr, 1.f, (__nv_bfloat16*)ao);
  } else {
    auto kern = topk_lane_restore_kernel<QBIT, LPR, true>;
    // two 4 KB tiles per warp: up to 64 KB per block, above the default limit (set per device)
    static bool attr[64] = {false};
    const int slot = current_device_slot();
    if (slot < 0 || !attr[slot]) {
      cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 8 * 8192);
      if (slot >= 0) attr[slot] = true;
    }
    lane_launch_shape(kern, rows, 32 / LPR, grid, threads, 8192);
    kern<<<grid, threads, (threads / 32) * 8192, st>>>((const __nv_bfloat16*)val, col, k, k > 0 ? 1.0f / (float)k : 0.f,
                                   (const uint8_t*)q, (const __nv_bfloat16*)scale, zp, rows,
                                   (const __nv_bfloat16*)grad, oscale, (__nv_bfloat16*)ao);
  }
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
                      int8_t* zp, const SoftmaxPrologue* sp, cudaStream_t st) {
  HYC_LANE_DISPATCH(launch_compress, a, rows, k, val, col, q, scale, zp, sp, st);
  return HYC_OK;
}
template <int QB>
static int restore_q(const void* val, const uint16_t* col, int k, const void* q, const void* scale, const int8_t* zp,
                     int64_t rows, int S, const void* grad, float oscale, void* ao, cudaStream_t st) {
  HYC_LANE_DISPATCH(launch_restore, val, col, k, q, scale, zp, rows, grad, oscale, ao, st);
  return HYC_OK;
}

int topk_lane_compress(const void* a, int64_t rows, int S, int k, void* val_out, uint16_t* col_out,
                       void* q_out, void* scale_out, int8_t* zp_out, int q_bit, cudaStream_t st) {
  if (!topk_lane_ok(S, k)) return HYC_ERR_SHAPE;
  if (q_bit == 2) return compress_q<2>(a, rows, S, k, val_out, col_out, q_out, scale_out, zp_out, nullptr, st);
  if (q_bit == 4) return compress_q<4>(a, rows, S, k, val_out, col_out, q_out, scale_out, zp_out, nullptr, st);
  return compress_q<8>(a, rows, S, k, val_out, col_out, q_out, scale_out, zp_out, nullptr, st);
}

// scores [rows, S] -> probabilities (written to `dense`) and their saved form, one pass.  Covered: the shapes of
// topk_lane_ok with M a multiple of the rows a warp takes and mask rows S apart; HYC_ERR_UNSUPPORTED otherwise
// (nothing launched: the caller runs the softmax and the compress kernels one after the other).
int topk_lane_softmax_compress(const void* scores, float sc, const void* mask, int64_t mb, int64_t mh, int64_t mr, int heads,
                               int M, int64_t rows, int S, int k, void* dense, void* val_out, uint16_t* col_out,
                               void* q_out, void* scale_out, int8_t* zp_out, int q_bit, cudaStream_t st) {
  if (!topk_lane_ok(S, k)) return HYC_ERR_UNSUPPORTED;
  const int rpw = 32 / (S / 64);
  if (M % rpw != 0 || (mask != nullptr && mr != S) || !aligned(scores, 32) || !aligned(dense, 32) || !aligned(q_out, 32) ||
      (mask != nullptr && (!aligned(mask, 32) || (mb & 15) != 0 || (mh & 15) != 0)))
    return HYC_ERR_UNSUPPORTED;
  SoftmaxPrologue sp;
  sp.scale = sc; sp.mask = (const __nv_bfloat16*)mask; sp.mb = mb; sp.mh = mh; sp.heads = heads; sp.M = M;
  sp.dense = (__nv_bfloat16*)dense;
  if (q_bit == 2) return compress_q<2>(scores, rows, S, k, val_out, col_out, q_out, scale_out, zp_out, &sp, st);
  if (q_bit == 4) return compress_q<4>(scores, rows, S, k, val_out, col_out, q_out, scale_out, zp_out, &sp, st);
  return compress_q<8>(scores, rows, S, k, val_out, col_out, q_out, scale_out, zp_out, &sp, st);
}
int topk_lane_restore(const void* val, const uint16_t* col, int k, const void* q, const void* scale,
                      const int8_t* zp, int64_t rows, int S, const void* grad_or_null, float out_scale, void* a_out,
                      int q_bit, cudaStream_t st) {
  if (!topk_lane_ok(S, k)) return HYC_ERR_SHAPE;
  if (q_bit == 2) return restore_q<2>(val, col, k, q, scale, zp, rows, S, grad_or_null, out_scale, a_out, st);
  if (q_bit == 4) return restore_q<4>(val, col, k, q, scale, zp, rows, S, grad_or_null, out_scale, a_out, st);
  return restore_q<8>(val, col, k, q, scale, zp, rows, S, grad_or_null, out_scale, a_out, st);
}

}  // namespace hyc

// 64-wide group quantization and the per-row top-k attention-map path.
//
// One warp works on 512 consecutive columns of a row at a time ("step"): lane l holds the
// 16 consecutive columns [16 l, 16 l + 16) of the step as eight packed bf16 pairs (two
// 128-bit loads, 32 contiguous bytes per lane).  A group of 64 columns is four adjacent
// lanes, so group min/max needs two shuffle rounds.  In the reference byte layout the two
// halves of a 32-column block sit in the two lanes of a pair; one shuffle per pair
// exchanges the half-finished bytes.
//
// Top-k (attention map): the whole row (<= 4096 columns) stays in registers.  The k-th
// largest magnitude is found by bisection on the 15-bit bf16 magnitude pattern; each probe
// counts "magnitude >= candidate" with packed bf16x2 compares and one warp reduction.  The
// selected elements are emitted in ascending column order through a warp prefix scan.
#include "group_math.cuh"
#include "topk_lane.cuh"
#include "lane_group.cuh"

namespace hyc {

constexpr int kStageEntries = 256;   // outlier-list entries a warp stages in shared memory

// Quantize the 16 values of a lane and store them in the reference byte layout.
// qrow points at the packed row; `lane_g` = 32*step + lane (global lane index in the row).
template <int QBIT>
__device__ __forceinline__ void quant_store16(const uint32_t (&xw)[8], const GroupParams& p,
                                              uint8_t* __restrict__ qrow, int lane_g, bool valid) {
  uint32_t w[4];   // w[i] = codes 4i..4i+3, one per byte
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint32_t b[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int idx = 4 * i + e;
      float xf = (idx & 1) ? bf16hi_to_f32(xw[idx >> 1]) : bf16lo_to_f32(xw[idx >> 1]);
      b[e] = group_code_bits<QBIT>(xf, p);
    }
    // low bytes of b0..b3 -> one word
    w[i] = __byte_perm(__byte_perm(b[0], b[1], 0x0040), __byte_perm(b[2], b[3], 0x0040), 0x5410);
  }
  const uint32_t w0 = w[0], w1 = w[1], w2 = w[2], w3 = w[3];
  const bool odd = lane_g & 1;
  if (QBIT == 8) {
    if (valid) st_stream_v4(qrow + 16 * (int64_t)lane_g, make_uint4(w0, w1, w2, w3));
  } else if (QBIT == 4) {
    // even lane: columns 0..15 of the block (low nibbles); odd lane: columns 16..31 (high)
    uint32_t s0 = odd ? w0 : w2, s1 = odd ? w1 : w3;
    uint32_t r0 = __shfl_xor_sync(kFull, s0, 1), r1 = __shfl_xor_sync(kFull, s1, 1);
    uint2 o;
    if (!odd) { o.x = w0 | (r0 << 4); o.y = w1 | (r1 << 4); }   // bytes 0..7
    else      { o.x = r0 | (w2 << 4); o.y = r1 | (w3 << 4); }   // bytes 8..15
    if (valid) st_stream_v2(qrow + 8 * (int64_t)lane_g, o);
  } else {
    // byte j = c[j] | c[8+j]<<2 | c[16+j]<<4 | c[24+j]<<6 ; even lane holds c[0..15], odd c[16..31]
    uint32_t p0, p1;
    if (!odd) { p0 = w0 | (w2 << 2); p1 = w1 | (w3 << 2); }
    else      { p0 = (w0 << 4) | (w2 << 6); p1 = (w1 << 4) | (w3 << 6); }
    uint32_t send = odd ? p0 : p1;
    uint32_t recv = __shfl_xor_sync(kFull, send, 1);
    uint32_t o = (odd ? p1 : p0) | recv;   // even: bytes 0..3, odd: bytes 4..7
    if (valid) st_stream_u32(qrow + 4 * (int64_t)lane_g, o);
  }
}

// Load the packed codes of the lane's 16 columns and dequantize them:
// x_hat = bf16( (code - half - z) * s ).  (code - half - z) is an exact small integer.
//   q = 2, 4 : packed bf16x2: 0x4300 | code is the bf16 128 + code; subtract 128 + half, subtract z
//              (both exact), multiply by the scale (one rounding, like the reference's bf16 multiply).
//   q = 8    : through fp32 (codes reach 255): 0x4B000000 | code is 2^23 + code.
template <int QBIT>
__device__ __forceinline__ void load_dequant16(const uint8_t* __restrict__ qrow, int lane_g,
                                               float s, float z, uint32_t (&out)[8]) {
  constexpr uint32_t MASK = (1u << QBIT) - 1u;
  if (QBIT == 8) {
    const float off = 8388608.f + (float)(1 << (QBIT - 1)) + z;
    const uint4 v = ld_stream_v4(qrow + 16 * (int64_t)lane_g);
    const uint32_t b[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float f0 = (byte_to_magic_float(b[j >> 1], (2 * j) & 3) - off) * s;
      const float f1 = (byte_to_magic_float(b[j >> 1], ((2 * j) & 3) + 1) - off) * s;
      out[j] = pack_bf16x2_rn(f0, f1);
    }
  } else {
    constexpr uint32_t BM = MASK * 0x01010101u;
    constexpr uint32_t C1 = 0x4300u | (uint32_t)(1 << (QBIT - 1));      // bf16 bits of 128 + half
    const uint32_t c1 = C1 | (C1 << 16);
    const uint32_t zb = f32_to_bf16bits_rn(z), z2 = zb | (zb << 16);
    const uint32_t sb = f32_to_bf16bits_rn(s), s2 = sb | (sb << 16);
    uint32_t w[4];    // codes of columns 4i..4i+3, one per byte
    if (QBIT == 4) {
      const uint4 v = ld_stream_v4(qrow + 16 * (int64_t)(lane_g >> 1));
      const int sh = 4 * (lane_g & 1);          // even lane: low nibbles, odd lane: high nibbles
      w[0] = (v.x >> sh) & BM; w[1] = (v.y >> sh) & BM; w[2] = (v.z >> sh) & BM; w[3] = (v.w >> sh) & BM;
    } else {
      const uint2 v = ld_stream_v2(qrow + 8 * (int64_t)(lane_g >> 1));
      const int sh = 4 * (lane_g & 1);          // columns 0..7: field sh, columns 8..15: field sh + 2
      w[0] = (v.x >> sh) & BM; w[1] = (v.y >> sh) & BM; w[2] = (v.x >> (sh + 2)) & BM; w[3] = (v.y >> (sh + 2)) & BM;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const uint32_t pr = __byte_perm(w[j >> 1], 0x43434343u, (j & 1) ? 0x4342u : 0x4140u);
      __nv_bfloat162 t = __hsub2(*reinterpret_cast<const __nv_bfloat162*>(&pr), *reinterpret_cast<const __nv_bfloat162*>(&c1));
      t = __hsub2(t, *reinterpret_cast<const __nv_bfloat162*>(&z2));
      t = __hmul2(t, *reinterpret_cast<const __nv_bfloat162*>(&s2));
      out[j] = *reinterpret_cast<const uint32_t*>(&t);
    }
  }
}

__device__ __forceinline__ int warp_excl_scan(int v, int lane, int& total) {
  int incl = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    int t = __shfl_up_sync(kFull, incl, o);
    if (lane >= o) incl += t;
  }
  total = __shfl_sync(kFull, incl, 31);
  return incl - v;
}

// ---------------------------------------------------------------- group mode (activations)
// items = rows * steps_per_row, one warp per item.
template <int QBIT>
__global__ void __launch_bounds__(256)
group_quant_kernel(const __nv_bfloat16* __restrict__ x, int64_t rows, int N, int64_t ldx,
                   uint8_t* __restrict__ q, __nv_bfloat16* __restrict__ scale, int8_t* __restrict__ zp) {
  const int lane = threadIdx.x & 31;
  const int steps = (N + 511) / 512;
  const int64_t items = rows * steps;
  const int64_t qld = (int64_t)N * QBIT / 8, gld = N / 64;
  for (int64_t it = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5); it < items; it += (int64_t)gridDim.x * 8) {
    const int64_t row = it / steps;
    const int st = (int)(it % steps);
    const int lane_g = 32 * st + lane;
    const int col = 16 * lane_g;
    const bool valid = col < N;
    uint32_t xw[8];
    if (valid) {
      ld_stream_v8(x + row * ldx + col, xw);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) xw[j] = 0u;
    }
    float mn, mx;
    group_minmax(xw, mn, mx);
    GroupParams p = group_params<QBIT>(mn, mx);
    quant_store16<QBIT>(xw, p, q + row * qld, lane_g, valid);
    if (valid && (lane & 3) == 0) {
      scale[row * gld + (col >> 6)] = __ushort_as_bfloat16(f32_to_bf16bits_rn(p.s));
      zp[row * gld + (col >> 6)] = (int8_t)(int)p.z;
    }
  }
}

template <int QBIT>
__global__ void __launch_bounds__(256)
group_dequant_kernel(const uint8_t* __restrict__ q, int64_t rows, int N,
                     const __nv_bfloat16* __restrict__ scale, const int8_t* __restrict__ zp,
                     __nv_bfloat16* __restrict__ xo, int64_t ldx) {
  const int lane = threadIdx.x & 31;
  const int steps = (N + 511) / 512;
  const int64_t items = rows * steps;
  const int64_t qld = (int64_t)N * QBIT / 8, gld = N / 64;
  for (int64_t it = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5); it < items; it += (int64_t)gridDim.x * 8) {
    const int64_t row = it / steps;
    const int st = (int)(it % steps);
    const int lane_g = 32 * st + lane;
    const int col = 16 * lane_g;
    if (col < N) {
      float s = __bfloat162float(scale[row * gld + (col >> 6)]);
      float z = (float)zp[row * gld + (col >> 6)];
      uint32_t o[8];
      load_dequant16<QBIT>(q + row * qld, lane_g, s, z, o);
      st_stream_v8(xo + row * ldx + col, o);
    }
  }
}

// ---------------------------------------------------------------- group mode, contiguous rows
// With ldx == N the tensor is a flat list of groups; one lane per group, 32 consecutive groups (4 KB)
// per warp and round, moved through shared memory so that every global access is a full 1 KB run.
template <int QBIT>
__global__ void __launch_bounds__(256, HYC_LANE_MINB)
group_flat_quant_kernel(const __nv_bfloat16* __restrict__ x, int64_t n_groups, uint8_t* __restrict__ q,
                        __nv_bfloat16* __restrict__ scale, int8_t* __restrict__ zp) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  __shared__ __align__(16) uint32_t s_x[8][32 * 32];
  const int64_t items = (n_groups + 31) / 32;
  for (int64_t item = (int64_t)blockIdx.x * nwarps + warp; item < items; item += (int64_t)gridDim.x * nwarps) {
    const int64_t g0 = item * 32, left = n_groups - g0;
    const int nv = (int)(left < 32 ? left : 32);
    lane_run_to_shared(x + g0 * 64, nv * 4, s_x[warp], lane);
    __syncwarp();
    uint32_t xw[32];
    lane_slot_load(s_x[warp] + lane * 32, lane, xw);
    float mn, mx;
    lane_minmax(xw, mn, mx);
    const GroupParams p = group_params<QBIT>(mn, mx);
    if (lane < nv) {
      lane_quant_store<QBIT>(xw, p, q + (g0 + lane) * (64 * QBIT / 8));
      scale[g0 + lane] = __ushort_as_bfloat16(f32_to_bf16bits_rn(p.s));
      zp[g0 + lane] = (int8_t)(int)p.z;
    }
    __syncwarp();
  }
}

template <int QBIT>
__global__ void __launch_bounds__(256, HYC_LANE_MINB)
group_flat_dequant_kernel(const uint8_t* __restrict__ q, int64_t n_groups, const __nv_bfloat16* __restrict__ scale,
                          const int8_t* __restrict__ zp, __nv_bfloat16* __restrict__ xo) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  __shared__ __align__(16) uint32_t s_x[8][32 * 32];
  const int64_t items = (n_groups + 31) / 32;
  for (int64_t item = (int64_t)blockIdx.x * nwarps + warp; item < items; item += (int64_t)gridDim.x * nwarps) {
    const int64_t g0 = item * 32, left = n_groups - g0;
    const int nv = (int)(left < 32 ? left : 32);
    if (lane < nv) {
      const float s = __bfloat162float(scale[g0 + lane]);
      const float z = (float)zp[g0 + lane];
      uint32_t o[32];
      lane_load_dequant<QBIT>(q + (g0 + lane) * (64 * QBIT / 8), s, z, o);
      lane_slot_store(s_x[warp] + lane * 32, lane, o);
    }
    __syncwarp();
    lane_shared_to_run(s_x[warp], xo + g0 * 64, nv * 4, lane);
    __syncwarp();
  }
}

// ---------------------------------------------------------------- per-row top-k (attention map)
__device__ __forceinline__ __nv_bfloat162 as_bf162(uint32_t v) { return *reinterpret_cast<__nv_bfloat162*>(&v); }
__device__ __forceinline__ uint32_t as_u32(__nv_bfloat162 v) { return *reinterpret_cast<uint32_t*>(&v); }

// number of keys >= cand over the whole warp; keys are 15-bit magnitude patterns, which
// order like the positive bf16 values they spell, so packed bf16x2 compares count them
template <int NREG>
__device__ __forceinline__ int count_ge(const uint32_t (&m)[NREG], uint32_t cand) {
  const __nv_bfloat162 cb = as_bf162(cand | (cand << 16));
  __nv_bfloat162 acc = __float2bfloat162_rn(0.f);
#pragma unroll
  for (int j = 0; j < NREG; ++j) acc = __hadd2(acc, __hge2(as_bf162(m[j]), cb));
  int c = (int)(__bfloat162float(acc.x) + __bfloat162float(acc.y));
  return __reduce_add_sync(kFull, c);
}

template <int QBIT, int STEPS>
__global__ void __launch_bounds__(256)
topk_compress_kernel(const __nv_bfloat16* __restrict__ a, int64_t rows, int S, int k,
                     __nv_bfloat16* __restrict__ val_out, uint16_t* __restrict__ col_out,
                     uint8_t* __restrict__ q, __nv_bfloat16* __restrict__ scale, int8_t* __restrict__ zp) {
  const int lane = threadIdx.x & 31;
  const int64_t qld = (int64_t)S * QBIT / 8, gld = S / 64;
  __shared__ __align__(16) uint32_t s_x[8][32][8];          // the lane's 16 values, per warp
  __shared__ uint32_t s_out[8][kStageEntries];              // staged (column, value) words, per warp
  for (int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5); row < rows; row += (int64_t)gridDim.x * 8) {
    const __nv_bfloat16* arow = a + row * S;
    uint32_t xw[STEPS][8];
    uint32_t m[STEPS * 8];
#pragma unroll
    for (int st = 0; st < STEPS; ++st) {
      const int col = 16 * (32 * st + lane);
      if (col < S) {
        ld_stream_v8(arow + col, xw[st]);
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) xw[st][j] = 0u;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) m[st * 8 + j] = xw[st][j] & 0x7fff7fffu;
    }

    if (k > 0) {
      // ---- a lower bound from few candidates: the two largest keys of each of the lane's
      // 2*STEPS eight-element streams (the low and the high halves of the packed registers).
      // They are distinct elements of the row, so the k-th largest of them is <= the k-th
      // largest of the row, and usually equal to it.
      uint32_t cand[2 * STEPS];
      uint32_t lane_max = 0u;
#pragma unroll
      for (int st = 0; st < STEPS; ++st) {
        __nv_bfloat162 m1 = as_bf162(m[st * 8]), m2 = __float2bfloat162_rn(0.f);
#pragma unroll
        for (int j = 1; j < 8; ++j) {
          const __nv_bfloat162 v = as_bf162(m[st * 8 + j]);
          m2 = __hmax2(m2, __hmin2(m1, v));
          m1 = __hmax2(m1, v);
        }
        cand[2 * st] = as_u32(m1);
        cand[2 * st + 1] = as_u32(m2);
        const uint32_t c1 = as_u32(m1);
        lane_max = max(lane_max, max(c1 & 0xffffu, c1 >> 16));
      }
      const uint32_t U = __reduce_max_sync(kFull, lane_max);     // largest key of the row
      uint32_t L = 0u;
      if (k <= 128 * STEPS) {
        // bitwise bisection over the candidates: largest L with count_cand(>= L) >= k
        for (int bit = 14; bit >= 0; --bit) {
          const uint32_t c = L | (1u << bit);
          if (c > U) continue;
          const int cnt = count_ge<2 * STEPS>(cand, c);
          if (cnt >= k) { L = c; if (cnt == k) break; }
        }
      }
      // ---- exact threshold on the full row: largest T in [L, U] with count(>= T) >= k
      uint32_t T = L;
      int n_ge = count_ge<8 * STEPS>(m, L);
      // more than k keys >= L: either equal keys at L (then T = L and the tie rule decides), or a
      // stream held more than two of the k largest (rare; bisect on the whole row above L)
      if (n_ge > k) {
        const int n_gt = count_ge<8 * STEPS>(m, L + 1u);
        if (n_gt >= k) {
          uint32_t lo = L + 1u, hi = U + 1u;   // count(>= lo) >= k, count(>= hi) < k
          n_ge = n_gt;
          while (n_ge != k && hi - lo > 1u) {
            const uint32_t mid = (lo + hi) >> 1;
            const int cnt = count_ge<8 * STEPS>(m, mid);
            if (cnt >= k) { lo = mid; n_ge = cnt; } else { hi = mid; }
          }
          T = lo;
        }
      }
      // ---- selection masks (0xffff per selected half)
      const __nv_bfloat162 Tb = as_bf162(T | (T << 16));
      uint32_t sel[STEPS][8];
      if (n_ge == k) {
#pragma unroll
        for (int st = 0; st < STEPS; ++st)
#pragma unroll
          for (int j = 0; j < 8; ++j) sel[st][j] = __hge2_mask(as_bf162(m[st * 8 + j]), Tb);
      } else {
        // more than k keys are >= T: all keys > T, and the ties in ascending column order
        int need = k - count_ge<8 * STEPS>(m, T + 1u);
        int tie_base = 0;
#pragma unroll
        for (int st = 0; st < STEPS; ++st) {
          uint32_t eq[8];
          int neq = 0;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            eq[j] = __heq2_mask(as_bf162(m[st * 8 + j]), Tb);
            neq += __popc(eq[j]) >> 4;
          }
          int tot;
          int rank = tie_base + warp_excl_scan(neq, lane, tot);
          tie_base += tot;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            uint32_t take = 0u;
            if (eq[j] & 0xffffu) { if (rank < need) take |= 0xffffu; ++rank; }
            if (eq[j] >> 16) { if (rank < need) take |= 0xffff0000u; ++rank; }
            sel[st][j] = __hgt2_mask(as_bf162(m[st * 8 + j]), Tb) | take;
          }
        }
      }
      // ---- emit in ascending column order, then zero the selected positions.
      // The lane's registers are parked in shared memory so that the few selected elements can be
      // picked by index; (column << 16 | value bits) words are gathered per warp and written out
      // as one coalesced pass.  Lists longer than the staging area go straight to global memory.
      const bool staged = k <= kStageEntries;
      uint32_t* sx = s_x[threadIdx.x >> 5][lane];
      uint32_t* so = s_out[threadIdx.x >> 5];
      __nv_bfloat16* vrow = val_out + row * k;
      uint16_t* crow = col_out + row * k;
      int base = 0;
#pragma unroll
      for (int st = 0; st < STEPS; ++st) {
        // bit e: element e of this step is selected.  A mask register is 0xffff per selected
        // half, so bit 2j of its low half and bit 2j+1 of its high half are picked out.
        uint32_t acc = 0u;
#pragma unroll
        for (int j = 0; j < 8; ++j) acc |= sel[st][j] & ((1u << (2 * j)) | (1u << (17 + 2 * j)));
        uint32_t bits = (acc | (acc >> 16)) & 0xffffu;
        int tot;
        int slot = base + warp_excl_scan(__popc(bits), lane, tot);
        base += tot;
        *reinterpret_cast<uint4*>(sx) = make_uint4(xw[st][0], xw[st][1], xw[st][2], xw[st][3]);
        *reinterpret_cast<uint4*>(sx + 4) = make_uint4(xw[st][4], xw[st][5], xw[st][6], xw[st][7]);
        const uint32_t col0 = (uint32_t)(16 * (32 * st + lane));
        while (bits) {
          const int e = __ffs(bits) - 1;
          bits &= bits - 1u;
          const uint32_t v = reinterpret_cast<const uint16_t*>(sx)[e];
          if (slot < k) {
            if (staged) so[slot] = ((col0 + e) << 16) | v;
            else { vrow[slot] = __ushort_as_bfloat16((uint16_t)v); crow[slot] = (uint16_t)(col0 + e); }
          }
          ++slot;
        }
        __syncwarp();
#pragma unroll
        for (int j = 0; j < 8; ++j) xw[st][j] &= ~sel[st][j];
      }
      if (staged) {
        __syncwarp();
        for (int j = lane; j < k; j += 32) {
          const uint32_t w = so[j];
          vrow[j] = __ushort_as_bfloat16((uint16_t)(w & 0xffffu));
          crow[j] = (uint16_t)(w >> 16);
        }
        __syncwarp();
      }
    }

#pragma unroll
    for (int st = 0; st < STEPS; ++st) {
      const int lane_g = 32 * st + lane;
      const int col = 16 * lane_g;
      const bool valid = col < S;
      if (16 * 32 * st < S) {   // warp-uniform: the step holds at least one valid group
        float mn, mx;
        group_minmax(xw[st], mn, mx);
        GroupParams p = group_params<QBIT>(mn, mx);
        quant_store16<QBIT>(xw[st], p, q + row * qld, lane_g, valid);
        if (valid && (lane & 3) == 0) {
          scale[row * gld + (col >> 6)] = __ushort_as_bfloat16(f32_to_bf16bits_rn(p.s));
          zp[row * gld + (col >> 6)] = (int8_t)(int)p.z;
        }
      }
    }
  }
}

template <int QBIT>
__global__ void __launch_bounds__(256)
topk_restore_kernel(const __nv_bfloat16* __restrict__ val, const uint16_t* __restrict__ colv, int k,
                    const uint8_t* __restrict__ q, const __nv_bfloat16* __restrict__ scale,
                    const int8_t* __restrict__ zp, int64_t rows, int S, __nv_bfloat16* __restrict__ ao) {
  const int lane = threadIdx.x & 31;
  const int steps = (S + 511) / 512;
  const int64_t qld = (int64_t)S * QBIT / 8, gld = S / 64;
  for (int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5); row < rows; row += (int64_t)gridDim.x * 8) {
    // the outlier list of the row is fetched first so that its latency overlaps the de-quantization
    constexpr int PRE = 4;
    uint16_t pc[PRE], pv[PRE];
#pragma unroll
    for (int i = 0; i < PRE; ++i) {
      const int j = lane + 32 * i;
      pc[i] = 0; pv[i] = 0;
      if (j < k) { pc[i] = colv[row * k + j]; pv[i] = __bfloat16_as_ushort(val[row * k + j]); }
    }
    for (int st = 0; st < steps; ++st) {
      const int lane_g = 32 * st + lane;
      const int col = 16 * lane_g;
      if (col < S) {
        float s = __bfloat162float(scale[row * gld + (col >> 6)]);
        float z = (float)zp[row * gld + (col >> 6)];
        uint32_t o[8];
        load_dequant16<QBIT>(q + row * qld, lane_g, s, z, o);
        st_stream_v8(ao + row * S + col, o);
      }
    }
    __syncwarp();   // orders this warp's row stores before the overwrites below
#pragma unroll
    for (int i = 0; i < PRE; ++i) {
      const int j = lane + 32 * i;
      if (j < k) ao[row * S + pc[i]] = __ushort_as_bfloat16(pv[i]);
    }
    for (int j = lane + 32 * PRE; j < k; j += 32) ao[row * S + colv[row * k + j]] = val[row * k + j];
  }
}

static inline int warp_grid(int64_t items) {
  int64_t blocks = (items + 7) / 8;
  int64_t cap = (int64_t)num_sms() * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}

}  // namespace hyc

using namespace hyc;

static int check_group(const void* a, const void* b, int64_t rows, int N, int64_t ldx, int q_bit) {
  if (!a || !b) return HYC_ERR_NULL;
  if (q_bit != 2 && q_bit != 4 && q_bit != 8) return HYC_ERR_QBIT;
  if (rows < 0 || N <= 0 || N % 64 != 0 || ldx < N) return HYC_ERR_SHAPE;
  if (ldx % 16 != 0) return HYC_ERR_ALIGN;   // 256-bit row accesses
  return HYC_OK;
}

extern "C" HYC_API int hyc_group_quant_pack(const void* x, int64_t rows, int N, int64_t ldx,
                                    void* q_out, void* scale_out, int8_t* zp_out, int q_bit, void* stream) {
  int rc = check_group(x, q_out, rows, N, ldx, q_bit);
  if (rc) return rc;
  if (!scale_out || !zp_out) return HYC_ERR_NULL;
  if (!aligned(x, 32) || !aligned(q_out, 16)) return HYC_ERR_ALIGN;
  if (rows == 0) return HYC_OK;
  cudaStream_t st = (cudaStream_t)stream;
  if (ldx == N && aligned(q_out, 32)) {
    const int64_t n_groups = rows * (N / 64);
    int grid, threads;
#define GFQ(QB) do { auto kern = group_flat_quant_kernel<QB>; lane_launch_shape(kern, n_groups, 32, grid, threads); \
      kern<<<grid, threads, 0, st>>>((const __nv_bfloat16*)x, n_groups, (uint8_t*)q_out, (__nv_bfloat16*)scale_out, zp_out); } while (0)
    if (q_bit == 2) GFQ(2); else if (q_bit == 4) GFQ(4); else GFQ(8);
#undef GFQ
    HYC_CHECK_LAUNCH();
    return HYC_OK;
  }
  const int64_t items = rows * ((N + 511) / 512);
#define GQ(QB) group_quant_kernel<QB><<<warp_grid(items), 256, 0, st>>>((const __nv_bfloat16*)x, rows, N, ldx, \
      (uint8_t*)q_out, (__nv_bfloat16*)scale_out, zp_out)
  if (q_bit == 2) GQ(2); else if (q_bit == 4) GQ(4); else GQ(8);
#undef GQ
  HYC_CHECK_LAUNCH();
  return HYC_OK;
}

extern "C" HYC_API int hyc_group_unpack_dequant(const void* q, int64_t rows, int N,
                                        const void* scale, const int8_t* zp,
                                        void* x_out, int64_t ldx, int q_bit, void* stream) {
  int rc = check_group(q, x_out, rows, N, ldx, q_bit);
  if (rc) return rc;
  if (!scale || !zp) return HYC_ERR_NULL;
  if (!aligned(x_out, 32) || !aligned(q, 16)) return HYC_ERR_ALIGN;
  if (rows == 0) return HYC_OK;
  cudaStream_t st = (cudaStream_t)stream;
  if (ldx == N && aligned(q, 32)) {
    const int64_t n_groups = rows * (N / 64);
    int grid, threads;
#define GFD(QB) do { auto kern = group_flat_dequant_kernel<QB>; lane_launch_shape(kern, n_groups, 32, grid, threads); \
      kern<<<grid, threads, 0, st>>>((const uint8_t*)q, n_groups, (const __nv_bfloat16*)scale, zp, (__nv_bfloat16*)x_out); } while (0)
    if (q_bit == 2) GFD(2); else if (q_bit == 4) GFD(4); else GFD(8);
#undef GFD
    HYC_CHECK_LAUNCH();
    return HYC_OK;
  }
  const int64_t items = rows * ((N + 511) / 512);
#define GD(QB) group_dequant_kernel<QB><<<warp_grid(items), 256, 0, st>>>((const uint8_t*)q, rows, N, \
      (const __nv_bfloat16*)scale, zp, (__nv_bfloat16*)x_out, ldx)
  if (q_bit == 2) GD(2); else if (q_bit == 4) GD(4); else GD(8);
#undef GD
  HYC_CHECK_LAUNCH();
  return HYC_OK;
}

extern "C" HYC_API int hyc_softmax_fwd_topk_save(const void* scores, float scale, const void* mask_or_null, int64_t mask_stride_b,
                                                 int64_t mask_stride_h, int64_t mask_stride_row, int heads, int M,
                                                 int64_t rows, int S, int k, void* a_out, void* val_out, uint16_t* col_out,
                                                 void* q_out, void* scale_out, int8_t* zp_out, int q_bit, void* stream) {
  if (!scores || !a_out || !q_out || !scale_out || !zp_out) return HYC_ERR_NULL;
  if (k > 0 && (!val_out || !col_out)) return HYC_ERR_NULL;
  if (q_bit != 2 && q_bit != 4 && q_bit != 8) return HYC_ERR_QBIT;
  if (rows < 0 || S <= 0 || S % 64 != 0 || k < 0 || k > S || heads < 1 || M < 1 || rows % M != 0) return HYC_ERR_SHAPE;
  if (rows == 0) return HYC_OK;
  const int rc = topk_lane_softmax_compress(scores, scale, mask_or_null, mask_stride_b, mask_stride_h, mask_stride_row, heads, M,
                                            rows, S, k, a_out, val_out, col_out, q_out, scale_out, zp_out, q_bit,
                                            (cudaStream_t)stream);
  if (rc) return rc;
  HYC_CHECK_LAUNCH();
  return HYC_OK;
}

extern "C" HYC_API int hyc_softmax_topk_compress(const void* a, int64_t rows, int S, int k,
                                         void* val_out, uint16_t* col_out,
                                         void* q_out, void* scale_out, int8_t* zp_out, int q_bit, void* stream) {
  if (!a || !q_out || !scale_out || !zp_out) return HYC_ERR_NULL;
  if (k > 0 && (!val_out || !col_out)) return HYC_ERR_NULL;
  if (q_bit != 2 && q_bit != 4 && q_bit != 8) return HYC_ERR_QBIT;
  if (rows < 0 || S <= 0 || S % 64 != 0 || S > 4096 || k < 0 || k > S) return HYC_ERR_SHAPE;
  if (!aligned(a, 32) || !aligned(q_out, 16)) return HYC_ERR_ALIGN;
  if (rows == 0) return HYC_OK;
  cudaStream_t st = (cudaStream_t)stream;
  if (topk_lane_ok(S, k) && aligned(q_out, 32)) {
    const int rc = topk_lane_compress(a, rows, S, k, val_out, col_out, q_out, scale_out, zp_out, q_bit, st);
    if (rc) return rc;
    HYC_CHECK_LAUNCH();
    return HYC_OK;
  }
  const int steps = (S + 511) / 512;
  const int grid = warp_grid(rows);
#define TK(QB, ST) topk_compress_kernel<QB, ST><<<grid, 256, 0, st>>>((const __nv_bfloat16*)a, rows, S, k, \
      (__nv_bfloat16*)val_out, col_out, (uint8_t*)q_out, (__nv_bfloat16*)scale_out, zp_out)
#define TKQ(QB) do { if (steps <= 1) TK(QB, 1); else if (steps <= 2) TK(QB, 2); else if (steps <= 4) TK(QB, 4); else TK(QB, 8); } while (0)
  if (q_bit == 2) TKQ(2); else if (q_bit == 4) TKQ(4); else TKQ(8);
#undef TKQ
#undef TK
  HYC_CHECK_LAUNCH();
  return HYC_OK;
}

extern "C" HYC_API int hyc_softmax_topk_restore(const void* val, const uint16_t* col, int k,
                                        const void* q, const void* scale, const int8_t* zp,
                                        int64_t rows, int S, void* a_out, int q_bit, void* stream) {
  if (!q || !scale || !zp || !a_out) return HYC_ERR_NULL;
  if (k > 0 && (!val || !col)) return HYC_ERR_NULL;
  if (q_bit != 2 && q_bit != 4 && q_bit != 8) return HYC_ERR_QBIT;
  if (rows < 0 || S <= 0 || S % 64 != 0 || S > 4096 || k < 0 || k > S) return HYC_ERR_SHAPE;
  if (!aligned(a_out, 32) || !aligned(q, 16)) return HYC_ERR_ALIGN;
  if (rows == 0) return HYC_OK;
  cudaStream_t st = (cudaStream_t)stream;
  if (topk_lane_ok(S, k) && aligned(q, 32)) {
    const int rc = topk_lane_restore(val, col, k, q, scale, zp, rows, S, nullptr, 1.f, a_out, q_bit, st);
    if (rc) return rc;
    HYC_CHECK_LAUNCH();
    return HYC_OK;
  }
#define TR(QB) topk_restore_kernel<QB><<<warp_grid(rows), 256, 0, st>>>((const __nv_bfloat16*)val, col, k, \
      (const uint8_t*)q, (const __nv_bfloat16*)scale, zp, rows, S, (__nv_bfloat16*)a_out)
  if (q_bit == 2) TR(2); else if (q_bit == 4) TR(4); else TR(8);
#undef TR
  HYC_CHECK_LAUNCH();
  return HYC_OK;
}

extern "C" HYC_API int hyc_softmax_topk_restore_bwd(const void* val, const uint16_t* col, int k,
                                                    const void* q, const void* scale, const int8_t* zp,
                                                    int64_t rows, int S, const void* grad, void* out, int q_bit,
                                                    float out_scale, void* stream) {
  if (!q || !scale || !zp || !grad || !out) return HYC_ERR_NULL;
  if (k > 0 && (!val || !col)) return HYC_ERR_NULL;
  if (q_bit != 2 && q_bit != 4 && q_bit != 8) return HYC_ERR_QBIT;
  if (rows < 0 || S <= 0 || S % 64 != 0 || S > 4096 || k < 0 || k > S) return HYC_ERR_SHAPE;
  if (!aligned(out, 32) || !aligned(grad, 32) || !aligned(q, 16)) return HYC_ERR_ALIGN;
  if (!topk_lane_ok(S, k) || !aligned(q, 32)) return HYC_ERR_UNSUPPORTED;   // caller: restore, then hyc_softmax_bwd
  if (rows == 0) return HYC_OK;
  const int rc = topk_lane_restore(val, col, k, q, scale, zp, rows, S, grad, out_scale, out, q_bit, (cudaStream_t)stream);
  if (rc) return rc;
  HYC_CHECK_LAUNCH();
  return HYC_OK;
}

// Device helpers of the "one lane = one group of 64 columns" kernels (group mode and per-row top-k).
//
// A warp works on 32 consecutive groups = one contiguous run of 4 KB of bf16 data.  The run moves between
// global and shared memory as four fully coalesced 1 KB accesses (lane t handles the 32-byte piece 32 i + t);
// in shared memory every lane owns a 128-byte slot whose 16-byte chunks are rotated by the lane number, so
// that both the piece-wise and the slot-wise 128-bit accesses are free of bank conflicts.
#pragma once
#include "group_math.cuh"

#ifndef HYC_LANE_MINB
#define HYC_LANE_MINB 4      // resident blocks per SM the lane kernels are compiled for (register cap 64)
#endif

namespace hyc {

// address (in 32-bit words) of 16-byte chunk c of a lane's 128-byte slot: chunks are rotated by the
// lane number so that 128-bit accesses of eight adjacent lanes fall on distinct banks
__device__ __forceinline__ int park_chunk(int c, int lane) { return ((c ^ (lane & 7)) << 2); }

__device__ __forceinline__ uint32_t mad_u32(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("mad.lo.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}

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
  // group_code_bits leaves 0x4B000000 + code.  Four of them are merged with integer multiply-adds (the
  // FMA pipe; the logic pipe is the busy one here): b0 + (b1 << 8) + (b2 << 16) + (b3 << 24) keeps one
  // 0x4B000000, the others are shifted out.  w[i] = 0x4B000000 + codes of columns 4i..4i+3, one per byte.
  uint32_t w[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const uint32_t b0 = group_code_bits<QBIT>(bf16lo_to_f32(xw[2 * i]), p);
    const uint32_t b1 = group_code_bits<QBIT>(bf16hi_to_f32(xw[2 * i]), p);
    const uint32_t b2 = group_code_bits<QBIT>(bf16lo_to_f32(xw[2 * i + 1]), p);
    const uint32_t b3 = group_code_bits<QBIT>(bf16hi_to_f32(xw[2 * i + 1]), p);
    w[i] = mad_u32(mad_u32(b3, 256u, b2), 65536u, mad_u32(b1, 256u, b0));
  }
  if (QBIT == 8) {
#pragma unroll
    for (int i = 0; i < 16; ++i) w[i] -= 0x4B000000u;
#pragma unroll
    for (int i = 0; i < 2; ++i) st_stream_v8(qgroup + 32 * i, *reinterpret_cast<const uint32_t(*)[8]>(&w[8 * i]));
  } else if (QBIT == 4) {
    // block h: byte j = code[j] | code[16 + j] << 4; the two offsets add up to 17 * 0x4B000000 = 0xFB000000
    uint32_t o[8];
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
      for (int i = 0; i < 4; ++i) o[4 * h + i] = mad_u32(w[8 * h + 4 + i], 16u, w[8 * h + i]) + 0x05000000u;
    st_stream_v8(qgroup, o);
  } else {
    // block h: byte j = code[j] | code[8 + j] << 2 | code[16 + j] << 4 | code[24 + j] << 6
    // the four offsets add up to 85 * 0x4B000000 = 0xE7000000 (mod 2^32)
    uint32_t o[4];
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
      for (int i = 0; i < 2; ++i)
        o[2 * h + i] = mad_u32(mad_u32(w[8 * h + 6 + i], 4u, w[8 * h + 4 + i]), 16u, mad_u32(w[8 * h + 2 + i], 4u, w[8 * h + i])) + 0x19000000u;
    st_stream_v4(qgroup, make_uint4(o[0], o[1], o[2], o[3]));
  }
}

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

// global -> shared: pieces [0, n_pieces) of the run, zeros beyond (slots = the warp's 32 x 32 words)
__device__ __forceinline__ void lane_run_to_shared(const __nv_bfloat16* __restrict__ run, int n_pieces, uint32_t* slots, int lane) {
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
    uint32_t* dst = slots + owner * 32;
    *reinterpret_cast<uint4*>(dst + park_chunk(c0, owner)) = make_uint4(t[0], t[1], t[2], t[3]);
    *reinterpret_cast<uint4*>(dst + park_chunk(c0 + 1, owner)) = make_uint4(t[4], t[5], t[6], t[7]);
  }
}
// global -> shared without passing through registers (cp.async): the same placement as lane_run_to_shared.  The
// copy is in flight while the warp does other work; lane_async_wait() + __syncwarp() before the slots are read.
__device__ __forceinline__ void lane_run_to_shared_async(const __nv_bfloat16* __restrict__ run, int n_pieces, uint32_t* slots, int lane) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int p = 32 * i + lane;
    const int owner = p >> 2, c0 = 2 * (p & 3);
    uint32_t* dst = slots + owner * 32;
    const bool in = p < n_pieces;
    const __nv_bfloat16* src = run + 16 * (in ? p : 0);
    const int nbytes = in ? 16 : 0;                 // 0: the 16 bytes are filled with zeros
    const uint32_t d0 = (uint32_t)__cvta_generic_to_shared(dst + park_chunk(c0, owner));
    const uint32_t d1 = (uint32_t)__cvta_generic_to_shared(dst + park_chunk(c0 + 1, owner));
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d0), "l"(src), "r"(nbytes) : "memory");
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d1), "l"(src + 8), "r"(nbytes) : "memory");
  }
  asm volatile("cp.async.commit_group;" ::: "memory");
}
__device__ __forceinline__ void lane_async_wait() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }
// shared -> global
__device__ __forceinline__ void lane_shared_to_run(const uint32_t* slots, __nv_bfloat16* __restrict__ run, int n_pieces, int lane) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int p = 32 * i + lane;
    const int owner = p >> 2, c0 = 2 * (p & 3);
    const uint32_t* src = slots + owner * 32;
    const uint4 t0 = *reinterpret_cast<const uint4*>(src + park_chunk(c0, owner));
    const uint4 t1 = *reinterpret_cast<const uint4*>(src + park_chunk(c0 + 1, owner));
    const uint32_t t[8] = {t0.x, t0.y, t0.z, t0.w, t1.x, t1.y, t1.z, t1.w};
    if (p < n_pieces) st_stream_v8(run + 16 * p, t);
  }
}
// the lane's own slot <-> registers
__device__ __forceinline__ void lane_slot_load(const uint32_t* sx, int lane, uint32_t (&xw)[32]) {
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    const uint4 t = *reinterpret_cast<const uint4*>(sx + park_chunk(c, lane));
    xw[4 * c] = t.x; xw[4 * c + 1] = t.y; xw[4 * c + 2] = t.z; xw[4 * c + 3] = t.w;
  }
}
__device__ __forceinline__ void lane_slot_store(uint32_t* sx, int lane, const uint32_t (&o)[32]) {
#pragma unroll
  for (int c = 0; c < 8; ++c)
    *reinterpret_cast<uint4*>(sx + park_chunk(c, lane)) = make_uint4(o[4 * c], o[4 * c + 1], o[4 * c + 2], o[4 * c + 3]);
}

// Grid and block width.  Every warp walks the items (groups of 32 / LPR rows) with a fixed stride, so the
// kernel ends when the busiest warp ends: with R resident warps on the GPU the efficiency is
// items / (ceil(items / R) * R).  The block width (5..8 warps) is picked to make that largest.
template <typename K>
inline void lane_launch_shape(K kern, int64_t rows, int rows_per_warp, int& grid, int& threads, int smem_per_warp = 0) {
  const int64_t items = (rows + rows_per_warp - 1) / rows_per_warp;
  double best = -1.0;
  grid = 1; threads = 256;
  for (int w = 8; w >= 5; --w) {
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, 32 * w, (size_t)w * smem_per_warp) != cudaSuccess || per_sm < 1) per_sm = 1;
    const int64_t resident = (int64_t)num_sms() * per_sm * w;
    int64_t blocks = (items + w - 1) / w;
    if (blocks > (int64_t)num_sms() * per_sm) blocks = (int64_t)num_sms() * per_sm;
    const int64_t rounds = (items + resident - 1) / resident;
    const double eff = items <= resident ? 1.0 + 1e-3 * w : (double)items / (double)(rounds * resident);
    if (eff > best + 1e-9) { best = eff; grid = (int)(blocks < 1 ? 1 : blocks); threads = 32 * w; }
  }
}

}  // namespace hyc

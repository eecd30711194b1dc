// Per-channel codes of ONE OCTET (eight consecutive columns, 16 bytes of bf16) of a row, for kernels whose
// threads own octets: adjacent lanes own adjacent octets, so the four lanes that share a 32-column block of
// the reference byte layout (byte j = columns j, j + 32/epp, ... at rising bit positions) are lanes
// 4m .. 4m+3 of a warp and combine their bit fields with butterfly shuffles.
#pragma once
#include "hyc_common.cuh"

namespace hyc {

// Quantize the octet (four packed bf16 pairs) with the per-column scales `sv` (eight packed bf16) and return
// one code per byte.  Bit e of `zero_mask` forces column e to encode as zero (an outlier column).
template <int QBIT>
__device__ __forceinline__ void octet_quant(const uint32_t (&xw)[4], const uint4& sv, uint32_t zero_mask, uint32_t (&k)[2]) {
  const uint32_t sw[4] = {sv.x, sv.y, sv.z, sv.w};
  uint32_t b[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    const float xf = (e & 1) ? bf16hi_to_f32(xw[e >> 1]) : bf16lo_to_f32(xw[e >> 1]);
    const float sf = (e & 1) ? bf16hi_to_f32(sw[e >> 1]) : bf16lo_to_f32(sw[e >> 1]);
    float rcs = fastq_scale<QBIT>(__frcp_rn(sf));
    if ((zero_mask >> e) & 1u) rcs = 0.f;
    b[e] = fastq_code_bits<QBIT>(xf, rcs);
  }
  k[0] = gather_low_bytes(b[0], b[1], b[2], b[3]);
  k[1] = gather_low_bytes(b[4], b[5], b[6], b[7]);
}

// The same with the per-column constants already formed (fastq_scale of the reciprocal; 0 = encode as zero)
template <int QBIT>
__device__ __forceinline__ void octet_quant_rcs(const uint32_t (&xw)[4], const float (&rcs)[8], uint32_t (&k)[2]) {
  uint32_t b[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    const float xf = (e & 1) ? bf16hi_to_f32(xw[e >> 1]) : bf16lo_to_f32(xw[e >> 1]);
    b[e] = fastq_code_bits<QBIT>(xf, rcs[e]);
  }
  k[0] = gather_low_bytes(b[0], b[1], b[2], b[3]);
  k[1] = gather_low_bytes(b[4], b[5], b[6], b[7]);
}
template <int QBIT>
__device__ __forceinline__ void octet_rcs(const uint4& sv, uint32_t zero_mask, float (&rcs)[8]) {
  const uint32_t sw[4] = {sv.x, sv.y, sv.z, sv.w};
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    const float sf = (e & 1) ? bf16hi_to_f32(sw[e >> 1]) : bf16lo_to_f32(sw[e >> 1]);
    rcs[e] = ((zero_mask >> e) & 1u) ? 0.f : fastq_scale<QBIT>(__frcp_rn(sf));
  }
}

// Store the codes of the octet that starts at column `col` (a multiple of 8) of the packed row `qrow`.
// EVERY lane of the warp must call this (shuffles); `ok` = this lane's octet exists.
template <int QBIT>
__device__ __forceinline__ void octet_store(uint8_t* __restrict__ qrow, int col, const uint32_t (&k)[2], bool ok) {
  const int blk = col >> 5, cg = (col >> 3) & 3;
  if (QBIT == 8) {
    if (ok) st_stream_v2(qrow + col, make_uint2(k[0], k[1]));
  } else if (QBIT == 4) {
    // octets 0, 1: low nibbles of bytes 0..7, 8..15; octets 2, 3: high nibbles of the same bytes
    const int sh = 4 * (cg >> 1);
    uint32_t p0 = ok ? (k[0] << sh) : 0u, p1 = ok ? (k[1] << sh) : 0u;
    p0 |= __shfl_xor_sync(0xffffffffu, p0, 2);
    p1 |= __shfl_xor_sync(0xffffffffu, p1, 2);
    if (ok && cg < 2) st_stream_v2(qrow + 16 * blk + 8 * cg, make_uint2(p0, p1));
  } else {
    // octet cg supplies bit field cg of bytes 0..7
    const int sh = 2 * cg;
    uint32_t p0 = ok ? (k[0] << sh) : 0u, p1 = ok ? (k[1] << sh) : 0u;
    p0 |= __shfl_xor_sync(0xffffffffu, p0, 1); p0 |= __shfl_xor_sync(0xffffffffu, p0, 2);
    p1 |= __shfl_xor_sync(0xffffffffu, p1, 1); p1 |= __shfl_xor_sync(0xffffffffu, p1, 2);
    if (ok && cg == 0) st_stream_v2(qrow + 8 * blk, make_uint2(p0, p1));
  }
}

// Load and de-quantize the octet at column `col`: x_hat = bf16((code - half) * scale) as four packed pairs
// (exact: see unpack_dequant_kernel).  No shuffles; partner lanes read the same bytes.
template <int QBIT>
__device__ __forceinline__ void octet_load_dequant(const uint8_t* __restrict__ qrow, int col, const uint4& sv, uint32_t (&out)[4]) {
  constexpr uint32_t BM = ((1u << QBIT) - 1u) * 0x01010101u;
  const int blk = col >> 5, cg = (col >> 3) & 3;
  const uint32_t sw[4] = {sv.x, sv.y, sv.z, sv.w};
  uint2 a;
  int sh;
  if (QBIT == 8) { a = ld_stream_v2(qrow + col); sh = 0; }
  else if (QBIT == 4) { a = ld_stream_v2(qrow + 16 * blk + 8 * (cg & 1)); sh = 4 * (cg >> 1); }
  else { a = ld_stream_v2(qrow + 8 * blk); sh = 2 * cg; }
  const uint32_t k[2] = {(a.x >> sh) & BM, (a.y >> sh) & BM};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const uint32_t w = k[j >> 1];
    if (QBIT == 8) {
      const float f0 = (byte_to_magic_float(w, (2 * j) & 3) - 8388736.f) * bf16lo_to_f32(sw[j]);
      const float f1 = (byte_to_magic_float(w, ((2 * j) & 3) + 1) - 8388736.f) * bf16hi_to_f32(sw[j]);
      out[j] = pack_bf16x2_rn(f0, f1);
    } else {
      constexpr uint32_t C1 = 0x4300u | (uint32_t)(1 << (QBIT - 1));
      const uint32_t c1 = C1 | (C1 << 16);
      const uint32_t pr = __byte_perm(w, 0x43434343u, (j & 1) ? 0x4342u : 0x4140u);
      __nv_bfloat162 t = __hsub2_rn(*reinterpret_cast<const __nv_bfloat162*>(&pr), *reinterpret_cast<const __nv_bfloat162*>(&c1));
      t = __hmul2_rn(t, *reinterpret_cast<const __nv_bfloat162*>(&sw[j]));
      out[j] = *reinterpret_cast<const uint32_t*>(&t);
    }
  }
}

}  // namespace hyc

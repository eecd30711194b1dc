// Shared device helpers for the HyC activation-compression kernels (sm_100a).
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include "../../include/hyc.h"

#define HYC_CHECK_LAUNCH()                                                     \
  do {                                                                         \
    cudaError_t e__ = cudaGetLastError();                                      \
    if (e__ != cudaSuccess) { hyc_set_last_cuda_error((int)e__); return HYC_ERR_LAUNCH; } \
  } while (0)

#define HYC_API __attribute__((visibility("default")))
extern "C" HYC_API void hyc_set_last_cuda_error(int e);

namespace hyc {

// Multiprocessor count of the current device (launch geometry), asked once per device.  The cache is written
// without a lock: concurrent callers store the same value.
inline int num_sms() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n < 1) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}
// index of the current device for per-device one-time set-up (-1: no device)
inline int current_device_slot() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -1;
  return dev;
}

__host__ __device__ inline bool aligned(const void* p, size_t a) {
  return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0;
}

// ---- bf16 <-> f32 bit tricks -------------------------------------------------
__device__ __forceinline__ float bf16lo_to_f32(uint32_t packed) { return __uint_as_float(packed << 16); }
__device__ __forceinline__ float bf16hi_to_f32(uint32_t packed) { return __uint_as_float(packed & 0xffff0000u); }
__device__ __forceinline__ float bf16bits_to_f32(uint16_t b) { return __uint_as_float(((uint32_t)b) << 16); }

// round-to-nearest-even f32 pair -> packed bf16x2 (lo = a, hi = b)
__device__ __forceinline__ uint32_t pack_bf16x2_rn(float a, float b) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(b), "f"(a));
  return r;
}
__device__ __forceinline__ uint16_t f32_to_bf16bits_rn(float a) {
  return (uint16_t)(pack_bf16x2_rn(a, 0.f) & 0xffffu);
}

// ---- exact quotient ----------------------------------------------------------
// RN(x / s) from a correctly rounded reciprocal rc = RN(1/s): one multiply and two
// fused multiply-adds give the IEEE quotient (checked exhaustively on the host over all
// bf16 operand pairs; results that differ sit far below 1e-20 and cannot change a code).
// Domain: |x / s| must stay below the fp32 range (an overflowing first estimate would turn
// into a NaN); every caller clamps the result to the code range.  rc == 0 yields exactly 0.
__device__ __forceinline__ float quotient_rn(float x, float s, float rc) {
  float q0 = x * rc;
  float rem = fmaf(-q0, s, x);
  return fmaf(rem, rc, q0);
}

// C roundf (halves away from zero) of a value already clamped to [-2^(q-1), 2^(q-1)-1],
// returned as a signed integer.  RZ(r + copysign(0.5, r)) followed by truncation never
// rounds across an integer, so 0.49999997 -> 0.
__device__ __forceinline__ int round_half_away_i(float r) {
  float h = __uint_as_float((__float_as_uint(r) & 0x80000000u) | 0x3f000000u);
  return __float2int_rz(__fadd_rz(r, h));
}

template <int QBIT>
__device__ __forceinline__ int quant_code_signed(float x, float s, float rc) {
  constexpr float lo = -(float)(1 << (QBIT - 1));
  constexpr float hi = (float)((1 << (QBIT - 1)) - 1);
  float r = quotient_rn(x, s, rc);
  r = fminf(fmaxf(r, lo), hi);
  return round_half_away_i(r);
}
template <int QBIT>
__device__ __forceinline__ int quant_code_signed_zp(float x, float s, float rc, float z) {
  constexpr float lo = -(float)(1 << (QBIT - 1));
  constexpr float hi = (float)((1 << (QBIT - 1)) - 1);
  float r = quotient_rn(x, s, rc) + z;
  r = fminf(fmaxf(r, lo), hi);
  return round_half_away_i(r);
}

// ---- fast exact per-channel quantizer (no zero point) ---------------------------
// code = clamp(roundf(RN(x / s)), -2^(q-1), 2^(q-1)-1) + 2^(q-1) without a division, a clamp pair
// or a float->int conversion.  Why it is exact: x and s are bf16 (8-bit significands), so a
// quotient that is not exactly a half-integer stays at least 1/510 away from every half-integer,
// while an exact half-integer quotient is reproduced by x * RN(1/s) to within 2^-23 relative.
// Multiplying by (1 + delta) pushes ties away from zero (C roundf) by more than that error and
// moves every other value by far less than 1/510; round-to-nearest then gives the reference code.
// Checked exhaustively on the host over all bf16 scale significands and all bf16 inputs.
//   q = 2, 4 : u = sat(fma(x, rcs, 2^(q-1)/L)),  rcs = RN(1/s) * (1 + 2^-16) / L,  L = 2^q - 1,
//              code = low mantissa bits of fma(u, L, 2^23).  Saturation at 0 and 1 IS the clamp to
//              [-2^(q-1), 2^(q-1)-1]; the inexact constants cost < 1e-6 code units, far inside the margin.
//   q = 8    : t = clamp(x * rc, -128, 127),  code = low byte of fma(t, 1 + 2^-18, 1.5 * 2^23) ^ 0x80
// A column with rcs == 0 (outlier column) encodes as zero.
template <int QBIT>
__device__ __forceinline__ float fastq_scale(float rc) {
  if (QBIT == 8) return rc;
  return rc * ((1.0f + 1.0f / 65536.0f) / (float)((1 << QBIT) - 1));
}
// offset-binary code in the low byte of the returned word (upper bits are not zero)
template <int QBIT>
__device__ __forceinline__ uint32_t fastq_code_bits(float x, float rcs) {
  if (QBIT == 8) {
    const float t = fminf(fmaxf(x * rcs, -128.f), 127.f);
    return __float_as_uint(fmaf(t, 1.0f + 1.0f / 262144.0f, 12582912.f)) ^ 0x80u;
  } else {
    constexpr float L = (float)((1 << QBIT) - 1);
    constexpr float C2 = (float)(1 << (QBIT - 1)) / L;
    float u;
    asm("fma.rn.sat.f32 %0, %1, %2, %3;" : "=f"(u) : "f"(x), "f"(rcs), "f"(C2));
    return __float_as_uint(fmaf(u, L, 8388608.f));
  }
}
// low bytes of four words -> one word (byte k = low byte of bk)
__device__ __forceinline__ uint32_t gather_low_bytes(uint32_t b0, uint32_t b1, uint32_t b2, uint32_t b3) {
  return __byte_perm(__byte_perm(b0, b1, 0x0040), __byte_perm(b2, b3, 0x0040), 0x5410);
}
// byte k (0..3) of w as the float 2^23 + byte
__device__ __forceinline__ float byte_to_magic_float(uint32_t w, int k) {
  return __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7540u + (uint32_t)k));
}

// ---- streaming 128-bit / 64-bit global access --------------------------------
__device__ __forceinline__ uint4 ld_stream_v4(const void* p) {
  uint4 v;
  asm volatile("ld.global.cs.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ uint2 ld_stream_v2(const void* p) {
  uint2 v;
  asm volatile("ld.global.cs.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
  return v;
}
__device__ __forceinline__ uint32_t ld_stream_u32(const void* p) {
  uint32_t v;
  asm volatile("ld.global.cs.u32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}
// 256-bit accesses (sm_100): p must be 32-byte aligned
__device__ __forceinline__ void ld_stream_v8(const void* p, uint32_t (&v)[8]) {
  asm volatile("ld.global.cs.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]) : "l"(p));
}
__device__ __forceinline__ void st_stream_v8(void* p, const uint32_t (&v)[8]) {
  asm volatile("st.global.cs.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]),
               "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]) : "memory");
}
__device__ __forceinline__ void st_stream_v4(void* p, uint4 v) {
  asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ void st_stream_v2(void* p, uint2 v) {
  asm volatile("st.global.cs.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(v.x), "r"(v.y) : "memory");
}
__device__ __forceinline__ void st_stream_u32(void* p, uint32_t v) {
  asm volatile("st.global.cs.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Pack eight signed codes (two's complement, low QBIT bits significant) held as the
// bytes of two 32-bit words per slab into the reference byte layout: output byte j
// carries slab i in bits [QBIT*i, QBIT*(i+1)).  `w[i][h]` = bytes 4h..4h+3 of slab i.
template <int QBIT>
__device__ __forceinline__ uint2 interleave_slabs(const uint32_t (&w)[8 / QBIT][2]) {
  constexpr int EPP = 8 / QBIT;
  constexpr uint32_t M = ((1u << QBIT) - 1u) * 0x01010101u;
  constexpr uint32_t HALF = (1u << (QBIT - 1));
  uint32_t xorv = 0;
#pragma unroll
  for (int i = 0; i < EPP; ++i) xorv |= (HALF << (QBIT * i));
  xorv *= 0x01010101u;  // two's complement -> offset binary: flip the top bit of every code
  uint2 o = make_uint2(0u, 0u);
#pragma unroll
  for (int i = 0; i < EPP; ++i) {
    o.x |= (w[i][0] & M) << (QBIT * i);
    o.y |= (w[i][1] & M) << (QBIT * i);
  }
  o.x ^= xorv;
  o.y ^= xorv;
  return o;
}

// four signed ints -> four bytes (two's complement truncation), byte k = c_k
__device__ __forceinline__ uint32_t pack4_s8(int c0, int c1, int c2, int c3) {
  // cvt.pack.sat.s8.s32.b32 d, a, b, c  ==  d = (c << 16) | (sat8(a) << 8) | sat8(b)
  uint32_t hi, r;
  asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(hi) : "r"(c3), "r"(c2), "r"(0));
  asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(c1), "r"(c0), "r"(hi));
  return r;
}

}  // namespace hyc

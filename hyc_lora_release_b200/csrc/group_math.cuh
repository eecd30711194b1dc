// Arithmetic of the 64-wide group quantizer, shared by the group-mode and top-k kernels.
#pragma once
#include "hyc_common.cuh"

namespace hyc {

constexpr unsigned kFull = 0xffffffffu;

struct GroupParams { float s, rcl, zcl, z; };

// Group-mode arithmetic (fp32, one rounding per operation):
//   d = bf16(mx - mn);  il = 1/levels;  s = bf16(d * il), 1e-3 when zero;  rc = 1/s
//   z = clamp(rint(clamp(-mn*rc, +-300)) - half, -128, 127)
//   u = sat01(fma(x, rc*il, (z + half)*il));   code = rint(u * levels)     rint = half to even
// Per element that is one saturating fma and one fma with 2^23 as addend (the integer
// lands in the low mantissa bits): both run on the FMA pipe, no min/max, no conversion.
template <int QBIT>
__device__ __forceinline__ GroupParams group_params(float mn, float mx) {
  constexpr float il = 1.0f / (float)((1 << QBIT) - 1);
  constexpr float half = (float)(1 << (QBIT - 1));
  float d = bf16bits_to_f32(f32_to_bf16bits_rn(__fsub_rn(mx, mn)));
  float s = bf16bits_to_f32(f32_to_bf16bits_rn(__fmul_rn(d, il)));
  if (s == 0.f) s = bf16bits_to_f32(f32_to_bf16bits_rn(1e-3f));
  GroupParams p;
  p.s = s;
  const float rc = __frcp_rn(s);
  float t = fminf(fmaxf(__fmul_rn(-mn, rc), -300.f), 300.f);
  float zr = __fadd_rn(__fadd_rn(t, 12582912.f), -12582912.f);   // rint, |t| <= 300
  p.z = fminf(fmaxf(zr - half, -128.f), 127.f);
  p.rcl = __fmul_rn(rc, il);
  p.zcl = __fmul_rn(p.z + half, il);
  return p;
}

// min / max of the 16 values of a lane (packed pairs), then over the 4 lanes of the group
__device__ __forceinline__ void group_minmax(const uint32_t (&xw)[8], float& mn, float& mx) {
  __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&xw[0]);
  __nv_bfloat162 lo = a, hi = a;
#pragma unroll
  for (int j = 1; j < 8; ++j) {
    __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(&xw[j]);
    lo = __hmin2(lo, v);
    hi = __hmax2(hi, v);
  }
  mn = fminf(__bfloat162float(lo.x), __bfloat162float(lo.y));
  mx = fmaxf(__bfloat162float(hi.x), __bfloat162float(hi.y));
#pragma unroll
  for (int o = 1; o <= 2; o <<= 1) {
    mn = fminf(mn, __shfl_xor_sync(kFull, mn, o));
    mx = fmaxf(mx, __shfl_xor_sync(kFull, mx, o));
  }
}

// unsigned code of one value, left in the low byte of a float's bit pattern (2^23 + code)
template <int QBIT>
__device__ __forceinline__ uint32_t group_code_bits(float x, const GroupParams& p) {
  constexpr float levels = (float)((1 << QBIT) - 1);
  float u, r;
  asm("fma.rn.sat.f32 %0, %1, %2, %3;" : "=f"(u) : "f"(x), "f"(p.rcl), "f"(p.zcl));
  asm("fma.rn.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(u), "f"(levels), "f"(8388608.f));
  return __float_as_uint(r);
}

}  // namespace hyc

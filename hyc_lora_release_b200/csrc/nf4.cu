// De-quantizer of 4-bit block-wise weights in the layout of bitsandbytes 0.43.2 (`functional.dequantize_4bit`,
// which the reference calls as `BF.dequantize_nf4(w, quant_state)`, models/utils/compute_utils.py:19, 29 and
// models/llama/fused_llama_layer_intra_inter_full_fuse.py:218-219, 359, 367, 379).  That library is not part of
// this build; what is restated here is its published storage format:
//   * two 4-bit codes per byte, the HIGH nibble first: element 2 i in bits 7..4 of byte i, element 2 i + 1 in bits 3..0;
//   * value = code_table[code] * absmax[element / blocksize], computed in fp32, rounded once to bf16;
//   * the 16-entry code table travels with the quant state (NF4 or FP4: whatever the table holds);
//   * "double quantization": absmax itself stored as 8-bit codes, absmax = table256[code] * absmax2[block / blocksize2]
//     + offset (fp32).
// One thread turns 16 packed bytes into 32 bf16 values (64 bytes out); purely HBM-bound: 0.5 + 2 bytes per element.
#include "hyc_common.cuh"

namespace hyc {

template <bool NESTED>
__global__ void __launch_bounds__(256)
dequant_nf4_kernel(const uint8_t* __restrict__ packed, const float* __restrict__ code16,
                   const float* __restrict__ absmax, const uint8_t* __restrict__ absmax_q,
                   const float* __restrict__ code256, const float* __restrict__ absmax2, int blocksize2, float offset,
                   int64_t numel, int blocksize, __nv_bfloat16* __restrict__ out) {
  __shared__ float s_code[16];
  if (threadIdx.x < 16) s_code[threadIdx.x] = code16[threadIdx.x];
  __syncthreads();
  const int64_t n_chunks = (numel + 31) / 32;           // 32 elements = 16 bytes per chunk
  for (int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; c < n_chunks; c += (int64_t)gridDim.x * blockDim.x) {
    const int64_t e0 = c * 32;
    const bool whole = e0 + 32 <= numel;
    uint32_t w[4] = {0u, 0u, 0u, 0u};
    if (whole) {
      const uint4 v = ld_stream_v4(packed + c * 16);
      w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w;
    } else {
      const int64_t nbytes = (numel - e0 + 1) / 2;
      for (int64_t b = 0; b < nbytes; ++b) w[b >> 2] |= (uint32_t)packed[c * 16 + b] << (8 * (b & 3));
    }
    auto scale_of = [&](int64_t e) -> float {
      const int64_t blk = e / blocksize;
      if (!NESTED) return absmax[blk];
      // two roundings, as the library's two steps (block-wise de-quantization of the codes, then `+= offset`)
      return __fadd_rn(__fmul_rn(code256[absmax_q[blk]], absmax2[blk / blocksize2]), offset);
    };
    // blocks are at least 32 elements wide in every configuration the library offers (64 ... 4096); smaller
    // block sizes look the scale up per element
    const bool one_scale = (blocksize % 32) == 0;
    const float s_all = scale_of(e0);
    uint32_t o[16];
#pragma unroll
    for (int b = 0; b < 16; ++b) {
      const uint32_t byte = (w[b >> 2] >> (8 * (b & 3))) & 0xffu;
      const float s0 = one_scale ? s_all : scale_of(e0 + 2 * b);
      const float s1 = one_scale ? s_all : scale_of(e0 + 2 * b + 1);
      const float hi = __fmul_rn(s_code[byte >> 4], s0);          // element 2 b: the high nibble
      const float lo = __fmul_rn(s_code[byte & 15u], s1);         // element 2 b + 1
      o[b] = pack_bf16x2_rn(hi, lo);
    }
    if (whole) {
#pragma unroll
      for (int i = 0; i < 4; ++i)
        st_stream_v4(out + e0 + 8 * i, make_uint4(o[4 * i], o[4 * i + 1], o[4 * i + 2], o[4 * i + 3]));
    } else {
      for (int64_t e = e0; e < numel; ++e) {
        const uint32_t pr = o[(e - e0) >> 1];
        out[e] = __ushort_as_bfloat16((uint16_t)(((e - e0) & 1) ? (pr >> 16) : (pr & 0xffffu)));
      }
    }
  }
}

}  // namespace hyc

using namespace hyc;

extern "C" HYC_API int hyc_dequant_nf4(const void* packed, const float* code16, const float* absmax_f32,
                                       const uint8_t* absmax_q, const float* code256, const float* absmax2,
                                       int blocksize2, float offset, int64_t numel, int blocksize, void* out,
                                       void* stream) {
  if (!packed || !code16 || !out) return HYC_ERR_NULL;
  const bool nested = absmax_f32 == nullptr;
  if (nested && (!absmax_q || !code256 || !absmax2)) return HYC_ERR_NULL;
  if (numel < 0 || blocksize <= 0 || (nested && blocksize2 <= 0)) return HYC_ERR_SHAPE;
  if (!aligned(packed, 16) || !aligned(out, 16)) return HYC_ERR_ALIGN;
  if (numel == 0) return HYC_OK;
  const int64_t n_chunks = (numel + 31) / 32;
  int64_t grid = (n_chunks + 255) / 256;
  const int64_t cap = (int64_t)num_sms() * 8;
  if (grid > cap) grid = cap;
  cudaStream_t st = (cudaStream_t)stream;
  if (nested)
    dequant_nf4_kernel<true><<<(int)grid, 256, 0, st>>>((const uint8_t*)packed, code16, nullptr, absmax_q, code256, absmax2,
                                                      blocksize2, offset, numel, blocksize, (__nv_bfloat16*)out);
  else
    dequant_nf4_kernel<false><<<(int)grid, 256, 0, st>>>((const uint8_t*)packed, code16, absmax_f32, nullptr, nullptr, nullptr,
                                                       1, 0.f, numel, blocksize, (__nv_bfloat16*)out);
  HYC_CHECK_LAUNCH();
  return HYC_OK;
}

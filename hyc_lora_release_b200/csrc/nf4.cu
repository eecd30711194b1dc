// De-quantizer of 4-bit block-wise weights in the layout of bitsandbytes 0.43.2 (`functional.dequantize_4bit`,
// which the reference calls as `BF.dequantize_nf4(w, quant_state)`, models/utils/compute_utils.py:19, 29 and
// models/llama/fused_llama_layer_intra_inter_full_fuse.py:218-219, 359, 367, 379).  That library is not part of
// this build; what is restated here is its published storage format:
//   * two 4-bit codes per byte, the HIGH nibble first: element 2 i in bits 7..4 of byte i, element 2 i + 1 in bits 3..0;
//   * value = code_table[code] * absmax[element / blocksize], computed in fp32, rounded once to bf16;
//   * the 16-entry code table travels with the quant state (NF4 or FP4: whatever the table holds);
//   * "double quantization": absmax itself stored as 8-bit codes, absmax = table256[code] * absmax2[block / blocksize2]
//     + offset (fp32).
// A warp turns runs of 512 packed bytes into 1024 bf16 values with coalesced loads and stores; HBM-bound: 0.5 + 2
// bytes per element.
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
  auto scale_of = [&](int64_t e) -> float {
    const int64_t blk = e / blocksize;
    if (!NESTED) return absmax[blk];
    // two roundings, as the library's two steps (block-wise de-quantization of the codes, then `+= offset`)
    return __fadd_rn(__fmul_rn(code256[absmax_q[blk]], absmax2[blk / blocksize2]), offset);
  };
  // A warp takes runs of 1024 elements: four coalesced 128-byte loads (4 bytes = 8 elements per lane and load), four
  // coalesced 512-byte stores (16 bytes per lane and store).  All loads of a run are issued before the first use.
  const int lane = threadIdx.x & 31;
  const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t n_warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  const int64_t n_runs = numel / 1024;
  const bool one_scale = (blocksize % 8) == 0;        // the 8 elements of a lane share a block
  for (int64_t r = warp; r < n_runs; r += n_warps) {
    const int64_t e_run = r * 1024;
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) w[i] = __ldcs(reinterpret_cast<const uint32_t*>(packed + e_run / 2) + 32 * i + lane);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int64_t e0 = e_run + 256 * i + 8 * lane;
      const float s_all = scale_of(e0);
      uint32_t o[4];
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        const uint32_t byte = (w[i] >> (8 * b)) & 0xffu;
        const float s0 = one_scale ? s_all : scale_of(e0 + 2 * b);
        const float s1 = one_scale ? s_all : scale_of(e0 + 2 * b + 1);
        o[b] = pack_bf16x2_rn(__fmul_rn(s_code[byte >> 4], s0),           // element 2 b: the high nibble
                              __fmul_rn(s_code[byte & 15u], s1));         // element 2 b + 1
      }
      st_stream_v4(out + e0, make_uint4(o[0], o[1], o[2], o[3]));
    }
  }
  // what is left of the tensor (fewer than 1024 elements): one element per thread of the first block
  if (blockIdx.x == 0) {
    for (int64_t e = n_runs * 1024 + threadIdx.x; e < numel; e += blockDim.x) {
      const uint32_t byte = packed[e >> 1];
      const uint32_t code = (e & 1) ? (byte & 15u) : (byte >> 4);
      out[e] = __float2bfloat16_rn(__fmul_rn(s_code[code], scale_of(e)));
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
  if (!aligned(packed, 4) || !aligned(out, 16)) return HYC_ERR_ALIGN;
  if (numel == 0) return HYC_OK;
  const int64_t n_runs = numel / 1024;                 // one warp per run, eight warps per block
  int64_t grid = (n_runs + 7) / 8;
  const int64_t cap = (int64_t)num_sms() * 8;
  if (grid > cap) grid = cap;
  if (grid < 1) grid = 1;
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

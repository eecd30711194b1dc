// Per-row top-k kernels in the "one lane = one group of 64 columns" layout (rows of 64 * 2^n columns).
#pragma once
#include "group_math.cuh"

namespace hyc {

constexpr int kLaneStageEntries = 256;   // (column, value) words a warp stages in shared memory

// rows of 64, 128, ..., 2048 columns whose outlier lists (all rows of a warp) fit the staging area
inline bool topk_lane_ok(int S, int k) {
  if (S < 64 || S > 2048 || (S & (S - 1)) != 0) return false;
  const int rows_per_warp = 32 / (S / 64);
  return (int64_t)rows_per_warp * k <= kLaneStageEntries;
}

// both return 0 or a negative HYC_ERR_* (arguments already validated by the caller)
int topk_lane_compress(const void* a, int64_t rows, int S, int k, void* val_out, uint16_t* col_out,
                       void* q_out, void* scale_out, int8_t* zp_out, int q_bit, cudaStream_t st);
// scale + mask + softmax of raw scores fused with the save of the resulting map (see topk_lane.cu);
// HYC_ERR_UNSUPPORTED when the shape is not covered (nothing launched)
int topk_lane_softmax_compress(const void* scores, float scale, const void* mask, int64_t mb, int64_t mh, int64_t mr, int heads,
                               int M, int64_t rows, int S, int k, void* dense, void* val_out, uint16_t* col_out,
                               void* q_out, void* scale_out, int8_t* zp_out, int q_bit, cudaStream_t st);
// grad_or_null != NULL: a_out receives bf16(softmax_backward(restored map, grad) * out_scale) instead of the
// restored map (out_scale == 1: no second operation)
int topk_lane_restore(const void* val, const uint16_t* col, int k, const void* q, const void* scale,
                      const int8_t* zp, int64_t rows, int S, const void* grad_or_null, float out_scale, void* a_out,
                      int q_bit, cudaStream_t st);

// softmax backward on dense maps in the same layout; false = shape or alignment not covered, nothing launched
bool softmax_bwd_lane(const void* y, const void* g, int64_t rows, int S, float out_scale, void* out, cudaStream_t st);

}  // namespace hyc

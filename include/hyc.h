/*
 * libhyc -- C ABI of the B200 (sm_100a) activation-compression kernels.
 *
 * Every entry point replaces one launch wrapper (or one pure-PyTorch helper) of the
 * HyC-LoRA-release operator layer; the comment above each declaration cites it
 * (paths relative to that project's root).  Conventions:
 *   - all pointers are DEVICE pointers unless the name says `host`;
 *   - activations are bf16, row-major, last dimension contiguous; `rows` is the product
 *     of the leading dimensions (batch * sequence), `ld*` a row stride in ELEMENTS;
 *   - packed codes use the reference byte layout: inside every 32-column block, byte j
 *     holds the codes of columns j, j+32/epp, j+2*32/epp, ... (epp = 8 / q_bit) in
 *     ascending bit position (operators/compress_function_kernel.py:78-110);
 *   - `stream` is a cudaStream_t passed as void*; work is stream-ordered, nothing
 *     synchronises, nothing allocates (scratch is caller-provided and sized by the
 *     matching *_workspace_bytes query);
 *   - the return value is 0 or a negative HYC_ERR_* code; hyc_strerror() names it.
 */
#ifndef HYC_H_
#define HYC_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  HYC_OK = 0,
  HYC_ERR_NULL = -1,        /* a required pointer is null */
  HYC_ERR_QBIT = -2,        /* q_bit not in {2,4,8} */
  HYC_ERR_SHAPE = -3,       /* a dimension violates the documented divisibility / range */
  HYC_ERR_ALIGN = -4,       /* pointer or stride not aligned for 128-bit access */
  HYC_ERR_WORKSPACE = -5,   /* workspace missing or too small */
  HYC_ERR_LAUNCH = -6,      /* CUDA launch failed; see hyc_last_cuda_error() */
  HYC_ERR_CAPACITY = -7,    /* output capacity too small for the data */
  HYC_ERR_UNSUPPORTED = -8  /* feature not available in this build */
};

const char* hyc_strerror(int code);
int hyc_last_cuda_error(void);   /* cudaError_t of the last HYC_ERR_LAUNCH, else 0 */
int hyc_version(void);

/* ---- statistics (calibration iterations only) ------------------------------------ */

/* Per-channel scale of batch sample 0: scale[n] = bf16((max_m x0[m,n] - min_m x0[m,n]) / (2^q - 1)).
 * Replaces get_statistics_only_quant(..., 'per-channel')  (operators/compress_function.py:45-59).
 * If outlier_idx != NULL (k entries) those columns are treated as zero and zero scales become
 * bf16(1e-3): the scale half of get_statistics_channel_base (compress_function.py:94-104).
 * If zp_out != NULL it also writes the int8 zero point of
 * get_statistics_only_quant_zero_point (compress_function.py:62-77).
 * x0: [M, N] bf16, N % 8 == 0. */
int hyc_colstats_scale(const void* x0, int M, int N, int64_t ldx, int q_bit,
                       const int64_t* outlier_idx, int k,
                       void* scale_out, int8_t* zp_out, void* stream);

/* Column L2 norm of sample 0 as bf16 and the k largest channels ordered by
 * (norm descending, index ascending).  Replaces the norm/topk half of
 * get_statistics_channel_base (compress_function.py:86-87).  N <= 32768.
 * norm_out: [N] bf16 scratch/result; idx_out: [k] int64. */
int hyc_channel_norm_topk(const void* x0, int M, int N, int64_t ldx, int k,
                          void* norm_out, int64_t* idx_out, void* stream);

/* ---- per-channel quantize-and-pack / unpack-dequantize ---------------------------- */

/* Replaces compression_quantization (+kernel) (compress_function.py:178-210,
 * compress_function_kernel.py:47-112), compression_quantization_with_zero_point
 * (compress_function.py:245-275, kernel :229-301) when zp != NULL, and
 * outlier_subtraction_fuse_compression_quantization (compress_function.py:111-143) when
 * outlier_idx != NULL: the k outlier columns are gathered into outlier_out [rows, k] bf16 and
 * encoded as zero; x itself is NOT modified.
 * x [rows, N] bf16 (N % 32 == 0), scale [N] bf16, zp [N] int8 or NULL,
 * q_out [rows, N*q_bit/8] uint8. */
int hyc_quant_pack(const void* x, int64_t rows, int N, int64_t ldx,
                   const void* scale, const int8_t* zp,
                   const int64_t* outlier_idx, int k,
                   void* q_out, void* outlier_out, int q_bit, void* stream);

/* Replaces decompression_dequantization (+kernel) (compress_function.py:214-241, kernel
 * :150-206), ..._with_zero_point (compress_function.py:278-306, kernel :324-388) when
 * zp != NULL, and outlier_addition_fuse_decompression_dequantization
 * (compress_function.py:147-174) when outlier_idx != NULL (x[:, idx[j]] = outlier[:, j]).
 * x_out [rows, N] bf16 with row stride ldx. */
int hyc_unpack_dequant(const void* q, int64_t rows, int N,
                       const void* scale, const int8_t* zp,
                       const int64_t* outlier_idx, int k, const void* outlier,
                       void* x_out, int64_t ldx, int q_bit, void* stream);

/* ---- 64-wide group mode (no counterpart in the reference: scale and zero point are
 *      taken from each group of 64 values of a row; same arithmetic as
 *      compress_function.py:62-77 / compress_function_kernel.py:279-299, 376-387) ------ */
int hyc_group_quant_pack(const void* x, int64_t rows, int N, int64_t ldx,
                         void* q_out, void* scale_out, int8_t* zp_out, int q_bit, void* stream);
int hyc_group_unpack_dequant(const void* q, int64_t rows, int N,
                             const void* scale, const int8_t* zp,
                             void* x_out, int64_t ldx, int q_bit, void* stream);

/* ---- attention map: threshold prune (the reference's behaviour) --------------------- */

/* compression_softmax (compress_function.py:309-313): keep a[i] > bf16(threshold) and
 * a[i] != 0, as the COO list of the flattened map.  Two phases because the caller owns the
 * output: phase 1 counts per tile and leaves exclusive offsets plus the total in `workspace`
 * (copy the int64 at workspace[0] to the host to size idx/val); phase 2 writes them.
 * workspace bytes: hyc_softmax_prune_workspace_bytes(numel). */
size_t hyc_softmax_prune_workspace_bytes(int64_t numel);
int hyc_softmax_prune_count(const void* a, int64_t numel, float threshold,
                            void* workspace, size_t workspace_bytes, void* stream);
int hyc_softmax_prune_fill(const void* a, int64_t numel, float threshold,
                           const void* workspace, int64_t* idx_out, void* val_out,
                           int64_t capacity, void* stream);
/* to_dense (compress_function.py:316-317): zero-fill and scatter. */
int hyc_softmax_prune_restore(const int64_t* idx, const void* val, int64_t nnz,
                              void* a_out, int64_t numel, void* stream);

/* to_dense for a list whose length lives in device memory (the count hyc_softmax_prune_static left in nnz_out and
 * nobody copied to the host): zero-fill, then scatter min(*nnz_dev, capacity) entries.  No host synchronisation. */
int hyc_softmax_prune_restore_counted(const int64_t* idx, const void* val, const int64_t* nnz_dev, int64_t capacity,
                                      void* a_out, int64_t numel, void* stream);

/* The same threshold prune in ONE pass over the map, in a tiled form, for callers that only ever restore the map
 * (the restore of the layers is to_dense, compress_function.py:316-317; nothing reads the COO list itself): no
 * second pass over the map, 4 bytes per kept entry instead of 10.  The map is cut into batches of 2048 consecutive
 * elements; the entries of a batch go into a span of words_out as (offset in the batch << 16 | bf16 bits), in no
 * particular order inside the span, and directory_out[batch] = {first word of the span, entries written} (two
 * uint32).  directory_out holds hyc_softmax_prune_tiled_directory_bytes(numel) bytes (the directory and, behind it,
 * 8 KB of counters the call clears and uses: one per sub-list and a ticket by which the block that finishes last
 * knows to write *nnz_out, so the whole save is one memset and one kernel) and must be 128-byte aligned.  words_out is used as up to 64 equal
 * sub-lists (one per 32 batches of the map, a single one for maps below 131072 elements); a batch takes its span
 * from the sub-list that a hash of its index names, by one atomic add on that sub-list's counter, so the order of
 * the spans depends on the run and the sub-lists fill evenly but not identically (give `capacity` a margin); the set of (index, value) pairs is that of
 * compression_softmax (compress_function.py:309-313).  *nnz_out (device int64) = the number of kept entries if
 * every span fit its sub-list, else capacity + the number of dropped entries (so "nnz > capacity" means entries
 * were dropped).  capacity <= 2^32 - 1. */
size_t hyc_softmax_prune_tiled_directory_bytes(int64_t numel);
int hyc_softmax_prune_tiled(const void* a, int64_t numel, float threshold,
                            uint32_t* words_out, int64_t capacity, void* directory_out,
                            int64_t* nnz_out, void* stream);
/* to_dense for the tiled form, one pass: every batch's 4 KB are built on chip and written once (no zero-fill pass,
 * no scattered 2-byte stores). */
int hyc_softmax_prune_tiled_restore(const uint32_t* words, int64_t capacity, const void* directory,
                                    void* a_out, int64_t numel, void* stream);

/* No counterpart in the reference.  The same threshold prune for callers that must not allocate
 * device memory at call time (a fixed up-front memory plan, or a host that forbids allocation inside
 * operator callbacks) and so have no workspace to pass: the tile offsets live in a 512 KiB array built
 * into the library (resident on every GPU that loads it), count + scan + fill run in this one call,
 * and nothing is allocated.  nnz_out (device int64) receives the number of kept entries; entries
 * beyond `capacity` are dropped, so compare the two.  Limit: numel <= 268,435,456 (else
 * HYC_ERR_CAPACITY).  The first call on each device resolves the array's address and should be made
 * outside of stream capture.  Calls share the array: do not let two of them overlap on one GPU.  A map that
 * lives on another GPU than the current one is refused (HYC_ERR_UNSUPPORTED): the scratch is per device. */
int hyc_softmax_prune_static(const void* a, int64_t numel, float threshold,
                             int64_t* idx_out, void* val_out, int64_t capacity,
                             int64_t* nnz_out, void* stream);

/* ---- attention map: per-row top-k + grouped remainder (no counterpart in the reference;
 *      the reference prunes by one global threshold, compress_function.py:30-32, 309-313) -- */
/* a [rows, S] bf16 (S % 64 == 0, S <= 4096, k <= S): the k largest magnitudes of every row
 * (equal magnitudes: lower column first) go to val_out [rows,k] bf16 / col_out [rows,k] uint16 in
 * ascending column order; the row with those positions zeroed is group-quantized. */
int hyc_softmax_topk_compress(const void* a, int64_t rows, int S, int k,
                              void* val_out, uint16_t* col_out,
                              void* q_out, void* scale_out, int8_t* zp_out, int q_bit, void* stream);
/* The forward side of the attention map in ONE pass: s = q k^T / sqrt(d) is already computed (library batched GEMM);
 * this call does  a = softmax(bf16(bf16(s * scale) + mask))  (fused_llama_layer_intra_inter_full_fuse.py:152-167, the
 * three tensor operations of the layer with their bf16 rounding points), writes the dense probabilities to a_out
 * (the P.V product needs them; a_out may be the scores buffer) AND saves them in the top-k form of
 * hyc_softmax_topk_compress -- the row never leaves the registers in between, so the map is read once instead of
 * twice.  mask: additive bf16, row m of (batch b, head h) at mask + b * mask_stride_b + h * mask_stride_h +
 * m * mask_stride_row (strides in elements, 0 = broadcast).  rows = batch * heads * M.  Returns
 * HYC_ERR_UNSUPPORTED without launching anything for shapes outside the fused kernel (S not 64 * 2^n <= 2048, M not a
 * multiple of 32 / (S / 64), mask_stride_row != S, buffers not 32-byte aligned): run hyc_softmax_fwd_scale_mask and
 * hyc_softmax_topk_compress then. */
int hyc_softmax_fwd_topk_save(const void* scores, float scale, const void* mask_or_null, int64_t mask_stride_b,
                              int64_t mask_stride_h, int64_t mask_stride_row, int heads, int M,
                              int64_t rows, int S, int k, void* a_out, void* val_out, uint16_t* col_out,
                              void* q_out, void* scale_out, int8_t* zp_out, int q_bit, void* stream);
int hyc_softmax_topk_restore(const void* val, const uint16_t* col, int k,
                             const void* q, const void* scale, const int8_t* zp,
                             int64_t rows, int S, void* a_out, int q_bit, void* stream);
/* Restore fused with softmax_backward (fused_llama_layer_intra_inter_full_fuse.py:414-433: `a_o.to_dense()`
 * followed by `softmax_backward`): out = (g - sum_row(bf16(y * g))) * y with y the restored map, which is
 * never written to HBM.  grad, out [rows, S] bf16.  out_scale != 1 multiplies the bf16 result once more (a second
 * bf16 operation: the layer's `grad_s / sqrt(head_dim)`, :436).  Returns HYC_ERR_UNSUPPORTED for shapes outside the
 * lane-per-group kernels (S not 64 * 2^n <= 2048, very large k): restore, then hyc_softmax_bwd. */
int hyc_softmax_topk_restore_bwd(const void* val, const uint16_t* col, int k,
                                 const void* q, const void* scale, const int8_t* zp,
                                 int64_t rows, int S, const void* grad, void* out, int q_bit, float out_scale,
                                 void* stream);

/* ---- fused LoRA-SiLU-Hadamard elementwise kernels ------------------------------------- */

/* triton_fuse_silu_forward (operators/triton_fuse_lora_silu_hadamard_forward_kernels.py:28-181).
 * xa* [rows, R] bf16 (R == 16), bt* [N, R] bf16 (the LoRA-B weight as stored, i.e. b^T),
 * x* [rows, N] bf16 (the frozen-weight products), s* [N] bf16.  N % 32 == 0.
 * Writes q1, q2 [rows, N*q_bit/8] and o [rows, N] bf16. */
int hyc_fused_lora_silu_hadamard_fwd(const void* xa1, const void* bt1, const void* x1, const void* s1,
                                     const void* xa2, const void* bt2, const void* x2, const void* s2,
                                     void* q1, void* q2, void* o,
                                     int64_t rows, int N, int R, int q_bit, void* stream);
/* triton_fuse_silu_backward (operators/triton_fuse_lora_silu_hadamard_backward_kernels.py:28-178).
 * Writes o, grad_gate, grad_up [rows, N] bf16. */
int hyc_fused_lora_silu_hadamard_bwd(const void* xa1, const void* bt1, const void* q1, const void* s1,
                                     const void* xa2, const void* bt2, const void* q2, const void* s2,
                                     const void* grad_o, void* o, void* grad_gate, void* grad_up,
                                     int64_t rows, int N, int R, int q_bit, void* stream);

/* De-quantize + LoRA re-add: y = bf16( decompression_dequantization(q, scale) + bf16(xa * bt^T) ), the
 * backward-side reconstruction of a LoRA projection whose main branch was saved as codes (q/k/v:
 * fused_llama_layer_intra_inter_full_fuse.py:416-452, `decompression_dequantization` then `+ x_lora_a @ w_lora_b`).
 * q [rows, N*q_bit/8], scale [N] bf16, xa [rows, 16] bf16, bt [N, 16] bf16, y [rows, N] bf16.  N % 32 == 0. */
int hyc_dequant_lora_add(const void* q, const void* scale, const void* xa, const void* bt,
                         void* y, int64_t rows, int N, int R, int q_bit, void* stream);

/* ---- producers / consumers of the saved tensors ----------------------------------------- */

/* rmsnorm_forward / rmsnorm_backward (operators/rmsnorm_kernels.py:10-54, 58-113, wrappers
 * :116-185).  rstd [rows] fp32.  The backward keeps the reference's LayerNorm-style mean term. */
int hyc_rmsnorm_fwd(const void* x, const void* w, float eps, void* y, float* rstd,
                    int64_t rows, int N, void* stream);
int hyc_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, void* dx,
                    int64_t rows, int N, void* stream);

/* RMSNorm fused with the saves of the fused layer (fused_llama_layer_intra_inter_full_fuse.py:203-216: the
 * norm, `compression_pack_channel_base(x_medium)` and `compression_pack_quant_base(x_norm)` of the MLP half; the
 * attention half has the same pattern at :99-112): one pass over x writes y = x_norm and rstd, the packed
 * per-channel codes of x (qx [rows, N*q_bit/8]) with its outlier channels moved to outlier_out [rows, k], and,
 * when scale_y/qy are given, the packed codes of the bf16 y.  Bit-identical to hyc_rmsnorm_fwd followed by
 * hyc_quant_pack on x (with the outlier list) and on y.  Statistics are the caller's (steady state of the
 * calibration): scale_x [N] (zero-guarded), outlier_idx int64 [k], scale_y [N].  N % 32 == 0, N <= 16384. */
int hyc_rmsnorm_fwd_save(const void* x, const void* w, float eps, int64_t rows, int N,
                         const void* scale_x, const int64_t* outlier_idx, int k, const void* scale_y_or_null,
                         void* y, float* rstd, void* qx, void* outlier_out, void* qy_or_null, int q_bit, void* stream);

/* RMSNorm backward reading the packed x directly (:388-395, :484-491: `outlier_addition_fuse_decompression_
 * dequantization` followed by `rmsnorm_backward`): x is de-quantized and its outlier channels restored inside
 * the kernel, then the arithmetic of hyc_rmsnorm_bwd.  residual_grad (optional, [rows, N] bf16) is added to the
 * result as a bf16 tensor add (the residual branch of the layer input's gradient). */
int hyc_rmsnorm_bwd_packed(const void* dy, const void* qx, const void* scale_x, const int64_t* outlier_idx, int k,
                           const void* outlier, const void* w, const float* rstd, const void* residual_grad_or_null,
                           void* dx, int64_t rows, int N, int q_bit, void* stream);
/* rope_forward / rope_backward (operators/rope_kernels.py:81-131, called from
 * fused_llama_layer_intra_inter_full_fuse.py:142-143, 441, 449, 459-460): rotary embedding in the rotate-half
 * form on the hidden layout.  x, out [rows, n_heads*head_dim] bf16 with row strides ldx / ldo (elements,
 * multiples of 8; out may alias x), position of a row = row % seq_len, cos/sin tables [>= seq_len, ld_table]
 * of which the first head_dim/2 columns are read, bf16 (table_is_f32 = 0) or fp32 (1).
 *   out[j] = x[j]*cos[j] - x[j+h]*sin[j];  out[j+h] = x[j+h]*cos[j] + x[j]*sin[j];  backward: sin negated.
 * fp32 arithmetic, one rounding to bf16.  head_dim % 16 == 0. */
int hyc_rope(const void* x, int64_t ldx, void* out, int64_t ldo, const void* cos_table, const void* sin_table,
             int64_t ld_table, int table_is_f32, int64_t rows, int seq_len, int n_heads, int head_dim,
             int backward, void* stream);
/* Attention probabilities from raw scores in one pass (fused_llama_layer_intra_inter_full_fuse.py:150-160:
 * `s = q @ k^T / sqrt(d)`, `s + attention_mask`, `softmax(s, -1, dtype=bf16)`): a = softmax(bf16(bf16(scores * scale)
 * + mask)) per row, fp32 inside, bf16 result.  scores, a [rows, S] bf16 (a may alias scores), rows = batch * heads * M;
 * the optional additive bf16 mask is read at mask[b*stride_b + head*stride_h + m*stride_row + column] (strides in
 * elements, multiples of 8; stride_h = 0 for a mask shared by the heads).  S % 8 == 0, S <= 4096. */
int hyc_softmax_fwd_scale_mask(const void* scores, float scale, const void* mask_or_null, int64_t mask_stride_b,
                               int64_t mask_stride_h, int64_t mask_stride_row, int heads, int M, void* a,
                               int64_t rows, int S, void* stream);
/* softmax_backward (operators/softmax_kernels.py:7-56): o = (g - sum(y*g)) * y per row; out_scale != 1 multiplies
 * the bf16 result once more (o = bf16(o * out_scale)). */
int hyc_softmax_bwd(const void* y, const void* g, void* o, int64_t rows, int S, float out_scale, void* stream);

/* ---- frozen weights stored as 4-bit block-wise codes -------------------------------------------
 * De-quantizer for weights in the storage format of bitsandbytes 0.43.2 (requirements.txt:3), which the reference
 * calls as BF.dequantize_nf4(w, quant_state) before every frozen matmul (models/utils/compute_utils.py:19, 29;
 * models/llama/fused_llama_layer_intra_inter_full_fuse.py:218-219, 359, 367, 379).  The library itself is not part
 * of this build; its published format is restated: two codes per byte, high nibble first; value = code16[code] *
 * absmax[element / blocksize] in fp32, rounded to bf16; with "double quantization" absmax_f32 is NULL and absmax =
 * code256[absmax_q[block]] * absmax2[block / blocksize2] + offset.  packed: numel/2 bytes (4-byte aligned);
 * code16: 16 floats (the table of the quant state: NF4 or FP4); out: numel bf16.  Parity unpinned (no copy of the
 * library to compare with). */
int hyc_dequant_nf4(const void* packed, const float* code16, const float* absmax_f32,
                    const uint8_t* absmax_q, const float* code256, const float* absmax2,
                    int blocksize2, float offset, int64_t numel, int blocksize, void* out, void* stream);

/* ---- tcgen05 / TMEM GEMMs of the LoRA MLP (activation compression in the epilogue) ------------
 * bf16 operands, fp32 accumulation in tensor memory, operands staged by TMA.  `status` is a
 * caller-provided device int, zero before the call; a non-zero value afterwards means a bounded
 * wait inside the kernel gave up (1 producer, 2 MMA issuer, 3 epilogue) and the output is invalid.
 * LoRA operands: xa* is the [rows, 16] activation of the LoRA-A projection; bt* addresses the LoRA-B
 * factor as element (column, r) at bt[column * ld_col + r * ld_r], so both the [out, r] weight and
 * its [r, out] transpose can be passed without a copy. */

/* D[M,N] = A[M,K] * B (+ A2[M,K2] * B2) (+ A3[M,K3] * B3) (+ xa0 * bt0^T) (+ xa1 * bt1^T) (+ residual).
 * Up to three (A, B) pairs accumulate in the same tensor-memory tile; K2, K3 may be 0.  A rank-16 LoRA
 * product can be passed either as an extra pair whose K is padded with zeros to 64 (it then costs one more
 * MMA block and nothing in the epilogue) or as xa/bt, evaluated per element in the epilogue and rounded to
 * bf16 separately like the reference's tensor-by-tensor code.
 * b_is_kn = 0: every B is [N,K] row-major (an nn.Linear weight, forward use); 1: every B is [K,N] row-major
 * (the same weight used for a backward product, read in place).  N % 256 == 0, K, K2, K3 % 64 == 0.
 * Replaces the matmuls of lora_forward / lora_backward (models/utils/compute_utils.py:18-36) and the
 * hand-inlined copies (models/llama/fused_llama_layer_intra_inter_full_fuse.py:247, 359-364, 379-384). */
int hyc_gemm_bf16_tcgen05(const void* A, const void* B, int M, int N, int K, int b_is_kn,
                          const void* A2, const void* B2, int K2, const void* A3, const void* B3, int K3,
                          const void* xa0, const void* bt0, int64_t bt0_ld_col, int64_t bt0_ld_r,
                          const void* xa1, const void* bt1, int64_t bt1_ld_col, int64_t bt1_ld_r,
                          const void* residual, void* D, int* status, void* stream);

/* A LoRA projection with the save of its main branch in the GEMM epilogue (the q/k/v/o projections of the
 * attention half: `lora_forward` followed by `compression_pack_quant_base(x=q_main, ...)`,
 * fused_llama_layer_intra_inter_full_fuse.py:112-142; models/utils/compute_utils.py:18-25):
 *   main = bf16(x * w^T)   q_out = quantize + pack(main, scale)   y = bf16(main + bf16(xa * bt^T))
 * x [T,K], w [N,K] (nn.Linear layout), xa [T,16] = x * A^T (or NULL: no LoRA term), bt element (col, r) at
 * bt[col*bt_ld_col + r*bt_ld_r], scale [N] bf16 (calibrated; during calibration run hyc_gemm_bf16_tcgen05, the
 * statistics and hyc_quant_pack instead), q_out [T, N*q_bit/8], y [T,N]; main_or_null receives the bf16 main
 * branch for inspection.  N % 256 == 0, K % 64 == 0. */
int hyc_linear_lora_save_fwd_tcgen05(const void* x, const void* w, int T, int K, int N,
                                     const void* xa, const void* bt, int64_t bt_ld_col, int64_t bt_ld_r,
                                     const void* scale, void* q_out, void* y, void* main_or_null, int q_bit,
                                     int* status, void* stream);

/* gate/up projections and triton_fuse_silu_forward in one kernel
 * (fused_llama_layer_intra_inter_full_fuse.py:218-235 + triton_fuse_lora_silu_hadamard_forward_kernels.py):
 * gate_main = x * wg^T and up_main = x * wu^T stay in tensor memory; the epilogue rounds them to bf16,
 * quantizes and packs them (q1, q2), adds the LoRA terms, applies SiLU and the Hadamard product (o).
 * x [T,H], wg/wu [I,H], s1/s2 [I] bf16, q1/q2 [T, I*q_bit/8], o [T,I].  I % 128 == 0, H % 64 == 0.
 * main1/main2 (optional, [T,I] bf16) receive the bf16 main branches for inspection. */
int hyc_mlp_gateup_fwd_tcgen05(const void* x, const void* wg, const void* wu, int T, int H, int I,
                               const void* xa1, const void* b1t, int64_t b1_ld_col, int64_t b1_ld_r,
                               const void* xa2, const void* b2t, int64_t b2_ld_col, int64_t b2_ld_r,
                               const void* s1, const void* s2, void* q1, void* q2, void* o,
                               void* main1_or_null, void* main2_or_null, int q_bit, int* status, void* stream);

/* grad_down = g * wd (+ a_lora * b_lora) and triton_fuse_silu_backward in one kernel
 * (fused_llama_layer_intra_inter_full_fuse.py:359-369 + triton_fuse_lora_silu_hadamard_backward_kernels.py):
 * the epilogue unpacks and de-quantizes the saved gate/up codes, recomputes the forward and writes
 * o (hadamard), grad_gate, grad_up [T,I].  g [T,H], wd [H,I] (the down weight as stored).  I % 256 == 0.
 * The LoRA part of grad_down, (g * Bd^T) * Ad, is passed as a zero-padded extra K block:
 * a_lora [T, k_lora] (the rank-16 product g * Bd^T in its first columns), b_lora [k_lora, I] (Ad in its
 * first rows), k_lora a multiple of 64 or 0.
 * The LoRA terms of the gate and up branches that the recomputation needs, bf16(xa1 * b1t^T) and
 * bf16(xa2 * b2t^T), are either computed in the epilogue (16 FMAs per element each: lora_gate = lora_up = NULL)
 * or read from lora_gate / lora_up ([T, ld_lora] bf16, ld_lora >= I, a multiple of 8), which one launch of
 * hyc_gemm_bf16_tcgen05 on the zero-padded rank-16 operands prepares; xa1/b1t/xa2/b2t may then be NULL. */
int hyc_mlp_graddown_bwd_tcgen05(const void* g, const void* wd, int T, int H, int I,
                                 const void* a_lora, const void* b_lora, int k_lora,
                                 const void* xa1, const void* b1t, int64_t b1_ld_col, int64_t b1_ld_r,
                                 const void* xa2, const void* b2t, int64_t b2_ld_col, int64_t b2_ld_r,
                                 const void* q1, const void* s1, const void* q2, const void* s2,
                                 const void* lora_gate, const void* lora_up, int64_t ld_lora,
                                 void* o, void* grad_gate, void* grad_up, int q_bit, int* status, void* stream);

/* LoRA-A gradient with the de-quantizer inside the contraction:
 *   out[r, h] = sum_t gm[t, r] * x_hat[t, h],   x_hat = decompression_dequantization(q, scale)
 * Replaces `decompression_dequantization` followed by `x.mT @ grad_medium` of lora_backward
 * (models/utils/compute_utils.py:30-32; call sites fused_llama_layer_intra_inter_full_fuse.py:375-383): the
 * packed codes are unpacked into shared-memory tiles and fed to the tensor cores; x_hat is never written to
 * HBM.  q [T, H*q_bit/8], scale [H] bf16, gm [T, ldg] bf16 of which the first R2 columns are used (R2 a
 * multiple of 16, <= 64: several LoRA adapters that share the input can be stacked), out [R2, H] bf16.
 * H % 128 == 0.  workspace: hyc_lora_grad_a_workspace_bytes(T, H, R2) bytes of fp32 partial sums. */
size_t hyc_lora_grad_a_workspace_bytes(int T, int H, int R2);
int hyc_lora_grad_a_dequant(const void* q, const void* scale, const void* gm, int64_t ldg, int R2,
                            int T, int H, int q_bit, void* out, void* workspace, size_t workspace_bytes,
                            void* stream);

#ifdef __cplusplus
}
#endif
#endif /* HYC_H_ */

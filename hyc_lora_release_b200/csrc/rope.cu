// Rotary position embedding (rotate-half form) on the hidden layout [rows, n_heads * head_dim], the
// operation the fused layer applies to q and k after their projections and re-applies in the backward pass
// to the reconstructed q and k (models/llama/fused_llama_layer_intra_inter_full_fuse.py:142-143, 441, 449,
// 459-460 call rope_forward / rope_backward of operators/rope_kernels.py).
//
//   position p = row % seq_len,  h = head_dim / 2,  c = cos[p, j],  s = sin[p, j]   (j < h: the tables
//   repeat their first half in the second)
//   out[j]     = x[j] * c - x[j + h] * s
//   out[j + h] = x[j + h] * c + x[j] * s            backward: the same with s negated
//
// Arithmetic: that of the reference's kernel, which computes in the dtype of the sine table
// (operators/rope_kernels.py:73-78: `Q1 = tl.load(...).to(sin1.dtype)`): with bf16 tables every product and the
// sum are bf16 operations (three roundings per output); with fp32 tables they are separate fp32 operations and the
// store rounds to bf16.  No multiply-add contraction in either form.
// One thread owns eight adjacent j of one head: two 16-byte loads and two 16-byte stores of x, 16 (bf16
// tables) or 2 x 32 (fp32 tables) bytes of each table; the tables stay in L1/L2 (seq_len * head_dim values).
#include "hyc_common.cuh"

namespace hyc {

template <bool TABLE_F32>
__global__ void __launch_bounds__(256)
rope_kernel(const __nv_bfloat16* __restrict__ x, int64_t ldx, __nv_bfloat16* __restrict__ out, int64_t ldo,
            const void* __restrict__ cos_t, const void* __restrict__ sin_t, int64_t ld_table,
            int64_t rows, int seq_len, int n_heads, int head_dim, float sin_sign) {
  const int half = head_dim >> 1;
  const int per_head = half >> 3;                       // octets of j per head
  const int per_row = n_heads * per_head;
  const int64_t total = rows * per_row;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = i / per_row;
    const int w = (int)(i - row * per_row);
    const int head = w / per_head, j0 = (w - head * per_head) << 3;
    const int pos = (int)(row % seq_len);
    const __nv_bfloat16* xp = x + row * ldx + (int64_t)head * head_dim + j0;
    const uint4 a = *reinterpret_cast<const uint4*>(xp);
    const uint4 b = *reinterpret_cast<const uint4*>(xp + half);
    const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
    uint32_t o1[4], o2[4];
    if (TABLE_F32) {
      float c[8], s[8];
      const float* cp = reinterpret_cast<const float*>(cos_t) + pos * ld_table + j0;
      const float* sp = reinterpret_cast<const float*>(sin_t) + pos * ld_table + j0;
#pragma unroll
      for (int e = 0; e < 8; e += 4) {
        const float4 cv = *reinterpret_cast<const float4*>(cp + e), sv = *reinterpret_cast<const float4*>(sp + e);
        c[e] = cv.x; c[e + 1] = cv.y; c[e + 2] = cv.z; c[e + 3] = cv.w;
        s[e] = sv.x; s[e + 1] = sv.y; s[e + 2] = sv.z; s[e + 3] = sv.w;
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float x1l = bf16lo_to_f32(aw[e]), x1h = bf16hi_to_f32(aw[e]);
        const float x2l = bf16lo_to_f32(bw[e]), x2h = bf16hi_to_f32(bw[e]);
        const float sl = s[2 * e] * sin_sign, sh = s[2 * e + 1] * sin_sign;
        const float cl = c[2 * e], ch = c[2 * e + 1];
        o1[e] = pack_bf16x2_rn(__fsub_rn(__fmul_rn(x1l, cl), __fmul_rn(x2l, sl)), __fsub_rn(__fmul_rn(x1h, ch), __fmul_rn(x2h, sh)));
        o2[e] = pack_bf16x2_rn(__fadd_rn(__fmul_rn(x2l, cl), __fmul_rn(x1l, sl)), __fadd_rn(__fmul_rn(x2h, ch), __fmul_rn(x1h, sh)));
      }
    } else {
      const uint4 cv = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(cos_t) + pos * ld_table + j0);
      const uint4 sv = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(sin_t) + pos * ld_table + j0);
      const uint32_t cw[4] = {cv.x, cv.y, cv.z, cv.w}, sw[4] = {sv.x, sv.y, sv.z, sv.w};
      const uint32_t flip = sin_sign < 0.f ? 0x80008000u : 0u;     // backward: the sine negated (exact)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const uint32_t sn = sw[e] ^ flip;
        const __nv_bfloat162 x1 = *reinterpret_cast<const __nv_bfloat162*>(&aw[e]);
        const __nv_bfloat162 x2 = *reinterpret_cast<const __nv_bfloat162*>(&bw[e]);
        const __nv_bfloat162 c2 = *reinterpret_cast<const __nv_bfloat162*>(&cw[e]);
        const __nv_bfloat162 s2 = *reinterpret_cast<const __nv_bfloat162*>(&sn);
        const __nv_bfloat162 r1 = __hsub2_rn(__hmul2_rn(x1, c2), __hmul2_rn(x2, s2));
        const __nv_bfloat162 r2 = __hadd2_rn(__hmul2_rn(x2, c2), __hmul2_rn(x1, s2));
        o1[e] = *reinterpret_cast<const uint32_t*>(&r1);
        o2[e] = *reinterpret_cast<const uint32_t*>(&r2);
      }
    }
    __nv_bfloat16* op = out + row * ldo + (int64_t)head * head_dim + j0;
    *reinterpret_cast<uint4*>(op) = make_uint4(o1[0], o1[1], o1[2], o1[3]);
    *reinterpret_cast<uint4*>(op + half) = make_uint4(o2[0], o2[1], o2[2], o2[3]);
  }
}

}  // namespace hyc

using namespace hyc;

extern "C" HYC_API int hyc_rope(const void* x, int64_t ldx, void* out, int64_t ldo, const void* cos_t, const void* sin_t,
                                int64_t ld_table, int table_is_f32, int64_t rows, int seq_len, int n_heads, int head_dim,
                                int backward, void* stream) {
  if (!x || !out || !cos_t || !sin_t) return HYC_ERR_NULL;
  if (rows < 0 || seq_len < 1 || n_heads < 1 || head_dim < 16 || (head_dim & 15) != 0) return HYC_ERR_SHAPE;
  if (ldx < (int64_t)n_heads * head_dim || ldo < (int64_t)n_heads * head_dim || ld_table < head_dim / 2) return HYC_ERR_SHAPE;
  if ((ldx & 7) != 0 || (ldo & 7) != 0 || (ld_table & (table_is_f32 ? 3 : 7)) != 0) return HYC_ERR_ALIGN;
  if (!aligned(x, 16) || !aligned(out, 16) || !aligned(cos_t, 16) || !aligned(sin_t, 16)) return HYC_ERR_ALIGN;
  if (rows == 0) return HYC_OK;
  const int64_t total = rows * n_heads * (head_dim / 16);
  int64_t blocks = (total + 255) / 256;
  const int64_t cap = (int64_t)num_sms() * 8;
  if (blocks > cap) blocks = cap;
  const float sgn = backward ? -1.f : 1.f;
  if (table_is_f32)
    rope_kernel<true><<<(int)blocks, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, ldx, (__nv_bfloat16*)out, ldo, cos_t, sin_t,
                                                                    ld_table, rows, seq_len, n_heads, head_dim, sgn);
  else
    rope_kernel<false><<<(int)blocks, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, ldx, (__nv_bfloat16*)out, ldo, cos_t, sin_t,
                                                                     ld_table, rows, seq_len, n_heads, head_dim, sgn);
  HYC_CHECK_LAUNCH();
  return HYC_OK;
}

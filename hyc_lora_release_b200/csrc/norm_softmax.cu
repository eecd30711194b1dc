// RMSNorm forward/backward and softmax backward: the producers and consumers of the
// compressed tensors.  Plain streaming kernels, one row per block (norm) or per warp
// (softmax), the row held in registers between the reduction and the second pass.
#include "octet_codes.cuh"
#include "topk_lane.cuh"

namespace hyc {

constexpr int kNormThreads = 256;
constexpr int kNormMaxVec = 8;     // 8 x (256 threads x 8 elements) = 16384 columns

__device__ __forceinline__ float block_sum(float v) {
  __shared__ float s_p[kNormThreads / 32];
  __shared__ float s_tot;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if ((threadIdx.x & 31) == 0) s_p[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < kNormThreads / 32; ++i) t += s_p[i];
    s_tot = t;
  }
  __syncthreads();
  float r = s_tot;
  __syncthreads();
  return r;
}

// two sums with one pair of barriers
__device__ __forceinline__ void block_sum2(float a, float b, float& ra, float& rb) {
  __shared__ float2 s_p2[kNormThreads / 32];
  __shared__ float2 s_tot2;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) { a += __shfl_xor_sync(0xffffffffu, a, o); b += __shfl_xor_sync(0xffffffffu, b, o); }
  if ((threadIdx.x & 31) == 0) s_p2[threadIdx.x >> 5] = make_float2(a, b);
  __syncthreads();
  if (threadIdx.x == 0) {
    float ta = 0.f, tb = 0.f;
#pragma unroll
    for (int i = 0; i < kNormThreads / 32; ++i) { ta += s_p2[i].x; tb += s_p2[i].y; }
    s_tot2 = make_float2(ta, tb);
  }
  __syncthreads();
  ra = s_tot2.x; rb = s_tot2.y;
  __syncthreads();
}

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  f[0] = bf16lo_to_f32(v.x); f[1] = bf16hi_to_f32(v.x); f[2] = bf16lo_to_f32(v.y); f[3] = bf16hi_to_f32(v.y);
  f[4] = bf16lo_to_f32(v.z); f[5] = bf16hi_to_f32(v.z); f[6] = bf16lo_to_f32(v.w); f[7] = bf16hi_to_f32(v.w);
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  return make_uint4(pack_bf16x2_rn(f[0], f[1]), pack_bf16x2_rn(f[2], f[3]), pack_bf16x2_rn(f[4], f[5]), pack_bf16x2_rn(f[6], f[7]));
}

template <int NV>
__global__ void __launch_bounds__(kNormThreads)
rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w, float eps,
                   __nv_bfloat16* __restrict__ y, float* __restrict__ rstd, int64_t rows, int N) {
  const int nvec = N / 8;
  // NV octets per thread; the next row of the block is in flight while the current one is reduced and written
  uint4 xnext[NV];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int v = threadIdx.x + i * kNormThreads;
    xnext[i] = make_uint4(0u, 0u, 0u, 0u);
    if (v < nvec && (int64_t)blockIdx.x < rows) xnext[i] = ld_stream_v4(x + (int64_t)blockIdx.x * N + 8 * v);
  }
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    uint4 xv[NV];
    float ss = 0.f;
    const int64_t nrow = row + gridDim.x;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int v = threadIdx.x + i * kNormThreads;
      xv[i] = xnext[i];
      if (v < nvec) {
        if (nrow < rows) xnext[i] = ld_stream_v4(x + nrow * N + 8 * v);
        float f[8]; unpack8(xv[i], f);
#pragma unroll
        for (int e = 0; e < 8; ++e) ss = fmaf(f[e], f[e], ss);
      }
    }
    const float var = block_sum(ss) / (float)N;
    const float rs = 1.f / sqrtf(var + eps);
    if (threadIdx.x == 0) rstd[row] = rs;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int v = threadIdx.x + i * kNormThreads;
      if (v < nvec) {
        float f[8], wf[8];
        unpack8(xv[i], f);
        unpack8(*reinterpret_cast<const uint4*>(w + 8 * v), wf);
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] = (f[e] * rs) * wf[e];
        st_stream_v4(y + row * N + 8 * v, pack8(f));
      }
    }
  }
}

template <int NV>
__global__ void __launch_bounds__(kNormThreads, NV <= 2 ? 4 : 1)
rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                   const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd,
                   __nv_bfloat16* __restrict__ dx, int64_t rows, int N) {
  const int nvec = N / 8;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const float rs = rstd[row];
    uint4 xv[NV], gv[NV];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int v = threadIdx.x + i * kNormThreads;
      if (v < nvec) {
        xv[i] = ld_stream_v4(x + row * N + 8 * v);
        gv[i] = ld_stream_v4(dy + row * N + 8 * v);
        float xf[8], gf[8], wf[8];
        unpack8(xv[i], xf); unpack8(gv[i], gf);
        unpack8(*reinterpret_cast<const uint4*>(w + 8 * v), wf);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float wdy = wf[e] * gf[e];
          s1 = fmaf(xf[e] * rs, wdy, s1);
          s2 += wdy;
        }
      }
    }
    float c1, c2;
    block_sum2(s1, s2, c1, c2);
    c1 /= (float)N; c2 /= (float)N;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int v = threadIdx.x + i * kNormThreads;
      if (v < nvec) {
        float xf[8], gf[8], wf[8];
        unpack8(xv[i], xf); unpack8(gv[i], gf);
        unpack8(*reinterpret_cast<const uint4*>(w + 8 * v), wf);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float wdy = wf[e] * gf[e];
          xf[e] = (wdy - ((xf[e] * rs) * c1 + c2)) * rs;
        }
        st_stream_v4(dx + row * N + 8 * v, pack8(xf));
      }
    }
  }
}

// ---------------------------------------------------------------- RMSNorm fused with the activation saves
// Forward: one pass over x produces x_norm, rstd AND the saved forms of the layer's fused MLP path: the packed
// per-channel codes of x with its outlier channels moved to the outlier slab, and (optionally) the packed
// codes of x_norm.  The results are bit-identical to rmsnorm_fwd_kernel followed by quant_pack_kernel on x
// and on the bf16 x_norm.  A thread owns octets (8 columns); see octet_codes.cuh for the byte layout.
// s_map (dynamic shared memory, N int16): column -> position in the outlier list, -1 = none.
__device__ __forceinline__ void build_full_map(int16_t* s_map, int N, const int64_t* __restrict__ oidx, int k) {
  for (int i = threadIdx.x; i < N / 2; i += blockDim.x) reinterpret_cast<uint32_t*>(s_map)[i] = 0xffffffffu;
  __syncthreads();
  for (int j = threadIdx.x; j < k; j += blockDim.x) {
    const int64_t c = oidx[j];
    if (c >= 0 && c < N) s_map[c] = (int16_t)j;
  }
  __syncthreads();
}

// NV = octets per thread the kernel is built for (N <= NV * 2048 columns).  With NV <= 2 (hidden sizes up to
// 4096) the per-column quantizer constants and the norm weights of the thread's octets stay in registers
// across rows; wider rows form them on the fly.
template <int QBIT, int NV>
__global__ void __launch_bounds__(kNormThreads, NV <= 2 ? 3 : 1)
rmsnorm_fwd_save_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w, float eps,
                        const __nv_bfloat16* __restrict__ scale_x, const int64_t* __restrict__ oidx, int k,
                        const __nv_bfloat16* __restrict__ scale_y,
                        __nv_bfloat16* __restrict__ y, float* __restrict__ rstd, uint8_t* __restrict__ qx,
                        __nv_bfloat16* __restrict__ oout, uint8_t* __restrict__ qy, int64_t rows, int N) {
  extern __shared__ __align__(16) int16_t s_map[];
  constexpr bool CACHED = NV <= 2;
  if (k > 0) build_full_map(s_map, N, oidx, k);
  const int nvec = N / 8;
  const int64_t qld = (int64_t)N * QBIT / 8;
  const uint4 one = make_uint4(0x3f803f80u, 0x3f803f80u, 0x3f803f80u, 0x3f803f80u);
  // per-octet state that does not depend on the row
  uint32_t zmask[NV];
  float rx[CACHED ? NV : 1][8], ry[CACHED ? NV : 1][8];
  uint4 wv[CACHED ? NV : 1];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int v = threadIdx.x + i * kNormThreads;
    zmask[i] = 0u;
    if (v < nvec && k > 0) {
      const uint4 mv = *reinterpret_cast<const uint4*>(s_map + 8 * v);
      const uint32_t mw[4] = {mv.x, mv.y, mv.z, mv.w};
#pragma unroll
      for (int e = 0; e < 8; ++e)
        if ((int)(int16_t)((mw[e >> 1] >> (16 * (e & 1))) & 0xffffu) >= 0) zmask[i] |= 1u << e;
    }
    if (CACHED) {
      const bool ok = v < nvec;
      octet_rcs<QBIT>(ok ? *reinterpret_cast<const uint4*>(scale_x + 8 * v) : one, zmask[i], rx[i]);
      octet_rcs<QBIT>(ok && qy != nullptr ? *reinterpret_cast<const uint4*>(scale_y + 8 * v) : one, 0u, ry[i]);
      wv[i] = ok ? *reinterpret_cast<const uint4*>(w + 8 * v) : one;
    }
  }
  // the next row of the block is fetched while the current one is reduced and written (a block holds one
  // row at a time, so without this every row pays a full memory latency)
  uint4 xnext[NV];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int v = threadIdx.x + i * kNormThreads;
    xnext[i] = make_uint4(0u, 0u, 0u, 0u);
    if (v < nvec && (int64_t)blockIdx.x < rows) xnext[i] = ld_stream_v4(x + (int64_t)blockIdx.x * N + 8 * v);
  }
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    uint4 xv[NV];
    float ss = 0.f;
    const int64_t nrow = row + gridDim.x;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int v = threadIdx.x + i * kNormThreads;
      xv[i] = xnext[i];
      if (v < nvec) {
        if (nrow < rows) xnext[i] = ld_stream_v4(x + nrow * N + 8 * v);
        float f[8]; unpack8(xv[i], f);
#pragma unroll
        for (int e = 0; e < 8; ++e) ss = fmaf(f[e], f[e], ss);
      }
    }
    const float var = block_sum(ss) / (float)N;
    const float rs = 1.f / sqrtf(var + eps);
    if (threadIdx.x == 0) rstd[row] = rs;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      if (i * kNormThreads < nvec) {             // block-uniform: every lane takes part in the shuffles below
        const int v = threadIdx.x + i * kNormThreads;
        const bool ok = v < nvec;
        const int col = 8 * v;
        uint32_t xw[4] = {0u, 0u, 0u, 0u}, yw[4] = {0u, 0u, 0u, 0u};
        if (ok) {
          xw[0] = xv[i].x; xw[1] = xv[i].y; xw[2] = xv[i].z; xw[3] = xv[i].w;
          float f[8], wf[8];
          unpack8(xv[i], f);
          unpack8(CACHED ? wv[CACHED ? i : 0] : *reinterpret_cast<const uint4*>(w + col), wf);
#pragma unroll
          for (int e = 0; e < 8; ++e) f[e] = (f[e] * rs) * wf[e];
          const uint4 yv = pack8(f);
          st_stream_v4(y + row * N + col, yv);
          yw[0] = yv.x; yw[1] = yv.y; yw[2] = yv.z; yw[3] = yv.w;
          if (zmask[i] != 0u) {                  // rare: outlier columns in this octet go to the slab
            for (uint32_t bits = zmask[i]; bits; bits &= bits - 1u) {
              const int e = __ffs(bits) - 1;
              oout[row * k + s_map[col + e]] = __ushort_as_bfloat16((uint16_t)((xw[e >> 1] >> (16 * (e & 1))) & 0xffffu));
            }
          }
        }
        uint32_t kx[2];
        if (CACHED) {
          octet_quant_rcs<QBIT>(xw, rx[CACHED ? i : 0], kx);
        } else {
          octet_quant<QBIT>(xw, ok ? *reinterpret_cast<const uint4*>(scale_x + col) : one, zmask[i], kx);
        }
        octet_store<QBIT>(qx + row * qld, col, kx, ok);
        if (qy != nullptr) {
          uint32_t ky[2];
          if (CACHED) {
            octet_quant_rcs<QBIT>(yw, ry[CACHED ? i : 0], ky);
          } else {
            octet_quant<QBIT>(yw, ok ? *reinterpret_cast<const uint4*>(scale_y + col) : one, 0u, ky);
          }
          octet_store<QBIT>(qy + row * qld, col, ky, ok);
        }
      }
    }
  }
}

// Backward reading the packed x directly: x_hat = de-quantized codes with the outlier columns put back,
// then the arithmetic of rmsnorm_bwd_kernel; `res` (optional) is added to the result as a bf16 tensor add
// (the residual branch of the layer's input gradient).
// NV = octets of a row per thread: rows of up to 4096 columns (NV = 2) leave room for four resident blocks per SM,
// which matters because a block's row is one dependent chain (loads -> two block sums -> stores)
template <int QBIT, int NV>
__global__ void __launch_bounds__(kNormThreads, NV <= 2 ? 4 : 1)
rmsnorm_bwd_packed_kernel(const __nv_bfloat16* __restrict__ dy, const uint8_t* __restrict__ qx,
                          const __nv_bfloat16* __restrict__ scale_x, const int64_t* __restrict__ oidx, int k,
                          const __nv_bfloat16* __restrict__ oin, const __nv_bfloat16* __restrict__ w,
                          const float* __restrict__ rstd, const __nv_bfloat16* __restrict__ res,
                          __nv_bfloat16* __restrict__ dx, int64_t rows, int N) {
  extern __shared__ __align__(16) int16_t s_map[];
  if (k > 0) build_full_map(s_map, N, oidx, k);
  const int nvec = N / 8;
  const int64_t qld = (int64_t)N * QBIT / 8;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const float rs = rstd[row];
    uint4 xv[NV], gv[NV], rv[NV];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int v = threadIdx.x + i * kNormThreads;
      if (v < nvec) {
        const int col = 8 * v;
        gv[i] = ld_stream_v4(dy + row * N + col);
        if (res != nullptr) rv[i] = ld_stream_v4(res + row * N + col);     // needed last, fetched with the rest
        uint32_t xw[4];
        octet_load_dequant<QBIT>(qx + row * qld, col, *reinterpret_cast<const uint4*>(scale_x + col), xw);
        if (k > 0) {
          const uint4 mv = *reinterpret_cast<const uint4*>(s_map + col);
          if ((mv.x & mv.y & mv.z & mv.w) != 0xffffffffu) {
            const uint32_t mw[4] = {mv.x, mv.y, mv.z, mv.w};
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              const int jv = (int)(int16_t)((mw[e >> 1] >> (16 * (e & 1))) & 0xffffu);
              if (jv >= 0) {
                const uint32_t val = (uint32_t)__bfloat16_as_ushort(oin[row * k + jv]);
                xw[e >> 1] = (e & 1) ? ((xw[e >> 1] & 0x0000ffffu) | (val << 16)) : ((xw[e >> 1] & 0xffff0000u) | val);
              }
            }
          }
        }
        xv[i] = make_uint4(xw[0], xw[1], xw[2], xw[3]);
        float xf[8], gf[8], wf[8];
        unpack8(xv[i], xf); unpack8(gv[i], gf);
        unpack8(*reinterpret_cast<const uint4*>(w + col), wf);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float wdy = wf[e] * gf[e];
          s1 = fmaf(xf[e] * rs, wdy, s1);
          s2 += wdy;
        }
      }
    }
    float c1, c2;
    block_sum2(s1, s2, c1, c2);
    c1 /= (float)N; c2 /= (float)N;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int v = threadIdx.x + i * kNormThreads;
      if (v < nvec) {
        float xf[8], gf[8], wf[8];
        unpack8(xv[i], xf); unpack8(gv[i], gf);
        unpack8(*reinterpret_cast<const uint4*>(w + 8 * v), wf);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float wdy = wf[e] * gf[e];
          xf[e] = (wdy - ((xf[e] * rs) * c1 + c2)) * rs;
        }
        uint4 o = pack8(xf);
        if (res != nullptr) {
          const uint4 r = rv[i];
          const __nv_bfloat162* op = reinterpret_cast<const __nv_bfloat162*>(&o);
          const __nv_bfloat162* rp = reinterpret_cast<const __nv_bfloat162*>(&r);
          __nv_bfloat162 t[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) t[j] = __hadd2_rn(op[j], rp[j]);
          o = *reinterpret_cast<const uint4*>(t);
        }
        st_stream_v4(dx + row * N + 8 * v, o);
      }
    }
  }
}

constexpr int kSmMaxVec = 16;   // 16 x (32 lanes x 8 elements) = 4096 columns
__global__ void __launch_bounds__(256)
softmax_bwd_kernel(const __nv_bfloat16* __restrict__ y, const __nv_bfloat16* __restrict__ g,
                   __nv_bfloat16* __restrict__ o, int64_t rows, int S, float oscale) {
  const int lane = threadIdx.x & 31;
  const int nvec = S / 8;
  for (int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5); row < rows; row += (int64_t)gridDim.x * 8) {
    uint4 yv[kSmMaxVec], gv[kSmMaxVec];
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < kSmMaxVec; ++i) {
      const int v = lane + 32 * i;
      if (v < nvec) {
        yv[i] = ld_stream_v4(y + row * S + 8 * v);
        gv[i] = ld_stream_v4(g + row * S + 8 * v);
        float yf[8], gf[8];
        unpack8(yv[i], yf); unpack8(gv[i], gf);
#pragma unroll
        for (int e = 0; e < 8; ++e) acc += bf16bits_to_f32(f32_to_bf16bits_rn(yf[e] * gf[e]));   // y*g is a bf16 product
      }
    }
#pragma unroll
    for (int of = 16; of > 0; of >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, of);
#pragma unroll
    for (int i = 0; i < kSmMaxVec; ++i) {
      const int v = lane + 32 * i;
      if (v < nvec) {
        float yf[8], gf[8];
        unpack8(yv[i], yf); unpack8(gv[i], gf);
#pragma unroll
        for (int e = 0; e < 8; ++e) gf[e] = (gf[e] - acc) * yf[e];
        uint4 r = pack8(gf);
        if (oscale != 1.f) {       // a second bf16 operation on the result
          unpack8(r, gf);
#pragma unroll
          for (int e = 0; e < 8; ++e) gf[e] *= oscale;
          r = pack8(gf);
        }
        st_stream_v4(o + row * S + 8 * v, r);
      }
    }
  }
}


// Attention probabilities from raw scores in one pass (fused_llama_layer_intra_inter_full_fuse.py:150-160:
// `s = q @ k^T / sqrt(d)`, `s = s + attention_mask`, `a = softmax(s, dim=-1, dtype=bf16)`), with the
// reference's rounding points: t = bf16(s * scale), u = bf16(t + mask), fp32 softmax of u, bf16 result.
// One warp per row, the row in registers (NV chunks of 32 lanes x 8 columns).  The mask is addressed as
// mask[b * mb + head * mh + m * mr + column] for row = (b * heads + head) * M + m.
// The exponentials are evaluated twice (once for the row sum, once for the result) instead of keeping the row as
// fp32 values: 80 registers instead of 128, three resident blocks instead of two, half as many bytes again in flight
// (measured at rows of 2048: 115 -> 107 us for the [1,32,2048,2048] map; no difference at rows of 512).
template <int NV>
__global__ void __launch_bounds__(256, NV <= 8 ? 3 : 1)
softmax_fwd_kernel(const __nv_bfloat16* __restrict__ sc, float scale, const __nv_bfloat16* __restrict__ mask,
                   int64_t mb, int64_t mh, int64_t mr, int heads, int M, __nv_bfloat16* __restrict__ a,
                   int64_t rows, int S) {
  const int lane = threadIdx.x & 31;
  const int nvec = S / 8;
  constexpr float kLog2e = 1.4426950408889634f;
  for (int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5); row < rows; row += (int64_t)gridDim.x * 8) {
    const int m = (int)(row % M);
    const int64_t bh = row / M;
    const __nv_bfloat16* mrow = mask ? mask + (bh / heads) * mb + (bh % heads) * mh + (int64_t)m * mr : nullptr;
    // every load of the row is issued before the first use (the scores stream from HBM, the mask comes from L2)
    uint4 raw[NV], mk[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int v = lane + 32 * i;
      raw[i] = make_uint4(0xff80ff80u, 0xff80ff80u, 0xff80ff80u, 0xff80ff80u);      // -inf: columns beyond S
      if (v < nvec) raw[i] = ld_stream_v4(sc + row * S + 8 * v);
    }
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int v = lane + 32 * i;
      mk[i] = make_uint4(0u, 0u, 0u, 0u);
      if (mrow && v < nvec) mk[i] = __ldg(reinterpret_cast<const uint4*>(mrow + 8 * v));
    }
    // t = bf16(bf16(s * scale) + mask), kept as packed bf16 in place of the raw scores
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      float u[8], mf[8];
      unpack8(raw[i], u);
      unpack8(mk[i], mf);
#pragma unroll
      for (int e = 0; e < 8; ++e) u[e] *= scale;
      raw[i] = pack8(u);
      if (mrow) {
        unpack8(raw[i], u);
#pragma unroll
        for (int e = 0; e < 8; ++e) u[e] += mf[e];
        raw[i] = pack8(u);
      }
      unpack8(raw[i], u);
#pragma unroll
      for (int e = 0; e < 8; ++e) mx = fmaxf(mx, u[e]);
    }
#pragma unroll
    for (int of = 16; of > 0; of >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, of));
    const float mxl = mx * kLog2e;
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      float ef[8];
      unpack8(raw[i], ef);
#pragma unroll
      for (int e = 0; e < 8; ++e) sum += exp2f(fmaf(ef[e], kLog2e, -mxl));
    }
#pragma unroll
    for (int of = 16; of > 0; of >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, of);
    const float inv = 1.0f / sum;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int v = lane + 32 * i;
      float ef[8];
      unpack8(raw[i], ef);
#pragma unroll
      for (int e = 0; e < 8; ++e) ef[e] = exp2f(fmaf(ef[e], kLog2e, -mxl)) * inv;
      if (v < nvec) st_stream_v4(a + row * S + 8 * v, pack8(ef));
    }
  }
}

}  // namespace hyc

using namespace hyc;

extern "C" HYC_API int hyc_rmsnorm_fwd(const void* x, const void* w, float eps, void* y, float* rstd,
                               int64_t rows, int N, void* stream) {
  if (!x || !w || !y || !rstd) return HYC_ERR_NULL;
  if (rows < 0 || N <= 0 || N % 8 != 0 || N > kNormThreads * 8 * kNormMaxVec) return HYC_ERR_SHAPE;
  if (!aligned(x, 16) || !aligned(w, 16) || !aligned(y, 16)) return HYC_ERR_ALIGN;
  if (rows == 0) return HYC_OK;
  int64_t grid = rows < (int64_t)num_sms() * 8 ? rows : (int64_t)num_sms() * 8;
  if (N <= 2 * kNormThreads * 8)
    rmsnorm_fwd_kernel<2><<<(int)grid, kNormThreads, 0, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, eps, (__nv_bfloat16*)y, rstd, rows, N);
  else
    rmsnorm_fwd_kernel<kNormMaxVec><<<(int)grid, kNormThreads, 0, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, eps, (__nv_bfloat16*)y, rstd, rows, N);
  HYC_CHECK_LAUNCH();
  return HYC_OK;
}

extern "C" HYC_API int hyc_rmsnorm_fwd_save(const void* x, const void* w, float eps, int64_t rows, int N,
                                            const void* scale_x, const int64_t* outlier_idx, int k, const void* scale_y,
                                            void* y, float* rstd, void* qx, void* outlier_out, void* qy, int q_bit,
                                            void* stream) {
  if (!x || !w || !y || !rstd || !scale_x || !qx) return HYC_ERR_NULL;
  if ((qy != nullptr) != (scale_y != nullptr)) return HYC_ERR_NULL;
  if (q_bit != 2 && q_bit != 4 && q_bit != 8) return HYC_ERR_QBIT;
  if (rows < 0 || N <= 0 || N % 32 != 0 || N > kNormThreads * 8 * kNormMaxVec || k < 0 || k > N || k > 32767) return HYC_ERR_SHAPE;
  if (k > 0 && (!outlier_idx || !outlier_out)) return HYC_ERR_NULL;
  if (!aligned(x, 16) || !aligned(w, 16) || !aligned(y, 16) || !aligned(scale_x, 16) || !aligned(qx, 8) ||
      (qy && (!aligned(qy, 8) || !aligned(scale_y, 16)))) return HYC_ERR_ALIGN;
  if (rows == 0) return HYC_OK;
  // resident blocks only: a block computes its per-column constants and the outlier-column map once, then walks
  // rows with the next row's loads in flight
  const int64_t cap = (int64_t)num_sms() * (N <= 2 * kNormThreads * 8 ? 3 : 1);
  const int64_t grid = rows < cap ? rows : cap;
  const size_t smem = k > 0 ? (size_t)N * 2 : 0;
#define FS(QB) if (N <= 2 * kNormThreads * 8) FSV(QB, 2); else FSV(QB, kNormMaxVec)
#define FSV(QB, NVV) rmsnorm_fwd_save_kernel<QB, NVV><<<(int)grid, kNormThreads, smem, (cudaStream_t)stream>>>(       \
      (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, eps, (const __nv_bfloat16*)scale_x, outlier_idx, k,          \
      (const __nv_bfloat16*)scale_y, (__nv_bfloat16*)y, rstd, (uint8_t*)qx, (__nv_bfloat16*)outlier_out, (uint8_t*)qy, rows, N)
  if (q_bit == 2) { FS(2); } else if (q_bit == 4) { FS(4); } else { FS(8); }
#undef FS
#undef FSV
  HYC_CHECK_LAUNCH();
  return HYC_OK;
}

extern "C" HYC_API int hyc_rmsnorm_bwd_packed(const void* dy, const void* qx, const void* scale_x,
                                              const int64_t* outlier_idx, int k, const void* outlier, const void* w,
                                              const float* rstd, const void* residual_grad, void* dx,
                                              int64_t rows, int N, int q_bit, void* stream) {
  if (!dy || !qx || !scale_x || !w || !rstd || !dx) return HYC_ERR_NULL;
  if (q_bit != 2 && q_bit != 4 && q_bit != 8) return HYC_ERR_QBIT;
  if (rows < 0 || N <= 0 || N % 32 != 0 || N > kNormThreads * 8 * kNormMaxVec || k < 0 || k > N || k > 32767) return HYC_ERR_SHAPE;
  if (k > 0 && (!outlier_idx || !outlier)) return HYC_ERR_NULL;
  if (!aligned(dy, 16) || !aligned(w, 16) || !aligned(dx, 16) || !aligned(scale_x, 16) || !aligned(qx, 8) ||
      (residual_grad && !aligned(residual_grad, 16))) return HYC_ERR_ALIGN;
  if (rows == 0) return HYC_OK;
  // resident blocks only (each block builds the outlier-column map once and then walks rows)
  const int64_t cap = (int64_t)num_sms() * (N <= 2 * kNormThreads * 8 ? 4 : 1);
  const int64_t grid = rows < cap ? rows : cap;
  const size_t smem = k > 0 ? (size_t)N * 2 : 0;
#define BPN(QB, NV) rmsnorm_bwd_packed_kernel<QB, NV><<<(int)grid, kNormThreads, smem, (cudaStream_t)stream>>>(      \
      (const __nv_bfloat16*)dy, (const uint8_t*)qx, (const __nv_bfloat16*)scale_x, outlier_idx, k,                   \
      (const __nv_bfloat16*)outlier, (const __nv_bfloat16*)w, rstd, (const __nv_bfloat16*)residual_grad,             \
      (__nv_bfloat16*)dx, rows, N)
#define BP(QB) do { if (N <= 2 * kNormThreads * 8) BPN(QB, 2); else BPN(QB, kNormMaxVec); } while (0)
  if (q_bit == 2) BP(2); else if (q_bit == 4) BP(4); else BP(8);
#undef BPN
#undef BP
  HYC_CHECK_LAUNCH();
  return HYC_OK;
}

extern "C" HYC_API int hyc_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, void* dx,
                               int64_t rows, int N, void* stream) {
  if (!dy || !x || !w || !rstd || !dx) return HYC_ERR_NULL;
  if (rows < 0 || N <= 0 || N % 8 != 0 || N > kNormThreads * 8 * kNormMaxVec) return HYC_ERR_SHAPE;
  if (!aligned(x, 16) || !aligned(w, 16) || !aligned(dy, 16) || !aligned(dx, 16)) return HYC_ERR_ALIGN;
  if (rows == 0) return HYC_OK;
  int64_t grid = rows < (int64_t)num_sms() * 8 ? rows : (int64_t)num_sms() * 8;
  if (N <= 2 * kNormThreads * 8)
    rmsnorm_bwd_kernel<2><<<(int)grid, kNormThreads, 0, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, rstd, (__nv_bfloat16*)dx, rows, N);
  else
    rmsnorm_bwd_kernel<kNormMaxVec><<<(int)grid, kNormThreads, 0, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, rstd, (__nv_bfloat16*)dx, rows, N);
  HYC_CHECK_LAUNCH();
  return HYC_OK;
}

extern "C" HYC_API int hyc_softmax_bwd(const void* y, const void* g, void* o, int64_t rows, int S, float out_scale, void* stream) {
  if (!y || !g || !o) return HYC_ERR_NULL;
  if (rows < 0 || S <= 0 || S % 8 != 0 || S > 32 * 8 * kSmMaxVec) return HYC_ERR_SHAPE;
  if (!aligned(y, 16) || !aligned(g, 16) || !aligned(o, 16)) return HYC_ERR_ALIGN;
  if (rows == 0) return HYC_OK;
  if (softmax_bwd_lane(y, g, rows, S, out_scale, o, (cudaStream_t)stream)) {   // rows of 64 * 2^n columns: staged, coalesced
    HYC_CHECK_LAUNCH();
    return HYC_OK;
  }
  int64_t grid = (rows + 7) / 8;
  if (grid > (int64_t)num_sms() * 8) grid = (int64_t)num_sms() * 8;
  softmax_bwd_kernel<<<(int)grid, 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)y, (const __nv_bfloat16*)g, (__nv_bfloat16*)o, rows, S, out_scale);
  HYC_CHECK_LAUNCH();
  return HYC_OK;
}

extern "C" HYC_API int hyc_softmax_fwd_scale_mask(const void* scores, float scale, const void* mask_or_null, int64_t mask_stride_b,
                                                  int64_t mask_stride_h, int64_t mask_stride_row, int heads, int M, void* a,
                                                  int64_t rows, int S, void* stream) {
  if (!scores || !a) return HYC_ERR_NULL;
  if (rows < 0 || S <= 0 || S % 8 != 0 || S > 32 * 8 * kSmMaxVec || heads < 1 || M < 1) return HYC_ERR_SHAPE;
  if (!aligned(scores, 16) || !aligned(a, 16)) return HYC_ERR_ALIGN;
  if (mask_or_null && (!aligned(mask_or_null, 16) || (mask_stride_b & 7) || (mask_stride_h & 7) || (mask_stride_row & 7))) return HYC_ERR_ALIGN;
  if (rows == 0) return HYC_OK;
  int64_t grid = (rows + 7) / 8;
  if (grid > (int64_t)num_sms() * 8) grid = (int64_t)num_sms() * 8;
#define SF(NV) softmax_fwd_kernel<NV><<<(int)grid, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)scores, scale, \
      (const __nv_bfloat16*)mask_or_null, mask_stride_b, mask_stride_h, mask_stride_row, heads, M, (__nv_bfloat16*)a, rows, S)
  if (S <= 512) SF(2); else if (S <= 1024) SF(4); else if (S <= 2048) SF(8); else SF(16);
#undef SF
  HYC_CHECK_LAUNCH();
  return HYC_OK;
}

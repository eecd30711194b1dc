// Attention-map threshold prune: the COO list of the flattened map entries above a global
// threshold, and its dense restore.  The list is ordered by flattened index, so the
// compaction is a two-phase stream compaction: per-tile counts, a scan of the counts,
// then the ordered fill.  The workspace holds [0] = total, [1 + t] = exclusive offset of tile t.
#include "hyc_common.cuh"
#include <string.h>

namespace hyc {

constexpr int kTileThreads = 256;
constexpr int kTileElems = kTileThreads * 16;   // 4096 elements (8 KiB) per tile

__device__ __forceinline__ uint32_t keep_mask16(const uint32_t (&w)[8], float thr, int64_t base, int64_t numel) {
  uint32_t mk = 0u;
#pragma unroll
  for (int e = 0; e < 16; ++e) {
    float f = (e & 1) ? bf16hi_to_f32(w[e >> 1]) : bf16lo_to_f32(w[e >> 1]);
    if (f > thr && f != 0.f && (base + e) < numel) mk |= 1u << e;
  }
  return mk;
}

__device__ __forceinline__ void load16(const __nv_bfloat16* a, int64_t base, int64_t numel, uint32_t (&w)[8]) {
  if (base + 16 <= numel) {
    uint4 u = ld_stream_v4(a + base), v = ld_stream_v4(a + base + 8);
    w[0] = u.x; w[1] = u.y; w[2] = u.z; w[3] = u.w; w[4] = v.x; w[5] = v.y; w[6] = v.z; w[7] = v.w;
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      uint32_t lo = (base + 2 * j < numel) ? __bfloat16_as_ushort(a[base + 2 * j]) : 0u;
      uint32_t hi = (base + 2 * j + 1 < numel) ? __bfloat16_as_ushort(a[base + 2 * j + 1]) : 0u;
      w[j] = lo | (hi << 16);
    }
  }
}

__device__ __forceinline__ int block_excl_scan(int v, int& total) {
  __shared__ int s_w[kTileThreads / 32];
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  int incl = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    int t = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += t;
  }
  if (lane == 31) s_w[wid] = incl;
  __syncthreads();
  int wbase = 0, tot = 0;
#pragma unroll
  for (int i = 0; i < kTileThreads / 32; ++i) {
    int c = s_w[i];
    if (i < wid) wbase += c;
    tot += c;
  }
  total = tot;
  __syncthreads();
  return wbase + incl - v;
}

__global__ void __launch_bounds__(kTileThreads)
prune_count_kernel(const __nv_bfloat16* __restrict__ a, int64_t numel, float thr, int64_t n_tiles,
                   int64_t* __restrict__ ws) {
  for (int64_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
    const int64_t base = tile * kTileElems + 16 * (int64_t)threadIdx.x;
    uint32_t w[8];
    int c = 0;
    if (base < numel) { load16(a, base, numel, w); c = __popc(keep_mask16(w, thr, base, numel)); }
    int total;
    block_excl_scan(c, total);
    if (threadIdx.x == 0) ws[1 + tile] = total;
  }
}

// single block: counts -> exclusive offsets, total into ws[0]
__global__ void __launch_bounds__(1024)
prune_scan_kernel(int64_t* __restrict__ ws, int64_t n_tiles) {
  __shared__ int64_t s_part[1024];
  const int64_t per = (n_tiles + 1023) / 1024;
  const int64_t b = threadIdx.x * per, e = (b + per < n_tiles) ? b + per : n_tiles;
  int64_t sum = 0;
  for (int64_t i = b; i < e; ++i) sum += ws[1 + i];
  s_part[threadIdx.x] = sum;
  __syncthreads();
  if (threadIdx.x == 0) {
    int64_t run = 0;
    for (int i = 0; i < 1024; ++i) { int64_t t = s_part[i]; s_part[i] = run; run += t; }
    ws[0] = run;
  }
  __syncthreads();
  int64_t run = s_part[threadIdx.x];
  for (int64_t i = b; i < e; ++i) { int64_t t = ws[1 + i]; ws[1 + i] = run; run += t; }
}

__global__ void __launch_bounds__(kTileThreads)
prune_fill_kernel(const __nv_bfloat16* __restrict__ a, int64_t numel, float thr, int64_t n_tiles,
                  const int64_t* __restrict__ ws, int64_t* __restrict__ idx_out,
                  __nv_bfloat16* __restrict__ val_out, int64_t capacity) {
  for (int64_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
    const int64_t base = tile * kTileElems + 16 * (int64_t)threadIdx.x;
    uint32_t w[8];
    uint32_t mk = 0u;
    if (base < numel) { load16(a, base, numel, w); mk = keep_mask16(w, thr, base, numel); }
    int total;
    int64_t pos = ws[1 + tile] + block_excl_scan(__popc(mk), total);
#pragma unroll
    for (int e = 0; e < 16; ++e) {
      if (mk & (1u << e)) {
        if (pos < capacity) {
          idx_out[pos] = base + e;
          const uint32_t ww = w[e >> 1];
          val_out[pos] = __ushort_as_bfloat16((e & 1) ? (uint16_t)(ww >> 16) : (uint16_t)(ww & 0xffffu));
        }
        ++pos;
      }
    }
  }
}

__global__ void __launch_bounds__(256)
prune_scatter_kernel(const int64_t* __restrict__ idx, const __nv_bfloat16* __restrict__ val, int64_t nnz,
                     __nv_bfloat16* __restrict__ out, int64_t numel) {
  for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < nnz; i += (int64_t)gridDim.x * 256) {
    const int64_t p = idx[i];
    if (p >= 0 && p < numel) out[p] = val[i];
  }
}

static inline int64_t n_tiles_of(int64_t numel) { return (numel + kTileElems - 1) / kTileElems; }
static inline int tile_grid(int64_t n_tiles) {
  int64_t g = n_tiles < (int64_t)kNumSMs * 8 ? n_tiles : (int64_t)kNumSMs * 8;
  return (int)(g < 1 ? 1 : g);
}
// the comparison of the reference runs in bf16: the fp32 threshold is rounded to bf16 first
static inline float thr_bf16(float t) {
  uint32_t u; memcpy(&u, &t, 4);
  if ((u & 0x7f800000u) != 0x7f800000u) u += 0x7fffu + ((u >> 16) & 1u);
  u &= 0xffff0000u;
  float r; memcpy(&r, &u, 4);
  return r;
}

}  // namespace hyc

using namespace hyc;

extern "C" HYC_API size_t hyc_softmax_prune_workspace_bytes(int64_t numel) {
  if (numel < 0) return 0;
  return (size_t)(1 + n_tiles_of(numel)) * sizeof(int64_t);
}

extern "C" HYC_API int hyc_softmax_prune_count(const void* a, int64_t numel, float threshold,
                                       void* workspace, size_t workspace_bytes, void* stream) {
  if (!a || !workspace) return HYC_ERR_NULL;
  if (numel <= 0) return HYC_ERR_SHAPE;
  if (!aligned(a, 16) || !aligned(workspace, 8)) return HYC_ERR_ALIGN;
  if (workspace_bytes < hyc_softmax_prune_workspace_bytes(numel)) return HYC_ERR_WORKSPACE;
  const int64_t nt = n_tiles_of(numel);
  cudaStream_t st = (cudaStream_t)stream;
  prune_count_kernel<<<tile_grid(nt), kTileThreads, 0, st>>>((const __nv_bfloat16*)a, numel, thr_bf16(threshold), nt,
                                                              (int64_t*)workspace);
  HYC_CHECK_LAUNCH();
  prune_scan_kernel<<<1, 1024, 0, st>>>((int64_t*)workspace, nt);
  HYC_CHECK_LAUNCH();
  return HYC_OK;
}

extern "C" HYC_API int hyc_softmax_prune_fill(const void* a, int64_t numel, float threshold,
                                      const void* workspace, int64_t* idx_out, void* val_out,
                                      int64_t capacity, void* stream) {
  if (!a || !workspace) return HYC_ERR_NULL;
  if (capacity > 0 && (!idx_out || !val_out)) return HYC_ERR_NULL;
  if (numel <= 0 || capacity < 0) return HYC_ERR_SHAPE;
  if (!aligned(a, 16) || !aligned(workspace, 8)) return HYC_ERR_ALIGN;
  if (capacity == 0) return HYC_OK;
  const int64_t nt = n_tiles_of(numel);
  prune_fill_kernel<<<tile_grid(nt), kTileThreads, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)a, numel, thr_bf16(threshold), nt, (const int64_t*)workspace, idx_out,
      (__nv_bfloat16*)val_out, capacity);
  HYC_CHECK_LAUNCH();
  return HYC_OK;
}

extern "C" HYC_API int hyc_softmax_prune_restore(const int64_t* idx, const void* val, int64_t nnz,
                                         void* a_out, int64_t numel, void* stream) {
  if (!a_out || (nnz > 0 && (!idx || !val))) return HYC_ERR_NULL;
  if (numel <= 0 || nnz < 0) return HYC_ERR_SHAPE;
  cudaStream_t st = (cudaStream_t)stream;
  if (cudaMemsetAsync(a_out, 0, (size_t)numel * 2, st) != cudaSuccess) { hyc_set_last_cuda_error((int)cudaGetLastError()); return HYC_ERR_LAUNCH; }
  if (nnz > 0) {
    int64_t g = (nnz + 255) / 256;
    if (g > (int64_t)kNumSMs * 16) g = (int64_t)kNumSMs * 16;
    prune_scatter_kernel<<<(int)g, 256, 0, st>>>(idx, (const __nv_bfloat16*)val, nnz, (__nv_bfloat16*)a_out, numel);
    HYC_CHECK_LAUNCH();
  }
  return HYC_OK;
}

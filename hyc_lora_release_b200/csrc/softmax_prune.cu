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

// the same with the number of entries read from device memory (a count that was never copied to the host)
__global__ void __launch_bounds__(256)
prune_scatter_counted_kernel(const int64_t* __restrict__ idx, const __nv_bfloat16* __restrict__ val,
                             const int64_t* __restrict__ nnz_dev, int64_t capacity,
                             __nv_bfloat16* __restrict__ out, int64_t numel) {
  int64_t nnz = *nnz_dev;
  if (nnz > capacity) nnz = capacity;
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

extern "C" HYC_API int hyc_softmax_prune_restore_counted(const int64_t* idx, const void* val, const int64_t* nnz_dev,
                                                         int64_t capacity, void* a_out, int64_t numel, void* stream) {
  if (!a_out || !nnz_dev || (capacity > 0 && (!idx || !val))) return HYC_ERR_NULL;
  if (numel <= 0 || capacity < 0) return HYC_ERR_SHAPE;
  cudaStream_t st = (cudaStream_t)stream;
  if (cudaMemsetAsync(a_out, 0, (size_t)numel * 2, st) != cudaSuccess) { hyc_set_last_cuda_error((int)cudaGetLastError()); return HYC_ERR_LAUNCH; }
  if (capacity > 0) {
    int64_t g = (capacity + 255) / 256;
    if (g > (int64_t)kNumSMs * 16) g = (int64_t)kNumSMs * 16;
    prune_scatter_counted_kernel<<<(int)g, 256, 0, st>>>(idx, (const __nv_bfloat16*)val, nnz_dev, capacity,
                                                         (__nv_bfloat16*)a_out, numel);
    HYC_CHECK_LAUNCH();
  }
  return HYC_OK;
}

// ---------------------------------------------------------------------------------------------
// Variant for callers that must not allocate device memory when they call: a training loop whose
// HBM is handed out up front by a fixed memory plan, or a host framework that forbids allocation
// inside an operator callback, has no buffer to offer as the count/fill workspace.  Here the tile
// offsets live in a file-scope device array instead, so the whole compaction is ONE call that
// allocates nothing.
//
//   * The array holds kStaticMaxTiles + 1 int64 (512 KiB + 8 B) and stays resident on every GPU
//     that loads the library until the process exits.  Maps of more than kStaticMaxTiles * 4096
//     elements (268,435,456) are refused with HYC_ERR_CAPACITY.
//   * The first call on a device looks the array's device address up (cudaGetSymbolAddress, with
//     that device current) and remembers it; make that first call outside of any stream capture.
//   * All calls on a device share the array.  Every entry a call reads is written by that same
//     call first (the count kernel writes each tile's slot, the scan writes the total), so nothing
//     has to be cleared between calls; but two calls that overlap on the GPU (different streams)
//     would race on it.  Serialise them.
constexpr int64_t kStaticMaxTiles = 65536;
static __device__ __align__(256) int64_t g_prune_offsets[1 + kStaticMaxTiles];

static int64_t* static_offsets_for_current_device(int* err) {
  static int64_t* cached[64] = {nullptr};
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= 64) { *err = (int)(e != cudaSuccess ? e : cudaErrorInvalidDevice); return nullptr; }
  if (cached[dev] == nullptr) {
    // g_prune_offsets is a host-side handle here, not a device address: ask the runtime for the address
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_prune_offsets);
    if (e != cudaSuccess || p == nullptr) { *err = (int)e; return nullptr; }
    cached[dev] = reinterpret_cast<int64_t*>(p);
  }
  return cached[dev];
}

extern "C" HYC_API int hyc_softmax_prune_static(const void* a, int64_t numel, float threshold,
                                                int64_t* idx_out, void* val_out, int64_t capacity,
                                                int64_t* nnz_out, void* stream) {
  if (!a || !nnz_out) return HYC_ERR_NULL;
  if (capacity > 0 && (!idx_out || !val_out)) return HYC_ERR_NULL;
  if (numel <= 0 || capacity < 0) return HYC_ERR_SHAPE;
  if (!aligned(a, 16) || !aligned(nnz_out, 8)) return HYC_ERR_ALIGN;
  const int64_t nt = n_tiles_of(numel);
  if (nt > kStaticMaxTiles) return HYC_ERR_CAPACITY;   // map too large for the built-in scratch
  int err = 0;
  int64_t* ws = static_offsets_for_current_device(&err);
  if (!ws) { hyc_set_last_cuda_error(err); return HYC_ERR_LAUNCH; }
  cudaStream_t st = (cudaStream_t)stream;
  const float thr = thr_bf16(threshold);
  prune_count_kernel<<<tile_grid(nt), kTileThreads, 0, st>>>((const __nv_bfloat16*)a, numel, thr, nt, ws);
  HYC_CHECK_LAUNCH();
  prune_scan_kernel<<<1, 1024, 0, st>>>(ws, nt);
  HYC_CHECK_LAUNCH();
  if (capacity > 0) {
    prune_fill_kernel<<<tile_grid(nt), kTileThreads, 0, st>>>((const __nv_bfloat16*)a, numel, thr, nt, ws, idx_out,
                                                              (__nv_bfloat16*)val_out, capacity);
    HYC_CHECK_LAUNCH();
  }
  if (cudaMemcpyAsync(nnz_out, ws, sizeof(int64_t), cudaMemcpyDeviceToDevice, st) != cudaSuccess) {
    hyc_set_last_cuda_error((int)cudaGetLastError());
    return HYC_ERR_LAUNCH;
  }
  return HYC_OK;
}

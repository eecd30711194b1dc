// Attention-map threshold prune: the COO list of the flattened map entries above a global
// threshold, and its dense restore.  The list is ordered by flattened index, so the
// compaction is a two-phase stream compaction: per-tile counts, a scan of the counts,
// then the ordered fill.  The workspace holds [0] = total, [1 + t] = exclusive offset of tile t.
// Both passes over the map give a tile of 4096 elements to a warp (no block-wide barriers) and test two
// elements per instruction with packed bf16 compares.
#include "hyc_common.cuh"
#include <string.h>

namespace hyc {

constexpr int kTileThreads = 256;
constexpr int kTileElems = 4096;                // elements (8 KiB) per tile: the unit of the offsets in the workspace
constexpr int kWarpsPerBlock = kTileThreads / 32;

// A WARP owns a tile.  Chunk c of the tile (8 elements, 16 bytes) is read by lane c % 32 in trip c / 32, so that every
// load instruction of the warp covers 512 contiguous bytes and a lane has several independent loads in flight.

// one chunk of 8 elements starting at element `base` (a multiple of 8); elements at or beyond numel read as zero.
// LAST: the final read of the map (evict-first); the counting pass reads with the default policy so that a map
// smaller than the L2 is still there when the fill pass comes.
template <bool LAST>
__device__ __forceinline__ uint4 load_chunk(const __nv_bfloat16* a, int64_t base, int64_t numel) {
  if (base + 8 <= numel) return LAST ? ld_stream_v4(a + base) : __ldg(reinterpret_cast<const uint4*>(a + base));
  uint32_t w[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const uint32_t lo = (base + 2 * j < numel) ? __bfloat16_as_ushort(a[base + 2 * j]) : 0u;
    const uint32_t hi = (base + 2 * j + 1 < numel) ? __bfloat16_as_ushort(a[base + 2 * j + 1]) : 0u;
    w[j] = lo | (hi << 16);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

// The keep test `x > thr && x != 0` (a zero is no entry of a sparse tensor) on packed bf16 pairs: one compare
// instruction per two elements gives 0xffff per kept half.  For thr >= 0 the first condition implies the second
// (NEG = false); a NaN is never kept, as in the fp32 comparison.
template <bool NEG>
__device__ __forceinline__ uint32_t pair_mask(uint32_t w, __nv_bfloat162 t2) {
  const __nv_bfloat162 x = *reinterpret_cast<const __nv_bfloat162*>(&w);
  uint32_t m = __hgt2_mask(x, t2);
  if (NEG) m &= __hne2_mask(x, __float2bfloat162_rn(0.f));
  return m;
}
// one bit per kept element of the chunk: element 2j at bit 2j, element 2j + 1 at bit 16 + 2j + 1
template <bool NEG>
__device__ __forceinline__ uint32_t keep_bits(const uint4& u, __nv_bfloat162 t2) {
  return (pair_mask<NEG>(u.x, t2) & 0x00020001u) | (pair_mask<NEG>(u.y, t2) & 0x00080004u) |
         (pair_mask<NEG>(u.z, t2) & 0x00200010u) | (pair_mask<NEG>(u.w, t2) & 0x00800040u);
}
// bit e set: element e of the chunk is kept
template <bool NEG>
__device__ __forceinline__ uint32_t keep_mask8(const uint4& u, __nv_bfloat162 t2) {
  const uint32_t t = keep_bits<NEG>(u, t2);
  return (t | (t >> 16)) & 0xffu;
}

__device__ __forceinline__ int warp_excl_scan(int v, int lane, int& total) {
  int incl = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int t = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += t;
  }
  total = __shfl_sync(0xffffffffu, incl, 31);
  return incl - v;
}

// (four loads in flight per lane and 32 registers: all 64 warp slots of an SM are taken, one wave for 9472 tiles)
template <bool NEG>
__global__ void __launch_bounds__(kTileThreads, 8)
prune_count_kernel(const __nv_bfloat16* __restrict__ a, int64_t numel, float thr, int64_t n_tiles,
                   int64_t* __restrict__ ws) {
  constexpr int CB = 4;
  const __nv_bfloat162 t2 = __float2bfloat162_rn(thr);
  const int lane = threadIdx.x & 31;
  const int64_t warp0 = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  for (int64_t tile = warp0; tile < n_tiles; tile += (int64_t)gridDim.x * kWarpsPerBlock) {
    const int64_t t0 = tile * kTileElems + 8 * lane;
    int c = 0;
#pragma unroll
    for (int b = 0; b < kTileElems / (256 * CB); ++b) {
      uint4 u[CB];
#pragma unroll
      for (int j = 0; j < CB; ++j) {
        const int64_t base = t0 + 256 * (b * CB + j);
        u[j] = base < numel ? load_chunk<false>(a, base, numel) : make_uint4(0u, 0u, 0u, 0u);
      }
#pragma unroll
      for (int j = 0; j < CB; ++j) c += __popc(keep_bits<NEG>(u[j], t2));
    }
    c = (int)__reduce_add_sync(0xffffffffu, (unsigned)c);
    if (lane == 0) ws[1 + tile] = c;
  }
}

// single block: counts -> exclusive offsets, total into ws[0] (and into *total_out when given).  The counts are
// taken 8192 at a time: every thread fetches eight of them (coalesced, all eight loads in flight), then eight
// block-wide scans chained by a carry.
__global__ void __launch_bounds__(1024)
prune_scan_kernel(int64_t* __restrict__ ws, int64_t n_tiles, int64_t* __restrict__ total_out) {
  constexpr int U = 8;
  __shared__ int64_t s_off[U][32];      // per scan: inclusive warp totals, then the warps' exclusive offsets
  __shared__ int64_t s_tot[U];
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  int64_t carry = 0;
  for (int64_t c0 = 0; c0 < n_tiles; c0 += 1024 * U) {
    int64_t v[U], incl[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t i = c0 + 1024 * u + threadIdx.x;
      v[u] = i < n_tiles ? ws[1 + i] : 0;
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      int64_t x = v[u];
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int64_t t = __shfl_up_sync(0xffffffffu, x, o);
        if (lane >= o) x += t;
      }
      incl[u] = x;
      if (lane == 31) s_off[u][wid] = x;
    }
    __syncthreads();
    if (wid < U) {
      const int64_t t0 = s_off[wid][lane];
      int64_t x = t0;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int64_t t = __shfl_up_sync(0xffffffffu, x, o);
        if (lane >= o) x += t;
      }
      s_off[wid][lane] = x - t0;
      if (lane == 31) s_tot[wid] = x;
    }
    __syncthreads();
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t i = c0 + 1024 * u + threadIdx.x;
      if (i < n_tiles) ws[1 + i] = carry + s_off[u][wid] + incl[u] - v[u];
      carry += s_tot[u];
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    ws[0] = carry;
    if (total_out) *total_out = carry;
  }
}

// Ordered fill.  The entries of four trips (1024 elements) are first packed into a per-warp staging area in list
// order as (offset within the 1024 << 16 | value), then written out by consecutive lanes: a list entry is 8 + 2
// bytes, and one store instruction per entry and lane would cost a 32-byte memory transaction for each of them.
// The work per trip does not depend on how the kept entries are spread over the lanes (in a causal map they
// cluster: the first rows keep everything, the masked half keeps nothing); a trip without any entry is skipped.
constexpr int kBatch = 8;                       // chunks a lane has in flight: a tile is two batches
constexpr int kFillTrips = 4;

template <bool NEG>
__global__ void __launch_bounds__(kTileThreads, 4)
prune_fill_kernel(const __nv_bfloat16* __restrict__ a, int64_t numel, float thr, int64_t n_tiles,
                  const int64_t* __restrict__ ws, int64_t* __restrict__ idx_out,
                  __nv_bfloat16* __restrict__ val_out, int64_t capacity) {
  __shared__ uint32_t s_stage[kWarpsPerBlock][256 * kFillTrips];
  const __nv_bfloat162 t2 = __float2bfloat162_rn(thr);
  const int lane = threadIdx.x & 31;
  uint32_t* stage = s_stage[threadIdx.x >> 5];
  const int64_t warp0 = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  for (int64_t tile = warp0; tile < n_tiles; tile += (int64_t)gridDim.x * kWarpsPerBlock) {
    const int64_t t0 = tile * kTileElems + 8 * lane;
    int64_t run = ws[1 + tile];            // list position of the tile's first entry
#pragma unroll
    for (int b = 0; b < kTileElems / (256 * kBatch); ++b) {
      uint4 u[kBatch];
#pragma unroll
      for (int j = 0; j < kBatch; ++j) {
        const int64_t base = t0 + 256 * (b * kBatch + j);
        u[j] = base < numel ? load_chunk<true>(a, base, numel) : make_uint4(0u, 0u, 0u, 0u);
      }
#pragma unroll
      for (int g = 0; g < kBatch / kFillTrips; ++g) {
        int n_staged = 0;
#pragma unroll
        for (int jj = 0; jj < kFillTrips; ++jj) {
          // the entries of one trip (256 consecutive elements) are consecutive in the list: lanes in order
          const int j = g * kFillTrips + jj;
          const uint32_t mk = keep_mask8<NEG>(u[j], t2);
          if (__any_sync(0xffffffffu, mk != 0u)) {
            int total;
            int pos = n_staged + warp_excl_scan(__popc(mk), lane, total);
            n_staged += total;
            const uint32_t w[4] = {u[j].x, u[j].y, u[j].z, u[j].w};
            const uint32_t off = (uint32_t)(256 * jj + 8 * lane);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              if (mk & (1u << e)) stage[pos++] = __byte_perm(w[e >> 1], off + e, (e & 1) ? 0x5432 : 0x5410);
            }
          }
        }
        if (n_staged) {
          __syncwarp();
          const int64_t g0 = tile * kTileElems + 256 * (b * kBatch + g * kFillTrips);   // element index of offset 0
          for (int i = lane; i < n_staged; i += 32) {
            const int64_t p = run + i;
            if (p < capacity) {
              const uint32_t wv = stage[i];
              idx_out[p] = g0 + (int64_t)(wv >> 16);
              val_out[p] = __ushort_as_bfloat16((uint16_t)(wv & 0xffffu));
            }
          }
          run += n_staged;
          __syncwarp();
        }
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

// One-pass, tiled form for callers that only ever restore the map (the fused layer in steady state): the map is
// read once, there is no offset array and no second launch, and an entry costs 4 bytes instead of 10.
// A BATCH is 2048 consecutive elements (half a tile).  A warp stages the entries of a batch in shared memory as
// (offset within the batch << 16 | bf16 value) words, reserves a span of the word list with ONE atomic add on the
// device-side count, writes the span with consecutive lanes and records {span start, entries} in the batch's
// directory slot.  Which span a batch gets depends on the order in which the warps arrive; inside a span the
// entries of a lane are adjacent (the order is fixed, but not ascending).
// One counter for the whole list would be the bottleneck: sixteen thousand atomic adds on ONE address take about as
// long as reading the map.  The word list is therefore cut into kSubLists equal sub-lists with a counter each (128
// bytes apart, behind the directory), and a batch takes its span from the sub-list its hashed index names, so every
// sub-list receives a pseudo-random sample of the batches and fills evenly.  A span that does not fit its sub-list is
// cut short (the directory records what was written); a last one-block kernel adds the counters up: *nnz_out = the
// number of kept entries if everything fit, else capacity + the number of entries that were dropped.  Small maps
// use fewer sub-lists (at least 32 batches each, so that the sample averages out), down to a single one, which
// never drops anything that `capacity` could hold.
constexpr int kBatchElems = 256 * kBatch;       // 2048
constexpr int kSubLists = 64;
constexpr int kCounterStride = 16;              // unsigned long long per counter slot (128 bytes)

__host__ __device__ inline uint32_t tiled_sub_lists(int64_t numel) {
  const int64_t nb = (numel + kBatchElems - 1) / kBatchElems;
  const int64_t n = nb / 32;
  return (uint32_t)(n < 1 ? 1 : (n > kSubLists ? kSubLists : n));
}
__host__ __device__ inline int64_t tiled_dir_entries(int64_t numel) {
  const int64_t nb = (numel + kBatchElems - 1) / kBatchElems;
  return (nb + 15) & ~(int64_t)15;              // the counters behind it start on a 128-byte boundary
}

// sub-list counters -> *nnz_out: kept entries, or capacity + dropped entries when a sub-list overflowed
__device__ __forceinline__ void tiled_finish(const unsigned long long* counters, uint32_t capacity, uint32_t n_sub,
                                             int64_t* __restrict__ nnz_out, unsigned long long* s_kd) {
  if (threadIdx.x < 64) {
    const uint32_t sub_cap = capacity / n_sub;
    const unsigned long long c = threadIdx.x < n_sub ? __ldcg(counters + threadIdx.x * kCounterStride) : 0ull;
    unsigned long long kept = c, dropped = c > sub_cap ? c - sub_cap : 0ull;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      kept += __shfl_xor_sync(0xffffffffu, kept, o);
      dropped += __shfl_xor_sync(0xffffffffu, dropped, o);
    }
    if ((threadIdx.x & 31) == 0) { s_kd[threadIdx.x >> 5] = kept; s_kd[2 + (threadIdx.x >> 5)] = dropped; }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned long long k = s_kd[0] + s_kd[1], d = s_kd[2] + s_kd[3];
    *nnz_out = (int64_t)(d ? (unsigned long long)capacity + d : k);
  }
}

template <bool NEG>
__global__ void __launch_bounds__(kTileThreads, 4)
prune_tiled_kernel(const __nv_bfloat16* __restrict__ a, int64_t numel, float thr, int64_t n_tiles,
                   uint32_t* __restrict__ words, uint32_t capacity, uint2* __restrict__ dir,
                   unsigned long long* __restrict__ counters, int64_t* __restrict__ nnz_out) {
  // A warp walks batches with a fixed stride.  Per batch: masks and counts from the eight chunks in registers, ONE
  // atomic add for the span, the entries staged in shared memory, and -- before anything waits for the atomic's
  // answer -- the loads of the warp's NEXT batch: the round trip of the atomic and the write-out of this batch run
  // while those loads are in flight.  (A batch with more than 1024 entries, i.e. more than the staging area holds,
  // takes the plain sequence: group by group, next loads afterwards.)
  __shared__ uint32_t s_stage[kWarpsPerBlock][256 * kFillTrips];
  const __nv_bfloat162 t2 = __float2bfloat162_rn(thr);
  const int lane = threadIdx.x & 31;
  uint32_t* stage = s_stage[threadIdx.x >> 5];
  const int64_t n_batches = (numel + kBatchElems - 1) / kBatchElems;
  const int64_t stride = (int64_t)gridDim.x * kWarpsPerBlock;
  int64_t batch = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  const uint32_t n_sub = tiled_sub_lists(numel);
  const uint32_t sub_cap = capacity / n_sub;          // words per sub-list
  (void)n_tiles;
  uint4 u[kBatch];
  auto load_batch = [&](int64_t bt) {
    const int64_t t0 = bt * kBatchElems + 8 * lane;
#pragma unroll
    for (int j = 0; j < kBatch; ++j) {
      const int64_t base = t0 + 256 * j;
      u[j] = base < numel ? load_chunk<true>(a, base, numel) : make_uint4(0u, 0u, 0u, 0u);
    }
  };
  // entries of group g (four trips) into the staging area from position `pos` on, lanes in order
  auto stage_group = [&](int g, uint32_t mkg, int pos) {
#pragma unroll
    for (int jj = 0; jj < kFillTrips; ++jj) {
      const int j = g * kFillTrips + jj;
      const uint32_t w[4] = {u[j].x, u[j].y, u[j].z, u[j].w};
      const uint32_t off = (uint32_t)(256 * j + 8 * lane);        // offset inside the batch
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        if (mkg & (1u << (8 * jj + e))) stage[pos++] = __byte_perm(w[e >> 1], off + e, (e & 1) ? 0x5432 : 0x5410);
      }
    }
  };
  if (batch < n_batches) load_batch(batch);
  while (batch < n_batches) {
    uint32_t mk[kBatch / kFillTrips];      // the keep masks of a group's four trips, one byte each
    int cg[kBatch / kFillTrips];
#pragma unroll
    for (int g = 0; g < kBatch / kFillTrips; ++g) {
      mk[g] = 0u;
#pragma unroll
      for (int jj = 0; jj < kFillTrips; ++jj) mk[g] |= keep_mask8<NEG>(u[g * kFillTrips + jj], t2) << (8 * jj);
      cg[g] = __popc(mk[g]);
    }
    // both group totals in one reduction (a group holds at most 1024 entries)
    const unsigned packed = __reduce_add_sync(0xffffffffu, (unsigned)cg[0] | ((unsigned)cg[1] << 16));
    const int n0 = (int)(packed & 0xffffu), n1 = (int)(packed >> 16);
    const unsigned n_batch = (unsigned)(n0 + n1);
    // span = {first word, words that fit}: from the sub-list the hashed batch index names
    uint2 span = make_uint2(0u, 0u);
    if (lane == 0) {
      if (n_batch) {
        const uint32_t sub = __umulhi((uint32_t)batch * 0x9E3779B1u, n_sub);
        const unsigned long long at = atomicAdd(counters + sub * kCounterStride, (unsigned long long)n_batch);
        const uint32_t room = at < sub_cap ? sub_cap - (uint32_t)at : 0u;
        span = make_uint2(sub * sub_cap + (uint32_t)(at < sub_cap ? at : 0), n_batch < room ? n_batch : room);
      }
      dir[batch] = span;
    }
    const int64_t next = batch + stride;
    if (n_batch <= 256 * kFillTrips) {
      if (n_batch) {
        int total;
        const int p0 = warp_excl_scan(cg[0], lane, total);
        stage_group(0, mk[0], p0);
        if (n1) {
          const int p1 = n0 + warp_excl_scan(cg[1], lane, total);
          stage_group(1, mk[1], p1);
        }
      }
      if (next < n_batches) load_batch(next);          // in flight while the atomic answers and the span is written
      if (n_batch) {
        __syncwarp();
        const uint32_t run = __shfl_sync(0xffffffffu, span.x, 0), fit = __shfl_sync(0xffffffffu, span.y, 0);
        for (unsigned i = lane; i < fit; i += 32) words[run + i] = stage[i];
        __syncwarp();
      }
    } else {
      uint32_t run = __shfl_sync(0xffffffffu, span.x, 0), fit = __shfl_sync(0xffffffffu, span.y, 0);
#pragma unroll
      for (int g = 0; g < kBatch / kFillTrips; ++g) {
        const int n_staged = g == 0 ? n0 : n1;
        if (n_staged == 0) continue;
        int total;
        stage_group(g, mk[g], warp_excl_scan(cg[g], lane, total));
        __syncwarp();
        const uint32_t n_out = (uint32_t)n_staged < fit ? (uint32_t)n_staged : fit;
        for (uint32_t i = lane; i < n_out; i += 32) words[run + i] = stage[i];
        run += n_out;
        fit -= n_out;
        __syncwarp();
      }
      if (next < n_batches) load_batch(next);
    }
    batch = next;
  }
  // the block that finishes last adds the counters up (no second launch): every block takes a ticket once all its
  // atomics have returned
  __shared__ unsigned long long s_kd[4];
  __shared__ bool s_last;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned long long ticket = atomicAdd(counters + kSubLists * kCounterStride, 1ull);
    s_last = ticket == (unsigned long long)gridDim.x - 1ull;
  }
  __syncthreads();
  if (s_last) {
    __threadfence();
    tiled_finish(counters, capacity, n_sub, nnz_out, s_kd);
  }
}

// Restore of the tiled form in one pass: a warp builds a batch's 4 KB of the dense map in shared memory (zeros, then
// the batch's entries from its span) and writes it with 16-byte stores.  One directory read and one dependent
// round of list reads per batch; every output byte is written exactly once.
__global__ void __launch_bounds__(kTileThreads, 4)
prune_tiled_restore_kernel(const uint32_t* __restrict__ words, uint32_t capacity, const uint2* __restrict__ dir,
                           __nv_bfloat16* __restrict__ out, int64_t numel, int64_t n_batches) {
  __shared__ __align__(16) uint16_t s_tile[kWarpsPerBlock][kBatchElems];
  const int lane = threadIdx.x & 31;
  uint16_t* tile = s_tile[threadIdx.x >> 5];
  uint4* tile4 = reinterpret_cast<uint4*>(tile);
  const int64_t warp0 = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  const int64_t stride = (int64_t)gridDim.x * kWarpsPerBlock;
  uint2 d = warp0 < n_batches ? __ldg(dir + warp0) : make_uint2(0u, 0u);
  for (int64_t batch = warp0; batch < n_batches; batch += stride) {
    const uint2 cur = d;
    if (batch + stride < n_batches) d = __ldg(dir + batch + stride);     // the next batch's slot, one round ahead
    // entries first (the loads are in flight while the tile is cleared)
    uint32_t n = cur.y;
    if (cur.x >= capacity) n = 0u;
    else if (n > capacity - cur.x) n = capacity - cur.x;
    constexpr int PRE = 4;
    uint32_t w[PRE];
#pragma unroll
    for (int i = 0; i < PRE; ++i) {
      const uint32_t j = lane + 32u * i;
      w[i] = j < n ? __ldg(words + cur.x + j) : 0xffffffffu;
    }
#pragma unroll
    for (int c = 0; c < kBatchElems / (8 * 32); ++c) tile4[c * 32 + lane] = make_uint4(0u, 0u, 0u, 0u);
    __syncwarp();
#pragma unroll
    for (int i = 0; i < PRE; ++i) {
      const uint32_t j = lane + 32u * i;
      if (j < n) tile[(w[i] >> 16) & (kBatchElems - 1)] = (uint16_t)(w[i] & 0xffffu);
    }
    for (uint32_t j = lane + 32u * PRE; j < n; j += 32u) {
      const uint32_t wv = __ldg(words + cur.x + j);
      tile[(wv >> 16) & (kBatchElems - 1)] = (uint16_t)(wv & 0xffffu);
    }
    __syncwarp();
    const int64_t e0 = batch * kBatchElems;
#pragma unroll
    for (int c = 0; c < kBatchElems / (8 * 32); ++c) {
      const int64_t e = e0 + 8 * (c * 32 + lane);
      if (e + 8 <= numel) {
        st_stream_v4(out + e, tile4[c * 32 + lane]);
      } else {
        for (int t = 0; t < 8 && e + t < numel; ++t) out[e + t] = __ushort_as_bfloat16(tile[8 * (c * 32 + lane) + t]);
      }
    }
    __syncwarp();
  }
}

static inline int64_t n_tiles_of(int64_t numel) { return (numel + kTileElems - 1) / kTileElems; }
// one warp per tile, eight tiles per block; very large maps wrap around a grid of 32 blocks per SM
static inline int tile_grid(int64_t n_tiles) {
  int64_t g = (n_tiles + kWarpsPerBlock - 1) / kWarpsPerBlock;
  if (g > (int64_t)num_sms() * 32) g = (int64_t)num_sms() * 32;
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

// thr is the bf16-rounded threshold; a negative one (or NaN) takes the kernels that also test for zero
static inline void launch_count(const __nv_bfloat16* a, int64_t numel, float thr, int64_t nt, int64_t* ws, cudaStream_t st) {
  if (thr >= 0.f) prune_count_kernel<false><<<tile_grid(nt), kTileThreads, 0, st>>>(a, numel, thr, nt, ws);
  else prune_count_kernel<true><<<tile_grid(nt), kTileThreads, 0, st>>>(a, numel, thr, nt, ws);
}
static inline void launch_fill(const __nv_bfloat16* a, int64_t numel, float thr, int64_t nt, const int64_t* ws,
                               int64_t* idx_out, __nv_bfloat16* val_out, int64_t capacity, cudaStream_t st) {
  if (thr >= 0.f) prune_fill_kernel<false><<<tile_grid(nt), kTileThreads, 0, st>>>(a, numel, thr, nt, ws, idx_out, val_out, capacity);
  else prune_fill_kernel<true><<<tile_grid(nt), kTileThreads, 0, st>>>(a, numel, thr, nt, ws, idx_out, val_out, capacity);
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
  launch_count((const __nv_bfloat16*)a, numel, thr_bf16(threshold), nt, (int64_t*)workspace, st);
  HYC_CHECK_LAUNCH();
  prune_scan_kernel<<<1, 1024, 0, st>>>((int64_t*)workspace, nt, nullptr);
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
  launch_fill((const __nv_bfloat16*)a, numel, thr_bf16(threshold), nt, (const int64_t*)workspace, idx_out,
              (__nv_bfloat16*)val_out, capacity, (cudaStream_t)stream);
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
    if (g > (int64_t)num_sms() * 16) g = (int64_t)num_sms() * 16;
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
    if (g > (int64_t)num_sms() * 16) g = (int64_t)num_sms() * 16;
    prune_scatter_counted_kernel<<<(int)g, 256, 0, st>>>(idx, (const __nv_bfloat16*)val, nnz_dev, capacity,
                                                         (__nv_bfloat16*)a_out, numel);
    HYC_CHECK_LAUNCH();
  }
  return HYC_OK;
}

extern "C" HYC_API size_t hyc_softmax_prune_tiled_directory_bytes(int64_t numel) {
  if (numel < 0) return 0;
  // directory, the sub-lists' counters, and one more slot: the ticket of the blocks that have finished
  return (size_t)tiled_dir_entries(numel) * sizeof(uint2) + (size_t)(kSubLists + 1) * kCounterStride * sizeof(unsigned long long);
}

extern "C" HYC_API int hyc_softmax_prune_tiled(const void* a, int64_t numel, float threshold,
                                               uint32_t* words_out, int64_t capacity, void* directory_out,
                                               int64_t* nnz_out, void* stream) {
  if (!a || !nnz_out || !directory_out) return HYC_ERR_NULL;
  if (capacity > 0 && !words_out) return HYC_ERR_NULL;
  if (numel <= 0 || capacity < 0 || capacity > 0xffffffffll) return HYC_ERR_SHAPE;
  if (!aligned(a, 16) || !aligned(nnz_out, 8) || !aligned(directory_out, 128) || !aligned(words_out, 4)) return HYC_ERR_ALIGN;
  cudaStream_t st = (cudaStream_t)stream;
  unsigned long long* counters = reinterpret_cast<unsigned long long*>(reinterpret_cast<uint2*>(directory_out) + tiled_dir_entries(numel));
  if (cudaMemsetAsync(counters, 0, (size_t)(kSubLists + 1) * kCounterStride * sizeof(unsigned long long), st) != cudaSuccess) {
    hyc_set_last_cuda_error((int)cudaGetLastError());
    return HYC_ERR_LAUNCH;
  }
  const int64_t nt = n_tiles_of(numel);
  const float thr = thr_bf16(threshold);
  // four resident blocks of eight warps per multiprocessor, a warp per batch; larger maps wrap around
  const int64_t nbt = (numel + kBatchElems - 1) / kBatchElems;
  int64_t g = (nbt + kWarpsPerBlock - 1) / kWarpsPerBlock;
  if (g > (int64_t)num_sms() * 4) g = (int64_t)num_sms() * 4;
  if (thr >= 0.f)
    prune_tiled_kernel<false><<<(int)g, kTileThreads, 0, st>>>((const __nv_bfloat16*)a, numel, thr, nt, words_out, (uint32_t)capacity,
                                                            (uint2*)directory_out, counters, nnz_out);
  else
    prune_tiled_kernel<true><<<(int)g, kTileThreads, 0, st>>>((const __nv_bfloat16*)a, numel, thr, nt, words_out, (uint32_t)capacity,
                                                           (uint2*)directory_out, counters, nnz_out);
  HYC_CHECK_LAUNCH();
  return HYC_OK;
}

extern "C" HYC_API int hyc_softmax_prune_tiled_restore(const uint32_t* words, int64_t capacity, const void* directory,
                                                       void* a_out, int64_t numel, void* stream) {
  if (!a_out || !directory || (capacity > 0 && !words)) return HYC_ERR_NULL;
  if (numel <= 0 || capacity < 0 || capacity > 0xffffffffll) return HYC_ERR_SHAPE;
  if (!aligned(a_out, 16) || !aligned(directory, 128)) return HYC_ERR_ALIGN;
  const int64_t nb = (numel + kBatchElems - 1) / kBatchElems;
  int64_t g = (nb + kWarpsPerBlock - 1) / kWarpsPerBlock;
  if (g > (int64_t)num_sms() * 4) g = (int64_t)num_sms() * 4;
  prune_tiled_restore_kernel<<<(int)g, kTileThreads, 0, (cudaStream_t)stream>>>(words, (uint32_t)capacity, (const uint2*)directory,
                                                                             (__nv_bfloat16*)a_out, numel, nb);
  HYC_CHECK_LAUNCH();
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
  // one slot per device, filled on that device's first call.  Written without a lock: the documented use is one
  // host thread per GPU, and two threads racing on a slot would store the same address.
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
  // the built-in scratch is the CURRENT device's copy: a map that lives on another GPU is refused before any launch
  {
    cudaPointerAttributes pa;
    int cur = -1;
    if (cudaPointerGetAttributes(&pa, a) == cudaSuccess && pa.type == cudaMemoryTypeDevice &&
        cudaGetDevice(&cur) == cudaSuccess && pa.device != cur)
      return HYC_ERR_UNSUPPORTED;
    (void)cudaGetLastError();      // an unregistered (host test) pointer leaves an error state behind: clear it
  }
  int err = 0;
  int64_t* ws = static_offsets_for_current_device(&err);
  if (!ws) { hyc_set_last_cuda_error(err); return HYC_ERR_LAUNCH; }
  cudaStream_t st = (cudaStream_t)stream;
  const float thr = thr_bf16(threshold);
  launch_count((const __nv_bfloat16*)a, numel, thr, nt, ws, st);
  HYC_CHECK_LAUNCH();
  prune_scan_kernel<<<1, 1024, 0, st>>>(ws, nt, nnz_out);
  HYC_CHECK_LAUNCH();
  if (capacity > 0) {
    launch_fill((const __nv_bfloat16*)a, numel, thr, nt, ws, idx_out, (__nv_bfloat16*)val_out, capacity, st);
    HYC_CHECK_LAUNCH();
  }
  return HYC_OK;
}

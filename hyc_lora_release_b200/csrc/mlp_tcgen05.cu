// tcgen05 / TMEM GEMMs of the LoRA MLP with the activation-compression work in the epilogue.
//
// One persistent kernel, three epilogues:
//   STORE    : D = A * B (+ rank-16 LoRA terms, + residual), bf16 out.  Down projection, grad_x.
//   GATEUP   : [gate_main | up_main] tile = x * [Wg ; Wu]^T, then per element: quantize-and-pack
//              both main branches, add the LoRA terms, SiLU, Hadamard product (forward).
//   GRADDOWN : grad_down tile = g * Wd (+ LoRA), then per element: unpack-dequantize the saved
//              gate/up codes, recompute the forward, emit hadamard, grad_gate, grad_up (backward).
//
// Two CTAs on neighbouring SMs (a cluster of 2) work on one 256 x 256 tile with the pair form of the MMA
// (cta_group::2): CTA r of the pair holds rows 128 r .. 128 r + 127 of the A tile and columns 128 r .. of the
// B tile in its shared memory, the tensor core of each SM reads both halves of B, and each CTA's tensor memory
// receives its own 128 rows of the result.  Per 64-wide k-block an SM therefore pulls 32 KB from L2 instead of
// the 48 KB a 128 x 256 tile of its own would need: the L2-to-SM feed is what bounds the main loop.
//
// Structure of a CTA (320 threads, one CTA per SM, pair tiles dealt round-robin over the pairs):
//   warp 0      : TMA producer (both CTAs): its 128x64 A block and its 128x64 B block per stage (128-byte
//                 swizzle), 6 stages of 32 KB.  The loads of both CTAs complete on the LEADER's (CTA 0 of the
//                 pair) "full" barrier; each CTA waits on its own "empty" barrier.
//   warp 1      : allocates all 512 TMEM columns (two 128x256 fp32 accumulators per CTA; both CTAs take part);
//                 in the leader one lane issues tcgen05.mma.cta_group::2 (M256 N256 K16, bf16 -> fp32) and
//                 commits to the "empty" / "accumulator full" barriers of BOTH CTAs (tcgen05.commit with a CTA
//                 mask; the loads themselves are plain, no multicast).
//   warps 2..9  : epilogue (both CTAs).  Warp w reads TMEM lanes 32*(w%4).. (tcgen05.ld 32x32b.x32) for half
//                 of the tile's columns, so the epilogue of tile i overlaps the MMAs of tile i+1; when a warp
//                 is done with an accumulator it arrives on the leader's "accumulator empty" barrier.
// The B operand is either K-major ([N,K] row-major, the forward weights) or MN-major ([K,N]
// row-major: the same weights read for the backward products, no transposed copy).
// Every wait is bounded: when a limit is hit the kernel records a code in *status and drains; both CTAs of a
// pair then still meet at the cluster barrier before the tensor memory is released.
// The same kernel also exists without the pairing (template argument PAIR = false: a 128 x 256 tile per CTA,
// 4 stages of 48 KB, cta_group::1 everywhere, no cluster); the grad_down product uses that form (see UsePair).
#include "hyc_common.cuh"
#include <cuda.h>

#ifdef HYC_TC_PROF
#define TC_STAMP(role, it, j) do { if (p.prof != nullptr && blockIdx.x < 2 && (it) < 16) p.prof[blockIdx.x * 384 + ((role) * 16 + (it)) * 8 + (j)] = clock64(); } while (0)
static long long* g_tc_prof = nullptr;
extern "C" __attribute__((visibility("default"))) void hyc_tc_debug_profile(void* buf) { g_tc_prof = (long long*)buf; }
#else
#define TC_STAMP(role, it, j) do { } while (0)
#endif

namespace hyc {
namespace tc {

constexpr int BM = 128, BN = 256, BK = 64;       // per CTA: 128 rows x 256 columns of accumulator
constexpr int STAGE_A_BYTES = BM * BK * 2;
// PAIR: two CTAs share a 256 x 256 tile, each loads 128 columns of the B block (6 stages of 32 KB);
// otherwise a CTA has a 128 x 256 tile of its own and loads the whole B block (4 stages of 48 KB)
template <bool PAIR> struct Geo {
  static constexpr int TILE_M = PAIR ? 2 * BM : BM;
  static constexpr int B_COLS = PAIR ? BN / 2 : BN;
  static constexpr int STAGE_B_BYTES = B_COLS * BK * 2;
  static constexpr int STAGE_BYTES = STAGE_A_BYTES + STAGE_B_BYTES;
  static constexpr int STAGES = PAIR ? 6 : 4;
};
constexpr int MAX_STAGES = 6;
constexpr int PIPE_BYTES = 6 * (STAGE_A_BYTES + (BN / 2) * BK * 2);
static_assert(PIPE_BYTES == Geo<true>::STAGES * Geo<true>::STAGE_BYTES && PIPE_BYTES == Geo<false>::STAGES * Geo<false>::STAGE_BYTES,
              "both forms use the same amount of shared memory");
constexpr int EPI_WARPS = 8;
constexpr int THREADS = 64 + 32 * EPI_WARPS;
constexpr int TMEM_COLS = 512;
// epilogue scratch: 32 KB of tiles followed by BN floats of per-column constants.
//   STORE    two fp32 LoRA-B tiles [BN][16], then BN quantizer constants
//   GATEUP   two fp32 LoRA-B tiles [BN/2][16], then (inside the 32 KB) two float vectors of BN/2 constants
//   GRADDOWN per epilogue warp two [32 rows][32 columns] bf16 tiles (LoRA terms in, results out), then two bf16
//            scale vectors of BN
constexpr int EPI_SMEM_BYTES = 2 * BN * 16 * 4 + BN * 4;
constexpr int SMEM_BYTES = 1024 + PIPE_BYTES + EPI_SMEM_BYTES + 256;
constexpr uint32_t SPIN_LIMIT = 1u << 22;

enum { EPI_STORE = 0, EPI_GATEUP = 1, EPI_GRADDOWN = 2 };
enum { ST_OK = 0, ST_TIMEOUT_PRODUCER = 1, ST_TIMEOUT_MMA = 2, ST_TIMEOUT_EPILOGUE = 3 };

struct LoraTerm {
  const __nv_bfloat16* xa;    // [M, 16] row-major, or null
  const __nv_bfloat16* bt;    // element (col, r) at bt[col * ld_col + r * ld_r]
  int64_t ld_col, ld_r;
};

struct Params {
  int M, N, K1, K2, K3;       // K2, K3 > 0: further (A, B) pairs accumulated into the same tile
  int epi, q_bit;
  LoraTerm l0, l1, l2;        // STORE: l0/l1 added; GATEUP: l0 gate, l1 up; GRADDOWN: l0 grad LoRA, l1 gate, l2 up
  const __nv_bfloat16* residual;   // STORE, [M, N] or null
  __nv_bfloat16* out0;        // STORE: D ; GATEUP: o ; GRADDOWN: o (hadamard)
  __nv_bfloat16* out1;        // GRADDOWN: grad_gate
  __nv_bfloat16* out2;        // GRADDOWN: grad_up
  __nv_bfloat16* dbg1;        // GATEUP: optional bf16 copy of gate_main
  __nv_bfloat16* dbg2;        // GATEUP: optional bf16 copy of up_main
  uint8_t* q1;                // GATEUP: out ; GRADDOWN: in
  uint8_t* q2;
  const __nv_bfloat16* s1;    // per-channel scales [N]
  const __nv_bfloat16* s2;
  const __nv_bfloat16* lpre1; // GRADDOWN: optional precomputed LoRA terms bf16(xa1 B1^T), bf16(xa2 B2^T), [M, ld_pre]
  const __nv_bfloat16* lpre2;
  int64_t ld_pre;
  int* status;
#ifdef HYC_TC_PROF
  long long* prof;            // debug builds only: clock64 stamps of CTA 0, [role][tile][8]
#endif
};

// ------------------------------------------------------------------ PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
// bounded wait; false = gave up (either the limit was hit here or another role raised abort)
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  for (uint32_t i = 0; i < SPIN_LIMIT; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 63u) == 63u && *abort_flag) return false;
  }
  return false;
}
// a tile into this CTA's shared memory; the bytes are counted on the barrier at shared::cluster address `bar`,
// which in the pair form may belong to the other CTA of the pair (that is what .cta_group::2 permits)
template <bool PAIR>
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1) {
  if (PAIR)
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1) : "memory");
  else
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of the same variable in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(const void* p, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_u32(p)), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// arrives on the barrier once the MMAs issued so far are done; pair form: on the barrier at this offset in BOTH CTAs
template <bool PAIR>
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  if (PAIR)
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(smem_u32(bar)), "h"((uint16_t)3) : "memory");
  else
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
template <bool PAIR>
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  if (PAIR)
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
  else
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
        "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
        "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr) : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// shared-memory matrix descriptor, 128-byte swizzle, descriptor version 1
__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3ffffu) >> 4);
  d |= (uint64_t)(lbo_bytes >> 4) << 16;
  d |= (uint64_t)(sbo_bytes >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

__device__ __forceinline__ void epi_bar_sync() { asm volatile("bar.sync 1, %0;" ::"n"(32 * EPI_WARPS) : "memory"); }

// round to bf16 and back: the value goes into the high half of the packed conversion, where its
// bits already are the float
__device__ __forceinline__ float bfr(float v) { return __uint_as_float(pack_bf16x2_rn(0.f, v) & 0xffff0000u); }

// ---- packed bf16x2 arithmetic.  The reference's element-wise chain works on bf16 tensors (every
// operation rounds to bf16).  For bf16 operands a packed add/sub/mul is the same thing: the fp32 product of
// two bf16 values is exact and the fp32 sum is exact unless the operands are more than 16 binades apart (then
// both forms return the larger one), so one rounding to bf16 is all that ever happens.  Two columns per
// instruction, no conversion instruction: those are the scarce resource of an epilogue that has only two
// warps per scheduler.
typedef __nv_bfloat162 bf2;
__device__ __forceinline__ bf2 as_bf2(uint32_t v) { return *reinterpret_cast<bf2*>(&v); }
__device__ __forceinline__ uint32_t as_u32(bf2 v) { return *reinterpret_cast<uint32_t*>(&v); }
// (the _rn forms: a multiply followed by an add must NOT be contracted into one fused operation, the
// reference rounds after each)
__device__ __forceinline__ uint32_t add2(uint32_t a, uint32_t b) { return as_u32(__hadd2_rn(as_bf2(a), as_bf2(b))); }
__device__ __forceinline__ uint32_t sub2(uint32_t a, uint32_t b) { return as_u32(__hsub2_rn(as_bf2(a), as_bf2(b))); }
__device__ __forceinline__ uint32_t mul2(uint32_t a, uint32_t b) { return as_u32(__hmul2_rn(as_bf2(a), as_bf2(b))); }
constexpr uint32_t kOne2 = 0x3f803f80u;   // (1.0, 1.0)
// bf16(sigmoid(y)) of both halves; the sigmoid itself is fp32 as in the reference kernels
__device__ __forceinline__ uint32_t sigmoid2(uint32_t y) {
  const float a = bf16lo_to_f32(y), b = bf16hi_to_f32(y);
  return pack_bf16x2_rn(__fdividef(1.f, 1.f + __expf(-a)), __fdividef(1.f, 1.f + __expf(-b)));
}
// dot with an fp32 LoRA-B row in shared memory: eight packed two-wide fp32 FMAs (even and odd ranks accumulate
// side by side, one add joins them) on four 128-bit broadcast loads
__device__ __forceinline__ uint64_t pair_f32(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ float lora_dot_f32(const float (&xa)[16], const float* __restrict__ brow) {
  uint64_t acc = 0ull;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float4 b = *reinterpret_cast<const float4*>(brow + 4 * j);
    asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(acc) : "l"(pair_f32(xa[4 * j], xa[4 * j + 1])), "l"(pair_f32(b.x, b.y)));
    asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(acc) : "l"(pair_f32(xa[4 * j + 2], xa[4 * j + 3])), "l"(pair_f32(b.z, b.w)));
  }
  float lo, hi;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(acc));
  return lo + hi;
}

// LoRA terms of the GRADDOWN epilogue on the legacy tensor path (a rank-16 side product of a tcgen05 kernel)
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(0.f), "f"(0.f), "f"(0.f), "f"(0.f));
}

__device__ __forceinline__ void load_xa_row(const __nv_bfloat16* xa, int64_t row, bool valid, float (&out)[16]) {
  uint4 u = make_uint4(0u, 0u, 0u, 0u), v = u;
  if (valid && xa != nullptr) {
    u = *reinterpret_cast<const uint4*>(xa + row * 16);
    v = *reinterpret_cast<const uint4*>(xa + row * 16 + 8);
  }
  const uint32_t w[8] = {u.x, u.y, u.z, u.w, v.x, v.y, v.z, v.w};
#pragma unroll
  for (int j = 0; j < 8; ++j) { out[2 * j] = bf16lo_to_f32(w[j]); out[2 * j + 1] = bf16hi_to_f32(w[j]); }
}

// cooperative staging of a LoRA-B tile as fp32 rows (ncols x 16 floats)
__device__ __forceinline__ void stage_lora_tile_f32(const LoraTerm& t, int n0, int ncols, float* dst, int et) {
  if (t.bt == nullptr) return;
  if (t.ld_r == 1 && t.ld_col == 16 && (reinterpret_cast<uintptr_t>(t.bt) & 15) == 0) {
    // [columns, 16] row-major (the layout of a lora_B weight): 128-bit loads, eight values each
    const uint4* src = reinterpret_cast<const uint4*>(t.bt + (int64_t)n0 * 16);
    for (int i = et; i < ncols * 2; i += 32 * EPI_WARPS) {
      const uint4 v = src[i];
      float4 a, b;
      a.x = bf16lo_to_f32(v.x); a.y = bf16hi_to_f32(v.x); a.z = bf16lo_to_f32(v.y); a.w = bf16hi_to_f32(v.y);
      b.x = bf16lo_to_f32(v.z); b.y = bf16hi_to_f32(v.z); b.z = bf16lo_to_f32(v.w); b.w = bf16hi_to_f32(v.w);
      reinterpret_cast<float4*>(dst)[2 * i] = a;
      reinterpret_cast<float4*>(dst)[2 * i + 1] = b;
    }
    return;
  }
  for (int i = et; i < ncols * 16; i += 32 * EPI_WARPS) {
    const int c = i >> 4, r = i & 15;
    dst[i] = __bfloat162float(t.bt[(int64_t)(n0 + c) * t.ld_col + (int64_t)r * t.ld_r]);
  }
}
// The reference byte layout of a 32-column block: byte j carries, at bit QBIT*i, the code of
// column j + i*SLAB (SLAB = 32/EPP columns, EPP = 8/QBIT).  A block is SLAB bytes = NW words.
template <int QBIT> struct BlockGeo {
  static constexpr int EPP = 8 / QBIT, SLAB = 32 / EPP, NW = SLAB / 4;
  static constexpr uint32_t CM = (1u << QBIT) - 1u;
};

template <int QBIT>
__device__ __forceinline__ void put_code(uint32_t (&words)[BlockGeo<QBIT>::NW], int c, uint32_t code) {
  using G = BlockGeo<QBIT>;
  const int j = c % G::SLAB, i = c / G::SLAB;
  words[j >> 2] |= code << (8 * (j & 3) + QBIT * i);
}
template <int QBIT>
__device__ __forceinline__ uint32_t get_code(const uint32_t (&words)[BlockGeo<QBIT>::NW], int c) {
  using G = BlockGeo<QBIT>;
  const int j = c % G::SLAB, i = c / G::SLAB;
  return (words[j >> 2] >> (8 * (j & 3) + QBIT * i)) & G::CM;
}
template <int QBIT>
__device__ __forceinline__ void store_block_words(uint8_t* dst, const uint32_t (&w)[BlockGeo<QBIT>::NW]) {
  if constexpr (QBIT == 8) {
    *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
    *reinterpret_cast<uint4*>(dst + 16) = make_uint4(w[4], w[5], w[6], w[7]);
  } else if constexpr (QBIT == 4) {
    *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
  } else {
    *reinterpret_cast<uint2*>(dst) = make_uint2(w[0], w[1]);
  }
}
template <int QBIT>
__device__ __forceinline__ void load_block_words(const uint8_t* src, bool valid, uint32_t (&w)[BlockGeo<QBIT>::NW]) {
#pragma unroll
  for (int i = 0; i < BlockGeo<QBIT>::NW; ++i) w[i] = 0u;
  if (!valid) return;
  if constexpr (QBIT == 8) {
    const uint4 a = *reinterpret_cast<const uint4*>(src), b = *reinterpret_cast<const uint4*>(src + 16);
    w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w; w[4] = b.x; w[5] = b.y; w[6] = b.z; w[7] = b.w;
  } else if constexpr (QBIT == 4) {
    const uint4 a = *reinterpret_cast<const uint4*>(src);
    w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w;
  } else {
    const uint2 a = *reinterpret_cast<const uint2*>(src);
    w[0] = a.x; w[1] = a.y;
  }
}

// ------------------------------------------------------------------ epilogues (one 32-column chunk per call)
// cb = column offset of the chunk inside the tile, ncol0 = first output column of the tile.  The thread owns
// one row; columns are handled two at a time as packed bf16 pairs.
__device__ __forceinline__ void store4_pairs(__nv_bfloat16* dst, const uint32_t (&v)[4]) {
  *reinterpret_cast<uint4*>(dst) = make_uint4(v[0], v[1], v[2], v[3]);
}

template <int QBIT>
__device__ __forceinline__ void epi_gateup_block(const Params& p, int64_t row, bool valid, int ncol0, int cb,
                                                 const uint32_t (&g)[32], const uint32_t (&u)[32],
                                                 const float (&xa1)[16], const float (&xa2)[16],
                                                 const float* sB1, const float* sB2, const float* sR1, const float* sR2) {
  using G = BlockGeo<QBIT>;
  const int64_t n = (int64_t)ncol0 + cb;
  uint32_t w1[G::NW], w2[G::NW];
#pragma unroll
  for (int i = 0; i < G::NW; ++i) { w1[i] = 0u; w2[i] = 0u; }
#pragma unroll
  for (int c8 = 0; c8 < 4; ++c8) {
    uint32_t o[4];
#pragma unroll
    for (int e2 = 0; e2 < 4; ++e2) {
      const int c = 8 * c8 + 2 * e2, tc = cb + c;
      // the frozen-weight products are bf16 tensors in the reference before anything else touches them
      const uint32_t x1 = pack_bf16x2_rn(__uint_as_float(g[c]), __uint_as_float(g[c + 1]));
      const uint32_t x2 = pack_bf16x2_rn(__uint_as_float(u[c]), __uint_as_float(u[c + 1]));
      put_code<QBIT>(w1, c, fastq_code_bits<QBIT>(bf16lo_to_f32(x1), sR1[tc]) & G::CM);
      put_code<QBIT>(w1, c + 1, fastq_code_bits<QBIT>(bf16hi_to_f32(x1), sR1[tc + 1]) & G::CM);
      put_code<QBIT>(w2, c, fastq_code_bits<QBIT>(bf16lo_to_f32(x2), sR2[tc]) & G::CM);
      put_code<QBIT>(w2, c + 1, fastq_code_bits<QBIT>(bf16hi_to_f32(x2), sR2[tc + 1]) & G::CM);
      const uint32_t l1 = pack_bf16x2_rn(lora_dot_f32(xa1, sB1 + tc * 16), lora_dot_f32(xa1, sB1 + (tc + 1) * 16));
      const uint32_t l2 = pack_bf16x2_rn(lora_dot_f32(xa2, sB2 + tc * 16), lora_dot_f32(xa2, sB2 + (tc + 1) * 16));
      const uint32_t y1 = add2(x1, l1);
      const uint32_t y1s = mul2(y1, sigmoid2(y1));
      o[e2] = mul2(y1s, add2(x2, l2));
    }
    if (valid) store4_pairs(p.out0 + row * p.N + n + 8 * c8, o);
  }
  if (valid) {
    store_block_words<QBIT>(p.q1 + (row * p.N + n) * QBIT / 8, w1);
    store_block_words<QBIT>(p.q2 + (row * p.N + n) * QBIT / 8, w2);
    if (p.dbg1 != nullptr) {
#pragma unroll
      for (int c8 = 0; c8 < 4; ++c8) {
        uint32_t a[4], b[4];
#pragma unroll
        for (int e2 = 0; e2 < 4; ++e2) {
          a[e2] = pack_bf16x2_rn(__uint_as_float(g[8 * c8 + 2 * e2]), __uint_as_float(g[8 * c8 + 2 * e2 + 1]));
          b[e2] = pack_bf16x2_rn(__uint_as_float(u[8 * c8 + 2 * e2]), __uint_as_float(u[8 * c8 + 2 * e2 + 1]));
        }
        store4_pairs(p.dbg1 + row * p.N + n + 8 * c8, a);
        store4_pairs(p.dbg2 + row * p.N + n + 8 * c8, b);
      }
    }
  }
}

// the saved codes of columns c, c + 1 of a 32-column block as the bf16 pair (x_hat[c], x_hat[c + 1]),
// x_hat = bf16((code - half) * scale); sc2 = the two scales as a packed pair
template <int QBIT>
__device__ __forceinline__ uint32_t dequant_pair(const uint32_t (&w)[BlockGeo<QBIT>::NW], int c, uint32_t sc2) {
  const uint32_t c0 = get_code<QBIT>(w, c), c1 = get_code<QBIT>(w, c + 1);
  if constexpr (QBIT == 8) {
    // codes reach 255: through fp32 (2^23 + code), one rounding in the packed conversion
    const float f0 = (__uint_as_float(0x4B000000u | c0) - 8388736.f) * bf16lo_to_f32(sc2);
    const float f1 = (__uint_as_float(0x4B000000u | c1) - 8388736.f) * bf16hi_to_f32(sc2);
    return pack_bf16x2_rn(f0, f1);
  } else {
    // 0x4300 | code is the bf16 128 + code; minus (128 + half) is exact, the product rounds once
    constexpr uint32_t C1 = 0x4300u | (uint32_t)(1 << (QBIT - 1));
    const uint32_t pr = 0x43004300u | c0 | (c1 << 16);
    return mul2(sub2(pr, C1 | (C1 << 16)), sc2);
  }
}

// Word index of 16-byte chunk c (eight columns) of a row in a [32 rows][32 columns] bf16 tile of one epilogue warp.
// The chunks of a row are permuted by the row number so that the three access patterns of the GRADDOWN epilogue
// are free of bank conflicts: 32-bit stores in the mma fragment layout (rows g, g + 8 / word t of chunk nt), 128-bit
// accesses of a lane to its own row, and 128-bit reads of eight rows x four chunks for the coalesced flush.
__device__ __forceinline__ int gd_chunk(int row, int c) { return row * 16 + ((c ^ ((row >> 1) & 3)) << 2); }

// rows [8k, 8k + 8) of the warp's tile leave as 64 contiguous bytes per row (four lanes per row)
__device__ __forceinline__ void gd_flush(const uint32_t* R, __nv_bfloat16* out, int64_t row0, int64_t M, int64_t ldo,
                                         int64_t n, int lane) {
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int r = 8 * k + (lane >> 2), c = lane & 3;
    const uint4 v = *reinterpret_cast<const uint4*>(R + gd_chunk(r, c));
    if (row0 + r < M) *reinterpret_cast<uint4*>(out + (row0 + r) * ldo + n + 8 * c) = v;
  }
}

// What a GRADDOWN block reads from global memory, fetched one block ahead: the packed codes of the lane's row and
// the LoRA-B fragments (mma B operands) of the block's 32 columns for both branches.
template <int QBIT>
struct GdInputs {
  uint32_t w1[BlockGeo<QBIT>::NW], w2[BlockGeo<QBIT>::NW];
  uint32_t bf[16];      // [nt][b1a, b1b, b2a, b2b]
};
template <int QBIT>
__device__ __forceinline__ void gd_fetch(const Params& p, int64_t row0, int lane, int64_t n, GdInputs<QBIT>& in) {
  const int64_t row = row0 + lane;
  const bool valid = row < p.M;
  const int g = lane >> 2, t = lane & 3;
  load_block_words<QBIT>(p.q1 + (row * p.N + n) * QBIT / 8, valid, in.w1);
  load_block_words<QBIT>(p.q2 + (row * p.N + n) * QBIT / 8, valid, in.w2);
  if (p.lpre1 != nullptr) return;      // kernel-uniform: the LoRA terms come from a launch that prepared them
  const bool fast = p.l1.ld_r == 1 && p.l2.ld_r == 1 && ((p.l1.ld_col | p.l2.ld_col) & 1) == 0;
#pragma unroll
  for (int nt = 0; nt < 4; ++nt) {
    const int64_t nn = n + 8 * nt + g;
    const __nv_bfloat16* b1p = p.l1.bt + nn * p.l1.ld_col;
    const __nv_bfloat16* b2p = p.l2.bt + nn * p.l2.ld_col;
    if (fast) {
      in.bf[4 * nt] = *reinterpret_cast<const uint32_t*>(b1p + 2 * t);
      in.bf[4 * nt + 1] = *reinterpret_cast<const uint32_t*>(b1p + 2 * t + 8);
      in.bf[4 * nt + 2] = *reinterpret_cast<const uint32_t*>(b2p + 2 * t);
      in.bf[4 * nt + 3] = *reinterpret_cast<const uint32_t*>(b2p + 2 * t + 8);
    } else {
      auto two = [](const __nv_bfloat16* q, int64_t r, int64_t ld) {
        return (uint32_t)__bfloat16_as_ushort(q[r * ld]) | ((uint32_t)__bfloat16_as_ushort(q[(r + 1) * ld]) << 16);
      };
      in.bf[4 * nt] = two(b1p, 2 * t, p.l1.ld_r); in.bf[4 * nt + 1] = two(b1p, 2 * t + 8, p.l1.ld_r);
      in.bf[4 * nt + 2] = two(b2p, 2 * t, p.l2.ld_r); in.bf[4 * nt + 3] = two(b2p, 2 * t + 8, p.l2.ld_r);
    }
  }
}

// One block of 32 rows x 32 columns of the GRADDOWN epilogue, a whole warp at a time (lane = row for the
// accumulator and the element-wise chain).  The LoRA terms of the two branches are rank-16 products on the legacy
// tensor path: fragments -> bf16 pairs -> the warp's two shared-memory tiles, from which every lane reads its own
// row.  The same tiles then collect the results so that they leave as coalesced 64-byte row segments: a lane
// storing 16 bytes of its own row would make every store instruction touch 32 lines, which throttled the
// load/store unit and slowed the TMA loads of the main loop.
template <int QBIT>
__device__ __forceinline__ void epi_graddown_block(const Params& p, int64_t row0, int lane, int ncol0, int cb,
                                                   const uint32_t (&acc)[32], const GdInputs<QBIT>& in,
                                                   const uint32_t (&fa1)[2][4], const uint32_t (&fa2)[2][4],
                                                   uint32_t* R1, uint32_t* R2,
                                                   const uint32_t* sS1, const uint32_t* sS2) {
  const int64_t n = (int64_t)ncol0 + cb;
  const int64_t row = row0 + lane;
  const bool valid = row < p.M;
  const int g = lane >> 2, t = lane & 3;
  const bool pre = p.lpre1 != nullptr;      // kernel-uniform
  if (!pre) {
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
      for (int mt = 0; mt < 2; ++mt) {
        float c1[4], c2[4];
        mma_bf16_16816(c1, fa1[mt], in.bf[4 * nt], in.bf[4 * nt + 1]);
        mma_bf16_16816(c2, fa2[mt], in.bf[4 * nt + 2], in.bf[4 * nt + 3]);
        // fragment: (row 16 mt + g, columns 8 nt + 2t, +1) and (row 16 mt + g + 8, same columns)
        R1[gd_chunk(16 * mt + g, nt) + t] = pack_bf16x2_rn(c1[0], c1[1]);
        R1[gd_chunk(16 * mt + g + 8, nt) + t] = pack_bf16x2_rn(c1[2], c1[3]);
        R2[gd_chunk(16 * mt + g, nt) + t] = pack_bf16x2_rn(c2[0], c2[1]);
        R2[gd_chunk(16 * mt + g + 8, nt) + t] = pack_bf16x2_rn(c2[2], c2[3]);
      }
    }
    __syncwarp();
  }
  uint32_t gu_all[16];
#pragma unroll
  for (int c8 = 0; c8 < 4; ++c8) {
    uint32_t o[4], gg[4];
    // the LoRA terms of the lane's row: from the warp's tiles, or from a launch that prepared them
    uint4 pl1, pl2;
    if (pre) {
      pl1 = make_uint4(0u, 0u, 0u, 0u); pl2 = pl1;
      if (valid) {
        pl1 = *reinterpret_cast<const uint4*>(p.lpre1 + row * p.ld_pre + n + 8 * c8);
        pl2 = *reinterpret_cast<const uint4*>(p.lpre2 + row * p.ld_pre + n + 8 * c8);
      }
    } else {
      pl1 = *reinterpret_cast<const uint4*>(R1 + gd_chunk(lane, c8));
      pl2 = *reinterpret_cast<const uint4*>(R2 + gd_chunk(lane, c8));
    }
    const uint32_t pw1[4] = {pl1.x, pl1.y, pl1.z, pl1.w}, pw2[4] = {pl2.x, pl2.y, pl2.z, pl2.w};
#pragma unroll
    for (int e2 = 0; e2 < 4; ++e2) {
      const int c = 8 * c8 + 2 * e2, tc = cb + c;
      // the LoRA part of grad_down arrived as an extra K block
      const uint32_t gd = pack_bf16x2_rn(__uint_as_float(acc[c]), __uint_as_float(acc[c + 1]));
      const uint32_t x1 = dequant_pair<QBIT>(in.w1, c, sS1[tc >> 1]);
      const uint32_t x2 = dequant_pair<QBIT>(in.w2, c, sS2[tc >> 1]);
      const uint32_t y1 = add2(x1, pw1[e2]), sig = sigmoid2(y1), y1s = mul2(y1, sig), y2 = add2(x2, pw2[e2]);
      o[e2] = mul2(y1s, y2);
      gu_all[4 * c8 + e2] = mul2(gd, y1s);
      const uint32_t inner = add2(kOne2, mul2(y1, sub2(kOne2, sig)));
      gg[e2] = mul2(mul2(gd, y2), mul2(sig, inner));
    }
    // chunk c8 of the lane's own row is dead now: the results take its place
    *reinterpret_cast<uint4*>(R1 + gd_chunk(lane, c8)) = make_uint4(o[0], o[1], o[2], o[3]);
    *reinterpret_cast<uint4*>(R2 + gd_chunk(lane, c8)) = make_uint4(gg[0], gg[1], gg[2], gg[3]);
  }
  __syncwarp();
  gd_flush(R1, p.out0, row0, p.M, p.N, n, lane);
  gd_flush(R2, p.out1, row0, p.M, p.N, n, lane);
  __syncwarp();
#pragma unroll
  for (int c8 = 0; c8 < 4; ++c8)
    *reinterpret_cast<uint4*>(R1 + gd_chunk(lane, c8)) = make_uint4(gu_all[4 * c8], gu_all[4 * c8 + 1], gu_all[4 * c8 + 2], gu_all[4 * c8 + 3]);
  __syncwarp();
  gd_flush(R1, p.out2, row0, p.M, p.N, n, lane);
  __syncwarp();     // the tiles are rewritten by the next block
}

template <int QBIT>
__device__ __forceinline__ void epi_store_block(const Params& p, int64_t row, bool valid, int ncol0, int cb,
                                                const uint32_t (&acc)[32], const float (&xa0)[16], const float (&xa1)[16],
                                                const float* sB0, const float* sB1, const float* sR) {
  using G = BlockGeo<QBIT>;
  const int64_t n = (int64_t)ncol0 + cb;
  const bool has0 = p.l0.bt != nullptr, has1 = p.l1.bt != nullptr;
  const bool has_res = p.residual != nullptr && valid;
  const bool save = p.q1 != nullptr;
  uint32_t w1[G::NW];
#pragma unroll
  for (int i = 0; i < G::NW; ++i) w1[i] = 0u;
#pragma unroll
  for (int c8 = 0; c8 < 4; ++c8) {
    uint4 rq = make_uint4(0u, 0u, 0u, 0u);
    if (has_res) rq = *reinterpret_cast<const uint4*>(p.residual + row * p.N + n + 8 * c8);
    const uint32_t r[4] = {rq.x, rq.y, rq.z, rq.w};
    uint32_t o[4], m[4];
#pragma unroll
    for (int e2 = 0; e2 < 4; ++e2) {
      const int c = 8 * c8 + 2 * e2, tc = cb + c;
      uint32_t v = pack_bf16x2_rn(__uint_as_float(acc[c]), __uint_as_float(acc[c + 1]));
      m[e2] = v;
      if (save) {
        put_code<QBIT>(w1, c, fastq_code_bits<QBIT>(bf16lo_to_f32(v), sR[tc]) & G::CM);
        put_code<QBIT>(w1, c + 1, fastq_code_bits<QBIT>(bf16hi_to_f32(v), sR[tc + 1]) & G::CM);
      }
      if (has0) v = add2(v, pack_bf16x2_rn(lora_dot_f32(xa0, sB0 + tc * 16), lora_dot_f32(xa0, sB0 + (tc + 1) * 16)));
      if (has1) v = add2(v, pack_bf16x2_rn(lora_dot_f32(xa1, sB1 + tc * 16), lora_dot_f32(xa1, sB1 + (tc + 1) * 16)));
      if (has_res) v = add2(v, r[e2]);
      o[e2] = v;
    }
    if (valid) {
      store4_pairs(p.out0 + row * p.N + n + 8 * c8, o);
      if (p.dbg1 != nullptr) store4_pairs(p.dbg1 + row * p.N + n + 8 * c8, m);
    }
  }
  if (save && valid) store_block_words<QBIT>(p.q1 + (row * p.N + n) * QBIT / 8, w1);
}

// ------------------------------------------------------------------ the kernel
template <int EPI, int QBIT, bool B_MN, bool PAIR>
__global__ void __launch_bounds__(THREADS, 1)
mlp_gemm_kernel(const __grid_constant__ CUtensorMap mapA1, const __grid_constant__ CUtensorMap mapB1,
                const __grid_constant__ CUtensorMap mapA2, const __grid_constant__ CUtensorMap mapB2,
                const __grid_constant__ CUtensorMap mapA3, const __grid_constant__ CUtensorMap mapB3,
                const Params p) {
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment for the 128-byte swizzle atoms
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* stage_base = smem;
  constexpr int STAGES = Geo<PAIR>::STAGES, STAGE_BYTES = Geo<PAIR>::STAGE_BYTES, TILE_M = Geo<PAIR>::TILE_M;
  constexpr int B_COLS = Geo<PAIR>::B_COLS;
  __nv_bfloat16* epi_b = reinterpret_cast<__nv_bfloat16*>(smem + PIPE_BYTES);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + PIPE_BYTES + EPI_SMEM_BYTES);
  uint64_t* full = bars;                           // [STAGES]
  uint64_t* empty = bars + MAX_STAGES;             // [STAGES]
  uint64_t* tmem_full = bars + 2 * MAX_STAGES;     // [2]
  uint64_t* tmem_empty = bars + 2 * MAX_STAGES + 2;  // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * MAX_STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // rank 0: leader of the pair (issues the MMAs), 1: its peer; a CTA on its own is its own leader
  const uint32_t rank = PAIR ? cluster_ctarank() : 0u;
  const int pair = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x, num_pairs = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;
  const int tiles_m = (p.M + TILE_M - 1) / TILE_M;
  constexpr int TILE_N = (EPI == EPI_GATEUP) ? BN / 2 : BN;     // output columns per tile
  const int tiles_n = p.N / TILE_N;
  const int num_tiles = tiles_m * tiles_n;
  const int kb1 = p.K1 / BK, kb2 = (p.K1 + p.K2) / BK, kb_total = (p.K1 + p.K2 + p.K3) / BK;

  if (threadIdx.x == 0) {
    // full / tmem_empty are used in the leader only: the loads of both CTAs and the epilogue warps of both CTAs
    // arrive there; empty / tmem_full exist in both CTAs and are signalled together by the leader's commits
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&tmem_full[b], 1); mbar_init(&tmem_empty[b], (PAIR ? 2 : 1) * EPI_WARPS); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    if (PAIR) {
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    } else {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
  }
  tc_fence_before();
  __syncthreads();
  if (PAIR) cluster_sync_all();      // the peer's barriers are initialised before anything is signalled there
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int pit = 0;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, ++pit) {
        const int m0 = (tile % tiles_m) * TILE_M + (int)rank * BM, n0 = (tile / tiles_m) * TILE_N;
        TC_STAMP(0, pit, 0);
        for (int kb = 0; kb < kb_total; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1u, abort_flag)) {
            if (!*abort_flag) { *abort_flag = 1; atomicExch(p.status, ST_TIMEOUT_PRODUCER); }
            ok = false;
            break;
          }
          const int seg = kb < kb1 ? 0 : (kb < kb2 ? 1 : 2);
          const CUtensorMap* ma = seg == 0 ? &mapA1 : (seg == 1 ? &mapA2 : &mapA3);
          const CUtensorMap* mb = seg == 0 ? &mapB1 : (seg == 1 ? &mapB2 : &mapB3);
          const int k0 = (seg == 0 ? kb : (seg == 1 ? kb - kb1 : kb - kb2)) * BK;
          const uint32_t sa = smem_u32(stage_base + stage * STAGE_BYTES);
          const uint32_t sb = sa + STAGE_A_BYTES;
          // pair form: the leader's barrier counts both CTAs' bytes
          const uint32_t fbar = PAIR ? map_to_cta(&full[stage], 0) : smem_u32(&full[stage]);
          if (rank == 0) mbar_expect_tx(&full[stage], (PAIR ? 2 : 1) * STAGE_BYTES);
          tma_load_2d<PAIR>(sa, ma, fbar, k0, m0);
          if (EPI == EPI_GATEUP) {
            // B columns 0..127 of the tile are 128 rows of Wg, columns 128..255 the same rows of Wu (pair form: the
            // leader fetches the former, the peer the latter)
            if (PAIR) {
              tma_load_2d<PAIR>(sb, rank == 0 ? &mapB1 : &mapB2, fbar, k0, n0);
            } else {
              tma_load_2d<PAIR>(sb, &mapB1, fbar, k0, n0);
              tma_load_2d<PAIR>(sb + 16384, &mapB2, fbar, k0, n0);
            }
          } else if (B_MN) {
            // [K, N] row-major: this CTA's columns as boxes of 64 k-rows x 64 columns (8 KB each)
#pragma unroll
            for (int j = 0; j < B_COLS / 64; ++j) tma_load_2d<PAIR>(sb + j * 8192, mb, fbar, n0 + (int)rank * B_COLS + 64 * j, k0);
          } else {
            tma_load_2d<PAIR>(sb, mb, fbar, k0, n0 + (int)rank * B_COLS);      // one box of B_COLS rows x 64 k
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        TC_STAMP(0, pit, 1);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------ MMA issuer (leader CTA only)
    if (lane == 0 && rank == 0) {
      // instruction descriptor: fp32 accumulate, bf16 x bf16, M = 256 (the pair) or 128, N = 256, B major as given
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((B_MN ? 1u : 0u) << 16) |
                             ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(TILE_M >> 4) << 24);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, ++it) {
        const int buf = it & 1;
        const uint32_t bphase = (uint32_t)(it >> 1) & 1u;
        TC_STAMP(1, it, 0);
        if (!mbar_wait(&tmem_empty[buf], bphase ^ 1u, abort_flag)) {
          if (!*abort_flag) { *abort_flag = 1; atomicExch(p.status, ST_TIMEOUT_MMA); }
          break;
        }
        tc_fence_after();
        TC_STAMP(1, it, 1);
        const uint32_t d_tmem = tmem_base + (uint32_t)(buf * BN);
        for (int kb = 0; kb < kb_total; ++kb) {
          if (!mbar_wait(&full[stage], phase, abort_flag)) {
            if (!*abort_flag) { *abort_flag = 1; atomicExch(p.status, ST_TIMEOUT_MMA); }
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(stage_base + stage * STAGE_BYTES);
          const uint32_t sb = sa + STAGE_A_BYTES;
          const uint64_t adesc = make_desc(sa, 16, 1024);
          const uint64_t bdesc = B_MN ? make_desc(sb, 64 * 128, 1024) : make_desc(sb, 16, 1024);
#pragma unroll
          for (int kk = 0; kk < BK / 16; ++kk) {
            // K-major: 16 elements = 32 bytes further along the swizzled row; MN-major: 16 k-rows of 128 bytes
            const uint64_t a = adesc + (uint64_t)(kk * 2);
            const uint64_t b = bdesc + (uint64_t)(B_MN ? kk * 128 : kk * 2);
            tc_mma<PAIR>(d_tmem, a, b, idesc, (kb > 0 || kk > 0) ? 1u : 0u);
          }
          tc_commit<PAIR>(&empty[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok) tc_commit<PAIR>(&tmem_full[buf]);
        TC_STAMP(1, it, 2);
      }
    }
  } else {
    // ------------------------------------------------ epilogue warps
    const int et = threadIdx.x - 64;
    const int quad = warp & 3;
    const int chalf = (warp - 2) >> 2;
    // scratch of the epilogue warps (layout: see EPI_SMEM_BYTES)
    float* sG1 = reinterpret_cast<float*>(epi_b);                 // STORE: two fp32 LoRA-B tiles of BN columns
    float* sG2 = sG1 + BN * 16;
    float* sGV = sG2 + BN * 16;                                   // STORE: BN quantizer constants
    __nv_bfloat16* sGS = reinterpret_cast<__nv_bfloat16*>(sGV);   // GRADDOWN: two bf16 scale vectors of BN
    uint32_t* sR1 = reinterpret_cast<uint32_t*>(epi_b) + (warp - 2) * 1024;   // GRADDOWN: this warp's two tiles
    uint32_t* sR2 = sR1 + 512;
    float* sF0 = sG1;                                             // GATEUP: two tiles of BN/2 columns ...
    float* sF1 = sF0 + (BN / 2) * 16;
    float* sV = sG2;                                              // ... and two float vectors at sV, sV + BN
    int it = 0;
    const uint32_t tmem_empty_leader[2] = {PAIR ? map_to_cta(&tmem_empty[0], 0) : smem_u32(&tmem_empty[0]),
                                           PAIR ? map_to_cta(&tmem_empty[1], 0) : smem_u32(&tmem_empty[1])};
    for (int tile = pair; tile < num_tiles; tile += num_pairs, ++it) {
      const int m0 = (tile % tiles_m) * TILE_M + (int)rank * BM, n0 = (tile / tiles_m) * TILE_N;
      const int buf = it & 1;
      const uint32_t bphase = (uint32_t)(it >> 1) & 1u;
      const int64_t row = (int64_t)m0 + quad * 32 + lane;
      const bool valid = row < p.M;
      if (et == 0) TC_STAMP(2, it, 0);

      // stage the per-tile LoRA-B rows and scales (previous tile's readers are done: barrier at the end)
      if (EPI == EPI_STORE) {
        stage_lora_tile_f32(p.l0, n0, BN, sG1, et);
        stage_lora_tile_f32(p.l1, n0, BN, sG2, et);
        if (p.q1 != nullptr) sGV[et] = fastq_scale<QBIT>(__frcp_rn(__bfloat162float(p.s1[n0 + et])));
      } else if (EPI == EPI_GATEUP) {
        // 128 output columns per tile: the two LoRA-B tiles fit as fp32 rows (2 x 8 KB)
        stage_lora_tile_f32(p.l0, n0, TILE_N, sF0, et);
        stage_lora_tile_f32(p.l1, n0, TILE_N, sF1, et);
        if (et < TILE_N) {
          sV[et] = fastq_scale<QBIT>(__frcp_rn(__bfloat162float(p.s1[n0 + et])));
          sV[BN + et] = fastq_scale<QBIT>(__frcp_rn(__bfloat162float(p.s2[n0 + et])));
        }
      } else {
        // the scales stay bf16: column pairs are read as one packed word
        sGS[et] = p.s1[n0 + et];
        sGS[BN + et] = p.s2[n0 + et];
      }
      float xa0[16], xa1[16];
      uint32_t fa1[2][4], fa2[2][4];       // GRADDOWN: the warp's LoRA-A rows as mma A fragments (two tiles of 16 rows)
      GdInputs<QBIT> gin;                  // GRADDOWN: global inputs of the next block, fetched one block ahead
      if (EPI != EPI_GRADDOWN) {
        load_xa_row(p.l0.xa, row, valid, xa0);
        load_xa_row(p.l1.xa, row, valid, xa1);
      } else {
        const int g = lane >> 2, t = lane & 3;
#pragma unroll
        for (int mt = 0; mt < 2; ++mt) {
          const int64_t ra = (int64_t)m0 + quad * 32 + 16 * mt + g, rb = ra + 8;
#pragma unroll
          for (int j = 0; j < 4; ++j) { fa1[mt][j] = 0u; fa2[mt][j] = 0u; }
          if (p.l1.xa != nullptr && p.l2.xa != nullptr) {
            if (ra < p.M) {
              fa1[mt][0] = *reinterpret_cast<const uint32_t*>(p.l1.xa + ra * 16 + 2 * t);
              fa1[mt][2] = *reinterpret_cast<const uint32_t*>(p.l1.xa + ra * 16 + 2 * t + 8);
              fa2[mt][0] = *reinterpret_cast<const uint32_t*>(p.l2.xa + ra * 16 + 2 * t);
              fa2[mt][2] = *reinterpret_cast<const uint32_t*>(p.l2.xa + ra * 16 + 2 * t + 8);
            }
            if (rb < p.M) {
              fa1[mt][1] = *reinterpret_cast<const uint32_t*>(p.l1.xa + rb * 16 + 2 * t);
              fa1[mt][3] = *reinterpret_cast<const uint32_t*>(p.l1.xa + rb * 16 + 2 * t + 8);
              fa2[mt][1] = *reinterpret_cast<const uint32_t*>(p.l2.xa + rb * 16 + 2 * t);
              fa2[mt][3] = *reinterpret_cast<const uint32_t*>(p.l2.xa + rb * 16 + 2 * t + 8);
            }
          }
        }
        // the first block's inputs are on their way while the warp waits for the accumulator
        gd_fetch<QBIT>(p, (int64_t)m0 + quad * 32, lane, (int64_t)n0 + 128 * chalf, gin);
      }
      epi_bar_sync();
      if (et == 0) TC_STAMP(2, it, 1);

      if (!mbar_wait(&tmem_full[buf], bphase, abort_flag)) {
        if (!*abort_flag) { *abort_flag = 1; atomicExch(p.status, ST_TIMEOUT_EPILOGUE); }
        break;
      }
      tc_fence_after();
      if (et == 0) TC_STAMP(2, it, 2);
      const uint32_t t_lane = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(buf * BN);
      if (EPI == EPI_GATEUP) {
        // gate columns [0, 128) and up columns [128, 256) of the accumulator; this warp takes 64 of each
#pragma unroll 1
        for (int ch = 0; ch < 2; ++ch) {
          uint32_t g[32], u[32];
          const int cb = 64 * chalf + 32 * ch;
          tc_ld32(t_lane + (uint32_t)cb, g);
          tc_ld32(t_lane + (uint32_t)(TILE_N + cb), u);
          epi_gateup_block<QBIT>(p, row, valid, n0, cb, g, u, xa0, xa1, sF0, sF1, sV, sV + BN);
        }
      } else {
#pragma unroll 1
        for (int ch = 0; ch < 4; ++ch) {
          uint32_t acc[32];
          const int cb = 128 * chalf + 32 * ch;
          tc_ld32(t_lane + (uint32_t)cb, acc);
          if (EPI == EPI_STORE) {
            epi_store_block<QBIT>(p, row, valid, n0, cb, acc, xa0, xa1, sG1, sG2, sGV);
          } else {
            const GdInputs<QBIT> cur = gin;
            if (ch < 3) gd_fetch<QBIT>(p, (int64_t)m0 + quad * 32, lane, (int64_t)n0 + cb + 32, gin);
            epi_graddown_block<QBIT>(p, (int64_t)m0 + quad * 32, lane, n0, cb, acc, cur, fa1, fa2, sR1, sR2,
                                     reinterpret_cast<const uint32_t*>(sGS), reinterpret_cast<const uint32_t*>(sGS + BN));
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (et == 0) TC_STAMP(2, it, 3);
      if (lane == 0) mbar_arrive_cluster(tmem_empty_leader[buf]);
      epi_bar_sync();    // everyone is done with the staged tile before the next one overwrites it
      if (et == 0) TC_STAMP(2, it, 4);
    }
  }

  // ------------------------------------------------ teardown
  // both CTAs are done with each other's barriers and tensor memory before either leaves
  tc_fence_before();
  __syncthreads();
  if (PAIR) cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    if (PAIR) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    else asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
      return nullptr;
    fn = reinterpret_cast<EncodeTiledFn>(sym);
  }
  return fn;
}

// row-major bf16 matrix [rows, cols] (cols contiguous), box = 64 columns x box_rows rows, 128-byte swizzle
static bool make_map(CUtensorMap* m, const void* ptr, int64_t rows, int64_t cols, int box_rows) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return false;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
  cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1u, 1u};
  return enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// The grad_down kernel stays on single CTAs: measured 175 us single against 197 us as pairs at the Llama-2-7B
// shapes (its epilogue runs mma.sync products on the same tensor pipe, and in a pair a stall of either SM holds
// up both); the other three products gain 5-16 % as pairs.
#ifndef HYC_GD_PAIR
#define HYC_GD_PAIR 0          // 1: build the grad_down kernel as pairs too (for measurements)
#endif
template <int EPI> struct UsePair { static constexpr bool value = EPI != EPI_GRADDOWN || HYC_GD_PAIR != 0; };

template <int EPI, int QBIT, bool B_MN>
static int launch(const CUtensorMap& a1, const CUtensorMap& b1, const CUtensorMap& a2, const CUtensorMap& b2,
                  const CUtensorMap& a3, const CUtensorMap& b3, const Params& p, cudaStream_t st) {
  constexpr bool PAIR = UsePair<EPI>::value;
  auto kern = mlp_gemm_kernel<EPI, QBIT, B_MN, PAIR>;
  // the attribute belongs to a (function, device) pair: set once per device (unknown device: every time)
  static bool attr[64] = {false};
  const int slot = current_device_slot();
  if (slot < 0 || !attr[slot]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess) {
      hyc_set_last_cuda_error((int)cudaGetLastError());
      return HYC_ERR_LAUNCH;
    }
    if (slot >= 0) attr[slot] = true;
  }
  constexpr int TILE_N = (EPI == EPI_GATEUP) ? BN / 2 : BN;
  const int tiles = ((p.M + Geo<PAIR>::TILE_M - 1) / Geo<PAIR>::TILE_M) * (p.N / TILE_N);
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = SMEM_BYTES;
  cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = 2; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
  cfg.attrs = at;
  cfg.numAttrs = PAIR ? 1 : 0;
  // the kernel is persistent: one CTA per SM, or one pair per two neighbouring SMs (as many as can be resident)
  int units = num_sms();
  if (PAIR) {
    static int pairs_on[64] = {0};
    int pairs = slot >= 0 ? pairs_on[slot] : 0;
    if (pairs == 0) {
      cfg.gridDim = dim3(2 * (unsigned)(num_sms() / 2));
      int n = 0;
      if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n < 1) { cudaGetLastError(); n = num_sms() / 2; }
      pairs = n < num_sms() / 2 ? n : num_sms() / 2;
      if (pairs < 1) pairs = 1;
      if (slot >= 0) pairs_on[slot] = pairs;
    }
    units = pairs;
  }
  cfg.gridDim = dim3((unsigned)((PAIR ? 2 : 1) * (tiles < units ? tiles : units)));
  Params pp = p;
#ifdef HYC_TC_PROF
  pp.prof = g_tc_prof;
#endif
  if (cudaLaunchKernelEx(&cfg, kern, a1, b1, a2, b2, a3, b3, pp) != cudaSuccess) {
    hyc_set_last_cuda_error((int)cudaGetLastError());
    return HYC_ERR_LAUNCH;
  }
  return HYC_OK;
}

}  // namespace tc
}  // namespace hyc

using namespace hyc;
using namespace hyc::tc;

static LoraTerm make_term(const void* xa, const void* bt, int64_t ld_col, int64_t ld_r) {
  LoraTerm t;
  t.xa = (const __nv_bfloat16*)xa;
  t.bt = (const __nv_bfloat16*)bt;
  t.ld_col = ld_col;
  t.ld_r = ld_r;
  return t;
}

extern "C" HYC_API int hyc_gemm_bf16_tcgen05(
    const void* A, const void* B, int M, int N, int K, int b_is_kn,
    const void* A2, const void* B2, int K2, const void* A3, const void* B3, int K3,
    const void* xa0, const void* bt0, int64_t bt0_ld_col, int64_t bt0_ld_r,
    const void* xa1, const void* bt1, int64_t bt1_ld_col, int64_t bt1_ld_r,
    const void* residual, void* D, int* status, void* stream) {
  if (!A || !B || !D || !status) return HYC_ERR_NULL;
  if ((K2 > 0) != (A2 != nullptr && B2 != nullptr)) return HYC_ERR_NULL;
  if ((K3 > 0) != (A3 != nullptr && B3 != nullptr)) return HYC_ERR_NULL;
  if (M <= 0 || N <= 0 || K <= 0 || N % BN != 0 || K % BK != 0 || K2 < 0 || K2 % BK != 0 || K3 < 0 || K3 % BK != 0)
    return HYC_ERR_SHAPE;
  if (!aligned(A, 16) || !aligned(B, 16) || !aligned(D, 16) || (residual && !aligned(residual, 16)) ||
      (xa0 && !aligned(xa0, 16)) || (xa1 && !aligned(xa1, 16)) || (A2 && (!aligned(A2, 16) || !aligned(B2, 16))) ||
      (A3 && (!aligned(A3, 16) || !aligned(B3, 16)))) return HYC_ERR_ALIGN;
  if ((bt0 != nullptr) != (xa0 != nullptr) || (bt1 != nullptr) != (xa1 != nullptr)) return HYC_ERR_NULL;
  CUtensorMap a1, b1, a2, b2, a3, b3;
  bool ok = make_map(&a1, A, M, K, BM);
  ok = ok && (b_is_kn ? make_map(&b1, B, K, N, 64) : make_map(&b1, B, N, K, 128));
  a2 = a1; b2 = b1;
  if (K2 > 0) {
    ok = ok && make_map(&a2, A2, M, K2, BM);
    ok = ok && (b_is_kn ? make_map(&b2, B2, K2, N, 64) : make_map(&b2, B2, N, K2, 128));
  }
  a3 = a1; b3 = b1;
  if (K3 > 0) {
    ok = ok && make_map(&a3, A3, M, K3, BM);
    ok = ok && (b_is_kn ? make_map(&b3, B3, K3, N, 64) : make_map(&b3, B3, N, K3, 128));
  }
  if (!ok) return HYC_ERR_UNSUPPORTED;
  Params p = {};
  p.M = M; p.N = N; p.K1 = K; p.K2 = K2; p.K3 = K3; p.epi = EPI_STORE; p.q_bit = 0;
  p.l0 = make_term(xa0, bt0, bt0_ld_col, bt0_ld_r);
  p.l1 = make_term(xa1, bt1, bt1_ld_col, bt1_ld_r);
  p.l2 = make_term(nullptr, nullptr, 0, 0);
  p.residual = (const __nv_bfloat16*)residual;
  p.out0 = (__nv_bfloat16*)D;
  p.status = status;
  cudaStream_t st = (cudaStream_t)stream;
  return b_is_kn ? launch<EPI_STORE, 4, true>(a1, b1, a2, b2, a3, b3, p, st)
                 : launch<EPI_STORE, 4, false>(a1, b1, a2, b2, a3, b3, p, st);
}

extern "C" HYC_API int hyc_mlp_gateup_fwd_tcgen05(
    const void* x, const void* wg, const void* wu, int T, int H, int I,
    const void* xa1, const void* b1t, int64_t b1_ld_col, int64_t b1_ld_r,
    const void* xa2, const void* b2t, int64_t b2_ld_col, int64_t b2_ld_r,
    const void* s1, const void* s2, void* q1, void* q2, void* o, void* main1_or_null, void* main2_or_null,
    int q_bit, int* status, void* stream) {
  if (!x || !wg || !wu || !xa1 || !b1t || !xa2 || !b2t || !s1 || !s2 || !q1 || !q2 || !o || !status) return HYC_ERR_NULL;
  if (q_bit != 2 && q_bit != 4 && q_bit != 8) return HYC_ERR_QBIT;
  if (T <= 0 || H <= 0 || I <= 0 || I % (BN / 2) != 0 || H % BK != 0) return HYC_ERR_SHAPE;
  const void* al[] = {x, wg, wu, xa1, xa2, q1, q2, o};
  for (const void* q : al) if (!aligned(q, 16)) return HYC_ERR_ALIGN;
  CUtensorMap a1, bg, bu;
  if (!make_map(&a1, x, T, H, BM) || !make_map(&bg, wg, I, H, 128) || !make_map(&bu, wu, I, H, 128)) return HYC_ERR_UNSUPPORTED;
  Params p = {};
  p.M = T; p.N = I; p.K1 = H; p.K2 = 0; p.K3 = 0; p.epi = EPI_GATEUP; p.q_bit = q_bit;
  p.l0 = make_term(xa1, b1t, b1_ld_col, b1_ld_r);
  p.l1 = make_term(xa2, b2t, b2_ld_col, b2_ld_r);
  p.l2 = make_term(nullptr, nullptr, 0, 0);
  p.out0 = (__nv_bfloat16*)o;
  p.dbg1 = (__nv_bfloat16*)main1_or_null; p.dbg2 = (__nv_bfloat16*)main2_or_null;
  p.q1 = (uint8_t*)q1; p.q2 = (uint8_t*)q2;
  p.s1 = (const __nv_bfloat16*)s1; p.s2 = (const __nv_bfloat16*)s2;
  p.status = status;
  cudaStream_t st = (cudaStream_t)stream;
  // the A2 slot is unused; mapB2 carries the up-projection weight
  if (q_bit == 2) return launch<EPI_GATEUP, 2, false>(a1, bg, a1, bu, a1, bg, p, st);
  if (q_bit == 4) return launch<EPI_GATEUP, 4, false>(a1, bg, a1, bu, a1, bg, p, st);
  return launch<EPI_GATEUP, 8, false>(a1, bg, a1, bu, a1, bg, p, st);
}

extern "C" HYC_API int hyc_mlp_graddown_bwd_tcgen05(
    const void* g, const void* wd, int T, int H, int I,
    const void* a_lora, const void* b_lora, int k_lora,
    const void* xa1, const void* b1t, int64_t b1_ld_col, int64_t b1_ld_r,
    const void* xa2, const void* b2t, int64_t b2_ld_col, int64_t b2_ld_r,
    const void* q1, const void* s1, const void* q2, const void* s2,
    const void* lora_gate, const void* lora_up, int64_t ld_lora,
    void* o, void* grad_gate, void* grad_up, int q_bit, int* status, void* stream) {
  if (!g || !wd || !q1 || !s1 || !q2 || !s2 || !o || !grad_gate || !grad_up || !status) return HYC_ERR_NULL;
  const bool pre = lora_gate != nullptr || lora_up != nullptr;
  if (pre) {
    if (!lora_gate || !lora_up) return HYC_ERR_NULL;
    if (ld_lora < I || ld_lora % 8 != 0) return HYC_ERR_SHAPE;
    if (!aligned(lora_gate, 16) || !aligned(lora_up, 16)) return HYC_ERR_ALIGN;
  } else if (!xa1 || !b1t || !xa2 || !b2t) {
    return HYC_ERR_NULL;
  }
  if ((k_lora > 0) != (a_lora != nullptr && b_lora != nullptr)) return HYC_ERR_NULL;
  if (q_bit != 2 && q_bit != 4 && q_bit != 8) return HYC_ERR_QBIT;
  if (T <= 0 || H <= 0 || I <= 0 || I % BN != 0 || H % BK != 0 || k_lora < 0 || k_lora % BK != 0) return HYC_ERR_SHAPE;
  const void* al[] = {g, wd, q1, q2, o, grad_gate, grad_up};
  for (const void* q : al) if (!aligned(q, 16)) return HYC_ERR_ALIGN;
  if (!pre && (!aligned(xa1, 16) || !aligned(xa2, 16))) return HYC_ERR_ALIGN;
  if (a_lora && (!aligned(a_lora, 16) || !aligned(b_lora, 16))) return HYC_ERR_ALIGN;
  CUtensorMap a1, b1, a2, b2;
  // wd is [H, I] row-major: the K = H rows are the reduction dimension, so B is MN-major
  if (!make_map(&a1, g, T, H, BM) || !make_map(&b1, wd, H, I, 64)) return HYC_ERR_UNSUPPORTED;
  a2 = a1; b2 = b1;
  if (k_lora > 0 && (!make_map(&a2, a_lora, T, k_lora, BM) || !make_map(&b2, b_lora, k_lora, I, 64))) return HYC_ERR_UNSUPPORTED;
  Params p = {};
  p.M = T; p.N = I; p.K1 = H; p.K2 = k_lora; p.K3 = 0; p.epi = EPI_GRADDOWN; p.q_bit = q_bit;
  p.l0 = make_term(nullptr, nullptr, 0, 0);
  p.l1 = pre ? make_term(nullptr, nullptr, 0, 0) : make_term(xa1, b1t, b1_ld_col, b1_ld_r);
  p.l2 = pre ? make_term(nullptr, nullptr, 0, 0) : make_term(xa2, b2t, b2_ld_col, b2_ld_r);
  p.lpre1 = (const __nv_bfloat16*)lora_gate; p.lpre2 = (const __nv_bfloat16*)lora_up; p.ld_pre = ld_lora;
  p.out0 = (__nv_bfloat16*)o; p.out1 = (__nv_bfloat16*)grad_gate; p.out2 = (__nv_bfloat16*)grad_up;
  p.q1 = (uint8_t*)const_cast<void*>(q1); p.q2 = (uint8_t*)const_cast<void*>(q2);
  p.s1 = (const __nv_bfloat16*)s1; p.s2 = (const __nv_bfloat16*)s2;
  p.status = status;
  cudaStream_t st = (cudaStream_t)stream;
  if (q_bit == 2) return launch<EPI_GRADDOWN, 2, true>(a1, b1, a2, b2, a1, b1, p, st);
  if (q_bit == 4) return launch<EPI_GRADDOWN, 4, true>(a1, b1, a2, b2, a1, b1, p, st);
  return launch<EPI_GRADDOWN, 8, true>(a1, b1, a2, b2, a1, b1, p, st);
}

extern "C" HYC_API int hyc_linear_lora_save_fwd_tcgen05(
    const void* x, const void* w, int T, int K, int N,
    const void* xa, const void* bt, int64_t bt_ld_col, int64_t bt_ld_r,
    const void* scale, void* q_out, void* y, void* main_or_null, int q_bit, int* status, void* stream) {
  if (!x || !w || !scale || !q_out || !y || !status) return HYC_ERR_NULL;
  if ((xa != nullptr) != (bt != nullptr)) return HYC_ERR_NULL;
  if (q_bit != 2 && q_bit != 4 && q_bit != 8) return HYC_ERR_QBIT;
  if (T <= 0 || N <= 0 || K <= 0 || N % BN != 0 || K % BK != 0) return HYC_ERR_SHAPE;
  if (!aligned(x, 16) || !aligned(w, 16) || !aligned(y, 16) || !aligned(q_out, 16) || (xa && !aligned(xa, 16)) ||
      (main_or_null && !aligned(main_or_null, 16))) return HYC_ERR_ALIGN;
  CUtensorMap a1, b1;
  if (!make_map(&a1, x, T, K, BM) || !make_map(&b1, w, N, K, 128)) return HYC_ERR_UNSUPPORTED;
  Params p = {};
  p.M = T; p.N = N; p.K1 = K; p.K2 = 0; p.K3 = 0; p.epi = EPI_STORE; p.q_bit = q_bit;
  p.l0 = make_term(xa, bt, bt_ld_col, bt_ld_r);
  p.l1 = make_term(nullptr, nullptr, 0, 0);
  p.l2 = make_term(nullptr, nullptr, 0, 0);
  p.out0 = (__nv_bfloat16*)y;
  p.dbg1 = (__nv_bfloat16*)main_or_null;
  p.q1 = (uint8_t*)q_out;
  p.s1 = (const __nv_bfloat16*)scale;
  p.status = status;
  cudaStream_t st = (cudaStream_t)stream;
  if (q_bit == 2) return launch<EPI_STORE, 2, false>(a1, b1, a1, b1, a1, b1, p, st);
  if (q_bit == 4) return launch<EPI_STORE, 4, false>(a1, b1, a1, b1, a1, b1, p, st);
  return launch<EPI_STORE, 8, false>(a1, b1, a1, b1, a1, b1, p, st);
}

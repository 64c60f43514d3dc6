// patina_gemm_kernel.cuh -- the persistent, warp-specialised tcgen05 GEMM.
//
//   C[M,N] = alpha * A[M,K] * B[N,K]^T      (both operands K-major, "TN")
//
// One CTA = 6 and more warps with fixed roles, the split the reference's generated
// kernel uses (crates/patina/tests/golden/v2_gemm_pipelined.ptx:89-94) and a few more:
//   warp 0      TMA producer   (one lane per load of a stage: each A slab, B)
//   warp 1      MMA issuer     (one elected lane; the whole warp owns TMEM alloc/dealloc)
//   warps 2..   epilogue       (TMEM -> registers -> swizzled SMEM -> TMA store),
//               four warps per accumulator sub-tile, one per TMEM lane quarter
//   then, where they exist: the scale producer of block-scaled kernels, and a second
//               MMA issuer in kernels with two accumulators to multiply into at once
//               (two sub-tiles, or the even and odd k-blocks of a narrow tile)
//
// What is different from that kernel (which runs one 128x128 tile in one CTA):
//   * persistent: each CTA (or CTA pair) walks a list of output tiles
//     (patina::tile_coord), so prologue cost is paid once per SM;
//   * 128-byte-swizzled K-major stages of 128 bytes of K, kStages deep;
//   * kMSub == 1: two accumulators in TMEM (2 x BN columns) so the epilogue of
//     tile i overlaps the mainloop of tile i+1;
//     kMSub == 2: each CTA owns two 128-row sub-tiles that share every B stage
//     (a 256 x BN tile per CTA, 512 x BN per pair), which cuts operand traffic
//     from L2 by a quarter; the accumulators then fill TMEM, so the epilogue
//     (eight warps) is not overlapped with the next mainloop, only with its
//     operand prefetch;
//   * optional CTA pair (kCtaGroup == 2): tcgen05.mma.cta_group::2 computes a
//     256 x BN tile; each CTA loads its own 128 rows of A and its own BN/2 rows
//     of B; the pair leader issues the MMAs. No TMA load is multicast: each
//     CTA's loads land in its own shared memory and count on the leader's
//     barrier (the one multicast in the file is the commit that signals both CTAs);
//   * every wait is bounded (WaitCtx): on expiry the CTA records a status code,
//     raises an abort flag that all roles poll, drains and returns.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include "patina_desc.h"
#include "patina_ptx.cuh"

namespace patina {

// Where a finished sub-tile of C is stored: one tensor map per destination. One destination is
// the normal case; several are the column-shard scatter, where every GPU of a node writes its
// column block into each GPU's full-width C (the other maps point into peer memory mapped
// over NVLink; TMA *stores* there are plain peer writes, nothing is multicast or loaded).
// A plain launch carries one map; only the scatter's instantiations carry kMaxDests of them
// (a kilobyte of kernel parameters that every other launch would pay for in launch latency).
constexpr int kMaxDests = 8;
template <int kDests>
struct CStoreMaps {
  CUtensorMap map[kDests];
};

struct GemmParams {
  uint32_t M, N, K;
  uint32_t tiles_m, tiles_n, num_tiles;  // in units of the cluster tile
  uint32_t k_blocks;                     // ceil(K / elements per 128 bytes)
  uint32_t group_m;                      // scheduler band height (tiles)
  float alpha;
  // fused epilogue (kernels instantiated with kFused): C = act(alpha*acc + bias[n] + beta*R[m,n])
  const float* bias;            // N floats or null
  const __nv_bfloat16* residual;  // [M, ldr] bf16 or null
  int64_t ldr;
  float beta;
  uint32_t activation;     // Activation
  // e4m3 output (kernels instantiated with kOutE4M3): C = e4m3_sat(out_scale * act(...)); the
  // largest |act(...)| of the launch is folded into *amax with an atomic max (may be null)
  float out_scale;
  float* amax;
  uint32_t n_dests;        // destinations of C (1..kMaxDests)
  // Two-sub-tile kernels, plain launch: scheduler indices from split_from on are HALF tiles
  // (index split_from + 2 i + h is sub-tile h of tile split_from + i); num_tiles counts
  // scheduler indices. The host splits the tiles of a last wave that fills at most half of the
  // clusters: the wave then takes half as long. Every accumulator still sees the same MMAs in the
  // same order, so results do not change. No split: split_from >= num_tiles.
  uint32_t split_from;
  // grouped launch (kernels instantiated with kGrouped): A and C hold the groups' rows one
  // after another, B holds one [N, K] block per group; M above is the total row count
  const int32_t* group_rows;  // device array, rows of A and C per group
  const float* group_alpha;   // device array, one more factor per group (e.g. an expert's weight
                              // scale for fp8 inputs), or null
  uint32_t n_groups;          // <= kMaxGroups
  // C itself (every destination), for boxes the TMA store cannot clip: TMA stores clip at
  // 16-byte granularity, so a box that crosses column N when N * element size is not a
  // multiple of 16 bytes, and (grouped launch) a box that crosses a group's last row, are
  // written row by row from the registers instead.
  void* c_dests[kMaxDests];
  int64_t ldc;
  // block-scaled operands (kernels instantiated with kMXE4M3): extents of the scale buffers in
  // atoms of 128 rows x 128 K elements, so that tiles hanging over the edge read inside them
  uint32_t sf_m_blocks, sf_n_blocks, sf_k_atoms;
  uint32_t* status;        // [0] first error code, [1] block, [2] detail; 0 = ok
  uint64_t wait_limit_ns;  // bound for every barrier wait
#ifdef PATINA_TRACE
  unsigned long long* trace;  // [grid][64]: time stamps of a trace build (never in the shipped library);
                              // words 32..47: cycle counter when the MMA issuer's wait for k-block i of
                              // its first tile returned, 48..63: when the producer issued its loads
  uint32_t l2_hint_a, l2_hint_b;  // trace builds: L2 eviction hint on operand loads of pair kernels
                                  // (0 none, 1 evict-first, 2 evict-last)
#endif
};

// Time stamps for a trace build (-DPATINA_TRACE): slot s of this CTA gets the global timer,
// slot 16 + s the SM's cycle counter. The shipped library compiles these to nothing.
#ifdef PATINA_TRACE
#define PATINA_TRACE_AT(slot)                                                     \
  do {                                                                            \
    if (p.trace) {                                                                \
      p.trace[(size_t)blockIdx.x * 64u + (slot)] = ptx::globaltimer_ns();         \
      p.trace[(size_t)blockIdx.x * 64u + 16u + (slot)] = (unsigned long long)clock64(); \
    }                                                                             \
  } while (0)
#define PATINA_TRACE_KB(base, i)                                                             \
  do {                                                                                      \
    if (p.trace && (i) < 16u) p.trace[(size_t)blockIdx.x * 64u + (base) + (i)] = (unsigned long long)clock64(); \
  } while (0)
#else
#define PATINA_TRACE_AT(slot) \
  do {                        \
  } while (0)
#define PATINA_TRACE_KB(base, i) \
  do {                           \
  } while (0)
#endif

constexpr uint32_t kMaxGroups = 128;
constexpr uint32_t kGroupTableBytes = 2u * (kMaxGroups + 1u) * 4u + 8u;  // row and tile prefix sums

enum Activation : uint32_t { kActNone = 0, kActRelu = 1, kActGelu = 2, kActSilu = 3 };

// erf to about 1e-6 absolute (Abramowitz & Stegun 7.1.26 with approximate reciprocal and
// exponential): two special-function instructions and a degree-5 polynomial; far inside the
// rounding of a bf16 result.
__device__ __forceinline__ float fast_erf(float x) {
  const float ax = fabsf(x);
  const float t = __fdividef(1.0f, fmaf(0.3275911f, ax, 1.0f));  // approximate reciprocal: 1 ulp-ish
  float poly = fmaf(1.061405429f, t, -1.453152027f);
  poly = fmaf(poly, t, 1.421413741f);
  poly = fmaf(poly, t, -0.284496736f);
  poly = fmaf(poly, t, 0.254829592f);
  const float y = 1.0f - poly * t * __expf(-ax * ax);
  return copysignf(y, x);
}

__device__ __forceinline__ float apply_activation(float x, uint32_t act) {
  switch (act) {
    case kActRelu: return fmaxf(x, 0.0f);
    case kActGelu: return 0.5f * x * (1.0f + fast_erf(x * 0.70710678118654752f));
    case kActSilu: return __fdividef(x, 1.0f + __expf(-x));
    default: return x;
  }
}

enum StatusCode : uint32_t {
  kStatusOk = 0,
  kTimeoutProducerEmpty = 1,
  kTimeoutMmaFull = 2,
  kTimeoutMmaTmemEmpty = 3,
  kTimeoutEpilogueTmemFull = 4,
  kTimeoutMmaDrain = 5,
};

struct WaitCtx {
  volatile uint32_t* abort_flag;  // this CTA's flag (shared memory)
  uint32_t peer_abort_addr;       // shared::cluster address of the partner's flag (pair only)
  uint32_t* status;
  uint64_t limit_ns;
  bool has_peer;
};

__device__ __noinline__ void raise_abort(const WaitCtx& w, uint32_t code, uint32_t detail) {
  *w.abort_flag = 1u;
  if (w.has_peer) ptx::st_cluster_u32(w.peer_abort_addr, 1u);
  if (atomicCAS(w.status, 0u, code) == 0u) {
    w.status[1] = blockIdx.x;
    w.status[2] = detail;
  }
  __threadfence();
}

// Returns false when the wait was abandoned (limit reached here, or another
// role raised the abort flag).
//
// try_wait itself blocks for a hardware-defined slice, so a few failed polls already mean
// microseconds; the abort flag and the clock are looked at every fourth one. (Looking at them
// only every 64th or 1024th poll, or polling with the non-blocking test_wait, was measured on
// twenty load- and compute-bound shapes: no difference in time anywhere, and an expired wait is
// noticed later, so the frequent check stays.)
constexpr uint32_t kWaitCheckEvery = 4u;
template <bool kClusterScope>
__device__ __forceinline__ bool bounded_wait(uint32_t bar, uint32_t parity, const WaitCtx& w,
                                             uint32_t code, uint32_t detail) {
  uint64_t t0 = 0;
  uint32_t spins = 0;
  for (;;) {
    const bool done = kClusterScope ? ptx::mbar_try_wait_cluster(bar, parity)
                                    : ptx::mbar_try_wait(bar, parity);
    if (done) return true;
    if ((++spins & (kWaitCheckEvery - 1u)) == 0u) {
      if (*w.abort_flag) return false;
      const uint64_t now = ptx::globaltimer_ns();
      if (t0 == 0) {
        t0 = now;
      } else if (now - t0 > w.limit_ns) {
        raise_abort(w, code, detail);
        return false;
      }
    }
  }
}

template <int kCtaGroup, int kMSub, int BN, int kStages, int kIn, int kOut, bool kFusedEpi = false,
          int kKChunks = 1>
struct GemmTraits {
  static constexpr uint32_t kEpiWarps = 4 * kMSub;            // one warp per (sub-tile, lane quarter)
  // producer + MMA + epilogue warps (+ the scale-producer warp of block-scaled kernels)
  // (+ a second MMA-issuing warp when there are two accumulator sub-tiles)
  // Two k-blocks per stage also means two accumulators per tile: the stage's first k-block is
  // multiplied into the first by one issuing thread, its second into the second by another, and
  // the epilogue adds the two (C = sum over even k-blocks + sum over odd k-blocks, in fp32: a
  // fixed order, but not the order of the one-accumulator kernels). One thread cannot issue the
  // MMAs of a narrow tile as fast as the tensor pipe retires them (85 cycles of issue against
  // 48 / 64 of pipe at 64 / 128 columns), and two threads may not share an accumulator.
  static constexpr bool kDualAcc = (kKChunks == 2);
  static constexpr uint32_t kIssuers = kDualAcc ? 2u : (uint32_t)kMSub;   // MMA-issuing threads
  static constexpr uint32_t kThreads =
      64 + 32 * kEpiWarps + (is_block_scaled(kIn) ? 32u : 0u) + (kIssuers == 2 ? 32u : 0u);
  static constexpr uint32_t kSecondIssuerWarp = 2 + kEpiWarps + (is_block_scaled(kIn) ? 1u : 0u);
  static constexpr uint32_t kBlockKElems = kBlockKBytes / input_bytes(kIn);
  static constexpr uint32_t kUmmaK = umma_k(kIn);
  static constexpr uint32_t kUmmaPerStage = kBlockKElems / kUmmaK;  // 4
  static constexpr uint32_t kTileM = kCtaRows * kCtaGroup * kMSub;  // rows of one cluster tile
  static constexpr uint32_t kBRows = BN / kCtaGroup;                // B rows this CTA loads
  // A stage holds kKChunks consecutive 128-byte spans of K ("k-blocks"). With more than one, each
  // operand slab of the stage is fetched by ONE 3-D TMA box {128 bytes, rows, kKChunks}, which lands
  // as [chunk][row][128 bytes]: an issuing lane spends 150 - 400 cycles per box whatever its size
  // (1024^3 on 128 x 256 tiles with one lane issuing: 9.9 us with one box per slab and k-block,
  // 12.7 / 20.3 / 26.2 us with the same bytes cut into 2 / 4 / 8 boxes), so narrow tiles, whose
  // k-block of MMAs is short, want few and large boxes.
  static constexpr uint32_t kChunkABytes = kCtaRows * kBlockKBytes;  // one 128-row slab of A, one k-block
  static constexpr uint32_t kChunkBBytes = kBRows * kBlockKBytes;
  static constexpr uint32_t kASubBytes = kChunkABytes * kKChunks;    // one slab of A, one stage
  static constexpr uint32_t kABytes = kMSub * kASubBytes;
  static constexpr uint32_t kBBytes = kChunkBBytes * kKChunks;
  static constexpr uint32_t kStageBytes = kABytes + kBBytes;
  static constexpr uint32_t kAccCols = kMSub * BN * (kKChunks == 2 ? 2 : 1);   // TMEM columns of one tile
  // Block-scaled operands: every stage also carries the scale atoms of its A slabs and of the
  // rows of B under the tile (512 bytes each), and TMEM holds one 4-column copy of each behind
  // the accumulators, rewritten for every k-block (tcgen05.cp and tcgen05.mma run in issue order).
  static constexpr bool kMx = is_block_scaled(kIn);
  static constexpr uint32_t kSfbAtoms = kMx ? mx_sfb_atoms(BN) : 0u;
  static constexpr uint32_t kSfAtoms = kMx ? (kMSub + kSfbAtoms) : 0u;
  static constexpr uint32_t kSfStageBytes = kSfAtoms * kSfAtomBytes;
  static constexpr uint32_t kSfCols = 4u * kSfAtoms;
  // One set of scale columns per MMA-issuing lane (one lane per sub-tile: each copies what its
  // own MMAs read). (A second set for alternate k-blocks, so that the next k-block's copy need
  // not wait for the MMAs still reading this one's, was measured: no gain.)
  static constexpr uint32_t kSfCopies = kMSub;
  static constexpr uint32_t kAccBufs = (2 * kAccCols + kSfCopies * kSfCols <= 512) ? 2 : 1;
  static constexpr uint32_t kSfCol0 = kAccBufs * kAccCols;          // first scale column
  static constexpr uint32_t kTmemUsed = kAccBufs * kAccCols + kSfCopies * kSfCols;
  // tcgen05.alloc takes powers of two (32..512): round the request up
  static constexpr uint32_t kTmemCols = kTmemUsed <= 32 ? 32 : kTmemUsed <= 64 ? 64 : kTmemUsed <= 128 ? 128
                                        : kTmemUsed <= 256 ? 256 : 512;
  static constexpr uint32_t kStageBufs = staging_bufs(kMSub, output_bytes(kOut), kFusedEpi);  // per epilogue warp
  static constexpr uint32_t kRowBytes = staging_row_bytes(kMSub, output_bytes(kOut), kFusedEpi);  // 128 or 64
  static constexpr uint32_t kBufBytes = staging_buf_bytes(kMSub, output_bytes(kOut), kFusedEpi);
  static constexpr uint32_t kChunkCols = kRowBytes / output_bytes(kOut);  // columns per store box
  // A width that is not a whole number of store boxes ends with one box moved left so that it
  // finishes at the tile's edge; the columns it shares with its neighbour are written twice
  // with the same values.
  static constexpr uint32_t kChunks = (BN + kChunkCols - 1) / kChunkCols;
  static constexpr bool kOverlapLastChunk = (BN % kChunkCols) != 0;
  static constexpr uint32_t kSmemBytes =
      smem_plan(kCtaGroup, kMSub, BN, kStages, output_bytes(kOut), kSfStageBytes, kFusedEpi, kKChunks).total_bytes;
  static_assert(kKChunks == 1 || (kKChunks == 2 && kCtaGroup == 1 && kMSub == 1 && !is_block_scaled(kIn) && !kFusedEpi),
                "two k-blocks per stage: single-CTA kernels with one sub-tile, plain epilogue");
  static_assert(!kMx || BN % 64 == 0, "block-scaled tiles: B's scales must start an even number of TMEM columns into an atom");
  static_assert(kMSub == 1 || kMSub == 2, "one or two accumulator sub-tiles per CTA");
  static_assert(umma_shape_ok(128 * kCtaGroup, BN), "illegal tcgen05.mma shape");
  static_assert(kTmemUsed <= 512, "accumulators exceed the 512 TMEM columns");
  static_assert(BN >= kChunkCols && BN % 16 == 0, "tile width: at least one store box, multiple of 16");
  static_assert((kBBytes % 1024) == 0, "swizzle atoms must stay 1024-byte aligned");
  static_assert(kSmemBytes <= kMaxDynSmem, "shared-memory plan exceeds 227 KB");
  static_assert((2 * kStages + 4) * 8 + 8 <= kBarrierRegionBytes, "barrier region too small");
};

// The kernel body; the __global__ entries below differ only in their parameter lists (the
// block-scaled one carries two more tensor maps, for the scales of A and B).
template <int kCtaGroup, int kMSub, int BN, int kStages, int kIn, int kOut, bool kFused, bool kGrouped,
          int kDests, int kKChunks = 1>
__device__ __forceinline__ void gemm_tn_body(const CUtensorMap& tm_a, const CUtensorMap& tm_b,
                                             const CStoreMaps<kDests>& tm_c, const GemmParams& p,
                                             const CUtensorMap* tm_sfa, const CUtensorMap* tm_sfb) {
  using T = GemmTraits<kCtaGroup, kMSub, BN, kStages, kIn, kOut, kFused, kKChunks>;
  constexpr bool kPair = (kCtaGroup == 2);
  constexpr bool kMx = T::kMx;
  static_assert(kKChunks == 1 || !kGrouped, "multi-chunk stages: plain launches");
  // stages of the K loop: kKChunks k-blocks each (the last may be partly past K: zero-filled, not multiplied)
  const uint32_t k_steps = (p.k_blocks + (uint32_t)kKChunks - 1u) / (uint32_t)kKChunks;
  constexpr int kKind = (kIn == kE4M3) ? 1 : 0;
  static_assert(!kMx || (!kFused && !kGrouped && kDests == 1 && kOut == kOutBF16),
                "block-scaled operands: plain bf16 epilogue only");
  constexpr uint32_t kEpiWarps = T::kEpiWarps;
  // A stage is fetched by one TMA load per A slab and one for B, each issued by its own lane of
  // the producer warp. What bounds a producer is not bytes but rounds: one lane's {wait for the
  // slot, announce the bytes, issue} takes about 390 cycles and a further issue 150 - 200,
  // whatever the box holds (8 to 32 KB measured alike), so a lane that issues a stage's two or
  // three loads alone delivers a stage per 550 - 640 cycles -- slower than the MMAs of every
  // tile narrower than 256 x 256 per pair. Lanes overlap: two lanes of one warp retire a load per
  // 231 cycles, four per 148 (separate warps: 199 and 100); one SM takes in 120 bytes per clock
  // when few SMs load and about 84 when 128 do.
  constexpr uint32_t kLoadLanes = (uint32_t)kMSub + 1u;
  constexpr uint32_t kIssuers = T::kIssuers;   // MMA-issuing threads: one per accumulator (sub-tile, or k-block parity)
  // The fused epilogue may read C itself as the residual, so no column may be produced twice.
  static_assert(!(kFused && T::kOverlapLastChunk), "fused epilogue needs whole store boxes");
  static_assert(!(kFused && kGrouped), "the grouped kernel has the plain epilogue only");
  static_assert(kOut != kOutE4M3 || kFused, "e4m3 output goes through the fused epilogue (scale, amax)");

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t ring = smem_base;
  const uint32_t staging = ring + kStages * T::kStageBytes;
  const uint32_t sf_ring = staging + kEpiWarps * T::kStageBufs * T::kBufBytes;  // [kStages] scale atoms
  const uint32_t bars = sf_ring + kStages * T::kSfStageBytes;
  const uint32_t full_bar = bars;                      // [kStages]
  const uint32_t empty_bar = bars + 8u * kStages;      // [kStages]
  const uint32_t tfull_bar = bars + 16u * kStages;     // [2]
  const uint32_t tempty_bar = tfull_bar + 16u;         // [2]
  const uint32_t tmem_slot = tempty_bar + 16u;         // u32
  const uint32_t abort_slot = tmem_slot + 4u;          // u32
  // grouped launch: prefix sums over the groups, [n_groups + 1] each, behind the barrier region
  uint32_t* const grp_row_begin = reinterpret_cast<uint32_t*>(
      smem_raw + (bars + kBarrierRegionBytes - ptx::smem_u32(smem_raw)));
  uint32_t* const grp_tile_begin = grp_row_begin + (kMaxGroups + 1u);
  uint8_t* const smem_generic = smem_raw + (smem_base - ptx::smem_u32(smem_raw));
  volatile uint32_t* const tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(
      smem_generic + (tmem_slot - smem_base));
  volatile uint32_t* const abort_ptr = reinterpret_cast<volatile uint32_t*>(
      smem_generic + (abort_slot - smem_base));

  const uint32_t warp_idx = threadIdx.x >> 5;
  const uint32_t lane = threadIdx.x & 31u;
  const uint32_t cta_rank = kPair ? ptx::cluster_ctarank() : 0u;
  const uint32_t peer_rank = cta_rank ^ 1u;
  const uint32_t cluster_id = blockIdx.x / kCtaGroup;
  const uint32_t num_clusters = gridDim.x / kCtaGroup;

  WaitCtx w;
  w.abort_flag = abort_ptr;
  w.peer_abort_addr = kPair ? ptx::mapa(abort_slot, peer_rank) : 0u;
  w.status = p.status;
  w.limit_ns = p.wait_limit_ns;
  w.has_peer = kPair;

  // ---------------------------------------------------------------- prologue
  if (threadIdx.x == 0) {
    PATINA_TRACE_AT(0);
    ptx::prefetch_tensormap(&tm_a);
    ptx::prefetch_tensormap(&tm_b);
    for (uint32_t d = 0; d < (uint32_t)kDests && d < p.n_dests; ++d) ptx::prefetch_tensormap(&tm_c.map[d]);
    if constexpr (kMx) {
      ptx::prefetch_tensormap(tm_sfa);
      ptx::prefetch_tensormap(tm_sfb);
    }
    for (uint32_t s = 0; s < (uint32_t)kStages; ++s) {
      ptx::mbar_init(full_bar + 8u * s, 1);
      ptx::mbar_init(empty_bar + 8u * s, kIssuers);
    }
    for (uint32_t b = 0; b < 2; ++b) {
      ptx::mbar_init(tfull_bar + 8u * b, kIssuers);
      ptx::mbar_init(tempty_bar + 8u * b, kEpiWarps * kCtaGroup);
    }
    *abort_ptr = 0u;
    ptx::fence_mbar_init();
  }
  // Single-CTA kernels: the producer lanes issue the first pass through
  // the ring right here, before TMEM allocation and the set-up barrier, so that those hide
  // behind the first loads' latency. Every stage is free, so no wait is needed. (A pair's loads
  // complete on the leader's barriers, which the partner may only use after the cluster-wide
  // barrier below; a grouped launch needs its tables first.)
  uint32_t pre_kb = 0;
  if constexpr (!kPair && !kGrouped && !kMx) {
    if (warp_idx == 0) {
      __syncwarp();  // the barriers thread 0 has just initialised, seen by the other issuing lanes
      if (lane < kLoadLanes && cluster_id < p.num_tiles) {
        ptx::fence_proxy_async_smem();
        const TileCoord c0 = tile_coord(cluster_id, p.tiles_m, p.tiles_n, p.group_m);
        const bool is_b = (lane == (uint32_t)kMSub);
        const CUtensorMap* const tm = is_b ? &tm_b : &tm_a;
        const int32_t row = is_b ? (int32_t)(c0.n * BN) : (int32_t)(c0.m * T::kTileM + lane * kCtaRows);
        const uint32_t dst_off = is_b ? T::kABytes : lane * T::kASubBytes;
        const uint32_t n_pre = k_steps < (uint32_t)kStages ? k_steps : (uint32_t)kStages;
        for (uint32_t kb = 0; kb < n_pre; ++kb) {
          const uint32_t dst = ring + kb * T::kStageBytes + dst_off;
          if (lane == 0) ptx::mbar_arrive_expect_tx(full_bar + 8u * kb, T::kStageBytes);
          if constexpr (kKChunks == 1)
            ptx::tma_load_2d(dst, tm, full_bar + 8u * kb, (int32_t)(kb * T::kBlockKElems), row);
          else
            ptx::tma_load_3d(dst, tm, full_bar + 8u * kb, 0, row, (int32_t)(kb * kKChunks));
        }
        pre_kb = n_pre;
      }
    }
  }
  if constexpr (kGrouped) {
    // Every CTA derives the same tables from the device-resident group sizes: first row and
    // first tile of every group (a group's tiles: its row blocks x all column blocks).
    for (uint32_t g = threadIdx.x; g < p.n_groups; g += blockDim.x) {
      const int32_t r = __ldg(p.group_rows + g);
      grp_row_begin[g + 1u] = r > 0 ? (uint32_t)r : 0u;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      uint32_t row = 0, tile = 0;
      grp_row_begin[0] = 0u;
      grp_tile_begin[0] = 0u;
      for (uint32_t g = 0; g < p.n_groups; ++g) {
        uint32_t r = grp_row_begin[g + 1u];
        if (r > p.M - row) r = p.M - row;  // never past the end of A and C
        row += r;
        tile += ((r + T::kTileM - 1u) / T::kTileM) * p.tiles_n;
        grp_row_begin[g + 1u] = row;
        grp_tile_begin[g + 1u] = tile;
      }
    }
  }
  if (warp_idx == 1) {
    ptx::tmem_alloc<kCtaGroup>(tmem_slot, T::kTmemCols);
    ptx::tmem_relinquish<kCtaGroup>();
  }
  ptx::tc_fence_before_sync();
  if constexpr (kPair) {
    ptx::cluster_arrive();
    ptx::cluster_wait();
  } else {
    __syncthreads();
  }
  ptx::tc_fence_after_sync();
  if (threadIdx.x == 0) PATINA_TRACE_AT(1);
  const uint32_t tmem_base = *tmem_slot_ptr;
  const uint32_t num_tiles = kGrouped ? grp_tile_begin[p.n_groups] : p.num_tiles;
  // Where tile t lies. Plain launch: one problem. Grouped launch: the group is found by moving
  // a cursor forward (tile indices only grow), rows are offset by the group's first row and
  // the rows of B by the group's block of N rows.
  struct TileSpot {
    uint32_t m, n;        // block coordinates inside the (group's) problem
    uint32_t row_base;    // first row of the problem in A and C
    uint32_t row_end;     // one past its last row
    uint32_t b_row_base;  // first row of the problem in B
    uint32_t sub_mask;    // accumulator sub-tiles of the tile that this scheduler index covers
  };
  auto locate = [&](uint32_t t, uint32_t& g) -> TileSpot {
    TileSpot sp;
    if constexpr (kGrouped) {
      while (g + 1u < p.n_groups && t >= grp_tile_begin[g + 1u]) ++g;
      const uint32_t rows = grp_row_begin[g + 1u] - grp_row_begin[g];
      const TileCoord c = tile_coord(t - grp_tile_begin[g], (rows + T::kTileM - 1u) / T::kTileM,
                                     p.tiles_n, p.group_m);
      sp.m = c.m;
      sp.n = c.n;
      sp.row_base = grp_row_begin[g];
      sp.row_end = grp_row_begin[g + 1u];
      sp.b_row_base = g * p.N;
      // the last row block of a group often needs only the first of its two 128-row (256 per
      // pair) sub-tiles: the second is then neither loaded nor multiplied
      sp.sub_mask = (kMSub == 2 && sp.row_base + c.m * T::kTileM + kCtaRows * kCtaGroup < sp.row_end) ? 3u : 1u;
    } else {
      sp.sub_mask = (1u << kMSub) - 1u;
      if constexpr (kMSub == 2) {
        if (t >= p.split_from) {   // a half tile of the last wave
          const uint32_t v = t - p.split_from;
          t = p.split_from + (v >> 1);
          sp.sub_mask = 1u << (v & 1u);
        }
      }
      const TileCoord c = tile_coord(t, p.tiles_m, p.tiles_n, p.group_m);
      sp.m = c.m;
      sp.n = c.n;
      sp.row_base = 0u;
      sp.row_end = p.M;
      sp.b_row_base = 0u;
    }
    return sp;
  };
  // ------------------------------------------------------------ TMA producer
  if (warp_idx == 0) {
    if (lane < kLoadLanes) {
      // (pre_kb k-blocks of the first tile are already in flight: see the prologue)
      uint32_t s = pre_kb == (uint32_t)kStages ? 0u : pre_kb, ph = pre_kb == (uint32_t)kStages ? 1u : 0u;
      uint32_t kb_first = pre_kb;
      const uint32_t leader_full = kPair ? ptx::mapa(full_bar, 0) : full_bar;
      const bool is_b = (lane == (uint32_t)kMSub);
      const CUtensorMap* const tm = is_b ? &tm_b : &tm_a;
      const uint32_t dst_off = is_b ? T::kABytes : lane * T::kASubBytes;
#ifdef PATINA_TRACE
      const uint32_t hint = is_b ? p.l2_hint_b : p.l2_hint_a;
      const uint64_t policy = hint == 1 ? ptx::l2_policy_evict_first() : ptx::l2_policy_evict_last();
#endif
      uint32_t grp = 0;
      for (uint32_t t = cluster_id; t < num_tiles; t += num_clusters) {
        const TileSpot c = locate(t, grp);
        // Sub-tile s of this CTA covers rows a_row + s * (128 * kCtaGroup). In a grouped launch
        // the last row block of a group also loads rows of the next group (or zeros past the
        // end): they only feed accumulator rows that are never stored.
        const int32_t row = is_b ? (int32_t)(c.b_row_base + c.n * BN + cta_rank * T::kBRows)
                                 : (int32_t)(c.row_base + c.m * T::kTileM + cta_rank * kCtaRows +
                                             lane * (kCtaRows * kCtaGroup));
        const bool live = is_b || ((c.sub_mask >> lane) & 1u) != 0u;
        // bytes this CTA loads per stage
        const uint32_t stage_tx = (uint32_t)__popc(c.sub_mask) * T::kASubBytes + T::kBBytes + T::kSfStageBytes;
        // (block scales of a stage are loaded by the scale-producer warp, onto the same barrier)
        bool ok = true;
        for (uint32_t kb = kb_first; kb < k_steps; ++kb) {
          ok = bounded_wait<kPair>(empty_bar + 8u * s, ph ^ 1u, w, kTimeoutProducerEmpty, t);
          if (!ok) break;
          if (lane == 0 && t == cluster_id) PATINA_TRACE_KB(48u, kb);
          const uint32_t dst = ring + s * T::kStageBytes + dst_off;
          const int32_t k0 = (int32_t)(kb * T::kBlockKElems);
          // One arrival per stage (the leader's lane 0) announces the bytes of all lanes and both
          // CTAs; a load that lands before it only drives the pending byte count negative.
          if (lane == 0 && cta_rank == 0) ptx::mbar_arrive_expect_tx(full_bar + 8u * s, (uint32_t)kCtaGroup * stage_tx);
          if (live) {
            if constexpr (kPair) {
#ifdef PATINA_TRACE
              if (hint) ptx::tma_load_2d_pair_hint(dst, tm, leader_full + 8u * s, k0, row, policy);
              else
#endif
              ptx::tma_load_2d_pair(dst, tm, leader_full + 8u * s, k0, row);
            } else if constexpr (kKChunks > 1) {
              ptx::tma_load_3d(dst, tm, full_bar + 8u * s, 0, row, (int32_t)(kb * kKChunks));
            } else {
              ptx::tma_load_2d(dst, tm, full_bar + 8u * s, k0, row);
            }
          }
          if (++s == (uint32_t)kStages) { s = 0; ph ^= 1u; }
        }
        kb_first = 0;
        if (!ok) break;
      }
    }
  }
  // -------------------------------------------------------------- MMA issuer
  // One warp (its lane 0) of the leader CTA per accumulator sub-tile: a thread issues one tcgen05 instruction
  // (mma, cp, commit) per 71 - 85 cycles, however short the instruction's work -- measured back to
  // back: 128 x 64 x 16 and 128 x 128 x 16 MMAs both retire one per 85 cycles from one thread, one
  // per 48 and 64 from two -- so a k-block of a two-sub-tile kernel (8 MMAs, 2 commits, a wait, and
  // 4 scale copies when block-scaled) is 11 to 16 issue slots against 768 - 1024 cycles of
  // tensor-pipe work. The sub-tiles' MMAs are independent, so each issuer multiplies its own
  // sub-tile (every accumulator sees the same MMAs in the same order whoever issues them), copies
  // the scales it needs into its own TMEM columns (tcgen05.cp is ordered before the MMAs of the
  // same thread only) and commits for itself: the `empty` and `tmem full` barriers count
  // kIssuers arrivals. Warp 1 takes sub-tile 0, the last warp of the block sub-tile 1.
  else if (warp_idx == 1 || (kIssuers == 2 && warp_idx == T::kSecondIssuerWarp)) {
    if (lane == 0 && cta_rank == 0) {
      const uint32_t my = (warp_idx == 1) ? 0u : 1u;  // the accumulator this thread multiplies into: sub-tile
                                                      // `my`, or (kDualAcc) the stages' k-block `my`
      const uint32_t idesc_v = idesc(kIn, kCtaRows * kCtaGroup, BN);
      uint32_t s = 0, ph = 0, it = 0, grp = 0;
      bool ok = true;
      for (uint32_t t = cluster_id; t < num_tiles && ok; t += num_clusters, ++it) {
        const TileSpot c = locate(t, grp);
        const bool live = T::kDualAcc || ((c.sub_mask >> my) & 1u) != 0u;
        const uint32_t buf = it % T::kAccBufs, acc_ph = (it / T::kAccBufs) & 1u;
        // block scales in TMEM, one set of columns per issuer: A's slabs first, then B's
        // atoms; the tile's first row of B may lie 64 rows into its first atom, i.e. 2 columns in
        // (widths are multiples of 64)
        const uint32_t tsfa0 = tmem_base + T::kSfCol0 + my * T::kSfCols;
        const uint32_t tsfb0 = tsfa0 + 4u * (uint32_t)kMSub + ((c.n * BN) % kSfAtomRows) / 32u;
        ok = bounded_wait<kPair>(tempty_bar + 8u * buf, acc_ph ^ 1u, w, kTimeoutMmaTmemEmpty, t);
        if (!ok) break;
        ptx::tc_fence_after_sync();
        const uint32_t tmem_d = tmem_base + buf * T::kAccCols + my * BN;
        for (uint32_t kb = 0; kb < k_steps; ++kb) {
          ok = bounded_wait<kPair>(full_bar + 8u * s, ph, w, kTimeoutMmaFull, t);
          if (!ok) break;
          ptx::tc_fence_after_sync();
          if (my == 0 && it == 0 && kb == 0) PATINA_TRACE_AT(2);
          if (my == 0 && it == 0) PATINA_TRACE_KB(32u, kb);
          const uint32_t sa = ring + s * T::kStageBytes;
          const uint64_t db = smem_desc_sw128_kmajor(sa + T::kABytes);
          if constexpr (kMx) {
            // this k-block's scales: shared memory -> TMEM, 32 lines of 16 bytes per atom (8-line
            // groups 128 bytes apart, no swizzle): this lane's slab of A and all atoms of B
            const uint32_t sfs = sf_ring + s * T::kSfStageBytes;
#pragma unroll
            for (uint32_t j = 0; j < T::kSfAtoms; ++j)
              if (live && (j == my || j >= (uint32_t)kMSub))
                ptx::tmem_cp_32x128b_warpx4<kCtaGroup>(tsfa0 + 4u * j,
                                                       smem_desc(sfs + j * kSfAtomBytes, 0, 128, kSwizzleNone));
          }
#pragma unroll
          for (uint32_t ch = 0; ch < (uint32_t)kKChunks; ++ch) {
            if (T::kDualAcc && ch != my) continue;      // the other issuer's k-block
            // (a stage's k-block past K holds TMA's zero fill: not multiplied)
            if (kKChunks > 1 && kb * (uint32_t)kKChunks + ch >= p.k_blocks) break;
            const uint64_t db_c = db + (uint64_t)((ch * T::kChunkBBytes) >> 4);
            const uint64_t da = smem_desc_sw128_kmajor(sa + (T::kDualAcc ? 0u : my) * T::kASubBytes + ch * T::kChunkABytes);
#pragma unroll
            for (uint32_t k = 0; k < T::kUmmaPerStage; ++k) {
              const uint32_t adv = k_advance_units_sw128(k * T::kUmmaK, kIn);
              if (live) {
                if constexpr (kMx) {
                  // the k-th 32-element block of this stage uses byte k of each scale column
                  ptx::umma_mx<kCtaGroup>(tmem_d, da + adv, db_c + adv, idesc_mx(kCtaRows * kCtaGroup, BN, k, k),
                                          (tsfa0 + 4u * my) | (k << 30), tsfb0 | (k << 30), (kb | k) != 0u);
                } else {
                  // (an accumulator's first MMA overwrites it: k-block 0, or 1 for the second of two)
                  ptx::umma<kCtaGroup, kKind>(tmem_d, da + adv, db_c + adv, idesc_v,
                                              (T::kDualAcc ? (kb | k) : (kb | ch | k)) != 0u);
                }
              }
            }
          }
          // (a lane without MMAs in this stage arrives at once)
          if constexpr (kPair) ptx::umma_commit_pair(empty_bar + 8u * s);   // both CTAs' slots
          else ptx::umma_commit<kCtaGroup>(empty_bar + 8u * s);
          if (++s == (uint32_t)kStages) { s = 0; ph ^= 1u; }
        }
        if (!ok) break;
        if constexpr (kPair) ptx::umma_commit_pair(tfull_bar + 8u * buf);
        else ptx::umma_commit<kCtaGroup>(tfull_bar + 8u * buf);
        if (my == 0) PATINA_TRACE_AT(3);  // (overwritten per tile: the last tile's stamp stays)
      }
      // Every MMA must have retired before shared memory or TMEM is released:
      // wait for the last accumulator's completion here as well.
      if (ok && it > 0) {
        const uint32_t last = it - 1;
        bounded_wait<kPair>(tfull_bar + 8u * (last % T::kAccBufs), (last / T::kAccBufs) & 1u, w,
                            kTimeoutMmaDrain, it);
      }
    }
  }
  // ---------------------------------------------------- scale producer (block-scaled kernels)
  // One more warp behind the epilogue warps: it walks the same tiles and stages as the TMA
  // producer and issues the stage's scale atoms (512 bytes each: the atom row of each A slab,
  // and the atoms under the tile's rows of B -- all of them in both CTAs of a pair, since every
  // CTA's accumulator has all BN columns) onto the same `full` barrier, whose expected byte
  // count, set by the TMA producer, includes them. Issuing a TMA load costs the issuing lane
  // over a hundred cycles, and a stage has up to four scale atoms: they are kept off the operand
  // producer's lane (measured at 8192^3: 457 us against 463 us with one lane issuing everything).
  // Atom indices are clamped into the buffers; an atom past the edge only scales rows or columns
  // that are never stored.
  else if (kMx && warp_idx == 2u + kEpiWarps) {
    if constexpr (kMx) {
      if (lane < T::kSfAtoms) {   // one lane per scale atom of a stage (lanes overlap their issue latency)
        uint32_t s = 0, ph = 0, grp = 0;
        const uint32_t leader_full = kPair ? ptx::mapa(full_bar, 0) : full_bar;
        const bool is_b = lane >= (uint32_t)kMSub;
        const CUtensorMap* const tm = is_b ? tm_sfb : tm_sfa;
        for (uint32_t t = cluster_id; t < num_tiles; t += num_clusters) {
          const TileSpot c = locate(t, grp);
          uint32_t blk, last;
          if (is_b) {
            blk = (c.n * BN) / kSfAtomRows + (lane - (uint32_t)kMSub);
            last = p.sf_n_blocks - 1u;
          } else {
            blk = (c.row_base + c.m * T::kTileM + cta_rank * kCtaRows + lane * kCtaRows * kCtaGroup) / kSfAtomRows;
            last = p.sf_m_blocks - 1u;
          }
          const uint32_t atom0 = (blk < last ? blk : last) * p.sf_k_atoms;
          bool ok = true;
          for (uint32_t kb = 0; kb < p.k_blocks; ++kb) {
            ok = bounded_wait<kPair>(empty_bar + 8u * s, ph ^ 1u, w, kTimeoutProducerEmpty, t);
            if (!ok) break;
            const uint32_t dst = sf_ring + s * T::kSfStageBytes + lane * kSfAtomBytes;
            if constexpr (kPair) ptx::tma_load_2d_pair(dst, tm, leader_full + 8u * s, 0, (int32_t)(atom0 + kb));
            else ptx::tma_load_2d(dst, tm, full_bar + 8u * s, 0, (int32_t)(atom0 + kb));
            if (++s == (uint32_t)kStages) { s = 0; ph ^= 1u; }
          }
          if (!ok) break;
        }
      }
    }
  }
  // ---------------------------------------------------------------- epilogue
  else {
    const uint32_t q = warp_idx & 3u;          // TMEM lane quarter this warp may touch
    const uint32_t e = warp_idx - 2u;          // epilogue warp index
    const uint32_t ms = e >> 2;                // accumulator sub-tile this warp drains
    const uint32_t stg0 = staging + e * (T::kStageBufs * T::kBufBytes);
    const uint32_t leader_tempty = kPair ? ptx::mapa(tempty_bar, 0) : tempty_bar;
    // Swizzled position of 16-byte piece j of this lane's row, matching the store's tensor map:
    // 128-byte rows: j ^ (row & 7); 64-byte rows: j ^ ((row >> 1) & 3).
    const uint32_t row_sw = (T::kRowBytes == 128u) ? (lane & 7u) : ((lane >> 1) & 3u);
    uint32_t it = 0, sbuf = 0;
    bool ok = true;
    uint32_t grp = 0;
    for (uint32_t t = cluster_id; t < num_tiles && ok; t += num_clusters, ++it) {
      const TileSpot c = locate(t, grp);
      const uint32_t buf = it % T::kAccBufs, acc_ph = (it / T::kAccBufs) & 1u;
      ok = bounded_wait<kPair>(tfull_bar + 8u * buf, acc_ph, w, kTimeoutEpilogueTmemFull, t);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      ptx::tc_fence_after_sync();
      if (warp_idx == 2 && lane == 0) PATINA_TRACE_AT(4);
      const uint32_t row0 = c.row_base + c.m * T::kTileM + ms * (kCtaRows * kCtaGroup) +
                            cta_rank * kCtaRows + q * kStoreBoxRows;
      // A grouped launch must not write past its group: a box beyond the group's last row is
      // dropped, one that straddles it is written row by row from the registers.
      float tile_alpha = p.alpha;
      if constexpr (kGrouped) {
        if (p.group_alpha != nullptr) tile_alpha *= __ldg(p.group_alpha + grp);
      }
      const bool live_sub = ((c.sub_mask >> ms) & 1u) != 0u;   // else: another index's half, or past the group
      const bool box_outside = !live_sub || row0 >= c.row_end;
      const bool box_straddles = kGrouped && !box_outside && row0 + kStoreBoxRows > c.row_end;
      const uint32_t col0 = c.n * BN;
      const uint32_t taddr = tmem_base + tmem_lane_offset(q) + buf * T::kAccCols + ms * BN;
      constexpr uint32_t kFp32PerChunk = T::kChunkCols;            // accumulator words per chunk
      constexpr uint32_t kPieces = T::kRowBytes / 16u;             // 16-byte pieces per staged row
      float tile_amax = 0.0f;   // e4m3 output: largest magnitude this thread produced in the tile
      auto chunk_col = [](uint32_t ch) -> uint32_t {
        return (T::kOverlapLastChunk && ch == T::kChunks - 1) ? (uint32_t)BN - T::kChunkCols
                                                               : ch * T::kChunkCols;
      };
      auto request = [&](uint32_t ch, uint32_t* v) {
        const uint32_t c0 = chunk_col(ch);
#pragma unroll
        for (uint32_t h = 0; h < kFp32PerChunk; h += 32u) ptx::tmem_ld_32x32b_x32(taddr + c0 + h, &v[h]);
      };
      auto finish = [&](uint32_t ch, uint32_t* v) {
        const uint32_t ch_col = chunk_col(ch);
        if (ch == T::kChunks - 1) {
          // Accumulator fully read: hand the TMEM buffer back to the MMA issuer.
          ptx::tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) {
            if constexpr (kPair) ptx::mbar_arrive_cluster(leader_tempty + 8u * buf);
            else ptx::mbar_arrive(tempty_bar + 8u * buf);
          }
        }
        if constexpr (kFused) {
          // v := act(alpha * v + bias[col] + beta * R[row, col]) in fp32; every lane of the warp
          // reads the same bias words (one broadcast transaction per load), and its own row of R.
          const uint32_t cc = col0 + ch_col;
          const uint32_t r = row0 + lane;
          float add[kFp32PerChunk];
          if (p.bias == nullptr) {
#pragma unroll
            for (uint32_t i = 0; i < kFp32PerChunk; ++i) add[i] = 0.0f;
          } else if (cc + kFp32PerChunk <= p.N && (reinterpret_cast<uintptr_t>(p.bias) & 15u) == 0) {
#pragma unroll
            for (uint32_t g = 0; g < kFp32PerChunk / 4u; ++g) {
              const float4 b4 = __ldg(reinterpret_cast<const float4*>(p.bias + cc) + g);
              add[4u * g] = b4.x;
              add[4u * g + 1u] = b4.y;
              add[4u * g + 2u] = b4.z;
              add[4u * g + 3u] = b4.w;
            }
          } else {
#pragma unroll
            for (uint32_t i = 0; i < kFp32PerChunk; ++i)
              add[i] = (cc + i < p.N) ? __ldg(p.bias + cc + i) : 0.0f;
          }
          if (p.residual != nullptr && r < p.M) {
            const __nv_bfloat16* rr = p.residual + (size_t)r * p.ldr + cc;
#pragma unroll
            for (uint32_t g = 0; g < kFp32PerChunk / 8u; ++g) {
              if (cc + 8u * g + 8u <= p.N) {
                const uint4 raw = __ldg(reinterpret_cast<const uint4*>(rr + 8u * g));
                const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
                for (uint32_t e2 = 0; e2 < 4; ++e2) {
                  const float2 f = __bfloat1622float2(h2[e2]);
                  add[8u * g + 2u * e2] += p.beta * f.x;
                  add[8u * g + 2u * e2 + 1u] += p.beta * f.y;
                }
              } else {
#pragma unroll
                for (uint32_t e1 = 0; e1 < 8; ++e1)
                  if (cc + 8u * g + e1 < p.N) add[8u * g + e1] += p.beta * __bfloat162float(rr[8u * g + e1]);
              }
            }
          }
          // one branch per chunk, not per element: the activation is the same for the launch
          switch (p.activation) {
            case kActRelu:
#pragma unroll
              for (uint32_t i = 0; i < kFp32PerChunk; ++i)
                v[i] = __float_as_uint(apply_activation(__uint_as_float(v[i]) * p.alpha + add[i], kActRelu));
              break;
            case kActGelu:
#pragma unroll
              for (uint32_t i = 0; i < kFp32PerChunk; ++i)
                v[i] = __float_as_uint(apply_activation(__uint_as_float(v[i]) * p.alpha + add[i], kActGelu));
              break;
            case kActSilu:
#pragma unroll
              for (uint32_t i = 0; i < kFp32PerChunk; ++i)
                v[i] = __float_as_uint(apply_activation(__uint_as_float(v[i]) * p.alpha + add[i], kActSilu));
              break;
            default:
#pragma unroll
              for (uint32_t i = 0; i < kFp32PerChunk; ++i)
                v[i] = __float_as_uint(__uint_as_float(v[i]) * p.alpha + add[i]);
              break;
          }
          if constexpr (kOut == kOutE4M3) {
            // rows past M carry act(bias) and must not count; columns past N are exactly zero
            if (r < p.M && live_sub) {
#pragma unroll
              for (uint32_t i = 0; i < kFp32PerChunk; ++i)
                if (cc + i < p.N) tile_amax = fmaxf(tile_amax, fabsf(__uint_as_float(v[i])));
            }
          }
        }
        const float out_scale = (kOut == kOutE4M3) ? p.out_scale : (kFused ? 1.0f : tile_alpha);
        static_assert(!kGrouped || kOut == kOutBF16, "grouped launches write bf16");
        if (box_outside) return;
        {
          const uint32_t cc = col0 + ch_col;
          constexpr uint32_t kOutBytes = output_bytes(kOut);
          const bool ragged_n = cc < p.N && cc + T::kChunkCols > p.N && ((p.N * kOutBytes) & 15u) != 0u;
          if (box_straddles || ragged_n) {
            // Each lane holds one row of the box: lanes whose row exists write their columns
            // themselves, 16 bytes at a time, element by element in the piece that crosses N.
            const uint32_t r = row0 + lane;
            if (r < c.row_end) {
              constexpr uint32_t kPerPiece = 16u / kOutBytes;   // elements per 16-byte piece
              for (uint32_t d = 0; d < p.n_dests; ++d) {
                uint8_t* crow = static_cast<uint8_t*>(p.c_dests[d]) +
                                ((size_t)r * (size_t)p.ldc + cc) * kOutBytes;
#pragma unroll
                for (uint32_t j = 0; j < kPieces; ++j) {
                  uint32_t w[4];
                  if constexpr (kOut == kOutBF16) {
#pragma unroll
                    for (uint32_t e2 = 0; e2 < 4; ++e2) {
                      const __nv_bfloat162 h = __floats2bfloat162_rn(
                          __uint_as_float(v[8 * j + 2 * e2]) * out_scale,
                          __uint_as_float(v[8 * j + 2 * e2 + 1]) * out_scale);
                      w[e2] = (uint32_t)__bfloat16_as_ushort(h.x) | ((uint32_t)__bfloat16_as_ushort(h.y) << 16);
                    }
                  } else if constexpr (kOut == kOutE4M3) {
#pragma unroll
                    for (uint32_t e4 = 0; e4 < 4; ++e4) {
                      const uint32_t i0 = 16 * j + 4 * e4;
                      const uint32_t lo = __nv_cvt_float2_to_fp8x2(
                          make_float2(__uint_as_float(v[i0]) * out_scale, __uint_as_float(v[i0 + 1]) * out_scale),
                          __NV_SATFINITE, __NV_E4M3);
                      const uint32_t hi = __nv_cvt_float2_to_fp8x2(
                          make_float2(__uint_as_float(v[i0 + 2]) * out_scale,
                                      __uint_as_float(v[i0 + 3]) * out_scale),
                          __NV_SATFINITE, __NV_E4M3);
                      w[e4] = lo | (hi << 16);
                    }
                  } else {
#pragma unroll
                    for (uint32_t e = 0; e < 4; ++e)
                      w[e] = __float_as_uint(__uint_as_float(v[4 * j + e]) * out_scale);
                  }
                  const uint32_t c_first = cc + kPerPiece * j;
                  if (c_first + kPerPiece <= p.N) {
                    *reinterpret_cast<uint4*>(crow + 16u * j) = make_uint4(w[0], w[1], w[2], w[3]);
                  } else {
#pragma unroll
                    for (uint32_t e = 0; e < kPerPiece; ++e) {
                      if (c_first + e < p.N) {
                        if constexpr (kOutBytes == 4u) {
                          reinterpret_cast<uint32_t*>(crow + 16u * j)[e] = w[e];
                        } else if constexpr (kOutBytes == 2u) {
                          reinterpret_cast<uint16_t*>(crow + 16u * j)[e] =
                              (uint16_t)(w[e >> 1] >> (16u * (e & 1u)));
                        } else {
                          (crow + 16u * j)[e] = (uint8_t)(w[e >> 2] >> (8u * (e & 3u)));
                        }
                      }
                    }
                  }
                }
              }
            }
            return;
          }
        }
        // The staging buffer about to be rewritten must have been read by its store.
        if (lane == 0) ptx::tma_store_wait_read<T::kStageBufs - 1>();
        __syncwarp();
        const uint32_t row_addr = stg0 + sbuf * T::kBufBytes + lane * T::kRowBytes;
#pragma unroll
        for (uint32_t j = 0; j < kPieces; ++j) {
          uint32_t w0, w1, w2, w3;
          if constexpr (kOut == kOutBF16) {
            auto pack = [&](uint32_t a, uint32_t b) -> uint32_t {
              __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(a) * out_scale,
                                                       __uint_as_float(b) * out_scale);
              return *reinterpret_cast<uint32_t*>(&h);
            };
            w0 = pack(v[8 * j + 0], v[8 * j + 1]);
            w1 = pack(v[8 * j + 2], v[8 * j + 3]);
            w2 = pack(v[8 * j + 4], v[8 * j + 5]);
            w3 = pack(v[8 * j + 6], v[8 * j + 7]);
          } else if constexpr (kOut == kOutE4M3) {
            // sixteen values per 16-byte piece; round to nearest even, saturate to +-448
            auto pack4 = [&](uint32_t i0) -> uint32_t {
              const uint32_t lo = __nv_cvt_float2_to_fp8x2(
                  make_float2(__uint_as_float(v[i0]) * out_scale, __uint_as_float(v[i0 + 1]) * out_scale),
                  __NV_SATFINITE, __NV_E4M3);
              const uint32_t hi = __nv_cvt_float2_to_fp8x2(
                  make_float2(__uint_as_float(v[i0 + 2]) * out_scale, __uint_as_float(v[i0 + 3]) * out_scale),
                  __NV_SATFINITE, __NV_E4M3);
              return lo | (hi << 16);
            };
            w0 = pack4(16 * j + 0);
            w1 = pack4(16 * j + 4);
            w2 = pack4(16 * j + 8);
            w3 = pack4(16 * j + 12);
          } else {
            w0 = __float_as_uint(__uint_as_float(v[4 * j + 0]) * out_scale);
            w1 = __float_as_uint(__uint_as_float(v[4 * j + 1]) * out_scale);
            w2 = __float_as_uint(__uint_as_float(v[4 * j + 2]) * out_scale);
            w3 = __float_as_uint(__uint_as_float(v[4 * j + 3]) * out_scale);
          }
          const uint32_t dst = row_addr + ((j ^ row_sw) << 4);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(w0), "r"(w1),
                       "r"(w2), "r"(w3)
                       : "memory");
        }
        ptx::fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          const uint32_t cc = col0 + ch_col;
          if (row0 < p.M && cc < p.N) {
            if constexpr (kDests == 1) {
              ptx::tma_store_2d(&tm_c.map[0], stg0 + sbuf * T::kBufBytes, (int32_t)cc, (int32_t)row0);
            } else {
              for (uint32_t d = 0; d < p.n_dests; ++d)
                ptx::tma_store_2d(&tm_c.map[d], stg0 + sbuf * T::kBufBytes, (int32_t)cc, (int32_t)row0);
            }
          }
          ptx::tma_store_commit();
        }
        sbuf = (sbuf + 1u) % T::kStageBufs;   // one or two staging buffers per warp
      };
      // (Requesting chunk ch + 1 from TMEM before chunk ch is converted was measured: nothing
      // gained on the plain epilogue, and the fused one lost 10 % to the second register set.)
      uint32_t v[kFp32PerChunk];
#pragma unroll 1
      for (uint32_t ch = 0; ch < T::kChunks; ++ch) {
        request(ch, v);
        if constexpr (T::kDualAcc) {
          // the odd k-blocks' accumulator, BN columns further on (never written when K is one k-block)
          if (p.k_blocks > 1u) {
            uint32_t v2[kFp32PerChunk];
            const uint32_t c0 = chunk_col(ch);
#pragma unroll
            for (uint32_t h = 0; h < kFp32PerChunk; h += 32u) ptx::tmem_ld_32x32b_x32(taddr + (uint32_t)BN + c0 + h, &v2[h]);
            ptx::tmem_ld_wait();
#pragma unroll
            for (uint32_t i = 0; i < kFp32PerChunk; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) + __uint_as_float(v2[i]));
          }
        }
        ptx::tmem_ld_wait();
        finish(ch, v);
      }
      if constexpr (kOut == kOutE4M3) {
        if (p.amax != nullptr) {
          // magnitudes are non-negative floats: their bit patterns order like unsigned integers
          const uint32_t m = __reduce_max_sync(0xffffffffu, __float_as_uint(tile_amax));
          if (lane == 0 && m != 0u) atomicMax(reinterpret_cast<unsigned int*>(p.amax), m);
        }
      }
    }
    // The staging buffers must have been read before the CTA gives its shared memory back; the
    // writes themselves are complete, as every write of a grid, when the grid completes.
    if (warp_idx == 2 && lane == 0) PATINA_TRACE_AT(5);
    if (lane == 0) ptx::tma_store_wait_read<0>();
    if (warp_idx == 2 && lane == 0) PATINA_TRACE_AT(6);
  }

  // ---------------------------------------------------------------- teardown
  __syncwarp();
  if (*abort_ptr) {
    // Give copies and MMAs that are still in flight time to land before the
    // shared memory and TMEM they target are released.
    const uint64_t t0 = ptx::globaltimer_ns();
    while (ptx::globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  __syncwarp();
  ptx::tc_fence_before_sync();
  if constexpr (kPair) {
    ptx::cluster_arrive();
    ptx::cluster_wait();
  } else {
    __syncthreads();
  }
  ptx::tc_fence_after_sync();
  if (warp_idx == 1) ptx::tmem_dealloc<kCtaGroup>(tmem_base, T::kTmemCols);
  if (threadIdx.x == 32) PATINA_TRACE_AT(7);
}

template <int kCtaGroup, int kMSub, int BN, int kStages, int kIn, int kOut, bool kFused = false,
          bool kGrouped = false, int kDests = 1>
__global__ void __launch_bounds__(64 + 128 * kMSub + (kMSub == 2 ? 32 : 0), 1)
gemm_tn_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
               const __grid_constant__ CStoreMaps<kDests> tm_c, const GemmParams p) {
  gemm_tn_body<kCtaGroup, kMSub, BN, kStages, kIn, kOut, kFused, kGrouped, kDests>(tm_a, tm_b, tm_c, p,
                                                                                   nullptr, nullptr);
}

// Single-CTA kernel whose stages hold two k-blocks, each operand slab of a stage fetched by one
// 3-D box (tensor maps of rank 3: {128 bytes of K, rows, K / 128 bytes}), the two k-blocks
// multiplied into two accumulators by two issuing threads; plain epilogue.
template <int kMSub, int BN, int kStages, int kIn, int kOut, int kKChunks>
__global__ void __launch_bounds__(64 + 128 * kMSub + 32, 1)   // + the second MMA-issuing warp
gemm_tn_chunked_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                       const __grid_constant__ CStoreMaps<1> tm_c, const GemmParams p) {
  gemm_tn_body<1, kMSub, BN, kStages, kIn, kOut, false, false, 1, kKChunks>(tm_a, tm_b, tm_c, p, nullptr, nullptr);
}

// Block-scaled operands (e4m3 elements, one E8M0 scale per 32 K elements of a row): the same
// kernel with the scale buffers of A and B as two more tensor maps.
template <int kCtaGroup, int kMSub, int BN, int kStages>
__global__ void __launch_bounds__(64 + 128 * kMSub + 32 + (kMSub == 2 ? 32 : 0), 1)   // + the scale-producer warp
gemm_mx_tn_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                  const __grid_constant__ CStoreMaps<1> tm_c, const __grid_constant__ CUtensorMap tm_sfa,
                  const __grid_constant__ CUtensorMap tm_sfb, const GemmParams p) {
  gemm_tn_body<kCtaGroup, kMSub, BN, kStages, kMXE4M3, kOutBF16, false, false, 1>(tm_a, tm_b, tm_c, p,
                                                                                 &tm_sfa, &tm_sfb);
}

}  // namespace patina

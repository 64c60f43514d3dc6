// patina_gemm_splitk.cuh -- few output tiles, deep K, more than 128 rows: K is cut across the
// CTAs of a thread-block cluster and the partial tiles are summed through distributed shared
// memory, never through global memory.
//
//   C[M,N] = alpha * A[M,K] * B[N,K]^T,   bf16 in, bf16 out
//
// Why: one tcgen05.mma of 128 rows takes about as long for 64 columns as for 256 (measured: a
// 128-byte k-block costs ~525 cycles on a CTA whatever the tile width), so narrower tiles do not
// spread a small problem over more SMs any faster; cutting K does. The large-tile kernel
// (patina_gemm_kernel.cuh) leaves a 1024^3 problem on 32 SMs for 16 k-blocks each; here the same
// 32 tiles run on 128 SMs for 4 k-blocks each. The stream-K kernel (patina_gemm_streamk.cuh)
// covers M <= 128; the reference's kernel is one tile on one SM
// (crates/patina/tests/golden/v2_gemm_pipelined.ptx, grid 1).
//
// One cluster of kSplit CTAs per 128 x 256 output tile. CTA r of the cluster:
//   1. runs the usual TMA -> ring -> tcgen05.mma mainloop (same 1 + 1 + 4 warp roles as the
//      reference's generated kernel, v2_gemm_pipelined.ptx:89-94) over ITS k-blocks only, into
//      one 256-column accumulator in TMEM;
//   2. after a cluster barrier (every CTA's ring is idle from then on) its epilogue warps copy,
//      for every other CTA o, the 256/kSplit columns that o owns, as fp32, from TMEM through a
//      local staging area into o's shared memory with bulk copies (cp.async.bulk shared::cta ->
//      shared::cluster, completing on o's receive barrier). Plain st.shared::cluster stores were
//      measured first: about 10 bytes per clock per SM, 6.5 us for the 96 KB a CTA of a 4-cluster
//      sends; the copy engine moves the same bytes several times faster;
//   3. waits for its own receive barrier (all parts for its columns have landed), sums them in
//      rank order with its own part from TMEM, so the result does not depend on timing, scales,
//      rounds to bf16 and stores through swizzled staging and TMA like the large-tile kernel.
// A last cluster barrier (arrive after the receive wait, wait before exit) keeps every CTA's
// shared memory alive until the copies that read it are done. Every mbarrier wait is bounded; a
// CTA whose wait ran out still joins the cluster barriers.
#pragma once

#include <cuda_bf16.h>

#include "patina_desc.h"
#include "patina_gemm_kernel.cuh"
#include "patina_ptx.cuh"

namespace patina {

constexpr uint32_t kSplitBN = 256;        // tile width
constexpr uint32_t kSplitStages = 4;      // 4 x (16 KB of A + 32 KB of B) = 192 KB
constexpr uint32_t kSplitStageBytes = kCtaRows * kBlockKBytes + kSplitBN * kBlockKBytes;
constexpr uint32_t kSplitStagingBytes = 4u * 2u * kStoreBoxRows * 64u;   // 4 warps x 2 buffers x 32 rows x 64 B
PATINA_HD constexpr uint32_t splitk_smem_bytes() {
  return 1024u + kSplitStages * kSplitStageBytes + kSplitStagingBytes + kBarrierRegionBytes;
}
// k-blocks [begin, end) of CTA r when k_blocks are cut into `split` nearly equal ranges.
PATINA_HD constexpr uint32_t splitk_kb_begin(uint32_t r, uint32_t k_blocks, uint32_t split) {
  return (uint32_t)(((uint64_t)r * k_blocks) / split);
}

namespace ptx {
__device__ __forceinline__ void st_cluster_v4(uint32_t cluster_addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared::cluster.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(cluster_addr), "r"(a), "r"(b), "r"(c),
               "r"(d)
               : "memory");
}
// Bulk copy from this CTA's shared memory into another CTA's of the cluster; the bytes count on
// an mbarrier of the destination CTA (both destination addresses are shared::cluster addresses).
// Addresses and size are multiples of 16 bytes.
__device__ __forceinline__ void bulk_copy_to_cluster(uint32_t dst_cluster, uint32_t src_cta, uint32_t bytes,
                                                     uint32_t bar_cluster) {
  asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   dst_cluster),
               "r"(src_cta), "r"(bytes), "r"(bar_cluster)
               : "memory");
}
__device__ __forceinline__ uint4 ld_shared_v4(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
}  // namespace ptx

template <int kSplit>
__global__ void __launch_bounds__(192, 1)
gemm_splitk_cluster_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                           const __grid_constant__ CUtensorMap tm_c, const GemmParams p) {
  static_assert(kSplit == 2 || kSplit == 4, "cluster sizes 2 and 4: receive and send areas of 8 would not fit the ring");
  constexpr uint32_t kOwnCols = kSplitBN / kSplit;       // columns of the tile this CTA finishes
  constexpr uint32_t kOwnChunks = kOwnCols / 32u;        // 32-column chunks of them
  constexpr uint32_t kBlockKElems = kBlockKBytes / 2u;   // bf16
  constexpr uint32_t kABytes = kCtaRows * kBlockKBytes;
  // One 32-column chunk of one lane quarter from one sender: [8 pieces of 16 bytes][32 lanes],
  // so that a warp's store or load of one piece is 512 contiguous bytes.
  constexpr uint32_t kChunkBytes = 8u * 32u * 16u;
  constexpr uint32_t kSlotBytes = 4u * kOwnChunks * kChunkBytes;   // one sender's part: 128 rows x kOwnCols fp32
  // ring, once idle: [kSplit - 1 receive slots][kSplit - 1 send slots]
  constexpr uint32_t kRecvBytes = (kSplit - 1u) * kSlotBytes;
  static_assert(2u * kRecvBytes <= kSplitStages * kSplitStageBytes, "receive and send areas must fit in the ring");

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t ring = smem_base;
  const uint32_t staging = ring + kSplitStages * kSplitStageBytes;
  const uint32_t bars = staging + kSplitStagingBytes;
  const uint32_t full_bar = bars;
  const uint32_t empty_bar = bars + 8u * kSplitStages;
  const uint32_t tfull_bar = bars + 16u * kSplitStages;
  const uint32_t recv_bar = tfull_bar + 8u;         // completes when every other CTA's part has landed
  const uint32_t tmem_slot = recv_bar + 8u;
  const uint32_t abort_slot = tmem_slot + 4u;
  uint8_t* const smem_generic = smem_raw + (smem_base - ptx::smem_u32(smem_raw));
  volatile uint32_t* const tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(smem_generic + (tmem_slot - smem_base));
  volatile uint32_t* const abort_ptr = reinterpret_cast<volatile uint32_t*>(smem_generic + (abort_slot - smem_base));

  const uint32_t warp_idx = threadIdx.x >> 5;
  const uint32_t lane = threadIdx.x & 31u;
  const uint32_t rank = ptx::cluster_ctarank();
  const uint32_t tile = blockIdx.x / kSplit;
  const TileCoord tc = tile_coord(tile, p.tiles_m, p.tiles_n, p.group_m);
  const uint32_t kb0 = splitk_kb_begin(rank, p.k_blocks, kSplit);
  const uint32_t kb1 = splitk_kb_begin(rank + 1u, p.k_blocks, kSplit);

  WaitCtx w;
  w.abort_flag = abort_ptr;
  w.peer_abort_addr = 0u;
  w.status = p.status;
  w.limit_ns = p.wait_limit_ns;
  w.has_peer = false;

  // ---------------------------------------------------------------- prologue
  if (threadIdx.x == 0) {
    PATINA_TRACE_AT(0);
    ptx::prefetch_tensormap(&tm_a);
    ptx::prefetch_tensormap(&tm_b);
    ptx::prefetch_tensormap(&tm_c);
    for (uint32_t s = 0; s < kSplitStages; ++s) {
      ptx::mbar_init(full_bar + 8u * s, 1);
      ptx::mbar_init(empty_bar + 8u * s, 1);
    }
    ptx::mbar_init(tfull_bar, 1);
    ptx::mbar_init(recv_bar, 1);
    *abort_ptr = 0u;
    ptx::fence_mbar_init();
    ptx::fence_proxy_async_smem();
    // what this CTA will receive: kSplit - 1 parts of 128 rows x kOwnCols fp32
    ptx::mbar_arrive_expect_tx(recv_bar, kRecvBytes);
  }
  // The producer lane starts the first pass through the ring before the set-up barrier.
  uint32_t pre = 0;
  if (threadIdx.x == 0) {
    const uint32_t n_pre = (kb1 - kb0) < kSplitStages ? (kb1 - kb0) : kSplitStages;
    for (uint32_t i = 0; i < n_pre; ++i) {
      const uint32_t sa = ring + i * kSplitStageBytes;
      const int32_t k0 = (int32_t)((kb0 + i) * kBlockKElems);
      ptx::mbar_arrive_expect_tx(full_bar + 8u * i, kSplitStageBytes);
      ptx::tma_load_2d(sa, &tm_a, full_bar + 8u * i, k0, (int32_t)(tc.m * kCtaRows));
      ptx::tma_load_2d(sa + kABytes, &tm_b, full_bar + 8u * i, k0, (int32_t)(tc.n * kSplitBN));
    }
    pre = n_pre;
  }
  if (warp_idx == 1) {
    ptx::tmem_alloc<1>(tmem_slot, 256);
    ptx::tmem_relinquish<1>();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot_ptr;
  if (threadIdx.x == 0) PATINA_TRACE_AT(1);

  if (warp_idx == 0) {
    // ---------------------------------------------------------- TMA producer
    if (lane == 0) {
      uint32_t s = pre == kSplitStages ? 0u : pre, ph = pre == kSplitStages ? 1u : 0u;
      for (uint32_t kb = kb0 + pre; kb < kb1; ++kb) {
        if (!bounded_wait<false>(empty_bar + 8u * s, ph ^ 1u, w, kTimeoutProducerEmpty, tile)) break;
        const uint32_t sa = ring + s * kSplitStageBytes;
        const int32_t k0 = (int32_t)(kb * kBlockKElems);
        ptx::mbar_arrive_expect_tx(full_bar + 8u * s, kSplitStageBytes);
        ptx::tma_load_2d(sa, &tm_a, full_bar + 8u * s, k0, (int32_t)(tc.m * kCtaRows));
        ptx::tma_load_2d(sa + kABytes, &tm_b, full_bar + 8u * s, k0, (int32_t)(tc.n * kSplitBN));
        if (++s == kSplitStages) { s = 0; ph ^= 1u; }
      }
    }
  } else if (warp_idx == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc_v = idesc(kBF16, kCtaRows, kSplitBN);
      uint32_t s = 0, ph = 0;
      bool ok = true;
      for (uint32_t kb = kb0; kb < kb1; ++kb) {
        ok = bounded_wait<false>(full_bar + 8u * s, ph, w, kTimeoutMmaFull, tile);
        if (!ok) break;
        ptx::tc_fence_after_sync();
        if (kb == kb0) PATINA_TRACE_AT(2);
        const uint32_t sa = ring + s * kSplitStageBytes;
        const uint64_t da = smem_desc_sw128_kmajor(sa), db = smem_desc_sw128_kmajor(sa + kABytes);
#pragma unroll
        for (uint32_t k = 0; k < 4u; ++k) {
          const uint32_t adv = k_advance_units_sw128(k * 16u, kBF16);
          ptx::umma<1, 0>(tmem_base, da + adv, db + adv, idesc_v, (kb != kb0 || k != 0u) ? 1u : 0u);
        }
        ptx::umma_commit<1>(empty_bar + 8u * s);
        if (++s == kSplitStages) { s = 0; ph ^= 1u; }
      }
      if (ok) {
        ptx::umma_commit<1>(tfull_bar);
        // every MMA has retired (and so every load was consumed) before the ring changes hands
        bounded_wait<false>(tfull_bar, 0u, w, kTimeoutMmaDrain, tile);
        PATINA_TRACE_AT(3);
      }
    }
  } else {
    // -------------------------------------------- epilogue warps: accumulator complete
    bool ok = bounded_wait<false>(tfull_bar, 0u, w, kTimeoutEpilogueTmemFull, tile);
    ok = __all_sync(0xffffffffu, ok);
    (void)ok;
    ptx::tc_fence_after_sync();
  }

  // ---- barrier 1: every CTA of the cluster is done with its ring -----------------------------
  __syncwarp();
  ptx::cluster_arrive();
  ptx::cluster_wait();
  if (threadIdx.x == 64) PATINA_TRACE_AT(4);       // first cluster barrier passed

  const uint32_t q = warp_idx & 3u;                                  // TMEM lane quarter of an epilogue warp
  const uint32_t taddr = tmem_base + tmem_lane_offset(q);
  const bool live = (*abort_ptr == 0u);
  if (warp_idx >= 2 && live) {
    // ---- 2. my accumulator's columns that other CTAs own -> local send area -> their receive slot
    const uint32_t send_area = ring + kRecvBytes;
    const uint32_t my_slot = rank;                                     // slot index at a receiver: senders in rank order,
#pragma unroll 1                                                       // the receiver's own rank left out
    for (uint32_t o = 0; o < (uint32_t)kSplit; ++o) {
      if (o == rank) continue;
      const uint32_t oi = o < rank ? o : o - 1u;                        // my send slot for destination o
      const uint32_t local = send_area + oi * kSlotBytes + q * (kOwnChunks * kChunkBytes);
#pragma unroll 1
      for (uint32_t c = 0; c < kOwnChunks; ++c) {
        uint32_t v[32];
        ptx::tmem_ld_32x32b_x32(taddr + o * kOwnCols + c * 32u, v);
        ptx::tmem_ld_wait();
#pragma unroll
        for (uint32_t j = 0; j < 8u; ++j)
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(local + c * kChunkBytes + (j * 32u + lane) * 16u),
                       "r"(v[4 * j]), "r"(v[4 * j + 1]), "r"(v[4 * j + 2]), "r"(v[4 * j + 3])
                       : "memory");
      }
      ptx::fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        const uint32_t si = my_slot < o ? my_slot : my_slot - 1u;     // my slot at receiver o
        const uint32_t remote = ptx::mapa(ring + si * kSlotBytes + q * (kOwnChunks * kChunkBytes), o);
        ptx::bulk_copy_to_cluster(remote, local, kOwnChunks * kChunkBytes, ptx::mapa(recv_bar, o));
      }
    }
  }

  if (threadIdx.x == 64) PATINA_TRACE_AT(5);       // my parts are staged and their copies issued
  // ---- all parts for my columns have landed -------------------------------------------------
  bool got = true;
  if (warp_idx >= 2) {
    got = bounded_wait<true>(recv_bar, 0u, w, kTimeoutEpilogueTmemFull, tile);
    got = __all_sync(0xffffffffu, got);
  }
  // Everything this CTA will ever read from a partner has arrived; tell the cluster (the matching
  // wait is at the very end: nobody's shared memory may go away while a copy still reads it).
  if (threadIdx.x == 64) PATINA_TRACE_AT(6);       // received everything
  __syncwarp();
  ptx::cluster_arrive();

  if (warp_idx >= 2 && live && got && (*abort_ptr == 0u)) {
    // ---- 3. sum my columns over the CTAs in rank order, scale, round, store ------------------
    const uint32_t e = warp_idx - 2u;
    const uint32_t stg0 = staging + e * (2u * kStoreBoxRows * 64u);
    const uint32_t row0 = tc.m * kCtaRows + q * kStoreBoxRows;
    const uint32_t row_sw = (lane >> 1) & 3u;                         // 64-byte rows, 64-byte swizzle
    uint32_t sbuf = 0;
#pragma unroll 1
    for (uint32_t c = 0; c < kOwnChunks; ++c) {
      uint32_t own[32];
      ptx::tmem_ld_32x32b_x32(taddr + rank * kOwnCols + c * 32u, own);
      ptx::tmem_ld_wait();
      float acc[32];
#pragma unroll
      for (uint32_t i = 0; i < 32u; ++i) acc[i] = 0.0f;
#pragma unroll
      for (uint32_t src = 0; src < (uint32_t)kSplit; ++src) {
        if (src == rank) {
#pragma unroll
          for (uint32_t i = 0; i < 32u; ++i) acc[i] = (src == 0u) ? __uint_as_float(own[i]) : acc[i] + __uint_as_float(own[i]);
        } else {
          const uint32_t si = src < rank ? src : src - 1u;
          const uint32_t base = ring + si * kSlotBytes + q * (kOwnChunks * kChunkBytes) + c * kChunkBytes;
#pragma unroll
          for (uint32_t j = 0; j < 8u; ++j) {
            const uint4 x = ptx::ld_shared_v4(base + (j * 32u + lane) * 16u);
            acc[4 * j] = (src == 0u) ? __uint_as_float(x.x) : acc[4 * j] + __uint_as_float(x.x);
            acc[4 * j + 1] = (src == 0u) ? __uint_as_float(x.y) : acc[4 * j + 1] + __uint_as_float(x.y);
            acc[4 * j + 2] = (src == 0u) ? __uint_as_float(x.z) : acc[4 * j + 2] + __uint_as_float(x.z);
            acc[4 * j + 3] = (src == 0u) ? __uint_as_float(x.w) : acc[4 * j + 3] + __uint_as_float(x.w);
          }
        }
      }
      // staging buffer about to be rewritten must have been read by its store
      if (lane == 0) ptx::tma_store_wait_read<1>();
      __syncwarp();
      const uint32_t row_addr = stg0 + sbuf * (kStoreBoxRows * 64u) + lane * 64u;
#pragma unroll
      for (uint32_t j = 0; j < 4u; ++j) {
        uint32_t wv[4];
#pragma unroll
        for (uint32_t e2 = 0; e2 < 4u; ++e2) {
          __nv_bfloat162 h = __floats2bfloat162_rn(acc[8 * j + 2 * e2] * p.alpha, acc[8 * j + 2 * e2 + 1] * p.alpha);
          wv[e2] = *reinterpret_cast<uint32_t*>(&h);
        }
        const uint32_t dst = row_addr + ((j ^ row_sw) << 4);
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(wv[0]), "r"(wv[1]), "r"(wv[2]),
                     "r"(wv[3])
                     : "memory");
      }
      ptx::fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        const uint32_t cc = tc.n * kSplitBN + rank * kOwnCols + c * 32u;
        if (row0 < p.M && cc < p.N) ptx::tma_store_2d(&tm_c, stg0 + sbuf * (kStoreBoxRows * 64u), (int32_t)cc, (int32_t)row0);
        ptx::tma_store_commit();
      }
      sbuf ^= 1u;
    }
    if (lane == 0) ptx::tma_store_wait_read<0>();
  }

  // ---------------------------------------------------------------- teardown
  __syncwarp();
  if (*abort_ptr) {
    const uint64_t t0 = ptx::globaltimer_ns();
    while (ptx::globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  __syncwarp();
  ptx::cluster_wait();        // every CTA of the cluster has received all its parts: no copy still reads my send area
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  if (warp_idx == 1) ptx::tmem_dealloc<1>(tmem_base, 256);
  if (threadIdx.x == 32) PATINA_TRACE_AT(7);
}

}  // namespace patina

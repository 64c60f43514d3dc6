// patina_gemm_streamk.cuh -- the skinny ("decode-shaped") GEMM: few rows of A,
// many rows of B, deep K. Memory-bound: the job is to stream B from HBM once,
// at full bandwidth, on every SM.
//
//   C[M,N] = alpha * X[M,K] * W[N,K]^T,   M <= 128 (X = activations, W = weights)
//
// Differences from the large-tile kernel (patina_gemm_kernel.cuh):
//   * operands swapped for the tensor core: 128 rows of W are the MMA's M side
//     (TMEM lanes), the M rows of X (padded to a multiple of 16) its N side
//     (TMEM columns), so a skinny M wastes no tensor-core rows;
//   * work is the flat list of (weight tile, k-block) units, cut into one
//     contiguous range per CTA ("stream-K"), so all SMs pull bytes until the
//     end whatever the number of weight tiles;
//   * a weight tile whose K range is shared by several CTAs is reduced through
//     global scratch memory without any CTA waiting for another: every
//     contributor writes its fp32 partial tile, bumps the tile's counter, and the
//     contributor that arrives last adds the partials up in contributor order
//     (so the result does not depend on who was last) and writes C.
//
// Roles are the same 1 + 1 + 4 warps as the reference's generated kernel
// (crates/patina/tests/golden/v2_gemm_pipelined.ptx:89-94).
#pragma once

#include <cuda_bf16.h>

#include "patina_desc.h"
#include "patina_gemm_kernel.cuh"
#include "patina_ptx.cuh"

namespace patina {

struct StreamKParams {
  uint32_t M, N, K;
  uint32_t m_pad;          // M rounded up to 16: the MMA's N extent
  uint32_t tiles;          // 128-row tiles of W
  uint32_t k_blocks;       // 128-byte k-blocks per tile
  uint64_t units;          // tiles * k_blocks
  uint32_t max_contrib;    // partial slots reserved per tile
  uint32_t stages;         // ring depth (<= kSkMaxStages)
  uint32_t stage_stride;   // bytes per stage: 16 KB of W + m_pad * 128 bytes of X
  uint32_t burst;          // stages the producer fills back to back, so that adjacent k-blocks
                           // of the same rows of W reach DRAM together (measured: 1 -> 4 stages
                           // lifts a 470 MB stream from 4.8 to 5.8 TB/s)
  float alpha;
  void* C;                 // bf16 [M, ldc], or fp32 when out_f32
  uint32_t out_f32;        // 1: C is fp32 (the reference's f16 -> f32 types), 0: bf16
  int64_t ldc;
  float* partials;         // [tiles][max_contrib][m_pad / 4][128 rows][4] fp32
  uint32_t* counters;      // [tiles], zero between launches
  uint32_t split_reduce;   // 1: shared tiles are only published here and summed by
                           // streamk_reduce_kernel, launched right after on the same stream
  uint32_t* status;
  uint64_t wait_limit_ns;
#ifdef PATINA_TRACE
  unsigned long long* trace;  // trace builds only: [grid][64] time stamps (see patina_gemm_kernel.cuh)
#endif
};

enum : uint32_t { kTimeoutStreamK = 6 };

constexpr uint32_t kSkTileRows = 128;
constexpr uint32_t kSkMaxStages = 13;       // what the barrier region has room for
constexpr uint32_t kSkTmemCols = 256;       // two accumulators of up to 128 columns

// One stage holds a 128-row slab of W and an m_pad-row slab of X, 128 bytes of K each. The
// ring takes whatever shared memory allows: a skinny X leaves room for more stages, i.e. more
// bytes of W in flight per SM, which is what a bandwidth-bound kernel lives on.
PATINA_HD constexpr uint32_t streamk_stage_stride(uint32_t m_pad) {
  return kSkTileRows * kBlockKBytes + m_pad * kBlockKBytes;
}
PATINA_HD constexpr uint32_t streamk_stages(uint32_t m_pad) {
  const uint32_t fit = (kMaxDynSmem - 1024 - kBarrierRegionBytes) / streamk_stage_stride(m_pad);
  return fit < kSkMaxStages ? fit : kSkMaxStages;
}
PATINA_HD constexpr uint32_t streamk_smem_bytes(uint32_t m_pad) {
  return 1024 + streamk_stages(m_pad) * streamk_stage_stride(m_pad) + kBarrierRegionBytes;
}

// First unit of CTA c's range, and the CTA that owns unit u, for `units` units cut into
// `parts` contiguous ranges whose lengths differ by at most one.
PATINA_HD uint64_t streamk_range_start(uint64_t c, uint64_t units, uint64_t parts) {
  return c * units / parts;
}
PATINA_HD uint32_t streamk_owner(uint64_t u, uint64_t units, uint64_t parts) {
  return (uint32_t)(((u + 1) * parts - 1) / units);
}
// Upper bound on the CTAs that can share one tile of `k_blocks` units.
PATINA_HD uint32_t streamk_max_contrib(uint64_t units, uint64_t parts, uint32_t k_blocks) {
  const uint64_t min_len = units / parts ? units / parts : 1;
  return (uint32_t)((k_blocks - 1) / min_len) + 2;
}

// True when at least one tile's k-blocks are split between CTAs (a CTA boundary that is not a
// tile boundary). Without one every tile is computed whole and nothing needs summing.
PATINA_HD bool streamk_any_shared_tile(uint64_t units, uint64_t parts, uint32_t k_blocks) {
  for (uint64_t c = 1; c < parts; ++c)
    if (streamk_range_start(c, units, parts) % k_blocks != 0) return true;
  return false;
}

// One element of C, rounded to the output type.
__device__ __forceinline__ void streamk_store(const StreamKParams& p, size_t index, float v) {
  if (p.out_f32) static_cast<float*>(p.C)[index] = v;
  else static_cast<__nv_bfloat16*>(p.C)[index] = __float2bfloat16_rn(v);
}

template <int kIn>
__global__ void __launch_bounds__(192, 1)
gemm_streamk_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x,
                    const StreamKParams p) {
  constexpr int kKind = (kIn == kE4M3) ? 1 : 0;
  constexpr uint32_t kBlockKElems = kBlockKBytes / input_bytes(kIn);
  constexpr uint32_t kUmmaK = umma_k(kIn);
  constexpr uint32_t kWBytes = kSkTileRows * kBlockKBytes;
  static_assert((2 * kSkMaxStages + 4) * 8 + 16 <= kBarrierRegionBytes, "barrier region too small");
  const uint32_t kStages = p.stages;
  const uint32_t kSkStageStride = p.stage_stride;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t ring = smem_base;
  const uint32_t bars = ring + kStages * kSkStageStride;
  const uint32_t full_bar = bars;
  const uint32_t empty_bar = bars + 8u * kSkMaxStages;
  const uint32_t tfull_bar = bars + 16u * kSkMaxStages;
  const uint32_t tempty_bar = tfull_bar + 16u;
  const uint32_t tmem_slot = tempty_bar + 16u;
  const uint32_t abort_slot = tmem_slot + 4u;
  const uint32_t last_slot = abort_slot + 4u;
  uint8_t* const smem_generic = smem_raw + (smem_base - ptx::smem_u32(smem_raw));
  volatile uint32_t* const tmem_slot_ptr =
      reinterpret_cast<volatile uint32_t*>(smem_generic + (tmem_slot - smem_base));
  volatile uint32_t* const abort_ptr =
      reinterpret_cast<volatile uint32_t*>(smem_generic + (abort_slot - smem_base));
  volatile uint32_t* const last_ptr =
      reinterpret_cast<volatile uint32_t*>(smem_generic + (last_slot - smem_base));

  const uint32_t warp_idx = threadIdx.x >> 5;
  const uint32_t lane = threadIdx.x & 31u;
  const uint64_t parts = gridDim.x;
  const uint64_t u_begin = streamk_range_start(blockIdx.x, p.units, parts);
  const uint64_t u_end = streamk_range_start(blockIdx.x + 1ull, p.units, parts);
  const uint32_t x_bytes = p.m_pad * kBlockKBytes;

  WaitCtx w;
  w.abort_flag = abort_ptr;
  w.peer_abort_addr = 0u;
  w.status = p.status;
  w.limit_ns = p.wait_limit_ns;
  w.has_peer = false;

  // Producer state lives outside the role branch: the producer lanes start the first ring pass
  // before the CTA-wide set-up barrier, so that TMEM allocation and the barrier hide behind DRAM
  // latency.
  uint32_t prod_s = 0, prod_ph = 0;
  uint64_t prod_u = u_begin;
  uint32_t prod_t = (uint32_t)(u_begin / p.k_blocks);
  uint32_t prod_kb = (uint32_t)(u_begin - (uint64_t)prod_t * p.k_blocks);
  // W is read exactly once: keep it from displacing X (re-read by every CTA) in L2.
  uint64_t stream_once = 0, keep = 0;
  if (threadIdx.x == 0) {
    PATINA_TRACE_AT(0);
    ptx::prefetch_tensormap(&tm_w);
    ptx::prefetch_tensormap(&tm_x);
    for (uint32_t s = 0; s < kStages; ++s) {
      ptx::mbar_init(full_bar + 8u * s, 1);
      ptx::mbar_init(empty_bar + 8u * s, 1);
    }
    for (uint32_t b = 0; b < 2; ++b) {
      ptx::mbar_init(tfull_bar + 8u * b, 1);
      ptx::mbar_init(tempty_bar + 8u * b, 4);
    }
    *abort_ptr = 0u;
    *last_ptr = 0u;
    ptx::fence_mbar_init();
    ptx::fence_proxy_async_smem();
  }
  // Two producer lanes: lane 0 announces the stage's bytes and loads the slab of W, lane 1 loads
  // the slab of X (an issuing lane spends 150 - 200 cycles per TMA load and 390 per {wait,
  // announce, issue} round; two lanes overlap theirs).
  const bool is_producer = (warp_idx == 0 && lane < 2u);
  if (warp_idx == 0) {
    __syncwarp();   // thread 0's barriers, seen by lane 1
    if (is_producer) {
      ptx::fence_proxy_async_smem();
      stream_once = ptx::l2_policy_evict_first();
      keep = ptx::l2_policy_evict_last();
      // First pass through the ring: every stage is free, no wait needed.
      while (prod_u < u_end && prod_ph == 0u) {
        const uint32_t sw = ring + prod_s * kSkStageStride;
        const int32_t k0 = (int32_t)(prod_kb * kBlockKElems);
        if (lane == 0) {
          ptx::mbar_arrive_expect_tx(full_bar + 8u * prod_s, kWBytes + x_bytes);
          ptx::tma_load_2d_hint(sw, &tm_w, full_bar + 8u * prod_s, k0, (int32_t)(prod_t * kSkTileRows), stream_once);
        } else {
          ptx::tma_load_2d_hint(sw + kWBytes, &tm_x, full_bar + 8u * prod_s, k0, 0, keep);
        }
        ++prod_u;
        if (++prod_s == kStages) { prod_s = 0; prod_ph = 1u; }
        if (++prod_kb == p.k_blocks) { prod_kb = 0; ++prod_t; }
      }
    }
  }
  if (warp_idx == 1) {
    ptx::tmem_alloc<1>(tmem_slot, kSkTmemCols);
    ptx::tmem_relinquish<1>();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot_ptr;
  if (threadIdx.x == 0) PATINA_TRACE_AT(1);
  // Let the follow-up reduce kernel's blocks take their places now; they wait for this grid to
  // complete before touching memory.
  if (p.split_reduce) ptx::launch_dependents();

  // ------------------------------------------------------------ TMA producer
  if (warp_idx == 0) {
    if (is_producer) {
      uint32_t s = prod_s, ph = prod_ph;
      bool ok = true;
      uint64_t u = prod_u;
      uint32_t t = prod_t;
      uint32_t kb = prod_kb;
      while (u < u_end && ok) {
        const uint64_t left = u_end - u;
        const uint32_t group = left < p.burst ? (uint32_t)left : p.burst;
        // all stages of the group must be free before any of it is issued
        uint32_t s2 = s, ph2 = ph;
        for (uint32_t g = 0; g < group && ok; ++g) {
          ok = bounded_wait<false>(empty_bar + 8u * s2, ph2 ^ 1u, w, kTimeoutProducerEmpty, t);
          if (++s2 == kStages) { s2 = 0; ph2 ^= 1u; }
        }
        if (!ok) break;
        for (uint32_t g = 0; g < group; ++g, ++u) {
          const uint32_t sw = ring + s * kSkStageStride;
          const int32_t k0 = (int32_t)(kb * kBlockKElems);
          if (lane == 0) {
            ptx::mbar_arrive_expect_tx(full_bar + 8u * s, kWBytes + x_bytes);
            ptx::tma_load_2d_hint(sw, &tm_w, full_bar + 8u * s, k0, (int32_t)(t * kSkTileRows), stream_once);
          } else {
            ptx::tma_load_2d_hint(sw + kWBytes, &tm_x, full_bar + 8u * s, k0, 0, keep);
          }
          if (++s == kStages) { s = 0; ph ^= 1u; }
          if (++kb == p.k_blocks) { kb = 0; ++t; }
        }
      }
    }
  }
  // -------------------------------------------------------------- MMA issuer
  else if (warp_idx == 1) {
    if (lane == 0) {
      const uint32_t idesc_v = idesc(kIn, kSkTileRows, p.m_pad);
      uint32_t s = 0, ph = 0, seg = 0;
      bool ok = true;
      uint64_t u = u_begin;
      while (u < u_end && ok) {
        const uint32_t t = (uint32_t)(u / p.k_blocks);
        const uint32_t kb0 = (uint32_t)(u - (uint64_t)t * p.k_blocks);
        const uint64_t left = u_end - u;
        const uint32_t kb1 = (uint64_t)(p.k_blocks - kb0) <= left ? p.k_blocks : kb0 + (uint32_t)left;
        const uint32_t buf = seg & 1u, acc_ph = (seg >> 1) & 1u;
        ok = bounded_wait<false>(tempty_bar + 8u * buf, acc_ph ^ 1u, w, kTimeoutMmaTmemEmpty, t);
        if (!ok) break;
        ptx::tc_fence_after_sync();
        const uint32_t tmem_d = tmem_base + buf * 128u;
        for (uint32_t kb = kb0; kb < kb1; ++kb) {
          ok = bounded_wait<false>(full_bar + 8u * s, ph, w, kTimeoutMmaFull, t);
          if (!ok) break;
          ptx::tc_fence_after_sync();
          if (u == u_begin && kb == kb0) PATINA_TRACE_AT(2);
          if (seg == 0) PATINA_TRACE_KB(32u, kb - kb0);
          const uint32_t sw = ring + s * kSkStageStride;
          const uint64_t dw = smem_desc_sw128_kmajor(sw);
          const uint64_t dx = smem_desc_sw128_kmajor(sw + kWBytes);
#pragma unroll
          for (uint32_t k = 0; k < kBlockKElems / kUmmaK; ++k) {
            const uint32_t adv = k_advance_units_sw128(k * kUmmaK, kIn);
            ptx::umma<1, kKind>(tmem_d, dw + adv, dx + adv, idesc_v, (kb != kb0 || k != 0u) ? 1u : 0u);
          }
          ptx::umma_commit<1>(empty_bar + 8u * s);
          if (++s == kStages) { s = 0; ph ^= 1u; }
        }
        if (!ok) break;
        ptx::umma_commit<1>(tfull_bar + 8u * buf);
        PATINA_TRACE_AT(3);
        u += kb1 - kb0;
        ++seg;
      }
      if (ok && seg > 0) {
        const uint32_t last = seg - 1;
        bounded_wait<false>(tfull_bar + 8u * (last & 1u), (last >> 1) & 1u, w, kTimeoutMmaDrain, seg);
      }
    }
  }
  // ---------------------------------------------------------------- epilogue
  else {
    const uint32_t q = warp_idx & 3u;
    const uint32_t epi_tid = threadIdx.x - 64u;
    uint32_t seg = 0;
    // A warp whose wait was abandoned goes "dead": it touches no more data but still walks
    // the segment list and joins the named barriers, so the other epilogue warps (which may
    // have passed the same wait a moment earlier) can never be left waiting for it.
    bool dead = false;
    uint64_t u = u_begin;
    while (u < u_end) {
      const uint32_t t = (uint32_t)(u / p.k_blocks);
      const uint32_t kb0 = (uint32_t)(u - (uint64_t)t * p.k_blocks);
      const uint64_t left = u_end - u;
      const uint32_t kb1 = (uint64_t)(p.k_blocks - kb0) <= left ? p.k_blocks : kb0 + (uint32_t)left;
      const uint32_t buf = seg & 1u, acc_ph = (seg >> 1) & 1u;
      if (!dead) {
        bool ok = bounded_wait<false>(tfull_bar + 8u * buf, acc_ph, w, kTimeoutEpilogueTmemFull, t);
        ok = __all_sync(0xffffffffu, ok);
        dead = !ok;
      }
      ptx::tc_fence_after_sync();
      if (epi_tid == 0) PATINA_TRACE_AT(4);   // (last segment's stamp stays)
      const uint32_t taddr = tmem_base + tmem_lane_offset(q) + buf * 128u;
      const uint32_t n = t * kSkTileRows + q * 32u + lane;  // the column of C this thread owns
      const bool whole = (kb0 == 0u && kb1 == p.k_blocks);
      uint32_t my_j = 0, contribs = 1;
      bool is_last = !dead;
      if (!whole) {
        const uint64_t tile_u0 = (uint64_t)t * p.k_blocks;
        const uint32_t first_cta = streamk_owner(tile_u0, p.units, parts);
        contribs = streamk_owner(tile_u0 + p.k_blocks - 1, p.units, parts) - first_cta + 1u;
        my_j = blockIdx.x - first_cta;
        // 1. publish this CTA's partial tile. Slot layout [m / 4][128 weight rows][4]: a thread
        //    writes four consecutive m of its row as one 16-byte word, a warp 512 contiguous bytes.
        if (!dead) {
          float4* mine = reinterpret_cast<float4*>(
                             p.partials + ((size_t)t * p.max_contrib + my_j) * ((size_t)p.m_pad * 128u)) +
                         q * 32u + lane;
          for (uint32_t m0 = 0; m0 < p.m_pad; m0 += 16u) {
            uint32_t v[16];
            ptx::tmem_ld_32x32b_x16(taddr + m0, v);
            ptx::tmem_ld_wait();
#pragma unroll
            for (uint32_t g = 0; g < 4; ++g)
              __stcg(mine + (size_t)(m0 / 4u + g) * 128u,
                     make_float4(__uint_as_float(v[4 * g]), __uint_as_float(v[4 * g + 1]),
                                 __uint_as_float(v[4 * g + 2]), __uint_as_float(v[4 * g + 3])));
          }
          if (!p.split_reduce) __threadfence();
        }
        if (p.split_reduce) {
          // The sum over contributors is the follow-up kernel's job (all SMs share it; a
          // single finishing CTA would have to pull every contributor's tile through one SM).
          is_last = false;
        } else {
          ptx::named_bar_sync(1, 128);
          if (epi_tid == 0) {
            bool last = false;
            if (!dead && *abort_ptr == 0u) {
              const uint32_t seen = atomicAdd(p.counters + t, 1u);
              last = (seen == contribs - 1u);
              if (last) p.counters[t] = 0u;  // everybody has arrived: leave it clean for the next launch
            }
            *last_ptr = last ? 1u : 0u;
          }
          ptx::named_bar_sync(1, 128);
          is_last = !dead && (*last_ptr != 0u);
          if (is_last) __threadfence();
        }
      }
      if (epi_tid == 0) PATINA_TRACE_AT(5);   // partial published / arrival counted
      if (is_last) {
        // 2. sum the contributors in their fixed order (this CTA's part comes from TMEM), scale,
        //    round to bf16 and store C[m][n]. Sixteen values of m at a time; the partials of up
        //    to eight contributors (32 loads of 16 bytes per thread) are requested before any is
        //    used, so a tile shared by many CTAs costs one or two trips to L2, not one per CTA.
        const float4* slot0 = reinterpret_cast<const float4*>(
                                  p.partials + (size_t)t * p.max_contrib * ((size_t)p.m_pad * 128u)) +
                              q * 32u + lane;
        const size_t slot_quads = (size_t)p.m_pad * 32u;  // float4 words per slot
        for (uint32_t m0 = 0; m0 < p.m_pad; m0 += 16u) {
          uint32_t own[16];
          ptx::tmem_ld_32x32b_x16(taddr + m0, own);
          ptx::tmem_ld_wait();
          float acc[16];
#pragma unroll
          for (uint32_t i = 0; i < 16; ++i) acc[i] = 0.0f;
          for (uint32_t j0 = 0; j0 < contribs; j0 += 8u) {
            float4 x[8][4];
#pragma unroll
            for (uint32_t jj = 0; jj < 8; ++jj) {
              const uint32_t j = j0 + jj;
              if (j < contribs && j != my_j) {
                const float4* other = slot0 + (size_t)j * slot_quads + (size_t)(m0 / 4u) * 128u;
#pragma unroll
                for (uint32_t g = 0; g < 4; ++g) x[jj][g] = __ldcg(other + (size_t)g * 128u);
              }
            }
#pragma unroll
            for (uint32_t jj = 0; jj < 8; ++jj) {
              const uint32_t j = j0 + jj;
              if (j < contribs) {
                const bool mine = (j == my_j);
#pragma unroll
                for (uint32_t g = 0; g < 4; ++g) {
                  const float a0 = mine ? __uint_as_float(own[4 * g]) : x[jj][g].x;
                  const float a1 = mine ? __uint_as_float(own[4 * g + 1]) : x[jj][g].y;
                  const float a2 = mine ? __uint_as_float(own[4 * g + 2]) : x[jj][g].z;
                  const float a3 = mine ? __uint_as_float(own[4 * g + 3]) : x[jj][g].w;
                  acc[4 * g] = (j == 0u) ? a0 : acc[4 * g] + a0;
                  acc[4 * g + 1] = (j == 0u) ? a1 : acc[4 * g + 1] + a1;
                  acc[4 * g + 2] = (j == 0u) ? a2 : acc[4 * g + 2] + a2;
                  acc[4 * g + 3] = (j == 0u) ? a3 : acc[4 * g + 3] + a3;
                }
              }
            }
          }
          if (n < p.N) {
#pragma unroll
            for (uint32_t i = 0; i < 16; ++i)
              if (m0 + i < p.M) streamk_store(p, (size_t)(m0 + i) * p.ldc + n, acc[i] * p.alpha);
          }
        }
      }
      if (epi_tid == 0) PATINA_TRACE_AT(6);   // segment finished (C written if this CTA was last)
      // accumulator drained: hand the TMEM buffer back
      if (!dead) {
        ptx::tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(tempty_bar + 8u * buf);
      }
      u += kb1 - kb0;
      ++seg;
    }
  }

  // ---------------------------------------------------------------- teardown
  __syncwarp();
  if (*abort_ptr) {
    const uint64_t t0 = ptx::globaltimer_ns();
    while (ptx::globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  __syncwarp();
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  if (warp_idx == 1) ptx::tmem_dealloc<1>(tmem_base, kSkTmemCols);
  if (threadIdx.x == 32) PATINA_TRACE_AT(7);
}

// Second half of a split-reduce launch: sums the partial tiles that gemm_streamk_kernel
// published, in contributor order (so the result does not depend on timing), scales, rounds to
// bf16 and writes C. One block per (tile of 128 columns of C, 16 rows of C); thread = column.
// Tiles that one CTA computed whole were written by that CTA and are skipped.
__global__ void __launch_bounds__(128)
streamk_reduce_kernel(const StreamKParams p, const uint32_t parts) {
  const uint32_t chunks = p.m_pad / 16u;
  const uint32_t t = blockIdx.x / chunks;
  const uint32_t m0 = (blockIdx.x - t * chunks) * 16u;
  const uint64_t tile_u0 = (uint64_t)t * p.k_blocks;
  const uint32_t first_cta = streamk_owner(tile_u0, p.units, parts);
  const uint32_t contribs = streamk_owner(tile_u0 + p.k_blocks - 1, p.units, parts) - first_cta + 1u;
  // Every block waits, also one with nothing to sum: this grid must not complete before the GEMM
  // grid has, or work enqueued behind it on the stream could read C too early.
  ptx::grid_dependency_wait();  // the partial tiles are complete and visible from here on
  if (contribs < 2u) return;
  const uint32_t n = t * kSkTileRows + threadIdx.x;
  const float4* slot0 = reinterpret_cast<const float4*>(
                            p.partials + (size_t)t * p.max_contrib * ((size_t)p.m_pad * 128u)) +
                        (size_t)(m0 / 4u) * 128u + threadIdx.x;
  const size_t slot_quads = (size_t)p.m_pad * 32u;
  float acc[16];
#pragma unroll
  for (uint32_t i = 0; i < 16; ++i) acc[i] = 0.0f;
  for (uint32_t j0 = 0; j0 < contribs; j0 += 8u) {
    float4 x[8][4];
#pragma unroll
    for (uint32_t jj = 0; jj < 8; ++jj) {
      if (j0 + jj < contribs) {
#pragma unroll
        for (uint32_t g = 0; g < 4; ++g)
          x[jj][g] = __ldcg(slot0 + (size_t)(j0 + jj) * slot_quads + (size_t)g * 128u);
      }
    }
#pragma unroll
    for (uint32_t jj = 0; jj < 8; ++jj) {
      if (j0 + jj < contribs) {
        const bool first = (j0 + jj == 0u);
#pragma unroll
        for (uint32_t g = 0; g < 4; ++g) {
          acc[4 * g] = first ? x[jj][g].x : acc[4 * g] + x[jj][g].x;
          acc[4 * g + 1] = first ? x[jj][g].y : acc[4 * g + 1] + x[jj][g].y;
          acc[4 * g + 2] = first ? x[jj][g].z : acc[4 * g + 2] + x[jj][g].z;
          acc[4 * g + 3] = first ? x[jj][g].w : acc[4 * g + 3] + x[jj][g].w;
        }
      }
    }
  }
  if (n < p.N) {
#pragma unroll
    for (uint32_t i = 0; i < 16; ++i)
      if (m0 + i < p.M) streamk_store(p, (size_t)(m0 + i) * p.ldc + n, acc[i] * p.alpha);
  }
}

}  // namespace patina

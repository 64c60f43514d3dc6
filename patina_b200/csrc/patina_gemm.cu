// patina_gemm.cu -- C ABI (include/patina_gemm.h) over the tcgen05 GEMM kernels:
// argument validation, launch planning, TMA tensor-map construction and caching,
// kernel dispatch. Host side of what the reference does in
// harness/gemm_check.cpp:240-300 and crates/patina/src/run.rs:462-529, minus
// the allocation and copies (device pointers belong to the caller here).
#include "../../include/patina_gemm.h"

#include <cuda.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdarg>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "patina_desc.h"
#include "patina_gemm_kernel.cuh"
#include "patina_gemm_splitk.cuh"
#include "patina_gemm_streamk.cuh"

using namespace patina;

namespace {

char* dup_cstr(const std::string& s) {
  char* p = static_cast<char*>(std::malloc(s.size() + 1));
  if (p) std::memcpy(p, s.c_str(), s.size() + 1);
  return p;
}

std::string fmt(const char* f, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, f);
  std::vsnprintf(buf, sizeof(buf), f, ap);
  va_end(ap);
  return std::string(buf);
}

// ------------------------------------------------------------------ kernels
using KernelFn = void (*)(const CUtensorMap, const CUtensorMap, const CStoreMaps<1>, const GemmParams);
using ScatterFn = void (*)(const CUtensorMap, const CUtensorMap, const CStoreMaps<kMaxDests>, const GemmParams);

struct KernelEntry {
  int cta_group, m_sub, block_n, stages, in_type, out_type;
  KernelFn fn;
  KernelFn fn_fused;     // same kernel with the bias / residual / activation epilogue, or null
  ScatterFn fn_scatter;  // same kernel storing every tile to up to kMaxDests destinations, or null
  uint32_t smem_bytes;
  int k_chunks = 1;      // k-blocks per stage; above 1 the operands come in 3-D boxes (K % 128 bytes == 0)
};

#define PATINA_KERNEL(G, MS, BN, S, IN, OUT)                                    \
  { G, MS, BN, S, IN, OUT, gemm_tn_kernel<G, MS, BN, S, IN, OUT>, nullptr, nullptr, \
    GemmTraits<G, MS, BN, S, IN, OUT>::kSmemBytes }
// bf16 -> bf16 without a fused form (widths that end in half a store box), with the scatter form
#define PATINA_KERNEL_S(G, MS, BN, S, IN, OUT)                           \
  { G, MS, BN, S, IN, OUT, gemm_tn_kernel<G, MS, BN, S, IN, OUT>, nullptr, \
    gemm_tn_kernel<G, MS, BN, S, IN, OUT, false, false, kMaxDests>,      \
    GemmTraits<G, MS, BN, S, IN, OUT>::kSmemBytes }
// bf16 -> bf16 with the fused and the scatter form
#define PATINA_KERNEL_F(G, MS, BN, S, IN, OUT)                      \
  { G, MS, BN, S, IN, OUT, gemm_tn_kernel<G, MS, BN, S, IN, OUT>,     \
    gemm_tn_kernel<G, MS, BN, S, IN, OUT, true>,                    \
    gemm_tn_kernel<G, MS, BN, S, IN, OUT, false, false, kMaxDests>, \
    GemmTraits<G, MS, BN, S, IN, OUT>::kSmemBytes }

// single-CTA kernel with KC k-blocks per stage (3-D operand boxes), plain epilogue
#define PATINA_KERNEL_KC(MS, BN, S, IN, OUT, KC)                                                   \
  { 1, MS, BN, S, IN, OUT, gemm_tn_chunked_kernel<MS, BN, S, IN, OUT, KC>, nullptr, nullptr,       \
    GemmTraits<1, MS, BN, S, IN, OUT, false, KC>::kSmemBytes, KC }

// Listed best-first per type pair: an explicit request takes the first match.
#define PATINA_KERNEL_Q(G, MS, BN, S)                                           \
  { G, MS, BN, S, kBF16, kOutE4M3, gemm_tn_kernel<G, MS, BN, S, kBF16, kOutE4M3, true>, \
    gemm_tn_kernel<G, MS, BN, S, kBF16, kOutE4M3, true>, nullptr,                \
    GemmTraits<G, MS, BN, S, kBF16, kOutE4M3>::kSmemBytes }

const KernelEntry kKernels[] = {
    // bf16 -> bf16
    PATINA_KERNEL_F(2, 2, 256, 4, kBF16, kOutBF16),  // 512 x 256 per pair, accumulators fill TMEM
    PATINA_KERNEL_F(2, 1, 256, 6, kBF16, kOutBF16),  // 256 x 256 per pair, double-buffered TMEM
    PATINA_KERNEL_F(2, 1, 256, 4, kBF16, kOutBF16),  // (4 and 6 stages measured alike: not latency-bound)
    PATINA_KERNEL_F(1, 1, 256, 4, kBF16, kOutBF16),
    PATINA_KERNEL_F(2, 2, 224, 4, kBF16, kOutBF16),  // 512 x 224: widths like 1792 or 3584 (multiples of
                                                     // 224 with an awkward count of 256-wide tiles)
    PATINA_KERNEL_S(2, 2, 240, 4, kBF16, kOutBF16),  // widths with half a store box at the end:
    PATINA_KERNEL_S(2, 2, 208, 4, kBF16, kOutBF16),  // plain epilogue only
    PATINA_KERNEL_S(2, 2, 176, 4, kBF16, kOutBF16),
    PATINA_KERNEL_F(2, 2, 192, 4, kBF16, kOutBF16),
    PATINA_KERNEL_F(2, 2, 160, 4, kBF16, kOutBF16),
    PATINA_KERNEL_F(2, 2, 128, 4, kBF16, kOutBF16),  // 512 x 128 per pair, double-buffered
    PATINA_KERNEL_F(2, 1, 128, 8, kBF16, kOutBF16),
    // Two k-blocks per stage, one 3-D box per operand and stage (see GemmTraits::kChunkABytes):
    // listed before their one-k-block twins, so they win ties and take plain launches whose K is
    // whole k-blocks (1024^3: 7.6 - 7.9 us against 8.9; 2048 x 1024 x 1024: 8.4 against 9.6).
    PATINA_KERNEL_KC(1, 128, 3, kBF16, kOutBF16, 2),
    PATINA_KERNEL_F(1, 1, 128, 6, kBF16, kOutBF16),
    // narrow tiles for problems with fewer 128-wide tiles than SMs: every SM's share of the
    // operands shrinks with the tile count, and one SM takes in about 64 bytes per clock
    PATINA_KERNEL_F(2, 1, 64, 8, kBF16, kOutBF16),   // 256 x 64 per pair
    PATINA_KERNEL_KC(1, 64, 4, kBF16, kOutBF16, 2),
    PATINA_KERNEL_F(1, 1, 64, 8, kBF16, kOutBF16),   // 128 x 64
    // e4m3 -> bf16
    PATINA_KERNEL(2, 2, 256, 4, kE4M3, kOutBF16),
    PATINA_KERNEL(2, 2, 240, 4, kE4M3, kOutBF16),
    PATINA_KERNEL(2, 2, 224, 4, kE4M3, kOutBF16),
    PATINA_KERNEL(2, 1, 256, 6, kE4M3, kOutBF16),
    PATINA_KERNEL(1, 1, 256, 4, kE4M3, kOutBF16),
    PATINA_KERNEL_KC(1, 128, 3, kE4M3, kOutBF16, 2),
    PATINA_KERNEL(1, 1, 128, 6, kE4M3, kOutBF16),
    // bf16 -> e4m3 (scaled, with amax): fused epilogue only, so both slots hold that kernel
    PATINA_KERNEL_Q(2, 1, 256, 6),
    PATINA_KERNEL_Q(1, 1, 256, 4),
    PATINA_KERNEL_Q(1, 1, 128, 6),
    // f16 -> f32 (the reference kernel's types)
    PATINA_KERNEL(2, 1, 256, 6, kF16, kOutF32),
    PATINA_KERNEL(1, 1, 256, 4, kF16, kOutF32),
    PATINA_KERNEL_KC(1, 128, 3, kF16, kOutF32, 2),
    PATINA_KERNEL(1, 1, 128, 6, kF16, kOutF32),
};
constexpr int kNumKernels = sizeof(kKernels) / sizeof(kKernels[0]);

// Grouped launches (bf16 -> bf16): the same kernel, compiled with the group tables.
#define PATINA_GROUPED(G, MS, BN, S, IN)                                                 \
  { G, MS, BN, S, IN, kOutBF16, gemm_tn_kernel<G, MS, BN, S, IN, kOutBF16, false, true>, \
    nullptr, nullptr, GemmTraits<G, MS, BN, S, IN, kOutBF16>::kSmemBytes + kGroupTableBytes }
const KernelEntry kGroupedKernels[] = {
    PATINA_GROUPED(2, 2, 256, 4, kBF16),  // 512 x 256 per pair: groups of many hundred rows
    PATINA_GROUPED(2, 1, 256, 6, kBF16),  // 256 x 256 per pair
    PATINA_GROUPED(1, 1, 256, 4, kBF16),  // 128 x 256: small groups lose least to their ragged last block
    PATINA_GROUPED(2, 2, 256, 4, kE4M3),
    PATINA_GROUPED(2, 1, 256, 6, kE4M3),
    PATINA_GROUPED(1, 1, 256, 4, kE4M3),
};
constexpr int kNumGroupedKernels = sizeof(kGroupedKernels) / sizeof(kGroupedKernels[0]);
static_assert(GemmTraits<2, 2, 256, 4, kBF16, kOutBF16>::kSmemBytes + kGroupTableBytes <= kMaxDynSmem,
              "group tables do not fit behind the largest kernel's shared memory");

// Block-scaled e4m3 (MXFP8) -> bf16. Widths are multiples of 64: a tile's scales of B start a whole
// number of 64 rows into a scale atom, i.e. an even number of TMEM columns (an odd column offset
// faults with "misaligned address": measured with 224-wide tiles). 256-wide accumulators leave no
// room in TMEM for a second buffer next to the scale columns; 192 does.
using MxFn = void (*)(const CUtensorMap, const CUtensorMap, const CStoreMaps<1>, const CUtensorMap,
                      const CUtensorMap, const GemmParams);
struct MxKernelEntry {
  int cta_group, m_sub, block_n, stages;
  MxFn fn;
  uint32_t smem_bytes;
};
#define PATINA_MX(G, MS, BN, S) \
  { G, MS, BN, S, gemm_mx_tn_kernel<G, MS, BN, S>, GemmTraits<G, MS, BN, S, kMXE4M3, kOutBF16>::kSmemBytes }
const MxKernelEntry kMxKernels[] = {
    PATINA_MX(2, 2, 192, 4),  // 512 x 192 per pair: one accumulator set + scales
    PATINA_MX(2, 1, 192, 6),  // 256 x 192 per pair, double-buffered accumulators
    PATINA_MX(2, 1, 256, 5),  // 256 x 256 per pair, one accumulator
    PATINA_MX(1, 1, 192, 4),  // 128 x 192, double-buffered
    PATINA_MX(1, 1, 128, 5),  // 128 x 128, double-buffered: small problems
};
constexpr int kNumMxKernels = sizeof(kMxKernels) / sizeof(kMxKernels[0]);

bool type_pair_supported(int in_type, int out_type) {
  if (in_type == kMXE4M3) return out_type == kOutBF16;
  for (int i = 0; i < kNumKernels; ++i)
    if (kKernels[i].in_type == in_type && kKernels[i].out_type == out_type) return true;
  return false;
}

// ------------------------------------------------------------------ planning
uint32_t ceil_div(uint64_t a, uint64_t b) { return (uint32_t)((a + b - 1) / b); }

// Tiles of the last wave that a two-sub-tile kernel runs as two half tiles each (see
// GemmParams::split_from): all of them when they fill at most half of the clusters -- the wave
// then takes half as long -- none otherwise (two half waves cost what one wave costs).
uint32_t half_tile_tail(uint32_t num_tiles, uint32_t clusters, int m_sub) {
  if (m_sub != 2 || clusters == 0) return 0;
  const uint32_t tail = num_tiles % clusters;
  return (tail > 0 && 2u * tail <= clusters) ? tail : 0u;
}

// Useful work per unit of modelled time, as a fraction of what the 512 x 256 pair tile does on
// exactly filled waves. Two measured facts go in:
//  * the throughput of each tile shape on filled waves (M = 8192, K = 4096, 37 tile columns):
//    smaller tiles move more operand bytes from L2 per flop, and the part is bound by shared
//    L2 bandwidth and power, not by any one SM;
//  * for the same reason a partly filled last wave is cheaper than a full one: with half the
//    clusters active each tile ran 29 % faster, so a wave filled to f costs about 0.55 + 0.45 f.
double config_score(const KernelEntry& k, int64_t M, int64_t N, int64_t K, int num_sms) {
  const int64_t tile_m = 128 * k.cta_group * k.m_sub;
  const uint64_t tiles = (uint64_t)ceil_div(M, tile_m) * ceil_div(N, k.block_n);
  const uint64_t slots = (uint64_t)(num_sms / k.cta_group);
  if (slots == 0 || tiles == 0) return 0.0;
  const uint64_t waves = (tiles + slots - 1) / slots;
  if (k.k_chunks == 2) {
    // Two k-blocks per stage, two accumulators: a k-block takes a CTA 0.16 us at either width
    // (issue and operand intake, not the tensor pipe), 0.20 us for the 128-wide tile once more
    // than about 96 CTAs pull 32 KB per k-block each; the 128-wide tile's epilogue is 0.5 us
    // longer. Measured: 1024^3 6.7 us on 128 x 64 tiles and 7.2 on 128 x 128, 2048 x 1024 x 1024
    // 10.3 and 7.7, 1024 x 1024 x 4096 15.6 and 15.7, 2048^3 28.2 and 18.4.
    // For problems of at most one wave of 128 x 128 tiles; beyond, the wide tiles' lower operand
    // traffic per flop wins (2048^3: 15.7 us on 128 x 256 tiles against 18.4).
    if ((uint64_t)ceil_div(M, 128) * ceil_div(N, 128) > slots) return 0.0;
    const uint64_t ctas = tiles < slots ? tiles : slots;
    const double kb = (double)ceil_div(K, kBlockKBytes / input_bytes(k.in_type));
    const double t_kb = (k.block_n >= 128 && ctas > 96) ? 0.20 : 0.16;
    const double time_us = t_kb * kb * (double)waves + (k.block_n >= 128 ? 4.6 : 4.1);
    return 1.0e12 / (time_us * 82000.0);
  }
  const double last_fill = (double)(tiles - (waves - 1) * slots) / (double)slots;
  double speed = 0.6;
  if (k.cta_group == 2 && k.m_sub == 2) {
    speed = k.block_n >= 256 ? 1.0 : k.block_n >= 240 ? 0.99 : k.block_n >= 224 ? 0.985
            : k.block_n >= 208 ? 0.975 : k.block_n >= 192 ? 0.95 : k.block_n >= 176 ? 0.91
            : k.block_n >= 160 ? 0.86 : 0.80;
  } else if (k.cta_group == 2) {
    speed = k.block_n >= 256 ? 0.955 : k.block_n >= 128 ? 0.70 : 0.45;
    if (k.in_type == kE4M3) speed *= 0.97;  // twice the MMA rate: the smaller tile falls back further
  } else {
    speed = k.block_n >= 256 ? 0.895 : k.block_n >= 128 ? 0.62 : 0.40;
  }
  // Time in units of "one SM's share of one output element over one k-block at full speed";
  // measured: 81 000 - 83 000 of them per microsecond at bf16 (a 128 x 256 tile's k-block takes
  // 0.45 us on a lone CTA, a 256 x 256 tile's 0.41 us on a pair).
  const double k_blocks = (double)ceil_div(K, kBlockKBytes / input_bytes(k.in_type));
  const double per_sm_tile = (double)tile_m * (double)k.block_n / (speed * (double)k.cta_group);
  // (a last wave that is run as half tiles -- half_tile_tail() -- takes half as long, and is
  // filled twice as well)
  const bool halves = half_tile_tail((uint32_t)tiles, (uint32_t)slots, k.m_sub) != 0;
  // (A launch that is nothing but half tiles runs them 15 % slower than the one-sub-tile pair
  // kernel runs the same 256-row tiles -- 8192 x 512 x 4096: 33.5 against 29.3 us -- its ring
  // holds four stages with an idle slab each, its accumulators are not double-buffered.)
  const double last_wave = halves ? (waves == 1 ? 0.6 : 0.5) * (0.55 + 0.45 * 2.0 * last_fill)
                                  : 0.55 + 0.45 * last_fill;
  const double mainloop = per_sm_tile * k_blocks * ((double)(waves - 1) + last_wave);
  // What a launch costs besides: set-up, the first loads' latency, the last epilogue, teardown.
  // A pair pays about 2 us more (cluster launch, barriers across the two CTAs): at
  // 8192 x 512 x 4096 128 lone CTAs take 25.6 us and 64 pairs 27.9 us, at 2048^3 15.3 vs 17.4 us,
  // at 1024^3 9.1 vs 11.0 us; from K = 6144 on the pair's faster mainloop wins again (41.8 vs
  // 44.0 us).
  const double fixed = (k.cta_group == 2 ? 8.0 : 6.0) * 82000.0;
  return 1.0e12 / (mainloop + fixed);
}

// Threads of a block: producer and MMA warps, four epilogue warps per accumulator sub-tile, a
// second MMA-issuing warp when there are two sub-tiles or two k-blocks per stage, a scale-producer
// warp when block-scaled (GemmTraits::kThreads).
uint32_t block_threads(int m_sub, bool block_scaled, int k_chunks = 1) {
  return 64u + 128u * (uint32_t)m_sub + ((m_sub == 2 || k_chunks == 2) ? 32u : 0u) + (block_scaled ? 32u : 0u);
}

// Kernels with several k-blocks per stage view an operand as {128 bytes, rows, K / 128 bytes}:
// K must be whole k-blocks (a ragged last k-block cannot be a box of that tensor).
bool chunked_ok(int in_type, int64_t K) { return K % (int64_t)(kBlockKBytes / input_bytes(in_type)) == 0; }

int make_plan(int in_type, int out_type, int64_t M, int64_t N, int64_t K,
              const PatinaGemmConfig* cfg, int num_sms, PatinaGemmPlan* out,
              const KernelEntry** entry_out, std::string* err, bool need_fused = false,
              bool need_scatter = false) {
  if (!type_pair_supported(in_type, out_type)) {
    if (err) *err = fmt("unsupported type pair in=%d out=%d", in_type, out_type);
    return PATINA_GEMM_ERR_INVALID_ARG;
  }
  if (num_sms <= 0) {
    if (err) *err = "num_sms must be positive";
    return PATINA_GEMM_ERR_INVALID_ARG;
  }
  PatinaGemmConfig c{};
  if (cfg) c = *cfg;
  const KernelEntry* best = nullptr;
  if (c.cta_group != 0 || c.block_n != 0 || c.m_sub != 0) {
    // explicit request: fill in whatever was left open with the first match
    for (int i = 0; i < kNumKernels && !best; ++i) {
      const KernelEntry& k = kKernels[i];
      if (k.in_type != in_type || k.out_type != out_type) continue;
      if (c.cta_group != 0 && k.cta_group != c.cta_group) continue;
      if (c.block_n != 0 && k.block_n != c.block_n) continue;
      if (c.stages != 0 && k.stages != c.stages) continue;
      if (k.m_sub != (c.m_sub != 0 ? c.m_sub : 1)) continue;  // explicit requests default to m_sub = 1
      if (k.k_chunks > 1 && (!chunked_ok(in_type, K) || c.k_order == 1)) continue;
      if (need_fused && !k.fn_fused) continue;
      if (need_scatter && !k.fn_scatter) continue;
      best = &k;
    }
    if (!best) {
      if (err)
        *err = fmt("no kernel for cta_group=%d m_sub=%d block_n=%d stages=%d with these types",
                   c.cta_group, c.m_sub, c.block_n, c.stages);
      return PATINA_GEMM_ERR_INVALID_ARG;
    }
  } else {
    double best_score = -1.0;
    for (int i = 0; i < kNumKernels; ++i) {
      const KernelEntry& k = kKernels[i];
      if (k.in_type != in_type || k.out_type != out_type) continue;
      if (c.stages != 0 && k.stages != c.stages) continue;
      if (k.cta_group == 2 && num_sms < 2) continue;
      if (k.k_chunks > 1 && (!chunked_ok(in_type, K) || c.k_order == 1)) continue;
      if (need_fused && !k.fn_fused) continue;
      if (need_scatter && !k.fn_scatter) continue;
      // (Peer destinations: store boxes with 128-byte rows cross NVLink at 0.84 of the plain copy
      // rate, boxes with 64-byte rows at 0.55: measured on two GPUs, 621 vs 408 GB/s out of each
      // GPU, copy 744. Every plain epilogue stages 128-byte rows.)
      const double s = config_score(k, M, N, K, num_sms);
      if (s > best_score) {
        best_score = s;
        best = &k;
      }
    }
    if (!best) {
      if (err) *err = "no kernel matches the requested stage count";
      return PATINA_GEMM_ERR_INVALID_ARG;
    }
  }
  PatinaGemmPlan p{};
  p.cta_group = best->cta_group;
  p.block_n = best->block_n;
  p.stages = best->stages;
  p.m_sub = best->m_sub;
  p.tile_m = 128u * best->cta_group * best->m_sub;
  p.tiles_m = ceil_div(M, p.tile_m);
  p.tiles_n = ceil_div(N, best->block_n);
  p.num_tiles = p.tiles_m * p.tiles_n;
  const uint32_t kelems = kBlockKBytes / input_bytes(in_type);
  p.k_blocks = ceil_div(K, kelems);
  p.group_m = c.group_m > 0 ? c.group_m : 8;
  uint32_t slots = (uint32_t)(num_sms / best->cta_group);
  if (c.max_ctas > 0 && (uint32_t)(c.max_ctas / best->cta_group) < slots)
    slots = (uint32_t)(c.max_ctas / best->cta_group);
  if (slots == 0) slots = 1;
  p.half_tiles = half_tile_tail(p.num_tiles, slots, best->m_sub);
  const uint32_t work = p.num_tiles + p.half_tiles;
  const uint32_t clusters = work < slots ? work : slots;
  p.grid = clusters * best->cta_group;
  p.block = block_threads(best->m_sub, false, best->k_chunks);
  p.cluster = best->cta_group;
  p.smem_bytes = best->smem_bytes;
  const uint32_t acc_cols = (uint32_t)(best->m_sub * best->block_n * (best->k_chunks == 2 ? 2 : 1));
  p.tmem_cols = (2 * acc_cols <= 512 ? 2 : 1) * acc_cols;
  p.tmem_cols = p.tmem_cols <= 256 ? 256 : 512;  // allocation granularity: a power of two
  const SmemPlan sp = smem_plan(best->cta_group, best->m_sub, best->block_n, best->stages,
                                output_bytes(out_type), 0, false, (uint32_t)best->k_chunks);
  p.stage_bytes = sp.stage_bytes;
  p.expect_tx_bytes = sp.stage_bytes * best->cta_group;
  p.idesc = idesc(in_type, 128 * best->cta_group, best->block_n);
  if (out) *out = p;
  if (entry_out) *entry_out = best;
  return PATINA_GEMM_OK;
}

// Argument check shared by every entry point. The diagnostic is formatted into the caller's
// buffer (no heap: the allocation-free entry point uses it as it is).
int validate_args_buf(int in_type, int out_type, const void* A, int64_t lda, const void* B, int64_t ldb,
                      const void* C, int64_t ldc, int64_t M, int64_t N, int64_t K, char* err,
                      size_t err_len) {
  auto fail = [&](const char* f, ...) {
    if (err && err_len) {
      va_list ap;
      va_start(ap, f);
      std::vsnprintf(err, err_len, f, ap);
      va_end(ap);
    }
    return (int)PATINA_GEMM_ERR_INVALID_ARG;
  };
  if (err && err_len) err[0] = '\0';
  if (!type_pair_supported(in_type, out_type))
    return fail("unsupported type pair in=%d out=%d", in_type, out_type);
  if (M < 0 || N < 0 || K < 0)
    return fail("negative dimension M=%lld N=%lld K=%lld", (long long)M, (long long)N, (long long)K);
  if (M > 0x7fffffffLL || N > 0x7fffffffLL || K > 0x7fffffffLL) return fail("dimension exceeds 2^31-1");
  if (M == 0 || N == 0) return PATINA_GEMM_OK;
  if (!C) return fail("C is null");
  const int64_t ib = input_bytes(in_type), ob = output_bytes(out_type);
  if ((reinterpret_cast<uintptr_t>(C) & 15u) != 0) return fail("C is not 16-byte aligned");
  if (ldc < N) return fail("ldc=%lld < N=%lld", (long long)ldc, (long long)N);
  if ((ldc * ob) % 16 != 0) return fail("ldc=%lld: row pitch is not a multiple of 16 bytes", (long long)ldc);
  if (K == 0) return PATINA_GEMM_OK;
  if (!A) return fail("A is null");
  if (!B) return fail("B is null");
  if ((reinterpret_cast<uintptr_t>(A) & 15u) != 0) return fail("A is not 16-byte aligned");
  if ((reinterpret_cast<uintptr_t>(B) & 15u) != 0) return fail("B is not 16-byte aligned");
  if (lda < K) return fail("lda=%lld < K=%lld", (long long)lda, (long long)K);
  if (ldb < K) return fail("ldb=%lld < K=%lld", (long long)ldb, (long long)K);
  if ((lda * ib) % 16 != 0) return fail("lda=%lld: row pitch is not a multiple of 16 bytes", (long long)lda);
  if ((ldb * ib) % 16 != 0) return fail("ldb=%lld: row pitch is not a multiple of 16 bytes", (long long)ldb);
  return PATINA_GEMM_OK;
}

int validate_args(int in_type, int out_type, const void* A, int64_t lda, const void* B, int64_t ldb,
                  const void* C, int64_t ldc, int64_t M, int64_t N, int64_t K, std::string* err) {
  char buf[256];
  const int rc = validate_args_buf(in_type, out_type, A, lda, B, ldb, C, ldc, M, N, K, buf, sizeof(buf));
  if (rc != PATINA_GEMM_OK && err) *err = buf;
  return rc;
}

}  // namespace

// ------------------------------------------------------------------- context
struct TensorMapKey {
  const void* ptr;
  uint64_t rows, cols, ld;
  uint32_t box_rows, box_cols;
  int dtype;  // CUtensorMapDataType
  bool operator==(const TensorMapKey& o) const {
    // (the swizzle mode follows from box_cols * element size: 128 or 64 bytes)
    return ptr == o.ptr && rows == o.rows && cols == o.cols && ld == o.ld &&
           box_rows == o.box_rows && box_cols == o.box_cols && dtype == o.dtype;
  }
};

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

constexpr int kHostChunksMax = 8;
constexpr int kHostEvents = 3 + 2 * kHostChunksMax;

struct PatinaGemmContext {
  int device = 0;
  int num_sms = 0;
  int cc_major = 0, cc_minor = 0;
  uint32_t* d_status = nullptr;  // 4 words
  uint64_t wait_limit_ns = 2000000000ull;
  uint64_t launches = 0;
  std::string last_error;
  EncodeTiledFn encode = nullptr;
  std::vector<std::pair<TensorMapKey, CUtensorMap>> tmaps;  // small most-recent-first cache
  bool smem_attr_set[kNumKernels] = {};
  bool scatter_attr_set[kNumKernels] = {};
  bool grouped_attr_set[kNumGroupedKernels] = {};
  int grouped_max_clusters[kNumGroupedKernels] = {};
  int max_clusters[kNumKernels] = {};  // co-resident clusters per kernel (pairs only)
  // scratch of the stream-K path: fp32 partial tiles and per-tile arrival counters
  float* d_sk_partials = nullptr;
  uint32_t* d_sk_counters = nullptr;
  size_t cap_sk_partials = 0, cap_sk_counters = 0;
  bool sk_attr_set[3] = {false, false, false};
  bool ck_attr_set[3] = {false, false, false};   // cluster split-K kernels (2, 4, 8 CTAs)
  bool mx_attr_set[kNumMxKernels] = {};
  int mx_max_clusters[kNumMxKernels] = {};
  uint32_t sk_burst = 4;
  // copy streams and events of patina_gemm_host's pipelined form
  cudaStream_t s_in = nullptr, s_out = nullptr;
  cudaEvent_t ev[kHostEvents] = {};
  // device staging for patina_gemm_host
  void* d_a = nullptr;
  void* d_b = nullptr;
  void* d_c = nullptr;
  size_t cap_a = 0, cap_b = 0, cap_c = 0;
#ifdef PATINA_TRACE
  unsigned long long* trace = nullptr;  // trace builds only: [grid][32] time stamps of the next launch
  uint32_t l2_hint_a = 0, l2_hint_b = 0;
  PatinaGemmConfig scatter_cfg{};       // trace builds only: tile override for the scatter entry
  bool has_scatter_cfg = false;
#endif
};

namespace {

int set_error(PatinaGemmContext* ctx, int code, const std::string& msg) {
  if (ctx) ctx->last_error = msg;
  return code;
}

// The runtime keeps the last error of any earlier call until somebody reads it. Read (and so
// clear) it before a launch, so that a launch check never reports another call's failure.
void drain_stale_error() { (void)cudaGetLastError(); }

int cuda_fail(PatinaGemmContext* ctx, cudaError_t e, const char* what) {
  return set_error(ctx, PATINA_GEMM_ERR_CUDA,
                   fmt("%s: %s (%s)", what, cudaGetErrorName(e), cudaGetErrorString(e)));
}

struct DeviceGuard {
  int prev = -1;
  bool ok = true;
  explicit DeviceGuard(int dev) {
    if (cudaGetDevice(&prev) != cudaSuccess) prev = -1;
    if (prev != dev) ok = (cudaSetDevice(dev) == cudaSuccess);
  }
  ~DeviceGuard() {
    int cur = -1;
    if (prev >= 0 && cudaGetDevice(&cur) == cudaSuccess && cur != prev) cudaSetDevice(prev);
  }
};

// A K-major matrix [rows, cols] with row pitch ld elements, tiled in boxes of
// box_rows x box_cols where box_cols spans exactly one swizzle span: 128 bytes (128-byte
// swizzle: operands, and C from four-warp epilogues) or 64 bytes (64-byte swizzle: C from
// eight-warp epilogues).
// (The reference's map is 4-D, unswizzled: harness/gemm_check.cpp:127-147.)
int get_tensor_map(PatinaGemmContext* ctx, const void* ptr, CUtensorMapDataType dtype,
                   uint32_t elt_bytes, uint64_t rows, uint64_t cols, uint64_t ld,
                   uint32_t box_rows, uint32_t box_cols, CUtensorMap* out) {
  TensorMapKey key{ptr, rows, cols, ld, box_rows, box_cols, (int)dtype};
  for (size_t i = 0; i < ctx->tmaps.size(); ++i) {
    if (ctx->tmaps[i].first == key) {
      *out = ctx->tmaps[i].second;
      return PATINA_GEMM_OK;
    }
  }
  const uint32_t span = box_cols * elt_bytes;
  if ((span != 128 && span != 64) || box_rows == 0 || box_rows > 256)
    return set_error(ctx, PATINA_GEMM_ERR_INVALID_ARG, "internal: illegal TMA box");
  const cuuint64_t gdim[2] = {cols, rows};
  const cuuint64_t gstride[1] = {ld * elt_bytes};
  const cuuint32_t box[2] = {box_cols, box_rows};
  const cuuint32_t estride[2] = {1, 1};
  CUtensorMap tm;
  CUresult rc = ctx->encode(&tm, dtype, 2, const_cast<void*>(ptr), gdim, gstride, box, estride,
                            CU_TENSOR_MAP_INTERLEAVE_NONE,
                            span == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS)
    return set_error(ctx, PATINA_GEMM_ERR_CUDA,
                     fmt("cuTensorMapEncodeTiled failed (CUresult %d) for %llux%llu ld=%llu", (int)rc,
                         (unsigned long long)rows, (unsigned long long)cols, (unsigned long long)ld));
  if (ctx->tmaps.size() >= 64) ctx->tmaps.pop_back();
  ctx->tmaps.insert(ctx->tmaps.begin(), std::make_pair(key, tm));
  *out = tm;
  return PATINA_GEMM_OK;
}

// The same matrix as a rank-3 tensor {128 bytes of K, rows, K / 128 bytes} (cols must be whole
// 128-byte spans): a box {128 bytes, box_rows, chunks} lands in shared memory as `chunks`
// consecutive [box_rows][128 bytes] slabs, each swizzled like a 2-D box of one k-block.
int get_tensor_map_chunked(PatinaGemmContext* ctx, const void* ptr, CUtensorMapDataType dtype,
                           uint32_t elt_bytes, uint64_t rows, uint64_t cols, uint64_t ld,
                           uint32_t box_rows, uint32_t chunks, CUtensorMap* out) {
  const uint32_t span_elems = kBlockKBytes / elt_bytes;
  TensorMapKey key{ptr, rows, cols, ld, box_rows, span_elems | (chunks << 16), (int)dtype};
  for (size_t i = 0; i < ctx->tmaps.size(); ++i) {
    if (ctx->tmaps[i].first == key) {
      *out = ctx->tmaps[i].second;
      return PATINA_GEMM_OK;
    }
  }
  if (cols % span_elems != 0 || box_rows == 0 || box_rows > 256 || chunks == 0 || chunks > 8)
    return set_error(ctx, PATINA_GEMM_ERR_INVALID_ARG, "internal: illegal 3-D TMA box");
  const cuuint64_t gdim[3] = {span_elems, rows, cols / span_elems};
  const cuuint64_t gstride[2] = {ld * elt_bytes, kBlockKBytes};
  const cuuint32_t box[3] = {span_elems, box_rows, chunks};
  const cuuint32_t estride[3] = {1, 1, 1};
  CUtensorMap tm;
  CUresult rc = ctx->encode(&tm, dtype, 3, const_cast<void*>(ptr), gdim, gstride, box, estride,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS)
    return set_error(ctx, PATINA_GEMM_ERR_CUDA,
                     fmt("cuTensorMapEncodeTiled (rank 3) failed (CUresult %d) for %llux%llu ld=%llu", (int)rc,
                         (unsigned long long)rows, (unsigned long long)cols, (unsigned long long)ld));
  if (ctx->tmaps.size() >= 64) ctx->tmaps.pop_back();
  ctx->tmaps.insert(ctx->tmaps.begin(), std::make_pair(key, tm));
  *out = tm;
  return PATINA_GEMM_OK;
}

CUtensorMapDataType tmap_in_type(int in_type) {
  switch (in_type) {
    case kF16: return CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    case kBF16: return CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    default: return CU_TENSOR_MAP_DATA_TYPE_UINT8;
  }
}


// ------------------------------------------------------------ stream-K path
struct SkPlan {
  uint32_t grid, tiles, k_blocks, m_pad, max_contrib;
  uint64_t units, partial_bytes, counter_bytes;
};

bool streamk_supported(int in_type, int out_type, int64_t M) {
  const bool types = (out_type == kOutBF16 && (in_type == kBF16 || in_type == kE4M3)) ||
                     (out_type == kOutF32 && in_type == kF16);   // the reference's own types
  return types && M >= 1 && M <= 128;
}

constexpr uint64_t kSkMinUnits = 8;

SkPlan make_sk_plan(int in_type, int64_t M, int64_t N, int64_t K, int num_sms) {
  SkPlan s{};
  s.m_pad = (uint32_t)((M + 15) / 16 * 16);
  s.tiles = ceil_div(N, kSkTileRows);
  s.k_blocks = ceil_div(K, kBlockKBytes / input_bytes(in_type));
  s.units = (uint64_t)s.tiles * s.k_blocks;
  // every CTA gets at least kSkMinUnits units, so that its set-up is paid for by some streaming
  const uint64_t want = (s.units + kSkMinUnits - 1) / kSkMinUnits;
  s.grid = (uint32_t)((uint64_t)num_sms < want ? (uint64_t)num_sms : want);
  // Fewer tiles than SMs: cut every tile into the same number of ranges, so that each CTA has one
  // segment of one tile (one accumulator to drain, one partial tile to publish) -- as long as that
  // keeps nine SMs in ten busy.
  if (s.tiles < s.grid) {
    const uint32_t aligned = s.tiles * (s.grid / s.tiles);
    if (aligned * 10u >= s.grid * 9u) s.grid = aligned;
  }
  s.max_contrib = streamk_max_contrib(s.units, s.grid, s.k_blocks);
  s.partial_bytes = (uint64_t)s.tiles * s.max_contrib * s.m_pad * 128ull * sizeof(float);
  s.counter_bytes = (uint64_t)s.tiles * sizeof(uint32_t);
  return s;
}

// The automatic choice between the two kernels for M <= 128.
//  * Many weight tiles (N = 28672, K = 8192): stream-K leads at M <= 16 (75.3 vs 77 us); with
//    32 rows of X it is already behind (80.4 vs 78.3 us) and from M = 64 on the X slab is as large
//    as the W slab and the large-tile kernel, which loads one X slab per 256 rows of W, is well
//    ahead (80.1 vs 89.4 us) -- as long as it has a tile for most SMs.
//  * Few weight tiles (a narrow shard, or the reference's own 128 x 128 x K shape) leave the
//    large-tile kernel on a handful of SMs, each pulling its whole K through one SM's L2 port:
//    128 x 128 x 8192 takes 45 us there and 10 us when K is cut across CTAs (128 x 1024 x 4096:
//    22 vs 9.6 us; 32 x 2048 x 2048: 12.8 vs 8.6 us). Only a short K (16 k-blocks: 8.6 vs 9.2 us)
//    is not worth cutting.
bool streamk_preferred(int in_type, int out_type, int64_t M, int64_t N, int64_t K, int num_sms) {
  if (!streamk_supported(in_type, out_type, M)) return false;
  const SkPlan s = make_sk_plan(in_type, M, N, K, num_sms);
  if (M <= 16 && s.units >= 4ull * (uint64_t)num_sms) return true;
  const uint64_t large_tiles = (uint64_t)ceil_div(N, 256);  // one 128-row tile covers all of M
  const bool starved = large_tiles * 10 < (uint64_t)num_sms * 7;
  return starved && s.k_blocks >= 24;
}

template <int kIn>
cudaError_t launch_sk_kernel(const SkPlan& sp, cudaStream_t stream, const CUtensorMap& tm_w,
                             const CUtensorMap& tm_x, const StreamKParams& p, bool* attr_set) {
  auto fn = gemm_streamk_kernel<kIn>;
  const uint32_t smem = streamk_smem_bytes(p.m_pad);
  if (!*attr_set) {
    cudaError_t e = cudaFuncSetAttribute(reinterpret_cast<const void*>(fn),
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)kMaxDynSmem);
    if (e != cudaSuccess) return e;
    *attr_set = true;
  }
  fn<<<sp.grid, 192, smem, stream>>>(tm_w, tm_x, p);
  cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess && p.split_reduce) {
    cudaLaunchConfig_t lc{};
    lc.gridDim = dim3(sp.tiles * (p.m_pad / 16u), 1, 1);
    lc.blockDim = dim3(128, 1, 1);
    lc.dynamicSmemBytes = 0;
    lc.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    lc.attrs = attr;
    lc.numAttrs = 1;
    e = cudaLaunchKernelEx(&lc, streamk_reduce_kernel, p, (uint32_t)sp.grid);
  }
  return e;
}

int launch_streamk(PatinaGemmContext* ctx, int in_type, const void* A, int64_t lda, const void* B,
                   int64_t ldb, void* C, int64_t ldc, int64_t M, int64_t N, int64_t K, float alpha,
                   cudaStream_t stream, int reduce_mode = 0, bool out_f32 = false) {
  const SkPlan sp = make_sk_plan(in_type, M, N, K, ctx->num_sms);
  // scratch: grow-only; counters start (and are left) at zero
  if (ctx->cap_sk_partials < sp.partial_bytes) {
    if (ctx->d_sk_partials) cudaFree(ctx->d_sk_partials);
    ctx->d_sk_partials = nullptr;
    ctx->cap_sk_partials = 0;
    cudaError_t e = cudaMalloc(reinterpret_cast<void**>(&ctx->d_sk_partials), sp.partial_bytes);
    if (e != cudaSuccess) return cuda_fail(ctx, e, "cudaMalloc(stream-K partials)");
    ctx->cap_sk_partials = sp.partial_bytes;
  }
  if (ctx->cap_sk_counters < sp.counter_bytes) {
    if (ctx->d_sk_counters) cudaFree(ctx->d_sk_counters);
    ctx->d_sk_counters = nullptr;
    ctx->cap_sk_counters = 0;
    cudaError_t e = cudaMalloc(reinterpret_cast<void**>(&ctx->d_sk_counters), sp.counter_bytes);
    if (e == cudaSuccess) e = cudaMemset(ctx->d_sk_counters, 0, sp.counter_bytes);
    if (e != cudaSuccess) return cuda_fail(ctx, e, "cudaMalloc(stream-K counters)");
    ctx->cap_sk_counters = sp.counter_bytes;
  }
  const uint32_t ib = input_bytes(in_type);
  const uint32_t kelems = kBlockKBytes / ib;
  CUtensorMap tm_w, tm_x;
  int rc = get_tensor_map(ctx, B, tmap_in_type(in_type), ib, (uint64_t)N, (uint64_t)K, (uint64_t)ldb,
                          kSkTileRows, kelems, &tm_w);
  if (rc != PATINA_GEMM_OK) return rc;
  rc = get_tensor_map(ctx, A, tmap_in_type(in_type), ib, (uint64_t)M, (uint64_t)K, (uint64_t)lda,
                      sp.m_pad, kelems, &tm_x);
  if (rc != PATINA_GEMM_OK) return rc;
  drain_stale_error();
  StreamKParams p{};
  p.M = (uint32_t)M;
  p.N = (uint32_t)N;
  p.K = (uint32_t)K;
  p.m_pad = sp.m_pad;
  p.tiles = sp.tiles;
  p.k_blocks = sp.k_blocks;
  p.units = sp.units;
  p.max_contrib = sp.max_contrib;
  p.stages = streamk_stages(sp.m_pad);
  p.stage_stride = streamk_stage_stride(sp.m_pad);
  p.burst = ctx->sk_burst < p.stages / 2 ? ctx->sk_burst : p.stages / 2;
  p.alpha = alpha;
  p.C = C;
  p.out_f32 = out_f32 ? 1u : 0u;
  p.ldc = ldc;
  p.partials = ctx->d_sk_partials;
  p.counters = ctx->d_sk_counters;
  // Shared tiles are summed by a second small kernel that every SM takes part in: one finishing
  // CTA per tile pulling every contributor's partial tile through its own SM was measured at 15 us
  // for M = 128 (16 KB and more per contributor), and for 16 rows of X it is still behind
  // (16 x 3584 x 8192: 17.5 against 16.8 us; 16 x 28672 x 8192: 79.0 against 78.7).
  p.split_reduce = sp.grid > 1u ? 1u : 0u;
  if (reduce_mode == 2) p.split_reduce = 1u;  // explicit request (PatinaGemmConfig::stream_k = 2 / 3)
  if (reduce_mode == 3) p.split_reduce = 0u;
  // No tile is shared (every CTA boundary is a tile boundary): nothing to sum, no second kernel.
  if (p.split_reduce && !streamk_any_shared_tile(sp.units, sp.grid, sp.k_blocks)) p.split_reduce = 0u;
  p.status = ctx->d_status;
  p.wait_limit_ns = ctx->wait_limit_ns;
#ifdef PATINA_TRACE
  p.trace = ctx->trace;
#endif
  cudaError_t e = (in_type == kBF16)   ? launch_sk_kernel<kBF16>(sp, stream, tm_w, tm_x, p, &ctx->sk_attr_set[0])
                  : (in_type == kE4M3) ? launch_sk_kernel<kE4M3>(sp, stream, tm_w, tm_x, p, &ctx->sk_attr_set[1])
                                       : launch_sk_kernel<kF16>(sp, stream, tm_w, tm_x, p, &ctx->sk_attr_set[2]);
  if (e != cudaSuccess) return cuda_fail(ctx, e, "stream-K launch");
  ctx->launches += p.split_reduce ? 2 : 1;
  return PATINA_GEMM_OK;
}

// ------------------------------------------------ K cut across a cluster (few tiles, deep K)
// One cluster of S (2 or 4) CTAs per 128 x 256 tile, each CTA taking 1/S of the k-blocks; the partial tiles
// are summed through distributed shared memory (patina_gemm_splitk.cuh). Measured facts behind
// the choice: a 128-byte k-block costs a CTA about 560 cycles (0.3 us) whatever the tile width (a
// tcgen05.mma of 128 rows takes its 128 cycles whether it has 64 or 256 columns), so a problem
// with few tiles only gets faster by giving each CTA fewer k-blocks; the cluster launch, the
// exchange and its barriers cost 3 us (two CTAs) to 6 us (four), i.e. kClusterKMinSaved k-blocks
// must be saved per CTA before the cut pays (1024 x 2048 x 2048: 12.4 vs 14.5 us;
// 256 x 4096 x 4096: 15.8 vs 23.2 us; 512 x 512 x 4096: 13.0 vs 22.0 us; but 1024^3: 9.4 vs 8.7 us).
constexpr uint32_t kClusterKMinSaved = 16;

bool cluster_k_supported(int in_type, int out_type, int64_t M, int64_t N, int64_t K, int split) {
  if (in_type != kBF16 || out_type != kOutBF16) return false;
  if (split != 2 && split != 4) return false;
  if (M < 1 || N < 1 || (N % 8) != 0) return false;               // whole 16-byte pieces in every store box
  return (int64_t)ceil_div(K, kBlockKBytes / 2) >= split;          // every CTA gets at least one k-block
}

// 0: do not split; else the cluster size.
int cluster_k_choice(int in_type, int out_type, int64_t M, int64_t N, int64_t K, int num_sms) {
  if (M <= 128) return 0;                                          // the skinny paths cover these
  // Only where even 128 x 64 tiles leave a third of the SMs without one: the two-accumulator
  // single-CTA kernels run a k-block in 0.16 us whatever their width, and from 1024 x 1024 x 4096
  // on (128 such tiles) they are ahead of the split (15.4 against 16.0 us; 1024 x 2048 x 2048:
  // 10.7 against 12.8), while 512 x 512 x 4096 (32 tiles) is 13.1 us split and 14.3 whole, and
  // 512 x 1024 x 8192 (64 tiles) 18.4 and 25.0.
  if ((uint64_t)ceil_div(M, kCtaRows) * ceil_div(N, 64) * 3 > (uint64_t)num_sms * 2) return 0;
  const uint64_t tiles = (uint64_t)ceil_div(M, kCtaRows) * ceil_div(N, kSplitBN);
  const uint32_t kb = ceil_div(K, kBlockKBytes / 2);
  for (int split = 4; split >= 2; split /= 2) {
    if (!cluster_k_supported(in_type, out_type, M, N, K, split)) continue;
    if (tiles * (uint64_t)split > (uint64_t)num_sms) continue;     // one wave of clusters
    const uint32_t saved = kb - kb / (uint32_t)split;              // k-blocks every CTA no longer runs
    if (saved >= kClusterKMinSaved && kb / (uint32_t)split >= 2u) return split;
  }
  return 0;
}

int launch_cluster_k(PatinaGemmContext* ctx, const void* A, int64_t lda, const void* B, int64_t ldb, void* C,
                     int64_t ldc, int64_t M, int64_t N, int64_t K, float alpha, int split, int group_m,
                     cudaStream_t stream) {
  CUtensorMap tm_a, tm_b, tm_c;
  const uint32_t kelems = kBlockKBytes / 2;
  int rc = get_tensor_map(ctx, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)M, (uint64_t)K, (uint64_t)lda,
                          kCtaRows, kelems, &tm_a);
  if (rc != PATINA_GEMM_OK) return rc;
  rc = get_tensor_map(ctx, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, kSplitBN,
                      kelems, &tm_b);
  if (rc != PATINA_GEMM_OK) return rc;
  rc = get_tensor_map(ctx, C, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)M, (uint64_t)N, (uint64_t)ldc,
                      kStoreBoxRows, 32, &tm_c);
  if (rc != PATINA_GEMM_OK) return rc;
  using Fn = void (*)(const CUtensorMap, const CUtensorMap, const CUtensorMap, const GemmParams);
  const Fn fn = split == 2 ? gemm_splitk_cluster_kernel<2> : gemm_splitk_cluster_kernel<4>;
  const int fi = split == 2 ? 0 : 1;
  if (!ctx->ck_attr_set[fi]) {
    cudaError_t e = cudaFuncSetAttribute(reinterpret_cast<const void*>(fn), cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)splitk_smem_bytes());
    if (e != cudaSuccess) return cuda_fail(ctx, e, "cudaFuncSetAttribute(smem, cluster split-K)");
    ctx->ck_attr_set[fi] = true;
  }
  GemmParams p{};
  p.M = (uint32_t)M;
  p.N = (uint32_t)N;
  p.K = (uint32_t)K;
  p.tiles_m = ceil_div(M, kCtaRows);
  p.tiles_n = ceil_div(N, kSplitBN);
  p.num_tiles = p.tiles_m * p.tiles_n;
  p.k_blocks = ceil_div(K, kelems);
  p.group_m = group_m > 0 ? (uint32_t)group_m : 8u;
  p.alpha = alpha;
  p.n_dests = 1;
  p.c_dests[0] = C;
  p.ldc = ldc;
  p.status = ctx->d_status;
  p.wait_limit_ns = ctx->wait_limit_ns;
#ifdef PATINA_TRACE
  p.trace = ctx->trace;
  p.l2_hint_a = p.l2_hint_b = 0;
#endif
  cudaLaunchConfig_t lc{};
  lc.gridDim = dim3(p.num_tiles * (uint32_t)split, 1, 1);
  lc.blockDim = dim3(192, 1, 1);
  lc.dynamicSmemBytes = splitk_smem_bytes();
  lc.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)split;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  lc.attrs = attr;
  lc.numAttrs = 1;
  drain_stale_error();
  cudaError_t e = cudaLaunchKernelEx(&lc, fn, tm_a, tm_b, tm_c, p);
  if (e != cudaSuccess) return cuda_fail(ctx, e, "cudaLaunchKernelEx(cluster split-K)");
  ctx->launches += 1;
  return PATINA_GEMM_OK;
}

// Clusters of this kernel that can be resident at once (cached per kernel). A persistent grid
// must not exceed it, or the late clusters would start their tile lists after the others finish.
int resident_clusters(const KernelEntry* k, int num_sms, int* cache) {
  if (*cache != 0) return *cache;
  cudaLaunchConfig_t qc{};
  qc.gridDim = dim3((unsigned)(num_sms / k->cta_group) * k->cta_group, 1, 1);
  qc.blockDim = dim3(block_threads(k->m_sub, k->in_type == kMXE4M3), 1, 1);
  qc.dynamicSmemBytes = k->smem_bytes;
  cudaLaunchAttribute qa[1];
  qa[0].id = cudaLaunchAttributeClusterDimension;
  qa[0].val.clusterDim.x = (unsigned)k->cta_group;
  qa[0].val.clusterDim.y = 1;
  qa[0].val.clusterDim.z = 1;
  qc.attrs = qa;
  qc.numAttrs = 1;
  int n = 0;
  cudaError_t qe = cudaOccupancyMaxActiveClusters(&n, reinterpret_cast<const void*>(k->fn), &qc);
  if (qe != cudaSuccess || n <= 0) {
    cudaGetLastError();
    n = num_sms / k->cta_group;
  }
  *cache = n;
  return n;
}

int launch_gemm(PatinaGemmContext* ctx, int in_type, int out_type, const void* A, int64_t lda,
                const void* B, int64_t ldb, void* C, int64_t ldc, int64_t M, int64_t N, int64_t K,
                float alpha, const PatinaGemmConfig* cfg, cudaStream_t stream,
                void* const* extra_dests = nullptr, int n_extra = 0,
                const PatinaGemmEpilogue* epi = nullptr, float out_scale = 1.0f,
                float* amax = nullptr) {
  if (!ctx) return PATINA_GEMM_ERR_INVALID_ARG;
  std::string err;
  int rc = validate_args(in_type, out_type, A, lda, B, ldb, C, ldc, M, N, K, &err);
  if (rc != PATINA_GEMM_OK) return set_error(ctx, rc, err);
  if (n_extra < 0 || n_extra > kMaxDests - 1 || (n_extra > 0 && !extra_dests))
    return set_error(ctx, PATINA_GEMM_ERR_INVALID_ARG, "bad destination list");
  for (int d = 0; d < n_extra; ++d)
    if (!extra_dests[d] || (reinterpret_cast<uintptr_t>(extra_dests[d]) & 15u) != 0)
      return set_error(ctx, PATINA_GEMM_ERR_INVALID_ARG, "a destination of C is null or not 16-byte aligned");
  if (M == 0 || N == 0) return PATINA_GEMM_OK;
  DeviceGuard guard(ctx->device);
  if (!guard.ok) return set_error(ctx, PATINA_GEMM_ERR_CUDA, "cudaSetDevice failed");
  const uint32_t ob = output_bytes(out_type);
  if (K == 0) {
    cudaError_t e = cudaMemset2DAsync(C, (size_t)ldc * ob, 0, (size_t)N * ob, (size_t)M, stream);
    if (e != cudaSuccess) return cuda_fail(ctx, e, "cudaMemset2DAsync");
    return PATINA_GEMM_OK;
  }
  const int want_sk = cfg ? cfg->stream_k : 0;
  if (want_sk > 0 && !streamk_supported(in_type, out_type, M))
    return set_error(ctx, PATINA_GEMM_ERR_INVALID_ARG,
                     "stream_k needs M <= 128 and bf16 or e4m3 inputs with bf16 output, or f16 inputs with f32 output");
  const bool explicit_tile = cfg && (cfg->cta_group != 0 || cfg->block_n != 0 || cfg->m_sub != 0);
  if (n_extra == 0 && epi == nullptr &&
      (want_sk > 0 || (want_sk == 0 && !explicit_tile &&
                       streamk_preferred(in_type, out_type, M, N, K, ctx->num_sms))))
    return launch_streamk(ctx, in_type, A, lda, B, ldb, C, ldc, M, N, K, alpha, stream, want_sk, out_type == kOutF32);
  const int want_ck = cfg ? cfg->cluster_k : 0;
  if (want_ck > 0 && (n_extra > 0 || epi != nullptr || explicit_tile ||
                      !cluster_k_supported(in_type, out_type, M, N, K, want_ck)))
    return set_error(ctx, PATINA_GEMM_ERR_INVALID_ARG,
                     "cluster_k needs bf16 in and out, 2 or 4 CTAs, at least that many 128-byte k-blocks, "
                     "N a multiple of 8, the plain epilogue and no explicit tile");
  if (n_extra == 0 && epi == nullptr && !explicit_tile && want_ck >= 0 && want_sk <= 0 &&
      !(cfg && cfg->k_order == 1 && want_ck == 0)) {
    const int split = want_ck > 0 ? want_ck : cluster_k_choice(in_type, out_type, M, N, K, ctx->num_sms);
    if (split >= 2)
      return launch_cluster_k(ctx, A, lda, B, ldb, C, ldc, M, N, K, alpha, split, cfg ? cfg->group_m : 0, stream);
  }
  PatinaGemmPlan plan;
  const KernelEntry* k = nullptr;
  rc = make_plan(in_type, out_type, M, N, K, cfg, ctx->num_sms, &plan, &k, &err, epi != nullptr,
                 n_extra > 0);
  if (rc != PATINA_GEMM_OK) return set_error(ctx, rc, err);

  const uint32_t ib = input_bytes(in_type);
  const uint32_t kelems = kBlockKBytes / ib;
  CUtensorMap tm_a, tm_b;
  CStoreMaps<kMaxDests> tm_c;
  // One TMA box per operand slab and stage: a 128-row slab of A, this CTA's rows of B.
  const uint32_t a_box = kCtaRows, b_box = (uint32_t)(k->block_n / k->cta_group);
  if (k->k_chunks > 1) {
    rc = get_tensor_map_chunked(ctx, A, tmap_in_type(in_type), ib, (uint64_t)M, (uint64_t)K, (uint64_t)lda,
                                a_box, (uint32_t)k->k_chunks, &tm_a);
    if (rc != PATINA_GEMM_OK) return rc;
    rc = get_tensor_map_chunked(ctx, B, tmap_in_type(in_type), ib, (uint64_t)N, (uint64_t)K, (uint64_t)ldb,
                                b_box, (uint32_t)k->k_chunks, &tm_b);
  } else {
    rc = get_tensor_map(ctx, A, tmap_in_type(in_type), ib, (uint64_t)M, (uint64_t)K, (uint64_t)lda,
                        a_box, kelems, &tm_a);
    if (rc != PATINA_GEMM_OK) return rc;
    rc = get_tensor_map(ctx, B, tmap_in_type(in_type), ib, (uint64_t)N, (uint64_t)K, (uint64_t)ldb,
                        b_box, kelems, &tm_b);
  }
  if (rc != PATINA_GEMM_OK) return rc;
  for (int d = 0; d <= n_extra; ++d) {
    rc = get_tensor_map(ctx, d == 0 ? C : extra_dests[d - 1],
                        out_type == kOutF32    ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                        : out_type == kOutE4M3 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                               : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16,
                        ob, (uint64_t)M, (uint64_t)N, (uint64_t)ldc, kStoreBoxRows,
                        staging_row_bytes((uint32_t)k->m_sub, ob, epi != nullptr) / ob, &tm_c.map[d]);
    if (rc != PATINA_GEMM_OK) return rc;
  }
  for (int d = n_extra + 1; d < kMaxDests; ++d) tm_c.map[d] = tm_c.map[0];

  const int ki = (int)(k - kKernels);
  if (!ctx->smem_attr_set[ki]) {
    cudaError_t e = cudaFuncSetAttribute(reinterpret_cast<const void*>(k->fn),
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)k->smem_bytes);
    if (e == cudaSuccess && k->fn_fused)
      e = cudaFuncSetAttribute(reinterpret_cast<const void*>(k->fn_fused),
                               cudaFuncAttributeMaxDynamicSharedMemorySize, (int)k->smem_bytes);
    if (e != cudaSuccess) return cuda_fail(ctx, e, "cudaFuncSetAttribute(smem)");
    ctx->smem_attr_set[ki] = true;
  }

  if (k->cta_group > 1) {
    const uint32_t cap = (uint32_t)resident_clusters(k, ctx->num_sms, &ctx->max_clusters[ki]);
    const uint32_t slots = (uint32_t)(ctx->num_sms / k->cta_group);
    if (cap < slots) {
      // fewer clusters fit than the plan assumed: the waves, and with them the tail, change
      uint32_t clusters = cap;
      if (cfg && cfg->max_ctas > 0 && (uint32_t)(cfg->max_ctas / k->cta_group) < clusters)
        clusters = (uint32_t)(cfg->max_ctas / k->cta_group);
      if (clusters == 0) clusters = 1;
      plan.half_tiles = half_tile_tail(plan.num_tiles, clusters, k->m_sub);
      const uint32_t work = plan.num_tiles + plan.half_tiles;
      plan.grid = (work < clusters ? work : clusters) * k->cta_group;
    }
  }

  GemmParams p{};
  p.M = (uint32_t)M;
  p.N = (uint32_t)N;
  p.K = (uint32_t)K;
  p.tiles_m = plan.tiles_m;
  p.tiles_n = plan.tiles_n;
  p.num_tiles = plan.num_tiles + plan.half_tiles;   // scheduler indices
  p.split_from = plan.num_tiles - plan.half_tiles;
  p.k_blocks = plan.k_blocks;
  p.group_m = (uint32_t)plan.group_m;
  p.alpha = alpha;
  KernelFn fn = k->fn;
  if (epi) {
    if (!k->fn_fused) return set_error(ctx, PATINA_GEMM_ERR_INVALID_ARG, "no fused-epilogue kernel for these types");
    fn = k->fn_fused;
    p.bias = static_cast<const float*>(epi->bias);
    p.residual = static_cast<const __nv_bfloat16*>(epi->residual);
    p.ldr = epi->ldr;
    p.beta = epi->beta;
    p.activation = (uint32_t)epi->activation;
  }
  p.n_dests = (uint32_t)(1 + n_extra);
  p.c_dests[0] = C;
  for (int d = 0; d < n_extra; ++d) p.c_dests[d + 1] = extra_dests[d];
  p.ldc = ldc;
  p.out_scale = out_scale;
  p.amax = amax;
  p.status = ctx->d_status;
  p.wait_limit_ns = ctx->wait_limit_ns;
#ifdef PATINA_TRACE
  p.trace = ctx->trace;
  p.l2_hint_a = ctx->l2_hint_a;
  p.l2_hint_b = ctx->l2_hint_b;
#endif

  cudaLaunchConfig_t lc{};
  lc.gridDim = dim3(plan.grid, 1, 1);
  lc.blockDim = dim3(plan.block, 1, 1);
  lc.dynamicSmemBytes = k->smem_bytes;
  lc.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)k->cta_group;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  lc.attrs = attr;
  lc.numAttrs = (k->cta_group > 1) ? 1 : 0;
  drain_stale_error();
  cudaError_t e;
  if (n_extra > 0) {
    // the scatter's own instantiation: the only one whose parameters carry kMaxDests store maps
    if (!ctx->scatter_attr_set[ki]) {
      e = cudaFuncSetAttribute(reinterpret_cast<const void*>(k->fn_scatter),
                               cudaFuncAttributeMaxDynamicSharedMemorySize, (int)k->smem_bytes);
      if (e != cudaSuccess) return cuda_fail(ctx, e, "cudaFuncSetAttribute(smem, scatter)");
      ctx->scatter_attr_set[ki] = true;
    }
    e = cudaLaunchKernelEx(&lc, k->fn_scatter, tm_a, tm_b, tm_c, p);
  } else {
    CStoreMaps<1> one;
    one.map[0] = tm_c.map[0];
    e = cudaLaunchKernelEx(&lc, fn, tm_a, tm_b, one, p);
  }
  if (e != cudaSuccess) return cuda_fail(ctx, e, "cudaLaunchKernelEx");
  ctx->launches += 1;
  return PATINA_GEMM_OK;
}

// The scale buffer of a [rows, K] operand as a 2-D tensor of 32-bit words: one 512-byte atom per
// line, lines in (row block, k atom) order. One box = one atom.
int get_scale_tensor_map(PatinaGemmContext* ctx, const void* ptr, uint64_t atoms, CUtensorMap* out) {
  TensorMapKey key{ptr, atoms, 128, 128, 1, 128, (int)CU_TENSOR_MAP_DATA_TYPE_UINT32};
  for (size_t i = 0; i < ctx->tmaps.size(); ++i) {
    if (ctx->tmaps[i].first == key) {
      *out = ctx->tmaps[i].second;
      return PATINA_GEMM_OK;
    }
  }
  const cuuint64_t gdim[2] = {128, atoms};
  const cuuint64_t gstride[1] = {kSfAtomBytes};
  const cuuint32_t box[2] = {128, 1};
  const cuuint32_t estride[2] = {1, 1};
  CUtensorMap tm;
  CUresult rc = ctx->encode(&tm, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(ptr), gdim, gstride, box,
                            estride, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS)
    return set_error(ctx, PATINA_GEMM_ERR_CUDA,
                     fmt("cuTensorMapEncodeTiled failed (CUresult %d) for a scale buffer of %llu atoms", (int)rc,
                         (unsigned long long)atoms));
  if (ctx->tmaps.size() >= 64) ctx->tmaps.pop_back();
  ctx->tmaps.insert(ctx->tmaps.begin(), std::make_pair(key, tm));
  *out = tm;
  return PATINA_GEMM_OK;
}

// Same scoring as the other types, on the block-scaled table.
const MxKernelEntry* pick_mx_kernel(int64_t M, int64_t N, int64_t K, const PatinaGemmConfig* cfg, int num_sms) {
  const bool explicit_tile = cfg && (cfg->cta_group != 0 || cfg->block_n != 0 || cfg->m_sub != 0);
  const MxKernelEntry* best = nullptr;
  double best_score = -1.0;
  for (int i = 0; i < kNumMxKernels; ++i) {
    const MxKernelEntry& k = kMxKernels[i];
    if (explicit_tile) {
      if (cfg->cta_group != 0 && k.cta_group != cfg->cta_group) continue;
      if (cfg->block_n != 0 && k.block_n != cfg->block_n) continue;
      if (k.m_sub != (cfg->m_sub != 0 ? cfg->m_sub : 1)) continue;
      return &k;
    }
    if (k.cta_group == 2 && num_sms < 2) continue;
    KernelEntry as{k.cta_group, k.m_sub, k.block_n, k.stages, kE4M3, kOutBF16, nullptr, nullptr, nullptr, 0};
    double s = config_score(as, M, N, K, num_sms);
    if (k.block_n == 256) s *= 0.93;  // one accumulator: the epilogue is not hidden
    if (s > best_score) {
      best_score = s;
      best = &k;
    }
  }
  return best;
}

int launch_mx(PatinaGemmContext* ctx, const void* A, int64_t lda, const void* sfa, const void* B, int64_t ldb,
              const void* sfb, void* C, int64_t ldc, int64_t M, int64_t N, int64_t K, float alpha,
              const PatinaGemmConfig* cfg, cudaStream_t stream) {
  if (!ctx) return PATINA_GEMM_ERR_INVALID_ARG;
  std::string err;
  int rc = validate_args(kMXE4M3, kOutBF16, A, lda, B, ldb, C, ldc, M, N, K, &err);
  if (rc != PATINA_GEMM_OK) return set_error(ctx, rc, err);
  if (M == 0 || N == 0) return PATINA_GEMM_OK;
  if (K % kSfBlockElems != 0)
    return set_error(ctx, PATINA_GEMM_ERR_INVALID_ARG,
                     fmt("K=%lld: block-scaled operands need K to be a multiple of 32", (long long)K));
  DeviceGuard guard(ctx->device);
  if (!guard.ok) return set_error(ctx, PATINA_GEMM_ERR_CUDA, "cudaSetDevice failed");
  if (K == 0) {
    cudaError_t e = cudaMemset2DAsync(C, (size_t)ldc * 2, 0, (size_t)N * 2, (size_t)M, stream);
    if (e != cudaSuccess) return cuda_fail(ctx, e, "cudaMemset2DAsync");
    return PATINA_GEMM_OK;
  }
  if (!sfa || !sfb || (reinterpret_cast<uintptr_t>(sfa) & 15u) || (reinterpret_cast<uintptr_t>(sfb) & 15u))
    return set_error(ctx, PATINA_GEMM_ERR_INVALID_ARG, "a scale buffer is null or not 16-byte aligned");
  const MxKernelEntry* k = pick_mx_kernel(M, N, K, cfg, ctx->num_sms);
  if (!k) return set_error(ctx, PATINA_GEMM_ERR_INVALID_ARG, "no block-scaled kernel for this tile request");
  const int ki = (int)(k - kMxKernels);

  const uint32_t kelems = kBlockKBytes;  // one byte per element
  const uint32_t tile_m = 128u * k->cta_group * k->m_sub;
  CUtensorMap tm_a, tm_b, tm_sfa, tm_sfb;
  CStoreMaps<1> tm_c;
  rc = get_tensor_map(ctx, A, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)M, (uint64_t)K, (uint64_t)lda, kCtaRows,
                      kelems, &tm_a);
  if (rc != PATINA_GEMM_OK) return rc;
  rc = get_tensor_map(ctx, B, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)N, (uint64_t)K, (uint64_t)ldb,
                      (uint32_t)(k->block_n / k->cta_group), kelems, &tm_b);
  if (rc != PATINA_GEMM_OK) return rc;
  rc = get_tensor_map(ctx, C, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)M, (uint64_t)N, (uint64_t)ldc,
                      kStoreBoxRows, staging_row_bytes((uint32_t)k->m_sub, 2) / 2, &tm_c.map[0]);
  if (rc != PATINA_GEMM_OK) return rc;
  rc = get_scale_tensor_map(ctx, sfa, mx_scale_atoms((uint64_t)M, (uint64_t)K), &tm_sfa);
  if (rc != PATINA_GEMM_OK) return rc;
  rc = get_scale_tensor_map(ctx, sfb, mx_scale_atoms((uint64_t)N, (uint64_t)K), &tm_sfb);
  if (rc != PATINA_GEMM_OK) return rc;

  if (!ctx->mx_attr_set[ki]) {
    cudaError_t e = cudaFuncSetAttribute(reinterpret_cast<const void*>(k->fn),
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)k->smem_bytes);
    if (e != cudaSuccess) return cuda_fail(ctx, e, "cudaFuncSetAttribute(smem, block-scaled)");
    ctx->mx_attr_set[ki] = true;
  }
  GemmParams p{};
  p.M = (uint32_t)M;
  p.N = (uint32_t)N;
  p.K = (uint32_t)K;
  p.tiles_m = ceil_div(M, tile_m);
  p.tiles_n = ceil_div(N, k->block_n);
  p.num_tiles = p.tiles_m * p.tiles_n;
  p.k_blocks = ceil_div(K, kelems);
  p.group_m = (cfg && cfg->group_m > 0) ? (uint32_t)cfg->group_m : 8u;
  p.alpha = alpha;
  p.n_dests = 1;
  p.c_dests[0] = C;
  p.ldc = ldc;
  p.sf_m_blocks = ceil_div(M, kSfAtomRows);
  p.sf_n_blocks = ceil_div(N, kSfAtomRows);
  p.sf_k_atoms = ceil_div(K, 128);
  p.status = ctx->d_status;
  p.wait_limit_ns = ctx->wait_limit_ns;
#ifdef PATINA_TRACE
  p.trace = ctx->trace;
  p.l2_hint_a = p.l2_hint_b = 0;
#endif
  uint32_t slots = (uint32_t)(ctx->num_sms / k->cta_group);
  if (k->cta_group > 1) {
    KernelEntry as{k->cta_group, k->m_sub, k->block_n, k->stages, kMXE4M3, kOutBF16,
                   reinterpret_cast<KernelFn>(k->fn), nullptr, nullptr, k->smem_bytes};
    const uint32_t cap = (uint32_t)resident_clusters(&as, ctx->num_sms, &ctx->mx_max_clusters[ki]);
    if (cap < slots) slots = cap;
  }
  if (cfg && cfg->max_ctas > 0 && (uint32_t)(cfg->max_ctas / k->cta_group) < slots)
    slots = (uint32_t)(cfg->max_ctas / k->cta_group);
  if (slots == 0) slots = 1;
  const uint32_t halves = half_tile_tail(p.num_tiles, slots, k->m_sub);
  p.split_from = p.num_tiles - halves;
  p.num_tiles += halves;   // scheduler indices
  const uint32_t clusters = p.num_tiles < slots ? p.num_tiles : slots;

  cudaLaunchConfig_t lc{};
  lc.gridDim = dim3(clusters * k->cta_group, 1, 1);
  lc.blockDim = dim3(block_threads(k->m_sub, true), 1, 1);
  lc.dynamicSmemBytes = k->smem_bytes;
  lc.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)k->cta_group;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  lc.attrs = attr;
  lc.numAttrs = (k->cta_group > 1) ? 1 : 0;
  drain_stale_error();
  cudaError_t e = cudaLaunchKernelEx(&lc, k->fn, tm_a, tm_b, tm_c, tm_sfa, tm_sfb, p);
  if (e != cudaSuccess) return cuda_fail(ctx, e, "cudaLaunchKernelEx(block-scaled)");
  ctx->launches += 1;
  return PATINA_GEMM_OK;
}

// One launch for n_groups GEMMs that share N and K: A and C hold the groups' rows one after
// another, B one [N, K] block per group, the row counts live in device memory.
int launch_grouped(PatinaGemmContext* ctx, int in_type, const void* A, int64_t lda, const void* B,
                   int64_t ldb, void* C, int64_t ldc, const int32_t* group_rows, int n_groups,
                   int64_t total_rows, int64_t N, int64_t K, float alpha, const float* group_alpha,
                   const PatinaGemmConfig* cfg, cudaStream_t stream) {
  if (!ctx) return PATINA_GEMM_ERR_INVALID_ARG;
  if (n_groups < 0 || n_groups > (int)kMaxGroups)
    return set_error(ctx, PATINA_GEMM_ERR_INVALID_ARG,
                     fmt("n_groups=%d: a grouped launch takes 0..%u groups", n_groups, kMaxGroups));
  if (n_groups > 0 && !group_rows)
    return set_error(ctx, PATINA_GEMM_ERR_INVALID_ARG, "group_rows is null");
  if ((int64_t)n_groups * N > 0x7fffffffLL)
    return set_error(ctx, PATINA_GEMM_ERR_INVALID_ARG, "n_groups * N exceeds 2^31-1");
  std::string err;
  // A is [total_rows, K]; B is [n_groups * N, K]; C is [total_rows, N]
  int rc = validate_args(in_type, kOutBF16, A, lda, B, ldb, C, ldc, total_rows, N, K, &err);
  if (rc != PATINA_GEMM_OK) return set_error(ctx, rc, err);
  if (group_alpha && (reinterpret_cast<uintptr_t>(group_alpha) & 3u))
    return set_error(ctx, PATINA_GEMM_ERR_INVALID_ARG, "the per-group factors are not 4-byte aligned");
  if (total_rows == 0 || N == 0 || n_groups == 0) return PATINA_GEMM_OK;
  DeviceGuard guard(ctx->device);
  if (!guard.ok) return set_error(ctx, PATINA_GEMM_ERR_CUDA, "cudaSetDevice failed");
  if (K == 0) {
    cudaError_t e = cudaMemset2DAsync(C, (size_t)ldc * 2, 0, (size_t)N * 2, (size_t)total_rows, stream);
    if (e != cudaSuccess) return cuda_fail(ctx, e, "cudaMemset2DAsync");
    return PATINA_GEMM_OK;
  }
  // The row counts are on the device, so the tile shape follows the average group: a tall tile
  // wastes up to a tile of rows at every group's end.
  const int64_t avg = total_rows / n_groups;
  int want_group = avg >= 1024 ? 2 : avg >= 256 ? 2 : 1;
  int want_msub = avg >= 1024 ? 2 : 1;
  if (cfg && cfg->cta_group != 0) want_group = cfg->cta_group;
  if (cfg && cfg->m_sub != 0) want_msub = cfg->m_sub;
  if (ctx->num_sms < 2) want_group = 1;
  const KernelEntry* k = nullptr;
  int ki = -1;
  for (int i = 0; i < kNumGroupedKernels; ++i)
    if (kGroupedKernels[i].in_type == in_type && kGroupedKernels[i].cta_group == want_group &&
        kGroupedKernels[i].m_sub == want_msub) {
      k = &kGroupedKernels[i];
      ki = i;
    }
  if (!k)
    return set_error(ctx, PATINA_GEMM_ERR_INVALID_ARG,
                     fmt("no grouped kernel for cta_group=%d m_sub=%d", want_group, want_msub));

  const uint32_t ib = input_bytes(in_type);
  const uint32_t kelems = kBlockKBytes / ib;
  const uint32_t tile_m = 128u * k->cta_group * k->m_sub;
  const uint32_t tiles_n = ceil_div(N, k->block_n);
  // every group may end with one partly filled row block
  const uint64_t max_tiles = ((uint64_t)(total_rows / tile_m) + (uint64_t)n_groups) * tiles_n;
  CUtensorMap tm_a, tm_b;
  CStoreMaps<1> tm_c;
  rc = get_tensor_map(ctx, A, tmap_in_type(in_type), ib, (uint64_t)total_rows, (uint64_t)K,
                      (uint64_t)lda, kCtaRows, kelems, &tm_a);
  if (rc != PATINA_GEMM_OK) return rc;
  rc = get_tensor_map(ctx, B, tmap_in_type(in_type), ib, (uint64_t)n_groups * (uint64_t)N,
                      (uint64_t)K, (uint64_t)ldb, (uint32_t)(k->block_n / k->cta_group), kelems, &tm_b);
  if (rc != PATINA_GEMM_OK) return rc;
  rc = get_tensor_map(ctx, C, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)total_rows, (uint64_t)N,
                      (uint64_t)ldc, kStoreBoxRows, staging_row_bytes((uint32_t)k->m_sub, 2) / 2,
                      &tm_c.map[0]);
  if (rc != PATINA_GEMM_OK) return rc;

  if (!ctx->grouped_attr_set[ki]) {
    cudaError_t e = cudaFuncSetAttribute(reinterpret_cast<const void*>(k->fn),
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)k->smem_bytes);
    if (e != cudaSuccess) return cuda_fail(ctx, e, "cudaFuncSetAttribute(smem, grouped)");
    ctx->grouped_attr_set[ki] = true;
  }
  uint32_t slots = (uint32_t)(ctx->num_sms / k->cta_group);
  if (k->cta_group > 1) {
    const uint32_t cap = (uint32_t)resident_clusters(k, ctx->num_sms, &ctx->grouped_max_clusters[ki]);
    if (cap < slots) slots = cap;
  }
  if (cfg && cfg->max_ctas > 0 && (uint32_t)(cfg->max_ctas / k->cta_group) < slots)
    slots = (uint32_t)(cfg->max_ctas / k->cta_group);
  if (slots == 0) slots = 1;
  const uint32_t clusters = max_tiles < slots ? (uint32_t)max_tiles : slots;

  GemmParams p{};
  p.M = (uint32_t)total_rows;
  p.N = (uint32_t)N;
  p.K = (uint32_t)K;
  p.tiles_m = 0;
  p.tiles_n = tiles_n;
  p.num_tiles = 0;  // the kernel derives it from the group sizes
  p.split_from = 0xffffffffu;
  p.k_blocks = ceil_div(K, kelems);
  p.group_m = (cfg && cfg->group_m > 0) ? (uint32_t)cfg->group_m : 8u;
  p.alpha = alpha;
  p.n_dests = 1;
  p.group_rows = group_rows;
  p.group_alpha = group_alpha;
  p.n_groups = (uint32_t)n_groups;
  p.c_dests[0] = C;
  p.ldc = ldc;
  p.status = ctx->d_status;
  p.wait_limit_ns = ctx->wait_limit_ns;

  cudaLaunchConfig_t lc{};
  lc.gridDim = dim3(clusters * k->cta_group, 1, 1);
  lc.blockDim = dim3(block_threads(k->m_sub, false), 1, 1);
  lc.dynamicSmemBytes = k->smem_bytes;
  lc.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)k->cta_group;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  lc.attrs = attr;
  lc.numAttrs = (k->cta_group > 1) ? 1 : 0;
  drain_stale_error();
  cudaError_t e = cudaLaunchKernelEx(&lc, k->fn, tm_a, tm_b, tm_c, p);
  if (e != cudaSuccess) return cuda_fail(ctx, e, "cudaLaunchKernelEx(grouped)");
  ctx->launches += 1;
  return PATINA_GEMM_OK;
}

int grow(PatinaGemmContext* ctx, void** p, size_t* cap, size_t need) {
  if (*cap >= need) return PATINA_GEMM_OK;
  if (*p) cudaFree(*p);
  *p = nullptr;
  *cap = 0;
  cudaError_t e = cudaMalloc(p, need);
  if (e != cudaSuccess) return cuda_fail(ctx, e, "cudaMalloc(staging)");
  *cap = need;
  return PATINA_GEMM_OK;
}

}  // namespace

// =============================================================== C ABI ======
extern "C" {

#ifdef PATINA_TRACE
// Trace builds only (not declared in the public header): where the large-tile kernel writes its
// per-CTA time stamps, [grid][32] 64-bit words of device memory, or null to stop.
int patina_gemm_debug_set_trace(PatinaGemmContext* ctx, void* buf) {
  if (!ctx) return PATINA_GEMM_ERR_INVALID_ARG;
  ctx->trace = static_cast<unsigned long long*>(buf);
  return PATINA_GEMM_OK;
}
// Trace builds only: a tile configuration for the scatter entry point (null: the library's choice),
// for comparing store-box shapes over NVLink.
int patina_gemm_debug_set_scatter_config(PatinaGemmContext* ctx, const PatinaGemmConfig* cfg) {
  if (!ctx) return PATINA_GEMM_ERR_INVALID_ARG;
  ctx->has_scatter_cfg = cfg != nullptr;
  if (cfg) ctx->scatter_cfg = *cfg;
  return PATINA_GEMM_OK;
}
// Trace builds only: L2 eviction hints on the operand loads of pair kernels (0 none, 1 evict-first,
// 2 evict-last), for measuring what they do to DRAM traffic.
int patina_gemm_debug_set_l2_hints(PatinaGemmContext* ctx, uint32_t hint_a, uint32_t hint_b) {
  if (!ctx) return PATINA_GEMM_ERR_INVALID_ARG;
  ctx->l2_hint_a = hint_a;
  ctx->l2_hint_b = hint_b;
  return PATINA_GEMM_OK;
}
#endif

const char* patina_gemm_version(void) { return "patina-b200-gemm 0.1 (sm_100a, tcgen05)"; }

void patina_gemm_string_free(char* s) { std::free(s); }

char* patina_gemm_last_error(PatinaGemmContext* ctx) {
  if (!ctx || ctx->last_error.empty()) return nullptr;
  return dup_cstr(ctx->last_error);
}

int patina_gemm_context_create(int device, PatinaGemmContext** out) {
  if (!out) return PATINA_GEMM_ERR_INVALID_ARG;
  *out = nullptr;
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess || count <= 0) {
    cudaGetLastError();
    return PATINA_GEMM_ERR_UNSUPPORTED_ARCH;  // no CUDA device at all: nothing can run here
  }
  if (device < 0 || device >= count) return PATINA_GEMM_ERR_INVALID_ARG;
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) return PATINA_GEMM_ERR_CUDA;
  if (prop.major != 10) return PATINA_GEMM_ERR_UNSUPPORTED_ARCH;  // tcgen05 needs sm_100a
  PatinaGemmContext* ctx = new PatinaGemmContext();
  ctx->device = device;
  ctx->num_sms = prop.multiProcessorCount;
  ctx->cc_major = prop.major;
  ctx->cc_minor = prop.minor;
  DeviceGuard guard(device);
  if (!guard.ok) {
    delete ctx;
    return PATINA_GEMM_ERR_CUDA;
  }
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
  if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || !fn) {
    delete ctx;
    return PATINA_GEMM_ERR_CUDA;
  }
  ctx->encode = reinterpret_cast<EncodeTiledFn>(fn);
  e = cudaMalloc(reinterpret_cast<void**>(&ctx->d_status), 4 * sizeof(uint32_t));
  if (e == cudaSuccess) e = cudaMemset(ctx->d_status, 0, 4 * sizeof(uint32_t));
  if (e != cudaSuccess) {
    delete ctx;
    return PATINA_GEMM_ERR_CUDA;
  }
  *out = ctx;
  return PATINA_GEMM_OK;
}

void patina_gemm_context_destroy(PatinaGemmContext* ctx) {
  if (!ctx) return;
  {
    DeviceGuard guard(ctx->device);
    if (ctx->d_status) cudaFree(ctx->d_status);
    if (ctx->d_sk_partials) cudaFree(ctx->d_sk_partials);
    if (ctx->d_sk_counters) cudaFree(ctx->d_sk_counters);
    if (ctx->s_in) {
      cudaStreamDestroy(ctx->s_in);
      cudaStreamDestroy(ctx->s_out);
      for (int i = 0; i < kHostEvents; ++i)
        if (ctx->ev[i]) cudaEventDestroy(ctx->ev[i]);
    }
    if (ctx->d_a) cudaFree(ctx->d_a);
    if (ctx->d_b) cudaFree(ctx->d_b);
    if (ctx->d_c) cudaFree(ctx->d_c);
  }
  delete ctx;
}

int patina_gemm_set_wait_limit_ns(PatinaGemmContext* ctx, uint64_t ns) {
  if (!ctx || ns == 0) return PATINA_GEMM_ERR_INVALID_ARG;
  ctx->wait_limit_ns = ns;
  return PATINA_GEMM_OK;
}

uint64_t patina_gemm_launch_count(PatinaGemmContext* ctx) { return ctx ? ctx->launches : 0; }

int patina_gemm_status(PatinaGemmContext* ctx, void* stream) {
  if (!ctx) return PATINA_GEMM_ERR_INVALID_ARG;
  DeviceGuard guard(ctx->device);
  cudaError_t e = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail(ctx, e, "cudaStreamSynchronize");
  uint32_t st[4] = {0, 0, 0, 0};
  e = cudaMemcpy(st, ctx->d_status, sizeof(st), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return cuda_fail(ctx, e, "cudaMemcpy(status)");
  if (st[0] == 0) return PATINA_GEMM_OK;
  static const char* const names[] = {"ok",
                                      "producer waiting for an empty stage",
                                      "MMA issuer waiting for a full stage",
                                      "MMA issuer waiting for a free accumulator",
                                      "epilogue waiting for a finished accumulator",
                                      "MMA issuer draining its last accumulator",
                                      "split-K reducer"};
  const char* what = st[0] < sizeof(names) / sizeof(names[0]) ? names[st[0]] : "unknown";
  set_error(ctx, PATINA_GEMM_ERR_TIMEOUT,
            fmt("device wait expired: %s (code %u, block %u, detail %u)", what, st[0], st[1], st[2]));
  cudaMemset(ctx->d_status, 0, sizeof(st));
  // an abandoned stream-K launch may have left arrival counters half-way
  if (ctx->d_sk_counters) cudaMemset(ctx->d_sk_counters, 0, ctx->cap_sk_counters);
  return PATINA_GEMM_ERR_TIMEOUT;
}

int patina_gemm_ex(PatinaGemmContext* ctx, int in_type, int out_type, const void* A, int64_t lda,
                   const void* B, int64_t ldb, void* C, int64_t ldc, int64_t M, int64_t N,
                   int64_t K, float alpha, const PatinaGemmConfig* cfg, void* stream) {
  return launch_gemm(ctx, in_type, out_type, A, lda, B, ldb, C, ldc, M, N, K, alpha, cfg,
                     static_cast<cudaStream_t>(stream));
}

int patina_gemm_bf16_tn(PatinaGemmContext* ctx, const void* A, int64_t lda, const void* B,
                        int64_t ldb, void* C, int64_t ldc, int64_t M, int64_t N, int64_t K,
                        float alpha, void* stream) {
  return launch_gemm(ctx, kBF16, kOutBF16, A, lda, B, ldb, C, ldc, M, N, K, alpha, nullptr,
                     static_cast<cudaStream_t>(stream));
}

int patina_gemm_fp8e4m3_tn(PatinaGemmContext* ctx, const void* A, int64_t lda, const void* B,
                           int64_t ldb, void* C, int64_t ldc, int64_t M, int64_t N, int64_t K,
                           float scale_a, float scale_b, void* stream) {
  return launch_gemm(ctx, kE4M3, kOutBF16, A, lda, B, ldb, C, ldc, M, N, K, scale_a * scale_b,
                     nullptr, static_cast<cudaStream_t>(stream));
}

int patina_gemm_f16_tn_f32out(PatinaGemmContext* ctx, const void* A, int64_t lda, const void* B,
                              int64_t ldb, void* C, int64_t ldc, int64_t M, int64_t N, int64_t K,
                              float alpha, void* stream) {
  return launch_gemm(ctx, kF16, kOutF32, A, lda, B, ldb, C, ldc, M, N, K, alpha, nullptr,
                     static_cast<cudaStream_t>(stream));
}

static int check_epilogue(PatinaGemmContext* ctx, const PatinaGemmEpilogue* epi, int64_t N, int64_t K) {
  if (!epi) return set_error(ctx, PATINA_GEMM_ERR_INVALID_ARG, "epilogue description is null");
  if (epi->activation < 0 || epi->activation > 3)
    return set_error(ctx, PATINA_GEMM_ERR_INVALID_ARG, "unknown activation");
  if (epi->bias && (reinterpret_cast<uintptr_t>(epi->bias) & 3u))
    return set_error(ctx, PATINA_GEMM_ERR_INVALID_ARG, "bias is not 4-byte aligned");
  if (epi->residual) {
    if ((reinterpret_cast<uintptr_t>(epi->residual) & 15u) || epi->ldr < N || (epi->ldr * 2) % 16 != 0)
      return set_error(ctx, PATINA_GEMM_ERR_INVALID_ARG,
                       "residual must be 16-byte aligned with ldr >= N and a row pitch multiple of 16 bytes");
  }
  if (K == 0) return set_error(ctx, PATINA_GEMM_ERR_INVALID_ARG, "fused epilogue needs K > 0");
  return PATINA_GEMM_OK;
}

int patina_gemm_bf16_tn_fused_fp8out(PatinaGemmContext* ctx, const void* A, int64_t lda, const void* B,
                                     int64_t ldb, void* C, int64_t ldc, int64_t M, int64_t N, int64_t K,
                                     float alpha, const PatinaGemmEpilogue* epi, float out_scale,
                                     float* amax, void* stream) {
  if (!ctx) return PATINA_GEMM_ERR_INVALID_ARG;
  const PatinaGemmEpilogue none{};
  if (!epi) epi = &none;
  int rc = check_epilogue(ctx, epi, N, K);
  if (rc != PATINA_GEMM_OK) return rc;
  if (!(out_scale > 0.0f) || !std::isfinite(out_scale))
    return set_error(ctx, PATINA_GEMM_ERR_INVALID_ARG, "out_scale must be positive and finite");
  if (amax && (reinterpret_cast<uintptr_t>(amax) & 3u))
    return set_error(ctx, PATINA_GEMM_ERR_INVALID_ARG, "amax is not 4-byte aligned");
  return launch_gemm(ctx, kBF16, kOutE4M3, A, lda, B, ldb, C, ldc, M, N, K, alpha, nullptr,
                     static_cast<cudaStream_t>(stream), nullptr, 0, epi, out_scale, amax);
}

int patina_gemm_bf16_tn_fused(PatinaGemmContext* ctx, const void* A, int64_t lda, const void* B,
                              int64_t ldb, void* C, int64_t ldc, int64_t M, int64_t N, int64_t K,
                              float alpha, const PatinaGemmEpilogue* epi, void* stream) {
  if (!ctx) return PATINA_GEMM_ERR_INVALID_ARG;
  {
    const int rc = check_epilogue(ctx, epi, N, K);
    if (rc != PATINA_GEMM_OK) return rc;
  }
  // A transcendental per output is too much work for the epilogue of the TMEM-filling tile,
  // which runs between two mainloops: take the double-buffered 256 x 256 pair tile, whose
  // epilogue overlaps the next tile's mainloop (measured at 8192 x 14336 x 4096 with bias + GELU:
  // 0.747 ms against 0.760 ms on the TMEM-filling tile).
  PatinaGemmConfig overlap{};
  overlap.cta_group = 2;
  overlap.block_n = 256;
  overlap.m_sub = 1;
  const bool heavy = epi->activation == (int)kActGelu || epi->activation == (int)kActSilu;
  return launch_gemm(ctx, kBF16, kOutBF16, A, lda, B, ldb, C, ldc, M, N, K, alpha,
                     heavy ? &overlap : nullptr, static_cast<cudaStream_t>(stream), nullptr, 0, epi);
}

int patina_gemm_bf16_tn_scatter(PatinaGemmContext* ctx, const void* A, int64_t lda, const void* B,
                                int64_t ldb, void* const* C_dests, int n_dests, int64_t ldc,
                                int64_t M, int64_t N, int64_t K, float alpha, void* stream) {
  if (!ctx) return PATINA_GEMM_ERR_INVALID_ARG;
  if (!C_dests || n_dests < 1 || n_dests > kMaxDests)
    return set_error(ctx, PATINA_GEMM_ERR_INVALID_ARG, "n_dests must be 1..8 and C_dests non-null");
  const PatinaGemmConfig* cfg = nullptr;
#ifdef PATINA_TRACE
  if (ctx->has_scatter_cfg) cfg = &ctx->scatter_cfg;
#endif
  return launch_gemm(ctx, kBF16, kOutBF16, A, lda, B, ldb, C_dests[0], ldc, M, N, K, alpha, cfg,
                     static_cast<cudaStream_t>(stream), C_dests + 1, n_dests - 1);
}

int patina_gemm_bf16_tn_grouped(PatinaGemmContext* ctx, const void* A, int64_t lda, const void* B,
                                int64_t ldb, void* C, int64_t ldc, const int32_t* group_rows,
                                int n_groups, int64_t total_rows, int64_t N, int64_t K, float alpha,
                                const PatinaGemmConfig* config, void* stream) {
  return launch_grouped(ctx, kBF16, A, lda, B, ldb, C, ldc, group_rows, n_groups, total_rows, N, K,
                        alpha, nullptr, config, static_cast<cudaStream_t>(stream));
}

int patina_gemm_fp8e4m3_tn_grouped(PatinaGemmContext* ctx, const void* A, int64_t lda, const void* B,
                                   int64_t ldb, void* C, int64_t ldc, const int32_t* group_rows,
                                   int n_groups, int64_t total_rows, int64_t N, int64_t K, float scale_a,
                                   const float* group_scale_b, const PatinaGemmConfig* config,
                                   void* stream) {
  return launch_grouped(ctx, kE4M3, A, lda, B, ldb, C, ldc, group_rows, n_groups, total_rows, N, K,
                        scale_a, group_scale_b, config, static_cast<cudaStream_t>(stream));
}

void patina_gemm_column_shard(int64_t n, int world, int rank, int64_t* n0, int64_t* n1) {
  int64_t a = 0, b = 0;
  if (n > 0 && world > 0 && rank >= 0 && rank < world) {
    const int64_t blocks = (n + 255) / 256, per = (blocks + world - 1) / world;
    a = (int64_t)rank * per * 256 < n ? (int64_t)rank * per * 256 : n;
    b = (int64_t)(rank + 1) * per * 256 < n ? (int64_t)(rank + 1) * per * 256 : n;
  }
  if (n0) *n0 = a;
  if (n1) *n1 = b;
}

int patina_gemm_sharded_bf16_tn(PatinaGemmContext* const* ctxs, int n_shards, const void* const* A, int64_t lda,
                                const void* const* B_shards, int64_t ldb, void* const* C_shards, int64_t ldc,
                                int64_t M, int64_t N, int64_t K, float alpha, void* const* streams) {
  if (!ctxs || !A || !B_shards || !C_shards || n_shards < 1 || n_shards > kMaxDests) return PATINA_GEMM_ERR_INVALID_ARG;
  for (int g = 0; g < n_shards; ++g)
    if (!ctxs[g]) return PATINA_GEMM_ERR_INVALID_ARG;
  // One launch per shard, each on its own context's device and stream; nothing waits here, so
  // the shards run concurrently when the contexts are on different GPUs (or streams).
  for (int g = 0; g < n_shards; ++g) {
    int64_t n0, n1;
    patina_gemm_column_shard(N, n_shards, g, &n0, &n1);
    if (n1 == n0) continue;
    // (ascending k in one accumulator: every shard's columns equal the unsharded result's)
    PatinaGemmConfig cfg{};
    cfg.k_order = 1;
    const int rc = launch_gemm(ctxs[g], kBF16, kOutBF16, A[g], lda, B_shards[g], ldb, C_shards[g], ldc, M, n1 - n0,
                               K, alpha, &cfg, static_cast<cudaStream_t>(streams ? streams[g] : nullptr));
    if (rc != PATINA_GEMM_OK) return rc;
  }
  return PATINA_GEMM_OK;
}

int patina_gemm_mxfp8_tn(PatinaGemmContext* ctx, const void* A, int64_t lda, const void* scales_a,
                         const void* B, int64_t ldb, const void* scales_b, void* C, int64_t ldc, int64_t M,
                         int64_t N, int64_t K, float alpha, const PatinaGemmConfig* config, void* stream) {
  return launch_mx(ctx, A, lda, scales_a, B, ldb, scales_b, C, ldc, M, N, K, alpha, config,
                   static_cast<cudaStream_t>(stream));
}

uint64_t patina_gemm_mx_scale_bytes(int64_t rows, int64_t K) {
  if (rows <= 0 || K <= 0) return 0;
  return mx_scale_atoms((uint64_t)rows, (uint64_t)K) * kSfAtomBytes;
}

uint64_t patina_gemm_mx_scale_offset(int64_t row, int64_t k_block32, int64_t K) {
  return mx_scale_offset((uint64_t)row, (uint64_t)k_block32, (uint64_t)K);
}

uint32_t patina_gemm_idesc_mx(uint32_t umma_m, uint32_t umma_n, uint32_t a_sf_id, uint32_t b_sf_id) {
  return idesc_mx(umma_m, umma_n, a_sf_id, b_sf_id);
}

// ---- buffers that other processes on the node can write ------------------------------------
int patina_gemm_peer_alloc(PatinaGemmContext* ctx, size_t bytes, void** ptr, unsigned char handle_out[64]) {
  if (!ctx || !ptr || !handle_out || bytes == 0) return PATINA_GEMM_ERR_INVALID_ARG;
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handles are 64 bytes");
  DeviceGuard guard(ctx->device);
  *ptr = nullptr;
  cudaError_t e = cudaMalloc(ptr, bytes);
  if (e != cudaSuccess) return cuda_fail(ctx, e, "cudaMalloc(peer buffer)");
  cudaIpcMemHandle_t h;
  e = cudaIpcGetMemHandle(&h, *ptr);
  if (e != cudaSuccess) {
    cudaFree(*ptr);
    *ptr = nullptr;
    return cuda_fail(ctx, e, "cudaIpcGetMemHandle");
  }
  std::memcpy(handle_out, &h, 64);
  return PATINA_GEMM_OK;
}

int patina_gemm_peer_open(PatinaGemmContext* ctx, const unsigned char handle[64], void** ptr) {
  if (!ctx || !ptr || !handle) return PATINA_GEMM_ERR_INVALID_ARG;
  // Opened with THIS context's device current: the driver maps the exporter's memory for this
  // device and enables peer access between the two as part of the open.
  DeviceGuard guard(ctx->device);
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle, 64);
  *ptr = nullptr;
  const cudaError_t e = cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) return cuda_fail(ctx, e, "cudaIpcOpenMemHandle");
  return PATINA_GEMM_OK;
}

int patina_gemm_peer_close(PatinaGemmContext* ctx, void* ptr) {
  if (!ctx) return PATINA_GEMM_ERR_INVALID_ARG;
  if (!ptr) return PATINA_GEMM_OK;
  DeviceGuard guard(ctx->device);
  const cudaError_t e = cudaIpcCloseMemHandle(ptr);
  return e == cudaSuccess ? PATINA_GEMM_OK : cuda_fail(ctx, e, "cudaIpcCloseMemHandle");
}

int patina_gemm_peer_free(PatinaGemmContext* ctx, void* ptr) {
  if (!ctx) return PATINA_GEMM_ERR_INVALID_ARG;
  if (!ptr) return PATINA_GEMM_OK;
  DeviceGuard guard(ctx->device);
  const cudaError_t e = cudaFree(ptr);
  return e == cudaSuccess ? PATINA_GEMM_OK : cuda_fail(ctx, e, "cudaFree(peer buffer)");
}

int patina_gemm_host(PatinaGemmContext* ctx, int in_type, int out_type, const void* hostA,
                     int64_t lda, const void* hostB, int64_t ldb, void* hostC, int64_t ldc,
                     int64_t M, int64_t N, int64_t K, float alpha, const PatinaGemmConfig* cfg,
                     void* stream_v) {
  if (!ctx) return PATINA_GEMM_ERR_INVALID_ARG;
  if (!type_pair_supported(in_type, out_type))
    return set_error(ctx, PATINA_GEMM_ERR_INVALID_ARG, "unsupported type pair");
  if (M < 0 || N < 0 || K < 0 || lda < K || ldb < K || ldc < N)
    return set_error(ctx, PATINA_GEMM_ERR_INVALID_ARG, "bad dimensions or leading dimensions");
  if (M == 0 || N == 0) return PATINA_GEMM_OK;
  if (!hostC || (K > 0 && (!hostA || !hostB)))
    return set_error(ctx, PATINA_GEMM_ERR_INVALID_ARG, "null host pointer");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  DeviceGuard guard(ctx->device);
  // Ascending k in one accumulator, whether the call runs one GEMM or one per row block: the
  // result does not depend on how (or whether) the rows are cut.
  PatinaGemmConfig host_cfg{};
  if (cfg) host_cfg = *cfg;
  if (host_cfg.k_order == 0) host_cfg.k_order = 1;
  cfg = &host_cfg;
  const size_t ib = input_bytes(in_type), ob = output_bytes(out_type);
  // Device copies are dense with the pitch rounded up to 16 bytes.
  const int64_t dk = (int64_t)((((size_t)K * ib + 15) / 16) * 16 / ib);
  const int64_t dn = (int64_t)((((size_t)N * ob + 15) / 16) * 16 / ob);
  int rc;
  if ((rc = grow(ctx, &ctx->d_a, &ctx->cap_a, (size_t)M * dk * ib + 16)) != 0) return rc;
  if ((rc = grow(ctx, &ctx->d_b, &ctx->cap_b, (size_t)N * dk * ib + 16)) != 0) return rc;
  if ((rc = grow(ctx, &ctx->d_c, &ctx->cap_c, (size_t)M * dn * ob + 16)) != 0) return rc;
  cudaError_t e;
  // Large problems are cut into row blocks of A / C so that the copy of block i+1 to the
  // device, the GEMM of block i and the copy of block i-1 back overlap (PCIe is full duplex and
  // is what bounds this call). Two context-owned streams carry the copies; events tie them to
  // the caller's stream in both directions, so the call still behaves as work enqueued on it.
  const size_t total_bytes = ((size_t)M * K + (size_t)N * K) * ib + (size_t)M * N * ob;
  int chunks = 1;
  if (K > 0 && total_bytes >= ((size_t)32 << 20) && M >= 1024) {
    // (Sixteen blocks of 512 rows, for a shorter tail after the last byte of A, measured no
    // better than eight: 6.0 vs 5.9 ms per 8192^3 call.)
    chunks = (int)(M / 1024);
    if (chunks > kHostChunksMax) chunks = kHostChunksMax;
  }
  if (chunks <= 1) {
    if (K > 0) {
      e = cudaMemcpy2DAsync(ctx->d_a, (size_t)dk * ib, hostA, (size_t)lda * ib, (size_t)K * ib,
                            (size_t)M, cudaMemcpyHostToDevice, stream);
      if (e != cudaSuccess) return cuda_fail(ctx, e, "cudaMemcpy2DAsync(A)");
      e = cudaMemcpy2DAsync(ctx->d_b, (size_t)dk * ib, hostB, (size_t)ldb * ib, (size_t)K * ib,
                            (size_t)N, cudaMemcpyHostToDevice, stream);
      if (e != cudaSuccess) return cuda_fail(ctx, e, "cudaMemcpy2DAsync(B)");
    }
    rc = launch_gemm(ctx, in_type, out_type, ctx->d_a, dk, ctx->d_b, dk, ctx->d_c, dn, M, N, K, alpha,
                     cfg, stream);
    if (rc != PATINA_GEMM_OK) return rc;
    e = cudaMemcpy2DAsync(hostC, (size_t)ldc * ob, ctx->d_c, (size_t)dn * ob, (size_t)N * ob,
                          (size_t)M, cudaMemcpyDeviceToHost, stream);
    if (e != cudaSuccess) return cuda_fail(ctx, e, "cudaMemcpy2DAsync(C)");
    return PATINA_GEMM_OK;
  }

  if (!ctx->s_in) {
    e = cudaStreamCreateWithFlags(&ctx->s_in, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&ctx->s_out, cudaStreamNonBlocking);
    for (int i = 0; e == cudaSuccess && i < kHostEvents; ++i)
      e = cudaEventCreateWithFlags(&ctx->ev[i], cudaEventDisableTiming);
    if (e != cudaSuccess) return cuda_fail(ctx, e, "creating copy streams/events");
  }
  // Every row block takes the path the whole problem would take, so that the result does not
  // depend on how this call cuts the rows (a block alone might be small enough for the cluster
  // split, whose sums round differently).
  PatinaGemmConfig block_cfg{};
  if (cfg) block_cfg = *cfg;
  if (block_cfg.cluster_k == 0) {
    const bool tile_given = block_cfg.cta_group != 0 || block_cfg.block_n != 0 || block_cfg.m_sub != 0;
    const int whole = tile_given ? 0 : cluster_k_choice(in_type, out_type, M, N, K, ctx->num_sms);
    block_cfg.cluster_k = whole > 0 ? whole : -1;
  }
  if (block_cfg.stream_k == 0) block_cfg.stream_k = -1;   // M >= 1024 here
  cfg = &block_cfg;
  cudaEvent_t ev_start = ctx->ev[0], ev_b = ctx->ev[1], ev_done = ctx->ev[2];
  cudaEvent_t* ev_a = &ctx->ev[3];
  cudaEvent_t* ev_g = &ctx->ev[3 + kHostChunksMax];
  // rows per block: a whole number of 512-row tiles
  int64_t rows = (M + chunks - 1) / chunks;
  rows = (rows + 511) / 512 * 512;
#define PATINA_TRY(call, what)                       \
  do {                                               \
    e = (call);                                      \
    if (e != cudaSuccess) return cuda_fail(ctx, e, what); \
  } while (0)
  PATINA_TRY(cudaEventRecord(ev_start, stream), "cudaEventRecord");
  PATINA_TRY(cudaStreamWaitEvent(ctx->s_in, ev_start, 0), "cudaStreamWaitEvent");
  PATINA_TRY(cudaStreamWaitEvent(ctx->s_out, ev_start, 0), "cudaStreamWaitEvent");
  PATINA_TRY(cudaMemcpy2DAsync(ctx->d_b, (size_t)dk * ib, hostB, (size_t)ldb * ib, (size_t)K * ib,
                               (size_t)N, cudaMemcpyHostToDevice, ctx->s_in), "cudaMemcpy2DAsync(B)");
  PATINA_TRY(cudaEventRecord(ev_b, ctx->s_in), "cudaEventRecord");
  int used = 0;
  for (int64_t r0 = 0; r0 < M; r0 += rows, ++used) {
    const int64_t mr = (M - r0) < rows ? (M - r0) : rows;
    PATINA_TRY(cudaMemcpy2DAsync(static_cast<char*>(ctx->d_a) + (size_t)r0 * dk * ib, (size_t)dk * ib,
                                 static_cast<const char*>(hostA) + (size_t)r0 * lda * ib,
                                 (size_t)lda * ib, (size_t)K * ib, (size_t)mr, cudaMemcpyHostToDevice,
                                 ctx->s_in), "cudaMemcpy2DAsync(A block)");
    PATINA_TRY(cudaEventRecord(ev_a[used], ctx->s_in), "cudaEventRecord");
  }
  PATINA_TRY(cudaStreamWaitEvent(stream, ev_b, 0), "cudaStreamWaitEvent");
  used = 0;
  for (int64_t r0 = 0; r0 < M; r0 += rows, ++used) {
    const int64_t mr = (M - r0) < rows ? (M - r0) : rows;
    PATINA_TRY(cudaStreamWaitEvent(stream, ev_a[used], 0), "cudaStreamWaitEvent");
    rc = launch_gemm(ctx, in_type, out_type, static_cast<char*>(ctx->d_a) + (size_t)r0 * dk * ib, dk,
                     ctx->d_b, dk, static_cast<char*>(ctx->d_c) + (size_t)r0 * dn * ob, dn, mr, N, K,
                     alpha, cfg, stream);
    if (rc != PATINA_GEMM_OK) return rc;
    PATINA_TRY(cudaEventRecord(ev_g[used], stream), "cudaEventRecord");
    PATINA_TRY(cudaStreamWaitEvent(ctx->s_out, ev_g[used], 0), "cudaStreamWaitEvent");
    PATINA_TRY(cudaMemcpy2DAsync(static_cast<char*>(hostC) + (size_t)r0 * ldc * ob, (size_t)ldc * ob,
                                 static_cast<char*>(ctx->d_c) + (size_t)r0 * dn * ob, (size_t)dn * ob,
                                 (size_t)N * ob, (size_t)mr, cudaMemcpyDeviceToHost, ctx->s_out),
               "cudaMemcpy2DAsync(C block)");
  }
  PATINA_TRY(cudaEventRecord(ev_done, ctx->s_out), "cudaEventRecord");
  PATINA_TRY(cudaStreamWaitEvent(stream, ev_done, 0), "cudaStreamWaitEvent");
#undef PATINA_TRY
  return PATINA_GEMM_OK;
}

// ---- host-only helpers ------------------------------------------------------
int patina_gemm_validate(int in_type, int out_type, const void* A, int64_t lda, const void* B,
                         int64_t ldb, const void* C, int64_t ldc, int64_t M, int64_t N, int64_t K,
                         char** err_out) {
  std::string err;
  if (err_out) *err_out = nullptr;
  int rc = validate_args(in_type, out_type, A, lda, B, ldb, C, ldc, M, N, K, &err);
  if (rc != PATINA_GEMM_OK && err_out) *err_out = dup_cstr(err);
  return rc;
}

int patina_gemm_plan(int in_type, int out_type, int64_t M, int64_t N, int64_t K,
                     const PatinaGemmConfig* cfg, int num_sms, PatinaGemmPlan* out) {
  if (!out || M <= 0 || N <= 0 || K <= 0) return PATINA_GEMM_ERR_INVALID_ARG;
  return make_plan(in_type, out_type, M, N, K, cfg, num_sms, out, nullptr, nullptr);
}

int patina_gemm_streamk_chosen(int in_type, int out_type, int64_t M, int64_t N, int64_t K, int num_sms) {
  if (M <= 0 || N <= 0 || K <= 0 || num_sms <= 0) return 0;
  return streamk_preferred(in_type, out_type, M, N, K, num_sms) ? 1 : 0;
}

int patina_gemm_cluster_k_chosen(int in_type, int out_type, int64_t M, int64_t N, int64_t K, int num_sms) {
  if (M <= 0 || N <= 0 || K <= 0 || num_sms <= 0) return 0;
  if (streamk_preferred(in_type, out_type, M, N, K, num_sms)) return 0;
  return cluster_k_choice(in_type, out_type, M, N, K, num_sms);
}

int patina_gemm_streamk_plan(int in_type, int64_t M, int64_t N, int64_t K, int num_sms,
                             PatinaStreamKPlan* out) {
  if (!out || N <= 0 || K <= 0 || num_sms <= 0 ||
      !streamk_supported(in_type, in_type == kF16 ? kOutF32 : kOutBF16, M))
    return PATINA_GEMM_ERR_INVALID_ARG;
  const SkPlan s = make_sk_plan(in_type, M, N, K, num_sms);
  out->grid = s.grid;
  out->tiles = s.tiles;
  out->k_blocks = s.k_blocks;
  out->m_pad = s.m_pad;
  out->max_contrib = s.max_contrib;
  out->stages = streamk_stages(s.m_pad);
  out->smem_bytes = streamk_smem_bytes(s.m_pad);
  out->units = s.units;
  out->partial_bytes = s.partial_bytes;
  out->counter_bytes = s.counter_bytes;
  return PATINA_GEMM_OK;
}
void patina_gemm_streamk_range(uint64_t cta, uint64_t units, uint64_t parts, uint64_t* begin,
                               uint64_t* end) {
  if (begin) *begin = streamk_range_start(cta, units, parts);
  if (end) *end = streamk_range_start(cta + 1, units, parts);
}
uint32_t patina_gemm_streamk_owner(uint64_t unit, uint64_t units, uint64_t parts) {
  return streamk_owner(unit, units, parts);
}

uint64_t patina_gemm_smem_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes,
                               int swizzle_code) {
  return smem_desc(smem_addr, lbo_bytes, sbo_bytes, swizzle_code);
}
uint32_t patina_gemm_idesc(int in_type, uint32_t umma_m, uint32_t umma_n) {
  return idesc(in_type, umma_m, umma_n);
}
uint32_t patina_gemm_k_advance_units(uint32_t k_elems, int in_type) {
  return k_advance_units_sw128(k_elems, in_type);
}
uint32_t patina_gemm_tmem_lane_offset(uint32_t warp_quarter) { return tmem_lane_offset(warp_quarter); }
void patina_gemm_tile_coord(uint32_t t, uint32_t tiles_m, uint32_t tiles_n, uint32_t group_m,
                            uint32_t* m_block, uint32_t* n_block) {
  const TileCoord c = tile_coord(t, tiles_m, tiles_n, group_m);
  if (m_block) *m_block = c.m;
  if (n_block) *n_block = c.n;
}

}  // extern "C"

// ====================================================== allocation-free entry ======
// Some callers may not allocate device memory at all: code that runs inside a memory pool's
// own allocation callback, a serving process whose device memory is fully pre-partitioned
// and audited at start-up, or a latency-critical loop where cudaMalloc's implicit device
// synchronisation is forbidden. The context API above allocates (status word, stream-K
// scratch, growing on demand), so it is closed to them. This one entry point runs the
// stream-K skinny GEMM with its scratch in a fixed array that is part of the loaded module.
//
// The array exists once per GPU that loads the library and stays until the process exits.
// Every call on that GPU shares it and it keeps whatever the previous call left, so the
// part that must start at zero is cleared on the stream before each launch, and two calls
// that overlap on the same GPU (different streams, different threads) race on it.
namespace {

constexpr size_t kNoAllocStatusBytes = 256;                 // wait-expiry record
constexpr size_t kNoAllocCounterBytes = 64 * 1024;          // up to 16384 tiles of B
constexpr size_t kNoAllocPartialBytes = PATINA_GEMM_NOALLOC_PARTIAL_BYTES;
constexpr size_t kNoAllocScratchBytes = kNoAllocStatusBytes + kNoAllocCounterBytes + kNoAllocPartialBytes;

static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];

constexpr int kNoAllocMaxDevices = 64;
// Written once by the first call on a device and published with a release store of `ready`;
// later calls (any thread) read it after an acquire load. Two threads that both make the
// first call do the same set-up and store the same values.
struct NoAllocDevice {
  std::atomic<bool> ready{false};
  unsigned char* scratch = nullptr;  // DEVICE address of g_noalloc_scratch on this GPU
  int num_sms = 0;
};
NoAllocDevice g_noalloc_dev[kNoAllocMaxDevices];
std::atomic<EncodeTiledFn> g_noalloc_encode{nullptr};

int noalloc_fail(char* buf, size_t len, int code, const char* f, ...) {
  if (buf && len) {
    va_list ap;
    va_start(ap, f);
    std::vsnprintf(buf, len, f, ap);
    va_end(ap);
  }
  return code;
}

// The two maps the kernel needs, built on the stack; no cache, no heap.
int noalloc_encode(EncodeTiledFn enc, const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld,
                   uint32_t box_rows, CUtensorMap* out) {
  const cuuint64_t gdim[2] = {cols, rows};
  const cuuint64_t gstride[1] = {ld * 2};
  const cuuint32_t box[2] = {64, box_rows};
  const cuuint32_t estride[2] = {1, 1};
  CUresult rc = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), gdim, gstride,
                    box, estride, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return rc == CUDA_SUCCESS ? 0 : (int)rc;
}

}  // namespace

extern "C" int patina_gemm_bf16_tn_skinny_noalloc(const void* A, int64_t lda, const void* B,
                                                  int64_t ldb, void* C, int64_t ldc, int64_t M,
                                                  int64_t N, int64_t K, float alpha, void* stream_v,
                                                  char* err_buf, size_t err_buf_len) {
  if (err_buf && err_buf_len) err_buf[0] = '\0';
  if (M < 1 || M > 128)
    return noalloc_fail(err_buf, err_buf_len, PATINA_GEMM_ERR_INVALID_ARG,
                        "M=%lld is outside this entry point's range 1..128", (long long)M);
  if (N < 1 || K < 1)
    return noalloc_fail(err_buf, err_buf_len, PATINA_GEMM_ERR_INVALID_ARG, "N and K must be positive");
  // (the diagnostic goes straight into the caller's buffer: no host heap on any path)
  int rc = validate_args_buf(kBF16, kOutBF16, A, lda, B, ldb, C, ldc, M, N, K, err_buf, err_buf_len);
  if (rc != PATINA_GEMM_OK) return rc;

  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0) {
    cudaGetLastError();
    return noalloc_fail(err_buf, err_buf_len, PATINA_GEMM_ERR_UNSUPPORTED_ARCH, "no current CUDA device");
  }
  if (dev >= kNoAllocMaxDevices)
    return noalloc_fail(err_buf, err_buf_len, PATINA_GEMM_ERR_INVALID_ARG, "device index %d too large", dev);

  NoAllocDevice& d = g_noalloc_dev[dev];
  if (!d.ready.load(std::memory_order_acquire)) {
    // First call on this device: one-time set-up, with this device current. It queries the
    // device, resolves a driver entry point and asks the runtime for the DEVICE address of the
    // scratch array (in host code the array's name is only a host-side handle; passing it to a
    // kernel would hand the GPU a host address). Do this first call outside any stream capture.
    int major = 0, sms = 0;
    e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess)
      return noalloc_fail(err_buf, err_buf_len, PATINA_GEMM_ERR_CUDA, "cudaDeviceGetAttribute: %s",
                          cudaGetErrorString(e));
    if (major != 10)
      return noalloc_fail(err_buf, err_buf_len, PATINA_GEMM_ERR_UNSUPPORTED_ARCH,
                          "device %d is not sm_100 (tcgen05 needs Blackwell)", dev);
    if (!g_noalloc_encode.load(std::memory_order_acquire)) {
      void* fn = nullptr;
      cudaDriverEntryPointQueryResult q;
      e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
      if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !fn)
        return noalloc_fail(err_buf, err_buf_len, PATINA_GEMM_ERR_CUDA, "cuTensorMapEncodeTiled not found");
      g_noalloc_encode.store(reinterpret_cast<EncodeTiledFn>(fn), std::memory_order_release);
    }
    unsigned char* ptr = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_noalloc_scratch);
    if (e != cudaSuccess || !ptr)
      return noalloc_fail(err_buf, err_buf_len, PATINA_GEMM_ERR_CUDA, "cudaGetSymbolAddress(scratch): %s",
                          cudaGetErrorString(e));
    e = cudaFuncSetAttribute(reinterpret_cast<const void*>(gemm_streamk_kernel<kBF16>),
                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kMaxDynSmem);
    if (e != cudaSuccess)
      return noalloc_fail(err_buf, err_buf_len, PATINA_GEMM_ERR_CUDA, "cudaFuncSetAttribute: %s",
                          cudaGetErrorString(e));
    d.scratch = ptr;
    d.num_sms = sms;
    d.ready.store(true, std::memory_order_release);
  }

  const SkPlan sp = make_sk_plan(kBF16, M, N, K, d.num_sms);
  if (sp.partial_bytes > kNoAllocPartialBytes || sp.counter_bytes > kNoAllocCounterBytes)
    return noalloc_fail(err_buf, err_buf_len, PATINA_GEMM_ERR_INVALID_ARG,
                        "problem needs %llu bytes of partial-tile scratch and %llu of counters; this entry "
                        "point's fixed scratch holds %llu and %llu (use the context API for larger problems)",
                        (unsigned long long)sp.partial_bytes, (unsigned long long)sp.counter_bytes,
                        (unsigned long long)kNoAllocPartialBytes, (unsigned long long)kNoAllocCounterBytes);

  CUtensorMap tm_w, tm_x;
  const EncodeTiledFn enc = g_noalloc_encode.load(std::memory_order_acquire);
  if (noalloc_encode(enc, B, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, kSkTileRows, &tm_w) ||
      noalloc_encode(enc, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, sp.m_pad, &tm_x))
    return noalloc_fail(err_buf, err_buf_len, PATINA_GEMM_ERR_CUDA, "cuTensorMapEncodeTiled failed");

  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  // An error some earlier call left pending must not be reported as this launch's.
  drain_stale_error();
  // The previous call's leftovers: the status record and the arrival counters must be zero.
  e = cudaMemsetAsync(d.scratch, 0, kNoAllocStatusBytes + sp.counter_bytes, stream);
  if (e != cudaSuccess)
    return noalloc_fail(err_buf, err_buf_len, PATINA_GEMM_ERR_CUDA, "cudaMemsetAsync: %s", cudaGetErrorString(e));

  StreamKParams p{};
  p.M = (uint32_t)M;
  p.N = (uint32_t)N;
  p.K = (uint32_t)K;
  p.m_pad = sp.m_pad;
  p.tiles = sp.tiles;
  p.k_blocks = sp.k_blocks;
  p.units = sp.units;
  p.max_contrib = sp.max_contrib;
  p.stages = streamk_stages(sp.m_pad);
  p.stage_stride = streamk_stage_stride(sp.m_pad);
  p.burst = 4 < p.stages / 2 ? 4 : p.stages / 2;
  p.alpha = alpha;
  p.C = C;
  p.ldc = ldc;
  p.status = reinterpret_cast<uint32_t*>(d.scratch);
  p.counters = reinterpret_cast<uint32_t*>(d.scratch + kNoAllocStatusBytes);
  p.partials = reinterpret_cast<float*>(d.scratch + kNoAllocStatusBytes + kNoAllocCounterBytes);
  p.wait_limit_ns = 2000000000ull;
#ifdef PATINA_TRACE
  p.trace = nullptr;
#endif
  gemm_streamk_kernel<kBF16><<<sp.grid, 192, streamk_smem_bytes(sp.m_pad), stream>>>(tm_w, tm_x, p);
  e = cudaGetLastError();
  if (e != cudaSuccess)
    return noalloc_fail(err_buf, err_buf_len, PATINA_GEMM_ERR_CUDA, "kernel launch: %s", cudaGetErrorString(e));
  return PATINA_GEMM_OK;
}

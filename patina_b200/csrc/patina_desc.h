// patina_desc.h -- every derived encoding the GEMM depends on, as plain
// host+device constexpr functions so that host unit tests can pin them:
// the 64-bit UMMA shared-memory descriptor, the 32-bit instruction descriptor,
// the K-advance inside a swizzle atom, TMEM addressing, and the persistent
// tile scheduler's index map.
//
// Reference counterparts: crates/patina/src/layout.rs:162-228 (SWIZZLE_NONE,
// f16 only: LBO 128, SBO 256, idesc_f16, tmem_lane_offset) and the constants
// its PTX printer bakes in (mlir/lib/LowerToPTX.cpp:40-42). This header
// generalises them to 128-byte swizzle, bf16 / f16 / e4m3 operands,
// M in {128, 256} and N up to 256; the reference's own constants fall out as
// special cases and are checked in the tests.
#pragma once

#include <stdint.h>

#if defined(__CUDACC__)
#define PATINA_HD __host__ __device__ __forceinline__
#else
#define PATINA_HD inline
#endif

namespace patina {

// kMXE4M3: e4m3 elements with one E8M0 scale (a power of two) per 32 consecutive K elements of
// every row ("MXFP8"); the tensor core applies the scales (tcgen05.mma kind::mxf8f6f4.block_scale).
enum InputType : int { kF16 = 0, kBF16 = 1, kE4M3 = 2, kMXE4M3 = 3 };
enum OutputType : int { kOutBF16 = 0, kOutF32 = 1, kOutE4M3 = 2 };
enum SwizzleMode : int { kSwizzleNone = 0, kSwizzle128B = 2 };  // descriptor layout-type codes

PATINA_HD constexpr uint32_t input_bytes(int t) { return (t == kE4M3 || t == kMXE4M3) ? 1u : 2u; }
PATINA_HD constexpr bool is_block_scaled(int t) { return t == kMXE4M3; }
PATINA_HD constexpr uint32_t output_bytes(int t) { return t == kOutF32 ? 4u : t == kOutE4M3 ? 1u : 2u; }

// ---- shared-memory matrix descriptor (tcgen05, "version 1") --------------
//   [ 0,14) start address  >> 4      [16,30) leading-dim byte offset >> 4
//   [32,46) stride-dim byte offset >> 4   [46,48) version = 1
//   [61,64) layout type: 0 none, 2 = 128-byte swizzle
PATINA_HD constexpr uint64_t smem_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes,
                                       int swizzle) {
  return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | ((uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16) |
         ((uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32) | (1ull << 46) | ((uint64_t)swizzle << 61);
}

// K-major operand tile whose rows are exactly one 128-byte swizzle span:
// 8-row groups are 1024 bytes apart; the leading-dim offset is unused.
PATINA_HD constexpr uint64_t smem_desc_sw128_kmajor(uint32_t smem_addr) {
  return smem_desc(smem_addr, 0, 1024, kSwizzle128B);
}

// Descriptor units (16 bytes) to advance by `k_elems` along K inside the
// 128-byte span: +2 per K16 of bf16/f16, +2 per K32 of e4m3.
PATINA_HD constexpr uint32_t k_advance_units_sw128(uint32_t k_elems, int input_type) {
  return (k_elems * input_bytes(input_type)) >> 4;
}

// The reference's no-swizzle layout: K-adjacent core matrices 128 B apart,
// K advance = core matrices * LBO (layout.rs:176-179).
PATINA_HD constexpr uint32_t k_advance_units_noswizzle(uint32_t k_elems, uint32_t elt_bytes,
                                                       uint32_t lbo_bytes) {
  return ((k_elems * elt_bytes / 16) * lbo_bytes) >> 4;
}

// ---- instruction descriptor (kind::f16 and kind::f8f6f4, dense) -----------
//   [4,6) D format (1 = f32)   [7,10) A format   [10,13) B format
//   [15] A major, [16] B major (0 = K-major)   [17,23) N >> 3   [24,29) M >> 4
// kind::f16: 0 = f16, 1 = bf16.   kind::f8f6f4: 0 = e4m3.
PATINA_HD constexpr uint32_t idesc(int input_type, uint32_t umma_m, uint32_t umma_n) {
  uint32_t fmt = (input_type == kBF16) ? 1u : 0u;  // f16 -> 0, e4m3 -> 0 (in its own kind)
  return (1u << 4) | (fmt << 7) | (fmt << 10) | ((umma_n >> 3) << 17) | ((umma_m >> 4) << 24);
}

// ---- block-scaled instruction descriptor (kind::mxf8f6f4.block_scale) ------
//   [4,6) B scale-factor id   [7,10) A format (0 = e4m3)   [10,13) B format
//   [15] A major, [16] B major (0 = K-major)   [17,23) N >> 3   [23] scale format (1 = E8M0)
//   [24,29) M >> 4   [29,31) A scale-factor id
// The scale-factor id says which byte of the operand's 32-bit scale column this instruction uses:
// one column holds the scales of four consecutive 32-element k-blocks.
PATINA_HD constexpr uint32_t idesc_mx(uint32_t umma_m, uint32_t umma_n, uint32_t a_sf_id, uint32_t b_sf_id) {
  return ((b_sf_id & 3u) << 4) | ((umma_n >> 3) << 17) | (1u << 23) | ((umma_m >> 4) << 24) |
         ((a_sf_id & 3u) << 29);
}

// ---- block scales in memory ---------------------------------------------------
// The scales of a [rows, K] operand are stored in "atoms" of 512 bytes that cover 128 rows x
// 128 elements of K (4 scales per row): atom (rows / 128, k / 128), the K index running fastest;
// inside an atom the scale of row r, 32-element block j (0..3) is byte (r % 32) * 16 + (r / 32) * 4 + j.
// That is 32 lines of 16 bytes: exactly what one tcgen05.cp.32x128b.warpx4 moves into four
// TMEM columns (line l to lane l of every lane quarter), where the MMA expects row r's scales
// in lane r % 32, column r / 32. Buffers are padded to whole atoms in both directions.
constexpr uint32_t kSfAtomBytes = 512;
constexpr uint32_t kSfAtomRows = 128;
constexpr uint32_t kSfBlockElems = 32;   // K elements per scale
PATINA_HD constexpr uint64_t mx_scale_atoms(uint64_t rows, uint64_t k) {
  return ((rows + 127) / 128) * ((k + 127) / 128);
}
PATINA_HD constexpr uint64_t mx_scale_offset(uint64_t row, uint64_t k_block32, uint64_t k) {
  return ((row / 128) * ((k + 127) / 128) + k_block32 / 4) * kSfAtomBytes + (row % 32) * 16 +
         ((row % 128) / 32) * 4 + (k_block32 % 4);
}
// Atoms of B's scales that a tile of width block_n (a multiple of 64) can touch: tiles start at
// multiples of block_n, so at 0 or 64 rows into an atom.
PATINA_HD constexpr uint32_t mx_sfb_atoms(uint32_t block_n) {
  uint32_t most = 0;
  for (uint32_t j = 0; j < 4; ++j) {
    const uint32_t need = ((block_n * j) % 128 + block_n + 127) / 128;
    most = need > most ? need : most;
  }
  return most;
}

// Elements of K one MMA instruction consumes: 32 bytes of a K-major row.
PATINA_HD constexpr uint32_t umma_k(int input_type) { return 32u / input_bytes(input_type); }

// Legal (M, N) for one instruction: M=128 (one CTA) or 256 (CTA pair), N % 16 == 0, 16..256.
PATINA_HD constexpr bool umma_shape_ok(uint32_t m, uint32_t n) {
  return (m == 128 || m == 256) && n >= 16 && n <= 256 && (n % 16) == 0;
}

// ---- tensor memory ---------------------------------------------------------
// Address = lane << 16 | column. A warp may only touch the 32-lane quarter
// (warp_id % 4); lane quarter q starts at q << 21.
PATINA_HD constexpr uint32_t tmem_lane_offset(uint32_t quarter) { return quarter << 21; }
PATINA_HD constexpr uint32_t tmem_addr(uint32_t base, uint32_t lane, uint32_t col) {
  return base + (lane << 16) + col;
}

// ---- persistent tile scheduler ---------------------------------------------
// Linear tile index -> (m_block, n_block). Tiles are walked in bands of
// `group_m` M-blocks; inside a band M runs fastest, so the CTAs that are
// resident at the same time share a few A row-panels and B column-panels in L2.
struct TileCoord {
  uint32_t m, n;
};

PATINA_HD TileCoord tile_coord(uint32_t t, uint32_t tiles_m, uint32_t tiles_n, uint32_t group_m) {
  if (group_m == 0) group_m = 1;
  const uint32_t per_band = group_m * tiles_n;
  const uint32_t band = t / per_band;
  const uint32_t first_m = band * group_m;
  const uint32_t rows = (tiles_m - first_m) < group_m ? (tiles_m - first_m) : group_m;
  const uint32_t in_band = t - band * per_band;
  TileCoord c;
  c.m = first_m + in_band % rows;
  c.n = in_band / rows;
  return c;
}

// ---- shared-memory plan ------------------------------------------------------
struct SmemPlan {
  uint32_t a_bytes, b_bytes, stage_bytes, stages, staging_bytes, barrier_bytes, total_bytes;
};

constexpr uint32_t kBlockKBytes = 128;      // one swizzle span of K per stage
constexpr uint32_t kCtaRows = 128;          // accumulator rows (TMEM lanes) per CTA sub-tile
constexpr uint32_t kStoreBoxRows = 32;      // one epilogue warp's rows
constexpr uint32_t kBarrierRegionBytes = 256;
constexpr uint32_t kMaxDynSmem = 232448;    // 227 KB

// Epilogue staging, 32 KB in every configuration. With four epilogue warps each warp owns two
// buffers of 32 rows x 128 bytes (128-byte swizzle), double-buffered so that filling one overlaps
// the TMA store reading the other. With eight warps (m_sub = 2) the plain bf16 epilogue gives each
// warp ONE buffer of 32 rows x 128 bytes: half as many boxes per tile as 64-byte rows would take,
// and per box the proxy fence, the TMA store issue (235 cycles on one lane) and the buffer wait are
// paid once; the store's read of the buffer is waited out before it is refilled. (128-byte-row
// boxes also cross NVLink faster when the destinations are peer buffers.) The fused epilogue of
// the eight-warp tiles keeps two buffers of 64-byte rows (64-byte swizzle): 64 accumulator words
// plus 64 bias/residual words per thread would not fit its registers. One-byte outputs stage
// 64-byte rows (64 columns per box).
#ifndef PATINA_WIDE_EPILOGUE
#define PATINA_WIDE_EPILOGUE 1
#endif
PATINA_HD constexpr bool staging_wide(uint32_t m_sub, uint32_t out_bytes, bool fused) {
  return PATINA_WIDE_EPILOGUE != 0 && m_sub == 2 && out_bytes == 2 && !fused;
}
PATINA_HD constexpr uint32_t staging_bufs(uint32_t m_sub, uint32_t out_bytes = 2, bool fused = false) {
  return staging_wide(m_sub, out_bytes, fused) ? 1u : 2u;
}
PATINA_HD constexpr uint32_t staging_row_bytes(uint32_t m_sub, uint32_t out_bytes, bool fused = false) {
  if (staging_wide(m_sub, out_bytes, fused)) return 128u;
  return ((m_sub == 2 && out_bytes == 2) || out_bytes == 1) ? 64u : 128u;
}
PATINA_HD constexpr uint32_t staging_buf_bytes(uint32_t m_sub, uint32_t out_bytes, bool fused = false) {
  return kStoreBoxRows * staging_row_bytes(m_sub, out_bytes, fused);
}

PATINA_HD constexpr SmemPlan smem_plan(uint32_t cta_group, uint32_t m_sub, uint32_t block_n,
                                       uint32_t stages, uint32_t out_bytes = 2,
                                       uint32_t sf_stage_bytes = 0, bool fused = false,
                                       uint32_t k_chunks = 1) {
  SmemPlan p{};
  // (k_chunks: 128-byte spans of K per stage; more than one when a stage is fetched with 3-D boxes)
  p.a_bytes = m_sub * kCtaRows * kBlockKBytes * k_chunks;
  p.b_bytes = (block_n / cta_group) * kBlockKBytes * k_chunks;
  p.stage_bytes = p.a_bytes + p.b_bytes;
  p.stages = stages;
  p.staging_bytes = 4 * m_sub * staging_bufs(m_sub, out_bytes, fused) * staging_buf_bytes(m_sub, out_bytes, fused);
  p.barrier_bytes = kBarrierRegionBytes;
  // +1024: the ring is placed on the next 1024-byte boundary (swizzle atom).
  // (block-scaled operands: the scales of a stage sit in a ring of their own behind the staging)
  p.total_bytes = 1024 + stages * p.stage_bytes + p.staging_bytes + stages * sf_stage_bytes + p.barrier_bytes;
  return p;
}

}  // namespace patina

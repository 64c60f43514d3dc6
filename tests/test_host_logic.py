"""Host-side logic of the library, no GPU: the shared object loads and exports the
whole C ABI, every derived encoding matches the reference's pinned constants,
the tile scheduler is a bijection, plans and argument checks behave."""
import ctypes as C
import os
import re

import pytest

from patina_b200 import lib as L

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol(built_lib):
    header = open(os.path.join(ROOT, "include", "patina_gemm.h")).read()
    declared = set(re.findall(r"\b(patina_gemm_\w+)\s*\(", header))
    assert declared == set(L.SYMBOLS)
    for name in declared:
        assert hasattr(built_lib, name), name


def test_reference_constants(built_lib):
    # crates/patina/tests/golden/v2_gemm_pipelined.ptx:192,197; crates/patina/tests/layout.rs:33-68
    assert built_lib.patina_gemm_smem_desc(0, 128, 256, 0) == 70437464178688
    d = built_lib.patina_gemm_smem_desc(0x4000, 128, 256, 0)
    assert d & 0x3FFF == 0x4000 >> 4
    assert (d >> 16) & 0x3FFF == 128 >> 4 and (d >> 32) & 0x3FFF == 256 >> 4
    assert (d >> 46) & 3 == 1 and (d >> 61) == 0
    assert built_lib.patina_gemm_idesc(L.IN_F16, 128, 128) == 136314896
    assert built_lib.patina_gemm_idesc(L.IN_F16, 64, 256) == (1 << 4) | ((256 >> 3) << 17) | ((64 >> 4) << 24)
    assert built_lib.patina_gemm_tmem_lane_offset(0) == 0
    assert built_lib.patina_gemm_tmem_lane_offset(3) == 3 << 21


def test_generalised_encodings(built_lib):
    # 128-byte swizzle, K-major: SBO 1024, layout code 2, version 1
    d = built_lib.patina_gemm_smem_desc(0x8400, 0, 1024, 2)
    assert d & 0x3FFF == 0x8400 >> 4 and (d >> 32) & 0x3FFF == 64 and d >> 61 == 2 and (d >> 46) & 3 == 1
    bf = built_lib.patina_gemm_idesc(L.IN_BF16, 256, 256)
    assert (bf >> 4) & 3 == 1 and (bf >> 7) & 7 == 1 and (bf >> 10) & 7 == 1
    assert (bf >> 17) & 0x3F == 32 and (bf >> 24) & 0x1F == 16 and (bf >> 15) & 3 == 0
    f8 = built_lib.patina_gemm_idesc(L.IN_E4M3, 128, 256)
    assert (f8 >> 7) & 7 == 0 and (f8 >> 10) & 7 == 0 and (f8 >> 24) & 0x1F == 8
    # one MMA consumes 32 bytes of K: +2 descriptor units for K16 (16-bit) and K32 (8-bit)
    assert built_lib.patina_gemm_k_advance_units(16, L.IN_BF16) == 2
    assert built_lib.patina_gemm_k_advance_units(48, L.IN_F16) == 6
    assert built_lib.patina_gemm_k_advance_units(32, L.IN_E4M3) == 2


@pytest.mark.parametrize("tiles_m,tiles_n,group", [(1, 1, 8), (32, 32, 8), (5, 7, 3), (7, 3, 16), (64, 2, 8), (3, 112, 1)])
def test_tile_scheduler_is_a_bijection(built_lib, tiles_m, tiles_n, group):
    seen = set()
    m, n = C.c_uint32(), C.c_uint32()
    for t in range(tiles_m * tiles_n):
        built_lib.patina_gemm_tile_coord(t, tiles_m, tiles_n, group, C.byref(m), C.byref(n))
        assert m.value < tiles_m and n.value < tiles_n
        seen.add((m.value, n.value))
    assert len(seen) == tiles_m * tiles_n
    # within a band M runs fastest
    if tiles_m >= 2 and group >= 2:
        built_lib.patina_gemm_tile_coord(1, tiles_m, tiles_n, group, C.byref(m), C.byref(n))
        assert (m.value, n.value) == (1, 0)


def test_plan_ascending_k_order():
    """k_order = 1 keeps a small problem off the two-accumulator kernels (whose stages hold two
    k-blocks: 7 warps, 3 or 4 stages) and off the cluster split."""
    free = L.plan(L.IN_BF16, L.OUT_BF16, 1024, 1024, 1024)
    assert (free.cta_group, free.block_n, free.stages, free.block) == (1, 64, 4, 224)
    assert free.stage_bytes == 2 * (128 + 64) * 128 and free.tmem_cols == 256
    kept = L.plan(L.IN_BF16, L.OUT_BF16, 1024, 1024, 1024, L.GemmConfig(k_order=1))
    assert kept.block == 192 and kept.stage_bytes == (128 + kept.block_n) * 128
    with pytest.raises(ValueError):   # the two-k-block kernel by its stage count, and ascending k: no such kernel
        L.plan(L.IN_BF16, L.OUT_BF16, 1024, 1024, 1024, L.GemmConfig(1, 128, 3, k_order=1))
    # large problems are summed in ascending k anyway: the setting changes nothing there
    a, b = L.plan(L.IN_BF16, L.OUT_BF16, 8192, 8192, 8192), L.plan(L.IN_BF16, L.OUT_BF16, 8192, 8192, 8192, L.GemmConfig(k_order=1))
    assert (a.cta_group, a.m_sub, a.block_n, a.stages) == (b.cta_group, b.m_sub, b.block_n, b.stages)


def test_plan_half_tile_tail():
    """A last wave that fills at most half of the clusters is run as half tiles."""
    # 8192 x 4096: 16 x 16 = 256 tiles of 512 x 256 on 74 clusters: 3 waves and 34 tiles
    p = L.plan(L.IN_BF16, L.OUT_BF16, 8192, 4096, 14336)
    assert (p.m_sub, p.num_tiles, p.half_tiles, p.grid) == (2, 256, 34, 148)
    # 8192^3: 512 tiles = 6 waves and 68 tiles: more than half a wave, left whole
    assert L.plan(L.IN_BF16, L.OUT_BF16, 8192, 8192, 8192).half_tiles == 0
    # fewer tiles than half the clusters: all of them are split, and more CTAs run
    q = L.plan(L.IN_BF16, L.OUT_BF16, 4096, 1024, 4096, L.GemmConfig(2, 256, 0, 0, 0, 2))
    assert (q.num_tiles, q.half_tiles, q.grid) == (32, 32, 128)
    # one accumulator sub-tile per CTA: nothing to split
    assert L.plan(L.IN_BF16, L.OUT_BF16, 8192, 4096, 14336, L.GemmConfig(2, 256, 0, 0, 0, 1)).half_tiles == 0
    # a capped grid changes the waves: 6 tiles on 4 clusters leave 2, on 2 clusters none
    assert L.plan(L.IN_BF16, L.OUT_BF16, 1536, 512, 320, L.GemmConfig(2, 256, 0, 0, 8, 2)).half_tiles == 2
    assert L.plan(L.IN_BF16, L.OUT_BF16, 1536, 512, 320, L.GemmConfig(2, 256, 0, 0, 4, 2)).half_tiles == 0


def test_plan_headline_shape():
    p = L.plan(L.IN_BF16, L.OUT_BF16, 8192, 8192, 8192)
    assert (p.cta_group, p.m_sub, p.block_n, p.cluster, p.tile_m) == (2, 2, 256, 2, 512)
    assert (p.tiles_m, p.tiles_n, p.num_tiles, p.k_blocks) == (16, 32, 512, 128)
    assert p.grid == 148 and p.block == 352 and p.tmem_cols == 512
    assert p.smem_bytes <= 232448
    # bytes the full barrier expects == bytes of the TMA boxes that land on it
    # (the invariant the reference's verifier enforces, mlir/lib/PatinaOps.cpp:587-614):
    # per CTA two 128-row A slabs and 128 rows of B, 128 bytes of K each, times two CTAs
    assert p.stage_bytes == 2 * 128 * 128 + 128 * 128 and p.expect_tx_bytes == 2 * p.stage_bytes
    q = L.plan(L.IN_BF16, L.OUT_BF16, 8192, 8192, 8192, L.GemmConfig(2, 256, 0, 0, 0, 0))
    assert (q.m_sub, q.tile_m, q.num_tiles, q.block, q.tmem_cols, q.stages) == (1, 256, 1024, 192, 512, 6)
    assert q.stage_bytes == 128 * 128 + 128 * 128 and q.expect_tx_bytes == 2 * q.stage_bytes


def test_plan_variants():
    cfg = L.GemmConfig(1, 256, 0, 0, 0)
    p = L.plan(L.IN_BF16, L.OUT_BF16, 1000, 776, 520, cfg)
    assert (p.cta_group, p.block_n, p.tiles_m, p.tiles_n, p.k_blocks) == (1, 256, 8, 4, 9)
    assert p.grid == 32 and p.expect_tx_bytes == 128 * 128 + 256 * 128
    p = L.plan(L.IN_E4M3, L.OUT_BF16, 8192, 8192, 8192)
    assert p.k_blocks == 64
    p = L.plan(L.IN_F16, L.OUT_F32, 128, 128, 4096)
    assert p.num_tiles == 1 and p.grid == p.cluster
    cfg = L.GemmConfig(2, 256, 0, 0, 20)
    assert L.plan(L.IN_BF16, L.OUT_BF16, 8192, 8192, 64, cfg).grid == 20
    with pytest.raises(ValueError):
        L.plan(L.IN_BF16, L.OUT_F32, 128, 128, 128)          # unsupported type pair
    with pytest.raises(ValueError):
        L.plan(L.IN_BF16, L.OUT_BF16, 128, 128, 128, L.GemmConfig(4, 256, 0, 0, 0))
    with pytest.raises(ValueError):
        L.plan(L.IN_F16, L.OUT_F32, 128, 128, 128, L.GemmConfig(2, 256, 0, 0, 0, 2))  # no such f16 kernel
    p = L.plan(L.IN_BF16, L.OUT_BF16, 4096, 4096, 4096, L.GemmConfig(2, 128, 0, 0, 0, 2))
    assert (p.tile_m, p.tmem_cols, p.block) == (512, 512, 352)


def test_planner_picks_match_what_was_measured_fastest():
    """The planner's time model (tile speed x waves, a partly filled last wave costing less)
    against shapes whose alternatives were timed on a B200: the pick must be the measured
    winner. Tile widths in steps of 16 columns: every stage stays a whole number of 1 KB
    swizzle atoms and the instruction's N a multiple of 16."""
    picks = {
        (8192, 8192, 8192): (2, 2, 256),      # 6.92 waves of 512 x 256
        (4096, 4096, 4096): (2, 2, 240),      # 144 tiles = two waves of 74 pairs instead of 128 + idle
        (8192, 3584, 8192): (2, 2, 224),      # 1/8 of a 28672-wide projection: 3 waves and 34 tiles, those as
                                              # half tiles: 318 vs 324 (208, no tail) vs 326 us (256)
        (8192, 1792, 4096): (2, 2, 208),
        (8192, 14336, 4096): (2, 2, 240),
        (8192, 4096, 4096): (2, 2, 256),      # 3 waves and 34 tiles of 512 x 256, those as half tiles: 181.0 us;
                                              # 256 x 256 pair tiles (6.92 waves) 180.1
        (8192, 512, 4096): (1, 1, 256),       # one wave, short K: 128 lone CTAs 25.6 us, 64 pairs 27.9 us
        (8192, 512, 6144): (2, 1, 256),       # longer K: the pair is ahead again (41.8 vs 44.0 us)
        (2048, 2048, 2048): (1, 1, 256),      # 15.3 vs 17.4 us (128 x 128 tiles with two accumulators: 18.4)
        # at most one wave of 128 x 128 tiles: two k-blocks per stage, two accumulators
        (1024, 1024, 1024): (1, 1, 64),       # 6.7 us; 128 x 128 tiles 7.2; one accumulator 9.2
        (512, 512, 512): (1, 1, 64),          # 5.1 vs 5.5
        (2048, 1024, 1024): (1, 1, 128),      # 7.7 vs 10.3 on 128 x 64 tiles (two waves) vs 9.9 on 128 x 256
        (1024, 2048, 2048): (1, 1, 128),      # 10.7 vs 15.7
        (1536, 1536, 4096): (1, 1, 128),      # 17.7 vs 27.3
    }
    for shape, want in picks.items():
        p = L.plan(L.IN_BF16, L.OUT_BF16, *shape)
        assert (p.cta_group, p.m_sub, p.block_n) == want, (shape, (p.cta_group, p.m_sub, p.block_n))
        assert p.stage_bytes % 1024 == 0 and p.block_n % 16 == 0
        assert p.expect_tx_bytes == p.cta_group * p.stage_bytes
        assert p.smem_bytes <= 232448
    # every width is reachable by an explicit request and keeps the same invariants
    for bn in (256, 240, 224, 208, 192, 176, 160, 128):
        p = L.plan(L.IN_BF16, L.OUT_BF16, 8192, 8192, 8192, L.GemmConfig(2, bn, 0, 0, 0, 2))
        assert p.block_n == bn and p.tiles_n == -(-8192 // bn) and p.stage_bytes == 2 * 16384 + bn // 2 * 128
        assert p.tmem_cols == 512 and p.smem_bytes <= 232448
    # e4m3 output (fused epilogue with scale and amax) has its own kernels
    p = L.plan(L.IN_BF16, L.OUT_E4M3, 8192, 14336, 4096)
    assert (p.cta_group, p.m_sub, p.block_n) == (2, 1, 256)


def test_argument_validation(built_lib):
    ok = dict(in_type=L.IN_BF16, out_type=L.OUT_BF16, A=0x1000, lda=64, B=0x2000, ldb=64, Cp=0x3000,
              ldc=64, M=32, N=64, K=64)
    assert L.validate(**ok) is None
    bad = [({"A": 0}, "A is null"), ({"B": 0}, "B is null"), ({"Cp": 0}, "C is null"),
           ({"A": 0x1008}, "A is not 16-byte aligned"), ({"Cp": 0x3004}, "C is not 16-byte aligned"),
           ({"lda": 60}, "lda=60 < K=64"), ({"lda": 68}, "multiple of 16 bytes"),
           ({"ldc": 32}, "ldc=32 < N=64"), ({"ldc": 66}, "multiple of 16 bytes"),
           ({"M": -1}, "negative dimension"), ({"K": 2 ** 31}, "exceeds"),
           ({"out_type": L.OUT_F32}, "unsupported type pair")]
    for change, needle in bad:
        msg = L.validate(**{**ok, **change})
        assert msg is not None and needle in msg, (change, msg)
    # empty problems never dereference anything
    assert L.validate(**{**ok, "M": 0, "A": 0, "Cp": 0}) is None
    assert L.validate(**{**ok, "K": 0, "A": 0, "B": 0}) is None
    # fp8 rows are bytes: K=48 is a legal pitch, K=40 is not
    assert L.validate(L.IN_E4M3, L.OUT_BF16, 0x1000, 48, 0x2000, 48, 0x3000, 64, 32, 64, 48) is None
    assert "16 bytes" in L.validate(L.IN_E4M3, L.OUT_BF16, 0x1000, 40, 0x2000, 40, 0x3000, 64, 32, 64, 40)


def test_string_free_is_null_safe(built_lib):
    built_lib.patina_gemm_string_free(None)
    assert built_lib.patina_gemm_last_error(None) is None
    assert built_lib.patina_gemm_version().startswith(b"patina-b200-gemm")


def test_no_device_means_unsupported_not_fallback(built_lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    h = C.c_void_p()
    assert built_lib.patina_gemm_context_create(0, C.byref(h)) == L.ERR_UNSUPPORTED_ARCH
    assert not h.value
    import patina_b200
    with pytest.raises(patina_b200.PatinaGemmError):
        patina_b200.GemmContext(0)
    with pytest.raises(patina_b200.PatinaGemmError):
        patina_b200.compute_capability()


def test_inputs_are_deterministic():
    import torch
    from patina_b200 import inputs
    A1, B1 = inputs.make_operands("llm", 64, 48, 32)
    A2, B2 = inputs.make_operands("llm", 64, 48, 32)
    assert torch.equal(A1, A2) and torch.equal(B1, B2) and A1.dtype == torch.bfloat16
    assert 0.5 < float(A1.float().std()) < 1.5 and 0.01 < float(B1.float().std()) < 0.03
    U, _ = inputs.make_operands("uniform", 256, 8, 64)
    assert float(U.float().min()) >= -1 and float(U.float().max()) <= 1
    Aq, sa, Bq, sb = inputs.make_fp8_operands(32, 16, 64)
    assert Aq.dtype == torch.float8_e4m3fn and abs(float(Aq.float().abs().max()) - 448.0) < 1e-3
    assert sa > 0 and sb > 0


# ------------------------------------------------------------------ stream-K partition
@pytest.mark.parametrize("M,N,K,sms", [(16, 28672, 8192, 148), (128, 28672, 8192, 148), (64, 3584, 8192, 148),
                                       (1, 128, 64, 148), (128, 1000, 200, 148), (32, 4096, 14336, 132),
                                       (128, 28672, 8192, 7)])
def test_streamk_partition(built_lib, M, N, K, sms):
    p = L.streamk_plan(L.IN_BF16, M, N, K, sms)
    assert p.m_pad % 16 == 0 and M <= p.m_pad < M + 16
    assert p.tiles == -(-N // 128) and p.k_blocks == -(-K // 64) and p.units == p.tiles * p.k_blocks
    # at least 8 units per CTA; with fewer tiles than CTAs every tile is cut into the same number
    # of ranges (one segment per CTA) when that keeps nine SMs in ten busy
    want = min(sms, -(-p.units // 8))
    if p.tiles < want and p.tiles * (want // p.tiles) * 10 >= want * 9:
        want = p.tiles * (want // p.tiles)
    assert p.grid == want and p.smem_bytes <= 232448
    if (M, N, K, sms) == (64, 3584, 8192, 148):
        assert p.grid == 140                  # 28 tiles x 5 ranges
    assert p.partial_bytes == p.tiles * p.max_contrib * p.m_pad * 128 * 4 and p.counter_bytes == p.tiles * 4
    b, e = C.c_uint64(), C.c_uint64()
    prev_end, lens = 0, []
    for c in range(p.grid):
        built_lib.patina_gemm_streamk_range(c, p.units, p.grid, C.byref(b), C.byref(e))
        assert b.value == prev_end and e.value > b.value          # contiguous, never empty
        prev_end = e.value
        lens.append(e.value - b.value)
        # the owner function inverts the ranges at both ends
        assert built_lib.patina_gemm_streamk_owner(b.value, p.units, p.grid) == c
        assert built_lib.patina_gemm_streamk_owner(e.value - 1, p.units, p.grid) == c
    assert prev_end == p.units and max(lens) - min(lens) <= 1
    # contributors of every tile fit the slots reserved for it
    for t in range(0, p.tiles, max(1, p.tiles // 97)):
        first = built_lib.patina_gemm_streamk_owner(t * p.k_blocks, p.units, p.grid)
        last = built_lib.patina_gemm_streamk_owner((t + 1) * p.k_blocks - 1, p.units, p.grid)
        assert 1 <= last - first + 1 <= p.max_contrib


def test_streamk_plan_rejects_wide_m():
    with pytest.raises(ValueError):
        L.streamk_plan(L.IN_BF16, 129, 4096, 4096)
    assert L.streamk_plan(L.IN_F16, 16, 4096, 4096).tiles == 32    # f16 (-> f32): the reference's types


def test_automatic_choice_between_the_two_kernels(built_lib):
    """Which kernel a call without configuration takes for M <= 128, against the shapes that were
    timed on a B200 (microseconds: stream-K / large-tile)."""
    chosen = lambda M, N, K, t=L.IN_BF16, o=L.OUT_BF16: built_lib.patina_gemm_streamk_chosen(t, o, M, N, K, 148)
    assert chosen(16, 28672, 8192) == 1        # 75.3 / 77
    assert chosen(32, 28672, 8192) == 0        # 80.4 / 78.3
    assert chosen(64, 28672, 8192) == 0        # 88 / 78: enough 256-wide tiles for most SMs
    assert chosen(128, 28672, 8192) == 0       # 98 / 79
    assert chosen(64, 3584, 8192) == 1         # 16.8 / 23 (an 8-way shard: 14 tiles of 256)
    assert chosen(128, 3584, 8192) == 1        # 17.8 / 53
    assert chosen(128, 128, 4096) == 1         # 9.4 / 22: one tile, deep K
    assert chosen(64, 256, 8192) == 1          # 10.0 / 45
    assert chosen(128, 2048, 1024) == 0        # 9.2 / 8.6: K too short to be worth cutting
    assert chosen(16, 24, 40) == 0
    assert chosen(129, 3584, 8192) == 0        # the stream-K kernel holds at most 128 rows of X
    assert chosen(16, 28672, 8192, L.IN_E4M3) == 1
    assert chosen(128, 128, 4096, L.IN_F16, L.OUT_F32) == 1   # the reference's own types and shape: 9.6 / 15.1
    assert chosen(128, 128, 128, L.IN_F16, L.OUT_F32) == 0    # its test cases (K = 32, 128): one or two k-blocks
    assert chosen(128, 128, 4096, L.IN_F16, L.OUT_BF16) == 0  # no such type pair


def test_block_scaled_encodings(built_lib):
    """The block-scaled (MXFP8) instruction descriptor and the scale-buffer layout. Field
    positions as documented for tcgen05.mma kind::mxf8f6f4.block_scale: B scale id [4,6),
    N >> 3 at bit 17, E8M0 scale format bit 23, M >> 4 at bit 24, A scale id [29,31); the
    reference has no block-scaled path (its idesc 136314896 is the kind::f16 form)."""
    import torch
    from patina_b200 import inputs
    L = built_lib
    assert L.patina_gemm_idesc_mx(128, 256, 0, 0) == (32 << 17) | (1 << 23) | (8 << 24)
    assert L.patina_gemm_idesc_mx(256, 224, 3, 2) == (2 << 4) | (28 << 17) | (1 << 23) | (16 << 24) | (3 << 29)
    assert L.patina_gemm_mx_scale_bytes(128, 128) == 512
    assert L.patina_gemm_mx_scale_bytes(129, 160) == 2 * 2 * 512
    assert L.patina_gemm_mx_scale_bytes(0, 128) == 0
    # the packer and the library's offset function describe the same layout
    rows, K = 300, 416                      # 3 row blocks, 13 scales per row -> 4 atoms along K
    e = torch.arange(rows * (K // 32), dtype=torch.int64).reshape(rows, K // 32)
    e8 = (e % 251).to(torch.uint8)
    packed = inputs.pack_mx_scales(e8, fill=127)
    assert packed.numel() == L.patina_gemm_mx_scale_bytes(rows, K)
    seen = torch.zeros(packed.numel(), dtype=torch.bool)
    for r in (0, 1, 31, 32, 95, 127, 128, 200, 299):
        for kb in range(K // 32):
            off = L.patina_gemm_mx_scale_offset(r, kb, K)
            assert int(packed[off]) == int(e8[r, kb]), (r, kb)
            seen[off] = True
    assert int(packed[L.patina_gemm_mx_scale_offset(299 + 1, 0, K)]) == 127      # padding rows
    assert int(packed[L.patina_gemm_mx_scale_offset(0, 13, K)]) == 127           # padding scales
    # byte position inside an atom: (r % 32) * 16 + (r / 32) * 4 + j
    assert L.patina_gemm_mx_scale_offset(33, 2, 128) == 1 * 16 + 1 * 4 + 2
    assert L.patina_gemm_mx_scale_offset(128 + 5, 4 + 1, 256) == (1 * 2 + 1) * 512 + 5 * 16 + 1


def test_mx_quantiser_round_trip(oracle_mod):
    """quantize_mxfp8 + oracle.mx_dequant: every element within half an e4m3 step of its block's
    scale, blocks scaled independently."""
    import numpy as np
    import torch
    from patina_b200 import inputs
    g = torch.Generator().manual_seed(2)
    x = torch.randn((40, 96), generator=g) * torch.exp2(torch.randint(-5, 6, (40, 3, 1), generator=g).float()).expand(40, 3, 32).reshape(40, 96)
    q, e = inputs.quantize_mxfp8(x)
    back = oracle_mod.mx_dequant(q.view(torch.uint8).numpy(), e.numpy())
    amax = x.reshape(40, 3, 32).abs().amax(dim=2, keepdim=True).expand(40, 3, 32).reshape(40, 96).numpy()
    assert np.all(np.abs(back - x.numpy()) <= amax * 2.0 ** -3)      # e4m3: 3 mantissa bits, scale within 2x of amax/448
    assert np.all(np.abs(back) <= 448.0 * np.ldexp(1.0, e.numpy().astype(np.int32) - 127).repeat(32, axis=1) + 0)


def test_cluster_split_k_choice(built_lib):
    """Which problems get K cut across a cluster: more than 128 rows, so few tiles that even
    128 x 64 ones would leave a third of the SMs without one (above that the two-accumulator
    single-CTA kernels are ahead: timed on a B200, microseconds split / whole), enough k-blocks
    saved per CTA to pay for the exchange; never the skinny shapes (stream-K)."""
    from patina_b200 import lib as Lm
    c = lambda M, N, K: built_lib.patina_gemm_cluster_k_chosen(Lm.IN_BF16, Lm.OUT_BF16, M, N, K, 148)
    assert c(1024, 1024, 1024) == 0          # 16 k-blocks: the exchange costs more than it saves
    assert c(512, 512, 4096) == 4            # 32 tiles of 128 x 64: 13.1 / 14.3
    assert c(512, 1024, 8192) == 4           # 64 tiles: 18.4 / 25.0
    assert c(256, 256, 8192) == 4            # 17.4 / 24.6
    assert c(1024, 1024, 4096) == 0          # 128 tiles: 16.0 / 15.4
    assert c(256, 4096, 4096) == 0           # 16.1 / 15.5
    assert c(1024, 2048, 2048) == 0          # 12.8 / 10.7
    assert c(2048, 2048, 2048) == 0          # 128 tiles: no room for a second CTA per tile
    assert c(8192, 8192, 8192) == 0
    assert c(1024, 1024, 256) == 0           # 4 k-blocks: nothing to save
    assert c(128, 1024, 8192) == 0 and c(16, 28672, 8192) == 0      # skinny paths
    assert c(1024, 1028, 1024) == 0          # N not a multiple of 8
    assert built_lib.patina_gemm_cluster_k_chosen(Lm.IN_E4M3, Lm.OUT_BF16, 1024, 1024, 1024, 148) == 0

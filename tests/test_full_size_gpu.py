"""Parity at the stated sizes of the benchmark configurations, through the C ABI, on a B200.

The oracle (the reference's double-accumulating CPU GEMM restated, harness/gemm_check.cpp:165-178)
cannot produce a full 8192 x 28672 x 8192 result in test time, so every shape is checked on
samples that cover what can go wrong in a tiled kernel:

  * at least 64 whole rows of C (boundary rows of the row tiles plus random ones),
  * at least 64 whole columns of C (boundary columns of the column tiles plus random ones),
  * the four corners of every tile of the launch plan (a superset of "every 16th tile"): the
    grid of first/last tile rows x first/last tile columns,

each against bf16(alpha * double-accumulated reference) with the suite's tolerance
(|d| <= 1e-2 * max|ref| elementwise, relative Frobenius error <= 1e-3), and on properties that
need no oracle: a column shard equals the same columns of the full result bit for bit.
The tile plan is the library's automatic choice, so the 240-, 224- and 208-wide tiles the planner
picks for these widths run at size here.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

ELEM_TOL, FRO_TOL = 1e-2, 1e-3


@pytest.fixture(scope="module")
def ctx():
    import patina_b200
    c = patina_b200.GemmContext(0)
    yield c
    c.close()


def widen(oracle_mod, t: torch.Tensor) -> np.ndarray:
    t = t.contiguous()
    if t.dtype == torch.bfloat16:
        return oracle_mod.bf16_bits_to_f32(t.view(torch.int16).numpy().view(np.uint16))
    return oracle_mod.e4m3_bits_to_f32(t.view(torch.uint8).numpy())


def sample_indices(extent: int, tile: int, n_random: int, rng) -> np.ndarray:
    """First and last index of the first, second and last tile, plus n_random random ones."""
    edges = [0, tile - 1, tile, 2 * tile - 1, extent - tile, extent - 1]
    edges = [e for e in edges if 0 <= e < extent]
    return np.unique(np.concatenate([edges, rng.integers(0, extent, n_random)])).astype(np.int64)


def tile_edges(extent: int, tile: int) -> np.ndarray:
    first = np.arange(0, extent, tile)
    last = np.minimum(first + tile - 1, extent - 1)
    return np.unique(np.concatenate([first, last])).astype(np.int64)


def check_samples(oracle_mod, out: torch.Tensor, A: torch.Tensor, B: torch.Tensor, alpha: float,
                  tile_m: int, tile_n: int, what: str, seed: int = 5):
    """Rows, columns and tile corners of `out` against the oracle. Returns the three Frobenius errors."""
    M, N = out.shape
    wa, wb = widen(oracle_mod, A), widen(oracle_mod, B)
    rng = np.random.default_rng(seed)
    errs = []

    def compare(got: torch.Tensor, ref: np.ndarray, label: str):
        want = oracle_mod.scale_round_bf16(ref, alpha)
        ok, me, mx, fr = oracle_mod.compare_norm(got.float().cpu().numpy(), want, ELEM_TOL, FRO_TOL)
        assert ok, f"{what} {label}: max|d|={me:.4g} max|ref|={mx:.4g} fro_rel={fr:.4g}"
        errs.append(fr)

    rows = sample_indices(M, tile_m, 60, rng)
    assert rows.size >= 64
    compare(out[torch.from_numpy(rows).cuda()], oracle_mod.ref_gemm_tn(wa, wb, rows=rows), f"{rows.size} rows")
    cols = sample_indices(N, tile_n, 60, rng)
    assert cols.size >= 64
    # columns of C = rows of (B A^T): the same double accumulation over k, same order
    ref_t = oracle_mod.ref_gemm_tn(wb, wa, rows=cols)
    compare(out[:, torch.from_numpy(cols).cuda()], ref_t.T.copy(), f"{cols.size} columns")
    er, ec = tile_edges(M, tile_m), tile_edges(N, tile_n)
    ref_c = oracle_mod.ref_gemm_tn(wa, np.ascontiguousarray(wb[ec]), rows=er)
    got_c = out[torch.from_numpy(er).cuda()][:, torch.from_numpy(ec).cuda()]
    compare(got_c, ref_c, f"corners of {er.size // 2} x {ec.size // 2} tiles")
    return errs


def plan_of(M, N, K, in_type=None):
    from patina_b200 import lib as L
    return L.plan(L.IN_BF16 if in_type is None else in_type, L.OUT_BF16, M, N, K)


# ------------------------------------------------------------ bf16, square
def test_bf16_4096_cubed(ctx, oracle_mod):
    """4096^3, N(0,1)*0.1 operands (the second size of the square bf16 configuration)."""
    from patina_b200 import inputs
    n = 4096
    A, B = inputs.make_operands("normal_0p1", n, n, n)
    out = ctx.gemm_tn(A.cuda(), B.cuda())
    ctx.status()
    p = plan_of(n, n, n)
    check_samples(oracle_mod, out, A, B, 1.0, p.tile_m, p.block_n, "4096^3")


# ------------------------------------------------ LLM projections (bf16, M = 8192 tokens)
@pytest.mark.parametrize("N,K", [(4096, 4096), (14336, 4096), (4096, 14336), (28672, 8192)])
def test_llm_projection_full_size(ctx, oracle_mod, N, K):
    """The four projection shapes at full size: activations N(0,1), weights N(0,0.02), the
    library's own tile choice."""
    from patina_b200 import inputs
    M = 8192
    A, B = inputs.make_operands("llm", M, N, K, seed=N // 64 + K)
    out = ctx.gemm_tn(A.cuda(), B.cuda())
    ctx.status()
    p = plan_of(M, N, K)
    check_samples(oracle_mod, out, A, B, 1.0, p.tile_m, p.block_n, f"projection {M}x{N}x{K}")


def test_llm_projection_column_shards_equal_the_full_result(ctx, oracle_mod):
    """What N-sharding over GPUs relies on, on a projection shape: every rank's column shard
    (its own launch, its own tile plan: 1792 columns take 224-wide tiles, 3584 take 208-wide
    ones) holds exactly the bits the unsharded launch produces for those columns; one shard is
    also checked against the oracle at its own tile plan."""
    from patina_b200 import inputs, sharded
    M, N, K = 8192, 14336, 4096
    A, B = inputs.make_operands("llm", M, N, K, seed=77)
    dA, dB = A.cuda(), B.cuda()
    full = ctx.gemm_tn(dA, dB)
    ctx.status()
    for world in (2, 4, 8):
        for rank in sorted({0, world // 2, world - 1}):
            n0, n1 = sharded.column_shard(N, world, rank)
            shard = ctx.gemm_tn(dA, dB[n0:n1])
            ctx.status()
            assert torch.equal(shard, full[:, n0:n1]), f"shard {rank} of {world}"
    n0, n1 = sharded.column_shard(N, 8, 5)
    shard = ctx.gemm_tn(dA, dB[n0:n1])
    ctx.status()
    p = plan_of(M, n1 - n0, K)
    check_samples(oracle_mod, shard, A, B[n0:n1], 1.0, p.tile_m, p.block_n, "shard 5 of 8")


def test_widest_projection_shard_of_eight(ctx, oracle_mod):
    """One GPU's share of the 28672 x 8192 projection split over 8 GPUs (3584 columns)."""
    from patina_b200 import inputs
    M, N, K = 8192, 3584, 8192
    A, B = inputs.make_operands("llm", M, N, K, seed=3584)
    out = ctx.gemm_tn(A.cuda(), B.cuda())
    ctx.status()
    p = plan_of(M, N, K)
    check_samples(oracle_mod, out, A, B, 1.0, p.tile_m, p.block_n, f"shard {M}x{N}x{K}")


# ------------------------------------------------------------------ fp8 e4m3
def test_fp8_8192_cubed(ctx, oracle_mod):
    """fp8 e4m3, 8192^3: operands quantised from N(0,1) with per-tensor scales amax/448; the
    result is compared after dequantisation (bf16 of sa*sb * sum qa*qb in double)."""
    from patina_b200 import inputs, lib as L
    n = 8192
    Aq, sa, Bq, sb = inputs.make_fp8_operands(n, n, n)
    out = ctx.gemm_fp8e4m3_tn(Aq.cuda(), Bq.cuda(), sa, sb)
    ctx.status()
    p = plan_of(n, n, n, L.IN_E4M3)
    check_samples(oracle_mod, out, Aq, Bq, sa * sb, p.tile_m, p.block_n, "fp8 8192^3")


def test_fp8_16384_shard_of_eight(ctx, oracle_mod):
    """One GPU's share of the fp8 16384^3 problem split over 8 GPUs: M = K = 16384, 2048 columns
    (128 k-blocks of 128 bytes per tile on the 512 x 256 e4m3 kernel)."""
    from patina_b200 import inputs, lib as L
    M, N, K = 16384, 2048, 16384
    A32, B32 = inputs.make_operands("unit_normal", M, N, K, dtype=torch.float32, seed=16384)
    Aq, sa = inputs.quantize_e4m3(A32)
    Bq, sb = inputs.quantize_e4m3(B32)
    del A32, B32
    out = ctx.gemm_fp8e4m3_tn(Aq.cuda(), Bq.cuda(), sa, sb)
    ctx.status()
    p = plan_of(M, N, K, L.IN_E4M3)
    check_samples(oracle_mod, out, Aq, Bq, sa * sb, p.tile_m, p.block_n, "fp8 16384 x 2048 x 16384 shard")

"""Block-scaled fp8 (MXFP8: e4m3 elements, one E8M0 scale per 32 K elements of a row) through
`patina_gemm_mxfp8_tn`, against the CPU oracle: the dequantised operands (exact in float32) go
through the reference's double-accumulating loop (harness/gemm_check.cpp:165-178) and the result
is rounded once to bf16. Tolerance: |d| <= 1e-2 * max|ref| elementwise and relative Frobenius
error <= 1e-3, the same rule as the per-tensor fp8 path (compared after dequantisation).

The operands are drawn so that neighbouring 32-element blocks and neighbouring rows carry very
different scales (each block is multiplied by its own power of two between 2^-6 and 2^6 before
quantisation): a kernel that picked the wrong byte of a scale column, the wrong row's scale or
the wrong atom would be off by factors of two, not by rounding.
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


def make(M, N, K, seed):
    """Operands whose blocks differ in magnitude by up to 2^12; returns quantised tensors and scales."""
    from patina_b200 import inputs
    g = torch.Generator().manual_seed(seed)

    def draw(rows):
        x = torch.randn((rows, K // 32, 32), generator=g)
        lift = torch.randint(-6, 7, (rows, K // 32, 1), generator=g).float()
        return (x * torch.exp2(lift)).reshape(rows, K)
    Aq, ea = inputs.quantize_mxfp8(draw(M))
    Bq, eb = inputs.quantize_mxfp8(draw(N))
    return Aq, ea, Bq, eb


def expect(oracle_mod, Aq, ea, Bq, eb, alpha=1.0, rows=None):
    wa = oracle_mod.mx_dequant(Aq.view(torch.uint8).numpy(), ea.numpy())
    wb = oracle_mod.mx_dequant(Bq.view(torch.uint8).numpy(), eb.numpy())
    return oracle_mod.scale_round_bf16(oracle_mod.ref_gemm_tn(wa, wb, rows=rows), alpha)


def run(ctx, Aq, ea, Bq, eb, alpha=1.0, config=None, out=None):
    from patina_b200 import inputs
    got = ctx.gemm_mxfp8_tn(Aq.cuda(), inputs.pack_mx_scales(ea).cuda(), Bq.cuda(), inputs.pack_mx_scales(eb).cuda(),
                            alpha=alpha, config=config, out=out)
    ctx.status()
    return got


def check(oracle_mod, got, want, what):
    ok, me, mx, fr = oracle_mod.compare_norm(got.float().cpu().numpy(), want, ELEM_TOL, FRO_TOL)
    assert ok, f"{what}: max|d|={me:.4g} max|ref|={mx:.4g} fro_rel={fr:.4g}"


def mx_cfgs():
    from patina_b200 import GemmConfig
    return {"auto": None, "1cta_n128": GemmConfig(1, 128, 0, 0, 0), "1cta_n192": GemmConfig(1, 192, 0, 0, 0),
            "pair_n192": GemmConfig(2, 192, 0, 0, 0), "pair_n256": GemmConfig(2, 256, 0, 0, 0),
            "pair_2sub_n192": GemmConfig(2, 192, 0, 0, 0, 2)}


@pytest.mark.parametrize("name", ["1cta_n128", "1cta_n192", "pair_n192", "pair_n256", "pair_2sub_n192", "auto"])
def test_mxfp8_every_tile(ctx, oracle_mod, name):
    """One k-block and one tile, then many tiles and k-blocks with stage wraps, for every tile
    configuration (192-wide tiles start every other tile 64 rows into a scale atom of B)."""
    cfg = mx_cfgs()[name]
    for (M, N, K) in [(128, 128, 128), (256, 896, 1024), (1024, 1344, 2048)]:
        Aq, ea, Bq, eb = make(M, N, K, seed=M + N + K)
        got = run(ctx, Aq, ea, Bq, eb, config=cfg)
        check(oracle_mod, got, expect(oracle_mod, Aq, ea, Bq, eb), f"{name} {M}x{N}x{K}")


def test_mxfp8_half_tile_tail_wave(ctx, oracle_mod):
    """The two-sub-tile kernel splits the tiles of a short last wave into half tiles (6 tiles on
    4 clusters: the last 2 become 4 halves): equal, bit for bit, to the launch on one cluster,
    which splits nothing, and within tolerance of the oracle."""
    from patina_b200 import GemmConfig
    M, N, K = 1500, 384, 1152
    Aq, ea, Bq, eb = make(M, N, K, seed=11)
    split = run(ctx, Aq, ea, Bq, eb, alpha=0.5, config=GemmConfig(2, 192, 0, 0, 8, 2))
    whole = run(ctx, Aq, ea, Bq, eb, alpha=0.5, config=GemmConfig(2, 192, 0, 0, 2, 2))
    check(oracle_mod, split, expect(oracle_mod, Aq, ea, Bq, eb, alpha=0.5), "half-tile tail")
    assert torch.equal(split, whole)


@pytest.mark.parametrize("M,N,K", [(1, 8, 32), (200, 392, 352), (129, 257, 96), (520, 1000, 4128)])
def test_mxfp8_ragged_shapes(ctx, oracle_mod, M, N, K):
    """Ragged M, N and K (K a multiple of 32 but not of 128: the last scale atom is partly
    padding), alpha, padded output pitch with untouched columns behind N."""
    Aq, ea, Bq, eb = make(M, N, K, seed=7 * M + N)
    want = expect(oracle_mod, Aq, ea, Bq, eb, alpha=0.5)
    for name, cfg in mx_cfgs().items():
        ldc = (N + 7) // 8 * 8 + 8
        full = torch.full((M, ldc), float("nan"), dtype=torch.bfloat16, device="cuda")
        run(ctx, Aq, ea, Bq, eb, alpha=0.5, config=cfg, out=full[:, :N])
        check(oracle_mod, full[:, :N], want, f"{name} {M}x{N}x{K}")
        assert bool(torch.isnan(full[:, N:]).all()), f"{name}: columns behind N were written"


def test_mxfp8_equals_per_tensor_fp8_when_all_scales_are_one(ctx, oracle_mod):
    """With every scale 2^0 the block-scaled product is the plain e4m3 product: it must agree with
    the per-tensor fp8 entry point (scale 1) far inside the tolerance."""
    from patina_b200 import inputs
    M, N, K = 512, 768, 1024
    Aq, _, Bq, _ = inputs.make_fp8_operands(M, N, K, seed=5)
    ones_a = torch.full((M, K // 32), 127, dtype=torch.uint8)
    ones_b = torch.full((N, K // 32), 127, dtype=torch.uint8)
    got = run(ctx, Aq, ones_a, Bq, ones_b)
    plain = ctx.gemm_fp8e4m3_tn(Aq.cuda(), Bq.cuda(), 1.0, 1.0)
    ctx.status()
    check(oracle_mod, got, plain.float().cpu().numpy(), "all-ones scales vs per-tensor fp8")


def test_mxfp8_8192_cubed_samples(ctx, oracle_mod):
    """8192^3 at the library's own tile choice: 64 sampled rows against the oracle."""
    from patina_b200 import inputs
    n = 8192
    Aq, ea, Bq, eb = inputs.make_mxfp8_operands(n, n, n)
    got = run(ctx, Aq, ea, Bq, eb)
    rng = np.random.default_rng(5)
    rows = np.unique(np.concatenate([[0, 127, 128, 255, 256, 511, 512, n - 1], rng.integers(0, n, 58)])).astype(np.int64)
    want = expect(oracle_mod, Aq, ea, Bq, eb, rows=rows)
    check(oracle_mod, got[torch.from_numpy(rows).cuda()], want, "8192^3 sampled rows")


def test_mxfp8_arguments(ctx):
    import patina_b200
    Aq = torch.zeros((64, 48), dtype=torch.uint8, device="cuda")
    sf = torch.full((4096,), 127, dtype=torch.uint8, device="cuda")
    with pytest.raises(patina_b200.PatinaGemmError, match="multiple of 32"):
        ctx.gemm_mxfp8_tn(Aq, sf, Aq, sf)
    Aq = torch.zeros((64, 64), dtype=torch.uint8, device="cuda")
    with pytest.raises(patina_b200.PatinaGemmError, match="scale buffers"):
        ctx.gemm_mxfp8_tn(Aq, sf[:16], Aq, sf)
    ctx.status()

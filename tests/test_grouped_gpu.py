"""Grouped GEMM (`patina_gemm_bf16_tn_grouped`): ragged groups that share N and K, one launch.

The oracle is the reference's CPU GEMM restated (harness/gemm_check.cpp:165-178), run once per
group on that group's rows and weights; the tolerance is the bf16 rule of the other parity tests
(elementwise 1e-2 * max|C_ref|, relative Frobenius 1e-3 after bf16 rounding of the reference).
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    import patina_b200
    c = patina_b200.GemmContext(0)
    yield c
    c.close()


def widen(oracle_mod, t):
    return oracle_mod.bf16_bits_to_f32(t.view(torch.int16).numpy().view(np.uint16))


def check_norm(oracle_mod, got, want, what):
    ok, max_abs, max_ref, fro = oracle_mod.compare_norm(got.float().cpu().numpy(), want, 1e-2, 1e-3)
    assert ok, f"{what}: max abs {max_abs:.3e} (max ref {max_ref:.3e}), rel fro {fro:.3e}"


def configs():
    from patina_b200 import GemmConfig
    return {"auto": None, "1cta": GemmConfig(1, 0, 0, 0, 0, 1), "pair": GemmConfig(2, 0, 0, 0, 0, 1),
            "pair_2sub": GemmConfig(2, 0, 0, 0, 0, 2)}


def make_problem(rows, N, K, seed, extra_rows=0):
    from patina_b200 import inputs
    total = int(sum(max(r, 0) for r in rows)) + extra_rows
    A, _ = inputs.make_operands("llm", max(total, 1), 1, K, seed=seed)
    A = A[:total]
    _, B = inputs.make_operands("llm", 1, len(rows) * N, K, seed=seed + 1)
    return A, B.view(len(rows), N, K)


def expected_blocks(oracle_mod, A, B, rows, alpha=1.0):
    out, r0 = [], 0
    for g, r in enumerate(rows):
        r = max(r, 0)
        if r:
            ref = oracle_mod.ref_gemm_tn(widen(oracle_mod, A[r0:r0 + r]), widen(oracle_mod, B[g]))
            out.append((r0, r, oracle_mod.scale_round_bf16(ref, alpha)))
        r0 += r
    return out


@pytest.mark.parametrize("rows,N,K", [([300, 0, 1, 129, 512, 37, 5], 520, 264),
                                      ([31, 33, 32, 64, 1], 256, 72),
                                      ([1000, 600], 776, 520),
                                      ([70, 33, 200], 261, 72)])   # N not a multiple of 8 columns
def test_grouped_matches_oracle(ctx, oracle_mod, rows, N, K):
    """Every group against the oracle, on every tile height; rows behind the last group and
    the padding columns of C keep their contents; empty and one-row groups; group ends that
    fall inside a 32-row store box."""
    A, B = make_problem(rows, N, K, seed=len(rows) * 100 + N, extra_rows=40)
    total = A.shape[0]
    ldc = (N + 15) // 8 * 8
    want = expected_blocks(oracle_mod, A, B, rows, alpha=0.5)
    d_rows = torch.tensor(rows, dtype=torch.int32, device="cuda")
    dA, dB = A.cuda(), B.cuda()
    for name, cfg in configs().items():
        Cfull = torch.full((total, ldc), 7.0, dtype=torch.bfloat16, device="cuda")
        ctx.gemm_bf16_tn_grouped(dA, dB, d_rows, out=Cfull[:, :N], alpha=0.5, config=cfg)
        ctx.status()
        for r0, r, ref in want:
            check_norm(oracle_mod, Cfull[r0:r0 + r, :N], ref, f"{name} group at row {r0}")
        used = sum(rows)
        assert bool((Cfull[used:, :] == 7.0).all()), f"{name}: rows behind the last group were written"
        assert bool((Cfull[:, N:] == 7.0).all()), f"{name}: padding columns were written"


def test_grouped_equals_separate_calls(ctx):
    """Same kernel, same accumulation order: one grouped launch gives the bits that one plain
    call per group gives with the same tile shape."""
    from patina_b200 import GemmConfig
    rng = np.random.default_rng(5)
    rows = [int(x) for x in rng.multinomial(4096, [0.3, 0.05, 0.2, 0.0, 0.15, 0.1, 0.12, 0.08])]
    N, K = 1024, 512
    A, B = make_problem(rows, N, K, seed=3)
    dA, dB = A.cuda(), B.cuda()
    d_rows = torch.tensor(rows, dtype=torch.int32, device="cuda")
    for g_cfg, p_cfg in [(GemmConfig(2, 0, 0, 0, 0, 2), GemmConfig(2, 256, 0, 0, 0, 2)),
                         (GemmConfig(1, 0, 0, 0, 0, 1), GemmConfig(1, 256, 0, 0, 0, 1))]:
        out = ctx.gemm_bf16_tn_grouped(dA, dB, d_rows, config=g_cfg)
        ctx.status()
        r0 = 0
        for g, r in enumerate(rows):
            if r:
                single = ctx.gemm_tn(dA[r0:r0 + r], dB[g], config=p_cfg)
                ctx.status()
                assert torch.equal(out[r0:r0 + r], single), f"group {g}"
            r0 += r


def test_grouped_counts_beyond_the_buffer_are_dropped(ctx, oracle_mod):
    """Row counts that add up to more than A and C hold: the excess is ignored, nothing past
    the buffers is touched (C sits inside a larger sentinel-filled allocation)."""
    rows, N, K = [100, 200, 300], 256, 128
    A, B = make_problem(rows, N, K, seed=8)
    total = 250                      # the buffers end inside group 1
    guard = torch.full((total + 64, N), 3.0, dtype=torch.bfloat16, device="cuda")
    d_rows = torch.tensor(rows, dtype=torch.int32, device="cuda")
    ctx.gemm_bf16_tn_grouped(A[:total].cuda().contiguous(), B.cuda(), d_rows, out=guard[:total])
    ctx.status()
    want = expected_blocks(oracle_mod, A[:total], B, [100, 150])
    for r0, r, ref in want:
        check_norm(oracle_mod, guard[r0:r0 + r], ref, f"group at row {r0}")
    assert bool((guard[total:] == 3.0).all())


def test_grouped_fp8_with_a_scale_per_group(ctx, oracle_mod):
    """e4m3 operands, one weight scale per group: C_g = sa * sb[g] * (A_g B_g^T), against the
    oracle on the dequantised operands (the bound of the fp8 configurations: elementwise
    1e-2 * max|C_ref|, relative Frobenius 1e-3 after bf16 rounding of the reference)."""
    from patina_b200 import inputs
    rows, N, K = [200, 3, 0, 321], 392, 336
    total = sum(rows)
    Aq, sa, _, _ = inputs.make_fp8_operands(total, 8, K)
    Bqs, sbs = [], []
    for g in range(len(rows)):
        _, _, Bq, sb = inputs.make_fp8_operands(8, N, K, seed=40 + g)
        Bqs.append(Bq)
        sbs.append(sb * (1.0 + g))            # clearly different factors per group
    Bq = torch.stack(Bqs)
    d_rows = torch.tensor(rows, dtype=torch.int32, device="cuda")
    d_sb = torch.tensor(sbs, dtype=torch.float32, device="cuda")
    w8 = lambda t: oracle_mod.e4m3_bits_to_f32(t.view(torch.uint8).numpy())
    for name, cfg in configs().items():
        out = ctx.gemm_fp8e4m3_tn_grouped(Aq.cuda(), Bq.cuda(), d_rows, sa, d_sb, config=cfg)
        ctx.status()
        r0 = 0
        for g, r in enumerate(rows):
            if r:
                ref = oracle_mod.ref_gemm_tn(w8(Aq[r0:r0 + r]), w8(Bq[g]))
                check_norm(oracle_mod, out[r0:r0 + r], oracle_mod.scale_round_bf16(ref, sa * sbs[g]),
                           f"{name} fp8 group {g}")
            r0 += r


def test_grouped_invalid_arguments(ctx):
    import patina_b200
    A = torch.zeros((64, 64), dtype=torch.bfloat16, device="cuda")
    B = torch.zeros((129 * 8, 64), dtype=torch.bfloat16, device="cuda")
    rows = torch.zeros(129, dtype=torch.int32, device="cuda")
    with pytest.raises(patina_b200.PatinaGemmError, match="0..128 groups"):
        ctx.gemm_bf16_tn_grouped(A, B, rows)
    with pytest.raises(patina_b200.PatinaGemmError, match="CUDA tensors"):
        ctx.gemm_bf16_tn_grouped(A.cpu(), B, rows)
    # no groups, no rows: nothing to do, no error
    empty = ctx.gemm_bf16_tn_grouped(A[:0], B[:0], rows[:0], out=torch.empty((0, 8), dtype=torch.bfloat16, device="cuda"))
    assert empty.shape[0] == 0
    ctx.status()

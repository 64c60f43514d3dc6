"""Parity of the CUDA path against the CPU oracle, through the C ABI, on a B200.

Tolerances (stated where used):
  * reference-shape case (f16 in, f32 out, 128x128xK): the reference harness's own
    rule, zero elements with abs_err > 1e-3 AND abs_err/max(1,|ref|) > 1e-3
    (harness/gemm_check.cpp:303-321);
  * bf16 / fp8 cases: |d| <= 1e-2 * max|C_ref| elementwise and relative Frobenius
    error <= 1e-3, with C_ref = bf16(alpha * double-accumulated reference).
"""
import ctypes as C

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
    """Exact float32 view of a host f16/bf16/e4m3 tensor, via the oracle's own converters."""
    t = t.contiguous()
    if t.dtype == torch.bfloat16:
        return oracle_mod.bf16_bits_to_f32(t.view(torch.int16).numpy().view(np.uint16))
    if t.dtype == torch.float16:
        return oracle_mod.f16_bits_to_f32(t.view(torch.int16).numpy().view(np.uint16))
    return oracle_mod.e4m3_bits_to_f32(t.view(torch.uint8).numpy())


def expect_bf16(oracle_mod, A, B, alpha=1.0, rows=None):
    ref = oracle_mod.ref_gemm_tn(widen(oracle_mod, A), widen(oracle_mod, B), rows=rows)
    return oracle_mod.scale_round_bf16(ref, alpha)


def check_norm(oracle_mod, got: torch.Tensor, want: np.ndarray, what=""):
    ok, me, mx, fr = oracle_mod.compare_norm(got.float().cpu().numpy(), want, ELEM_TOL, FRO_TOL)
    assert ok, f"{what}: max|d|={me:.4g} max|ref|={mx:.4g} fro_rel={fr:.4g}"
    return fr


def cfgs():
    from patina_b200 import GemmConfig
    return {"auto": None, "1cta_n256": GemmConfig(1, 256, 0, 0, 0), "1cta_n128": GemmConfig(1, 128, 0, 0, 0),
            "pair_n256": GemmConfig(2, 256, 0, 0, 0), "pair_n128": GemmConfig(2, 128, 0, 0, 0),
            "pair_2sub_n256": GemmConfig(2, 256, 0, 0, 0, 2), "pair_2sub_n128": GemmConfig(2, 128, 0, 0, 0, 2),
            "pair_2sub_n224": GemmConfig(2, 224, 0, 0, 0, 2), "pair_2sub_n192": GemmConfig(2, 192, 0, 0, 0, 2),
            "pair_2sub_n160": GemmConfig(2, 160, 0, 0, 0, 2),
            # widths ending in half a store box (the last box overlaps its neighbour)
            "pair_2sub_n240": GemmConfig(2, 240, 0, 0, 0, 2), "pair_2sub_n208": GemmConfig(2, 208, 0, 0, 0, 2),
            "pair_2sub_n176": GemmConfig(2, 176, 0, 0, 0, 2),
            # narrow tiles for problems with few tiles
            "pair_n64": GemmConfig(2, 64, 0, 0, 0), "1cta_n64": GemmConfig(1, 64, 0, 0, 0),
            # (1cta_n128 / 1cta_n64 take the kernels with two k-blocks per stage when K is whole
            # k-blocks; these name the one-k-block kernels by their stage counts)
            "1cta_n128_6stages": GemmConfig(1, 128, 6, 0, 0), "1cta_n64_8stages": GemmConfig(1, 64, 8, 0, 0)}


# ------------------------------------------------------------ reference shape
@pytest.mark.parametrize("K", [32, 128, 4096])
def test_reference_shape_f16_f32(ctx, oracle_mod, golden, K):
    """The three hardware cases of the reference (crates/patina/tests/hw_run.rs:192-197;
    K=4096 added), same closed-form inputs, checked with the reference's rule against
    golden outputs of the reference's own CPU GEMM."""
    A, B = oracle_mod.fill_legacy_f16(K)
    dA = torch.from_numpy(A.view(np.int16)).view(torch.float16).cuda()
    dB = torch.from_numpy(B.view(np.int16)).view(torch.float16).cuda()
    out = ctx.gemm_f16_tn_f32out(dA, dB)
    ctx.status()
    bad, max_abs, max_rel, _ = oracle_mod.compare_legacy(out.cpu().numpy(), golden[f"C_ref_k{K}"])
    assert bad == 0, f"K={K}: {bad} mismatches, max abs {max_abs:.3e}, max rel {max_rel:.3e}"


def test_run_gemm_mirror(oracle_mod, golden):
    """The run.rs-shaped entry (float32 in, rounded to f16 on the host, C on the host)."""
    import patina_b200
    A, B = oracle_mod.fill_legacy_f16(128)
    c = patina_b200.run_gemm(128, oracle_mod.f16_bits_to_f32(A), oracle_mod.f16_bits_to_f32(B))
    assert c.shape == (128, 128) and c.dtype == torch.float32 and not c.is_cuda
    assert oracle_mod.compare_legacy(c.numpy(), golden["C_ref_k128"])[0] == 0
    with pytest.raises(patina_b200.PatinaGemmError):
        patina_b200.run_gemm(48, np.zeros((128, 48), np.float32), np.zeros((128, 48), np.float32))


@pytest.mark.parametrize("M,N,K", [(100, 130, 96), (300, 261, 200), (128, 127, 64)])
def test_f16_f32out_ragged_shapes(ctx, oracle_mod, M, N, K):
    """The reference's types (f16 in, f32 out) on shapes its kernel cannot run: ragged M, N, K, the
    reference's own pass rule against its CPU GEMM restated, every kernel of that type pair; N is
    not a multiple of 4 columns, so the last store box of a row is written from the registers,
    and not one column behind N may change."""
    from patina_b200 import GemmConfig
    g = torch.Generator().manual_seed(M + N)
    A = (torch.rand((M, K), generator=g) - 0.5).to(torch.float16)
    B = (torch.rand((N, K), generator=g) - 0.5).to(torch.float16)
    w = lambda t: oracle_mod.f16_bits_to_f32(t.view(torch.int16).numpy().view(np.uint16))
    ref = oracle_mod.ref_gemm_tn(w(A), w(B))
    ldc = (N + 3) // 4 * 4 + 4
    for name, cfg in {"auto": None, "1cta_n128": GemmConfig(1, 128, 0, 0, 0), "1cta_n256": GemmConfig(1, 256, 0, 0, 0),
                      "pair_n256": GemmConfig(2, 256, 0, 0, 0)}.items():
        full = torch.full((M, ldc), float("nan"), dtype=torch.float32, device="cuda")
        ctx.gemm_tn(A.cuda(), B.cuda(), out=full[:, :N], config=cfg)
        ctx.status()
        bad, max_abs, max_rel, _ = oracle_mod.compare_legacy(full[:, :N].cpu().numpy(), ref)
        assert bad == 0, f"{name}: {bad} mismatches, max abs {max_abs:.3e}, max rel {max_rel:.3e}"
        assert bool(torch.isnan(full[:, N:]).all()), f"{name}: columns behind N were written"


# ------------------------------------------------------------------ bf16 cases
def test_bf16_1024_cubed_all_configs(ctx, oracle_mod):
    """The 1024^3 check case: U(-1,1) operands, full compare, every tile configuration."""
    from patina_b200 import inputs
    A, B = inputs.make_operands("uniform", 1024, 1024, 1024)
    want = expect_bf16(oracle_mod, A, B)
    dA, dB = A.cuda(), B.cuda()
    outs = {}
    for name, cfg in cfgs().items():
        out = ctx.gemm_tn(dA, dB, config=cfg)
        ctx.status()
        check_norm(oracle_mod, out, want, name)
        outs[name] = out
    via_named_entry = ctx.gemm_bf16_tn(dA, dB)
    ctx.status()
    assert torch.equal(via_named_entry, outs["auto"])
    # configurations agree with each other far inside the tolerance
    for name, out in outs.items():
        check_norm(oracle_mod, out, outs["auto"].float().cpu().numpy(), f"{name} vs auto")


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (200, 136, 192), (1024, 1024, 1088), (520, 1000, 4096),
                                   (2048, 264, 960)])
def test_two_k_blocks_per_stage_kernels(ctx, oracle_mod, M, N, K):
    """The single-CTA kernels whose stages hold two k-blocks fetched as one 3-D box per operand
    (128 x 128 tiles with 3 stages, 128 x 64 with 4), the even k-blocks multiplied into one
    accumulator and the odd ones into a second by two issuing threads, the two added in the
    epilogue: odd and even counts of k-blocks (an odd count leaves the last stage half zero-filled;
    a single k-block leaves the second accumulator unused), ragged M and N. Against the oracle,
    and against the one-accumulator kernel of the same tile (another summation order: within
    the tolerance, and equal bit for bit when K is a single k-block)."""
    from patina_b200 import inputs, GemmConfig, lib as L
    assert K % 64 == 0
    A, B = inputs.make_operands("llm", M, N, K, seed=M + N + K)
    want = expect_bf16(oracle_mod, A, B, alpha=0.75)
    dA, dB = A.cuda(), B.cuda()
    for block_n, two, one in ((128, 3, 6), (64, 4, 8)):
        plan = L.plan(L.IN_BF16, L.OUT_BF16, M, N, K, GemmConfig(1, block_n, two, 0, 0))
        assert plan.stages == two and plan.stage_bytes == 2 * (128 + block_n) * 128
        assert plan.block == 224 and plan.tmem_cols == 4 * block_n
        assert L.plan(L.IN_BF16, L.OUT_BF16, M, N, K, GemmConfig(1, block_n, 0, 0, 0)).stages == two
        ldc = (N + 7) // 8 * 8 + 8
        full = torch.full((M, ldc), float("nan"), dtype=torch.bfloat16, device="cuda")
        for _ in range(2):   # twice: the second accumulator is reused
            ctx.gemm_tn(dA, dB, out=full[:, :N], alpha=0.75, config=GemmConfig(1, block_n, two, 0, 0))
            ctx.status()
            check_norm(oracle_mod, full[:, :N], want, f"128 x {block_n}, two k-blocks per stage, {M}x{N}x{K}")
            assert bool(torch.isnan(full[:, N:]).all())
        ref = ctx.gemm_tn(dA, dB, alpha=0.75, config=GemmConfig(1, block_n, one, 0, 0))
        ctx.status()
        check_norm(oracle_mod, full[:, :N], ref.float().cpu().numpy(), "two accumulators vs one")
        if K == 64:
            assert torch.equal(full[:, :N], ref)


@pytest.mark.parametrize("M,N,K", [(1536, 512, 320), (1400, 520, 136), (4096, 1024, 1024)])
def test_half_tile_tail_wave(ctx, oracle_mod, M, N, K):
    """Tiles of a last wave that fills at most half of the clusters are run as two half tiles
    (one accumulator sub-tile each, on different clusters). Every accumulator sees the same MMAs
    in the same order, so the result equals the unsplit launch bit for bit -- also with rows past
    M in the split tile and with the fused epilogue."""
    from patina_b200 import inputs, GemmConfig, lib as L
    A, B = inputs.make_operands("llm", M, N, K, seed=M + K)
    want = expect_bf16(oracle_mod, A, B, alpha=0.5)
    dA, dB = A.cuda(), B.cuda()
    split_cfg = GemmConfig(2, 256, 0, 0, 8 if M < 4096 else 0, 2)
    whole_cfg = GemmConfig(2, 256, 0, 0, 2, 2)       # one cluster: no tail wave
    assert L.plan(L.IN_BF16, L.OUT_BF16, M, N, K, split_cfg).half_tiles > 0
    assert L.plan(L.IN_BF16, L.OUT_BF16, M, N, K, whole_cfg).half_tiles == 0
    ldc = (N + 7) // 8 * 8 + 8
    full = torch.full((M, ldc), float("nan"), dtype=torch.bfloat16, device="cuda")
    ctx.gemm_tn(dA, dB, out=full[:, :N], alpha=0.5, config=split_cfg)
    ctx.status()
    check_norm(oracle_mod, full[:, :N], want, f"half-tile tail {M}x{N}x{K}")
    assert bool(torch.isnan(full[:, N:]).all())
    whole = ctx.gemm_tn(dA, dB, alpha=0.5, config=whole_cfg)
    ctx.status()
    assert torch.equal(full[:, :N], whole)


def test_half_tile_tail_wave_fused_epilogue(ctx, oracle_mod):
    """8192 x 4096 has 34 tiles in its last wave: the fused epilogue over half tiles (bias,
    residual and activation applied by the sub-tile's own epilogue warps only) against the plain
    kernel's result put through the same arithmetic in fp32."""
    from patina_b200 import inputs, lib as L
    M, N, K = 8192, 4096, 2048
    assert L.plan(L.IN_BF16, L.OUT_BF16, M, N, K).half_tiles == 34
    A, B = inputs.make_operands("llm", M, N, K, seed=9)
    dA, dB = A.cuda(), B.cuda()
    g = torch.Generator().manual_seed(3)
    bias = torch.randn(N, generator=g).cuda()
    resid = torch.randn((M, N), generator=g).to(torch.bfloat16).cuda()
    fused = ctx.gemm_bf16_tn_fused(dA, dB, alpha=0.5, bias=bias, residual=resid, beta=0.25, activation="relu")
    ctx.status()
    plain = ctx.gemm_tn(dA, dB, out_dtype=None)          # bf16 of the fp32 accumulators (alpha = 1)
    ctx.status()
    # the fused kernel rounds once, from fp32; redo it from the bf16 result: 1 bf16 ulp of slack
    ref = torch.relu(plain.float() * 0.5 + bias[None, :] + 0.25 * resid.float())
    err = (fused.float() - ref).abs().max().item()
    assert err <= 2.0 ** -7 * max(1.0, ref.abs().max().item()), err
    # and the plain kernel itself, split, equals the oracle on sampled rows
    rows = np.array([0, 255, 256, 511, 512, 4095, 7936, 8191])
    want = oracle_mod.scale_round_bf16(oracle_mod.ref_gemm_tn(
        oracle_mod.bf16_bits_to_f32(A.view(torch.int16).numpy().view(np.uint16)),
        oracle_mod.bf16_bits_to_f32(B.view(torch.int16).numpy().view(np.uint16)), rows=rows), 1.0)
    check_norm(oracle_mod, plain[torch.from_numpy(rows).cuda()], want, "split tail rows")


def test_two_k_blocks_per_stage_needs_whole_k_blocks(ctx):
    """K = 72 is not whole 64-element k-blocks: the 3-D operand view does not exist, the library's
    own choice falls back to the one-k-block kernel and an explicit request is refused."""
    from patina_b200 import GemmConfig, PatinaGemmError, lib as L
    assert L.plan(L.IN_BF16, L.OUT_BF16, 256, 256, 72, GemmConfig(1, 128, 0, 0, 0)).stages == 6
    A = torch.zeros((256, 72), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(PatinaGemmError):
        ctx.gemm_tn(A, A, config=GemmConfig(1, 128, 3, 0, 0))
    ctx.gemm_tn(A, A, config=GemmConfig(1, 128, 0, 0, 0))
    ctx.status()


@pytest.mark.parametrize("M,N,K", [(1, 8, 8), (16, 24, 40), (128, 128, 64), (129, 257, 72), (1000, 776, 520),
                                   (300, 1032, 2048), (2048, 264, 136)])
def test_bf16_ragged_shapes(ctx, oracle_mod, M, N, K):
    from patina_b200 import inputs
    A, B = inputs.make_operands("llm", M, N, K, seed=M * 7 + N)
    want = expect_bf16(oracle_mod, A, B, alpha=0.75)
    for name, cfg in cfgs().items():
        ldc = (N + 7) // 8 * 8 + 8  # row pitch must be a multiple of 16 bytes
        full = torch.full((M, ldc), float("nan"), dtype=torch.bfloat16, device="cuda")
        out = full[:, :N]
        ctx.gemm_tn(A.cuda(), B.cuda(), out=out, alpha=0.75, config=cfg)
        ctx.status()
        check_norm(oracle_mod, out, want, f"{name} {M}x{N}x{K}")
        # not one column behind N may be written, also when N is not a multiple of 8 columns
        # (TMA stores clip in units of 16 bytes; the kernel writes such boxes itself)
        assert bool(torch.isnan(full[:, N:]).all()), f"{name} {M}x{N}x{K}: columns behind N were written"


def test_leading_dimensions_and_untouched_padding(ctx, oracle_mod):
    """lda/ldb/ldc larger than the extents; K not a multiple of the K block; columns of C
    beyond N and rows beyond M must keep their contents."""
    from patina_b200 import inputs
    M, N, K, lda, ldb, ldc = 200, 136, 100, 104, 128, 160
    A, B = inputs.make_operands("uniform", M, N, K, seed=11)
    Ap = torch.zeros((M, lda), dtype=torch.bfloat16); Ap[:, :K] = A; Ap[:, K:] = 7.0
    Bp = torch.zeros((N, ldb), dtype=torch.bfloat16); Bp[:, :K] = B; Bp[:, K:] = -3.0
    Cp = torch.full((M + 8, ldc), 5.0, dtype=torch.bfloat16, device="cuda")
    want = expect_bf16(oracle_mod, A, B)
    for name, cfg in cfgs().items():
        Cp.fill_(5.0)
        ctx.gemm_tn(Ap.cuda()[:, :K], Bp.cuda()[:, :K], out=Cp[:M, :N], config=cfg)
        ctx.status()
        check_norm(oracle_mod, Cp[:M, :N], want, name)
        assert bool((Cp[:M, N:] == 5.0).all()) and bool((Cp[M:, :] == 5.0).all()), name


def test_empty_problems(ctx):
    A = torch.zeros((0, 64), dtype=torch.bfloat16, device="cuda")
    B = torch.ones((32, 64), dtype=torch.bfloat16, device="cuda")
    assert ctx.gemm_tn(A, B).shape == (0, 32)
    assert ctx.gemm_tn(B, A).shape == (32, 0)
    # K == 0: C = 0
    out = torch.full((32, 16), 3.0, dtype=torch.bfloat16, device="cuda")
    ctx.gemm_tn(torch.zeros((32, 0), dtype=torch.bfloat16, device="cuda"),
                torch.zeros((16, 0), dtype=torch.bfloat16, device="cuda"), out=out)
    ctx.status()
    assert bool((out == 0).all())


def test_invalid_arguments_are_diagnosed(ctx):
    import patina_b200
    from patina_b200 import lib as L
    A = torch.zeros((64, 64), dtype=torch.bfloat16, device="cuda")
    odd = torch.zeros((64, 60), dtype=torch.bfloat16, device="cuda")  # 120-byte row pitch
    with pytest.raises(patina_b200.PatinaGemmError, match="multiple of 16 bytes"):
        ctx.gemm_tn(odd, odd)
    with pytest.raises(patina_b200.PatinaGemmError, match="CUDA tensors"):
        ctx.gemm_tn(A.cpu(), A.cpu())
    with pytest.raises(patina_b200.PatinaGemmError, match="unsupported input dtypes"):
        ctx.gemm_tn(A.float(), A.float())
    lib = L.load()
    h = ctx._h
    rc = lib.patina_gemm_bf16_tn(h, None, 64, A.data_ptr(), 64, A.data_ptr(), 64, 64, 64, 64, 1.0, None)
    assert rc == L.ERR_INVALID_ARG
    assert "A is null" in L.take_string(lib.patina_gemm_last_error(h))
    rc = lib.patina_gemm_bf16_tn(h, A.data_ptr() + 2, 64, A.data_ptr(), 64, A.data_ptr(), 64, 8, 8, 8, 1.0, None)
    assert rc == L.ERR_INVALID_ARG
    rc = lib.patina_gemm_ex(h, L.IN_BF16, L.OUT_BF16, A.data_ptr(), 64, A.data_ptr(), 64, A.data_ptr(), 64,
                            64, 64, 64, 1.0, C.byref(L.GemmConfig(3, 256, 0, 0, 0)), None)
    assert rc == L.ERR_INVALID_ARG
    assert lib.patina_gemm_bf16_tn(None, A.data_ptr(), 64, A.data_ptr(), 64, A.data_ptr(), 64, 8, 8, 8, 1.0, None) == L.ERR_INVALID_ARG
    ctx.status()  # nothing was launched; the context is still usable


# ------------------------------------------------------------------- fp8 cases
@pytest.mark.parametrize("M,N,K", [(1024, 1024, 1024), (200, 392, 336)])
def test_fp8_e4m3(ctx, oracle_mod, M, N, K):
    from patina_b200 import inputs
    Aq, sa, Bq, sb = inputs.make_fp8_operands(M, N, K)
    want = expect_bf16(oracle_mod, Aq, Bq, alpha=sa * sb)  # dequantised: sa*sb * sum(qa*qb)
    out = ctx.gemm_fp8e4m3_tn(Aq.cuda(), Bq.cuda(), sa, sb)
    ctx.status()
    check_norm(oracle_mod, out, want, "fp8 auto")
    for name, cfg in cfgs().items():
        if name in ("pair_n128", "pair_2sub_n128", "pair_2sub_n192", "pair_2sub_n160", "pair_2sub_n208",
                    "pair_2sub_n176", "pair_n64", "1cta_n64", "1cta_n64_8stages"):
            continue  # no such fp8 kernels
        out = ctx.gemm_tn(Aq.cuda(), Bq.cuda(), alpha=sa * sb, config=cfg)
        ctx.status()
        check_norm(oracle_mod, out, want, f"fp8 {name}")


# ------------------------------------------------------------ skinny (stream-K) path
@pytest.mark.parametrize("M,N,K", [(16, 512, 256), (1, 136, 64), (64, 1000, 2120), (100, 3584, 1024),
                                   (128, 2048, 8192), (33, 28672, 512)])
def test_streamk_matches_oracle_and_large_tile_kernel(ctx, oracle_mod, M, N, K):
    """Skinny problems through the stream-K kernel (forced), against the oracle and against
    the large-tile kernel; run twice to check that the arrival counters are left clean."""
    from patina_b200 import inputs, GemmConfig
    A, B = inputs.make_operands("llm", M, N, K, seed=N + K)
    want = expect_bf16(oracle_mod, A, B, alpha=1.5)
    ldc = (N + 7) // 8 * 8
    dA, dB = A.cuda(), B.cuda()
    outs = []
    for _ in range(2):
        out = torch.full((M, ldc), float("nan"), dtype=torch.bfloat16, device="cuda")[:, :N]
        ctx.gemm_tn(dA, dB, out=out, alpha=1.5, config=GemmConfig(0, 0, 0, 0, 0, 0, 1))
        ctx.status()
        check_norm(oracle_mod, out, want, f"stream-K {M}x{N}x{K}")
        outs.append(out.clone())
    assert torch.equal(outs[0], outs[1])  # deterministic: fixed reduction order
    tiled = torch.empty((M, ldc), dtype=torch.bfloat16, device="cuda")[:, :N]
    ctx.gemm_tn(dA, dB, out=tiled, alpha=1.5, config=GemmConfig(0, 0, 0, 0, 0, 0, -1))
    ctx.status()
    check_norm(oracle_mod, tiled, outs[0].float().cpu().numpy(), "large-tile vs stream-K")


def test_streamk_whole_tiles_only_orders_the_stream(ctx, oracle_mod):
    """A partition in which every CTA owns whole tiles (100 tiles x 8 k-blocks over 100 CTAs) with
    a wide X, which would normally hand the sum to the follow-up kernel: nothing is shared, so no
    second kernel may be launched, and work enqueued right behind the call on the same stream
    must see the finished C."""
    from patina_b200 import inputs, GemmConfig
    M, N, K = 32, 12800, 512
    A, B = inputs.make_operands("llm", M, N, K, seed=31)
    dA, dB = A.cuda(), B.cuda()
    want = expect_bf16(oracle_mod, A, B)
    for mode in (1, 2):
        out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
        before = ctx.launch_count
        ctx.gemm_tn(dA, dB, out=out, config=GemmConfig(0, 0, 0, 0, 0, 0, mode))
        seen = out.clone()                       # a consumer on the same stream, no sync in between
        assert ctx.launch_count - before == 1, "no tile is shared: the reduce kernel must not run"
        ctx.status()
        check_norm(oracle_mod, seen, want, f"consumer right behind the call (stream_k={mode})")


def test_streamk_wait_expiry_is_reported_and_context_recovers(ctx, oracle_mod):
    """The skinny kernel's bounded waits: with a 1 ns limit on a problem whose CTAs stream for
    tens of microseconds each and share tiles, the launch is abandoned and status() says so;
    status() also clears the arrival counters the abandoned launch left half-way, so the next
    launches on the same context are right again (in-kernel sum and follow-up kernel)."""
    import patina_b200
    from patina_b200 import inputs, GemmConfig, lib as L
    M, N, K = 16, 12800, 16384                 # 100 tiles x 256 k-blocks over 148 CTAs: shared tiles
    A, B = inputs.make_operands("llm", M, N, K, seed=32)
    dA, dB = A.cuda(), B.cuda()
    ctx.set_wait_limit_ns(1)
    try:
        ctx.gemm_tn(dA, dB, config=GemmConfig(0, 0, 0, 0, 0, 0, 3))
        with pytest.raises(patina_b200.PatinaGemmError) as ei:
            ctx.status()
        assert ei.value.code == L.ERR_TIMEOUT and "wait expired" in str(ei.value)
    finally:
        ctx.set_wait_limit_ns(2_000_000_000)
    rng = np.random.default_rng(3)
    cols = np.unique(np.concatenate([[0, 127, 128, N - 1], rng.integers(0, N, 60)])).astype(np.int64)
    ref_t = oracle_mod.ref_gemm_tn(widen(oracle_mod, B), widen(oracle_mod, A), rows=cols)
    want = oracle_mod.scale_round_bf16(ref_t.T.copy(), 1.0)
    for mode in (3, 2):
        out = ctx.gemm_tn(dA, dB, config=GemmConfig(0, 0, 0, 0, 0, 0, mode))
        ctx.status()
        check_norm(oracle_mod, out[:, torch.from_numpy(cols).cuda()], want, f"after recovery (stream_k={mode})")


def test_streamk_decode_shapes_full_size(ctx, oracle_mod):
    """The decode-shaped configurations at full size (N=28672, K=8192, M in {16, 64, 128}):
    one launch each, or two where the stream-K kernel hands the sum over contributors to its
    follow-up kernel; 128 sampled columns of C against the
    oracle (computed as rows of B x A^T), and fp8 inputs on the same path."""
    from patina_b200 import inputs
    N, K = 28672, 8192
    rng = np.random.default_rng(9)
    cols = np.unique(np.concatenate([[0, 127, 128, N - 1], rng.integers(0, N, 124)])).astype(np.int64)
    for M in (16, 64, 128):
        A, B = inputs.make_operands("llm", M, N, K, seed=M)
        before = ctx.launch_count
        out = ctx.gemm_tn(A.cuda(), B.cuda())
        ctx.status()
        assert 1 <= ctx.launch_count - before <= 2
        ref_t = oracle_mod.ref_gemm_tn(widen(oracle_mod, B), widen(oracle_mod, A), rows=cols)  # [cols, M]
        want = oracle_mod.scale_round_bf16(ref_t.T.copy(), 1.0)
        check_norm(oracle_mod, out[:, torch.from_numpy(cols).cuda()], want, f"decode M={M}")
    Aq, sa, Bq, sb = inputs.make_fp8_operands(32, 4096, 4096)
    out = ctx.gemm_fp8e4m3_tn(Aq.cuda(), Bq.cuda(), sa, sb)
    ctx.status()
    check_norm(oracle_mod, out, expect_bf16(oracle_mod, Aq, Bq, alpha=sa * sb), "fp8 stream-K")


@pytest.mark.parametrize("activation", ["none", "relu", "gelu", "silu"])
def test_fused_epilogue(ctx, oracle_mod, activation):
    """bias + residual + activation applied to the fp32 accumulator inside the kernel, against the
    oracle's double-precision epilogue; ragged shape; also each term alone, and the empty
    epilogue, which must reproduce the plain entry point bit for bit."""
    from patina_b200 import inputs
    M, N, K = 1000, 776, 520
    A, B = inputs.make_operands("llm", M, N, K, seed=9)
    g = torch.Generator().manual_seed(4)
    bias = torch.randn(N, generator=g, dtype=torch.float32)
    res = (torch.randn((M, N), generator=g) * 0.5).to(torch.bfloat16)
    ref = oracle_mod.ref_gemm_tn(widen(oracle_mod, A), widen(oracle_mod, B))
    dA, dB = A.cuda(), B.cuda()
    ldc = (N + 7) // 8 * 8
    cases = [dict(bias=bias, residual=res, beta=0.75), dict(bias=bias), dict(residual=res, beta=-1.0)]
    for kw in cases:
        out = torch.full((M, ldc), float("nan"), dtype=torch.bfloat16, device="cuda")[:, :N]
        dev_kw = {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in kw.items()}
        ctx.gemm_bf16_tn_fused(dA, dB, out=out, alpha=1.25, activation=activation, **dev_kw)
        ctx.status()
        want = oracle_mod.fused_epilogue_bf16(
            ref, 1.25, bias=kw.get("bias").numpy() if "bias" in kw else None,
            residual=widen(oracle_mod, kw["residual"]) if "residual" in kw else None,
            beta=kw.get("beta", 1.0), activation=activation)
        check_norm(oracle_mod, out, want, f"fused {activation} {sorted(kw)}")
    if activation == "none":
        plain = ctx.gemm_tn(dA, dB, alpha=1.25)
        empty = ctx.gemm_bf16_tn_fused(dA, dB, alpha=1.25)
        ctx.status()
        assert torch.equal(plain, empty)
        # residual read from the output buffer itself (C += A B^T)
        acc = res.cuda().clone()
        ctx.gemm_bf16_tn_fused(dA, dB, out=acc, residual=acc, beta=1.0)
        ctx.status()
        check_norm(oracle_mod, acc, oracle_mod.fused_epilogue_bf16(ref, 1.0, residual=widen(oracle_mod, res)),
                   "in-place accumulate")


def test_stream_k_reduce_modes_agree(ctx, oracle_mod):
    """The sum over the CTAs that share a tile can run inside the stream-K kernel (the last CTA
    to reach a tile adds the others' parts) or in the follow-up kernel; both add in the same
    contributor order, so they must agree bit for bit, for skinny and for wide X."""
    from patina_b200 import inputs, GemmConfig
    for M, N, K in [(16, 1024, 4096), (40, 904, 2120), (128, 1536, 8192)]:
        A, B = inputs.make_operands("llm", M, N, K, seed=M + N)
        dA, dB = A.cuda(), B.cuda()
        follow_up = ctx.gemm_tn(dA, dB, config=GemmConfig(0, 0, 0, 0, 0, 0, 2))
        in_kernel = ctx.gemm_tn(dA, dB, config=GemmConfig(0, 0, 0, 0, 0, 0, 3))
        ctx.status()
        assert torch.equal(follow_up, in_kernel), (M, N, K)
        check_norm(oracle_mod, follow_up, expect_bf16(oracle_mod, A, B), f"stream-K {M}x{N}x{K}")


def test_calls_can_be_captured_in_a_cuda_graph(ctx, oracle_mod):
    """The calls only enqueue work, so after one eager call each (first calls set function
    attributes and grow scratch memory) they can be captured into a CUDA graph; replaying the
    graph on new operand values must give what eager calls give. Covers the large-tile kernel,
    the stream-K kernel alone and the stream-K kernel with its dependent reduce kernel."""
    from patina_b200 import inputs
    shapes = [(512, 520, 264), (16, 1024, 8192), (96, 1024, 8192)]   # the last two take stream-K
    ops, outs = [], []
    for i, (M, N, K) in enumerate(shapes):
        A, B = inputs.make_operands("llm", M, N, K, seed=50 + i)
        ops.append((A.cuda(), B.cuda()))
        outs.append(torch.empty((M, (N + 7) // 8 * 8), dtype=torch.bfloat16, device="cuda")[:, :N])
    for (dA, dB), out in zip(ops, outs):
        ctx.gemm_tn(dA, dB, out=out)           # eager first call
    ctx.status()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            for (dA, dB), out in zip(ops, outs):
                ctx.gemm_tn(dA, dB, out=out)
        for round_ in range(2):
            for i, (dA, dB) in enumerate(ops):  # new values in the captured buffers
                A2, B2 = inputs.make_operands("llm", *shapes[i], seed=70 + 10 * round_ + i)
                dA.copy_(A2.cuda()); dB.copy_(B2.cuda())
            for out in outs:
                out.fill_(float("nan"))
            graph.replay()
            side.synchronize()
            replayed = [o.clone() for o in outs]
            for (dA, dB), out, got in zip(ops, outs, replayed):
                eager = ctx.gemm_tn(dA, dB)
                ctx.status()
                assert torch.equal(got, eager)
    torch.cuda.current_stream().wait_stream(side)
    A2, B2 = inputs.make_operands("llm", *shapes[2], seed=70 + 10 + 2)
    check_norm(oracle_mod, replayed[2], expect_bf16(oracle_mod, A2, B2), "graph replay vs oracle")


@pytest.mark.parametrize("activation", ["none", "gelu"])
def test_fused_epilogue_fp8_output(ctx, oracle_mod, activation):
    """e4m3 result of the fused epilogue: C = sat_e4m3(rne(out_scale * y)), y as in the bf16 case,
    plus the running amax. Rule (written out because one e4m3 step is 6-12 % of a value, far
    above the bf16 tolerance): every code equals the oracle's (double-precision y, one rounding),
    or is the neighbouring code where the exact out_scale * y lies within 5 % of a step of the
    midpoint between the two (fp32 vs double accumulation may fall either side); at most 1 % of
    the codes may differ; saturated values are +-448, never NaN; amax within 1e-4 relative."""
    from patina_b200 import inputs
    M, N, K = 520, 392, 264
    A, B = inputs.make_operands("llm", M, N, K, seed=21)
    g = torch.Generator().manual_seed(6)
    bias = torch.randn(N, generator=g, dtype=torch.float32) * 0.1
    res = (torch.randn((M, N), generator=g) * 0.2).to(torch.bfloat16)
    ref = oracle_mod.ref_gemm_tn(widen(oracle_mod, A), widen(oracle_mod, B))
    table = oracle_mod.e4m3_bits_to_f32(np.arange(256, dtype=np.uint8)).astype(np.float64)
    dA, dB = A.cuda(), B.cuda()
    ldc = (N + 31) // 16 * 16
    for kw, scale_for in [(dict(bias=bias, residual=res, beta=0.5), 200.0), (dict(), 2000.0)]:
        _, amax_ref, y = oracle_mod.fused_epilogue_e4m3(
            ref, 1.0, alpha=1.5, bias=kw.get("bias").numpy() if "bias" in kw else None,
            residual=widen(oracle_mod, kw["residual"]) if "residual" in kw else None,
            beta=kw.get("beta", 1.0), activation=activation)
        out_scale = scale_for / amax_ref          # 200: inside the range; 2000: part of it saturates
        codes_ref = oracle_mod.f32_to_e4m3_bits((y * out_scale).astype(np.float32))
        full = torch.full((M, ldc), 0x55, dtype=torch.uint8, device="cuda")
        amax = torch.zeros(1, dtype=torch.float32, device="cuda")
        dev_kw = {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in kw.items()}
        ctx.gemm_bf16_tn_fused_fp8out(dA, dB, out_scale, out=full[:, :N], amax=amax, alpha=1.5,
                                      activation=activation, **dev_kw)
        ctx.status()
        got = full[:, :N].cpu().numpy()
        assert bool((full[:, N:] == 0x55).all()), "padding columns were written"
        assert not np.any((got & 0x7F) == 0x7F), "NaN code in the output"
        diff = got != codes_ref
        assert diff.mean() <= 0.01, f"{diff.mean():.4f} of the codes differ"
        a, b, x = table[got[diff]], table[codes_ref[diff]], (y * out_scale)[diff]
        step = np.abs(a - b)
        order = np.sort(np.unique(table[np.isfinite(table)]))
        adjacent = np.abs(np.searchsorted(order, a) - np.searchsorted(order, b)) == 1
        assert bool(adjacent.all()), "a differing code is not the oracle's neighbour"
        assert bool((np.abs(np.clip(x, -448, 448) - (a + b) / 2) <= 0.05 * step + 1e-6).all()), \
            "a differing code is not explained by a value on a rounding boundary"
        if scale_for > 448:
            assert np.any(np.abs(table[got]) == 448.0), "expected saturated values"
        assert abs(float(amax.item()) - amax_ref) <= 1e-4 * amax_ref
        # a second call with a smaller result must leave the running maximum where it is
        ctx.gemm_bf16_tn_fused_fp8out(dA, dB, out_scale, out=full[:, :N], amax=amax, alpha=0.5,
                                      activation=activation, **dev_kw)
        ctx.status()
        if not kw:
            assert abs(float(amax.item()) - amax_ref) <= 1e-4 * amax_ref


def test_scatter_to_several_destinations_on_one_gpu(ctx, oracle_mod):
    """patina_gemm_bf16_tn_scatter with three destinations that all live on this GPU: each must
    receive exactly what the single-destination call produces (on a multi-GPU node the extra
    destinations are peer buffers; the kernel path is the same)."""
    import patina_b200
    from patina_b200 import inputs, lib as L
    M, N, K, ldc = 1000, 520, 328, 2048
    A, B = inputs.make_operands("llm", M, N, K, seed=77)
    dA, dB = A.cuda(), B.cuda()
    single = ctx.gemm_tn(dA, dB)
    wide = [torch.full((M, ldc), 9.0, dtype=torch.bfloat16, device="cuda") for _ in range(3)]
    offs = [0, 256, 1024]                      # a different column offset in every destination
    ptrs = [w.data_ptr() + 2 * o for w, o in zip(wide, offs)]
    ctx.gemm_bf16_tn_scatter(dA, dB, ptrs, ldc)
    ctx.status()
    for w, o in zip(wide, offs):
        assert torch.equal(w[:, o:o + N], single)
        assert bool((w[:, :o] == 9.0).all()) and bool((w[:, o + N:] == 9.0).all())
    check_norm(oracle_mod, single, expect_bf16(oracle_mod, A, B), "scatter reference")
    # a width that is not a multiple of 8 columns: the last box of every row is written from the
    # registers, once per destination, and must not touch the neighbouring columns either
    N2 = 523
    A2, B2 = inputs.make_operands("llm", M, N2, K, seed=78)
    dA2, dB2 = A2.cuda(), B2.cuda()
    single2 = ctx.gemm_tn(dA2, dB2, out=torch.empty((M, 528), dtype=torch.bfloat16, device="cuda")[:, :N2])
    for w in wide:
        w.fill_(9.0)
    ctx.gemm_bf16_tn_scatter(dA2, dB2, ptrs, ldc)
    ctx.status()
    for w, o in zip(wide, offs):
        assert torch.equal(w[:, o:o + N2], single2)
        assert bool((w[:, :o] == 9.0).all()) and bool((w[:, o + N2:] == 9.0).all())
    with pytest.raises(patina_b200.PatinaGemmError, match="n_dests"):
        ctx.gemm_bf16_tn_scatter(dA, dB, ptrs * 3, ldc)            # nine destinations
    with pytest.raises(patina_b200.PatinaGemmError):
        ctx.gemm_bf16_tn_scatter(dA, dB, [ptrs[0], ptrs[1] + 2], ldc)   # misaligned destination


@pytest.mark.parametrize("M,N,K", [(1024, 1024, 1024), (256, 4096, 4096), (1000, 776, 2056), (129, 264, 520),
                                   (512, 512, 512)])
def test_cluster_split_k(ctx, oracle_mod, M, N, K):
    """K cut across a thread-block cluster (2 and 4 CTAs per 128 x 256 tile), partial tiles
    summed through distributed shared memory in rank order: every cluster size against the
    oracle, ragged M / N / K, padding columns untouched, two runs bit-identical, and the
    library's own choice for the shape."""
    from patina_b200 import inputs, GemmConfig, lib as L
    A, B = inputs.make_operands("llm", M, N, K, seed=M + K)
    want = expect_bf16(oracle_mod, A, B, alpha=0.5)
    dA, dB = A.cuda(), B.cuda()
    ldc = N + 8
    for split in (2, 4):
        if (K + 63) // 64 < split:
            continue
        outs = []
        for _ in range(2):
            full = torch.full((M, ldc), float("nan"), dtype=torch.bfloat16, device="cuda")
            before = ctx.launch_count
            ctx.gemm_tn(dA, dB, out=full[:, :N], alpha=0.5, config=GemmConfig(0, 0, 0, 0, 0, 0, 0, split))
            ctx.status()
            assert ctx.launch_count - before == 1
            check_norm(oracle_mod, full[:, :N], want, f"cluster_k={split} {M}x{N}x{K}")
            assert bool(torch.isnan(full[:, N:]).all()), f"cluster_k={split}: columns behind N were written"
            outs.append(full[:, :N].clone())
        assert torch.equal(outs[0], outs[1])
    auto = ctx.gemm_tn(dA, dB, alpha=0.5)
    never = ctx.gemm_tn(dA, dB, alpha=0.5, config=GemmConfig(0, 0, 0, 0, 0, 0, 0, -1))
    ctx.status()
    check_norm(oracle_mod, auto, want, "library's choice")
    check_norm(oracle_mod, never, auto.float().cpu().numpy(), "large-tile kernel vs library's choice")


def test_cluster_split_k_refusals(ctx):
    import patina_b200
    from patina_b200 import GemmConfig
    A = torch.zeros((256, 128), dtype=torch.bfloat16, device="cuda")
    B = torch.zeros((260, 128), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(patina_b200.PatinaGemmError, match="cluster_k"):
        ctx.gemm_tn(A, B[:256], config=GemmConfig(0, 0, 0, 0, 0, 0, 0, 4))       # 2 k-blocks < 4 CTAs
    with pytest.raises(patina_b200.PatinaGemmError, match="cluster_k"):
        ctx.gemm_tn(A, B, out=torch.empty((256, 264), dtype=torch.bfloat16, device="cuda")[:, :260],
                    config=GemmConfig(0, 0, 0, 0, 0, 0, 0, 2))                   # N = 260 is not a multiple of 8
    with pytest.raises(patina_b200.PatinaGemmError, match="cluster_k"):
        ctx.gemm_tn(A, B[:256], config=GemmConfig(0, 0, 0, 0, 0, 0, 0, 3))
    with pytest.raises(patina_b200.PatinaGemmError, match="cluster_k"):
        ctx.gemm_tn(A, B[:256], config=GemmConfig(0, 0, 0, 0, 0, 0, 0, 8))
    ctx.status()


@pytest.mark.parametrize("K", [520, 512])
def test_sharded_entry_point_on_one_gpu(oracle_mod, K):
    """patina_gemm_sharded_bf16_tn with several shards that all live on this GPU (one context and
    one stream per shard, as on a multi-GPU node one per GPU): each shard writes its column block
    of one full-width C through the leading dimension, and the result equals the unsharded call
    that sums in the same ascending k order (`k_order = 1`, which the sharded entry point asks
    for itself) bit for bit, for shard counts that split the width evenly and unevenly. K = 512
    is whole k-blocks: without that setting the unsharded call and the narrower shards would take
    the two-accumulator kernels, whose sums round differently."""
    import ctypes as C
    import patina_b200
    from patina_b200 import inputs, sharded, lib as L
    lib = L.load()
    M, N = 1000, 1800
    A, B = inputs.make_operands("llm", M, N, K, seed=12)
    dA, dB = A.cuda(), B.cuda()
    ctxs = [patina_b200.GemmContext(0) for _ in range(4)]
    single = ctxs[0].gemm_tn(dA, dB, config=sharded.ASCENDING_K)
    ctxs[0].status()
    for world in (1, 2, 3, 4):
        full = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
        streams = [torch.cuda.Stream() for _ in range(world)]
        for st in streams:
            st.wait_stream(torch.cuda.current_stream())
        spans = [sharded.column_shard(N, world, r) for r in range(world)]
        vp = C.c_void_p
        arr = lambda vals: (vp * world)(*vals)
        rc = lib.patina_gemm_sharded_bf16_tn(
            arr([c._h.value for c in ctxs[:world]]), world, arr([dA.data_ptr()] * world), dA.stride(0),
            arr([dB.data_ptr() + 2 * K * n0 for n0, _ in spans]), dB.stride(0),
            arr([full.data_ptr() + 2 * n0 for n0, _ in spans]), full.stride(0), M, N, K, 1.0,
            arr([st.cuda_stream for st in streams]))
        assert rc == L.OK
        for c, st in zip(ctxs, streams):
            with torch.cuda.stream(st):
                c.status()
        assert torch.equal(full, single), f"{world} shards"
    check_norm(oracle_mod, single, expect_bf16(oracle_mod, A, B), "sharded reference")
    for c in ctxs:
        c.close()


# ------------------------------------------------------- full benchmark sizes
def test_bf16_8192_cubed_samples_and_properties(ctx, oracle_mod):
    """8192^3 (the benchmark size): 64 sampled rows against the oracle, plus
    size-independent properties: column shards reproduce the full result bit for
    bit (what N-sharding over GPUs relies on), scaling alpha by 2 doubles every
    output exactly, and the two tile configurations agree."""
    from patina_b200 import inputs, GemmConfig
    n = 8192
    A, B = inputs.make_operands("normal_0p1", n, n, n)
    dA, dB = A.cuda(), B.cuda()
    out = ctx.gemm_tn(dA, dB)
    ctx.status()
    rng = np.random.default_rng(5)
    rows = np.unique(np.concatenate([[0, 127, 128, 255, 256, n - 1], rng.integers(0, n, 58)])).astype(np.int64)
    want = expect_bf16(oracle_mod, A, B, rows=rows)
    check_norm(oracle_mod, out[torch.from_numpy(rows).cuda()], want, "sampled rows")
    # column shards == full result
    for g in (2, 8):
        w = n // g
        for r in (0, g - 1):
            shard = ctx.gemm_tn(dA, dB[r * w:(r + 1) * w])
            assert torch.equal(shard, out[:, r * w:(r + 1) * w]), f"shard {r}/{g}"
    doubled = ctx.gemm_tn(dA, dB, alpha=2.0)
    assert torch.equal(doubled.float(), out.float() * 2.0)
    other = ctx.gemm_tn(dA, dB, config=GemmConfig(1, 256, 0, 0, 0))
    ctx.status()
    check_norm(oracle_mod, other, out.float().cpu().numpy(), "1-CTA vs pair")


def test_host_entry_point(ctx, oracle_mod):
    """patina_gemm_host: pinned host buffers in, pinned host buffer out."""
    from patina_b200 import inputs
    A, B = inputs.make_operands("uniform", 512, 384, 256, pin=True)
    Cn = torch.empty((512, 384), dtype=torch.bfloat16).pin_memory()
    ctx.gemm_host(A, B, Cn)
    ctx.status()
    check_norm(oracle_mod, Cn, expect_bf16(oracle_mod, A, B), "host entry")


def test_host_entry_point_pipelined_blocks(ctx, oracle_mod):
    """A problem large enough for patina_gemm_host to cut into row blocks whose copies and
    GEMMs overlap; ragged M, padded host pitches; two calls in a row on the same buffers."""
    from patina_b200 import inputs
    M, N, K = 4100, 2048, 2056
    A, B = inputs.make_operands("llm", M, N, K, seed=5)
    Ap = torch.zeros((M, K + 8), dtype=torch.bfloat16).pin_memory(); Ap[:, :K] = A
    Bp = torch.zeros((N, K + 24), dtype=torch.bfloat16).pin_memory(); Bp[:, :K] = B
    Cp = torch.full((M, N + 16), 3.0, dtype=torch.bfloat16).pin_memory()
    want_dev = ctx.gemm_tn(A.cuda(), B.cuda())
    ctx.status()
    for _ in range(2):
        Cp.fill_(3.0)
        ctx.gemm_host(Ap[:, :K], Bp[:, :K], Cp[:, :N])
        ctx.status()
        assert torch.equal(Cp[:, :N], want_dev.cpu())
        assert bool((Cp[:, N:] == 3.0).all())
    rows = np.arange(0, M, 41, dtype=np.int64)
    check_norm(oracle_mod, Cp[:, :N][torch.from_numpy(rows)], expect_bf16(oracle_mod, A, B, rows=rows), "pipelined host entry")


def test_wait_expiry_is_reported_and_context_survives(ctx, oracle_mod):
    """A wait that runs out must come back as PATINA_GEMM_ERR_TIMEOUT, not a hang.
    The limit is set to 1 ns on a single-tile problem with a long K loop, so the
    epilogue's wait for its accumulator expires while the mainloop is still
    healthy; afterwards the same context must compute correctly again."""
    import patina_b200
    from patina_b200 import inputs, lib as L
    A, B = inputs.make_operands("uniform", 128, 128, 131072, seed=3)
    dA, dB = A.cuda(), B.cuda()
    ctx.set_wait_limit_ns(1)
    try:
        ctx.gemm_tn(dA, dB)
        with pytest.raises(patina_b200.PatinaGemmError) as ei:
            ctx.status()
        assert ei.value.code == L.ERR_TIMEOUT and "wait expired" in str(ei.value)
    finally:
        ctx.set_wait_limit_ns(2_000_000_000)
    out = ctx.gemm_tn(dA, dB)
    ctx.status()
    check_norm(oracle_mod, out, expect_bf16(oracle_mod, A, B), "after recovery")

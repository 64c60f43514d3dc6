"""The CPU oracle against (1) golden vectors produced by the reference's own
functions, (2) the compiled reference itself when it is present, (3) independent
arithmetic (numpy / torch). No GPU."""
import hashlib

import numpy as np
import pytest
import torch


def _nan_equal_bits(a_bits, b_bits):
    a = a_bits.view(np.float32)
    b = b_bits.view(np.float32)
    both_nan = np.isnan(a) & np.isnan(b)
    return np.all(both_nan | (a_bits == b_bits))


def test_f16_to_f32_matches_reference_table(oracle_mod, golden):
    bits = np.arange(65536, dtype=np.uint16)
    mine = oracle_mod.f16_bits_to_f32(bits).view(np.uint32)
    assert _nan_equal_bits(mine, golden["f16_to_f32_bits"])


def test_f32_to_f16_matches_reference_samples(oracle_mod, golden):
    assert np.array_equal(oracle_mod.f32_to_f16_bits(golden["f32_inputs"]), golden["f32_to_f16"])


def test_f16_roundtrip_all_patterns(oracle_mod):
    bits = np.arange(65536, dtype=np.uint16)
    wide = oracle_mod.f16_bits_to_f32(bits)
    back = oracle_mod.f32_to_f16_bits(wide)
    finite = ~np.isnan(wide)
    assert np.array_equal(back[finite], bits[finite])
    assert np.array_equal(wide[finite], bits.view(np.float16).astype(np.float32)[finite])


def test_bf16_converters_all_patterns_and_vs_torch(oracle_mod):
    bits = np.arange(65536, dtype=np.uint16)
    wide = oracle_mod.bf16_bits_to_f32(bits)
    assert np.array_equal(wide.view(np.uint32), bits.astype(np.uint32) << 16)
    finite = ~np.isnan(wide)
    assert np.array_equal(oracle_mod.f32_to_bf16_bits(wide)[finite], bits[finite])
    rng = np.random.default_rng(1)
    x = (rng.standard_normal(1 << 16) * 10.0 ** rng.integers(-20, 20, 1 << 16)).astype(np.float32)
    # exact ties: halfway between neighbouring bf16 values
    ties = ((rng.integers(0, 1 << 15, 4096).astype(np.uint32) << 16) | 0x8000).view(np.float32)
    x = np.concatenate([x, ties])
    x = x[~np.isnan(x)]  # NaN payloads are implementation-defined
    want = torch.from_numpy(x).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(oracle_mod.f32_to_bf16_bits(x), want)


def test_e4m3_converters_all_patterns_and_vs_torch(oracle_mod):
    bits = np.arange(256, dtype=np.uint8)
    wide = oracle_mod.e4m3_bits_to_f32(bits)
    want = torch.from_numpy(bits).view(torch.float8_e4m3fn).float().numpy()
    nan = np.isnan(want)
    assert np.array_equal(np.isnan(wide), nan)
    assert np.array_equal(wide[~nan], want[~nan])
    assert np.array_equal(oracle_mod.f32_to_e4m3_bits(wide)[~nan], bits[~nan])
    rng = np.random.default_rng(2)
    x = (rng.standard_normal(1 << 16) * 10.0 ** rng.integers(-5, 3, 1 << 16)).astype(np.float32)
    x = x[np.abs(x) <= 448.0]  # torch overflows to NaN above the range; this converter saturates
    got = oracle_mod.f32_to_e4m3_bits(x)
    want = torch.from_numpy(x).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    assert np.array_equal(got, want)
    assert oracle_mod.f32_to_e4m3_bits(np.array([1e6, -1e6, 464.0, 463.9], np.float32)).tolist() == [0x7E, 0xFE, 0x7E, 0x7E]


@pytest.mark.parametrize("K", [32, 128, 4096])
def test_legacy_inputs_and_gemm_match_golden(oracle_mod, golden, K):
    A, B = oracle_mod.fill_legacy_f16(K)
    assert hashlib.sha256(A.tobytes()).digest() == golden[f"A_sha_k{K}"].tobytes()
    assert hashlib.sha256(B.tobytes()).digest() == golden[f"B_sha_k{K}"].tobytes()
    if K <= 128:
        assert np.array_equal(A, golden[f"A_k{K}"]) and np.array_equal(B, golden[f"B_k{K}"])
    C = oracle_mod.ref_gemm_tn(oracle_mod.f16_bits_to_f32(A), oracle_mod.f16_bits_to_f32(B))
    assert np.array_equal(C, golden[f"C_ref_k{K}"])  # bit-exact doubles
    for threads in (1, 3):
        C2 = oracle_mod.ref_gemm_tn(oracle_mod.f16_bits_to_f32(A), oracle_mod.f16_bits_to_f32(B), threads=threads)
        assert np.array_equal(C2, C)


def test_against_compiled_reference_when_present(oracle_mod):
    if not oracle_mod.have_ref():
        pytest.skip("oracle/_ref not built on this machine")
    R = oracle_mod.ref()
    assert (R.patina_ref_rows(), R.patina_ref_cols()) == (128, 128)
    for K in (32, 64, 96, 1024):
        A = np.empty((128, K), np.uint16)
        B = np.empty((128, K), np.uint16)
        R.patina_ref_fill_inputs(A.ctypes.data, B.ctypes.data, K)
        Cr = np.empty((128, 128), np.float64)
        R.patina_ref_reference_gemm(A.ctypes.data, B.ctypes.data, K, Cr.ctypes.data)
        A2, B2 = oracle_mod.fill_legacy_f16(K)
        assert np.array_equal(A, A2) and np.array_equal(B, B2)
        assert np.array_equal(oracle_mod.ref_gemm_tn(oracle_mod.f16_bits_to_f32(A), oracle_mod.f16_bits_to_f32(B)), Cr)


def test_general_shapes_vs_numpy(oracle_mod):
    rng = np.random.default_rng(3)
    for (M, N, K) in [(1, 1, 1), (5, 9, 17), (64, 33, 100), (130, 257, 72)]:
        A = rng.standard_normal((M, K)).astype(np.float32)
        B = rng.standard_normal((N, K)).astype(np.float32)
        C = oracle_mod.ref_gemm_tn(A, B)
        want = A.astype(np.float64) @ B.astype(np.float64).T
        assert np.allclose(C, want, rtol=1e-12, atol=1e-12)
        # strided operands (leading dimension > K)
        Ap = np.zeros((M, K + 8), np.float32); Ap[:, :K] = A
        Bp = np.zeros((N, K + 24), np.float32); Bp[:, :K] = B
        assert np.array_equal(oracle_mod.ref_gemm_tn(Ap[:, :K], Bp[:, :K]), C)
    rows = np.array([3, 0, 129], np.int64)
    A = rng.standard_normal((130, 40)).astype(np.float32)
    B = rng.standard_normal((20, 40)).astype(np.float32)
    assert np.array_equal(oracle_mod.ref_gemm_tn(A, B, rows=rows), oracle_mod.ref_gemm_tn(A, B)[rows])
    assert oracle_mod.ref_gemm_tn(np.zeros((0, 8), np.float32), B[:, :8].copy()).shape == (0, 20)


def test_compare_rules(oracle_mod):
    ref = np.array([0.0, 10.0, -2000.0, 0.5], np.float64)
    got = ref.astype(np.float32).copy()
    assert oracle_mod.compare_legacy(got, ref)[0] == 0
    got[0] += 2e-3          # abs > atol and rel (vs max(1,|ref|)) > rtol -> mismatch
    got[2] += 1.0           # abs > atol but rel = 5e-4 <= rtol -> not a mismatch
    bad, max_abs, max_rel, s = oracle_mod.compare_legacy(got, ref)
    assert bad == 1 and abs(max_abs - 1.0) < 1e-3 and abs(max_rel - 2e-3) < 1e-5
    got[3] = np.nan
    assert oracle_mod.compare_legacy(got, ref)[0] == 2
    r = np.linspace(-4, 4, 1000).astype(np.float32)
    ok, me, mx, fr = oracle_mod.compare_norm(r, r)
    assert ok and me == 0 and fr == 0 and mx == 4.0
    g = r.copy(); g[10] += 0.05  # > 1e-2 * max|ref|
    assert not oracle_mod.compare_norm(g, r)[0]
    g = r * np.float32(1.002)    # elementwise fine, Frobenius 2e-3 > 1e-3
    assert not oracle_mod.compare_norm(g, r)[0]
    g = r.copy(); g[0] = np.nan
    assert not oracle_mod.compare_norm(g, r)[0]


def test_bf16_output_rounding(oracle_mod):
    ref = np.array([1.00390625, 3.0, -2.5e-3], np.float64)  # first one is a bf16 tie -> even
    out = oracle_mod.scale_round_bf16(ref, alpha=1.0)
    assert out[0] == 1.0 and out[1] == 3.0
    assert oracle_mod.scale_round_bf16(ref, alpha=0.5)[1] == 1.5


def test_fused_epilogue_reference(oracle_mod):
    """The oracle's double-precision epilogue against torch float64, every activation."""
    rng = np.random.default_rng(8)
    ref = rng.standard_normal((9, 14)) * 3
    bias = rng.standard_normal(14).astype(np.float32)
    res = rng.standard_normal((9, 14)).astype(np.float32)
    t = torch.from_numpy(0.5 * ref) + torch.from_numpy(bias.astype(np.float64))[None, :] + 2.0 * torch.from_numpy(res.astype(np.float64))
    want = {"none": t, "relu": torch.relu(t), "gelu": torch.nn.functional.gelu(t), "silu": torch.nn.functional.silu(t)}
    for act, w in want.items():
        got = oracle_mod.fused_epilogue_bf16(ref, 0.5, bias=bias, residual=res, beta=2.0, activation=act)
        exp = w.to(torch.float32).to(torch.bfloat16).float().numpy()
        # double -> bf16 directly vs double -> float -> bf16 may differ by one bf16 ulp at a tie
        assert np.max(np.abs(got - exp)) <= np.max(np.abs(exp)) * 2 ** -7
        assert np.mean(got != exp) < 0.02
    with pytest.raises(ValueError):
        oracle_mod.fused_epilogue_bf16(ref, activation="tanh")


def test_fp8_output_epilogue_restatement(oracle_mod):
    """oracle.fused_epilogue_e4m3 (the expected output of the fp8-output entry point): its codes
    are the round-to-nearest-even, saturating e4m3 of out_scale * y, checked against torch's own
    float8_e4m3fn conversion where that is defined (|x| <= 448), and against +-448 beyond."""
    import torch
    rng = np.random.default_rng(12)
    ref = rng.normal(size=(37, 53)) * 3.0
    bias = rng.normal(size=53).astype(np.float32)
    codes, amax, y = oracle_mod.fused_epilogue_e4m3(ref, 40.0, alpha=1.5, bias=bias, activation="relu")
    want_y = np.maximum(1.5 * ref + bias.astype(np.float64)[None, :], 0.0)
    assert np.allclose(y, want_y, rtol=0, atol=0)
    assert amax == float(np.abs(want_y).max())
    x = (want_y * 40.0).astype(np.float32)
    inside = np.abs(x) <= 448.0
    t = torch.from_numpy(x).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    assert np.array_equal(codes[inside], t[inside])
    assert inside.sum() < x.size, "the case should also exercise saturation"
    assert np.all(codes[~inside & (x > 0)] == 0x7E) and np.all(codes[~inside & (x < 0)] == 0xFE)

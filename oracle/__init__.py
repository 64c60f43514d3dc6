"""CPU oracle for the Patina GEMM path -- TEST INFRASTRUCTURE ONLY.

numpy-facing wrappers over ``oracle/_build/libpatina_oracle.so`` (the CPU
restatement of the reference's check, ``patina_oracle.c``) and, when present,
``oracle/_ref/libpatina_ref.so`` (the reference's own functions compiled from
the reference sources by ``oracle/Makefile``).

Nothing in the shipped package imports this module. Only the test-suite, the
smoke check and the benchmark's CPU-baseline legs do, and only as the checker
or as the timed CPU baseline.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(_HERE, "_build", "libpatina_oracle.so")
REF_SO = os.path.join(_HERE, "_ref", "libpatina_ref.so")


def build(reference_root: str | None = None) -> None:
    """Compile the restatement; also the reference wrapper when its sources exist."""
    subprocess.check_call(["make", "-s", "-C", _HERE, "oracle"])
    root = (reference_root or os.environ.get("PATINA_REFERENCE_ROOT")
            or os.path.abspath(os.path.join(_HERE, "..", "..", "reference")))
    if os.path.isfile(os.path.join(root, "harness", "gemm_check.cpp")):
        subprocess.check_call(["make", "-s", "-C", _HERE, "ref", f"REF={root}"])


_lib = None
_ref = None


def _p(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.isfile(ORACLE_SO):
            build()
        L = C.CDLL(ORACLE_SO)
        L.po_f16_to_f32.restype = C.c_float
        L.po_f16_to_f32.argtypes = [C.c_uint16]
        L.po_f32_to_f16.restype = C.c_uint16
        L.po_f32_to_f16.argtypes = [C.c_float]
        for name in ("po_f16_to_f32_n", "po_f32_to_f16_n", "po_bf16_to_f32_n",
                     "po_f32_to_bf16_n", "po_e4m3_to_f32_n", "po_f32_to_e4m3_n"):
            getattr(L, name).restype = None
            getattr(L, name).argtypes = [C.c_void_p, C.c_void_p, C.c_size_t]
        L.po_fill_legacy_f16.restype = None
        L.po_fill_legacy_f16.argtypes = [C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint64]
        L.po_ref_gemm_tn.restype = C.c_int
        L.po_ref_gemm_tn.argtypes = [C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_void_p,
                                     C.c_int64, C.c_int64, C.c_int64, C.c_int64, C.c_int]
        L.po_ref_gemm_tn_rows.restype = C.c_int
        L.po_ref_gemm_tn_rows.argtypes = [C.c_void_p, C.c_int64, C.c_void_p, C.c_int64,
                                          C.c_void_p, C.c_int64, C.c_void_p, C.c_int64,
                                          C.c_int64, C.c_int64, C.c_int]
        L.po_scale_round_bf16.restype = None
        L.po_scale_round_bf16.argtypes = [C.c_void_p, C.c_double, C.c_void_p, C.c_size_t]
        L.po_compare_legacy.restype = C.c_uint64
        L.po_compare_legacy.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_double,
                                        C.c_double, C.POINTER(C.c_double),
                                        C.POINTER(C.c_double), C.POINTER(C.c_double)]
        L.po_compare_norm.restype = C.c_int
        L.po_compare_norm.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_double,
                                      C.c_double, C.POINTER(C.c_double),
                                      C.POINTER(C.c_double), C.POINTER(C.c_double)]
        L.po_host_threads.restype = C.c_int
        _lib = L
    return _lib


def have_ref() -> bool:
    return os.path.isfile(REF_SO)


def ref() -> C.CDLL:
    """The reference's own CPU functions (see ref_wrap.cpp)."""
    global _ref
    if _ref is None:
        R = C.CDLL(REF_SO)
        R.patina_ref_rows.restype = C.c_uint32
        R.patina_ref_cols.restype = C.c_uint32
        R.patina_ref_f16_to_f32.restype = C.c_float
        R.patina_ref_f16_to_f32.argtypes = [C.c_uint16]
        R.patina_ref_f32_to_f16.restype = C.c_uint16
        R.patina_ref_f32_to_f16.argtypes = [C.c_float]
        R.patina_ref_fill_inputs.restype = None
        R.patina_ref_fill_inputs.argtypes = [C.c_void_p, C.c_void_p, C.c_uint64]
        R.patina_ref_reference_gemm.restype = None
        R.patina_ref_reference_gemm.argtypes = [C.c_void_p, C.c_void_p, C.c_uint64, C.c_void_p]
        _ref = R
    return _ref


# ---------------------------------------------------------------- converters
def _conv(name, src, src_dt, dst_dt):
    src = np.ascontiguousarray(src, dtype=src_dt)
    dst = np.empty(src.shape, dtype=dst_dt)
    getattr(lib(), name)(_p(src), _p(dst), src.size)
    return dst


def f16_bits_to_f32(a): return _conv("po_f16_to_f32_n", a, np.uint16, np.float32)
def f32_to_f16_bits(a): return _conv("po_f32_to_f16_n", a, np.float32, np.uint16)
def bf16_bits_to_f32(a): return _conv("po_bf16_to_f32_n", a, np.uint16, np.float32)
def f32_to_bf16_bits(a): return _conv("po_f32_to_bf16_n", a, np.float32, np.uint16)
def e4m3_bits_to_f32(a): return _conv("po_e4m3_to_f32_n", a, np.uint8, np.float32)
def f32_to_e4m3_bits(a): return _conv("po_f32_to_e4m3_n", a, np.float32, np.uint8)


def fill_legacy_f16(K: int, rows: int = 128):
    """The reference's closed-form inputs as f16 bit patterns: (A, B), each [rows, K]."""
    A = np.empty((rows, K), np.uint16)
    B = np.empty((rows, K), np.uint16)
    lib().po_fill_legacy_f16(_p(A), _p(B), rows, K)
    return A, B


# ---------------------------------------------------------------------- GEMM
def ref_gemm_tn(A: np.ndarray, B: np.ndarray, rows=None, threads: int = 0) -> np.ndarray:
    """C = A @ B.T in the reference's arithmetic (double accumulate, k ascending).

    A [M, K] and B [N, K] are float32 arrays holding exactly-widened storage
    values; rows (optional int64 indices) restricts the output to those rows.
    """
    assert A.dtype == np.float32 and B.dtype == np.float32
    assert A.shape[1] == B.shape[1]
    if A.size == 0 or B.size == 0:
        n_out = A.shape[0] if rows is None else len(rows)
        return np.zeros((n_out, B.shape[0]), np.float64)
    assert A.strides[1] == 4 and B.strides[1] == 4
    lda, ldb = A.strides[0] // 4, B.strides[0] // 4
    N, K = B.shape
    if rows is None:
        out = np.empty((A.shape[0], N), np.float64)
        lib().po_ref_gemm_tn(_p(A), lda, _p(B), ldb, _p(out), N, A.shape[0], N, K, threads)
    else:
        rows = np.ascontiguousarray(rows, dtype=np.int64)
        out = np.empty((rows.size, N), np.float64)
        lib().po_ref_gemm_tn_rows(_p(A), lda, _p(B), ldb, _p(out), N, _p(rows), rows.size,
                                  N, K, threads)
    return out


def mx_dequant(q_bits: np.ndarray, e: np.ndarray) -> np.ndarray:
    """Block-scaled fp8 operand as exact float32 values: e4m3 element times 2^(e - 127), one E8M0
    byte e per 32 consecutive K elements of a row (OCP Microscaling formats v1.0, MXFP8). The
    reference has no block-scaled path; this extends its check: the dequantised operands go
    through the same double-accumulating loop (harness/gemm_check.cpp:165-178)."""
    q = e4m3_bits_to_f32(q_bits)
    rows, K = q.shape
    assert K % 32 == 0 and e.shape == (rows, K // 32) and e.dtype == np.uint8
    assert not np.any(e == 0xFF), "0xFF is the E8M0 NaN"
    scale = np.ldexp(np.float32(1.0), e.astype(np.int32) - 127).astype(np.float32)
    out = (q.reshape(rows, K // 32, 32) * scale[:, :, None]).reshape(rows, K)
    assert np.all(np.isfinite(out))
    return np.ascontiguousarray(out, dtype=np.float32)


def scale_round_bf16(ref: np.ndarray, alpha: float = 1.0) -> np.ndarray:
    """bf16(alpha * ref) (RNE), widened back to float32: the expected bf16 output."""
    ref = np.ascontiguousarray(ref, dtype=np.float64)
    out = np.empty(ref.shape, np.float32)
    lib().po_scale_round_bf16(_p(ref), float(alpha), _p(out), ref.size)
    return out


def fused_epilogue_f64(ref: np.ndarray, alpha=1.0, bias=None, residual=None, beta=1.0,
                       activation="none") -> np.ndarray:
    """act(alpha * ref + bias[n] + beta * residual[m, n]) in double, before any rounding.
    (The reference's kernel has no epilogue arithmetic; this extends its double-precision check.)"""
    import math
    x = alpha * np.asarray(ref, dtype=np.float64)
    if bias is not None:
        x = x + np.asarray(bias, dtype=np.float64)[None, :]
    if residual is not None:
        x = x + beta * np.asarray(residual, dtype=np.float64)
    if activation == "relu":
        x = np.maximum(x, 0.0)
    elif activation == "gelu":
        erf = np.vectorize(math.erf)
        x = 0.5 * x * (1.0 + erf(x / math.sqrt(2.0)))
    elif activation == "silu":
        x = x / (1.0 + np.exp(-x))
    elif activation != "none":
        raise ValueError(activation)
    return x


def fused_epilogue_bf16(ref: np.ndarray, alpha=1.0, bias=None, residual=None, beta=1.0,
                        activation="none") -> np.ndarray:
    """bf16 of the double-precision epilogue, widened to float32: the expected output of the
    fused-epilogue entry point (one rounding at the very end)."""
    return scale_round_bf16(fused_epilogue_f64(ref, alpha, bias, residual, beta, activation), 1.0)


def fused_epilogue_e4m3(ref: np.ndarray, out_scale: float, alpha=1.0, bias=None, residual=None,
                        beta=1.0, activation="none"):
    """The fp8-output epilogue: (e4m3 codes of out_scale * y rounded to nearest even and
    saturated, max|y|, y) with y the double-precision epilogue."""
    y = fused_epilogue_f64(ref, alpha, bias, residual, beta, activation)
    codes = f32_to_e4m3_bits((y * out_scale).astype(np.float32))
    return codes, float(np.abs(y).max()) if y.size else 0.0, y


# --------------------------------------------------------------- comparisons
def compare_legacy(got: np.ndarray, ref: np.ndarray, atol=1e-3, rtol=1e-3):
    """The reference harness's rule. Returns (mismatches, max_abs, max_rel, sum_got)."""
    got = np.ascontiguousarray(got, dtype=np.float32)
    ref = np.ascontiguousarray(ref, dtype=np.float64)
    assert got.size == ref.size
    ma, mr, sm = C.c_double(), C.c_double(), C.c_double()
    bad = lib().po_compare_legacy(_p(got), _p(ref), got.size, atol, rtol,
                                  C.byref(ma), C.byref(mr), C.byref(sm))
    return int(bad), ma.value, mr.value, sm.value


def compare_norm(got: np.ndarray, ref: np.ndarray, elem_tol=1e-2, fro_tol=1e-3):
    """|d| <= elem_tol*max|ref| elementwise and ||d||_F/||ref||_F <= fro_tol.

    Returns (ok, max_abs_err, max_abs_ref, fro_rel).
    """
    got = np.ascontiguousarray(got, dtype=np.float32)
    ref = np.ascontiguousarray(ref, dtype=np.float32)
    assert got.size == ref.size
    me, mx, fr = C.c_double(), C.c_double(), C.c_double()
    ok = lib().po_compare_norm(_p(got), _p(ref), got.size, elem_tol, fro_tol,
                               C.byref(me), C.byref(mx), C.byref(fr))
    return bool(ok), me.value, mx.value, fr.value


def host_threads() -> int:
    return int(lib().po_host_threads())

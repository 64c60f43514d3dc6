"""Host-side launch API over the C ABI, on torch CUDA tensors.

Mirrors the reference's Rust runner (crates/patina/src/run.rs): `compute_capability`
(run.rs:418-445), `run_gemm` (run.rs:462-529) for the reference kernel's own
128x128xK f16->f32 shape, and a `CudaError`-style exception carrying the
library's diagnostic. PyTorch is used only for device memory and streams; all
arithmetic runs in the library's tcgen05 kernels.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import lib as _l
from .lib import GemmConfig


class PatinaGemmError(RuntimeError):
    """Counterpart of run.rs `CudaError` (run.rs:106-115)."""

    def __init__(self, code: int, message: str):
        super().__init__(f"[patina_gemm error {code}] {message}")
        self.code = code


_IN = {torch.float16: _l.IN_F16, torch.bfloat16: _l.IN_BF16}
if hasattr(torch, "float8_e4m3fn"):
    _IN[torch.float8_e4m3fn] = _l.IN_E4M3
_OUT = {torch.bfloat16: _l.OUT_BF16, torch.float32: _l.OUT_F32}


def compute_capability(device: int = 0) -> tuple[int, int]:
    """(major, minor) of the device; raises if there is no CUDA device (run.rs:418-445)."""
    if not torch.cuda.is_available():
        raise PatinaGemmError(_l.ERR_UNSUPPORTED_ARCH, "no CUDA device is visible")
    return torch.cuda.get_device_capability(device)


def _stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


class GemmContext:
    """Owns one `PatinaGemmContext` (one per device; not thread-safe)."""

    def __init__(self, device: int | None = None):
        self._lib = _l.load()
        self._h = C.c_void_p()
        if device is None:
            device = torch.cuda.current_device() if torch.cuda.is_available() else 0
        self.device = int(device)
        rc = self._lib.patina_gemm_context_create(self.device, C.byref(self._h))
        if rc != _l.OK:
            why = {_l.ERR_UNSUPPORTED_ARCH: "device is not sm_100 (tcgen05 needs Blackwell); "
                                            "there is no fallback path",
                   _l.ERR_INVALID_ARG: "no such device"}.get(rc, "CUDA error")
            raise PatinaGemmError(rc, f"patina_gemm_context_create({self.device}): {why}")

    def close(self) -> None:
        if self._h:
            self._lib.patina_gemm_context_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    # ----------------------------------------------------------------- helpers
    def _raise(self, rc: int):
        msg = _l.take_string(self._lib.patina_gemm_last_error(self._h)) or "no diagnostic"
        raise PatinaGemmError(rc, msg)

    def set_wait_limit_ns(self, ns: int) -> None:
        rc = self._lib.patina_gemm_set_wait_limit_ns(self._h, int(ns))
        if rc != _l.OK:
            self._raise(rc)

    def status(self) -> None:
        """Synchronise the current stream; raise if a device-side wait expired."""
        rc = self._lib.patina_gemm_status(self._h, _stream_ptr(self.device))
        if rc != _l.OK:
            self._raise(rc)

    @property
    def launch_count(self) -> int:
        return int(self._lib.patina_gemm_launch_count(self._h))

    # -------------------------------------------------------------------- GEMM
    def gemm_tn(self, A: torch.Tensor, B: torch.Tensor, out: torch.Tensor | None = None,
                alpha: float = 1.0, out_dtype: torch.dtype | None = None,
                config: GemmConfig | None = None) -> torch.Tensor:
        """out[M,N] = alpha * A[M,K] @ B[N,K]^T. A, B: K-contiguous CUDA tensors of the
        same dtype (f16, bf16 or float8_e4m3fn); row strides are the leading dimensions."""
        if A.dtype != B.dtype or A.dtype not in _IN:
            raise PatinaGemmError(_l.ERR_INVALID_ARG, f"unsupported input dtypes {A.dtype}/{B.dtype}")
        if A.dim() != 2 or B.dim() != 2 or A.shape[1] != B.shape[1]:
            raise PatinaGemmError(_l.ERR_INVALID_ARG, "A must be [M,K] and B [N,K]")
        if not (A.is_cuda and B.is_cuda):
            raise PatinaGemmError(_l.ERR_INVALID_ARG, "A and B must be CUDA tensors (no CPU path)")
        M, K = A.shape
        N = B.shape[0]
        if out is None:
            if out_dtype is None:
                out_dtype = torch.float32 if A.dtype == torch.float16 else torch.bfloat16
            out = torch.empty((M, N), dtype=out_dtype, device=A.device)
        if out.dtype not in _OUT or tuple(out.shape) != (M, N):
            raise PatinaGemmError(_l.ERR_INVALID_ARG, "out must be [M,N] bf16 or f32")
        for name, t in (("A", A), ("B", B), ("out", out)):
            if t.numel() and t.stride(1) != 1:
                raise PatinaGemmError(_l.ERR_INVALID_ARG, f"{name} must be contiguous along its last dim")
        lda = A.stride(0) if M > 1 else max(K, 1)
        ldb = B.stride(0) if N > 1 else max(K, 1)
        ldc = out.stride(0) if M > 1 else max(N, 1)
        rc = self._lib.patina_gemm_ex(
            self._h, _IN[A.dtype], _OUT[out.dtype], A.data_ptr(), lda, B.data_ptr(), ldb,
            out.data_ptr(), ldc, M, N, K, float(alpha),
            C.byref(config) if config is not None else None, _stream_ptr(self.device))
        if rc != _l.OK:
            self._raise(rc)
        return out

    def gemm_bf16_tn(self, A, B, out=None, alpha=1.0):
        """The `patina_gemm_bf16_tn` entry point itself (no explicit config)."""
        M, K = A.shape
        N = B.shape[0]
        if out is None:
            out = torch.empty((M, N), dtype=torch.bfloat16, device=A.device)
        rc = self._lib.patina_gemm_bf16_tn(self._h, A.data_ptr(), A.stride(0), B.data_ptr(),
                                           B.stride(0), out.data_ptr(), out.stride(0), M, N, K,
                                           float(alpha), _stream_ptr(self.device))
        if rc != _l.OK:
            self._raise(rc)
        return out

    def gemm_fp8e4m3_tn(self, Aq, Bq, scale_a: float, scale_b: float, out=None):
        """bf16 out = scale_a*scale_b * Aq @ Bq^T for float8_e4m3fn (or uint8-viewed) inputs."""
        M, K = Aq.shape
        N = Bq.shape[0]
        if out is None:
            out = torch.empty((M, N), dtype=torch.bfloat16, device=Aq.device)
        rc = self._lib.patina_gemm_fp8e4m3_tn(self._h, Aq.data_ptr(), Aq.stride(0), Bq.data_ptr(),
                                              Bq.stride(0), out.data_ptr(), out.stride(0), M, N, K,
                                              float(scale_a), float(scale_b),
                                              _stream_ptr(self.device))
        if rc != _l.OK:
            self._raise(rc)
        return out

    def gemm_mxfp8_tn(self, Aq, scales_a, Bq, scales_b, out=None, alpha: float = 1.0,
                      config: GemmConfig | None = None):
        """bf16 out = alpha * (Aq * sa) @ (Bq * sb)^T for block-scaled fp8 operands: Aq [M, K] and
        Bq [N, K] float8_e4m3fn (or uint8-viewed) CUDA tensors, scales_a / scales_b uint8 CUDA
        tensors holding one E8M0 scale per 32 K elements of a row in the library's atom layout
        (`inputs.pack_mx_scales`); K a multiple of 32."""
        M, K = Aq.shape
        N = Bq.shape[0]
        if not (Aq.is_cuda and Bq.is_cuda and scales_a.is_cuda and scales_b.is_cuda):
            raise PatinaGemmError(_l.ERR_INVALID_ARG, "operands and scales must be CUDA tensors (no CPU path)")
        need_a = int(self._lib.patina_gemm_mx_scale_bytes(M, K))
        need_b = int(self._lib.patina_gemm_mx_scale_bytes(N, K))
        if scales_a.element_size() != 1 or scales_b.element_size() != 1 or scales_a.numel() < need_a \
                or scales_b.numel() < need_b or not scales_a.is_contiguous() or not scales_b.is_contiguous():
            raise PatinaGemmError(_l.ERR_INVALID_ARG,
                                  f"scale buffers must be contiguous bytes of at least {need_a} and {need_b}")
        if out is None:
            out = torch.empty((M, N), dtype=torch.bfloat16, device=Aq.device)
        rc = self._lib.patina_gemm_mxfp8_tn(
            self._h, Aq.data_ptr(), Aq.stride(0) if M > 1 else max(K, 1), scales_a.data_ptr(), Bq.data_ptr(),
            Bq.stride(0) if N > 1 else max(K, 1), scales_b.data_ptr(), out.data_ptr(),
            out.stride(0) if M > 1 else max(N, 1), M, N, K, float(alpha),
            C.byref(config) if config is not None else None, _stream_ptr(self.device))
        if rc != _l.OK:
            self._raise(rc)
        return out

    def gemm_f16_tn_f32out(self, A, B, out=None, alpha=1.0):
        M, K = A.shape
        N = B.shape[0]
        if out is None:
            out = torch.empty((M, N), dtype=torch.float32, device=A.device)
        rc = self._lib.patina_gemm_f16_tn_f32out(self._h, A.data_ptr(), A.stride(0), B.data_ptr(),
                                                 B.stride(0), out.data_ptr(), out.stride(0), M, N,
                                                 K, float(alpha), _stream_ptr(self.device))
        if rc != _l.OK:
            self._raise(rc)
        return out

    def _epilogue(self, M, N, bias, residual, beta, activation):
        acts = {"none": _l.ACT_NONE, "relu": _l.ACT_RELU, "gelu": _l.ACT_GELU, "silu": _l.ACT_SILU}
        if activation not in acts:
            raise PatinaGemmError(_l.ERR_INVALID_ARG, f"unknown activation {activation!r}")
        if bias is not None and (bias.dtype != torch.float32 or bias.numel() != N or not bias.is_contiguous()):
            raise PatinaGemmError(_l.ERR_INVALID_ARG, "bias must be a contiguous float32 vector of N elements")
        if residual is not None and (residual.dtype != torch.bfloat16 or tuple(residual.shape) != (M, N)
                                     or residual.stride(1) != 1):
            raise PatinaGemmError(_l.ERR_INVALID_ARG, "residual must be bf16 [M, N], contiguous rows")
        return _l.GemmEpilogue(bias.data_ptr() if bias is not None else None,
                               residual.data_ptr() if residual is not None else None,
                               residual.stride(0) if residual is not None else 0, float(beta), acts[activation])

    def gemm_bf16_tn_fused(self, A, B, out=None, alpha=1.0, bias=None, residual=None, beta=1.0,
                           activation="none"):
        """out = act(alpha * A @ B^T + bias[n] + beta * residual[m, n]) in one kernel
        (bias: float32 [N]; residual: bf16 [M, N]; activation: none | relu | gelu | silu)."""
        M, K = A.shape
        N = B.shape[0]
        if out is None:
            out = torch.empty((M, N), dtype=torch.bfloat16, device=A.device)
        epi = self._epilogue(M, N, bias, residual, beta, activation)
        rc = self._lib.patina_gemm_bf16_tn_fused(self._h, A.data_ptr(), A.stride(0), B.data_ptr(),
                                                 B.stride(0), out.data_ptr(), out.stride(0), M, N, K,
                                                 float(alpha), C.byref(epi), _stream_ptr(self.device))
        if rc != _l.OK:
            self._raise(rc)
        return out

    def gemm_bf16_tn_fused_fp8out(self, A, B, out_scale: float, out=None, amax=None, alpha=1.0, bias=None,
                                  residual=None, beta=1.0, activation="none"):
        """out (float8_e4m3fn) = saturate(out_scale * act(alpha * A @ B^T + bias + beta * residual));
        `amax`, a one-element float32 CUDA tensor, is raised to the largest |act(...)| seen."""
        M, K = A.shape
        N = B.shape[0]
        if out is None:
            ldc = (N + 15) // 16 * 16
            out = torch.empty((M, ldc), dtype=torch.float8_e4m3fn, device=A.device)[:, :N]
        if out.element_size() != 1 or tuple(out.shape) != (M, N) or out.stride(1) != 1:
            raise PatinaGemmError(_l.ERR_INVALID_ARG, "out must be [M, N] float8_e4m3fn (or uint8), contiguous rows")
        if amax is not None and (amax.dtype != torch.float32 or amax.numel() != 1 or not amax.is_cuda):
            raise PatinaGemmError(_l.ERR_INVALID_ARG, "amax must be a one-element float32 CUDA tensor")
        epi = self._epilogue(M, N, bias, residual, beta, activation)
        rc = self._lib.patina_gemm_bf16_tn_fused_fp8out(
            self._h, A.data_ptr(), A.stride(0), B.data_ptr(), B.stride(0), out.data_ptr(),
            out.stride(0) if M > 1 else max((N + 15) // 16 * 16, 16), M, N, K, float(alpha), C.byref(epi),
            float(out_scale), amax.data_ptr() if amax is not None else None, _stream_ptr(self.device))
        if rc != _l.OK:
            self._raise(rc)
        return out

    def gemm_bf16_tn_scatter(self, A, B, dest_ptrs, ldc: int, alpha=1.0):
        """C = alpha * A @ B^T stored to every device address in `dest_ptrs` (row stride `ldc`
        elements for all of them; the first is normally local, the others peer buffers opened
        with peer_open)."""
        M, K = A.shape
        N = B.shape[0]
        arr = (C.c_void_p * len(dest_ptrs))(*[int(p) for p in dest_ptrs])
        rc = self._lib.patina_gemm_bf16_tn_scatter(self._h, A.data_ptr(), A.stride(0), B.data_ptr(),
                                                   B.stride(0), arr, len(dest_ptrs), int(ldc), M, N, K,
                                                   float(alpha), _stream_ptr(self.device))
        if rc != _l.OK:
            self._raise(rc)

    def _grouped(self, A, B, group_rows, out, in_dtypes):
        if not (A.is_cuda and B.is_cuda and group_rows.is_cuda):
            raise PatinaGemmError(_l.ERR_INVALID_ARG, "A, B and group_rows must be CUDA tensors (no CPU path)")
        if A.dtype not in in_dtypes or B.dtype != A.dtype or group_rows.dtype != torch.int32:
            raise PatinaGemmError(_l.ERR_INVALID_ARG, f"A and B must be {in_dtypes[0]}, group_rows int32")
        n_groups = int(group_rows.numel())
        total_rows, K = A.shape
        if B.dim() == 3:
            if not B.is_contiguous():
                raise PatinaGemmError(_l.ERR_INVALID_ARG, "a 3-D B must be contiguous")
            N = B.shape[1]
            B2 = B.view(B.shape[0] * N, B.shape[2])
        else:
            B2 = B
            N = B.shape[0] // max(n_groups, 1)
        if B2.shape[0] != n_groups * N or B2.shape[1] != K or not group_rows.is_contiguous():
            raise PatinaGemmError(_l.ERR_INVALID_ARG, "B must hold one [N, K] block per group")
        if out is None:
            out = torch.empty((total_rows, N), dtype=torch.bfloat16, device=A.device)
        lda = A.stride(0) if total_rows > 1 else max(K, 1)
        ldb = B2.stride(0) if B2.shape[0] > 1 else max(K, 1)
        ldc = out.stride(0) if total_rows > 1 else max(N, 1)
        return B2, out, (A.data_ptr(), lda, B2.data_ptr(), ldb, out.data_ptr(), ldc, group_rows.data_ptr(),
                         n_groups, total_rows, N, K)

    def gemm_bf16_tn_grouped(self, A, B, group_rows, out=None, alpha=1.0, config=None):
        """One launch for the groups of a ragged batch: out[rows of group g] = alpha *
        A[rows of group g] @ B[g]^T. A: [total_rows, K] bf16 with the groups' rows one after
        another; B: [n_groups, N, K] (or [n_groups * N, K]) bf16; group_rows: int32 CUDA tensor
        of n_groups row counts (it stays on the device: nothing here synchronises)."""
        _, out, args = self._grouped(A, B, group_rows, out, (torch.bfloat16,))
        rc = self._lib.patina_gemm_bf16_tn_grouped(
            self._h, *args, float(alpha), C.byref(config) if config is not None else None,
            _stream_ptr(self.device))
        if rc != _l.OK:
            self._raise(rc)
        return out

    def gemm_fp8e4m3_tn_grouped(self, Aq, Bq, group_rows, scale_a: float, group_scale_b=None, out=None,
                                config=None):
        """The grouped launch for float8_e4m3fn operands, bf16 result: out[group g] = scale_a *
        group_scale_b[g] * Aq[group g] @ Bq[g]^T (group_scale_b: float32 CUDA tensor or None)."""
        if group_scale_b is not None and (group_scale_b.dtype != torch.float32 or not group_scale_b.is_cuda
                                          or group_scale_b.numel() != group_rows.numel()):
            raise PatinaGemmError(_l.ERR_INVALID_ARG, "group_scale_b must be a float32 CUDA tensor, one per group")
        _, out, args = self._grouped(Aq, Bq, group_rows, out, (torch.float8_e4m3fn, torch.uint8))
        rc = self._lib.patina_gemm_fp8e4m3_tn_grouped(
            self._h, *args, float(scale_a), group_scale_b.data_ptr() if group_scale_b is not None else None,
            C.byref(config) if config is not None else None, _stream_ptr(self.device))
        if rc != _l.OK:
            self._raise(rc)
        return out

    # ------------------------------------------------------------- peer buffers
    def peer_alloc(self, nbytes: int) -> tuple[int, bytes]:
        """Device memory other processes of the node can map: (pointer, 64-byte handle)."""
        ptr = C.c_void_p()
        handle = C.create_string_buffer(64)
        rc = self._lib.patina_gemm_peer_alloc(self._h, int(nbytes), C.byref(ptr), handle)
        if rc != _l.OK:
            self._raise(rc)
        return int(ptr.value), handle.raw

    def peer_open(self, handle: bytes) -> int:
        ptr = C.c_void_p()
        rc = self._lib.patina_gemm_peer_open(self._h, handle, C.byref(ptr))
        if rc != _l.OK:
            self._raise(rc)
        return int(ptr.value)

    def peer_close(self, ptr: int) -> None:
        rc = self._lib.patina_gemm_peer_close(self._h, ptr)
        if rc != _l.OK:
            self._raise(rc)

    def peer_free(self, ptr: int) -> None:
        rc = self._lib.patina_gemm_peer_free(self._h, ptr)
        if rc != _l.OK:
            self._raise(rc)

    def gemm_host(self, hA: torch.Tensor, hB: torch.Tensor, hC: torch.Tensor, alpha: float = 1.0,
                  config: GemmConfig | None = None) -> torch.Tensor:
        """End-to-end call on HOST (ideally pinned) tensors: H2D, GEMM, D2H on the current
        stream, no synchronisation (the shape of run.rs `run_gemm`)."""
        if hA.is_cuda or hB.is_cuda or hC.is_cuda:
            raise PatinaGemmError(_l.ERR_INVALID_ARG, "gemm_host takes host tensors")
        M, K = hA.shape
        N = hB.shape[0]
        rc = self._lib.patina_gemm_host(
            self._h, _IN[hA.dtype], _OUT[hC.dtype], hA.data_ptr(), hA.stride(0), hB.data_ptr(),
            hB.stride(0), hC.data_ptr(), hC.stride(0), M, N, K, float(alpha),
            C.byref(config) if config is not None else None, _stream_ptr(self.device))
        if rc != _l.OK:
            self._raise(rc)
        return hC


class _RawCuda:
    """A raw device pointer seen through the CUDA array interface (16-bit words)."""

    def __init__(self, ptr: int, shape: tuple[int, ...]):
        self.__cuda_array_interface__ = {"shape": shape, "typestr": "<i2", "data": (ptr, False),
                                         "version": 3, "strides": None}


def wrap_bf16(ptr: int, rows: int, cols: int, device: int) -> torch.Tensor:
    """A [rows, cols] bf16 tensor over memory this library (or a peer) allocated; no copy.
    The tensor does not own the memory."""
    t = torch.as_tensor(_RawCuda(ptr, (rows, cols)), device=torch.device("cuda", device))
    return t.view(torch.bfloat16)


_default_ctx: dict[int, GemmContext] = {}


def default_context(device: int | None = None) -> GemmContext:
    if device is None:
        device = torch.cuda.current_device() if torch.cuda.is_available() else 0
    ctx = _default_ctx.get(device)
    if ctx is None:
        ctx = _default_ctx[device] = GemmContext(device)
    return ctx


def run_gemm(k: int, a, b) -> torch.Tensor:
    """The reference runner's call shape (run.rs:462-529): A[128,k], B[128,k] given as
    float32, rounded to f16 on the host, C[128,128] float32 returned on the host.
    (The reference's `ptx` and `kernel` arguments select a generated kernel; here the
    library's own f16->f32 kernel runs.)"""
    a = torch.as_tensor(a, dtype=torch.float32).reshape(128, k)
    b = torch.as_tensor(b, dtype=torch.float32).reshape(128, k)
    if k % 32 != 0:
        raise PatinaGemmError(_l.ERR_INVALID_ARG, "K must be a multiple of 32 (run.rs:476)")
    major, minor = compute_capability()
    if major < 10:
        raise PatinaGemmError(_l.ERR_UNSUPPORTED_ARCH,
                              f"device is sm_{major}{minor}; tcgen05 needs sm_100a")
    ctx = default_context()
    dA = a.to(torch.float16).cuda()
    dB = b.to(torch.float16).cuda()
    out = ctx.gemm_f16_tn_f32out(dA, dB)
    ctx.status()
    return out.cpu()

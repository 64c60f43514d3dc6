"""Seeded synthetic inputs for the GEMM workloads (host side, deterministic).

The reference measures on no dataset: its only inputs are closed-form
(harness/gemm_check.cpp:152-163). The distributions here are the ones the
benchmark configurations name; values are drawn on the host with a seeded
generator, rounded once to the storage type, and shared by the device run and
whatever checks it, so both see bit-identical operands.
"""
from __future__ import annotations

import torch

DEFAULT_SEED = 0x5EED

# workload name -> (A distribution, B distribution); ("uniform", lo, hi) or ("normal", std)
DISTRIBUTIONS = {
    "uniform": (("uniform", -1.0, 1.0), ("uniform", -1.0, 1.0)),      # 1024^3 check case
    "normal_0p1": (("normal", 0.1), ("normal", 0.1)),                 # square bf16 benchmark
    "llm": (("normal", 1.0), ("normal", 0.02)),                       # activations x weights
    "unit_normal": (("normal", 1.0), ("normal", 1.0)),                # fp8 (before quantisation)
}


def _draw(spec, shape, gen):
    if spec[0] == "uniform":
        return torch.rand(shape, generator=gen, dtype=torch.float32) * (spec[2] - spec[1]) + spec[1]
    return torch.randn(shape, generator=gen, dtype=torch.float32) * spec[1]


def make_operands(workload: str, M: int, N: int, K: int, dtype: torch.dtype = torch.bfloat16,
                  seed: int = DEFAULT_SEED, pin: bool = False):
    """Host tensors (A[M,K], B[N,K]) in `dtype` for a named distribution."""
    da, db = DISTRIBUTIONS[workload]
    ga = torch.Generator().manual_seed(seed * 2 + 1)
    gb = torch.Generator().manual_seed(seed * 2 + 2)
    A = _draw(da, (M, K), ga).to(dtype)
    B = _draw(db, (N, K), gb).to(dtype)
    if pin:
        A, B = A.pin_memory(), B.pin_memory()
    return A, B


def quantize_e4m3(x: torch.Tensor):
    """Per-tensor fp8 quantisation: scale = amax/448, q = e4m3_rne(x/scale). Returns (q, scale)."""
    amax = float(x.abs().max()) if x.numel() else 0.0
    scale = amax / 448.0 if amax > 0 else 1.0
    q = (x.float() / scale).clamp_(-448.0, 448.0).to(torch.float8_e4m3fn)
    return q, scale


def make_fp8_operands(M: int, N: int, K: int, seed: int = DEFAULT_SEED):
    A, B = make_operands("unit_normal", M, N, K, dtype=torch.float32, seed=seed)
    Aq, sa = quantize_e4m3(A)
    Bq, sb = quantize_e4m3(B)
    return Aq, sa, Bq, sb


# ------------------------------------------------------------ block-scaled fp8 (MXFP8)
def quantize_mxfp8(x: torch.Tensor):
    """Block-scaled fp8 of a [rows, K] float tensor, K a multiple of 32: every 32 consecutive K
    elements of a row share a power-of-two scale 2^(e - 127), e = ceil(log2(amax / 448)) + 127
    stored as one E8M0 byte, and the elements are e4m3_rne(x / scale). Returns
    (q [rows, K] float8_e4m3fn, e [rows, K / 32] uint8)."""
    rows, K = x.shape
    assert K % 32 == 0
    blocks = x.float().reshape(rows, K // 32, 32)
    amax = blocks.abs().amax(dim=2)
    exp = torch.ceil(torch.log2(torch.clamp(amax, min=2.0 ** -120) / 448.0)).clamp_(-127, 127)
    scale = torch.exp2(exp)
    q = (blocks / scale[..., None]).clamp_(-448.0, 448.0).to(torch.float8_e4m3fn).reshape(rows, K)
    return q, (exp + 127).to(torch.uint8)


def pack_mx_scales(e: torch.Tensor, fill: int = 127) -> torch.Tensor:
    """Scales [rows, K / 32] (uint8) in the layout the library's block-scaled GEMM takes: atoms of
    512 bytes covering 128 rows x 4 scales, atom index (row / 128) * ceil(K / 128) + kb / 4, byte
    (row % 32) * 16 + ((row % 128) / 32) * 4 + kb % 4 inside; padded to whole atoms with `fill`
    (127 = the scale 1.0; padding must not be 0xFF, which is NaN)."""
    rows, kb = e.shape
    rb, ka = (rows + 127) // 128, (kb + 3) // 4
    padded = torch.full((rb * 128, ka * 4), fill, dtype=torch.uint8, device=e.device)
    padded[:rows, :kb] = e
    # [rb, 4 (row / 32), 32 (row % 32), ka, 4 (kb % 4)] -> [rb, ka, 32, 4, 4]
    v = padded.view(rb, 4, 32, ka, 4).permute(0, 3, 2, 1, 4).contiguous()
    return v.view(-1)


def make_mxfp8_operands(M: int, N: int, K: int, seed: int = DEFAULT_SEED, workload: str = "unit_normal"):
    """(Aq, ea, Bq, eb): block-scaled fp8 operands drawn from a named distribution."""
    A, B = make_operands(workload, M, N, K, dtype=torch.float32, seed=seed)
    Aq, ea = quantize_mxfp8(A)
    Bq, eb = quantize_mxfp8(B)
    return Aq, ea, Bq, eb

"""ctypes binding of include/patina_gemm.h (the library's C ABI).

There is no fallback: if the shared library is missing, loading fails loudly.
"""
from __future__ import annotations

import ctypes as C
import os

LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_lib", "libpatina_gemm.so")

OK, ERR_INVALID_ARG, ERR_UNSUPPORTED_ARCH, ERR_CUDA, ERR_TIMEOUT = 0, 1, 2, 3, 4
IN_F16, IN_BF16, IN_E4M3, IN_MXE4M3 = 0, 1, 2, 3
OUT_BF16, OUT_F32, OUT_E4M3 = 0, 1, 2

# every symbol include/patina_gemm.h declares
SYMBOLS = (
    "patina_gemm_context_create", "patina_gemm_context_destroy", "patina_gemm_last_error",
    "patina_gemm_string_free", "patina_gemm_set_wait_limit_ns", "patina_gemm_status",
    "patina_gemm_launch_count", "patina_gemm_bf16_tn", "patina_gemm_fp8e4m3_tn",
    "patina_gemm_f16_tn_f32out", "patina_gemm_ex", "patina_gemm_host", "patina_gemm_validate",
    "patina_gemm_plan", "patina_gemm_smem_desc", "patina_gemm_idesc",
    "patina_gemm_k_advance_units", "patina_gemm_tmem_lane_offset", "patina_gemm_tile_coord",
    "patina_gemm_version", "patina_gemm_streamk_plan", "patina_gemm_streamk_chosen", "patina_gemm_streamk_range",
    "patina_gemm_streamk_owner", "patina_gemm_cluster_k_chosen", "patina_gemm_bf16_tn_skinny_noalloc", "patina_gemm_bf16_tn_scatter", "patina_gemm_bf16_tn_fused", "patina_gemm_bf16_tn_fused_fp8out", "patina_gemm_bf16_tn_grouped", "patina_gemm_fp8e4m3_tn_grouped",
    "patina_gemm_mxfp8_tn", "patina_gemm_mx_scale_bytes", "patina_gemm_mx_scale_offset", "patina_gemm_idesc_mx",
    "patina_gemm_column_shard", "patina_gemm_sharded_bf16_tn",
    "patina_gemm_peer_alloc",
    "patina_gemm_peer_open", "patina_gemm_peer_close", "patina_gemm_peer_free",
)


class StreamKPlan(C.Structure):
    _fields_ = [("grid", C.c_uint32), ("tiles", C.c_uint32), ("k_blocks", C.c_uint32),
                ("m_pad", C.c_uint32), ("max_contrib", C.c_uint32), ("stages", C.c_uint32),
                ("smem_bytes", C.c_uint32), ("units", C.c_uint64), ("partial_bytes", C.c_uint64),
                ("counter_bytes", C.c_uint64)]


class GemmConfig(C.Structure):
    _fields_ = [("cta_group", C.c_int32), ("block_n", C.c_int32), ("stages", C.c_int32),
                ("group_m", C.c_int32), ("max_ctas", C.c_int32), ("m_sub", C.c_int32), ("stream_k", C.c_int32),
                ("cluster_k", C.c_int32), ("k_order", C.c_int32)]


class GemmEpilogue(C.Structure):
    _fields_ = [("bias", C.c_void_p), ("residual", C.c_void_p), ("ldr", C.c_int64), ("beta", C.c_float),
                ("activation", C.c_int32)]


ACT_NONE, ACT_RELU, ACT_GELU, ACT_SILU = 0, 1, 2, 3


class GemmPlan(C.Structure):
    _fields_ = [("cta_group", C.c_int32), ("block_n", C.c_int32), ("stages", C.c_int32),
                ("group_m", C.c_int32), ("m_sub", C.c_int32), ("tile_m", C.c_uint32),
                ("tiles_m", C.c_uint32), ("tiles_n", C.c_uint32),
                ("num_tiles", C.c_uint32), ("k_blocks", C.c_uint32), ("grid", C.c_uint32),
                ("block", C.c_uint32), ("cluster", C.c_uint32), ("smem_bytes", C.c_uint32),
                ("tmem_cols", C.c_uint32), ("stage_bytes", C.c_uint32),
                ("expect_tx_bytes", C.c_uint32), ("idesc", C.c_uint32), ("half_tiles", C.c_uint32)]


_lib = None


def load() -> C.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.isfile(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m patina_b200.build` "
            "(this package has no CPU or PyTorch fallback)")
    L = C.CDLL(LIB_PATH)
    vp, i64, i32, f32 = C.c_void_p, C.c_int64, C.c_int, C.c_float
    L.patina_gemm_context_create.argtypes = [i32, C.POINTER(vp)]
    L.patina_gemm_context_destroy.argtypes = [vp]
    L.patina_gemm_context_destroy.restype = None
    L.patina_gemm_last_error.argtypes = [vp]
    L.patina_gemm_last_error.restype = vp
    L.patina_gemm_string_free.argtypes = [vp]
    L.patina_gemm_string_free.restype = None
    L.patina_gemm_set_wait_limit_ns.argtypes = [vp, C.c_uint64]
    L.patina_gemm_status.argtypes = [vp, vp]
    L.patina_gemm_launch_count.argtypes = [vp]
    L.patina_gemm_launch_count.restype = C.c_uint64
    gemm_args = [vp, vp, i64, vp, i64, vp, i64, i64, i64, i64]
    L.patina_gemm_bf16_tn.argtypes = gemm_args + [f32, vp]
    L.patina_gemm_fp8e4m3_tn.argtypes = gemm_args + [f32, f32, vp]
    L.patina_gemm_f16_tn_f32out.argtypes = gemm_args + [f32, vp]
    ex_args = [vp, i32, i32, vp, i64, vp, i64, vp, i64, i64, i64, i64, f32,
               C.POINTER(GemmConfig), vp]
    L.patina_gemm_ex.argtypes = ex_args
    L.patina_gemm_host.argtypes = ex_args
    L.patina_gemm_validate.argtypes = [i32, i32, vp, i64, vp, i64, vp, i64, i64, i64, i64,
                                       C.POINTER(vp)]
    L.patina_gemm_plan.argtypes = [i32, i32, i64, i64, i64, C.POINTER(GemmConfig), i32,
                                   C.POINTER(GemmPlan)]
    L.patina_gemm_smem_desc.argtypes = [C.c_uint32, C.c_uint32, C.c_uint32, i32]
    L.patina_gemm_smem_desc.restype = C.c_uint64
    L.patina_gemm_idesc.argtypes = [i32, C.c_uint32, C.c_uint32]
    L.patina_gemm_idesc.restype = C.c_uint32
    L.patina_gemm_k_advance_units.argtypes = [C.c_uint32, i32]
    L.patina_gemm_k_advance_units.restype = C.c_uint32
    L.patina_gemm_tmem_lane_offset.argtypes = [C.c_uint32]
    L.patina_gemm_tmem_lane_offset.restype = C.c_uint32
    L.patina_gemm_tile_coord.argtypes = [C.c_uint32] * 4 + [C.POINTER(C.c_uint32)] * 2
    L.patina_gemm_tile_coord.restype = None
    L.patina_gemm_version.restype = C.c_char_p
    L.patina_gemm_streamk_plan.argtypes = [i32, i64, i64, i64, i32, C.POINTER(StreamKPlan)]
    L.patina_gemm_streamk_chosen.argtypes = [i32, i32, i64, i64, i64, i32]
    L.patina_gemm_cluster_k_chosen.argtypes = [i32, i32, i64, i64, i64, i32]
    L.patina_gemm_streamk_range.argtypes = [C.c_uint64] * 3 + [C.POINTER(C.c_uint64)] * 2
    L.patina_gemm_streamk_range.restype = None
    L.patina_gemm_streamk_owner.argtypes = [C.c_uint64] * 3
    L.patina_gemm_streamk_owner.restype = C.c_uint32
    L.patina_gemm_bf16_tn_scatter.argtypes = [vp, vp, i64, vp, i64, C.POINTER(vp), i32, i64, i64, i64, i64, f32, vp]
    L.patina_gemm_bf16_tn_fused_fp8out.argtypes = gemm_args + [f32, C.POINTER(GemmEpilogue), f32, vp, vp]
    L.patina_gemm_bf16_tn_grouped.argtypes = [vp, vp, i64, vp, i64, vp, i64, vp, i32, i64, i64, i64, f32,
                                              C.POINTER(GemmConfig), vp]
    L.patina_gemm_fp8e4m3_tn_grouped.argtypes = [vp, vp, i64, vp, i64, vp, i64, vp, i32, i64, i64, i64, f32,
                                                 vp, C.POINTER(GemmConfig), vp]
    L.patina_gemm_bf16_tn_fused.argtypes = gemm_args + [f32, C.POINTER(GemmEpilogue), vp]
    L.patina_gemm_peer_alloc.argtypes = [vp, C.c_size_t, C.POINTER(vp), C.c_char_p]
    L.patina_gemm_peer_open.argtypes = [vp, C.c_char_p, C.POINTER(vp)]
    L.patina_gemm_peer_close.argtypes = [vp, vp]
    L.patina_gemm_peer_free.argtypes = [vp, vp]
    L.patina_gemm_mxfp8_tn.argtypes = [vp, vp, i64, vp, vp, i64, vp, vp, i64, i64, i64, i64, f32,
                                       C.POINTER(GemmConfig), vp]
    L.patina_gemm_mx_scale_bytes.argtypes = [i64, i64]
    L.patina_gemm_mx_scale_bytes.restype = C.c_uint64
    L.patina_gemm_mx_scale_offset.argtypes = [i64, i64, i64]
    L.patina_gemm_mx_scale_offset.restype = C.c_uint64
    L.patina_gemm_idesc_mx.argtypes = [C.c_uint32] * 4
    L.patina_gemm_idesc_mx.restype = C.c_uint32
    L.patina_gemm_column_shard.argtypes = [i64, i32, i32, C.POINTER(i64), C.POINTER(i64)]
    L.patina_gemm_column_shard.restype = None
    L.patina_gemm_sharded_bf16_tn.argtypes = [C.POINTER(vp), i32, C.POINTER(vp), i64, C.POINTER(vp), i64,
                                              C.POINTER(vp), i64, i64, i64, i64, f32, C.POINTER(vp)]
    L.patina_gemm_bf16_tn_skinny_noalloc.argtypes = [vp, i64, vp, i64, vp, i64, i64, i64, i64, f32, vp,
                                                     C.c_char_p, C.c_size_t]
    _lib = L
    return L


def take_string(ptr) -> str | None:
    """Copy and free a heap string returned by the library (NULL -> None)."""
    if not ptr:
        return None
    s = C.cast(ptr, C.c_char_p).value.decode()
    load().patina_gemm_string_free(ptr)
    return s


def plan(in_type, out_type, M, N, K, config: GemmConfig | None = None, num_sms: int = 148) -> GemmPlan:
    p = GemmPlan()
    rc = load().patina_gemm_plan(in_type, out_type, M, N, K,
                                 C.byref(config) if config is not None else None, num_sms,
                                 C.byref(p))
    if rc != OK:
        raise ValueError(f"patina_gemm_plan failed with code {rc}")
    return p


def streamk_plan(in_type, M, N, K, num_sms: int = 148) -> StreamKPlan:
    p = StreamKPlan()
    rc = load().patina_gemm_streamk_plan(in_type, M, N, K, num_sms, C.byref(p))
    if rc != OK:
        raise ValueError(f"patina_gemm_streamk_plan failed with code {rc}")
    return p


def validate(in_type, out_type, A, lda, B, ldb, Cp, ldc, M, N, K) -> str | None:
    """None when the arguments are acceptable, else the library's diagnostic."""
    err = C.c_void_p()
    rc = load().patina_gemm_validate(in_type, out_type, A, lda, B, ldb, Cp, ldc, M, N, K,
                                     C.byref(err))
    msg = take_string(err.value)
    return None if rc == OK else (msg or f"error {rc}")

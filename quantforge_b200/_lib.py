"""ctypes binding of libquantforge_rt.so (the C ABI in include/quantforge_rt.h).

There is no fallback: if the shared library is missing the import of any compute entry
point raises, and every compute call needs a CUDA device.
"""
from __future__ import annotations

import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "lib", "libquantforge_rt.so")

QF_OK = 0
QF_F16, QF_BF16, QF_F32 = 0, 1, 2
QF_ZERO_CONST, QF_ZERO_U4, QF_ZERO_I8 = 0, 1, 2
QF_PATH_AUTO, QF_PATH_GEMV, QF_PATH_GEMM = 0, 1, 2
QF_LAYOUT_CANONICAL, QF_LAYOUT_INTERLEAVED, QF_LAYOUT_TILED, QF_LAYOUT_GEMV_SLAB = 0, 1, 2, 3
QF_EPI_NONE, QF_EPI_SILU_MUL, QF_EPI_RESIDUAL_ADD = 0, 1, 2
QF_SLAB_UNIT_BYTES = 4352
QF_SLAB_MAX_M = 32

# every symbol include/quantforge_rt.h declares
EXPORTS = [
    "qf_version", "qf_status_string", "qf_ctx_create", "qf_ctx_destroy", "qf_last_error", "qf_unpack_int4",
    "qf_dequant_w4", "qf_w4a16_workspace_bytes", "qf_w4a16_linear", "qf_w4a16_linear_host", "qf_w4a16_plan",
    "qf_launch_count", "qf_prepack_w4", "qf_prepack_w4_tiled", "qf_w4a16_gemv_static_scratch", "qf_ctx_status", "qf_ctx_clear_status",
    "qf_comm_create", "qf_comm_export", "qf_comm_connect", "qf_comm_destroy", "qf_w4a16_linear_allreduce",
    "qf_w4a16_linear_allgather", "qf_w4a16_linear_host_async", "qf_w4a16_linear_fused", "qf_w4a16_linear_batched",
    "qf_prepack_bytes", "qf_prepack_gemv_slab", "qf_unpack_gemv_slab", "qf_repack_kn_to_canonical",
]
QF_COMM_HANDLE_BYTES = 64


class LinearDesc(ctypes.Structure):
    _fields_ = [
        ("M", ctypes.c_int64), ("N", ctypes.c_int64), ("K", ctypes.c_int64),
        ("group_size", ctypes.c_int32), ("act_dtype", ctypes.c_int32), ("out_dtype", ctypes.c_int32),
        ("zero_mode", ctypes.c_int32), ("zero_const", ctypes.c_int32), ("path", ctypes.c_int32),
        ("split_k", ctypes.c_int32), ("weight_layout", ctypes.c_int32), ("epilogue", ctypes.c_int32),
        ("reserved", ctypes.c_int32 * 3),
    ]


class QuantForgeError(RuntimeError):
    def __init__(self, status: int, name: str, message: str):
        super().__init__(f"{name} ({status}): {message}")
        self.status = status
        self.name = name


_lib = None


def load() -> ctypes.CDLL:
    """Load the runtime library, or raise (no CPU path exists)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m quantforge_b200.build` (needs nvcc). "
            "quantforge_b200 has no CPU fallback.")
    lib = ctypes.CDLL(LIB_PATH)
    vp, i64, i32, sz = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int32, ctypes.c_size_t
    dp = ctypes.POINTER(LinearDesc)
    lib.qf_version.restype = ctypes.c_int
    lib.qf_status_string.restype = ctypes.c_char_p
    lib.qf_status_string.argtypes = [ctypes.c_int]
    lib.qf_ctx_create.argtypes = [ctypes.POINTER(vp), ctypes.c_int]
    lib.qf_ctx_destroy.argtypes = [vp]
    lib.qf_last_error.restype = ctypes.c_char_p
    lib.qf_last_error.argtypes = [vp]
    lib.qf_unpack_int4.argtypes = [vp, vp, vp, i64, i64, vp]
    lib.qf_dequant_w4.argtypes = [vp, dp, vp, vp, vp, vp, vp]
    lib.qf_w4a16_workspace_bytes.restype = sz
    lib.qf_w4a16_workspace_bytes.argtypes = [dp]
    lib.qf_w4a16_linear.argtypes = [vp, dp, vp, vp, vp, vp, vp, vp, sz, vp]
    lib.qf_w4a16_linear_fused.argtypes = [vp, dp, vp, vp, vp, vp, vp, vp, vp, sz, vp]
    pvp = ctypes.POINTER(vp)
    lib.qf_w4a16_linear_batched.argtypes = [vp, ctypes.c_int, dp, pvp, pvp, pvp, pvp, pvp, pvp, vp, sz, vp]
    lib.qf_prepack_bytes.restype = sz
    lib.qf_prepack_bytes.argtypes = [ctypes.c_int, i64, i64]
    lib.qf_prepack_gemv_slab.argtypes = [vp, dp, vp, vp, vp, vp, vp]
    lib.qf_unpack_gemv_slab.argtypes = [vp, i64, i64, vp, vp, vp]
    lib.qf_repack_kn_to_canonical.argtypes = [vp, vp, ctypes.c_int, i64, i64, vp, vp]
    lib.qf_w4a16_linear_host.argtypes = [vp, dp, vp, vp, vp, vp, vp, vp, sz, vp]
    lib.qf_w4a16_linear_host_async.argtypes = [vp, dp, vp, vp, vp, vp, vp, vp, sz, vp]
    lib.qf_w4a16_gemv_static_scratch.argtypes = [vp, dp, vp, vp, vp, vp, vp, vp]
    lib.qf_w4a16_plan.argtypes = [dp, ctypes.POINTER(i32), ctypes.POINTER(i32)]
    lib.qf_launch_count.restype = i64
    lib.qf_prepack_w4.argtypes = [vp, vp, vp, i64, ctypes.c_int, vp]
    lib.qf_prepack_w4_tiled.argtypes = [vp, vp, vp, i64, i64, ctypes.c_int, vp]
    lib.qf_ctx_status.argtypes = [vp]
    lib.qf_ctx_clear_status.argtypes = [vp]
    lib.qf_comm_create.argtypes = [vp, ctypes.c_int, ctypes.c_int, sz, ctypes.POINTER(vp)]
    lib.qf_comm_export.argtypes = [vp, vp]
    lib.qf_comm_connect.argtypes = [vp, vp, ctypes.c_int]
    lib.qf_comm_destroy.argtypes = [vp]
    lib.qf_w4a16_linear_allreduce.argtypes = [vp, vp, dp, vp, vp, vp, vp, vp, vp, sz, vp]
    lib.qf_w4a16_linear_allgather.argtypes = [vp, vp, dp, vp, vp, vp, vp, vp, vp, sz, vp]
    _lib = lib
    return lib


def status_name(status: int) -> str:
    return load().qf_status_string(status).decode()

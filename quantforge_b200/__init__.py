"""quantforge_b200: B200 (sm_100a) runtime for QuantForge's W4A16 hot path.

Host-side mirror of the reference's Python interface (python/quantforge/baseline.py:
pack_int4, unpack_int4, gemv_int4_baseline) on top of the C ABI in include/quantforge_rt.h.
"""
from .ops import (  # noqa: F401
    Comm, W4A16Linear, clear_device_status, dequant_w4, device_status, gemv_int4, launch_count, pack_int4, pack_zeros_u4,
    prepack_w4, unpack_int4, w4a16_linear, w4a16_linear_allgather, w4a16_linear_allreduce, w4a16_linear_host, workspace_bytes,
    SlabWeight, interleave_gate_up, prepack_gemv_slab, repack_kn_to_canonical, unpack_gemv_slab,
)
from ._lib import (QF_EPI_NONE, QF_EPI_RESIDUAL_ADD, QF_EPI_SILU_MUL, QF_LAYOUT_CANONICAL, QF_LAYOUT_GEMV_SLAB,  # noqa: F401
                   QF_LAYOUT_INTERLEAVED, QF_LAYOUT_TILED, QF_PATH_AUTO, QF_PATH_GEMM, QF_PATH_GEMV, QuantForgeError)

__version__ = "0.1.0"

"""Group-wise INT4 quantisation and packing of a floating-point weight (the inverse of qf.unpack + qf.dequant).

    codes, scales, zeros = quantize_w4(weight, group_size=128, symmetric=False)
    qweight = pack_int4(codes)                      # int8 [N, K/2], the canonical layout of the runtime
    qzeros  = pack_zeros_u4(zeros)                  # int32 [G, N/8]   (asymmetric only)

Layout helpers only (plain torch ops, any device); nothing here is on the inference hot path. The packing rule is the
reference's `pack_int4` (python/quantforge/baseline.py:17-31); quantisation itself has no counterpart in the reference,
which starts from already-quantised codes.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .ops import pack_int4, pack_zeros_u4  # noqa: F401  (re-exported for convenience)


def quantize_w4(weight: torch.Tensor, group_size: int = 128, symmetric: bool = False,
                scale_dtype: Optional[torch.dtype] = None) -> Tuple[torch.Tensor, torch.Tensor, Optional[torch.Tensor]]:
    """weight [N, K] float -> (codes int8 [N, K] in [0,15], scales [G, N], zeros int8 [G, N] or None).

    asymmetric: per (group, row) scale = (max - min) / 15, zero = round(-min / scale) clamped to [0, 15];
    symmetric : scale = max|w| / 7, zero is the constant 8.
    The scale is rounded to `scale_dtype` (default: weight dtype if 16-bit, else float16) BEFORE the codes are
    chosen, so that dequantising with the stored scale reproduces the quantiser's own reconstruction.
    """
    if weight.dim() != 2:
        raise ValueError("weight must be [N, K]")
    N, K = weight.shape
    if K % group_size != 0:
        raise ValueError("K must be a multiple of group_size")
    if scale_dtype is None:
        scale_dtype = weight.dtype if weight.dtype in (torch.float16, torch.bfloat16) else torch.float16
    G = K // group_size
    w = weight.float().reshape(N, G, group_size)
    if symmetric:
        amax = w.abs().amax(dim=-1)
        scale = (amax / 7.0).clamp_min(2.0 ** -14).to(scale_dtype).float()
        q = torch.round(w / scale.unsqueeze(-1)) + 8.0
        zeros = None
    else:
        wmin, wmax = w.amin(dim=-1), w.amax(dim=-1)
        scale = ((wmax - wmin) / 15.0).clamp_min(2.0 ** -14).to(scale_dtype).float()
        zero = torch.round(-wmin / scale).clamp_(0, 15)
        q = torch.round(w / scale.unsqueeze(-1)) + zero.unsqueeze(-1)
        zeros = zero.to(torch.int8).t().contiguous()          # [G, N]
    codes = q.clamp_(0, 15).to(torch.int8).reshape(N, K)
    scales = scale.to(scale_dtype).t().contiguous()            # [G, N]
    return codes, scales, zeros


def dequantize_reference(codes: torch.Tensor, scales: torch.Tensor, zeros: Optional[torch.Tensor], group_size: int,
                         zero_const: int = 8) -> torch.Tensor:
    """float32 reconstruction (q - z) * s, for checking a quantisation; not a compute path."""
    N, K = codes.shape
    G = K // group_size
    q = codes.float().reshape(N, G, group_size)
    z = (zeros.float().t() if zeros is not None else torch.full((N, G), float(zero_const), device=codes.device))
    return ((q - z.unsqueeze(-1)) * scales.float().t().unsqueeze(-1)).reshape(N, K)

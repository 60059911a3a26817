"""Quantise + pack tool: round trips and error bounds (CPU, layout helpers only)."""
import numpy as np
import pytest
import torch

from oracle import qf_oracle as O
from quantforge_b200 import quantize as Q


@pytest.mark.parametrize("symmetric", [False, True])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_quantise_error_is_within_half_a_step(symmetric, dtype):
    torch.manual_seed(0)
    w = (torch.randn(64, 512) * 0.05).to(dtype)
    codes, scales, zeros = Q.quantize_w4(w, 128, symmetric)
    assert codes.dtype == torch.int8 and codes.min() >= 0 and codes.max() <= 15
    assert scales.shape == (4, 64) and scales.dtype == dtype
    assert (zeros is None) == symmetric
    rec = Q.dequantize_reference(codes, scales, zeros, 128)
    step = scales.float().t().repeat_interleave(128, dim=1)
    # half a quantisation step, plus the slack of rounding the scale to 16 bits (the range is 16 steps wide)
    eps = 2.0 ** -11 if dtype == torch.float16 else 2.0 ** -8
    assert torch.all((rec - w.float()).abs() <= (0.5 + 16 * eps) * step + 1e-6) or symmetric
    if symmetric:  # the symmetric grid clips the positive extreme by at most one step
        assert torch.all((rec - w.float()).abs() <= 1.01 * step + 1e-6)


def test_pack_matches_oracle_and_dequant_matches_oracle():
    torch.manual_seed(1)
    w = (torch.randn(32, 256) * 0.02).half()
    codes, scales, zeros = Q.quantize_w4(w, 128, False)
    packed = Q.pack_int4(codes)
    assert np.array_equal(packed.numpy(), O.pack_int4(codes.numpy()))
    assert np.array_equal(O.unpack_int4(packed.numpy()), codes.numpy())
    want = O.dequant(codes.numpy(), scales.float().numpy(), zeros.numpy(), 128, "f16")
    rec = Q.dequantize_reference(codes, scales, zeros, 128).half().float().numpy()
    assert np.max(np.abs(rec - want)) <= np.max(np.abs(want)) * 2 ** -10
    zw = Q.pack_zeros_u4(zeros).numpy().view(np.uint32)
    assert np.array_equal(O.unpack_words(zw), zeros.numpy())

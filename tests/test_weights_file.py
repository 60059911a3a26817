"""On-disk container of quantised linears: round trip, corruption check (CPU); quantise -> save -> load -> prepack ->
kernel against the floating-point matmul (GPU)."""
import numpy as np
import pytest
import torch

from oracle import qf_oracle as O
from quantforge_b200 import weights_file as W


def _linears():
    torch.manual_seed(3)
    a = W.quantize_linear((torch.randn(64, 256) * 0.05).half(), 128, symmetric=False)
    b = W.quantize_linear((torch.randn(128, 512) * 0.02).bfloat16(), 256, symmetric=True)
    return {"layers.0.q_proj": a, "layers.0.down_proj": b}


def test_round_trip_is_bit_exact(tmp_path):
    lin = _linears()
    path = str(tmp_path / "w.qfw4")
    W.save_w4(path, lin)
    back = W.load_w4(path)
    assert sorted(back) == sorted(lin)
    for name in lin:
        a, b = lin[name], back[name]
        assert torch.equal(a.qweight, b.qweight) and a.scales.dtype == b.scales.dtype
        assert torch.equal(a.scales.view(torch.int16), b.scales.view(torch.int16))
        assert (a.zeros is None) == (b.zeros is None) and (a.zeros is None or torch.equal(a.zeros, b.zeros))
        assert (a.group_size, a.zero_const, a.N, a.K) == (b.group_size, b.zero_const, b.N, b.K)
    # the stored codes are the reference's packing: unpack gives the quantiser's codes back
    q = lin["layers.0.q_proj"]
    codes = O.unpack_int4(back["layers.0.q_proj"].qweight.numpy())
    assert codes.min() >= 0 and codes.max() <= 15 and np.array_equal(O.pack_int4(codes), q.qweight.numpy())


def test_corruption_is_detected(tmp_path):
    path = str(tmp_path / "w.qfw4")
    W.save_w4(path, _linears())
    raw = bytearray(open(path, "rb").read())
    raw[-100] ^= 0x40
    open(path, "wb").write(bytes(raw))
    with pytest.raises(ValueError):
        W.load_w4(path)
    with pytest.raises(ValueError):
        bad = str(tmp_path / "bad.qfw4")
        open(bad, "wb").write(b"not a weights file")
        W.load_w4(bad)


@pytest.mark.gpu
@pytest.mark.parametrize("M,symmetric,dtype", [(1, False, torch.bfloat16), (4, True, torch.float16), (24, False, torch.float16)])
def test_quantise_save_load_prepack_run(tmp_path, M, symmetric, dtype):
    """The whole chain a checkpoint goes through, against the matmul with the ORIGINAL floating-point weight: the error
    is what 4-bit quantisation allows (half a step per weight, accumulated over K), not more."""
    import quantforge_b200 as qf
    dev = torch.device("cuda:0")
    torch.manual_seed(M)
    N, K, g = 256, 1024, 128
    w = (torch.randn(N, K) * 0.05).to(dtype)
    x = torch.randn(M, K).to(dtype)
    path = str(tmp_path / "layer.qfw4")
    W.save_w4(path, {"lin": W.quantize_linear(w, g, symmetric)})
    lin = W.load_w4(path, device=dev)["lin"]
    xd = x.to(dev)
    y_canon = qf.w4a16_linear(xd, lin.qweight, lin.scales, lin.kernel_zeros(), g, lin.zero_const, torch.float32)
    outs = [y_canon]
    if M <= 32:
        outs.append(qf.w4a16_linear(xd, lin.to_slab(), out_dtype=torch.float32))
    torch.cuda.synchronize()
    # exact statement of what the kernels must compute from the stored tensors
    zeros_np = lin.zeros.cpu().numpy() if lin.zeros is not None else lin.zero_const
    act = "f16" if dtype == torch.float16 else "bf16"
    want = O.w4a16_linear(x.float().numpy(), lin.qweight.cpu().numpy(), lin.scales.float().cpu().numpy(), zeros_np, g,
                          act, O.F32, accumulate="f64")
    for y in outs:
        assert O.rel_err(y.cpu().numpy(), want) < 1e-4
    # and against the unquantised weight: bounded by the quantisation step (s/2 per weight, s for the clipped
    # extreme of the symmetric grid), summed in quadrature over K
    y_fp = x.double() @ w.double().t()
    step = lin.scales.float().cpu().t().repeat_interleave(g, dim=1).double()          # [N, K]
    bound = ((1.0 if symmetric else 0.5) * step * x.double().abs().max()).pow(2).sum(dim=1).sqrt()  # [N]
    err = (outs[0].cpu().double() - y_fp).abs().max(dim=0).values
    assert torch.all(err <= 4.0 * bound + 1e-3)

"""GPU parity: the CUDA kernels, called through the C ABI, against the CPU oracle and the golden fixtures."""
import os

import numpy as np
import pytest
import torch

from oracle import qf_oracle as O

pytestmark = pytest.mark.gpu

TOL = 1e-2  # max |y - y_ref| / rms(y_ref), the tolerance the parity target states


@pytest.fixture(scope="module")
def qf():
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    import quantforge_b200 as qf
    return qf


def _t(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a))
    if dtype is not None:
        t = t.to(dtype)
    return t.cuda()


_TD = {"f16": torch.float16, "bf16": torch.bfloat16, "f32": torch.float32}


# ------------------------------------------------------------------------------------------
# qf.unpack: bit-exact
# ------------------------------------------------------------------------------------------
def test_unpack_exhaustive_byte_table(qf, golden_dir):
    g = np.load(os.path.join(golden_dir, "unpack.npz"))
    got = qf.unpack_int4(_t(g["all_bytes"])).cpu().numpy()
    assert np.array_equal(got, g["unpacked_table"])


def test_unpack_golden_round_trip(qf, golden_dir):
    g = np.load(os.path.join(golden_dir, "unpack.npz"))
    got = qf.unpack_int4(_t(g["packed"])).cpu().numpy()
    assert np.array_equal(got, g["codes"])
    # pack (layout helper) then unpack (kernel) is the identity, as the reference script asserts
    packed = qf.pack_int4(_t(g["codes"]))
    assert np.array_equal(packed.cpu().numpy(), g["packed"])
    assert np.array_equal(qf.unpack_int4(packed).cpu().numpy(), g["codes"])


@pytest.mark.parametrize("shape", [(1, 1), (3, 5), (7, 16), (5, 48), (33, 100), (4096, 2048), (0, 8), (4, 0)])
def test_unpack_shapes_vs_oracle(qf, shape):
    rng = np.random.default_rng(sum(shape))
    packed = rng.integers(-128, 128, size=shape, dtype=np.int8)
    got = qf.unpack_int4(_t(packed)).cpu().numpy()
    assert got.shape == (shape[0], shape[1] * 2)
    assert np.array_equal(got, O.unpack_int4(packed))


def test_unpack_does_not_write_outside_output(qf):
    rng = np.random.default_rng(1)
    packed = _t(rng.integers(-128, 128, size=(9, 16), dtype=np.int8))
    import ctypes
    from quantforge_b200 import _lib, ops
    buf = torch.full((9 * 32 + 64,), 0x55, dtype=torch.int8, device="cuda")
    ctx = ops._ctx(packed.device)
    st = _lib.load().qf_unpack_int4(ctx, ctypes.c_void_p(packed.data_ptr()), ctypes.c_void_p(buf.data_ptr() + 32), 9, 16,
                                    None)
    assert st == 0
    torch.cuda.synchronize()
    out = buf.cpu().numpy()
    assert np.all(out[:32] == 0x55) and np.all(out[32 + 9 * 32:] == 0x55)
    assert np.array_equal(out[32:32 + 9 * 32].reshape(9, 32), O.unpack_int4(packed.cpu().numpy()))


# ------------------------------------------------------------------------------------------
# qf.dequant(qf.unpack): bit-exact per element against the oracle
# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("act", ["f16", "bf16"])
@pytest.mark.parametrize("zero_kind", ["u4", "const8", "const0", "i8"])
def test_dequant_bit_exact(qf, act, zero_kind):
    d = O.make_inputs(M=1, K=512, N=64, group_size=128, act_dtype=act, seed=5)
    if zero_kind == "u4":
        z_np, z_t, zc = d["zeros"], qf.pack_zeros_u4(_t(d["zeros"])), 0
    elif zero_kind == "i8":
        z_np = (d["zeros"].astype(np.int32) * 3 - 20).astype(np.int8)  # signed, outside [0, 15]
        z_t, zc = _t(z_np), 0
    else:
        zc = 8 if zero_kind == "const8" else 0
        z_np, z_t = zc, None
    want = O.dequant(d["codes"], d["scales"], z_np, 128, act)
    got = qf.dequant_w4(_t(d["qweight"]), _t(d["scales"], _TD[act]), z_t, 128, zc).float().cpu().numpy()
    assert np.array_equal(got, want)


# ------------------------------------------------------------------------------------------
# linear: golden fixtures of the reference function, then the oracle on wider cases
# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("case", ["m1", "m4", "m16", "signed"])
def test_gemv_int4_matches_reference_golden(qf, golden_dir, case):
    g = np.load(os.path.join(golden_dir, "gemv_per_channel.npz"))
    y = qf.gemv_int4(_t(g[f"{case}_x"]), _t(g[f"{case}_w_packed"]), _t(g[f"{case}_scale"]),
                     _t(g[f"{case}_zero_point"]))
    assert y.dtype == torch.float16
    want = g[f"{case}_y"].astype(np.float32)
    assert O.rel_err(y.float().cpu().numpy(), want) < TOL


def _run_linear(qf, M, K, N, g, act, zero_kind, out="f32", seed=0, path=0, split_k=0, sigma=0.02):
    d = O.make_inputs(M=M, K=K, N=N, group_size=g, act_dtype=act, seed=seed, sigma=sigma)
    if zero_kind == "u4":
        z_np, z_t, zc = d["zeros"], qf.pack_zeros_u4(_t(d["zeros"])), 0
    elif zero_kind == "i8":
        z_np = (d["zeros"].astype(np.int32) - 8).astype(np.int8)
        z_t, zc = _t(z_np), 0
    else:
        z_np, z_t, zc = 8, None, 8
    want = O.w4a16_linear(d["x"], d["qweight"], d["scales"], z_np, g, act, O.F32, accumulate="f64")
    y = qf.w4a16_linear(_t(d["x"], _TD[act]), _t(d["qweight"]), _t(d["scales"], _TD[act]), z_t, group_size=g,
                        zero_const=zc, out_dtype=_TD[out], path=path, split_k=split_k)
    return y.float().cpu().numpy(), want


@pytest.mark.parametrize("act", ["f16", "bf16"])
@pytest.mark.parametrize("M", [1, 2, 3, 5, 8])
@pytest.mark.parametrize("zero_kind", ["u4", "const", "i8"])
def test_gemv_small_vs_oracle(qf, act, M, zero_kind):
    got, want = _run_linear(qf, M, 512, 64, 128, act, zero_kind, seed=M)
    assert O.rel_err(got, want) < 1e-4  # fp32 output, identical weights: only accumulation order differs


@pytest.mark.parametrize("shape", [(1, 128, 16), (1, 256, 48), (4, 1024, 80), (8, 2048, 272), (7, 384, 1040)])
@pytest.mark.parametrize("split_k", [0, 1, 2, 3])
def test_gemv_ragged_shapes_and_splits(qf, shape, split_k):
    M, K, N = shape
    got, want = _run_linear(qf, M, K, N, 128, "bf16", "u4", seed=K + N, split_k=split_k)
    assert O.rel_err(got, want) < 1e-4


@pytest.mark.parametrize("g", [128, 256, 1024])
def test_group_sizes(qf, g):
    got, want = _run_linear(qf, 2, 1024, 128, g, "f16", "u4", seed=g)
    assert O.rel_err(got, want) < 1e-4


@pytest.mark.parametrize("out", ["f16", "bf16", "f32"])
def test_output_dtypes(qf, out):
    got, want = _run_linear(qf, 4, 1024, 256, 128, "bf16", "u4", out=out, seed=9)
    # bf16 output rounding alone is 2^-9 relative of the largest outputs (several rms): looser bound there
    bound = {"f32": 1e-4, "f16": 3e-3, "bf16": 2e-2}[out]
    assert O.rel_err(got, want) < bound
    assert np.array_equal(got, O.round_to(got, out))


def test_config0_reference_gemv_f16(qf):
    """M=1, K=N=4096, g128, asymmetric, f16 in/out: the benchmark's GEMV configuration."""
    got, want = _run_linear(qf, 1, 4096, 4096, 128, "f16", "u4", out="f16", seed=0)
    assert O.rel_err(got, want) < TOL


@pytest.mark.parametrize("M", [1, 4, 8, 16, 64])
@pytest.mark.parametrize("KN", [(4096, 4096), (4096, 14336), (14336, 4096)])
def test_config1_sweep_bf16(qf, M, KN):
    K, N = KN
    got, want = _run_linear(qf, M, K, N, 128, "bf16", "u4", out="f32", seed=1)
    assert O.rel_err(got, want) < TOL


def test_deterministic_and_workspace_reuse(qf):
    d = O.make_inputs(M=3, K=4096, N=512, group_size=128, act_dtype="bf16", seed=3)
    args = (_t(d["x"], torch.bfloat16), _t(d["qweight"]), _t(d["scales"], torch.bfloat16),
            qf.pack_zeros_u4(_t(d["zeros"])))
    ys = [qf.w4a16_linear(*args, out_dtype=torch.float32).clone() for _ in range(4)]
    for y in ys[1:]:
        assert torch.equal(y, ys[0])


def test_linearity_in_x_full_size(qf):
    """Size-independent property at a benchmark-size layer: the op is linear in X."""
    M, K, N = 4, 14336, 4096
    d = O.make_inputs(M=M, K=K, N=N, group_size=128, act_dtype="f16", seed=4)
    qw, s, z = _t(d["qweight"]), _t(d["scales"], torch.float16), qf.pack_zeros_u4(_t(d["zeros"]))
    x1 = _t(d["x"], torch.float16)
    x2 = torch.flip(x1, dims=[1]).contiguous()
    y1 = qf.w4a16_linear(x1, qw, s, z, out_dtype=torch.float32)
    y2 = qf.w4a16_linear(x2, qw, s, z, out_dtype=torch.float32)
    y12 = qf.w4a16_linear((x1.float() * 0.5 + x2.float() * 0.25).half(), qw, s, z, out_dtype=torch.float32)
    want = 0.5 * y1 + 0.25 * y2
    rms = want.pow(2).mean().sqrt()
    assert ((y12 - want).abs().max() / rms).item() < 5e-3  # x rounding to f16 only


def test_host_entry_point(qf):
    d = O.make_inputs(M=2, K=1024, N=256, group_size=128, act_dtype="f16", seed=6)
    x_host = torch.from_numpy(d["x"]).half().pin_memory()
    y = qf.w4a16_linear_host(x_host, _t(d["qweight"]), _t(d["scales"], torch.float16),
                             qf.pack_zeros_u4(_t(d["zeros"])), out_dtype=torch.float32)
    assert not y.is_cuda
    want = O.w4a16_linear(d["x"], d["qweight"], d["scales"], d["zeros"], 128, "f16", O.F32, accumulate="f64")
    assert O.rel_err(y.numpy(), want) < 1e-4


def test_host_entry_point_async(qf):
    """wait=False: several calls back to back on one stream, one synchronisation, same results as the waiting call."""
    outs, wants = [], []
    for seed, (M, K, N) in enumerate([(1, 1024, 512), (4, 2048, 256), (2, 512, 1024)]):
        d = O.make_inputs(M=M, K=K, N=N, group_size=128, act_dtype="f16", seed=20 + seed)
        x_host = torch.from_numpy(d["x"]).half().pin_memory()
        args = (_t(d["qweight"]), _t(d["scales"], torch.float16), qf.pack_zeros_u4(_t(d["zeros"])))
        wants.append(qf.w4a16_linear_host(x_host, *args, out_dtype=torch.float32).clone())
        out = torch.empty(M, N, dtype=torch.float32).pin_memory()
        outs.append((x_host, args, out))
    for x_host, args, out in outs:
        qf.w4a16_linear_host(x_host, *args, out_dtype=torch.float32, out_host=out, wait=False)
    torch.cuda.synchronize()
    for (_, _, out), want in zip(outs, wants):
        assert torch.equal(out, want)


def test_layer_object_host_path(qf):
    """W4A16Linear.forward_host (prepared descriptors, waiting and not waiting) equals the plain device call."""
    d = O.make_inputs(M=4, K=1024, N=512, group_size=128, act_dtype="bf16", seed=31)
    qw, sc, zr = _t(d["qweight"]), _t(d["scales"], torch.bfloat16), qf.pack_zeros_u4(_t(d["zeros"]))
    x_host = torch.from_numpy(d["x"]).to(torch.bfloat16).pin_memory()
    want = qf.w4a16_linear(x_host.cuda(), qw, sc, zr, out_dtype=torch.float32).cpu()
    for lin in (qf.W4A16Linear(qw, sc, zr), qf.W4A16Linear(qf.prepack_w4(qw), sc, zr, weight_layout=1)):
        out = torch.empty(4, 512, dtype=torch.float32).pin_memory()
        for wait in (True, False, False):
            out.zero_()
            lin.forward_host(x_host, out, wait=wait)
            torch.cuda.synchronize()
            assert O.rel_err(out.numpy(), want.numpy()) < 1e-5
    with pytest.raises(ValueError):
        lin.forward_host(x_host, torch.empty(3, 512, dtype=torch.float32))


def test_error_behaviour(qf):
    from quantforge_b200 import QuantForgeError
    x = torch.zeros(1, 256, dtype=torch.float16, device="cuda")
    qw = torch.zeros(32, 128, dtype=torch.int8, device="cuda")
    s = torch.ones(2, 32, dtype=torch.float16, device="cuda")
    y = qf.w4a16_linear(x, qw, s)
    assert torch.all(y == 0)
    with pytest.raises(QuantForgeError) as e:  # N not a multiple of 16
        qf.w4a16_linear(x, qw[:24].contiguous(), s[:, :24].contiguous())
    assert e.value.status == -1
    with pytest.raises(QuantForgeError) as e:  # unsupported group size
        qf.w4a16_linear(x, qw, torch.ones(4, 32, dtype=torch.float16, device="cuda"), group_size=64)
    assert e.value.status == -2
    with pytest.raises(ValueError):
        qf.w4a16_linear(x, qw, s[:1])
    # M == 0 is a no-op
    y0 = qf.w4a16_linear(x[:0], qw, s)
    assert y0.shape == (0, 32)


def test_kernels_were_launched(qf):
    before = qf.launch_count()
    qf.unpack_int4(torch.zeros(4, 16, dtype=torch.int8, device="cuda"))
    assert qf.launch_count() == before + 1

"""GPU parity of the tcgen05 GEMM path (forced with path=QF_PATH_GEMM) against the CPU oracle."""
import numpy as np
import pytest
import torch

from oracle import qf_oracle as O

pytestmark = pytest.mark.gpu

GEMM = 2  # QF_PATH_GEMM
INTERLEAVED = 1
TILED = 2
_TD = {"f16": torch.float16, "bf16": torch.bfloat16, "f32": torch.float32}


@pytest.fixture(scope="module")
def qf():
    assert torch.cuda.is_available()
    import quantforge_b200 as qf
    return qf


def _t(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a))
    if dtype is not None:
        t = t.to(dtype)
    return t.cuda()


def _run(qf, M, K, N, g=128, act="bf16", zero_kind="u4", out="f32", seed=0, split_k=0, interleaved=False, sigma=0.02):
    d = O.make_inputs(M=M, K=K, N=N, group_size=g, act_dtype=act, seed=seed, sigma=sigma)
    if zero_kind == "u4":
        z_np, z_t, zc = d["zeros"], qf.pack_zeros_u4(_t(d["zeros"])), 0
    elif zero_kind == "i8":
        z_np = (d["zeros"].astype(np.int32) - 8).astype(np.int8)
        z_t, zc = _t(z_np), 0
    else:
        z_np, z_t, zc = 8, None, 8
    want = O.w4a16_linear(d["x"], d["qweight"], d["scales"], z_np, g, act, O.F32, accumulate="f64")
    qw = _t(d["qweight"])
    if interleaved == "tiled":
        qw = qf.prepack_w4(qw, layout=TILED)
    elif interleaved:
        qw = qf.prepack_w4(qw)
    y = qf.w4a16_linear(_t(d["x"], _TD[act]), qw, _t(d["scales"], _TD[act]), z_t, group_size=g, zero_const=zc,
                        out_dtype=_TD[out], path=GEMM, split_k=split_k,
                        weight_layout=TILED if interleaved == "tiled" else INTERLEAVED if interleaved else 0)
    assert qf.device_status() == 0, "a bounded device wait expired"
    return y.float().cpu().numpy(), want


def test_prepack_is_a_permutation_and_round_trips(qf):
    rng = np.random.default_rng(0)
    packed = rng.integers(-128, 128, size=(128, 64), dtype=np.int8)
    qw = _t(packed)
    inter = qf.prepack_w4(qw)
    back = qf.prepack_w4(inter, to_canonical=True)
    assert torch.equal(back, qw)
    codes = O.unpack_int4(packed).reshape(128, -1, 8)
    codes_i = O.unpack_int4(inter.cpu().numpy()).reshape(128, -1, 8)
    assert np.array_equal(codes_i, codes[:, :, [0, 2, 4, 6, 1, 3, 5, 7]])


def test_tiled_prepack_round_trips(qf):
    rng = np.random.default_rng(1)
    packed = rng.integers(-128, 128, size=(256, 192), dtype=np.int8)  # N=256, K=384
    qw = _t(packed)
    tiled = qf.prepack_w4(qw, layout=TILED)
    assert tiled.shape == qw.shape and not torch.equal(tiled, qw)
    assert torch.equal(qf.prepack_w4(tiled, to_canonical=True, layout=TILED), qw)
    # same multiset of codes: a permutation
    assert np.array_equal(np.sort(O.unpack_int4(tiled.cpu().numpy()).ravel()), np.sort(O.unpack_int4(packed).ravel()))


@pytest.mark.parametrize("M", [16, 1, 9, 17, 32, 33, 64, 100, 128, 200, 256, 300])
@pytest.mark.parametrize("layout", [False, "tiled"])
def test_gemm_batch_tiles(qf, M, layout):
    got, want = _run(qf, M, 512, 256, seed=M, interleaved=layout)
    assert O.rel_err(got, want) < 2e-4


@pytest.mark.parametrize("act", ["f16", "bf16"])
@pytest.mark.parametrize("zero_kind", ["u4", "const", "i8"])
@pytest.mark.parametrize("interleaved", [False, True, "tiled"])
def test_gemm_dtypes_zero_modes_layouts(qf, act, zero_kind, interleaved):
    got, want = _run(qf, 24, 1024, 128, act=act, zero_kind=zero_kind, interleaved=interleaved, seed=3)
    assert O.rel_err(got, want) < 2e-4


@pytest.mark.parametrize("split_k", [1, 2, 3, 8])
@pytest.mark.parametrize("M", [16, 64, 272])
def test_gemm_split_k(qf, split_k, M):
    got, want = _run(qf, M, 2048, 256, split_k=split_k, seed=split_k)
    assert O.rel_err(got, want) < 2e-4


@pytest.mark.parametrize("g", [128, 256, 1024])
def test_gemm_group_sizes(qf, g):
    got, want = _run(qf, 40, 1024, 128, g=g, act="f16", seed=g)
    assert O.rel_err(got, want) < 2e-4


@pytest.mark.parametrize("out", ["f16", "bf16", "f32"])
def test_gemm_output_dtypes(qf, out):
    got, want = _run(qf, 48, 1024, 256, out=out, seed=12)
    bound = {"f32": 2e-4, "f16": 3e-3, "bf16": 2e-2}[out]
    assert O.rel_err(got, want) < bound
    assert np.array_equal(got, O.round_to(got, out))


@pytest.mark.parametrize("M", [16, 64])
@pytest.mark.parametrize("KN", [(4096, 4096), (4096, 14336), (14336, 4096)])
def test_gemm_config1_shapes(qf, M, KN):
    K, N = KN
    got, want = _run(qf, M, K, N, seed=2, interleaved="tiled")
    assert O.rel_err(got, want) < 1e-2


def test_gemm_prefill_slice_symmetric(qf):
    """M=512 rows of the prefill configuration's kind (symmetric zero 8, sigma 0.01, bf16) on a K=8192 slice."""
    got, want = _run(qf, 512, 8192, 512, zero_kind="const", sigma=0.01, seed=5, interleaved="tiled")
    assert O.rel_err(got, want) < 1e-2


def test_gemm_deterministic(qf):
    d = O.make_inputs(M=48, K=4096, N=256, group_size=128, act_dtype="bf16", seed=3)
    args = (_t(d["x"], torch.bfloat16), _t(d["qweight"]), _t(d["scales"], torch.bfloat16),
            qf.pack_zeros_u4(_t(d["zeros"])))
    ys = [qf.w4a16_linear(*args, out_dtype=torch.float32, path=GEMM).clone() for _ in range(3)]
    assert torch.equal(ys[0], ys[1]) and torch.equal(ys[0], ys[2])


def test_gemm_rejects_bad_n(qf):
    from quantforge_b200 import QuantForgeError
    x = torch.zeros(16, 256, dtype=torch.float16, device="cuda")
    qw = torch.zeros(64, 128, dtype=torch.int8, device="cuda")
    s = torch.ones(2, 64, dtype=torch.float16, device="cuda")
    with pytest.raises(QuantForgeError) as e:
        qf.w4a16_linear(x, qw, s, path=GEMM)
    assert e.value.status == -1
    # AUTO falls back to the GEMV kernel for such N
    assert torch.all(qf.w4a16_linear(x, qw, s) == 0)


def _device_inputs(qf, M, K, N, sym, sigma, seed, dtype=torch.bfloat16):
    """Inputs of a benchmark-size layer generated on the device (a CPU generator would take minutes)."""
    gen = torch.Generator(device="cuda")
    gen.manual_seed(seed)
    G = K // 128
    qw = torch.randint(-128, 128, (N, K // 2), dtype=torch.int8, device="cuda", generator=gen)
    sc = (torch.randn(G, N, device="cuda", generator=gen).abs() * (sigma / 7.0)).clamp_min(2.0 ** -14).to(dtype)
    zeros = None if sym else torch.randint(0, 16, (G, N), dtype=torch.int8, device="cuda", generator=gen)
    x = torch.randn(M, K, device="cuda", generator=gen).to(dtype)
    return qw, sc, zeros, x


def test_prefill_full_size_sampled_columns_vs_oracle(qf):
    """The prefill configuration at its full size (M=2048, K=8192, N=28672, symmetric, bf16): 48 output columns
    spread over the matrix are recomputed by the CPU oracle from the same device-generated inputs."""
    M, K, N = 2048, 8192, 28672
    qw, sc, _, x = _device_inputs(qf, M, K, N, sym=True, sigma=0.01, seed=11)
    y = qf.w4a16_linear(x, qf.prepack_w4(qw), sc, None, group_size=128, zero_const=8, out_dtype=torch.float32,
                        weight_layout=INTERLEAVED)
    assert qf.device_status() == 0
    cols = torch.linspace(0, N - 1, 48).long().cuda()
    want = O.w4a16_linear(x.float().cpu().numpy(), qw[cols].cpu().numpy(), sc[:, cols].float().cpu().numpy(), 8, 128,
                          "bf16", O.F32, accumulate="f64")
    assert O.rel_err(y[:, cols].cpu().numpy(), want) < 1e-2


@pytest.mark.parametrize("K,N", [(28672, 8192), (8192, 10240)])
def test_large_decode_linears_both_kernels_agree(qf, K, N):
    """Llama-3-70B-shaped linears at M=1 and 2: AUTO sends them to the tcgen05 kernel; the GEMV kernel must give
    the same result up to accumulation order, and 32 sampled columns must match the oracle."""
    for M in (1, 2):
        qw, sc, zeros, x = _device_inputs(qf, M, K, N, sym=False, sigma=0.02, seed=K + M)
        zp = qf.pack_zeros_u4(zeros)
        y_auto = qf.w4a16_linear(x, qf.prepack_w4(qw), sc, zp, out_dtype=torch.float32, weight_layout=INTERLEAVED)
        y_canon = qf.w4a16_linear(x, qw, sc, zp, out_dtype=torch.float32)                    # AUTO, canonical weights
        y_gemv = qf.w4a16_linear(x, qw, sc, zp, out_dtype=torch.float32, path=qf.QF_PATH_GEMV)
        assert qf.device_status() == 0
        rms = y_gemv.pow(2).mean().sqrt()
        assert ((y_auto - y_gemv).abs().max() / rms).item() < 1e-4
        assert ((y_canon - y_gemv).abs().max() / rms).item() < 1e-4
        cols = torch.linspace(0, N - 1, 32).long().cuda()
        want = O.w4a16_linear(x.float().cpu().numpy(), qw[cols].cpu().numpy(), sc[:, cols].float().cpu().numpy(),
                              zeros[:, cols].cpu().numpy(), 128, "bf16", O.F32, accumulate="f64")
        assert O.rel_err(y_auto[:, cols].cpu().numpy(), want) < 1e-2

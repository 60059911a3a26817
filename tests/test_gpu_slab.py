"""The streaming GEMV kernel on QF_LAYOUT_GEMV_SLAB weights (qf_prepack_gemv_slab + qf_w4a16_linear_fused)
against the CPU oracle: prepack permutation bit for bit, linear results within the parity tolerance, every way a
row block can be shared between thread blocks, CUDA-graph replays (the workspace cleans itself), fused epilogues.
"""
import numpy as np
import pytest
import torch

from oracle import qf_oracle as O

pytestmark = pytest.mark.gpu
TOL = 1e-2  # max |y - y_ref| / rms(y_ref), the tolerance the path is specified with; observed values are ~1e-5


def _t(a, dev, dt=None):
    t = torch.from_numpy(np.ascontiguousarray(a))
    return (t.to(dt) if dt else t).to(dev)


def _case(M, K, N, act, group=128, zmode="u4", seed=0):
    import quantforge_b200 as qf
    dev = torch.device("cuda:0")
    tdt = torch.float16 if act == "f16" else torch.bfloat16
    d = O.make_inputs(M=M, K=K, N=N, group_size=group, act_dtype=act, seed=seed, symmetric=zmode.startswith("const"))
    zeros_np, zeros_t, zc = d["zeros"], None, 8
    if zmode == "u4":
        zeros_t = qf.pack_zeros_u4(_t(d["zeros"], dev))
    elif zmode == "i8":
        zeros_np = (d["zeros"].astype(np.int16) * 17 - 128).astype(np.int8)  # signed zero points, -128..127
        zeros_t = _t(zeros_np, dev)
    elif zmode == "const0":
        zeros_np, zc = 0, 0
    else:
        zeros_np = 8
    x = _t(d["x"], dev, tdt)
    qw = _t(d["qweight"], dev)
    sc = _t(d["scales"], dev, tdt)
    slab = qf.prepack_gemv_slab(qw, sc, zeros_t, group_size=group, zero_const=zc)
    return d, zeros_np, x, qw, sc, zeros_t, slab


def test_prepack_is_a_permutation_of_the_codes():
    import quantforge_b200 as qf
    for (K, N) in [(128, 64), (1024, 192), (4096, 256)]:
        d, _z, _x, qw, _sc, _zt, slab = _case(1, K, N, "bf16", seed=K + N)
        assert slab.blob.numel() == (N // 64) * (K // 128) * 4352
        back = qf.unpack_gemv_slab(slab)
        assert torch.equal(back, qw)
        assert np.array_equal(O.unpack_int4(back.cpu().numpy()), d["codes"])


@pytest.mark.parametrize("M,K,N,act,group,zmode,grid", [
    (1, 4096, 4096, "f16", 128, "u4", 0),        # the headline GEMV case
    (1, 128, 64, "bf16", 128, "u4", 0),          # one unit, one thread block
    (1, 1024, 64, "bf16", 128, "u4", 3),         # one row block shared by three thread blocks
    (1, 1024, 64, "bf16", 128, "u4", 8),         # one unit per thread block
    (2, 1024, 192, "f16", 128, "i8", 5),
    (3, 512, 192, "bf16", 128, "const8", 7),
    (4, 2048, 256, "bf16", 256, "u4", 0),
    (5, 4096, 14336, "bf16", 128, "u4", 0),
    (8, 2048, 1024, "f16", 2048, "i8", 0),       # per-channel (group == K), signed zero points
    (8, 4096, 1024, "bf16", 128, "const0", 0),   # the zp == 0 fast path
    (1, 14336, 4096, "bf16", 128, "u4", 0),
    (1, 14336, 4096, "bf16", 128, "u4", 1000),   # more thread blocks than fit at once: owners wait for earlier blocks only
    (9, 1024, 512, "bf16", 128, "u4", 0),        # two batch tiles
    (16, 2048, 512, "f16", 128, "u4", 11),
    (17, 1024, 256, "bf16", 128, "i8", 0),       # four batch tiles, ragged
    (32, 4096, 256, "bf16", 128, "u4", 0),
    (1, 8192, 1280, "bf16", 128, "u4", 0),       # a tensor-parallel shard of a 70B q/k/v projection
    (3, 128, 512, "bf16", 128, "u4", 0),         # one K chunk per row block: every pair of units spans two row blocks
    (1, 128, 512, "f16", 128, "i8", 3),          # the same with ranges of 3, 3 and 2 units (an odd tail)
    (2, 384, 192, "f16", 128, "u4", 2),          # three chunks per row block: pairs straddle a row block every time
    (1, 640, 320, "bf16", 128, "u4", 7),         # 25 units over 7 thread blocks: odd and even ranges, odd chunk count
])
def test_slab_linear_matches_oracle(M, K, N, act, group, zmode, grid):
    import quantforge_b200 as qf
    d, zeros_np, x, _qw, _sc, _zt, slab = _case(M, K, N, act, group, zmode, seed=M + K + N)
    want = O.w4a16_linear(d["x"], d["qweight"], d["scales"], zeros_np, group, act, O.F32, accumulate="f64")
    y = qf.w4a16_linear(x, slab, out_dtype=torch.float32, split_k=grid)
    y2 = qf.w4a16_linear(x, slab, out_dtype=torch.float32, split_k=grid)
    torch.cuda.synchronize()
    assert qf.device_status() == 0
    assert O.rel_err(y.cpu().numpy(), want) < TOL
    assert O.rel_err(y.cpu().numpy(), want) < 1e-4  # same per-weight rounding as the oracle: only the summation order differs
    assert torch.equal(y, y2)  # deterministic, and the first call left the workspace clean
    # output in the activation type: one rounding of the same accumulators
    tdt = torch.float16 if act == "f16" else torch.bfloat16
    y16 = qf.w4a16_linear(x, slab, split_k=grid)
    assert torch.equal(y16, y.to(tdt))


@pytest.mark.parametrize("M,grid", [(1, 700), (1, 1000), (1, 0), (8, 900)])
def test_slab_repeated_launches_are_bit_identical(M, grid):
    """Thread blocks that start late (more blocks than fit on the GPU at once) get their refills within a few hundred
    nanoseconds; a stage released before its last read then shows as a few rows that differ in some launches. The
    sums are taken in a fixed order, so every launch must reproduce the first one bit for bit."""
    import quantforge_b200 as qf
    K, N = 14336, 4096
    d, zeros_np, x, _qw, _sc, _zt, slab = _case(M, K, N, "bf16", seed=grid + M)
    want = O.w4a16_linear(d["x"], d["qweight"], d["scales"], zeros_np, 128, "bf16", O.F32, accumulate="f64")
    first = qf.w4a16_linear(x, slab, out_dtype=torch.float32, split_k=grid).clone()
    assert np.abs(first.cpu().numpy() - want).max() / np.sqrt(np.mean(want ** 2)) < TOL
    outs = [torch.empty_like(first) for _ in range(8)]
    for _ in range(30):
        for o in outs:
            qf.w4a16_linear(x, slab, out_dtype=torch.float32, split_k=grid, out=o)
        torch.cuda.synchronize()
        for o in outs:
            assert torch.equal(o, first)
    assert qf.device_status() == 0


def test_slab_guard_rows_are_not_written():
    import quantforge_b200 as qf
    M, K, N = 3, 1024, 192
    d, zeros_np, x, _qw, _sc, _zt, slab = _case(M, K, N, "bf16", seed=5)
    buf = torch.full((M + 2, N), 7.0, dtype=torch.float32, device=x.device)
    qf.w4a16_linear(x, slab, out_dtype=torch.float32, out=buf[1:M + 1], split_k=5)
    torch.cuda.synchronize()
    assert torch.all(buf[0] == 7.0) and torch.all(buf[M + 1] == 7.0)
    want = O.w4a16_linear(d["x"], d["qweight"], d["scales"], zeros_np, 128, "bf16", O.F32, accumulate="f64")
    assert O.rel_err(buf[1:M + 1].cpu().numpy(), want) < 1e-4


def test_slab_in_cuda_graph_mixed_shapes_share_the_workspace():
    import quantforge_b200 as qf
    a = _case(1, 2048, 1024, "bf16", seed=1)
    b = _case(4, 1024, 192, "bf16", seed=2)
    outs = []
    for (d, zeros_np, x, _qw, _sc, _zt, slab), grid in ((a, 37), (b, 9)):
        want = O.w4a16_linear(d["x"], d["qweight"], d["scales"], zeros_np, 128, "bf16", O.F32, accumulate="f64")
        out = torch.empty(x.shape[0], slab.N, dtype=torch.float32, device=x.device)
        outs.append((x, slab, grid, out, want))
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        for (x, slab, grid, out, _w) in outs:
            qf.w4a16_linear(x, slab, out_dtype=torch.float32, out=out, split_k=grid)
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for _ in range(3):
            for (x, slab, grid, out, _w) in outs:
                qf.w4a16_linear(x, slab, out_dtype=torch.float32, out=out, split_k=grid)
    for _ in range(3):
        for (_x, _s, _g, out, _w) in outs:
            out.zero_()
        g.replay()
        torch.cuda.synchronize()
        for (_x, _s, _g, out, want) in outs:
            assert O.rel_err(out.cpu().numpy(), want) < 1e-4
    assert qf.device_status() == 0


def _gate_up_case(M, K, F, act, seed):
    """gate and up projections [F, K] each, interleaved in groups of 8 rows as QF_EPI_SILU_MUL expects."""
    dg = O.make_inputs(M=M, K=K, N=F, group_size=128, act_dtype=act, seed=seed)
    du = O.make_inputs(M=M, K=K, N=F, group_size=128, act_dtype=act, seed=seed + 1)
    qweight = O.interleave8(dg["qweight"], du["qweight"], 0)
    scales = O.interleave8(dg["scales"], du["scales"], 1)
    zeros = O.interleave8(dg["zeros"], du["zeros"], 1)
    y_gate = O.w4a16_linear(dg["x"], dg["qweight"], dg["scales"], dg["zeros"], 128, act, O.F32, accumulate="f64")
    y_up = O.w4a16_linear(dg["x"], du["qweight"], du["scales"], du["zeros"], 128, act, O.F32, accumulate="f64")
    return dg["x"], qweight, scales, zeros, O.silu_mul(y_gate, y_up)


@pytest.mark.parametrize("M,K,F,act,grid", [(1, 1024, 256, "bf16", 0), (3, 2048, 512, "f16", 13), (8, 1024, 1024, "bf16", 0),
                                            (20, 1024, 256, "bf16", 6)])
def test_slab_silu_mul_epilogue(M, K, F, act, grid):
    import quantforge_b200 as qf
    dev = torch.device("cuda:0")
    tdt = torch.float16 if act == "f16" else torch.bfloat16
    x_np, qweight, scales, zeros, want = _gate_up_case(M, K, F, act, seed=M + F)
    slab = qf.prepack_gemv_slab(_t(qweight, dev), _t(scales, dev, tdt), qf.pack_zeros_u4(_t(zeros, dev)))
    y = qf.w4a16_linear(_t(x_np, dev, tdt), slab, out_dtype=torch.float32, epilogue=qf.QF_EPI_SILU_MUL, split_k=grid)
    torch.cuda.synchronize()
    assert tuple(y.shape) == (M, F)
    assert O.rel_err(y.cpu().numpy(), want) < 1e-4


@pytest.mark.parametrize("M,K,N,out_dt,grid", [(1, 1024, 256, torch.float32, 0), (4, 2048, 512, torch.bfloat16, 9),
                                               (12, 1024, 192, torch.float32, 0)])
def test_slab_residual_epilogue(M, K, N, out_dt, grid):
    import quantforge_b200 as qf
    d, zeros_np, x, _qw, _sc, _zt, slab = _case(M, K, N, "bf16", seed=N)
    lin = O.w4a16_linear(d["x"], d["qweight"], d["scales"], zeros_np, 128, "bf16", O.F32, accumulate="f64")
    res_np = O.round_to(np.random.default_rng(3).normal(size=(M, N)).astype(np.float32), "bf16")
    res = _t(res_np, x.device, out_dt)
    y = res.clone()  # in place: the residual aliases the output
    qf.w4a16_linear(x, slab, out_dtype=out_dt, out=y, epilogue=qf.QF_EPI_RESIDUAL_ADD, residual=y)
    torch.cuda.synchronize()
    want = lin + res_np
    if out_dt == torch.float32:
        assert O.rel_err(y.cpu().numpy(), want) < 1e-4
    else:
        assert torch.equal(y, torch.from_numpy(O.round_to(want, "bf16")).to(torch.bfloat16).to(y.device)) or \
            O.rel_err(y.float().cpu().numpy(), want) < 2e-2  # one bf16 ulp of the largest outputs


@pytest.mark.parametrize("M,K,F,split_k,inter", [(16, 1024, 256, 1, False), (16, 2048, 256, 4, True), (40, 1024, 128, 2, True),
                                                 (64, 4096, 256, 12, False), (130, 1024, 128, 1, True)])
def test_tcgen05_silu_mul_epilogue(M, K, F, split_k, inter):
    """The same epilogue in the tcgen05 kernel: direct, cluster split-K and global split-K reductions."""
    import quantforge_b200 as qf
    dev = torch.device("cuda:0")
    x_np, qweight, scales, zeros, want = _gate_up_case(M, K, F, "bf16", seed=M + F)
    qw = _t(qweight, dev)
    layout = qf.QF_LAYOUT_CANONICAL
    if inter:
        qw, layout = qf.prepack_w4(qw), qf.QF_LAYOUT_INTERLEAVED
    y = qf.w4a16_linear(_t(x_np, dev, torch.bfloat16), qw, _t(scales, dev, torch.bfloat16),
                        qf.pack_zeros_u4(_t(zeros, dev)), out_dtype=torch.float32, split_k=split_k,
                        weight_layout=layout, epilogue=qf.QF_EPI_SILU_MUL)
    torch.cuda.synchronize()
    assert tuple(y.shape) == (M, F) and qf.device_status() == 0
    assert O.rel_err(y.cpu().numpy(), want) < 1e-4


@pytest.mark.parametrize("M,K,N,split_k", [(16, 1024, 256, 1), (33, 2048, 128, 4), (64, 4096, 256, 12), (200, 1024, 256, 1)])
def test_tcgen05_residual_epilogue(M, K, N, split_k):
    import quantforge_b200 as qf
    dev = torch.device("cuda:0")
    d = O.make_inputs(M=M, K=K, N=N, group_size=128, act_dtype="bf16", seed=M)
    lin = O.w4a16_linear(d["x"], d["qweight"], d["scales"], d["zeros"], 128, "bf16", O.F32, accumulate="f64")
    res_np = np.random.default_rng(4).normal(size=(M, N)).astype(np.float32)
    y = _t(res_np, dev)
    qf.w4a16_linear(_t(d["x"], dev, torch.bfloat16), _t(d["qweight"], dev), _t(d["scales"], dev, torch.bfloat16),
                    qf.pack_zeros_u4(_t(d["zeros"], dev)), out_dtype=torch.float32, out=y, split_k=split_k,
                    path=qf.QF_PATH_GEMM, epilogue=qf.QF_EPI_RESIDUAL_ADD, residual=y)
    torch.cuda.synchronize()
    assert O.rel_err(y.cpu().numpy(), lin + res_np) < 1e-4


def test_repack_kn_to_canonical_is_bit_exact():
    import quantforge_b200 as qf
    dev = torch.device("cuda:0")
    rng = np.random.default_rng(11)
    for (K, N) in [(128, 64), (1024, 48), (512, 1000)]:
        codes_kn = rng.integers(0, 16, size=(K, N), dtype=np.int8)
        want = O.repack_kn_to_canonical(codes_kn)
        got = qf.repack_kn_to_canonical(_t(codes_kn, dev), K, N)
        assert np.array_equal(got.cpu().numpy(), want)
        packed_n = O.pack_int4(codes_kn)  # two codes per byte along N, the reference tests' weight operand
        got2 = qf.repack_kn_to_canonical(_t(packed_n, dev), K, N)
        assert np.array_equal(got2.cpu().numpy(), want)
        assert np.array_equal(O.unpack_int4(got2.cpu().numpy()), codes_kn.T)


def test_slab_rejects_what_it_cannot_serve():
    import quantforge_b200 as qf
    d, _z, x, qw, sc, zt, slab = _case(1, 1024, 64, "bf16")
    big = torch.zeros(40, 1024, dtype=torch.bfloat16, device=x.device)
    with pytest.raises(qf.QuantForgeError):  # M > 32
        qf.w4a16_linear(big, slab)
    with pytest.raises(ValueError):  # N % 64 != 0
        qf.prepack_gemv_slab(qw[:48], sc[:, :48].contiguous(), None)
    with pytest.raises(qf.QuantForgeError):  # qf_dequant_w4 reads canonical weights only
        from quantforge_b200 import _lib, ops
        import ctypes
        desc = ops._make_desc(1, 64, 1024, 128, torch.bfloat16, torch.bfloat16, zt, 8, 0, 0, qf.QF_LAYOUT_INTERLEAVED)
        out = torch.empty(64, 1024, dtype=torch.bfloat16, device=x.device)
        ctx = ops._ctx(x.device)
        st = _lib.load().qf_dequant_w4(ctx, ctypes.byref(desc), ops._ptr(qw), ops._ptr(sc), ops._ptr(zt), ops._ptr(out), None)
        ops._check(st, ctx)

"""The linear kernels with the cross-GPU step in their epilogue (qf_w4a16_linear_allreduce / _allgather).

One GPU: a comm of world 1 runs the whole exchange (push, flag, wait, sum) against its own buffer, so the result
must equal the plain linear bit for bit, call after call (the slots alternate by call parity) and inside a CUDA
graph. Two GPUs: two processes, each with its K shard, against the unsharded CPU oracle and against each other.
"""
import os
import socket
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.gpu


def _t(a, dev, dt=None):
    t = torch.from_numpy(np.ascontiguousarray(a))
    return (t.to(dt) if dt else t).to(dev)


@pytest.mark.parametrize("M,K,N,act,split_k", [
    (1, 1024, 512, "f16", 0), (1, 4096, 4096, "bf16", 0), (2, 2048, 1040, "bf16", 0), (4, 1024, 256, "f16", 1),
    (8, 1024, 8192, "bf16", 1), (3, 512, 144, "bf16", 2), (1, 8192, 1024, "f16", 0),
])
def test_world1_equals_plain_linear(M, K, N, act, split_k):
    import quantforge_b200 as qf
    from oracle import qf_oracle as O
    dev = torch.device("cuda:0")
    tdt = torch.float16 if act == "f16" else torch.bfloat16
    d = O.make_inputs(M=M, K=K, N=N, group_size=128, act_dtype=act, seed=M + N)
    x, qw, sc = _t(d["x"], dev, tdt), _t(d["qweight"], dev), _t(d["scales"], dev, tdt)
    zr = qf.pack_zeros_u4(_t(d["zeros"], dev))
    comm = qf.Comm(M * N, device=dev, rank=0, world=1)
    try:
        want = qf.w4a16_linear(x, qw, sc, zr, 128, out_dtype=torch.float32, path=qf.QF_PATH_GEMV, split_k=split_k)
        for _ in range(3):  # both slot parities
            got = qf.w4a16_linear_allreduce(x, qw, sc, zr, comm, 128, out_dtype=torch.float32, split_k=split_k,
                                            path=qf.QF_PATH_GEMV)
            assert torch.equal(got, want)
        ref = O.w4a16_linear(d["x"], d["qweight"], d["scales"], d["zeros"], 128, act, O.F32, accumulate="f64")
        assert O.rel_err(got.cpu().numpy(), ref) < 1e-2
        torch.cuda.synchronize()
        assert qf.device_status(dev) == 0
    finally:
        comm.close()


def test_world1_in_cuda_graph():
    import quantforge_b200 as qf
    from oracle import qf_oracle as O
    dev = torch.device("cuda:0")
    d = O.make_inputs(M=2, K=2048, N=1024, group_size=128, act_dtype="bf16", seed=3)
    x, qw, sc = _t(d["x"], dev, torch.bfloat16), _t(d["qweight"], dev), _t(d["scales"], dev, torch.bfloat16)
    zr = qf.pack_zeros_u4(_t(d["zeros"], dev))
    comm = qf.Comm(2 * 1024, device=dev, rank=0, world=1)
    try:
        want = qf.w4a16_linear(x, qw, sc, zr, 128, path=qf.QF_PATH_GEMV)
        out = torch.empty_like(want)
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            qf.w4a16_linear_allreduce(x, qw, sc, zr, comm, 128, out=out, path=qf.QF_PATH_GEMV)
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(3):
                qf.w4a16_linear_allreduce(x, qw, sc, zr, comm, 128, out=out, path=qf.QF_PATH_GEMV)
        for _ in range(3):
            out.zero_()
            g.replay()
            torch.cuda.synchronize()
            assert torch.equal(out, want)
        assert qf.device_status(dev) == 0
    finally:
        comm.close()


@pytest.mark.parametrize("M,K,N,act,split_k,inter", [
    (16, 1024, 512, "bf16", 0, True), (64, 2048, 256, "f16", 1, False), (5, 4096, 1024, "bf16", 0, True),
    (33, 1024, 384, "bf16", 2, True),
])
@pytest.mark.parametrize("gather", [False, True])
def test_world1_tcgen05_kernel(M, K, N, act, split_k, inter, gather):
    import quantforge_b200 as qf
    from oracle import qf_oracle as O
    dev = torch.device("cuda:0")
    tdt = torch.float16 if act == "f16" else torch.bfloat16
    d = O.make_inputs(M=M, K=K, N=N, group_size=128, act_dtype=act, seed=M + N)
    x, qw, sc = _t(d["x"], dev, tdt), _t(d["qweight"], dev), _t(d["scales"], dev, tdt)
    zr = qf.pack_zeros_u4(_t(d["zeros"], dev))
    layout = qf.QF_LAYOUT_INTERLEAVED if inter else qf.QF_LAYOUT_CANONICAL
    if inter:
        qw = qf.prepack_w4(qw)
    comm = qf.Comm(M * N, device=dev, rank=0, world=1)
    fn = qf.w4a16_linear_allgather if gather else qf.w4a16_linear_allreduce
    try:
        want = qf.w4a16_linear(x, qw, sc, zr, 128, path=qf.QF_PATH_GEMM, split_k=split_k, weight_layout=layout)
        for _ in range(3):
            got = fn(x, qw, sc, zr, comm, 128, path=qf.QF_PATH_GEMM, split_k=split_k, weight_layout=layout)
            assert torch.equal(got, want)
        torch.cuda.synchronize()
        assert qf.device_status(dev) == 0
    finally:
        comm.close()


def test_rejects_what_the_kernel_cannot_do():
    import quantforge_b200 as qf
    from oracle import qf_oracle as O
    dev = torch.device("cuda:0")
    d = O.make_inputs(M=80, K=512, N=128, group_size=128, act_dtype="bf16", seed=1)
    x, qw, sc = _t(d["x"], dev, torch.bfloat16), _t(d["qweight"], dev), _t(d["scales"], dev, torch.bfloat16)
    zr = qf.pack_zeros_u4(_t(d["zeros"], dev))
    comm = qf.Comm(64, device=dev, rank=0, world=1)
    try:
        with pytest.raises(qf.QuantForgeError):   # M > 64
            qf.w4a16_linear_allreduce(x, qw, sc, zr, comm, 128)
        with pytest.raises(qf.QuantForgeError):   # M*N beyond the comm's capacity
            qf.w4a16_linear_allreduce(x[:1], qw, sc, zr, comm, 128)
    finally:
        comm.close()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    import datetime
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev,
                            timeout=datetime.timedelta(seconds=120))
    comm = None
    try:
        import quantforge_b200 as qf
        from oracle import qf_oracle as O
        from quantforge_b200 import tp
        comm = qf.Comm(16 * 4096, device=dev)
        res = []
        for (M, K, N, act, mode) in [(1, 2048, 4096, "bf16", "row"), (2, 1024, 528, "f16", "row"),
                                     (8, 4096, 1024, "bf16", "row"), (16, 2048, 512, "bf16", "row"),
                                     (64, 1024, 256, "f16", "row"), (1, 1024, 2048, "bf16", "col"),
                                     (16, 2048, 1024, "bf16", "col"), (4, 512, 96, "f16", "col")]:
            tdt = torch.float16 if act == "f16" else torch.bfloat16
            d = O.make_inputs(M=M, K=K, N=N, group_size=128, act_dtype=act, seed=K + M)
            prepack = M > 2 and N % 256 == 0
            if mode == "row":
                lin = tp.RowParallelLinear(_t(d["qweight"], dev), _t(d["scales"], dev, tdt),
                                           qf.pack_zeros_u4(_t(d["zeros"], dev)), 128, input_is_parallel=False,
                                           comm=comm, prepack=prepack)
            else:
                lin = tp.ColumnParallelLinear(_t(d["qweight"], dev), _t(d["scales"], dev, tdt),
                                              qf.pack_zeros_u4(_t(d["zeros"], dev)), 128, gather_output=True,
                                              comm=comm, prepack=prepack)
            x = _t(d["x"], dev, tdt)
            want = O.w4a16_linear(d["x"], d["qweight"], d["scales"], d["zeros"], 128, act, O.F32, accumulate="f64")
            for _ in range(3):
                y = lin(x, torch.float32)
            torch.cuda.synchronize()
            err = O.rel_err(y.cpu().numpy(), want)
            # every rank must hold the same bits
            both = [torch.empty_like(y) for _ in range(world)]
            dist.all_gather(both, y)
            same = all(torch.equal(both[0], b) for b in both)
            res.append((err, same, int(qf.device_status(dev))))
        if rank == 0:
            out.put(res)
    finally:
        if comm is not None:
            comm.close()
        dist.destroy_process_group()


def test_two_gpus_row_parallel_fused_sum():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    out = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
        assert p.exitcode == 0
    for err, same, status in out.get():
        assert err < 1e-3 and same and status == 0

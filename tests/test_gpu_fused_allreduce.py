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


@pytest.mark.parametrize("M,K,N,act,grid,gather", [
    (1, 1024, 256, "bf16", 0, False), (1, 4096, 4096, "f16", 200, False), (3, 2048, 192, "bf16", 37, False),
    (8, 1024, 1024, "bf16", 100, True), (20, 1024, 256, "f16", 50, False), (1, 8192, 1024, "bf16", 296, True),
])
def test_world1_slab_kernel(M, K, N, act, grid, gather):
    """The streaming GEMV kernel with the exchange in it: pushes as tiles finish, collects at the end of each
    thread block's life. With one rank the result must equal the plain kernel on the same split, bit for bit."""
    import quantforge_b200 as qf
    from oracle import qf_oracle as O
    dev = torch.device("cuda:0")
    tdt = torch.float16 if act == "f16" else torch.bfloat16
    d = O.make_inputs(M=M, K=K, N=N, group_size=128, act_dtype=act, seed=M + N)
    x = _t(d["x"], dev, tdt)
    slab = qf.prepack_gemv_slab(_t(d["qweight"], dev), _t(d["scales"], dev, tdt), qf.pack_zeros_u4(_t(d["zeros"], dev)))
    comm = qf.Comm(M * N, device=dev, rank=0, world=1)
    fn = qf.w4a16_linear_allgather if gather else qf.w4a16_linear_allreduce
    try:
        split = grid if grid else 2 * 148  # what the exchanging call uses by default
        want = qf.w4a16_linear(x, slab, out_dtype=torch.float32, split_k=split)
        for _ in range(3):  # both slot parities
            got = fn(x, slab, None, None, comm, out_dtype=torch.float32, split_k=grid)
            assert torch.equal(got, want)
        ref = O.w4a16_linear(d["x"], d["qweight"], d["scales"], d["zeros"], 128, act, O.F32, accumulate="f64")
        assert O.rel_err(got.cpu().numpy(), ref) < 1e-4
        assert qf.device_status(dev) == 0
    finally:
        comm.close()


@pytest.mark.parametrize("kind", ["slab", "gemv", "gemm"])
def test_wait_for_a_peer_runs_out_and_is_reported(kind):
    """A rank whose peer never makes the call: the collect's wait is bounded, so the kernel returns, the context
    reports QF_ERR_TIMEOUT, and after the comm is destroyed and the workspace zeroed again the GPU computes
    correctly. One process plays both ranks of a world-2 comm on one GPU, and only rank 0 ever launches (nothing
    waits on a kernel that is not running, nothing faults). The wait is shortened to 20 ms for the test."""
    import ctypes
    import quantforge_b200 as qf
    from oracle import qf_oracle as O
    from quantforge_b200 import _lib, ops
    lib = _lib.load()
    dev = torch.device("cuda:0")
    ctx = ops._ctx(dev)
    M, K, N = (16, 1024, 256) if kind == "gemm" else (2, 1024, 256)
    d = O.make_inputs(M=M, K=K, N=N, group_size=128, act_dtype="bf16", seed=9)
    x = _t(d["x"], dev, torch.bfloat16)
    qw, sc = _t(d["qweight"], dev), _t(d["scales"], dev, torch.bfloat16)
    zr = qf.pack_zeros_u4(_t(d["zeros"], dev))
    slab = qf.prepack_gemv_slab(qw, sc, zr)
    torch.cuda.synchronize()
    os.environ["QF_EXCHANGE_WAIT_MS"] = "20"
    comms = [ctypes.c_void_p(), ctypes.c_void_p()]
    try:
        for r in range(2):
            assert lib.qf_comm_create(ctx, r, 2, M * N, ctypes.byref(comms[r])) == 0, lib.qf_last_error(ctx)
    finally:
        del os.environ["QF_EXCHANGE_WAIT_MS"]
    try:
        handles = b""
        for r in range(2):
            buf = ctypes.create_string_buffer(_lib.QF_COMM_HANDLE_BYTES)
            assert lib.qf_comm_export(comms[r], buf) == 0
            handles += bytes(buf.raw)
        for r in range(2):
            assert lib.qf_comm_connect(comms[r], handles, 2) == 0, lib.qf_last_error(ctx)

        class _C:  # the Python wrapper only needs the handle and the world size
            _h, world = comms[0], 2
        assert qf.device_status(dev) == 0
        if kind == "slab":
            y = qf.w4a16_linear_allreduce(x, slab, None, None, _C, out_dtype=torch.float32)
        else:
            y = qf.w4a16_linear_allreduce(x, qw, sc, zr, _C, 128, out_dtype=torch.float32,
                                          path=qf.QF_PATH_GEMV if kind == "gemv" else qf.QF_PATH_GEMM)
        torch.cuda.synchronize()  # returns: the wait ran out after about 20 ms
        assert qf.device_status(dev) == -5  # QF_ERR_TIMEOUT
        del y
    finally:
        qf.clear_device_status(dev)
        for c in comms:
            if c:
                lib.qf_comm_destroy(c)
        for bufs in ops._workspaces.values():  # a call that gave up may leave split-K state behind: zero it again
            for ws in bufs:
                ws.zero_()
    want = O.w4a16_linear(d["x"], d["qweight"], d["scales"], d["zeros"], 128, "bf16", O.F32, accumulate="f64")
    got = qf.w4a16_linear(x, slab, out_dtype=torch.float32) if kind == "slab" else \
        qf.w4a16_linear(x, qw, sc, zr, 128, out_dtype=torch.float32)
    assert O.rel_err(got.cpu().numpy(), want) < 1e-4
    assert qf.device_status(dev) == 0


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
        # The ranks of this test are separate Python processes that prepare every case on the host (inputs, the CPU
        # oracle) before they launch; with eight of them sharing the host cores they drift apart by more than the
        # default limit of a wait for a peer (about a second). A longer limit and a barrier before each case keep a
        # slow host from reading as a lost peer; the time-out path has its own test.
        os.environ["QF_EXCHANGE_WAIT_MS"] = "10000"
        comm = qf.Comm(64 * 4096, device=dev)
        res = []
        # every shape shards for 2, 4 and 8 ranks (K/world a multiple of 128, N/world of 16; of 64 where slab is set)
        for (M, K, N, act, mode, slab) in [
                (1, 2048, 4096, "bf16", "row", False), (2, 1024, 528, "f16", "row", False),
                (8, 4096, 1024, "bf16", "row", False), (16, 2048, 512, "bf16", "row", False),
                (64, 1024, 256, "f16", "row", False), (1, 1024, 2048, "bf16", "col", False),
                (16, 2048, 1024, "bf16", "col", False), (4, 1024, 384, "f16", "col", False),
                (1, 8192, 1024, "bf16", "row", True), (8, 2048, 4096, "bf16", "row", True),
                (24, 1024, 512, "f16", "row", True), (1, 1024, 4096, "bf16", "col", True),
                (5, 2048, 1024, "f16", "col", True)]:
            tdt = torch.float16 if act == "f16" else torch.bfloat16
            d = O.make_inputs(M=M, K=K, N=N, group_size=128, act_dtype=act, seed=K + M)
            prepack = M > 2 and N % (128 * world) == 0
            if mode == "row":
                lin = tp.RowParallelLinear(_t(d["qweight"], dev), _t(d["scales"], dev, tdt),
                                           qf.pack_zeros_u4(_t(d["zeros"], dev)), 128, input_is_parallel=False,
                                           comm=comm, prepack=prepack, slab=slab)
            else:
                lin = tp.ColumnParallelLinear(_t(d["qweight"], dev), _t(d["scales"], dev, tdt),
                                              qf.pack_zeros_u4(_t(d["zeros"], dev)), 128, gather_output=True,
                                              comm=comm, prepack=prepack, slab=slab)
            x = _t(d["x"], dev, tdt)
            want = O.w4a16_linear(d["x"], d["qweight"], d["scales"], d["zeros"], 128, act, O.F32, accumulate="f64")
            torch.cuda.synchronize()
            dist.barrier()
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


@pytest.mark.parametrize("world", [2, 4, 8])
def test_ranks_exchange_inside_the_kernels(world):
    """One process per GPU: row-parallel sums and column-parallel gathers inside all three kernel families, against
    the unsharded CPU oracle and rank against rank (same bits everywhere)."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    out = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, out)) for r in range(world)]
    for p in procs:
        p.start()
    import time
    deadline = time.time() + 300  # one deadline for all ranks together
    codes = []
    for p in procs:
        p.join(max(1.0, deadline - time.time()))
        if p.is_alive():  # never leave a straggler behind on a shared GPU
            p.terminate()
            p.join(30)
        codes.append(p.exitcode)
    assert codes == [0] * world
    for err, same, status in out.get():
        assert err < 1e-3 and same and status == 0

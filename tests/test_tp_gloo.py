"""Column-/row-parallel sharding on 2 CPU ranks (gloo). The per-rank compute is the CPU oracle, injected in
place of the CUDA operator, so this checks the shard indexing and the exchange step only."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _oracle_compute(x, qweight, scales, zeros, group_size, zero_const, out_dtype):
    from oracle import qf_oracle as O
    z = zero_const if zeros is None else (O.unpack_words(zeros.numpy().view(np.uint32)) if zeros.dtype == torch.int32
                                          else zeros.numpy())
    y = O.w4a16_linear(x.float().numpy(), qweight.numpy(), scales.float().numpy(), z, group_size, "f16", O.F32,
                       accumulate="f64")
    return torch.from_numpy(y).to(out_dtype or torch.float32)


def _worker(rank, world, port, zero_kind, out):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import qf_oracle as O
        from quantforge_b200 import tp
        from quantforge_b200.ops import pack_zeros_u4
        M, K, N, g = 3, 512, 64, 128
        d = O.make_inputs(M=M, K=K, N=N, group_size=g, act_dtype="f16", seed=7)
        qw = torch.from_numpy(d["qweight"])
        sc = torch.from_numpy(d["scales"]).half()
        x = torch.from_numpy(d["x"]).half()
        if zero_kind == "u4":
            zeros, z_np = pack_zeros_u4(torch.from_numpy(d["zeros"])), d["zeros"]
        elif zero_kind == "i8":
            zeros, z_np = torch.from_numpy(d["zeros"]), d["zeros"]
        else:
            zeros, z_np = None, 8
        want = O.w4a16_linear(d["x"], d["qweight"], d["scales"], z_np, g, "f16", O.F32, accumulate="f64")

        col = tp.ColumnParallelLinear(qw, sc, zeros, g, compute=_oracle_compute)
        y_col = col(x, torch.float32)
        assert y_col.shape == (M, N)
        err_col = O.rel_err(y_col.numpy(), want)

        row = tp.RowParallelLinear(qw, sc, zeros, g, input_is_parallel=False, compute=_oracle_compute)
        y_row = row(x, torch.float32)
        err_row = O.rel_err(y_row.numpy(), want)

        # column-parallel (no gather) feeding row-parallel, the transformer MLP pattern: K2 = N of the first
        d2 = O.make_inputs(M=M, K=256, N=32, group_size=128, act_dtype="f16", seed=9)
        qw2, sc2 = torch.from_numpy(d2["qweight"]), torch.from_numpy(d2["scales"]).half()
        z2 = pack_zeros_u4(torch.from_numpy(d2["zeros"]))
        d1 = O.make_inputs(M=M, K=512, N=256, group_size=128, act_dtype="f16", seed=8)
        qw1, sc1 = torch.from_numpy(d1["qweight"]), torch.from_numpy(d1["scales"]).half()
        z1 = pack_zeros_u4(torch.from_numpy(d1["zeros"]))
        up = tp.ColumnParallelLinear(qw1, sc1, z1, 128, gather_output=False, compute=_oracle_compute)
        down = tp.RowParallelLinear(qw2, sc2, z2, 128, input_is_parallel=True, compute=_oracle_compute)
        h_local = up(x, torch.float16)
        assert h_local.shape == (M, 256 // world)
        y2 = down(h_local, torch.float32)
        h_full = O.w4a16_linear(d["x"], d1["qweight"], d1["scales"], d1["zeros"], 128, "f16", O.F16, accumulate="f64")
        want2 = O.w4a16_linear(h_full, d2["qweight"], d2["scales"], d2["zeros"], 128, "f16", O.F32, accumulate="f64")
        err_mlp = O.rel_err(y2.numpy(), want2)
        if rank == 0:
            out.put((err_col, err_row, err_mlp))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("zero_kind", ["u4", "i8", "const"])
def test_column_and_row_parallel_match_the_unsharded_oracle(zero_kind):
    ctx = mp.get_context("spawn")
    out = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, zero_kind, out)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    err_col, err_row, err_mlp = out.get()
    assert err_col < 1e-6          # gathering shards of the same computation
    assert err_row < 1e-5          # fp32 sum of two partials
    assert err_mlp < 2e-3          # f16 intermediate


def test_shard_shape_rules():
    from quantforge_b200 import tp
    with pytest.raises(ValueError):
        tp.check_shardable(4096, 4096, 128, 3, "column")
    with pytest.raises(ValueError):
        tp.check_shardable(4096, 4096 + 128, 128, 8, "row")
    tp.check_shardable(28672, 8192, 128, 8, "column")
    tp.check_shardable(8192, 28672, 128, 8, "row")
    qw = torch.zeros(64, 128, dtype=torch.int8)
    sc = torch.zeros(2, 64, dtype=torch.float16)
    z = torch.zeros(2, 8, dtype=torch.int32)
    a, b, c = tp.shard_column(qw, sc, z, 1, 2)
    assert a.shape == (32, 128) and b.shape == (2, 32) and c.shape == (2, 4)
    a, b, c = tp.shard_row(qw, sc, z, 1, 2)
    assert a.shape == (64, 64) and b.shape == (1, 64) and c.shape == (1, 8)


def test_every_shard_starts_on_a_16_byte_boundary():
    """The kernels refuse device pointers that are not 16-byte aligned. A row-parallel shard is a slice of whole rows
    of the scales / zero-point tables; with N = 528 a row of packed zero points is 264 bytes, so a view of the parent
    would start off the boundary on every odd rank of eight."""
    from quantforge_b200 import tp
    N, K, g = 528, 1024, 128
    qweight = torch.zeros(N, K // 2, dtype=torch.int8)
    scales = torch.zeros(K // g, N, dtype=torch.float16)
    zeros = torch.zeros(K // g, N // 8, dtype=torch.int32)
    for world in (2, 4, 8):
        for rank in range(world):
            for t in tp.shard_row(qweight, scales, zeros, rank, world):
                assert t.data_ptr() % 16 == 0 and t.is_contiguous()
    qweight = torch.zeros(384, K // 2, dtype=torch.int8)
    scales = torch.zeros(K // g, 384, dtype=torch.float16)
    zeros = torch.zeros(K // g, 384 // 8, dtype=torch.int32)
    for rank in range(8):
        for t in tp.shard_column(qweight, scales, zeros, rank, 8):
            assert t.data_ptr() % 16 == 0 and t.is_contiguous()

"""Tensor-parallel linears on 2 GPUs (NCCL), against the unsharded CPU oracle. Skipped on a single-GPU box."""
import os
import socket
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.gpu


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
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        import quantforge_b200 as qf
        from oracle import qf_oracle as O
        from quantforge_b200 import tp
        errs = []
        for M in (2, 24):
            d1 = O.make_inputs(M=M, K=1024, N=512, group_size=128, act_dtype="bf16", seed=8)
            d2 = O.make_inputs(M=M, K=512, N=256, group_size=128, act_dtype="bf16", seed=9)
            t = lambda a, dt=None: (torch.from_numpy(np.ascontiguousarray(a)).to(dt) if dt else
                                    torch.from_numpy(np.ascontiguousarray(a))).to(dev)
            x = t(d1["x"], torch.bfloat16)
            up = tp.ColumnParallelLinear(t(d1["qweight"]), t(d1["scales"], torch.bfloat16),
                                         qf.pack_zeros_u4(t(d1["zeros"])), 128, gather_output=False, prepack=True)
            down = tp.RowParallelLinear(t(d2["qweight"]), t(d2["scales"], torch.bfloat16),
                                        qf.pack_zeros_u4(t(d2["zeros"])), 128, input_is_parallel=True, prepack=True)
            full = tp.ColumnParallelLinear(t(d1["qweight"]), t(d1["scales"], torch.bfloat16),
                                           qf.pack_zeros_u4(t(d1["zeros"])), 128, gather_output=True)
            y_full = full(x, torch.float32)
            want_full = O.w4a16_linear(d1["x"], d1["qweight"], d1["scales"], d1["zeros"], 128, "bf16", O.F32,
                                       accumulate="f64")
            errs.append(O.rel_err(y_full.cpu().numpy(), want_full))
            h = up(x, torch.bfloat16)
            y = down(h, torch.float32)
            h_full = O.round_to(want_full, "bf16")
            want = O.w4a16_linear(h_full, d2["qweight"], d2["scales"], d2["zeros"], 128, "bf16", O.F32,
                                  accumulate="f64")
            errs.append(O.rel_err(y.cpu().numpy(), want))
        torch.cuda.synchronize()
        if rank == 0:
            out.put(errs)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_column_then_row_parallel(world):
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
        if p.is_alive():
            p.terminate()
            p.join(30)
        codes.append(p.exitcode)
    assert codes == [0] * world
    errs = out.get()
    assert errs[0] < 1e-4 and errs[2] < 1e-4          # all-gathered column-parallel output, fp32
    assert errs[1] < 1e-2 and errs[3] < 1e-2          # bf16 intermediate between the two linears

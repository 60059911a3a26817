"""The allocation-free entry point (qf_w4a16_gemv_static_scratch) against the regular one.

Some hosts of this library may not allocate device memory at all (a framework that owns the heap, a serving loop
that must never hit an implicit device synchronisation, a process whose budget is spent on weights). For them the
library carries its split-K scratch inside its own image. This test calls that entry point straight through the
C ABI, twice in a row on different inputs (the second call finds the first call's leftovers in the shared array),
and requires the same numbers as qf_w4a16_linear with a caller-provided workspace. The file name sorts last so a
failure here cannot hide the result of any other test.
"""
import ctypes

import numpy as np
import pytest
import torch

from oracle import qf_oracle as O

pytestmark = pytest.mark.gpu


def _vp(t):
    return ctypes.c_void_p(t.data_ptr() if t is not None else 0)


def _desc(_lib, M, N, K, split_k):
    d = _lib.LinearDesc()
    d.M, d.N, d.K, d.group_size = M, N, K, 128
    d.act_dtype, d.out_dtype = _lib.QF_BF16, _lib.QF_F32
    d.zero_mode = _lib.QF_ZERO_U4
    d.path = _lib.QF_PATH_GEMV
    d.split_k = split_k
    return d


def test_static_scratch_entry_point_matches_workspace_entry_point():
    assert torch.cuda.is_available()
    import quantforge_b200 as qf
    from quantforge_b200 import _lib, ops
    lib = _lib.load()
    dev = torch.device("cuda:0")
    ctx = ops._ctx(dev)
    stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)

    # Plans with more than 8 splits, or more than 8 chunks of K per split, cannot sum their splits inside a
    # thread-block cluster: their partial sums really travel through the static array (the first two cases; the
    # other two take the cluster route and only have the array's counters cleared).
    cases = [(1, 14336, 4096, 0, 20), (2, 4096, 512, 12, 23), (3, 2048, 512, 4, 21), (8, 4096, 1024, 0, 22)]
    used_scratch = 0
    for call, (M, K, N, split_k, seed) in enumerate(cases):
        d = O.make_inputs(M=M, K=K, N=N, group_size=128, act_dtype="bf16", seed=seed)
        x = torch.from_numpy(d["x"]).to(torch.bfloat16).to(dev)
        qw = torch.from_numpy(d["qweight"]).to(dev)
        sc = torch.from_numpy(d["scales"]).to(torch.bfloat16).to(dev)
        zr = qf.pack_zeros_u4(torch.from_numpy(d["zeros"]).to(dev))
        desc = _desc(_lib, M, N, K, split_k)

        ws_bytes = lib.qf_w4a16_workspace_bytes(ctypes.byref(desc))
        assert ws_bytes > 0, "the case must be a split-K plan"
        path, split = ctypes.c_int32(), ctypes.c_int32()
        assert lib.qf_w4a16_plan(ctypes.byref(desc), ctypes.byref(path), ctypes.byref(split)) == 0
        chunks_per_split = -(-(K // 128) // split.value)
        if split.value > 8 or chunks_per_split > 8:
            used_scratch += 1
        ws = torch.zeros(ws_bytes, dtype=torch.uint8, device=dev)
        y_ref = torch.full((M, N), float("nan"), dtype=torch.float32, device=dev)
        st = lib.qf_w4a16_linear(ctx, ctypes.byref(desc), _vp(x), _vp(qw), _vp(sc), _vp(zr), _vp(y_ref), _vp(ws),
                                 ws_bytes, stream)
        assert st == 0, lib.qf_last_error(ctx)

        y = torch.full((M, N), float("nan"), dtype=torch.float32, device=dev)
        st = lib.qf_w4a16_gemv_static_scratch(ctx, ctypes.byref(desc), _vp(x), _vp(qw), _vp(sc), _vp(zr), _vp(y),
                                              stream)
        assert st == 0, lib.qf_last_error(ctx)
        torch.cuda.synchronize()

        # same kernel, same split plan, same summation order: within the tolerance the other GPU tests use
        assert O.rel_err(y.cpu().numpy(), y_ref.cpu().numpy()) < 1e-4, f"call {call}"
        want = O.w4a16_linear(d["x"], d["qweight"], d["scales"], d["zeros"], 128, "bf16", O.F32, accumulate="f64")
        assert O.rel_err(y.cpu().numpy(), want) < 1e-4, f"call {call} vs oracle"
    assert used_scratch >= 2, "at least two of the calls must keep their partial sums in the static array"


def test_static_scratch_rejects_oversized_requests():
    import quantforge_b200 as qf  # noqa: F401
    from quantforge_b200 import _lib, ops
    lib = _lib.load()
    dev = torch.device("cuda:0")
    ctx = ops._ctx(dev)
    # 8 splits x 8 rows x 262144 columns x 4 bytes = 64 MiB of partial sums: more than the 16 MiB array
    desc = _desc(_lib, 8, 262144, 1024, 8)
    dummy = torch.zeros(64, dtype=torch.uint8, device=dev)
    st = lib.qf_w4a16_gemv_static_scratch(ctx, ctypes.byref(desc), _vp(dummy), _vp(dummy), _vp(dummy), _vp(dummy),
                                          _vp(dummy), None)
    assert st == -7  # QF_ERR_WORKSPACE, decided before any pointer is touched
    assert b"static array" in lib.qf_last_error(ctx)

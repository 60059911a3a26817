"""The C-ABI library loads without a GPU and exports every symbol include/quantforge_rt.h declares."""
import ctypes
import os
import re

import pytest

from quantforge_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    if not os.path.exists(_lib.LIB_PATH):
        from quantforge_b200 import build
        build.build()
    return _lib.load()


def _declared_symbols():
    with open(os.path.join(ROOT, "include", "quantforge_rt.h")) as f:
        text = f.read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(qf_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported(lib):
    declared = _declared_symbols()
    assert "qf_w4a16_linear" in declared and "qf_unpack_int4" in declared
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in the header but not exported"
    assert sorted(_lib.EXPORTS) == declared


def test_version_and_status_strings(lib):
    assert lib.qf_version() == 100
    assert _lib.status_name(0) == "QF_OK"
    assert _lib.status_name(-1) == "QF_ERR_BAD_ARG"
    assert _lib.status_name(-5) == "QF_ERR_TIMEOUT"
    assert _lib.status_name(-99) == "QF_ERR_UNKNOWN"


def _desc(M=1, N=4096, K=4096, g=128, act=_lib.QF_F16, out=_lib.QF_F16, zmode=_lib.QF_ZERO_U4, path=0, split=0):
    d = _lib.LinearDesc()
    d.M, d.N, d.K, d.group_size, d.act_dtype, d.out_dtype = M, N, K, g, act, out
    d.zero_mode, d.path, d.split_k = zmode, path, split
    return d


def test_plan_is_host_only_and_validates(lib):
    path, split = ctypes.c_int32(), ctypes.c_int32()
    assert lib.qf_w4a16_plan(ctypes.byref(_desc()), ctypes.byref(path), ctypes.byref(split)) == 0
    assert path.value == _lib.QF_PATH_GEMV and split.value >= 1
    ws = lib.qf_w4a16_workspace_bytes(ctypes.byref(_desc()))
    assert ws >= split.value * 8 * 4096 * 4 if split.value > 1 else ws == 0
    # shape rules
    assert lib.qf_w4a16_plan(ctypes.byref(_desc(K=4000)), None, None) == -1
    assert lib.qf_w4a16_plan(ctypes.byref(_desc(N=4100)), None, None) == -1
    assert lib.qf_w4a16_plan(ctypes.byref(_desc(g=64)), None, None) == -2
    assert lib.qf_w4a16_plan(ctypes.byref(_desc(act=_lib.QF_F32)), None, None) == -2
    assert lib.qf_w4a16_plan(ctypes.byref(_desc(zmode=7)), None, None) == -1
    assert lib.qf_w4a16_workspace_bytes(ctypes.byref(_desc(K=4000))) == 0
    bad = _desc()
    bad.reserved[2] = 1
    assert lib.qf_w4a16_plan(ctypes.byref(bad), None, None) == -1


def test_forced_split_sizes_workspace(lib):
    d = _desc(M=3, N=256, K=1024, split=4)
    split = ctypes.c_int32()
    assert lib.qf_w4a16_plan(ctypes.byref(d), None, ctypes.byref(split)) == 0
    assert split.value == 4
    assert lib.qf_w4a16_workspace_bytes(ctypes.byref(d)) >= 4 * 8 * 256 * 4


def test_no_device_means_error_not_fallback(lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    h = ctypes.c_void_p()
    assert lib.qf_ctx_create(ctypes.byref(h), 0) == -3  # QF_ERR_CUDA
    assert not h.value
    import quantforge_b200 as qf
    with pytest.raises(ValueError):
        qf.unpack_int4(torch.zeros(4, 4, dtype=torch.int8))
    with pytest.raises(ValueError):
        qf.w4a16_linear(torch.zeros(1, 128, dtype=torch.float16), torch.zeros(16, 64, dtype=torch.int8),
                        torch.zeros(1, 16, dtype=torch.float16))


def test_pack_helpers_match_oracle():
    import numpy as np
    import torch
    import quantforge_b200 as qf
    from oracle import qf_oracle as O
    rng = np.random.default_rng(0)
    codes = rng.integers(0, 16, size=(8, 64), dtype=np.int8)
    assert np.array_equal(qf.pack_int4(torch.from_numpy(codes)).numpy(), O.pack_int4(codes))
    z = rng.integers(0, 16, size=(3, 32), dtype=np.int8)
    got = qf.pack_zeros_u4(torch.from_numpy(z)).numpy().view(np.uint32)
    assert np.array_equal(got, O.pack_zeros_u4(z))

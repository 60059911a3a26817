"""Launch planning (host logic of qf_w4a16_plan): which kernel AUTO picks and how K is split. No GPU needed."""
import ctypes

import pytest

from quantforge_b200 import _lib


def _plan(M, K, N, layout=0, path=0, split_k=0):
    lib = _lib.load()
    d = _lib.LinearDesc(M=M, N=N, K=K, group_size=128, act_dtype=_lib.QF_BF16, out_dtype=_lib.QF_BF16,
                        zero_mode=_lib.QF_ZERO_U4, zero_const=8, path=path, split_k=split_k, weight_layout=layout)
    pa, sk = ctypes.c_int32(), ctypes.c_int32()
    st = lib.qf_w4a16_plan(ctypes.byref(d), ctypes.byref(pa), ctypes.byref(sk))
    assert st == 0
    return pa.value, sk.value


@pytest.mark.parametrize("M,K,N,layout,want", [
    (1, 4096, 4096, 0, _lib.QF_PATH_GEMV),        # small matrix, decode batch 1
    (2, 4096, 14336, 0, _lib.QF_PATH_GEMV),       # 29 MB: still the GEMV kernel
    (3, 4096, 4096, 0, _lib.QF_PATH_GEMM),        # M >= 3: tcgen05
    (1, 4096, 4096, 1, _lib.QF_PATH_GEMM),        # prepacked weights are read by the tcgen05 kernel only
    (1, 8192, 8192, 1, _lib.QF_PATH_GEMM),        # 32 MB prepacked: tcgen05
    (1, 8192, 8192, 0, _lib.QF_PATH_GEMV),        # 32 MB canonical: below the 40 MB crossover
    (1, 4096, 28672, 0, _lib.QF_PATH_GEMM),       # 56 MB canonical: tcgen05
    (1, 28672, 8192, 1, _lib.QF_PATH_GEMM),
    (16, 4096, 144, 0, _lib.QF_PATH_GEMV),        # N not a multiple of 128: only the GEMV kernel can
    (1, 16384, 4112, 0, _lib.QF_PATH_GEMV),       # large but N % 128 != 0
])
def test_auto_path(M, K, N, layout, want):
    assert _plan(M, K, N, layout)[0] == want


def test_forced_paths_are_respected():
    assert _plan(1, 8192, 57344, 0, path=_lib.QF_PATH_GEMV)[0] == _lib.QF_PATH_GEMV
    assert _plan(1, 4096, 4096, 0, path=_lib.QF_PATH_GEMM)[0] == _lib.QF_PATH_GEMM
    assert _plan(16, 4096, 4096, 1, split_k=3) == (_lib.QF_PATH_GEMM, 3)


def test_even_k_splits_are_preferred():
    # K = 14336 = 112 k-blocks of 128, 32 tiles: 296 block slots / 32 = 9 splits would leave a short last split
    assert _plan(16, 14336, 4096, 1) == (_lib.QF_PATH_GEMM, 8)
    assert _plan(64, 14336, 4096, 1) == (_lib.QF_PATH_GEMM, 8)
    # GEMV kernel: 112 chunks, 64 column blocks -> 9 splits by block count, 8 divides K evenly and fits a cluster
    assert _plan(1, 14336, 4096, 0) == (_lib.QF_PATH_GEMV, 8)
    # 4096 x 14336: 112 tiles, two splits fill the device
    assert _plan(16, 4096, 14336, 1) == (_lib.QF_PATH_GEMM, 2)


def test_no_split_when_tiles_fill_the_device():
    assert _plan(2048, 8192, 28672, 1) == (_lib.QF_PATH_GEMM, 1)
    assert _plan(64, 8192, 28672, 1) == (_lib.QF_PATH_GEMM, 1)


def test_splits_stay_within_one_wave_of_clusters():
    # tcgen05 kernel, narrow tiles: at most 8 splits and at most 256 blocks, so that the split-K sum stays on chip
    assert _plan(16, 4096, 6144, 1) == (_lib.QF_PATH_GEMM, 5)     # 48 tiles: 6 splits would be 288 blocks
    assert _plan(64, 4096, 5120, 1) == (_lib.QF_PATH_GEMM, 6)     # 40 tiles
    assert _plan(16, 8192, 1024, 1) == (_lib.QF_PATH_GEMM, 8)     # 8 tiles: not 16 splits through global memory
    assert _plan(16, 8192, 10240, 1) == (_lib.QF_PATH_GEMM, 3)    # 80 tiles
    assert _plan(16, 4096, 18944, 1) == (_lib.QF_PATH_GEMM, 2)    # 148 tiles: two splits fill every slot

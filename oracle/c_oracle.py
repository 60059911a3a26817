"""ctypes loader for the C restatement of the reference arithmetic (oracle/qf_oracle.c).

TEST INFRASTRUCTURE ONLY (checker + timed CPU baseline); never imported by the product package.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_DT = {"f16": 0, "bf16": 1, "f32": 2}
_lib = None


def build() -> None:
    subprocess.run(["make", "-C", _HERE, "-s", "all"], check=True)


def _has_avx2() -> bool:
    try:
        with open("/proc/cpuinfo") as f:
            flags = f.read()
        return " avx2" in flags and " f16c" in flags and " fma" in flags
    except OSError:
        return False


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        name = "libqf_oracle_v3.so" if _has_avx2() else "libqf_oracle_generic.so"
        path = os.path.join(_HERE, name)
        if not os.path.exists(path):
            build()
        _lib = ctypes.CDLL(path)
        _lib.qfo_num_threads.restype = ctypes.c_int
    return _lib


def num_threads() -> int:
    return int(lib().qfo_num_threads())


def set_num_threads(n: int) -> None:
    """Thread count of the following calls (torchrun exports OMP_NUM_THREADS=1 to its children)."""
    lib().qfo_set_num_threads(ctypes.c_int(int(n)))


def _p(a: np.ndarray):
    return a.ctypes.data_as(ctypes.c_void_p)


def unpack_int4(packed: np.ndarray) -> np.ndarray:
    packed = np.ascontiguousarray(packed)
    rows, pc = packed.reshape(-1, packed.shape[-1]).shape
    out = np.empty(packed.shape[:-1] + (pc * 2,), dtype=np.int8)
    lib().qfo_unpack_int4(_p(packed), _p(out), ctypes.c_int64(rows), ctypes.c_int64(pc))
    return out


def unpack_words(words: np.ndarray) -> np.ndarray:
    words = np.ascontiguousarray(words, dtype=np.uint32)
    rows, wc = words.reshape(-1, words.shape[-1]).shape
    out = np.empty(words.shape[:-1] + (wc * 8,), dtype=np.int8)
    lib().qfo_unpack_words(_p(words), _p(out), ctypes.c_int64(rows), ctypes.c_int64(wc))
    return out


def _zero_args(zeros, N):
    """-> (array_or_None, zero_mode, zero_const). Accepts scalar, packed uint32[G,N/8] or int8[G,N]."""
    if zeros is None:
        return None, 0, 8
    if np.isscalar(zeros):
        return None, 0, int(zeros)
    z = np.ascontiguousarray(zeros)
    if z.dtype == np.uint32:
        assert z.shape[1] * 8 == N
        return z, 1, 0
    return z.astype(np.int8), 2, 0


def w4a16_linear(x16: np.ndarray, qweight: np.ndarray, scales16: np.ndarray, zeros, group_size: int,
                 act_dtype: str, out_dtype: str = "f32") -> np.ndarray:
    """x16, scales16: uint16 bit patterns of act_dtype. qweight int8/uint8 [N,K/2]. Returns float32 [M,N]."""
    x16 = np.ascontiguousarray(x16, dtype=np.uint16)
    qweight = np.ascontiguousarray(qweight).view(np.uint8)
    scales16 = np.ascontiguousarray(scales16, dtype=np.uint16)
    M, K = x16.shape
    N = qweight.shape[0]
    z, zmode, zconst = _zero_args(zeros, N)
    y = np.empty((M, N), dtype=np.float32)
    lib().qfo_w4a16_linear(_p(x16), _p(qweight), _p(scales16), _p(z) if z is not None else None,
                           ctypes.c_int(zmode), ctypes.c_int(zconst), _p(y), ctypes.c_int64(M),
                           ctypes.c_int64(N), ctypes.c_int64(K), ctypes.c_int64(group_size),
                           ctypes.c_int(_DT[act_dtype]), ctypes.c_int(_DT[out_dtype]))
    return y


def to_bits(x_f32: np.ndarray, dtype: str) -> np.ndarray:
    """float32 values (already representable in dtype) -> uint16 bit patterns."""
    x_f32 = np.asarray(x_f32, dtype=np.float32)
    if dtype == "f16":
        return x_f32.astype(np.float16).view(np.uint16)
    return (x_f32.view(np.uint32) >> 16).astype(np.uint16)

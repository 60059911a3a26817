"""CPU oracle for the W4A16 unpack / dequant / matmul path (numpy).

TEST INFRASTRUCTURE ONLY.  This module restates, on the CPU, the arithmetic the
QuantForge reference defines for its `qf.unpack` / `qf.dequant` ops and the
matmul that consumes them.  It is the checker for the CUDA kernels; it is never
imported by the product package and is never a fallback.

Parity status
-------------
* unpack / pack / nibble order and the per-channel f16 GEMV are PINNED: they are
  checked against outputs of the reference's own Python functions
  (python/quantforge/baseline.py) stored under tests/golden/ (generator:
  tests/golden/make_golden.py).
* group-wise scales/zeros, bf16 activations and fp32 accumulation are extensions
  the reference does not implement; for those the oracle is the definition
  ("parity unpinned" by reference vectors) and is anchored by the degenerate case
  group == K, which must reproduce the pinned per-channel result.

Reference statements followed (paths inside the reference project):
  pack      python/quantforge/baseline.py:17-31
  unpack    lib/Transforms/LowerUnpackToArith.cpp:173-214,
            python/quantforge/baseline.py:34-49
  word      lib/Transforms/LowerUnpackToNVVM.cpp:221-280  (8 codes per uint32, LSB first)
  dequant   lib/Transforms/LowerDequantToArith.cpp:141-159 (sitofp, sitofp, subf, mulf in f16)
  zp == 0   lib/Transforms/CanonicalizeDequantZeroPoint.cpp:177-192
  matmul    lib/Transforms/ConvertLinalgToQuantForge.cpp:185-203,
            python/quantforge/baseline.py:64-72
"""
from __future__ import annotations

import numpy as np

F16 = "f16"
BF16 = "bf16"
F32 = "f32"


# --------------------------------------------------------------------------- #
# bf16 helpers (numpy has no bfloat16): values travel as uint16 bit patterns or
# as float32 arrays whose low 16 mantissa bits are zero.
# --------------------------------------------------------------------------- #
def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even float32 -> bfloat16 bit pattern (uint16)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    nan = (u & 0x7FFFFFFF) > 0x7F800000
    rounded = (u + (0x7FFF + ((u >> 16) & 1))) >> 16
    rounded = np.where(nan, (u >> 16) | 0x40, rounded)
    return rounded.astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def round_to(x: np.ndarray, dtype: str) -> np.ndarray:
    """Round a float32 array to `dtype` and return it as float32 again."""
    x = np.asarray(x, dtype=np.float32)
    if dtype == F32:
        return x
    if dtype == F16:
        return x.astype(np.float16).astype(np.float32)
    if dtype == BF16:
        return bf16_bits_to_f32(f32_to_bf16_bits(x))
    raise ValueError(dtype)


# --------------------------------------------------------------------------- #
# pack / unpack
# --------------------------------------------------------------------------- #
def pack_int4(codes: np.ndarray) -> np.ndarray:
    """codes int8[..., 2n] in [0,15] -> int8[..., n]; even index = low nibble.

    Follows python/quantforge/baseline.py:28-31.
    """
    codes = np.asarray(codes)
    assert codes.dtype == np.int8 and codes.shape[-1] % 2 == 0
    lo = codes[..., 0::2].astype(np.uint8) & 0x0F
    hi = codes[..., 1::2].astype(np.uint8) & 0x0F
    return (lo | (hi << 4)).astype(np.uint8).view(np.int8)


def unpack_int4(packed: np.ndarray) -> np.ndarray:
    """int8[..., n] -> int8[..., 2n]: out[2i] = b & 0xF, out[2i+1] = (b >>u 4) & 0xF.

    The shift is logical, on the raw 8-bit pattern
    (lib/Transforms/LowerUnpackToArith.cpp:173-202).
    """
    b = np.ascontiguousarray(packed).view(np.uint8)
    out = np.empty(b.shape[:-1] + (b.shape[-1] * 2,), dtype=np.int8)
    out[..., 0::2] = (b & 0x0F).astype(np.int8)
    out[..., 1::2] = ((b >> 4) & 0x0F).astype(np.int8)
    return out


def unpack_words(words: np.ndarray) -> np.ndarray:
    """uint32[..., n] -> int8[..., 8n]: code[8c+i] = (w >> 4i) & 0xF.

    Follows lib/Transforms/LowerUnpackToNVVM.cpp:233-280.  On a little-endian
    host this is identical to unpack_int4 of the same bytes.
    """
    w = np.ascontiguousarray(words, dtype=np.uint32)
    out = np.empty(w.shape[:-1] + (w.shape[-1] * 8,), dtype=np.int8)
    for i in range(8):
        out[..., i::8] = ((w >> np.uint32(4 * i)) & np.uint32(0xF)).astype(np.int8)
    return out


def pack_zeros_u4(zeros: np.ndarray) -> np.ndarray:
    """zero codes uint8/int8 [G, N] in [0,15] -> uint32[G, N/8], 8 per word along N, LSB first."""
    z = np.asarray(zeros).astype(np.uint32)
    G, N = z.shape
    assert N % 8 == 0
    z = z.reshape(G, N // 8, 8)
    out = np.zeros((G, N // 8), dtype=np.uint32)
    for i in range(8):
        out |= (z[..., i] & 0xF) << np.uint32(4 * i)
    return out


# --------------------------------------------------------------------------- #
# dequant
# --------------------------------------------------------------------------- #
def dequant(codes: np.ndarray, scales: np.ndarray, zeros, group_size: int, dtype: str) -> np.ndarray:
    """W[n,k] = round_dtype((q[n,k] - z[k/g, n]) * s[k/g, n]) as float32.

    codes  int8[N, K] (values 0..15)
    scales float32[G, N] holding values already representable in `dtype`
    zeros  int array [G, N] (signed, as the reference's i8 zero point) or a scalar
    The difference is exact in f16/bf16 (|q - z| < 2^8), so the reference's
    f16 `subf` then `mulf` (LowerDequantToArith.cpp:141-159) equals one exact
    subtraction followed by one round-to-nearest-even multiply; the product of a
    <=9-bit integer and an 8/11-bit significand is exact in float32, so rounding
    it once to `dtype` reproduces that multiply.
    """
    q = np.asarray(codes).astype(np.float32)
    N, K = q.shape
    G = K // group_size
    assert G * group_size == K
    s = np.asarray(scales, dtype=np.float32)
    assert s.shape == (G, N)
    if np.isscalar(zeros) or np.ndim(zeros) == 0:
        z = np.full((G, N), float(zeros), dtype=np.float32)
    else:
        z = np.asarray(zeros).astype(np.float32)
        assert z.shape == (G, N)
    s_full = np.repeat(s.T, group_size, axis=1)  # [N, K]
    z_full = np.repeat(z.T, group_size, axis=1)
    return round_to((q - z_full) * s_full, dtype)


# --------------------------------------------------------------------------- #
# linear
# --------------------------------------------------------------------------- #
def w4a16_linear(x: np.ndarray, qweight: np.ndarray, scales: np.ndarray, zeros, group_size: int,
                 act_dtype: str, out_dtype: str = F32, accumulate: str = "f32") -> np.ndarray:
    """Y[M,N] = X[M,K] . W^T with W = dequant(unpack(qweight)).

    x        float32[M, K], values already representable in act_dtype
    qweight  int8[N, K/2] (or uint32[N, K/8]) canonical packing along K
    Returns float32[M, N] rounded to out_dtype.
    accumulate: "f32" (numpy sgemm) or "f64".
    """
    if qweight.dtype == np.uint32:
        codes = unpack_words(qweight)
    else:
        codes = unpack_int4(qweight)
    w = dequant(codes, scales, zeros, group_size, act_dtype)  # [N, K] float32
    x = np.asarray(x, dtype=np.float32)
    if accumulate == "f64":
        y = (x.astype(np.float64) @ w.astype(np.float64).T).astype(np.float32)
    else:
        y = x @ w.T
    return round_to(y, out_dtype)


# --------------------------------------------------------------------------- #
# what follows the linear inside a decoder layer (no reference counterpart: definitions for the fused epilogues)
# --------------------------------------------------------------------------- #
def interleave8(a: np.ndarray, b: np.ndarray, axis: int = 0) -> np.ndarray:
    """Groups of 8 entries of `a` followed by the matching 8 of `b`, along `axis` (the gate|up row order)."""
    a = np.moveaxis(np.asarray(a), axis, 0)
    b = np.moveaxis(np.asarray(b), axis, 0)
    n = a.shape[0]
    assert a.shape == b.shape and n % 8 == 0
    both = np.stack([a.reshape(n // 8, 8, *a.shape[1:]), b.reshape(n // 8, 8, *b.shape[1:])], axis=1)
    return np.ascontiguousarray(np.moveaxis(both.reshape(2 * n, *a.shape[1:]), 0, axis))


def silu_mul(gate: np.ndarray, up: np.ndarray, out_dtype: str = F32) -> np.ndarray:
    """silu(gate) * up on fp32 accumulators, rounded once: silu(v) = v / (1 + exp(-v))."""
    g = np.asarray(gate, dtype=np.float64)
    u = np.asarray(up, dtype=np.float64)
    return round_to((g / (1.0 + np.exp(-g)) * u).astype(np.float32), out_dtype)


def repack_kn_to_canonical(codes_kn: np.ndarray) -> np.ndarray:
    """codes int8[K, N] (the matmul operand orientation of lib/Transforms/ConvertLinalgToQuantForge.cpp:185-203)
    -> canonical int8[N, K/2] packed along K (python/quantforge/baseline.py:58-71)."""
    return pack_int4(np.ascontiguousarray(np.asarray(codes_kn, dtype=np.int8).T))


def gemv_int4_per_channel(x: np.ndarray, w_packed: np.ndarray, scale: np.ndarray,
                          zero_point: np.ndarray) -> np.ndarray:
    """Restatement of python/quantforge/baseline.py:52-72 (f16 everywhere, per-row scale/zp).

    Returns float32 holding f16-representable values. The accumulation order of
    the reference's f16 matmul is unspecified; this one accumulates in fp32 and
    rounds once, which the golden test bounds against the reference output.
    """
    K = w_packed.shape[1] * 2
    s = np.asarray(scale, dtype=np.float32)[None, :]
    z = np.asarray(zero_point).astype(np.int32)[None, :]
    return w4a16_linear(x, w_packed, s, z, K, F16, F16)


# --------------------------------------------------------------------------- #
# seeded generators for the benchmark configurations
# --------------------------------------------------------------------------- #
def make_inputs(M: int, K: int, N: int, group_size: int = 128, act_dtype: str = F16, seed: int = 0,
                sigma: float = 0.02, symmetric: bool = False):
    """Synthetic tensors with the value distributions the benchmark configurations name.

    codes uniform uint4; scales |N(0, sigma)|/7 (floored at 2^-14) in act_dtype;
    zeros uniform uint4 per (group, n) or the constant 8; activations N(0,1).
    Returns dict of numpy arrays (float tensors as float32 already rounded to act_dtype).
    """
    rng = np.random.default_rng(seed)
    G = K // group_size
    codes = rng.integers(0, 16, size=(N, K), dtype=np.int8)
    scales = np.maximum(np.abs(rng.normal(0.0, sigma, size=(G, N))) / 7.0, 2.0 ** -14).astype(np.float32)
    scales = round_to(scales, act_dtype)
    if symmetric:
        zeros = None
    else:
        zeros = rng.integers(0, 16, size=(G, N), dtype=np.int8)
    x = round_to(rng.normal(0.0, 1.0, size=(M, K)).astype(np.float32), act_dtype)
    return {
        "codes": codes,
        "qweight": pack_int4(codes),
        "scales": scales,
        "zeros": zeros,
        "x": x,
    }


def rel_err(y: np.ndarray, y_ref: np.ndarray) -> float:
    """max |y - y_ref| / rms(y_ref): the quantity the parity tolerance (1e-2) is stated on."""
    y = np.asarray(y, dtype=np.float64)
    y_ref = np.asarray(y_ref, dtype=np.float64)
    rms = np.sqrt(np.mean(y_ref ** 2))
    return float(np.max(np.abs(y - y_ref)) / max(rms, 1e-30))

"""The oracle (numpy + C restatement) against fixtures made by the reference's own functions."""
import os

import numpy as np
import pytest

from oracle import c_oracle, qf_oracle as O


@pytest.fixture(scope="module")
def unpack_gold(golden_dir):
    return np.load(os.path.join(golden_dir, "unpack.npz"))


@pytest.fixture(scope="module")
def gemv_gold(golden_dir):
    return np.load(os.path.join(golden_dir, "gemv_per_channel.npz"))


def test_unpack_exhaustive_byte_table(unpack_gold):
    b = unpack_gold["all_bytes"]
    want = unpack_gold["unpacked_table"]
    assert np.array_equal(O.unpack_int4(b), want)
    assert np.array_equal(c_oracle.unpack_int4(b), want)
    # every output is a code in [0, 15], also for bytes >= 0x80 (logical shift)
    assert want.min() == 0 and want.max() == 15


def test_pack_matches_reference_and_round_trips(unpack_gold):
    codes, packed = unpack_gold["codes"], unpack_gold["packed"]
    assert np.array_equal(O.pack_int4(codes), packed)
    assert np.array_equal(O.unpack_int4(packed), codes)
    assert np.array_equal(c_oracle.unpack_int4(packed), codes)


def test_word_order_equals_byte_order(unpack_gold):
    packed = unpack_gold["packed"]
    words = np.ascontiguousarray(packed).view(np.uint32)
    assert np.array_equal(O.unpack_words(words), unpack_gold["codes"])
    assert np.array_equal(c_oracle.unpack_words(words), unpack_gold["codes"])


def test_zero_packing_round_trip():
    rng = np.random.default_rng(3)
    z = rng.integers(0, 16, size=(5, 64), dtype=np.int8)
    words = O.pack_zeros_u4(z)
    assert np.array_equal(O.unpack_words(words), z)


@pytest.mark.parametrize("case", ["m1", "m4", "m16", "signed"])
def test_per_channel_gemv_matches_reference(gemv_gold, case):
    x = gemv_gold[f"{case}_x"].astype(np.float32)
    wp = gemv_gold[f"{case}_w_packed"]
    s = gemv_gold[f"{case}_scale"].astype(np.float32)
    zp = gemv_gold[f"{case}_zero_point"]
    want = gemv_gold[f"{case}_y"].astype(np.float32)
    got = O.gemv_int4_per_channel(x, wp, s, zp)
    # the reference multiplies f16 matrices with torch's CPU kernel (accumulation order
    # unspecified, f16 output); the oracle accumulates in fp32: agreement well inside 1e-2 rms
    assert O.rel_err(got, want) < 4e-3
    # dequantised weights themselves are bit-identical to the reference formula in f16
    K = wp.shape[1] * 2
    w = O.dequant(O.unpack_int4(wp), s[None, :], zp[None, :].astype(np.int32), K, O.F16)
    codes = O.unpack_int4(wp).astype(np.float16)
    w_ref = (codes - zp[:, None].astype(np.float16)) * gemv_gold[f"{case}_scale"][:, None]
    assert np.array_equal(w.astype(np.float16).view(np.uint16), w_ref.view(np.uint16))


@pytest.mark.parametrize("act", ["f16", "bf16"])
@pytest.mark.parametrize("zero_kind", ["u4", "const", "i8"])
def test_c_oracle_equals_numpy_oracle(act, zero_kind):
    d = O.make_inputs(M=3, K=512, N=64, group_size=128, act_dtype=act, seed=11)
    if zero_kind == "u4":
        zeros_np, zeros_c = d["zeros"], O.pack_zeros_u4(d["zeros"])
    elif zero_kind == "const":
        zeros_np, zeros_c = 8, 8
    else:
        zeros_np = (d["zeros"].astype(np.int32) - 8).astype(np.int8)
        zeros_c = zeros_np
    want = O.w4a16_linear(d["x"], d["qweight"], d["scales"], zeros_np, 128, act, O.F32, accumulate="f64")
    got = c_oracle.w4a16_linear(c_oracle.to_bits(d["x"], act), d["qweight"], c_oracle.to_bits(d["scales"], act),
                                zeros_c, 128, act, "f32")
    assert O.rel_err(got, want) < 1e-5


def test_group_equal_k_reproduces_per_channel(gemv_gold):
    x = gemv_gold["m4_x"].astype(np.float32)
    wp = gemv_gold["m4_w_packed"]
    s = gemv_gold["m4_scale"].astype(np.float32)
    zp = gemv_gold["m4_zero_point"]
    K = wp.shape[1] * 2
    y_group = O.w4a16_linear(x, wp, s[None, :], zp[None, :].astype(np.int32), K, O.F16, O.F16)
    assert np.array_equal(y_group, O.gemv_int4_per_channel(x, wp, s, zp))


def test_bf16_rounding_helpers():
    x = np.array([1.0, 1.00390625, 1.01171875, -3.14159, 65504.0, 1e-30], dtype=np.float32)
    b = O.f32_to_bf16_bits(x)
    back = O.bf16_bits_to_f32(b)
    assert back[0] == 1.0
    assert back[1] == 1.0            # tie rounds to even (mantissa 0x00)
    assert back[2] == 1.015625       # tie rounds to even upward (mantissa 0x02)
    assert np.all(np.abs(back - x) <= np.abs(x) * 2.0 ** -8)

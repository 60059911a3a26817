"""Generate tests/golden/*.npz from the reference's own Python functions.

Run in a container where the reference checkout is present:
    python tests/golden/make_golden.py /path/to/reference      (or QF_REFERENCE_ROOT=/path/to/reference)
It imports python/quantforge/baseline.py of the reference (pack_int4, unpack_int4,
gemv_int4_baseline), runs them on seeded inputs on the CPU and stores inputs and
outputs.  The fixtures are committed; the tests read only the .npz files.
"""
import os
import sys

import numpy as np
import torch


def main() -> None:
    ref_root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("QF_REFERENCE_ROOT")
    if not ref_root:
        raise SystemExit("usage: make_golden.py /path/to/reference  (the QuantForge checkout)")
    sys.path.insert(0, os.path.join(ref_root, "python"))
    from quantforge.baseline import gemv_int4_baseline, pack_int4, unpack_int4  # noqa: E402

    out_dir = os.path.dirname(os.path.abspath(__file__))
    torch.manual_seed(42)  # the reference script's seed (baseline.py:104)

    # 1. exhaustive byte table: every byte value (incl. >= 0x80) through unpack_int4
    all_bytes = torch.arange(256, dtype=torch.int32).to(torch.uint8).view(torch.int8).reshape(4, 64)
    unpacked_table = unpack_int4(all_bytes)

    # 2. pack -> unpack round trip on random codes (baseline.py:115-116)
    codes = torch.randint(0, 16, (48, 256), dtype=torch.int8)
    packed = pack_int4(codes)
    roundtrip = unpack_int4(packed)
    assert torch.equal(roundtrip, codes)

    np.savez_compressed(
        os.path.join(out_dir, "unpack.npz"),
        all_bytes=all_bytes.numpy(), unpacked_table=unpacked_table.numpy(),
        codes=codes.numpy(), packed=packed.numpy(), roundtrip=roundtrip.numpy(),
    )

    # 3. per-channel f16 GEMV/GEMM, the only numeric form the reference function accepts
    cases = {}
    for name, (M, K, N) in {"m1": (1, 512, 256), "m4": (4, 256, 128), "m16": (16, 384, 64)}.items():
        x = torch.randn(M, K, dtype=torch.float16)
        w_full = torch.randint(0, 16, (N, K), dtype=torch.int8)
        w_packed = pack_int4(w_full)
        scale = torch.randn(N, dtype=torch.float16) * 0.01
        zero_point = torch.randint(0, 16, (N,), dtype=torch.int8)
        y = gemv_int4_baseline(x, w_packed, scale, zero_point)
        cases.update({
            f"{name}_x": x.numpy(), f"{name}_w_packed": w_packed.numpy(), f"{name}_scale": scale.numpy(),
            f"{name}_zero_point": zero_point.numpy(), f"{name}_y": y.numpy(),
        })
    # signed zero points (the dialect's zero_point is a signed i8, LowerDequantToArith.cpp:147-150)
    M, K, N = 2, 256, 64
    x = torch.randn(M, K, dtype=torch.float16)
    w_packed = pack_int4(torch.randint(0, 16, (N, K), dtype=torch.int8))
    scale = torch.randn(N, dtype=torch.float16) * 0.01
    zero_point = torch.randint(-8, 24, (N,), dtype=torch.int8)
    y = gemv_int4_baseline(x, w_packed, scale, zero_point)
    cases.update({"signed_x": x.numpy(), "signed_w_packed": w_packed.numpy(), "signed_scale": scale.numpy(),
                  "signed_zero_point": zero_point.numpy(), "signed_y": y.numpy()})
    np.savez_compressed(os.path.join(out_dir, "gemv_per_channel.npz"), **cases)
    print("wrote", sorted(os.listdir(out_dir)))


if __name__ == "__main__":
    main()

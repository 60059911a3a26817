"""Boundary tests of the re-hosted quantforge-opt: same flag names as the reference's driver, structural checks in
the style of its lit tests (ordered CHECK / CHECK-NOT on the printed IR), inputs under tests/mlir/."""
import os
import re
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
MLIR = os.path.join(ROOT, "tests", "mlir")


@pytest.fixture(scope="module")
def opt():
    from quantforge_b200 import build
    return build.build_opt()


def run(opt, args, path=None, stdin=None, expect=0):
    cmd = [opt] + args + ([os.path.join(MLIR, path)] if path else [])
    r = subprocess.run(cmd, input=stdin, capture_output=True, text=True)
    assert r.returncode == expect, r.stderr
    return r.stdout, r.stderr


def func_body(out, name):
    m = re.search(r"func\.func @" + name + r"\(.*?\n}\n", out, re.S)
    assert m, f"function {name} not printed"
    return m.group(0)


def check_order(text, patterns):
    pos = 0
    for p in patterns:
        m = re.compile(p).search(text, pos)
        assert m, f"pattern not found in order: {p}\n{text}"
        pos = m.end()


def test_round_trip_without_passes(opt):
    out, _ = run(opt, [], "unpack_dequant.mlir")
    out2, _ = run(opt, [], stdin=out)
    assert out == out2
    assert "qf.unpack %arg0 : tensor<4096x2048xi8> -> tensor<4096x4096xi8>" in out


def test_convert_linalg_to_quantforge(opt):
    out, _ = run(opt, ["--convert-linalg-to-quantforge"], "gemv.mlir")
    body = func_body(out, "gemv")
    check_order(body, [
        r"%\S+ = qf\.unpack %weight : tensor<4096x4096xi8> -> tensor<4096x4096xi8>",
        r"arith\.constant dense<5\.000000e-01> : tensor<f16>",       # harvested qf.scale
        r"arith\.constant dense<8> : tensor<i8>",                    # harvested qf.zp
        r"qf\.dequant %\S+, %\S+, %\S+ : tensor<4096x4096xi8>, tensor<f16>, tensor<i8> -> tensor<4096x4096xf16>",
        r"linalg\.matmul ins\(%act, %\S+ : tensor<1x4096xf16>, tensor<4096x4096xf16>\)",
    ])
    noop = func_body(out, "fp16_untouched")
    assert "qf.unpack" not in noop and "qf.dequant" not in noop and "linalg.matmul" in noop
    lhs = func_body(out, "int8_lhs")
    check_order(lhs, [r"qf\.unpack", r"arith\.constant dense<1\.000000e\+00> : tensor<f16>",
                      r"arith\.constant dense<0> : tensor<i8>", r"qf\.dequant",
                      r"arith\.sitofp %act : tensor<2x256xi8> to tensor<2x256xf16>",
                      r"linalg\.matmul ins\(%\S+, %\S+ : tensor<2x256xf16>, tensor<256x512xf16>\)"])


def test_pass_pipeline_syntax_and_bitwidth_option(opt):
    out, _ = run(opt, ["-pass-pipeline=builtin.module(func.func(convert-linalg-to-quantforge{qf-bitwidth=4}))"],
                 "gemv.mlir")
    assert "qf.unpack" in func_body(out, "gemv")
    run(opt, ["-pass-pipeline=builtin.module(func.func(convert-linalg-to-quantforge{qf-bitwidth=3}))"], "gemv.mlir",
        expect=1)


def test_fusion_pipeline(opt):
    out, _ = run(opt, ["--convert-linalg-to-quantforge", "--fuse-unpack-dequant"], "gemv.mlir")
    body = func_body(out, "gemv")
    assert "qf.unpack" not in body and "qf.dequant" not in body and "tensor.collapse_shape" not in body
    check_order(body, [r"linalg\.generic", r"arith\.andi", r"arith\.sitofp", r"arith\.subf", r"arith\.mulf",
                       r"linalg\.yield", r"linalg\.matmul ins\(%act, %\S+ : tensor<1x4096xf16>, tensor<4096x4096xf16>\)"])


def test_canonicalize_dequant_zp(opt):
    out, _ = run(opt, ["--canonicalize-dequant-zp"], "ops.mlir")
    sym = func_body(out, "dequant_symmetric")
    assert "qf.dequant" not in sym and "arith.subf" not in sym
    check_order(sym, [r"linalg\.generic", r"\^bb0\(%\S+: i8, %\S+: f16, %\S+: f16\):", r"arith\.sitofp %\S+ : i8 to f16\n\s*%\S+ = arith\.mulf",
                      r"linalg\.yield"])
    assert "qf.dequant" in func_body(out, "dequant_asymmetric")   # zero point 8: untouched


def test_lower_qf_to_runtime(opt):
    out, _ = run(opt, ["--convert-linalg-to-quantforge", "--lower-qf-to-runtime"], "gemv.mlir")
    body = func_body(out, "gemv")
    assert "qf.unpack" not in body and "qf.dequant" not in body and "linalg.matmul" not in body
    check_order(body, [r"%result = func\.call @qf_w4a16_linear_m1_k4096_n4096\(%act, %weight, %\S+, %\S+, %\S+\)",
                       r"qf\.weight_orientation = \"kn\""])
    assert re.search(r'func\.func private @qf_w4a16_linear_m1_k4096_n4096\(.*\) -> tensor<1x4096xf16> attributes '
                     r'\{qf\.runtime_symbol = "qf_w4a16_linear"\}', out)
    assert "linalg.matmul" in func_body(out, "fp16_untouched")
    out, _ = run(opt, ["--lower-qf-to-runtime"], "unpack_dequant.mlir")
    assert re.search(r"%0 = func\.call @qf_unpack_int4_4096x2048\(%arg0\)", func_body(out, "unpack_only"))
    d = func_body(out, "unpack_dequant")
    assert "qf." not in d.replace("qf.runtime", "")
    check_order(d, [r"%d = func\.call @qf_dequant_w4_256x64\(%w, %scale, %zp\) \{group_size = 128 : i64\}"])


def test_no_fallback_and_unknown_passes_fail(opt):
    # a qf.dequant on a plain tensor cannot become a runtime call: the pass fails (exit 1), nothing is emulated
    _, err = run(opt, ["--lower-qf-to-runtime"], "ops.mlir", expect=1)
    assert "no CPU fallback" in err
    _, err = run(opt, ["--quantforge-tiling"], "ops.mlir", expect=1)
    assert "not part of this build" in err
    run(opt, ["--no-such-pass"], "ops.mlir", expect=1)


def test_fuse_shape_doubling_form(opt):
    out, _ = run(opt, ["--fuse-unpack-dequant"], "unpack_dequant.mlir")
    body = func_body(out, "unpack_dequant")
    assert "qf.unpack" not in body and "qf.dequant" not in body
    check_order(body, [r"arith\.constant 15 : i8", r"arith\.constant 4 : i8", r"tensor\.empty\(\) : tensor<256x64x2xf16>",
                       r"linalg\.generic", r"arith\.andi", r"arith\.shrui", r"arith\.andi", r"arith\.select",
                       r"arith\.sitofp", r"arith\.subf", r"arith\.mulf", r"linalg\.yield",
                       r"tensor\.collapse_shape %\S+ \[\[0\], \[1, 2\]\] : tensor<256x64x2xf16> into tensor<256x128xf16>"])
    # a lone unpack has no dequant to fuse with: untouched
    assert "qf.unpack" in func_body(out, "unpack_only")


def test_fold_subf_zero(opt):
    out, _ = run(opt, ["--canonicalize-dequant-zp"], "unpack_dequant.mlir")
    body = func_body(out, "fold_subf_zero")
    assert "arith.subf" not in body and "return %x : f16" in body


def test_scalar_lowerings_of_unpack_and_dequant(opt):
    """The reference's scalar lowerings under their own flag names (the arithmetic the kernels implement)."""
    out, _ = run(opt, ["--lower-unpack-to-arith"], "unpack_dequant.mlir")
    assert re.search(r"^#map\d* = affine_map<\(d0, d1, d2\) -> \(d0, d1\)>", out, re.M)
    body = func_body(out, "unpack_only")
    assert "qf.unpack" not in body
    check_order(body, [r"arith\.constant 15 : i8", r"arith\.constant 4 : i8", r"tensor\.empty\(\) : tensor<4096x2048x2xi8>",
                       r"linalg\.generic \{indexing_maps = \[#map\d*, #map\d*\]", r"arith\.andi", r"arith\.shrui",
                       r"arith\.andi", r"arith\.select", r"linalg\.yield",
                       r"tensor\.collapse_shape %\S+ \[\[0\], \[1, 2\]\] : tensor<4096x2048x2xi8> into tensor<4096x4096xi8>"])

    out, _ = run(opt, ["--lower-unpack-branch-free"], "unpack_dequant.mlir")
    body = func_body(out, "unpack_only")
    assert "qf.unpack" not in body and "arith.select" not in body and "linalg.index" not in body
    check_order(body, [r"linalg\.generic", r"arith\.andi %b", r"linalg\.generic", r"arith\.shrui %b", r"arith\.andi",
                       r"tensor\.insert_slice %\S+ into %\S+\[0, 0\] \[4096, 2048\] \[1, 2\]",
                       r"tensor\.insert_slice %\S+ into %\S+\[0, 1\] \[4096, 2048\] \[1, 2\]"])

    for flag, marks in (("--lower-unpack-to-nvvm", [r"arith\.shrui", r"arith\.andi", r"arith\.trunci"]),
                        ("--lower-unpack-to-prmt", [r'llvm\.inline_asm "prmt\.b32', r'llvm\.inline_asm "prmt\.b32',
                                                    r"arith\.trunci"])):
        out, _ = run(opt, [flag], "unpack_dequant.mlir")
        body = func_body(out, "unpack_only")
        assert "qf.unpack" not in body and "linalg.generic" not in body
        check_order(body, [r"scf\.for", r"scf\.for"] + [r"tensor\.extract"] * 4 +
                    [r"arith\.extui", r"arith\.shli", r"arith\.ori"] + marks + [r"tensor\.insert "] * 8 + [r"scf\.yield"])

    out, _ = run(opt, ["--lower-dequant-to-arith"], "unpack_dequant.mlir")
    body = func_body(out, "unpack_dequant")
    assert "qf.dequant" not in body and "qf.unpack" in body
    check_order(body, [r"linalg\.generic", r"arith\.sitofp %\S+ : i8 to f16", r"arith\.sitofp %\S+ : i8 to f16",
                       r"arith\.subf", r"arith\.mulf", r"linalg\.yield"])

    out, _ = run(opt, ["--fuse-unpack-dequant-branch-free"], "unpack_dequant.mlir")
    body = func_body(out, "unpack_dequant")
    assert "qf." not in body and "arith.select" not in body
    check_order(body, [r"linalg\.generic", r"arith\.sitofp", r"linalg\.generic", r"arith\.shrui", r"arith\.sitofp",
                       r"tensor\.insert_slice .*\[0, 0\].*\[1, 2\]", r"tensor\.insert_slice .*\[0, 1\].*\[1, 2\]"])

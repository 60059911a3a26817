"""The reference's own lit files for the hot-path passes, run through the re-hosted quantforge-opt and FileCheck.

The RUN lines of the files are executed as written (tool names substituted), as the reference's lit.cfg.py does.
Skipped where the reference checkout or a FileCheck binary is absent (the checkout does not travel to GPU hosts);
tests/test_quantforge_opt.py covers the same passes on this repository's own inputs.
"""
import os
import re
import shutil
import subprocess

import pytest

REF = os.environ.get("QUANTFORGE_REFERENCE", "/root/reference")
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _filecheck():
    cand = [os.environ.get("FILECHECK"), shutil.which("FileCheck")]
    try:
        import triton
        cand.append(os.path.join(os.path.dirname(triton.__file__), "FileCheck"))
    except Exception:  # noqa: BLE001
        pass
    for c in cand:
        if c and os.path.exists(c) and os.access(c, os.X_OK):
            return c
    return None


FILECHECK = _filecheck()
pytestmark = pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "test")) or FILECHECK is None,
                                reason="needs the reference checkout and a FileCheck binary")

# The check files are used with two mechanical adjustments, applied to a temporary copy. They do not change what a
# line asks for; without them the lines cannot match ANY printer of the same IR, the reference's included (its
# repository has no lit site configuration or check target, the files were evidently never run):
#   * `%{{.*}}` (an SSA name) is greedy in FileCheck's POSIX regexes. linalg.generic prints `ins(...) outs(...)` on
#     one line, so `ins(%{{.*}} : T)` swallows the text up to the LAST ` : T)` of the line and the CHECK-SAME for
#     `outs(` that follows finds nothing. The wildcard is narrowed to the characters an SSA name can have.
#   * `llvm.inline_asm {{.*}} prmt.b32` demands a blank in front of the instruction name, but the asm string starts
#     with it (`"prmt.b32 $0, ...`, lib/Transforms/LowerUnpackToPRMT.cpp:234): the blank is dropped.
SSA_WILDCARD = (re.compile(r"%\{\{\.\*\}\}"), "%{{[A-Za-z0-9_.$#-]+}}")
ASM_BLANK = ("llvm.inline_asm {{.*}} prmt.b32", "llvm.inline_asm {{.*}}prmt.b32")

# file -> None (whole file) or the text at which the file is cut: lower_unpack_branch_free.mlir's last case expects
# qf.dequant to disappear under a RUN line that only runs --lower-unpack-branch-free, which no pass with that
# contract can satisfy (the reference's own pass leaves the op in place as well).
FILES = {
    "test/Dialect/QuantForge/basic.mlir": None,
    "test/Transforms/unpack_fusion_pipeline.mlir": None,
    "test/Transforms/canonicalize_dequant_zp.mlir": None,
    "test/Transforms/convert_linalg_to_qf.mlir": None,
    "test/Transforms/fuse_unpack_dequant.mlir": None,
    "test/Transforms/lower_unpack_to_arith.mlir": None,
    "test/Transforms/lower_unpack_branch_free.mlir": "// Test 5: Fused branch-free",
    "test/Transforms/lower_unpack_to_nvvm.mlir": None,
    "test/Transforms/lower_unpack_to_prmt.mlir": None,
    "test/Transforms/lower_dequant_to_arith.mlir": None,
}


@pytest.fixture(scope="module")
def opt():
    from quantforge_b200 import build
    return build.build_opt()


def run_lines(path):
    out = []
    with open(path) as f:
        for ln in f:
            m = re.match(r"\s*//\s*RUN:\s*(.*)$", ln)
            if m:
                out.append(m.group(1).strip())
    # lit joins RUN lines that end in a backslash
    joined, cur = [], ""
    for r in out:
        if r.endswith("\\"):
            cur += r[:-1] + " "
        else:
            joined.append(cur + r)
            cur = ""
    return joined


@pytest.mark.parametrize("rel", sorted(FILES))
def test_reference_lit_file(rel, opt, tmp_path):
    src = os.path.join(REF, rel)
    if not os.path.exists(src):
        pytest.skip(f"{rel} is not in this checkout")
    cut = FILES[rel]
    text = open(src).read()
    if cut is not None:
        pos = text.find(cut)
        assert pos > 0, "cut marker not found"
        # keep whole comment lines: cut at the start of the separator line above the marker
        pos = text.rfind("\n// ----", 0, pos)
        text = text[:pos] + "\n"
    text = SSA_WILDCARD[0].sub(SSA_WILDCARD[1], text).replace(*ASM_BLANK)
    path = str(tmp_path / os.path.basename(rel))
    with open(path, "w") as f:
        f.write(text)
    runs = run_lines(src)
    assert runs, "no RUN line"
    for r in runs:
        cmd = re.sub(r"\bquantforge-opt\b", opt, r)
        cmd = re.sub(r"\bFileCheck\b", FILECHECK, cmd)
        cmd = cmd.replace("%s", path)
        res = subprocess.run(["bash", "-o", "pipefail", "-c", cmd], capture_output=True, text=True)
        assert res.returncode == 0, f"{r}\n{res.stderr[-3000:]}"

"""Executes the runtime calls that `quantforge-opt --lower-qf-to-runtime` leaves in a function.

The lowering replaces `linalg.matmul(x, qf.dequant(qf.unpack(w), scale, zp))` by
`func.call @qf_w4a16_linear_m<M>_k<K>_n<N>(x, w, scale, zp, init) {group_size, qf.weight_orientation = "kn"}` whose
private declaration names the C entry point (`qf.runtime_symbol`). This module is the host side of such a call for
torch tensors: it binds the operands the way a compiled caller would -

  * the weight operand is the matmul's B operand, W[K, N] with one 4-bit code per byte (the same-shape `qf.unpack`
    of the reference's matcher only masks `& 0xF`, lib/Transforms/ConvertLinalgToQuantForge.cpp:118,185-203):
    it is converted once to the canonical [N, K/2] layout with qf_repack_kn_to_canonical;
  * a rank-0 scale is one quantisation group spanning K (`group_size = 0` on the call), replicated per output column;
  * a rank-0 i8 zero point is the constant-zero mode of the kernels;
  * the `init` operand is the zero-filled accumulator the matcher creates; the kernels start from zero themselves.

Only the operations the lowering emits around the call are interpreted (tensor constants, arith.sitofp of the
activations, func.call, return); anything else is an error - there is no CPU evaluation of the dialect here.
"""
from __future__ import annotations

import re
from typing import Dict

import torch

from . import ops

_CALL = re.compile(
    r"(%[\w.\-#]+) = func\.call (@[\w.]+)\(([^)]*)\)\s*(\{[^}]*\})?\s*:\s*\(([^)]*)\)\s*->\s*(tensor<[^>]*>)")
_CONST = re.compile(r"(%[\w.\-#]+) = arith\.constant\s+dense<([^>]*)>\s*:\s*tensor<(f16|i8)>")
_SITOFP = re.compile(r"(%[\w.\-#]+) = arith\.sitofp (%[\w.\-#]+) : tensor<[^>]*> to tensor<[^>]*xf16>")
_DECL = re.compile(r"func\.func private (@[\w.]+)\(.*?attributes \{qf\.runtime_symbol = \"(\w+)\"\}")
_RET = re.compile(r"return (%[\w.\-#]+)")


def _function_text(module: str, name: str) -> str:
    m = re.search(r"func\.func @" + re.escape(name) + r"\(.*?\n}\n", module, re.S)
    if not m:
        raise ValueError(f"function @{name} not found")
    return m.group(0)


def run_lowered(module: str, func: str, args: Dict[str, torch.Tensor]) -> torch.Tensor:
    """Runs function `func` of the lowered module text on CUDA tensors `args` (block-argument name -> tensor)."""
    symbols = dict(_DECL.findall(module))
    body = _function_text(module, func)
    if re.search(r"\bqf\.(unpack|dequant)\b", body):
        raise ValueError("the function still holds qf ops: run --lower-qf-to-runtime first (nothing evaluates them here)")
    env: Dict[str, object] = {("%" + k.lstrip("%")): v for k, v in args.items()}
    lines = body.splitlines()
    start = next(i for i, ln in enumerate(lines) if ln.rstrip().endswith("{")) + 1  # the header may span lines
    for line in lines[start:]:
        line = line.strip()
        if not line or line == "}":
            continue
        m = _CONST.match(line)
        if m:
            env[m.group(1)] = ("const", m.group(3), float(m.group(2)) if m.group(3) == "f16" else int(m.group(2)))
            continue
        m = _SITOFP.match(line)
        if m:
            env[m.group(1)] = env[m.group(2)].to(torch.float16)
            continue
        m = _CALL.match(line)
        if m:
            res, sym, operands, attrs = m.group(1), m.group(2), [o.strip() for o in m.group(3).split(",")], m.group(4) or ""
            entry = symbols.get(sym)
            if entry != "qf_w4a16_linear":
                raise NotImplementedError(f"call to {sym} ({entry}) is not bound here")
            if 'qf.weight_orientation = "kn"' not in attrs:
                raise ValueError("expected the [K, N] weight orientation the lowering emits")
            x, w_kn, scale, zp = (env[o] for o in operands[:4])
            if not (isinstance(scale, tuple) and isinstance(zp, tuple)):
                raise NotImplementedError("scale and zero point must be the rank-0 constants of the lowering")
            K, N = w_kn.shape
            qweight = ops.repack_kn_to_canonical(w_kn.contiguous(), K, N)
            g = re.search(r"group_size = (\d+)", attrs)
            group = int(g.group(1)) if g and int(g.group(1)) > 0 else K
            scales = torch.full((K // group, N), scale[2], dtype=torch.float16, device=x.device)
            env[res] = ops.w4a16_linear(x.contiguous(), qweight, scales, None, group_size=group, zero_const=zp[2],
                                        out_dtype=torch.float16)
            continue
        m = _RET.match(line)
        if m:
            return env[m.group(1)]
        if re.match(r"(%[\w.\-#]+ = )?(tensor\.empty|linalg\.fill|arith\.constant)", line):
            continue  # the accumulator the matcher builds (zero fill) and scalar constants feeding it
        raise NotImplementedError(f"cannot execute: {line}")
    raise ValueError("no return in function")

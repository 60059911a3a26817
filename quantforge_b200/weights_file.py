"""On-disk container for quantised linears: the canonical tensors of the runtime, nothing kernel-specific.

    save_w4(path, {"layers.0.q_proj": QuantizedLinear(qweight, scales, zeros, group_size, zero_const), ...})
    linears = load_w4(path, device="cuda:0")            # name -> QuantizedLinear on that device
    slab = linears["layers.0.q_proj"].to_slab()         # prepack for the streaming GEMV kernel (CUDA only)

File layout (little endian): magic b"QFW4\\0\\0\\0\\1" | u64 length of the JSON index | JSON index | padding to 64 B |
blobs, each 64-byte aligned. The index lists per linear: N, K, group_size, zero_const, scale dtype and for each of
`qweight` (int8 [N, K/2], two codes per byte along K, even index in the low nibble - the reference's pack_int4,
python/quantforge/baseline.py:17-31), `scales` ([K/group, N], f16 or bf16) and `zeros` (int8 [K/group, N] zero
points, absent for a constant zero) its offset, byte length and a CRC-32. Prepacked layouts are never stored:
they are a pure function of these tensors and of the kernel that reads them (qf_prepack_*), so files stay valid
when kernels change. The reference saves plain tensors the same way (python/quantforge/baseline.py:124-130).
"""
from __future__ import annotations

import json
import struct
import zlib
from dataclasses import dataclass
from typing import Dict, Optional

import numpy as np
import torch

MAGIC = b"QFW4\0\0\0\1"
_ALIGN = 64
_SCALE_DT = {"f16": torch.float16, "bf16": torch.bfloat16}


@dataclass
class QuantizedLinear:
    qweight: torch.Tensor            # int8 [N, K/2]
    scales: torch.Tensor             # f16 | bf16 [G, N]
    zeros: Optional[torch.Tensor]    # int8 [G, N] zero points, or None for the constant `zero_const`
    group_size: int = 128
    zero_const: int = 8

    @property
    def N(self) -> int:
        return self.qweight.shape[0]

    @property
    def K(self) -> int:
        return self.qweight.shape[1] * 2

    def check(self) -> None:
        N, K = self.N, self.K
        if self.qweight.dtype != torch.int8 or self.qweight.dim() != 2:
            raise ValueError("qweight must be int8 [N, K/2]")
        if self.group_size <= 0 or K % self.group_size != 0:
            raise ValueError("group_size must divide K")
        G = K // self.group_size
        if self.scales.dtype not in (torch.float16, torch.bfloat16) or tuple(self.scales.shape) != (G, N):
            raise ValueError(f"scales must be f16|bf16 [{G}, {N}]")
        if self.zeros is not None and (self.zeros.dtype != torch.int8 or tuple(self.zeros.shape) != (G, N)):
            raise ValueError(f"zeros must be int8 [{G}, {N}]")

    def to(self, device) -> "QuantizedLinear":
        return QuantizedLinear(self.qweight.to(device), self.scales.to(device),
                               None if self.zeros is None else self.zeros.to(device), self.group_size, self.zero_const)

    def kernel_zeros(self) -> Optional[torch.Tensor]:
        """Zero points as the linear calls take them: uint4 codes packed 8 per word when they fit, int8 otherwise."""
        from . import ops
        if self.zeros is None:
            return None
        if self.N % 8 == 0 and int(self.zeros.min()) >= 0 and int(self.zeros.max()) <= 15:
            return ops.pack_zeros_u4(self.zeros)
        return self.zeros

    def to_slab(self):
        """QF_LAYOUT_GEMV_SLAB prepack of this linear (tensors must live on a CUDA device)."""
        from . import ops
        return ops.prepack_gemv_slab(self.qweight, self.scales, self.kernel_zeros(), self.group_size, self.zero_const)


def _blob(t: torch.Tensor) -> bytes:
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().tobytes()
    return t.numpy().tobytes()


def save_w4(path: str, linears: Dict[str, QuantizedLinear]) -> None:
    index, blobs, offset = {}, [], 0
    for name, lin in linears.items():
        lin.check()
        entry = {"N": lin.N, "K": lin.K, "group_size": lin.group_size, "zero_const": lin.zero_const,
                 "scale_dtype": "f16" if lin.scales.dtype == torch.float16 else "bf16", "tensors": {}}
        for key, t in (("qweight", lin.qweight), ("scales", lin.scales), ("zeros", lin.zeros)):
            if t is None:
                continue
            b = _blob(t)
            entry["tensors"][key] = {"offset": offset, "nbytes": len(b), "crc32": zlib.crc32(b) & 0xFFFFFFFF}
            blobs.append(b)
            offset += -(-len(b) // _ALIGN) * _ALIGN
        index[name] = entry
    head = json.dumps({"version": 1, "linears": index}, sort_keys=True).encode()
    with open(path, "wb") as f:
        f.write(MAGIC)
        f.write(struct.pack("<Q", len(head)))
        f.write(head)
        f.write(b"\0" * (-(len(MAGIC) + 8 + len(head)) % _ALIGN))
        for b in blobs:
            f.write(b)
            f.write(b"\0" * (-len(b) % _ALIGN))


def load_w4(path: str, device="cpu", verify: bool = True) -> Dict[str, QuantizedLinear]:
    with open(path, "rb") as f:
        if f.read(len(MAGIC)) != MAGIC:
            raise ValueError(f"{path}: not a QFW4 weights file")
        (n,) = struct.unpack("<Q", f.read(8))
        head = json.loads(f.read(n))
        base = -(-(len(MAGIC) + 8 + n) // _ALIGN) * _ALIGN
        data = f.read()
    skip = base - (len(MAGIC) + 8 + n)
    out = {}
    for name, e in head["linears"].items():
        N, K, G = e["N"], e["K"], e["K"] // e["group_size"]

        def tensor(key, shape, np_dt, torch_dt=None):
            t = e["tensors"].get(key)
            if t is None:
                return None
            raw = data[skip + t["offset"]: skip + t["offset"] + t["nbytes"]]
            if len(raw) != t["nbytes"] or (verify and (zlib.crc32(raw) & 0xFFFFFFFF) != t["crc32"]):
                raise ValueError(f"{path}: tensor {name}.{key} is truncated or corrupt")
            arr = torch.from_numpy(np.frombuffer(raw, dtype=np_dt).reshape(shape).copy())
            return arr.view(torch_dt) if torch_dt is not None else arr

        sdt = _SCALE_DT[e["scale_dtype"]]
        lin = QuantizedLinear(tensor("qweight", (N, K // 2), np.int8),
                              tensor("scales", (G, N), np.int16, sdt),
                              tensor("zeros", (G, N), np.int8), e["group_size"], e["zero_const"])
        lin.check()
        out[name] = lin.to(device)
    return out


def quantize_linear(weight: torch.Tensor, group_size: int = 128, symmetric: bool = False) -> QuantizedLinear:
    """Floating-point weight [N, K] -> QuantizedLinear (quantize_w4 + pack_int4)."""
    from . import quantize as Q
    codes, scales, zeros = Q.quantize_w4(weight, group_size, symmetric)
    return QuantizedLinear(Q.pack_int4(codes), scales, zeros, group_size, 8)

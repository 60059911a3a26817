"""The quantised linears of a decoder layer stack, run back to back: the "decode-linear us/token" workload.

Each layer has q (H->H), k, v (H->KV), o (H->H), gate, up (H->F), down (F->H). Only the linears run; attention,
norms and activations are outside the W4A16 path, so outputs are chained where shapes agree (q feeds o, o feeds
gate/up, gate feeds down, down feeds the next layer). With tensor parallelism q/k/v/gate/up are column-parallel
(outputs stay sharded) and o/down are row-parallel followed by an all-reduce, one process per GPU.
Weights are random int4 codes with the distributions of the benchmark configurations (shapes only, no checkpoint).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from . import ops
from ._lib import QF_LAYOUT_CANONICAL, QF_LAYOUT_INTERLEAVED

LLAMA3_8B = {"hidden": 4096, "kv": 1024, "ffn": 14336, "layers": 32}
LLAMA3_70B = {"hidden": 8192, "kv": 1024, "ffn": 28672, "layers": 80}
GROUP = 128


BIG_WEIGHT_BYTES = 32 << 20  # from here on the tcgen05 kernel serves M <= 2 as well (prepacked weights)


def _rand_linear(N, K, dtype, dev, gen, prepack):
    qw = torch.randint(-128, 128, (N, K // 2), dtype=torch.int8, device=dev, generator=gen)
    layout = QF_LAYOUT_CANONICAL
    if (prepack or N * K // 2 >= BIG_WEIGHT_BYTES) and N % 128 == 0:
        qw = ops.prepack_w4(qw)
        layout = QF_LAYOUT_INTERLEAVED
    G = K // GROUP
    sc = (torch.randn(G, N, device=dev, generator=gen).abs() * (0.02 / 7.0)).clamp_min(2.0 ** -14).to(dtype)
    zr = ops.pack_zeros_u4(torch.randint(0, 16, (G, N), dtype=torch.int8, device=dev, generator=gen))
    return {"qw": qw, "sc": sc, "zr": zr, "layout": layout, "N": N, "K": K}


def linear_bytes(M, K, N, out_bytes=2):
    G = K // GROUP
    return K * N // 2 + G * N * 2 + G * N // 2 + M * K * 2 + M * N * out_bytes


class DecodeLinearStack:
    def __init__(self, cfg: dict, batch: int, dtype=torch.bfloat16, device=None, world: int = 1, rank: int = 0,
                 group: Optional[dist.ProcessGroup] = None, layers: Optional[int] = None, seed: int = 0,
                 fuse: bool = False, fused_allreduce: bool = False):
        """fuse=True runs q/k/v as ONE linear over the concatenated output rows and gate/up likewise (4 launches
        per layer instead of 7; same weights, same bytes, same results).
        fused_allreduce=True (world > 1, batch <= 64): the row-parallel o and down linears sum across ranks inside
        the kernel over peer memory instead of being followed by an NCCL all-reduce."""
        self.cfg, self.M, self.dtype = cfg, batch, dtype
        self.dev = device or torch.device("cuda", torch.cuda.current_device())
        self.world, self.rank, self.group = world, rank, group
        self.L = layers or cfg["layers"]
        H, KV, F = cfg["hidden"], cfg["kv"], cfg["ffn"]
        assert H % world == 0 and KV % world == 0 and F % world == 0
        gen = torch.Generator(device=self.dev)
        gen.manual_seed(seed + 7919 * rank)
        prepack = batch > 2  # the tcgen05 kernel serves M > 2 and reads the interleaved layout
        self.fuse = fuse
        self.comm = None
        if fused_allreduce and world > 1:
            if batch > 64:
                raise ValueError("fused_allreduce needs batch <= 64")
            self.comm = ops.Comm(batch * H, device=self.dev, group=group)
        prepack_row = prepack
        self.layers = []
        for _ in range(self.L):
            if fuse:
                self.layers.append({
                    "qkv": _rand_linear((H + 2 * KV) // world, H, dtype, self.dev, gen, prepack),
                    "o": _rand_linear(H, H // world, dtype, self.dev, gen, prepack_row),
                    "gate_up": _rand_linear(2 * F // world, H, dtype, self.dev, gen, prepack),
                    "down": _rand_linear(H, F // world, dtype, self.dev, gen, prepack_row),
                })
            else:
                self.layers.append({
                    "q": _rand_linear(H // world, H, dtype, self.dev, gen, prepack),
                    "k": _rand_linear(KV // world, H, dtype, self.dev, gen, prepack),
                    "v": _rand_linear(KV // world, H, dtype, self.dev, gen, prepack),
                    "o": _rand_linear(H, H // world, dtype, self.dev, gen, prepack_row),
                    "gate": _rand_linear(F // world, H, dtype, self.dev, gen, prepack),
                    "up": _rand_linear(F // world, H, dtype, self.dev, gen, prepack),
                    "down": _rand_linear(H, F // world, dtype, self.dev, gen, prepack_row),
                })
        M = batch
        self.h = torch.randn(M, H, device=self.dev, generator=gen).to(dtype)
        self.buf = {
            "q": torch.empty(M, H // world, dtype=dtype, device=self.dev),
            "k": torch.empty(M, KV // world, dtype=dtype, device=self.dev),
            "v": torch.empty(M, KV // world, dtype=dtype, device=self.dev),
            "o": torch.empty(M, H, dtype=dtype, device=self.dev),
            "gate": torch.empty(M, F // world, dtype=dtype, device=self.dev),
            "up": torch.empty(M, F // world, dtype=dtype, device=self.dev),
            "down": torch.empty(M, H, dtype=dtype, device=self.dev),
            "qkv": torch.empty(M, (H + 2 * KV) // world, dtype=dtype, device=self.dev),
            "gate_up": torch.empty(M, 2 * F // world, dtype=dtype, device=self.dev),
            # contiguous stand-ins for the attention output and the activation output of the fused variant
            "attn": torch.randn(M, H // world, device=self.dev, generator=gen).to(dtype),
            "act": torch.randn(M, F // world, device=self.dev, generator=gen).to(dtype),
        }

    def _lin(self, w, x, out):
        ops.w4a16_linear(x, w["qw"], w["sc"], w["zr"], group_size=GROUP, out=out, weight_layout=w["layout"])

    def _row(self, w, x, out):
        """Row-parallel linear + sum over ranks."""
        if self.comm is not None:
            ops.w4a16_linear_allreduce(x, w["qw"], w["sc"], w["zr"], self.comm, group_size=GROUP, out=out,
                                       weight_layout=w["layout"])
            return
        self._lin(w, x, out)
        if self.world > 1:
            dist.all_reduce(out, group=self.group)

    def close(self):
        if self.comm is not None:
            self.comm.close()
            self.comm = None

    def step(self) -> torch.Tensor:
        """One token step through all layers; returns the last hidden state buffer."""
        b = self.buf
        h = self.h
        for ly in self.layers:
            if self.fuse:
                self._lin(ly["qkv"], h, b["qkv"])
                self._row(ly["o"], b["attn"], b["o"])
                self._lin(ly["gate_up"], b["o"], b["gate_up"])
                self._row(ly["down"], b["act"], b["down"])
                h = b["down"]
                continue
            self._lin(ly["q"], h, b["q"])
            self._lin(ly["k"], h, b["k"])
            self._lin(ly["v"], h, b["v"])
            self._row(ly["o"], b["q"], b["o"])            # row-parallel: partial sums, summed over ranks
            self._lin(ly["gate"], b["o"], b["gate"])
            self._lin(ly["up"], b["o"], b["up"])
            self._row(ly["down"], b["gate"], b["down"])   # row-parallel: partial sums, summed over ranks
            h = b["down"]
        return h

    def capture(self) -> torch.cuda.CUDAGraph:
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            for _ in range(2):
                self.step()
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self.step()
        return g

    def launches_per_step(self) -> int:
        return (4 if self.fuse else 7) * self.L

    def bytes_per_step(self) -> int:
        """Algorithmic bytes of the whole (unsharded) token step."""
        H, KV, F, M = self.cfg["hidden"], self.cfg["kv"], self.cfg["ffn"], self.M
        per_layer = (2 * linear_bytes(M, H, H) + 2 * linear_bytes(M, H, KV) + 2 * linear_bytes(M, H, F) +
                     linear_bytes(M, F, H))
        return per_layer * self.L

"""The quantised linears of a decoder layer stack, run back to back: the "decode-linear us/token" workload.

Each layer has q (H->H), k, v (H->KV), o (H->H), gate, up (H->F), down (F->H). Only the linears run; attention,
norms and activations are outside the W4A16 path, so outputs are chained where shapes agree (q feeds o, o feeds
gate/up, gate feeds down, down feeds the next layer). With tensor parallelism q/k/v/gate/up are column-parallel
(outputs stay sharded) and o/down are row-parallel followed by a sum over the ranks, one process per GPU.
Weights are random int4 codes with the distributions of the benchmark configurations (shapes only, no checkpoint).

Modes
  fuse             q/k/v as ONE linear over the concatenated output rows and gate/up likewise (4 launches per
                   layer instead of 7; same weights, same bytes, same results)
  epilogues        (with fuse) gate/up runs with the SiLU * mul epilogue, so its output is the input of down, and
                   on one GPU o and down add the residual stream in their epilogue
  fused_allreduce  (world > 1, batch <= 64) the row-parallel o and down linears sum across ranks inside the kernel
                   over NVLink peer memory instead of being followed by an NCCL all-reduce
Batches of up to 8 rows read QF_LAYOUT_GEMV_SLAB weights (the streaming GEMV kernel), larger ones the
interleaved layout of the tcgen05 kernel.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.distributed as dist

from . import ops
from ._lib import QF_EPI_NONE, QF_EPI_RESIDUAL_ADD, QF_EPI_SILU_MUL, QF_LAYOUT_CANONICAL, QF_LAYOUT_INTERLEAVED

LLAMA3_8B = {"hidden": 4096, "kv": 1024, "ffn": 14336, "layers": 32}
LLAMA3_70B = {"hidden": 8192, "kv": 1024, "ffn": 28672, "layers": 80}
GROUP = 128
SLAB_BATCH = 8  # up to here the streaming GEMV kernel is the faster one (measured); beyond, the tcgen05 kernel
SAMPLE_COLUMNS = 64  # output columns per linear of layer 0 kept on the CPU for `check_parity`


def linear_bytes(M, K, N, out_bytes=2, out_cols=None):
    """Algorithmic bytes of one linear: codes + scales + zeros + X + Y."""
    G = K // GROUP
    return K * N // 2 + G * N * 2 + G * N // 2 + M * K * 2 + M * (out_cols if out_cols is not None else N) * out_bytes


class _Linear:
    """One quantised linear of the stack in the layout its kernel reads, plus (layer 0 only) a CPU copy of a few
    weight rows in canonical form for the parity check."""

    def __init__(self, N, K, dtype, dev, gen, batch, exchange: bool, silu: bool = False, sample: bool = False):
        self.N, self.K, self.silu = N, K, silu
        G = K // GROUP
        qw = torch.randint(-128, 128, (N, K // 2), dtype=torch.int8, device=dev, generator=gen)
        sc = (torch.randn(G, N, device=dev, generator=gen).abs() * (0.02 / 7.0)).clamp_min(2.0 ** -14).to(dtype)
        z8 = torch.randint(0, 16, (G, N), dtype=torch.int8, device=dev, generator=gen)
        self.sample = None
        if sample:
            n_out = N // 2 if silu else N
            cols = torch.randperm(n_out, generator=torch.Generator().manual_seed(N + K))[:SAMPLE_COLUMNS].sort().values
            if silu:  # output column j <- gate row (j // 8) * 16 + j % 8 and the up row 8 below it
                rows = torch.cat([(cols // 8) * 16 + cols % 8, (cols // 8) * 16 + cols % 8 + 8])
            else:
                rows = cols
            rd = rows.to(dev)
            self.sample = {"cols": cols.numpy(), "qweight": qw[rd].cpu().numpy(), "scales": sc[:, rd].float().cpu().numpy(),
                           "zeros": z8[:, rd].cpu().numpy()}
        zr = ops.pack_zeros_u4(z8)
        self.slab = None
        self.layout = QF_LAYOUT_CANONICAL
        if batch <= SLAB_BATCH and N % 64 == 0 and not exchange:
            self.slab = ops.prepack_gemv_slab(qw, sc, zr, GROUP)
            self.qw = self.sc = self.zr = None
        else:
            big = N * K // 2 >= (32 << 20)
            if (batch > 2 or big) and N % 128 == 0:
                qw = ops.prepack_w4(qw)
                self.layout = QF_LAYOUT_INTERLEAVED
            self.qw, self.sc, self.zr = qw, sc, zr

    def __call__(self, x, out, epilogue=QF_EPI_NONE, residual=None):
        if self.slab is not None:
            return ops.w4a16_linear(x, self.slab, out=out, out_dtype=out.dtype, epilogue=epilogue, residual=residual)
        return ops.w4a16_linear(x, self.qw, self.sc, self.zr, group_size=GROUP, out=out, out_dtype=out.dtype,
                                weight_layout=self.layout, epilogue=epilogue, residual=residual)


class DecodeLinearStack:
    def __init__(self, cfg: dict, batch: int, dtype=torch.bfloat16, device=None, world: int = 1, rank: int = 0,
                 group: Optional[dist.ProcessGroup] = None, layers: Optional[int] = None, seed: int = 0,
                 fuse: bool = False, fused_allreduce: bool = False, epilogues: bool = False,
                 exchange_in_slab_kernel: bool = True):
        """exchange_in_slab_kernel=False keeps the row-parallel linears of a fused_allreduce stack on the kernels
        that read canonical / interleaved weights (their last-arriving thread block exchanges each tile)."""
        self.cfg, self.M, self.dtype = cfg, batch, dtype
        self.dev = device or torch.device("cuda", torch.cuda.current_device())
        self.world, self.rank, self.group = world, rank, group
        self.L = layers or cfg["layers"]
        H, KV, F = cfg["hidden"], cfg["kv"], cfg["ffn"]
        assert H % world == 0 and KV % world == 0 and F % world == 0
        if epilogues and not fuse:
            raise ValueError("epilogues=True needs fuse=True (gate and up must be one linear)")
        gen = torch.Generator(device=self.dev)
        gen.manual_seed(seed + 7919 * rank)
        self.fuse, self.epilogues = fuse, epilogues
        self.residual = epilogues and world == 1
        self.comm = None
        if fused_allreduce and world > 1:
            if batch > 64:
                raise ValueError("fused_allreduce needs batch <= 64")
            self.comm = ops.Comm(batch * H, device=self.dev, group=group)
        exch = self.comm is not None and not exchange_in_slab_kernel
        self.layers = []
        for li in range(self.L):
            s = li == 0
            mk = lambda N, K, exchange=False, silu=False: _Linear(N, K, dtype, self.dev, gen, batch, exchange, silu, s)  # noqa: E731
            if fuse:
                self.layers.append({
                    "qkv": mk((H + 2 * KV) // world, H),
                    "o": mk(H, H // world, exch),
                    "gate_up": mk(2 * F // world, H, False, epilogues),
                    "down": mk(H, F // world, exch),
                })
            else:
                self.layers.append({
                    "q": mk(H // world, H), "k": mk(KV // world, H), "v": mk(KV // world, H),
                    "o": mk(H, H // world, exch),
                    "gate": mk(F // world, H), "up": mk(F // world, H),
                    "down": mk(H, F // world, exch),
                })
        M = batch
        self.h = torch.randn(M, H, device=self.dev, generator=torch.Generator(device=self.dev).manual_seed(seed + 1)).to(dtype)
        e = lambda *shape: torch.empty(*shape, dtype=dtype, device=self.dev)  # noqa: E731
        self.buf = {
            "q": e(M, H // world), "k": e(M, KV // world), "v": e(M, KV // world), "o": e(M, H),
            "gate": e(M, F // world), "up": e(M, F // world), "down": e(M, H),
            "qkv": e(M, (H + 2 * KV) // world), "gate_up": e(M, 2 * F // world),
            "h_in": e(M, H),  # the hidden state a token step starts from (step_host copies it in)
            # contiguous stand-ins for the attention output and the activation output of the fused variant
            "attn": torch.randn(M, H // world, device=self.dev, generator=gen).to(dtype),
            "act": torch.randn(M, F // world, device=self.dev, generator=gen).to(dtype),
        }
        self.buf["h_in"].copy_(self.h)
        self._graph = None
        self._h_host = None
        self._out_host = None

    # ------------------------------------------------------------------------------------------
    def _row(self, lin: _Linear, x, out, residual=None):
        """Row-parallel linear + sum over ranks (+ the residual stream on one GPU)."""
        if self.comm is not None:
            if lin.slab is not None:
                ops.w4a16_linear_allreduce(x, lin.slab, None, None, self.comm, out=out, out_dtype=out.dtype)
            else:
                ops.w4a16_linear_allreduce(x, lin.qw, lin.sc, lin.zr, self.comm, group_size=GROUP, out=out,
                                           out_dtype=out.dtype, weight_layout=lin.layout)
            return
        if residual is not None:
            lin(x, out, QF_EPI_RESIDUAL_ADD, residual)
        else:
            lin(x, out)
        if self.world > 1:
            dist.all_reduce(out, group=self.group)  # in the output's type (bf16 in the timed step, fp32 in the check)

    def close(self):
        self._graph = None
        if self.comm is not None:
            self.comm.close()
            self.comm = None

    def _layer(self, ly, h):
        b = self.buf
        if self.fuse:
            ly["qkv"](h, b["qkv"])
            self._row(ly["o"], b["attn"], b["o"], h if self.residual else None)
            if self.epilogues:
                ly["gate_up"](b["o"], b["act"], QF_EPI_SILU_MUL)
            else:
                ly["gate_up"](b["o"], b["gate_up"])
            self._row(ly["down"], b["act"], b["down"], b["o"] if self.residual else None)
            return b["down"]
        ly["q"](h, b["q"])
        ly["k"](h, b["k"])
        ly["v"](h, b["v"])
        self._row(ly["o"], b["q"], b["o"])            # row-parallel: partial sums, summed over ranks
        ly["gate"](b["o"], b["gate"])
        ly["up"](b["o"], b["up"])
        self._row(ly["down"], b["gate"], b["down"])   # row-parallel: partial sums, summed over ranks
        return b["down"]

    def step(self) -> torch.Tensor:
        """One token step through all layers, from buf["h_in"]; returns the last hidden state buffer."""
        h = self.buf["h_in"]
        for ly in self.layers:
            h = self._layer(ly, h)
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

    def step_host(self, h_host: torch.Tensor, out_host: torch.Tensor) -> torch.Tensor:
        """One token step for a caller whose hidden state lives in (pinned) host memory: copies it to the GPU, replays
        the captured step, copies the last hidden state back and waits. The same call on every rank of a tensor-
        parallel group; every rank ends with the full result."""
        if self._graph is None:
            self._graph = self.capture()
        self.buf["h_in"].copy_(h_host, non_blocking=True)
        self._graph.replay()
        out_host.copy_(self.buf["down"], non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return out_host

    def launches_per_step(self) -> int:
        return (4 if self.fuse else 7) * self.L

    def bytes_per_step(self) -> int:
        """Algorithmic bytes of the whole (unsharded) token step."""
        H, KV, F, M = self.cfg["hidden"], self.cfg["kv"], self.cfg["ffn"], self.M
        gate_up = (linear_bytes(M, H, 2 * F, out_cols=F) if self.epilogues else 2 * linear_bytes(M, H, F))
        per_layer = 2 * linear_bytes(M, H, H) + 2 * linear_bytes(M, H, KV) + gate_up + linear_bytes(M, F, H)
        if self.residual:
            per_layer += 2 * M * H * 2  # the residual stream read by o and down
        return per_layer * self.L

    # ------------------------------------------------------------------------------------------
    def check_parity(self, oracle_linear: Callable, silu_mul: Callable) -> dict:
        """Runs every linear of layer 0 through the call path `step` uses and compares SAMPLE_COLUMNS output columns
        with `oracle_linear(x, qweight_rows, scales, zeros, group) -> float array [M, rows]` (a CPU restatement the
        caller provides; this package has none). Row-parallel linears are compared after the sum over ranks, with
        the oracle's partial sums added across ranks in float64; every rank must also hold identical bits.
        The comparison is made on fp32 outputs of the same kernels (rounding an exact result to bf16 alone costs up
        to 1.3e-2 of the output's rms on layers this wide, more than the tolerance the path is specified with).
        Returns {"max_rel_err", "cases", "ranks_bit_identical"}; errors are max |y - ref| / rms(ref)."""
        import numpy as np
        b = self.buf
        ly = self.layers[0]
        M = self.M
        worst, cases, identical = 0.0, 0, True

        def ref_of(lin, x):
            s = lin.sample
            return oracle_linear(x.float().cpu().numpy(), s["qweight"], s["scales"], s["zeros"], GROUP)

        def err_of(y_cols, ref):
            rms = float(np.sqrt(np.mean(ref.astype(np.float64) ** 2)))
            return float(np.max(np.abs(y_cols.astype(np.float64) - ref)) / max(rms, 1e-30))

        def f32(t):
            return torch.empty(t.shape, dtype=torch.float32, device=t.device)

        def column(lin, x, buf, epilogue=QF_EPI_NONE):
            nonlocal worst, cases
            out = f32(buf)
            lin(x, out, epilogue)
            buf.copy_(out)  # the next linear of the layer reads it
            torch.cuda.synchronize()
            ref = ref_of(lin, x)
            if lin.silu:
                n = len(lin.sample["cols"])
                ref = silu_mul(ref[:, :n], ref[:, n:])
            y = out[:, torch.from_numpy(lin.sample["cols"]).to(out.device)].float().cpu().numpy()
            worst = max(worst, err_of(y, ref))
            cases += 1

        def row(lin, x, buf):
            nonlocal worst, cases, identical
            out = f32(buf)
            self._row(lin, x, out)
            buf.copy_(out)
            torch.cuda.synchronize()
            part = torch.from_numpy(np.ascontiguousarray(ref_of(lin, x), dtype=np.float64)).to(self.dev)
            if self.world > 1:
                dist.all_reduce(part, group=self.group)
                every = [torch.empty_like(out) for _ in range(self.world)]
                dist.all_gather(every, out.contiguous(), group=self.group)
                identical = identical and all(torch.equal(every[0], t) for t in every)
            y = out[:, torch.from_numpy(lin.sample["cols"]).to(out.device)].float().cpu().numpy()
            worst = max(worst, err_of(y, part.cpu().numpy()))
            cases += 1

        h = b["h_in"]
        if self.fuse:
            column(ly["qkv"], h, b["qkv"])
            row(ly["o"], b["attn"], b["o"])
            if self.epilogues:
                column(ly["gate_up"], b["o"], b["act"], QF_EPI_SILU_MUL)
            else:
                column(ly["gate_up"], b["o"], b["gate_up"])
            row(ly["down"], b["act"], b["down"])
        else:
            for name in ("q", "k", "v"):
                column(ly[name], h, b[name])
            row(ly["o"], b["q"], b["o"])
            column(ly["gate"], b["o"], b["gate"])
            column(ly["up"], b["o"], b["up"])
            row(ly["down"], b["gate"], b["down"])
        if self.world > 1:
            t = torch.tensor([worst, 0.0 if identical else 1.0], device=self.dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.group)
            worst, identical = float(t[0].item()), bool(t[1].item() == 0.0)
        return {"max_rel_err": worst, "cases": cases, "ranks_bit_identical": identical}

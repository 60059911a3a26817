#!/usr/bin/env python
"""Benchmark of the W4A16 hot path (INT4 unpack + dequant fused into GEMV / GEMM) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload stack70b|stack8b|sweep]

One JSON line on stdout (rank 0).

Default workload `stack70b`: the decode linears of a Llama-3-70B-shaped stack (80 layers of q/k/v 8192->10240 as one
linear, o 8192->8192, gate/up 8192->57344 as one linear, down 28672->8192; int4 g128 weights, asymmetric uint4
zeros, bf16 activations), batch 1. A step is one token step through all 320 linears (35.6 GB of weights, far above
L2), captured once as a CUDA graph. With N > 1 ranks the same stack runs tensor parallel: q/k/v/gate/up column-
parallel, o/down row-parallel with the sum over ranks inside the GEMV kernel over NVLink peer memory
(--nccl-collectives: an NCCL all-reduce after the linear instead). Total work is fixed: strong scaling.
`value` = algorithmic bytes of the whole token step / time (GB/s, all GPUs together).

`--workload sweep`: the batched GEMV / small-GEMM sweep, M in {1,4,8,16,64} x (K,N) in
{(4096,4096),(4096,14336),(14336,4096)}, 15 linears per step on 15 weight copies.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GROUP = 128
LAYOUT_CANONICAL, LAYOUT_INTERLEAVED = 0, 1
SWEEP_SHAPES = [(4096, 4096), (4096, 14336), (14336, 4096)]
SWEEP_MS = [1, 4, 8, 16, 64]
TIMED_BATCHES = 25  # the K-step bracket is repeated this often; the median is reported


def algo_bytes(M, K, N, out_bytes=2, zeros=True, group=GROUP):
    """Algorithmic bytes of one linear: codes + scales + zeros + X + Y (scratch and re-reads do not count)."""
    G = K // group
    return K * N // 2 + G * N * 2 + (G * N // 2 if zeros else 0) + M * K * 2 + M * N * out_bytes


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
                "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


# ------------------------------------------------------------------------------------------------
# clocks
# ------------------------------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.lines = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        # samples under load = upper half (the sampler also sees idle moments at both ends)
        sm_sorted = sorted(sm)
        under_load = sm_sorted[len(sm_sorted) // 2:]
        return {"sm_mhz": statistics.median(under_load), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm)}


# ------------------------------------------------------------------------------------------------
# CPU arm (the oracle's C port, timed on the host cores): cpu_baseline leg and --impl reference
# ------------------------------------------------------------------------------------------------
STACKS = {"stack8b": ("cfg2_llama3_8b_decode_linears", {"hidden": 4096, "kv": 1024, "ffn": 14336, "layers": 32}),
          "stack70b": ("cfg4_llama3_70b_decode_linears", {"hidden": 8192, "kv": 1024, "ffn": 28672, "layers": 80})}


def stack_layer_shapes(cfg, fuse=True):
    """(N, K) of the linears of one layer, in launch order."""
    H, KV, F = cfg["hidden"], cfg["kv"], cfg["ffn"]
    if fuse:
        return [(H + 2 * KV, H), (H, H), (2 * F, H), (H, F)]
    return [(H, H), (KV, H), (KV, H), (H, H), (F, H), (F, H), (H, F)]


def stack_config(workload, batch, layers, fuse):
    """The `config` object both arms print (what is computed; how it is run goes to `detail`)."""
    name, cfg = STACKS[workload]
    return {"workload": name, "batch": batch, "layers": layers or cfg["layers"], "group_size": GROUP,
            "zeros": "uint4 per (group,n)", "act_dtype": "bf16", "out_dtype": "bf16",
            "fused_qkv_gate_up": bool(fuse)}


class CpuLayer:
    """One layer of the stack on the host, for the C port of the reference arithmetic (seeded, same distributions)."""

    def __init__(self, cfg, batch, fuse=True):
        import numpy as np
        from oracle import c_oracle, qf_oracle as O
        self.c_oracle = c_oracle
        self.batch = batch
        self.linears = []
        rng = np.random.default_rng(17)
        for (N, K) in stack_layer_shapes(cfg, fuse):
            qw = rng.integers(0, 256, size=(N, K // 2), dtype=np.uint8)
            sc = np.maximum(np.abs(rng.normal(0, 0.02, size=(K // GROUP, N))) / 7.0, 2.0 ** -14).astype(np.float32)
            sc16 = c_oracle.to_bits(O.round_to(sc, "bf16"), "bf16")
            zw = rng.integers(0, 2 ** 32, size=(K // GROUP, N // 8), dtype=np.uint32)
            x16 = c_oracle.to_bits(O.round_to(rng.normal(size=(batch, K)).astype(np.float32), "bf16"), "bf16")
            self.linears.append((x16, qw, sc16, zw, N, K))
        self.bytes = sum(algo_bytes(batch, K, N) for (_x, _q, _s, _z, N, K) in self.linears)

    def run(self):
        t0 = time.perf_counter()
        for (x16, qw, sc16, zw, _N, _K) in self.linears:
            self.c_oracle.w4a16_linear(x16, qw, sc16, zw, GROUP, "bf16", "bf16")
        return time.perf_counter() - t0


def cpu_threads_all():
    """Use every host core, whatever a launcher exported (torchrun sets OMP_NUM_THREADS=1 for N > 1)."""
    from oracle import c_oracle
    n = os.cpu_count() or 1
    try:
        n = len(os.sched_getaffinity(0))
    except (AttributeError, OSError):
        pass
    c_oracle.set_num_threads(n)
    return c_oracle.num_threads()


def run_reference_arm(args):
    """The reference's arithmetic on the host cores (C port of the oracle; the reference itself ships no runnable
    lowering and its Python script needs the reference checkout, which is absent on the GPU box). Each step is a
    bounded sample of the arm's workload: one layer of the stack (every linear of the layer, same shapes, batch and
    dtypes); the rate does not depend on which layer runs."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import c_oracle
    c_oracle.lib()
    threads = cpu_threads_all()
    workload = args.workload if args.workload in STACKS else "stack70b"
    _name, cfg = STACKS[workload]
    fuse = not args.no_fuse
    layer = CpuLayer(cfg, args.batch, fuse)
    layers = args.layers or cfg["layers"]
    for _ in range(args.warmup):
        layer.run()
    secs = [layer.run() for _ in range(args.steps)]
    total_s = sum(secs)
    gbs = layer.bytes * args.steps / total_s / 1e9
    sample = (f"one of the {layers} layers per step ({len(layer.linears)} linears, {layer.bytes / 1e6:.0f} MB "
              f"algorithmic), {args.steps} steps")
    line = {
        "impl": "reference", "metric": "w4a16_linear_hbm_gbs", "value": gbs, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": total_s / args.steps * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": stack_config(workload, args.batch, args.layers, fuse),
        "detail": {"step": sample, "us_per_token_extrapolated": layer.bytes * layers / (gbs * 1e9) * 1e6,
                   "omp_threads": threads, "host_cores": os.cpu_count()},
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# helpers of the GPU arm
# ------------------------------------------------------------------------------------------------
class Env:
    """Process-wide handles of the GPU arm."""

    def __init__(self, torch, dist, qf, dev, world, rank, local_rank, pk):
        self.torch, self.dist, self.qf, self.dev = torch, dist, qf, dev
        self.world, self.rank, self.local_rank, self.pk = world, rank, local_rank, pk

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, values):
        if self.world == 1:
            return list(values)
        t = self.torch.tensor(list(values), device=self.dev, dtype=self.torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return [float(v) for v in t.tolist()]


def time_graph_batches(env, g, steps, warmup, batches):
    """`batches` brackets of exactly `steps` replays, each between a barrier + synchronize on both sides and timed
    with CUDA events on the launching stream; per bracket the max over ranks. Returns ms per bracket."""
    torch = env.torch
    for _ in range(warmup):
        g.replay()
    out = []
    for _ in range(batches):
        env.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            g.replay()
        e1.record()
        env.barrier()
        out.append(e0.elapsed_time(e1))
    return env.max_over_ranks(out)


def oracle_linear(x, qweight_rows, scales, zeros, group):
    """Checker handed to DecodeLinearStack.check_parity: the numpy restatement of the reference arithmetic."""
    from oracle import qf_oracle as O
    return O.w4a16_linear(x, qweight_rows, scales, zeros, group, "bf16", O.F32, accumulate="f64")


def oracle_silu_mul(gate, up):
    from oracle import qf_oracle as O
    return O.silu_mul(gate, up)


# ------------------------------------------------------------------------------------------------
# single-GPU extras: the sweep per case, cfg0, cfg2, cfg3, K1 bandwidth
# ------------------------------------------------------------------------------------------------
def time_case(env, M, K, N, act, out_dt, sym, sigma, slab, copies=None, reps=5, gen=None, stream_only=False):
    """One linear as a CUDA graph of one launch per weight copy, with enough copies (>= 300 MB) that every launch
    reads its weights from HBM; the figure is the average launch-to-launch time inside the graph (best of `reps`)."""
    torch, qf, dev = env.torch, env.qf, env.dev
    wbytes = K * N // 2
    n = copies or max(3, -(-300_000_000 // wbytes))
    G = K // GROUP
    use_slab = slab and M <= 8 and N % 64 == 0
    layout = LAYOUT_INTERLEAVED if ((M > 2 or N * K // 2 >= (32 << 20)) and N % 128 == 0) else LAYOUT_CANONICAL
    sets = []
    for _ in range(n):
        qw = torch.randint(-128, 128, (N, K // 2), dtype=torch.int8, device=dev, generator=gen)
        sc = (torch.randn(G, N, device=dev, generator=gen).abs() * (sigma / 7.0)).clamp_min(2.0 ** -14).to(act)
        zr = None if sym else qf.pack_zeros_u4(
            torch.randint(0, 16, (G, N), dtype=torch.int8, device=dev, generator=gen))
        if use_slab:
            sets.append((qf.prepack_gemv_slab(qw, sc, zr, GROUP, 8), None, None))
        else:
            if layout != LAYOUT_CANONICAL:
                qw = qf.prepack_w4(qw, layout=layout)
            sets.append((qw, sc, zr))
    x = torch.randn(M, K, device=dev, generator=gen).to(act)
    y = torch.empty(M, N, dtype=out_dt, device=dev)

    def run(i):
        qw, sc, zr = sets[i]
        if use_slab:
            qf.w4a16_linear(x, qw, out=y, out_dtype=out_dt)
        else:
            qf.w4a16_linear(x, qw, sc, zr, group_size=GROUP, zero_const=8, out=y, out_dtype=out_dt,
                            weight_layout=layout)
    if stream_only:
        # measurement mode of the slab kernel (read at launch, i.e. at capture): weights go through the copy pipeline,
        # nothing is converted or multiplied - the ceiling the weight stream alone allows in this very harness
        os.environ["QF_SLAB_STREAM_ONLY"] = "1"
    try:
        run(0)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for i in range(n):
                run(i)
    finally:
        os.environ.pop("QF_SLAB_STREAM_ONLY", None)
    best = None
    for it in range(reps + 2):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        if it >= 2:
            t = e0.elapsed_time(e1) * 1e3 / n
            best = t if best is None else min(best, t)
    del sets, g
    return best


def time_streaming(env, fn, in_bytes_per_call, reps=5):
    """A streaming kernel (unpack / dequant) on inputs that rotate over > L2 worth of data; best time per call (us)."""
    torch = env.torch
    n = len(fn)
    for f in fn:
        f()
    torch.cuda.synchronize()
    best = None
    for it in range(reps + 1):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for f in fn:
            f()
        e1.record()
        torch.cuda.synchronize()
        if it >= 1:
            t = e0.elapsed_time(e1) * 1e3 / n
            best = t if best is None else min(best, t)
    return best


def single_gpu_extras(env, args):
    torch, qf, dev, pk = env.torch, env.qf, env.dev, env.pk
    gen = torch.Generator(device=dev)
    gen.manual_seed(4321)
    detail, extra = [], {}
    hbm = pk["hbm_gbs"]
    for (K, N) in SWEEP_SHAPES:
        for M in SWEEP_MS:
            us = time_case(env, M, K, N, torch.bfloat16, torch.bfloat16, False, 0.02, True, gen=gen)
            b = algo_bytes(M, K, N)
            detail.append({"M": M, "K": K, "N": N, "us": round(us, 2), "gbs": round(b / us / 1e3, 1),
                           "frac_hbm": round(b / us / 1e3 / hbm, 3), "kernel": "gemv_slab" if M <= 8 else "gemm_tcgen05"})
    b = algo_bytes(1, 4096, 4096)
    us = time_case(env, 1, 4096, 4096, torch.float16, torch.float16, False, 0.02, True, gen=gen)
    us_old = time_case(env, 1, 4096, 4096, torch.float16, torch.float16, False, 0.02, False, gen=gen)
    us_read = time_case(env, 1, 4096, 4096, torch.float16, torch.float16, False, 0.02, True, gen=gen, stream_only=True)
    extra["cfg0_gemv_m1_4096x4096_f16"] = {
        "us": round(us, 2), "gbs": round(b / us / 1e3, 1), "frac_hbm": round(b / us / 1e3 / hbm, 3),
        "kernel": "qf::gemv_slab_kernel (prepacked slab)",
        "canonical_weights_gemv_kernel_us": round(us_old, 2),
        "weight_stream_only_us": round(us_read, 2),
        "weight_stream_only_frac_hbm": round(b / us_read / 1e3 / hbm, 3),
        "note": "weight_stream_only = the same launches in the same graph with the kernel moving its bytes through "
                "the bulk-copy pipeline and doing no arithmetic: the ceiling of a dependent-launch GEMV of this size"}
    bb = algo_bytes(1, 8192, 57344)
    us_big = time_case(env, 1, 8192, 57344, torch.bfloat16, torch.bfloat16, False, 0.02, True, copies=2, gen=gen)
    us_big_read = time_case(env, 1, 8192, 57344, torch.bfloat16, torch.bfloat16, False, 0.02, True, copies=2, gen=gen,
                            stream_only=True)
    extra["gemv_m1_8192x57344_bf16_70b_gate_up"] = {
        "us": round(us_big, 2), "gbs": round(bb / us_big / 1e3, 1), "frac_hbm": round(bb / us_big / 1e3 / hbm, 3),
        "weight_stream_only_us": round(us_big_read, 2),
        "weight_stream_only_frac_hbm": round(bb / us_big_read / 1e3 / hbm, 3)}
    from quantforge_b200 import stack as S
    for bsz in (1, 16):
        for mode in ("fused", "fused_epilogues"):
            st = S.DecodeLinearStack(S.LLAMA3_8B, bsz, torch.bfloat16, dev, fuse=True, epilogues=mode == "fused_epilogues")
            g = st.capture()
            ms = statistics.median(time_graph_batches(env, g, 20, 3, 5)) / 20
            nb = st.bytes_per_step()
            extra[f"cfg2_llama3_8b_decode_linears_batch{bsz}_{mode}"] = {
                "us_per_token": round(ms * 1e3, 1), "gbs": round(nb / ms / 1e6, 1),
                "frac_hbm": round(nb / ms / 1e6 / hbm, 3), "launches": st.launches_per_step()}
            del g
            st.close()
            del st
            torch.cuda.empty_cache()
    us = time_case(env, 2048, 8192, 28672, torch.bfloat16, torch.bfloat16, True, 0.01, False, copies=2, reps=3, gen=gen)
    tf = 2.0 * 2048 * 8192 * 28672 / us / 1e6
    extra["cfg3_gemm_m2048_k8192_n28672_bf16_sym"] = {
        "us": round(us, 1), "tflops": round(tf, 1), "frac_bf16_burst": round(tf / pk["bf16_tflops"], 3),
        "frac_bf16_sustained": round(tf / pk["bf16_tflops_sustained"], 3)}
    # K1: qf.unpack and the materialising qf.dequant as stand-alone streaming kernels (HBM roofline).
    # bytes: unpack 1 B read + 2 B written per packed byte; dequant 0.5 B read + 2 B written per weight (+ scales, zeros)
    for name, (Nn, Kk) in (("cfg0_4096x4096", (4096, 4096)), ("cfg3_28672x8192", (28672, 8192))):
        copies = max(2, -(-400_000_000 // (Nn * Kk * 2)))
        packed = [torch.randint(-128, 128, (Nn, Kk // 2), dtype=torch.int8, device=dev, generator=gen) for _ in range(copies)]
        us = time_streaming(env, [(lambda p=p: qf.unpack_int4(p)) for p in packed], Nn * Kk // 2)
        bts = Nn * Kk // 2 * 3
        extra[f"k1_unpack_{name}"] = {"us": round(us, 1), "gbs": round(bts / us / 1e3, 1),
                                      "frac_hbm": round(bts / us / 1e3 / hbm, 3)}
        sc = (torch.randn(Kk // GROUP, Nn, device=dev, generator=gen).abs() * (0.02 / 7)).clamp_min(2.0 ** -14).to(torch.bfloat16)
        zr = qf.pack_zeros_u4(torch.randint(0, 16, (Kk // GROUP, Nn), dtype=torch.int8, device=dev, generator=gen))
        us = time_streaming(env, [(lambda p=p: qf.dequant_w4(p, sc, zr, GROUP)) for p in packed], Nn * Kk // 2)
        bts = Nn * Kk // 2 + Nn * Kk * 2 + (Kk // GROUP) * Nn * 5 // 2
        extra[f"k1_dequant_{name}"] = {"us": round(us, 1), "gbs": round(bts / us / 1e3, 1),
                                       "frac_hbm": round(bts / us / 1e3 / hbm, 3)}
        del packed
        torch.cuda.empty_cache()
    return detail, extra


def cfg3_tensor_parallel_extra(env):
    """cfg3 sharded: the prefill GEMM (M=2048, K=8192, N=28672) column-parallel over the ranks + NCCL all-gather of
    the outputs; device time of the GEMM alone, the gather alone and both, max over ranks."""
    torch, qf, dist, dev, world = env.torch, env.qf, env.dist, env.dev, env.world
    M, K, N = 2048, 8192, 28672
    Nl = N // world
    gen = torch.Generator(device=dev)
    gen.manual_seed(99 + env.rank)
    qw = qf.prepack_w4(torch.randint(-128, 128, (Nl, K // 2), dtype=torch.int8, device=dev, generator=gen))
    sc = (torch.randn(K // GROUP, Nl, device=dev, generator=gen).abs() * (0.01 / 7)).clamp_min(2.0 ** -14).to(torch.bfloat16)
    x = torch.randn(M, K, device=dev, generator=torch.Generator(device=dev).manual_seed(5)).to(torch.bfloat16)
    y = torch.empty(M, Nl, dtype=torch.bfloat16, device=dev)
    yg = torch.empty(world, M, Nl, dtype=torch.bfloat16, device=dev)

    def gemm():
        qf.w4a16_linear(x, qw, sc, None, group_size=GROUP, zero_const=8, out=y, weight_layout=LAYOUT_INTERLEAVED)

    def gather():
        dist.all_gather_into_tensor(yg, y)

    def timed(fns, reps=10):
        for f in fns:
            f()
        env.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            for f in fns:
                f()
        e1.record()
        env.barrier()
        return env.max_over_ranks([e0.elapsed_time(e1) * 1e3 / reps])[0]

    t_gemm, t_gather, t_both = timed([gemm]), timed([gather]), timed([gemm, gather])
    # parity of the sharded result: a few gathered columns of this rank against the numpy oracle is covered by the
    # single-GPU tests; here every rank checks that its gathered copy of rank 0's shard equals rank 0's own output
    ref = y.clone() if env.rank == 0 else torch.empty_like(y)
    dist.broadcast(ref, 0)
    same = bool(torch.equal(yg[0], ref))
    flops = 2.0 * M * K * N
    return {"gemm_us": round(t_gemm, 1), "all_gather_us": round(t_gather, 1), "gemm_plus_gather_us": round(t_both, 1),
            "tflops_whole_job_gemm_only": round(flops / t_gemm / 1e6, 1),
            "tflops_whole_job_with_gather": round(flops / t_both / 1e6, 1),
            "gather_bytes_received_per_rank": (world - 1) * M * Nl * 2, "gathered_shard_matches_rank0": same}


# ------------------------------------------------------------------------------------------------
# decode-linear stack workloads (Llama-3-8B / 70B shaped layers, tensor parallel over the ranks)
# ------------------------------------------------------------------------------------------------
def run_stack_workload(env, args):
    from quantforge_b200 import stack as S
    torch, qf, dist, dev, world, rank, pk = env.torch, env.qf, env.dist, env.dev, env.world, env.rank, env.pk
    _name, cfg = STACKS[args.workload]
    fuse = not args.no_fuse
    in_kernel = world > 1 and not args.nccl_collectives and args.batch <= 64
    st = S.DecodeLinearStack(cfg, args.batch, torch.bfloat16, dev, world, rank, None, args.layers or None,
                             fuse=fuse, fused_allreduce=in_kernel, epilogues=args.epilogues,
                             exchange_in_slab_kernel=not args.legacy_exchange_kernels)
    # ---- parity before anything is timed: layer 0, every linear, sampled columns, against the CPU oracle ----
    parity = st.check_parity(oracle_linear, oracle_silu_mul)
    parity["tolerance"] = 1e-2
    parity["ok"] = bool(parity["max_rel_err"] < 1e-2 and parity["ranks_bit_identical"] and
                        qf.device_status(dev) == 0)
    parity["checked"] = ("every linear of layer 0 through the call path of the timed step, 64 sampled output columns "
                         "each, against the numpy restatement of the reference arithmetic (fp64 accumulation); "
                         "row-parallel linears after the sum over ranks, all ranks compared bit for bit")
    if not parity["ok"]:
        if rank == 0:
            print(json.dumps({"error": "parity check failed", "parity": parity}), flush=True)
        st.close()
        raise SystemExit(3)

    g = st.capture()
    sampler = ClockSampler(env.local_rank)
    if rank == 0:
        sampler.start()
    per_bracket = time_graph_batches(env, g, args.steps, args.warmup, TIMED_BATCHES)
    clocks = sampler.stop() if rank == 0 else None
    ms_bracket = statistics.median(per_bracket)
    ms = ms_bracket / args.steps
    nbytes = st.bytes_per_step()
    launches_per_step = st.launches_per_step()

    # ---- end to end: the hidden state comes from pinned host memory and the last hidden state goes back, every step ----
    H = cfg["hidden"]
    h_host = torch.randn(args.batch, H).to(torch.bfloat16).pin_memory()
    out_host = torch.empty(args.batch, H, dtype=torch.bfloat16).pin_memory()
    st._graph = g
    e2e_steps = max(3, min(args.steps, 50))
    for _ in range(3):
        st.step_host(h_host, out_host)
    env.barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        st.step_host(h_host, out_host)
    e2e_ms = (time.perf_counter() - t0) * 1e3 / e2e_steps
    env.barrier()
    e2e_ms = env.max_over_ranks([e2e_ms])[0]
    e2e = {"value": nbytes / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s", "h2d_bytes_per_step": args.batch * H * 2,
           "d2h_bytes_per_step": args.batch * H * 2, "ms_per_step": e2e_ms, "steps": e2e_steps,
           "us_per_token": e2e_ms * 1e3,
           "note": "DecodeLinearStack.step_host: hidden state from pinned host memory to the GPU, the captured token "
                   "step, last hidden state back to pinned host memory, stream synchronised, every step (host clock); "
                   "with N > 1 every rank does the same and ends with the full result"}

    detail_cases, extra = [], {}
    if not args.no_extras:
        if world == 1:
            # free the stack first: the extras allocate their own weights
            st._graph = None
            del g
            st.close()
            del st
            torch.cuda.empty_cache()
            st = None
            detail_cases, extra = single_gpu_extras(env, args)
        else:
            extra["cfg3_tp_prefill_gemm_column_parallel_nccl_all_gather"] = cfg3_tensor_parallel_extra(env)

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        threads = cpu_threads_all()
        layer = CpuLayer(cfg, args.batch, fuse)
        layer.run()
        s, passes = 0.0, 0
        while s < 12.0 and passes < 400:
            s += layer.run()
            passes += 1
        cpu_baseline = {"value": layer.bytes * passes / s / 1e9, "unit": "GB/s", "cores": threads, "kind": "port",
                        "sample": f"{passes} passes over one layer of the stack ({len(layer.linears)} linears, "
                                  f"{layer.bytes / 1e6:.0f} MB algorithmic; {s:.1f} s of CPU time)"}

    if rank == 0:
        gbs = nbytes / (ms * 1e-3) / 1e9
        per_launch_us = ms * 1e3 / launches_per_step
        kernel = "qf::gemv_slab_kernel" if args.batch <= 8 else "qf::gemm_kernel (tcgen05)"
        if in_kernel and args.batch <= 8:
            kernel += " + qf::gemv_slab_exch_kernel (row-parallel linears)"
        line = {
            "metric": "w4a16_linear_hbm_gbs", "value": gbs, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": stack_config(args.workload, args.batch, args.layers, fuse),
            "us_per_token": ms * 1e3,
            "detail": {
                "parallelism": "single GPU" if world == 1 else
                f"tensor parallel x{world}: column q/k/v/gate/up, row o/down + " +
                ("sum over ranks inside the GEMV kernel over NVLink peer memory (fp32 partials)"
                 if in_kernel else "NCCL all-reduce (bf16)"),
                "epilogues": bool(args.epilogues),
                "l2": f"weights of the step: {nbytes / 1e9:.2f} GB, far above L2",
                "timing": f"CUDA graph of one token step; {TIMED_BATCHES} brackets of exactly {args.steps} replays, "
                          "each between barrier + synchronize, CUDA events on the launching stream, max over ranks per "
                          "bracket, median bracket reported",
                "ms_per_step_min": min(per_bracket) / args.steps, "ms_per_step_max": max(per_bracket) / args.steps,
                "timed_region_s": sum(per_bracket) * 1e-3,
                "clock_sampling": "during the timed brackets"},
            "roofline": {"bound": "hbm", "kernel": kernel, "achieved": gbs / world, "peak": pk["hbm_gbs"],
                         "unit": "GB/s", "frac": gbs / world / pk["hbm_gbs"],
                         "traffic": nbytes / world / launches_per_step * 1.03,
                         "traffic_note": "algorithmic bytes per launch x 1.03, the DRAM/algorithmic ratio ncu measured "
                                         "on one captured launch of this kernel (profiles/): the slab layout stores a "
                                         "(constant, scale) pair per row and 128 codes",
                         "peak_source": pk["source"], "avg_launch_us": per_launch_us,
                         "launches_per_step": launches_per_step,
                         "algorithmic_bytes_per_launch": nbytes / world / launches_per_step,
                         "per_gpu": True},
            "parity": parity, "cpu_baseline": cpu_baseline, "e2e": e2e,
            "gpu_launches": launches_per_step * args.steps,
            "gpu_launches_all_brackets": launches_per_step * args.steps * TIMED_BATCHES, "clocks": clocks,
        }
        if detail_cases:
            line["cases"] = detail_cases
        if extra:
            line["extra"] = extra
        print(json.dumps(line), flush=True)
    if st is not None:
        st._graph = None
        del g
        st.close()


# ------------------------------------------------------------------------------------------------
# the sweep workload (15 linears per step)
# ------------------------------------------------------------------------------------------------
def run_sweep_workload(env, args):
    torch, qf, dist, dev, world, rank, pk = env.torch, env.qf, env.dist, env.dev, env.world, env.rank, env.pk
    gen = torch.Generator(device=dev)
    gen.manual_seed(1234 + rank)
    cases = []
    for (K, N) in SWEEP_SHAPES:
        assert N % world == 0
        Nl = N // world
        G = K // GROUP
        for M in SWEEP_MS:
            qw = torch.randint(-128, 128, (Nl, K // 2), dtype=torch.int8, device=dev, generator=gen)
            sc = (torch.randn(G, Nl, device=dev, generator=gen).abs() * (0.02 / 7.0)).clamp_min(2.0 ** -14).to(
                torch.bfloat16)
            zr = qf.pack_zeros_u4(torch.randint(0, 16, (G, Nl), dtype=torch.int8, device=dev, generator=gen))
            slab = None
            layout = LAYOUT_CANONICAL
            if M <= 8 and Nl % 64 == 0:
                slab = qf.prepack_gemv_slab(qw, sc, zr, GROUP)
            elif Nl % 128 == 0:
                qw = qf.prepack_w4(qw, layout=LAYOUT_INTERLEAVED)
                layout = LAYOUT_INTERLEAVED
            x = torch.randn(M, K, device=dev, generator=torch.Generator(device=dev).manual_seed(M + K)).to(torch.bfloat16)
            y = torch.empty(M, Nl, dtype=torch.bfloat16, device=dev)
            yg = torch.empty(M, world * Nl, dtype=torch.bfloat16, device=dev) if world > 1 else None
            ygt = torch.empty(world, M, Nl, dtype=torch.bfloat16, device=dev) if world > 1 else None  # rank-major
            cases.append({"M": M, "K": K, "N": N, "Nl": Nl, "layout": layout, "slab": slab, "qw": qw, "sc": sc,
                          "zr": zr, "x": x, "y": y, "yg": yg, "ygt": ygt})
    total_bytes = sum(algo_bytes(c["M"], c["K"], c["N"]) for c in cases)  # whole job, all ranks
    comm = None
    if world > 1 and not args.nccl_collectives:
        comm = qf.Comm(max(SWEEP_MS) * max(N for (_, N) in SWEEP_SHAPES) // world, device=dev)

    def launch(c):
        if comm is not None:
            if c["slab"] is not None:
                qf.w4a16_linear_allgather(c["x"], c["slab"], None, None, comm, out=c["yg"])
            else:
                qf.w4a16_linear_allgather(c["x"], c["qw"], c["sc"], c["zr"], comm, group_size=GROUP, out=c["yg"],
                                          weight_layout=c["layout"])
            return
        if c["slab"] is not None:
            qf.w4a16_linear(c["x"], c["slab"], out=c["y"])
        else:
            qf.w4a16_linear(c["x"], c["qw"], c["sc"], c["zr"], group_size=GROUP, out=c["y"], weight_layout=c["layout"])
        if world > 1:
            dist.all_gather_into_tensor(c["ygt"], c["y"])

    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        for _ in range(3):
            for c in cases:
                launch(c)
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for c in cases:
            launch(c)
    sampler = ClockSampler(env.local_rank)
    if rank == 0:
        sampler.start()
    per_bracket = time_graph_batches(env, g, args.steps, args.warmup, TIMED_BATCHES)
    clocks = sampler.stop() if rank == 0 else None
    ms = statistics.median(per_bracket) / args.steps
    if rank == 0:
        gbs = total_bytes / (ms * 1e-3) / 1e9
        line = {
            "metric": "w4a16_linear_hbm_gbs", "value": gbs, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "cfg1_sweep", "cases": "M in {1,4,8,16,64} x (K,N) in {(4096,4096),(4096,14336),(14336,4096)}",
                       "group_size": GROUP, "zeros": "uint4 per (group,n)", "out_dtype": "bf16"},
            "detail": {"parallelism": "single GPU" if world == 1 else
                       (f"column-parallel x{world}, outputs gathered inside the kernels over NVLink peer memory"
                        if comm is not None else f"column-parallel x{world} + NCCL all-gather"),
                       "l2": "inputs larger than L2: 15 weight copies, 335 MB touched per step",
                       "timed_region_s": sum(per_bracket) * 1e-3},
            "roofline": {"bound": "hbm", "kernel": "whole step (slab GEMV for M <= 8, tcgen05 for M = 16, 64)",
                         "achieved": gbs / world, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": gbs / world / pk["hbm_gbs"],
                         "traffic": None, "peak_source": pk["source"]},
            "cpu_baseline": None, "e2e": None, "gpu_launches": len(cases) * args.steps, "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    del g
    if comm is not None:
        comm.close()


# ------------------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="stack70b", choices=["stack70b", "stack8b", "sweep"])
    ap.add_argument("--batch", type=int, default=1, help="batch rows for the stack workloads")
    ap.add_argument("--layers", type=int, default=0, help="override the number of layers of a stack workload")
    ap.add_argument("--no-fuse", action="store_true", help="stack workloads: seven launches per layer instead of four")
    ap.add_argument("--epilogues", action="store_true",
                    help="stack workloads: SiLU*mul inside gate/up and (one GPU) the residual adds inside o / down")
    ap.add_argument("--nccl-collectives", action="store_true",
                    help="N > 1 GPUs: follow each linear with an NCCL collective instead of exchanging in-kernel")
    ap.add_argument("--legacy-exchange-kernels", action="store_true",
                    help="N > 1: row-parallel linears exchange inside the canonical-weight kernels, not the slab kernel")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3

    if args.impl == "reference":
        run_reference_arm(args)
        return

    import torch
    import torch.distributed as dist

    import quantforge_b200 as qf

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (the product has no CPU path)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        import datetime
        # a short collective timeout turns a rank mismatch into an error instead of a hang
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=300))
    env = Env(torch, dist, qf, dev, world, rank, local_rank, peaks())
    try:
        if args.workload == "sweep":
            run_sweep_workload(env, args)
        else:
            run_stack_workload(env, args)
    finally:
        if world > 1:
            import gc
            gc.collect()
            torch.cuda.synchronize()
            try:
                dist.barrier()
            except Exception:  # noqa: BLE001 - a failed rank must not mask the first error
                pass
            dist.destroy_process_group()


if __name__ == "__main__":
    main()

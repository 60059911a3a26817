"""Run one W4A16 linear configuration on the GPU and print its device time (for profiling a single kernel).

    python run_case.py --M 1 --K 4096 --N 14336 --act bf16 [--iters 5] [--copies 6] [--sym]

Inputs are seeded synthetic tensors (uniform uint4 codes, |N(0,0.02)|/7 scales, uniform uint4 zeros or the
constant 8 with --sym, N(0,1) activations).  `--copies` weight sets are rotated so that, with copies x weight
bytes above the 126 MB L2, every launch reads its weights from HBM.
"""
from __future__ import annotations

import argparse
import json

import torch

import quantforge_b200 as qf
from quantforge_b200._lib import QF_PATH_AUTO, QF_PATH_GEMM, QF_PATH_GEMV


def make_case(M, K, N, act, dev, sym=False, sigma=0.02, group=128, seed=0):
    gen = torch.Generator(device=dev)
    gen.manual_seed(seed)
    G = K // group
    qw = torch.randint(-128, 128, (N, K // 2), dtype=torch.int8, device=dev, generator=gen)
    sc = (torch.randn(G, N, device=dev, generator=gen).abs() * (sigma / 7.0)).clamp_min(2.0 ** -14).to(act)
    zr = None if sym else qf.pack_zeros_u4(torch.randint(0, 16, (G, N), dtype=torch.int8, device=dev, generator=gen))
    x = torch.randn(M, K, device=dev, generator=gen).to(act)
    return qw, sc, zr, x


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--M", type=int, default=1)
    ap.add_argument("--K", type=int, default=4096)
    ap.add_argument("--N", type=int, default=4096)
    ap.add_argument("--act", default="bf16", choices=["f16", "bf16"])
    ap.add_argument("--out", default=None, choices=[None, "f16", "bf16", "f32"])
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--copies", type=int, default=6)
    ap.add_argument("--sym", action="store_true")
    ap.add_argument("--sigma", type=float, default=0.02)
    ap.add_argument("--path", default="auto", choices=["auto", "gemv", "gemm"])
    ap.add_argument("--split-k", type=int, default=0)
    ap.add_argument("--interleaved", action="store_true", help="prepack the weights (QF_LAYOUT_INTERLEAVED)")
    ap.add_argument("--tiled", action="store_true", help="prepack the weights (QF_LAYOUT_TILED)")
    ap.add_argument("--slab", action="store_true",
                    help="prepack weights, scales and zeros for the streaming GEMV kernel (QF_LAYOUT_GEMV_SLAB)")
    ap.add_argument("--graph", action="store_true",
                    help="time a CUDA graph of one launch per weight copy instead of single launches")
    args = ap.parse_args()
    dt = {"f16": torch.float16, "bf16": torch.bfloat16, "f32": torch.float32}
    act = dt[args.act]
    out_dtype = dt[args.out] if args.out else act
    path = {"auto": QF_PATH_AUTO, "gemv": QF_PATH_GEMV, "gemm": QF_PATH_GEMM}[args.path]
    dev = torch.device("cuda:0")
    if args.graph:
        args.copies = max(args.copies, -(-300_000_000 // (args.K * args.N // 2)))
    sets = [make_case(args.M, args.K, args.N, act, dev, args.sym, args.sigma, seed=i) for i in range(args.copies)]
    layout = 0
    if args.interleaved:
        sets = [(qf.prepack_w4(qw), sc, zr, x) for (qw, sc, zr, x) in sets]
        layout = 1
    if args.tiled:
        sets = [(qf.prepack_w4(qw, layout=2), sc, zr, x) for (qw, sc, zr, x) in sets]
        layout = 2
    if args.slab:
        sets = [(qf.prepack_gemv_slab(qw, sc, zr, 128, 8), None, None, x) for (qw, sc, zr, x) in sets]
        layout = 3
    y = torch.empty(args.M, args.N, dtype=out_dtype, device=dev)

    def launch(i):
        qw, sc, zr, x = sets[i % args.copies]
        if args.slab:
            qf.w4a16_linear(x, qw, out_dtype=out_dtype, split_k=args.split_k, out=y)
            return
        qf.w4a16_linear(x, qw, sc, zr, group_size=128, zero_const=8, out_dtype=out_dtype, path=path,
                        split_k=args.split_k, out=y, weight_layout=layout)

    times = []
    if args.graph:
        launch(0)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for i in range(args.copies):
                launch(i)
        for it in range(args.iters + 2):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            g.replay()
            e1.record()
            torch.cuda.synchronize()
            if it >= 2:
                times.append(e0.elapsed_time(e1) * 1e3 / args.copies)
    else:
        for it in range(args.iters + 2):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            launch(it)
            e1.record()
            torch.cuda.synchronize()
            if it >= 2:
                times.append(e0.elapsed_time(e1) * 1e3)
    G = args.K // 128
    out_b = 4 if out_dtype == torch.float32 else 2
    nbytes = (args.K * args.N // 2 + G * args.N * 2 + (0 if args.sym else G * args.N // 2) + args.M * args.K * 2 +
              args.M * args.N * out_b)
    us = min(times)
    print(json.dumps({"M": args.M, "K": args.K, "N": args.N, "act": args.act, "path": args.path,
                      "layout": layout, "status": qf.device_status(), "us_min": round(us, 2),
                      "gbs": round(nbytes / us / 1e3, 1), "tflops": round(2 * args.M * args.K * args.N / us / 1e6, 1),
                      "us_all": [round(t, 2) for t in times]}))


if __name__ == "__main__":
    main()

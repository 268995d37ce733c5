"""Time one projection on one GPU:  python opbench.py --fmt q4 --n 28672 --k 8192 --m 1

Prints one JSON line: microseconds per launch (CUDA events around `reps` back-to-back launches
that rotate through enough weight copies to exceed L2), algorithmic GB/s and TFLOP/s.  Weights are
seeded synthetic tensors quantised the way the offline tools of the reference do it.  With
--reps 1..4 and --copies 1 it is also a small, self-ending command to put under a profiler.
"""
import argparse
import importlib
import importlib.util
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.join(HERE, "adreno-llms_b200")


def load_pkg():
    name = "adreno_llms_b200"
    if name in sys.modules:
        return sys.modules[name]
    spec = importlib.util.spec_from_file_location(name, os.path.join(PKG, "__init__.py"), submodule_search_locations=[PKG])
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--fmt", default="int8", choices=["fp16", "int8", "q4"])
    ap.add_argument("--n", type=int, default=151936)
    ap.add_argument("--k", type=int, default=896)
    ap.add_argument("--m", type=int, default=1)
    ap.add_argument("--op", default="linear", choices=["linear", "add", "swiglu"])
    ap.add_argument("--reps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--copies", type=int, default=0, help="resident weight copies (0: enough to exceed twice the L2)")
    ap.add_argument("--device", type=int, default=0)
    args = ap.parse_args()
    pkg = load_pkg()
    synth = importlib.import_module("adreno_llms_b200.synth")
    ctx = pkg.Context(args.device)
    _, l2, _ = ctx.device_info()
    rng = np.random.default_rng(1)
    fmt, N, K, M = args.fmt, args.n, args.k, args.m
    blk = min(N, 2048)   # timing does not depend on the values: quantise a block of rows and repeat it
    W, s = synth.weight(fmt, blk, K, rng)
    rep = (N + blk - 1) // blk
    W = np.tile(W, (rep, 1))[:N]
    if s is not None:
        s = np.tile(s, (rep, 1) if s.ndim == 2 else rep)[:N]
    nbytes = W.nbytes + (0 if s is None else s.nbytes)
    nw = 2 if args.op == "swiglu" else 1
    copies = args.copies if args.copies > 0 else int(max(2, min(256, -(-2 * l2 // (nbytes * nw)) + 1)))
    ws = [[pkg.QuantWeight(ctx, fmt, W, s) for _ in range(nw)] for _ in range(copies)]
    x = ctx.upload(synth.activations(M, K, rng).view(np.uint16))
    out = ctx.upload(synth.activations(M, N, rng).view(np.uint16))

    def run(i):
        w = ws[i % copies]
        if args.op == "linear":
            ctx.linear(M, N, K, x, w[0].buf, out)
        elif args.op == "add":
            ctx.linear_add(M, N, K, x, w[0].buf, out)
        else:
            ctx.fused_gate_up_silu(M, N, K, x, w[0].buf, w[1].buf, out)

    for i in range(args.warmup):
        run(i)
    a, b = ctx.event(), ctx.event()
    ctx.sync()
    l0 = ctx.launch_count()
    ctx.record(a)
    for i in range(args.reps):
        run(i)
    ctx.record(b)
    ms = ctx.elapsed_ms(a, b)
    us = ms * 1e3 / args.reps
    algo = nw * synth.linear_bytes(fmt, N, K, M) - (nw - 1) * (2 * M * K + 2 * M * N)
    print(json.dumps({"op": args.op, "fmt": fmt, "N": N, "K": K, "M": M, "us_per_launch": round(us, 3),
                      "algorithmic_bytes": algo, "gbps": round(algo / (us * 1e-6) / 1e9, 1),
                      "tflops": round(2.0 * nw * M * N * K / (us * 1e-6) / 1e12, 2),
                      "kernels_per_call": (ctx.launch_count() - l0) / args.reps, "weight_copies": copies}), flush=True)
    ctx.close()
    return 0


if __name__ == "__main__":
    sys.exit(main())

#!/usr/bin/env python3
"""Benchmark of the decode-step projection set (BASELINE.json configs[1]).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--fmt int8|fp16|q4]

A step is one pass over every projection of a SmolLM2-135M-shaped decode step
(30 x {QKV, o_proj+residual, gate/up/SiLU, down+residual} + tied lm_head; 211 GEMVs
recorded as 121 fused operators, the last of which also takes the greedy token) at M = 1 on
seeded synthetic weights and N(0,1) activations.  The recorded step is replayed as ONE resident
launch.  The metric is the achieved weight-stream rate: algorithmic bytes of the step / step
time, in GB/s.

  value     steps replayed from a recorded plan, operands resident in HBM, timed with
            CUDA events on the launching stream; consecutive steps use different
            resident weight copies so that every step streams from HBM, not L2
  e2e       the same step driven from HOST buffers through the C ABI: pinned-host
            hidden vector -> device, step, logits and token -> pinned host, every step
  roofline  the resident launch (the whole step is one kernel), against the HBM copy rate
  roofline_targets   the large single operators the north star names, each timed alone
  parity_checked     the replay's logits and token are compared inside the run with the same
            operators launched one by one (and, with several ranks, across the ranks)
  chained_step       the same projections with the model's data flow (layer norms fused into QKV and
            gate/up, o_proj reads q, down reads the SwiGLU output): every projection waits for the
            one before it, as in a real token
  cpu_baseline  the reference's own .cl kernels compiled for the CPU (oracle/_ref; the oracle
            port when that build is absent), all host cores, on a bounded sample of the step

  sharded_projections, prefill_gemm   the scaled-up operators of the other BASELINE configs
            (row-sharded int8 lm_head at M = 256, Q4 FFN matrix at M = 1..128; fp16 lm_head
            at M = 512 / 2048 on the tensor-core path), each timed alone

With --gpus N > 1 (launched under torchrun) the lm_head rows are sharded across the
ranks; every rank keeps its rows of the logits and the greedy pick exchanges one 8-byte
(value, row) key per rank over NVLink peer memory (the step with the logits gathered to
every rank instead is timed beside it); the per-layer projections stay replicated
(north star: only the large row-sharded projections are partitioned).
--impl reference times the reference's own CPU implementation of the path
(oracle/_ref when it was built, else the oracle port) on the host cores: whole steps, every
launch of the step executed.
"""
import argparse
import importlib.util
import json
import math
import os
import statistics
import subprocess
import sys
import tempfile
import time

import numpy as np

REPO = os.path.dirname(os.path.abspath(__file__))
METRIC = "int8/Q4 GEMV achieved HBM GB/s (decode-step projection set)"
UNIT = "GB/s"


class StdoutToStderr:
    """Send file descriptor 1 to stderr for a while: NCCL prints its version banner on stdout
    when a communicator is first made, and the bench prints exactly one JSON line there."""

    def __enter__(self):
        sys.stdout.flush()
        self.saved = os.dup(1)
        os.dup2(2, 1)

    def __exit__(self, *a):
        sys.stdout.flush()
        os.dup2(self.saved, 1)
        os.close(self.saved)


def load_pkg():
    name = "adreno_llms_b200"
    if name in sys.modules:
        return sys.modules[name]
    path = os.path.join(REPO, "adreno-llms_b200", "__init__.py")
    spec = importlib.util.spec_from_file_location(name, path, submodule_search_locations=[os.path.dirname(path)])
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def measured_peaks():
    p = os.path.join(REPO, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return 6650.0, "fallback (6.65 TB/s, earlier measurement on this pool)"


def measured_tensor_peak():
    p = os.path.join(REPO, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d["bf16_tflops"]), "measured (MEASURED_PEAKS.json bf16_tflops, burst)"
    return 1590.0, "fallback (1.59 PFLOP/s, earlier measurement on this pool)"


def prefill_gemm(pkg, ctx, synth, reps=6):
    """The prefill shapes of the Qwen-shaped lm_head (151936 x 896, fp16) on the tensor-core path:
    TFLOP/s = 2 M N K / device time, each launch timed alone with CUDA events (the 272 MB weight
    and the M x N output are larger than L2)."""
    peak, src = measured_tensor_peak()
    N, K = 151936, 896
    W, _ = synth.weight("fp16", 2048, K, np.random.default_rng(91))
    qw = pkg.QuantWeight(ctx, "fp16", np.tile(W, (N // 2048 + 1, 1))[:N], None)
    rows = []
    for M in (512, 2048):
        x = ctx.upload(synth.activations(M, K, np.random.default_rng(92)).view(np.uint16))
        out = ctx.alloc(M * N * 2)
        a, b = ctx.event(), ctx.event()
        best = []
        for i in range(reps + 2):
            ctx.record(a)
            ctx.linear(M, N, K, x, qw.buf, out)
            ctx.record(b)
            ctx.sync()
            if i >= 2:
                best.append(ctx.elapsed_ms(a, b))
        us = float(np.mean(best)) * 1e3
        tf = 2.0 * M * N * K / (us * 1e-6) / 1e12
        rows.append({"kernel": "linear_gemm_tc_kernel", "fmt": "fp16", "N": N, "K": K, "M": M, "us": us, "tflops": tf,
                     "peak_tflops": peak, "frac": tf / peak, "peak_source": src})
        ctx.free(out)
        ctx.free(x)
    qw.release()
    return rows


class ClockSampler:
    FIELDS = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.path, self.t0 = index, None, None, None

    def mark(self):
        """The load to be sampled starts now: samples taken before this moment (start-up, idle) are dropped."""
        import datetime
        self.t0 = datetime.datetime.now()

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if not self.proc:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        import datetime
        sm, mx, reasons = [], [], set()
        for line in open(self.path):
            f = [t.strip() for t in line.split(",")]
            if len(f) < 8:
                continue
            try:
                when = datetime.datetime.strptime(f[0], "%Y/%m/%d %H:%M:%S.%f")
                if self.t0 is not None and when < self.t0:
                    continue
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[4:8]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.path)
        if sm:
            out.update(sm_mhz=statistics.median(sm), sm_max_mhz=max(mx), reasons=sorted(reasons), samples=len(sm))
        return out


# ------------------------------------------------------------------------------------
# CPU arm: the oracle (checker code) used ONLY here as the timed CPU baseline
# ------------------------------------------------------------------------------------
def ref_build_present():
    return os.path.exists(os.path.join(REPO, "oracle", "_ref", "libsmollm2_block_fused_int8.so"))


def workload_text(shape, fmt, M):
    """config.workload: the same string in both arms."""
    synth = importlib.import_module("adreno_llms_b200.synth")
    return f"decode-step projection set, {shape.name} shape, {fmt}, M={M} ({synth.decode_step_gemvs(shape)} GEMVs, N(0,1) activations)"


def cpu_reference_steps(fmt, steps, budget_s=60.0):
    """Whole steps on the reference's OWN kernels (its .cl sources compiled for the CPU, oracle/_ref),
    all host cores: every launch of the step is executed, in order (per layer the three QKV GEMVs,
    o_proj+residual, gate/up/SiLU, down+residual; then the whole lm_head).  Timing does not depend on
    the values, so the thirty layers run on one layer's synthetic weights.  Returns
    (GB/s, cores, seconds per step, steps timed)."""
    sys.path.insert(0, REPO)
    from oracle import ref_cl  # noqa: E402  (CPU-baseline leg only)
    synth = importlib.import_module("adreno_llms_b200.synth")
    sh = synth.SMOLLM2_135M
    cores = os.cpu_count() or 1
    rng = np.random.default_rng(98)
    H, F = sh.hidden, sh.ffn
    x_h, x_f, r = synth.activations(1, H, rng), synth.activations(1, F, rng), synth.activations(1, H, rng)

    def w(n, k):
        return synth.weight(fmt, n, k, rng)

    Wq, Wk, Wv, Wo, Wg, Wu, Wd, Wl = w(sh.q_dim, H), w(sh.kv_dim, H), w(sh.kv_dim, H), w(H, sh.q_dim), w(F, H), w(F, H), w(H, F), w(sh.vocab, H)
    if fmt == "int8":
        lib = "smollm2_block_fused_int8"

        def gemv(W):
            return ref_cl.gemv_scaled(lib, "gemv_m1_k576_no4_img_int8", 4, x_h, W[0], W[1], cores)

        def layer():
            gemv(Wq), gemv(Wk), gemv(Wv)
            ref_cl.residual_scaled(lib, "fused_oproj_residual_m1_no4_img_int8", x_h, Wo[0], Wo[1], r, cores)
            ref_cl.swiglu_int8(x_h, Wg[0], Wg[1], Wu[0], Wu[1], cores)
            ref_cl.residual_scaled(lib, "fused_down_residual_m1_no4_img_int8", x_f, Wd[0], Wd[1], r, cores)
    else:
        lib = "smollm2_block_fused"

        def gemv(W):
            return ref_cl.gemv_fp16_img(lib, "gemv_m1_k576_no4_img", 4, x_h, W[0], cores)

        def layer():
            gemv(Wq), gemv(Wk), gemv(Wv)
            ref_cl.residual_fp16_img(lib, "fused_oproj_residual_m1_no4_img", x_h, Wo[0], r, cores)
            ref_cl.swiglu_fp16(x_h, Wg[0], Wu[0], cores)
            ref_cl.residual_fp16_img(lib, "fused_down_residual_m1_no4_img", x_f, Wd[0], r, cores)

    def one_step():
        for _ in range(sh.layers):
            layer()
        gemv(Wl)

    layer()  # warm (page in the libraries, start the worker threads)
    times, t_begin = [], time.perf_counter()
    while len(times) < steps and (not times or time.perf_counter() - t_begin < budget_s):
        t0 = time.perf_counter()
        one_step()
        times.append(time.perf_counter() - t0)
    t_step = statistics.median(times)
    return synth.decode_step_bytes(sh, fmt, 1) / t_step / 1e9, cores, t_step, len(times)


def cpu_port_steps(fmt, steps, budget_s=30.0):
    """Whole steps on the CPU restatement (oracle/oracle.c, -O3 -march=native, rows split over all
    host cores); same launch list and weight reuse as cpu_reference_steps."""
    sys.path.insert(0, REPO)
    from oracle import cpu as ocpu  # noqa: E402  (CPU-baseline leg only)
    synth = importlib.import_module("adreno_llms_b200.synth")
    sh = synth.SMOLLM2_135M
    cores = os.cpu_count() or 1
    rng = np.random.default_rng(99)
    H, F = sh.hidden, sh.ffn
    x_h, x_f = synth.activations(1, H, rng), synth.activations(1, F, rng)
    ws = {(n, k): synth.weight(fmt, n, k, rng) for _, _, lst in synth.decode_step_ops(sh) for n, k in lst}

    def one_step():
        for kind, _, lst in synth.decode_step_ops(sh):
            for n, k in lst:
                W, s = ws[(n, k)]
                ocpu.linear_acc(fmt, x_f if k == F else x_h, W, s, ocpu.ORDER_KERNEL, cores)

    ocpu.linear_acc(fmt, x_h, *ws[(sh.kv_dim, H)], ocpu.ORDER_KERNEL, cores)  # warm
    times, t_begin = [], time.perf_counter()
    while len(times) < steps and (not times or time.perf_counter() - t_begin < budget_s):
        t0 = time.perf_counter()
        one_step()
        times.append(time.perf_counter() - t0)
    t_step = statistics.median(times)
    return synth.decode_step_bytes(sh, fmt, 1) / t_step / 1e9, cores, t_step, len(times)


def cpu_arm(fmt, steps):
    """The CPU baseline as a dict: the reference's own kernels when they were built (kind
    "reference"), else the restatement (kind "port"); the other kind is reported beside it."""
    out = {}
    if ref_build_present() and fmt in ("int8", "fp16"):
        r, cores, t, n = cpu_reference_steps(fmt, steps)
        out = {"value": r, "unit": UNIT, "cores": cores, "kind": "reference", "seconds_per_step": t, "steps_timed": n, "extrapolated": False,
               "sample": f"{n} whole step(s): every launch of the step executed on the reference's .cl kernels compiled for the CPU "
                         f"(64 work-items of a group run as fibers), all {cores} cores; thirty layers on one layer's synthetic weights"}
    pr, pcores, pt, pn = cpu_port_steps(fmt, steps)
    port = {"value": pr, "unit": UNIT, "cores": pcores, "kind": "port", "seconds_per_step": pt, "steps_timed": pn, "extrapolated": False,
            "sample": f"{pn} whole step(s) on the C restatement of the kernels (-O3 -march=native), rows split over {pcores} cores"}
    if not out:
        return port
    out["port"] = port
    return out


def run_reference_arm(args, pkg, rank):
    if rank != 0:
        return
    fmt = args.fmt
    synth = importlib.import_module("adreno_llms_b200.synth")
    base = cpu_arm(fmt, max(1, min(args.steps, 3)))
    line = {
        "impl": "reference", "metric": METRIC, "value": base["value"], "unit": UNIT, "n_gpus": args.gpus,
        "steps": base["steps_timed"], "steps_requested": args.steps, "warmup": 1, "ms_per_step": base["seconds_per_step"] * 1e3,
        "extrapolated": False, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": f"{fmt} weights, fp16 activations, fp32 accumulate",
        "data": "synthetic",
        "config": {"workload": workload_text(synth.SMOLLM2_135M, fmt, 1)},
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------
def time_group(ctx, fn, reps):
    a, b = ctx.event(), ctx.event()
    ctx.sync()
    ctx.record(a)
    for i in range(reps):
        fn(i)
    ctx.record(b)
    ms = ctx.elapsed_ms(a, b)
    ctx.L.nn_event_destroy(a)
    ctx.L.nn_event_destroy(b)
    return ms


def sharded_projections(pkg, ctx, synth, comm, rank, world, dist, reps=12):
    """The scaled-up row-sharded projections: int8 lm_head 151936 x 896 at M=256 and a Q4 FFN
    matrix 28672 x 8192 at M in {1, 8, 32, 128}.  Rank g owns rows [g N/G, (g+1) N/G), writes its
    [M, N/G] block straight into slot g of the gather buffer, and an in-place all-gather fills
    the other slots (layout [G][M][N/G]).  Device-timed per operator with L2 flushed before each
    launch; the projection and the all-gather are reported separately, max over ranks."""
    rows = []
    cases = [("int8", 151936, 896, 256)] + [("q4", 28672, 8192, m) for m in (1, 8, 32, 128)]
    cache = {}
    for fmt, N, K, M in cases:
        n = N // world
        if (fmt, N, K) not in cache:
            for old in cache.values():
                old.release()
            cache.clear()
            # timing does not depend on the values: quantise a block of rows and repeat it
            blk = min(n, 1024)
            W, sc = synth.weight(fmt, blk, K, np.random.default_rng(77 + rank))
            rep = (n + blk - 1) // blk
            W = np.tile(W, (rep, 1))[:n]
            sc = np.tile(sc, (rep, 1) if sc.ndim == 2 else rep)[:n]
            cache[(fmt, N, K)] = pkg.QuantWeight(ctx, fmt, W, sc)
        qw = cache[(fmt, N, K)]
        x = ctx.upload(synth.activations(M, K, np.random.default_rng(78)).view(np.uint16))
        gathered = ctx.alloc(M * N * 2)
        mine = gathered + rank * M * n * 2
        ev = [ctx.event() for _ in range(3)]
        t_lin = t_ag = 0.0
        for i in range(reps + 2):
            ctx.l2_flush()
            if comm:   # line the ranks up on the device before the timed launches
                comm.signal()
                comm.wait()
            ctx.record(ev[0])
            ctx.linear(M, n, K, x, qw.buf, mine)
            ctx.record(ev[1])
            if comm:
                comm.all_gather(mine, gathered, M * n * 2)
            ctx.record(ev[2])
            ctx.sync()
            if i >= 2:
                t_lin += ctx.elapsed_ms(ev[0], ev[1])
                t_ag += ctx.elapsed_ms(ev[1], ev[2])
        t_fused = 0.0
        if comm:
            sym = [comm.symm_alloc(M * N * 2) for _ in range(2)]
            for i in range(reps + 2):
                ctx.l2_flush()
                comm.signal()
                comm.wait()
                ctx.record(ev[0])
                comm.linear_gather(M, n, K, x, qw.buf, sym[i & 1])
                ctx.record(ev[1])
                ctx.sync()
                if i >= 2:
                    t_fused += ctx.elapsed_ms(ev[0], ev[1])
            if dist:
                dist.barrier()
            for b in sym:
                comm.symm_free(b)
            # greedy tokens of the M rows without moving the logits: M keys per rank cross NVLink
            loc, toks = ctx.alloc(M * n * 2), ctx.alloc(M * 4)
            t_pick = 0.0
            for i in range(reps + 2):
                ctx.l2_flush()
                comm.signal()
                comm.wait()
                ctx.record(ev[0])
                comm.linear_argmax_sharded_rows(M, n, K, x, qw.buf, loc, toks)
                ctx.record(ev[1])
                ctx.sync()
                if i >= 2:
                    t_pick += ctx.elapsed_ms(ev[0], ev[1])
            if dist:
                dist.barrier()
            ctx.free(loc)
            ctx.free(toks)
        else:
            t_fused, t_ag = t_lin, 0.0   # one rank: nothing to gather
            t_pick = 0.0
        # the whole operator on one GPU, timed the same way, for the efficiency figure t1 / (G * tG)
        t_one = t_lin
        if world > 1:
            repn = (N + W.shape[0] - 1) // W.shape[0]
            Wf = np.tile(W, (repn, 1))[:N]
            sf = np.tile(sc, (repn, 1) if sc.ndim == 2 else repn)[:N]
            qf = pkg.QuantWeight(ctx, fmt, Wf, sf)
            t_one = 0.0
            for i in range(reps + 2):
                ctx.l2_flush()
                ctx.record(ev[0])
                ctx.linear(M, N, K, x, qf.buf, gathered)
                ctx.record(ev[1])
                ctx.sync()
                if i >= 2:
                    t_one += ctx.elapsed_ms(ev[0], ev[1])
            qf.release()
        t = [t_lin / reps * 1e3, t_ag / reps * 1e3, t_fused / reps * 1e3, t_one / reps * 1e3, t_pick / reps * 1e3]
        if dist:
            import torch
            tt = torch.tensor(t, dtype=torch.float64)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            t = tt.tolist()
        b = synth.linear_bytes(fmt, N, K, M)
        rows.append({"fmt": fmt, "N": N, "K": K, "M": M, "rows_per_rank": n, "linear_us": t[0], "nccl_all_gather_us": t[1],
                     "fused_gather_us": t[2],   # projection with peer stores + flag exchange, one call
                     "single_gpu_us": t[3],     # the unsharded operator on one GPU of this run
                     "efficiency_per_operator": t[3] / (world * t[2]) if t[2] > 0 else None,
                     # projection + greedy token of every row with one key per row and rank exchanged (no logits moved)
                     "sharded_pick_us": t[4] if world > 1 else None,
                     "efficiency_with_sharded_pick": t[3] / (world * t[4]) if (world > 1 and t[4] > 0) else None,
                     "gbps_aggregate": b / (t[2] * 1e-6) / 1e9,
                     "tflops_aggregate": 2.0 * M * N * K / (t[2] * 1e-6) / 1e12})
        for e in ev:
            ctx.L.nn_event_destroy(e)
        ctx.free(gathered)
        ctx.free(x)
    for old in cache.values():
        old.release()
    return rows


def roofline_targets(pkg, ctx, synth, l2_bytes, reps=40):
    """The large single operators the north star sets its HBM target on, each timed alone at M = 1:
    int8 and fp16 lm_head 151936 x 896, Q4 FFN matrix 28672 x 8192.  Two ways, both with CUDA events:
    "rotated back-to-back" = consecutive launches over enough weight copies to exceed twice the L2 (the
    next launch's weight stream starts under the tail of the previous one, as inside a decode loop);
    "isolated, L2 flushed" = one launch between two events after the L2 was rewritten."""
    peak, src = measured_peaks()
    rows = []
    for fmt, N, K in (("int8", 151936, 896), ("fp16", 151936, 896), ("q4", 28672, 8192)):
        blk = 2048
        W, s = synth.weight(fmt, blk, K, np.random.default_rng(61))
        rep = (N + blk - 1) // blk
        W = np.tile(W, (rep, 1))[:N]
        if s is not None:
            s = np.tile(s, (rep, 1) if s.ndim == 2 else rep)[:N]
        nbytes = W.nbytes + (0 if s is None else s.nbytes)
        copies = int(max(2, -(-2 * l2_bytes // nbytes) + 1))
        ws = [pkg.QuantWeight(ctx, fmt, W, s) for _ in range(copies)]
        x = ctx.upload(synth.activations(1, K, np.random.default_rng(62)).view(np.uint16))
        out = ctx.alloc(N * 2)
        for i in range(4):
            ctx.linear(1, N, K, x, ws[i % copies].buf, out)
        ms = time_group(ctx, lambda i: ctx.linear(1, N, K, x, ws[i % copies].buf, out), reps)
        us_rot = ms * 1e3 / reps
        a, b = ctx.event(), ctx.event()
        iso = []
        for i in range(8):
            ctx.l2_flush()
            ctx.record(a)
            ctx.linear(1, N, K, x, ws[i % copies].buf, out)
            ctx.record(b)
            ctx.sync()
            if i >= 2:
                iso.append(ctx.elapsed_ms(a, b) * 1e3)
        algo = synth.linear_bytes(fmt, N, K, 1)
        for mode, us in (("rotated back-to-back", us_rot), ("isolated, L2 flushed", float(np.mean(iso)))):
            rows.append({"kernel": "linear_stream_kernel", "fmt": fmt, "N": N, "K": K, "M": 1, "mode": mode, "us": us,
                         "algorithmic_bytes": algo, "achieved": algo / (us * 1e-6) / 1e9, "unit": "GB/s", "peak": peak,
                         "frac": algo / (us * 1e-6) / 1e9 / peak, "peak_source": src})
        for w in ws:
            w.release()
        ctx.free(x)
        ctx.free(out)
    return rows


def timed_steps(ctx, step, n_sets, steps, warmup):
    for i in range(warmup):
        step.launch(i % n_sets)
    ctx.sync()
    return time_group(ctx, lambda i: step.launch(i % n_sets), steps)


def record_separate(step):
    """Record the step's plans again as separate launches (one graph node per operator)."""
    for pl in step.plans:
        if pl:
            step.ctx.L.nn_plan_free(pl)
    os.environ["NNB_PLAN_SEPARATE"] = "1"
    try:
        n = step.record()
    finally:
        del os.environ["NNB_PLAN_SEPARATE"]
    return n


def results_of(ctx, step):
    sh = step.shape
    return (step.read_logits().view(np.uint16).copy(), step.read_token(),
            ctx.download(step.resid, (step.M, sh.hidden), np.uint16).copy())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--fmt", default="int8", choices=["int8", "fp16", "q4"])
    ap.add_argument("--shape", default="smollm2", choices=["smollm2", "qwen", "lfm2"],
                    help="model shape of the step (default: the configuration the metric is quoted on)")
    ap.add_argument("--m", type=int, default=1, help="activation rows per projection (batched decode), 1..16")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--only", default=None, choices=["qkv", "o_add", "gate_up", "down_add", "lm_head"],
                    help="profiling aid: the step consists of this launch group only")
    ap.add_argument("--quick", action="store_true", help="the step only: none of the other configurations' operators")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.warmup < 3:
        args.warmup = 3

    pkg = load_pkg()
    if args.impl == "reference":
        run_reference_arm(args, pkg, rank)
        return 0

    synth = importlib.import_module("adreno_llms_b200.synth")
    dstep = importlib.import_module("adreno_llms_b200.decode_step")
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist = dist_mod
        dist.init_process_group(backend="gloo", rank=rank, world_size=world)

    ctx = pkg.Context(local_rank)
    sm_count, l2_bytes, _ = ctx.device_info()
    shape = {"smollm2": synth.SMOLLM2_135M, "qwen": synth.QWEN25_05B, "lfm2": synth.LFM25_350M}[args.shape]
    fmt, MM = args.fmt, max(1, min(16, args.m))
    default_workload = args.shape == "smollm2" and MM == 1 and args.only is None
    if shape.vocab % world:
        raise SystemExit(f"vocab {shape.vocab} is not divisible by {world} ranks")
    vrows = shape.vocab // world
    step_bytes_full = sum(synth.linear_bytes(fmt, n, k, MM) for kind, _, ws in synth.decode_step_ops(shape)
                          if args.only in (None, kind) for n, k in ws)
    n_sets = min(64, max(2, math.ceil(2.0 * l2_bytes / step_bytes_full) + 1))
    comm = None
    if world > 1:
        import torch
        idbuf = torch.zeros(128, dtype=torch.uint8)
        if rank == 0:
            idbuf = torch.tensor(list(pkg.Comm.unique_id()), dtype=torch.uint8)
        dist.broadcast(idbuf, 0)
        with StdoutToStderr():
            comm = pkg.Comm(ctx, bytes(idbuf.tolist()), rank, world)
            comm.symm_free(comm.symm_alloc(256))   # first collective on the communicator
    # The step of the metric (BASELINE configs[1]): every projection reads its own N(0,1) activation
    # buffer; the in-place residual adds are the only data that flows from one projection to the next.
    # The same projections with the model's data flow (every projection waits for the one before it)
    # are timed further down as `chained_step`.
    step = dstep.DecodeStep(ctx, shape, fmt, M=MM, n_sets=n_sets, vocab_rows=(rank * vrows, vrows), only=args.only, comm=comm)

    def barrier():
        ctx.sync()
        if dist:
            dist.barrier()

    def max_over_ranks(v):
        if not dist:
            return v
        import torch
        tt = torch.tensor([v], dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        return float(tt.item())

    kernels_per_step = step.record(with_argmax=(args.only is None))
    resident_runs = step.resident_runs()
    recorded = ctx.L.nn_plan_num_recorded(step.plans[0])
    sampler = ClockSampler(local_rank)
    sampler.start()   # the sampling process needs a moment to come up: started before the warm-up, marked at the timed region
    for i in range(args.warmup):
        step.launch(i % n_sets)
    barrier()
    sampler.mark()

    # ---- value: K steps, device-timed ----
    launches0 = ctx.launch_count()
    barrier()
    ms = time_group(ctx, lambda i: step.launch(i % n_sets), args.steps)
    barrier()
    launches = ctx.launch_count() - launches0
    ms = max_over_ranks(ms)
    ms_per_step = ms / args.steps
    value = step_bytes_full / (ms_per_step * 1e-3) / 1e9

    # ---- e2e: hidden vector from pinned host memory in, logits and token to pinned host memory out, every step ----
    e2e_steps = max(50, min(args.steps, 500))
    import ctypes
    hx = pkg.load().nn_host_alloc(MM * shape.hidden * 2)
    hl = pkg.load().nn_host_alloc(MM * shape.vocab * 2)
    hl_tok = pkg.load().nn_host_alloc(64)
    ctypes.memmove(hx, step.resid0.ctypes.data, MM * shape.hidden * 2)
    x_in = step.resid if step.chained else step.x_h     # where the token's hidden vector enters the step
    keys_pick = bool(comm) and MM == 1 and args.only is None
    d2h_bytes = (MM * step.vocab_n * 2 + 4) if (keys_pick or not comm) else MM * shape.vocab * 2

    # The host program's own copies are recorded with the step, as the reference records its whole token into the
    # replayed queue: one plan per weight copy holds the host -> device copy of the hidden vector, the step, and the
    # device -> host reads of the logits and the token; a step is one nn_plan_launch and one nn_sync.
    io_plans = []
    for i in range(n_sets):
        ctx.plan_begin()
        pkg._check(ctx.L.nn_buf_write(ctx.h, x_in, 0, hx, MM * shape.hidden * 2))
        step.enqueue(i, with_argmax=(args.only is None))
        if keys_pick or not comm:
            pkg._check(ctx.L.nn_buf_read(ctx.h, hl, step.logits, 0, MM * step.vocab_n * 2))
            pkg._check(ctx.L.nn_buf_read(ctx.h, hl_tok, step.token, 0, 4))
        else:
            pkg._check(ctx.L.nn_buf_read(ctx.h, hl, step.gathered[i], 0, MM * shape.vocab * 2))
        io_plans.append(ctx.plan_end())

    def e2e_step(i):
        ctx.plan_launch(io_plans[i % n_sets])
        ctx.sync()

    for i in range(5):
        e2e_step(i)
    barrier()
    t0 = time.perf_counter()
    for i in range(e2e_steps):
        e2e_step(i)
    e2e_s = max_over_ranks(time.perf_counter() - t0)
    e2e_value = step_bytes_full / (e2e_s / e2e_steps) / 1e9
    # short runs: the same load is kept up (untimed) until the clock sampler has had half a second of it
    # (the count is derived from the max-over-ranks timings, so every rank launches the same number of steps)
    spent = ms * 1e-3 + e2e_s
    if spent < 0.5:
        for i in range(int((0.5 - spent) / (ms_per_step * 1e-3)) + 1):
            step.launch(i % n_sets)
        ctx.sync()
    # what came back through the recorded copies is what the device holds
    e2e_step(0)
    e2e_logits = np.ctypeslib.as_array(ctypes.cast(hl, ctypes.POINTER(ctypes.c_uint16)), (MM * step.vocab_n,)).copy() if (keys_pick or not comm) else None
    e2e_token = int(ctypes.cast(hl_tok, ctypes.POINTER(ctypes.c_int32))[0]) if (keys_pick or not comm) else None
    for pl in io_plans:
        ctx.L.nn_plan_free(pl)
    clocks = sampler.stop()

    # ---- parity, inside the run: the replay against the same operators launched one by one ----
    parity = {"checked": False}
    if args.only is None:
        step.reset_residual()
        step.launch(0)
        ctx.sync()
        got = results_of(ctx, step)
        sep_n = record_separate(step)
        step.reset_residual()
        step.launch(0)
        ctx.sync()
        want = results_of(ctx, step)
        same = bool(np.array_equal(got[0], want[0]) and got[1] == want[1] and np.array_equal(got[2], want[2]))
        lg = want[0].view(np.float16).astype(np.float32)
        if e2e_logits is not None:
            e2e_same = bool(np.array_equal(e2e_logits, got[0].reshape(-1)) and e2e_token == got[1])
            same = same and e2e_same
        parity = {"checked": True, "resident_equals_separate_launches": same, "logits_finite": bool(np.isfinite(lg).all()),
                  "token": int(got[1]), "separate_launches": int(sep_n)}
        if keys_pick:
            # across the ranks: the exchanged pick must be the arg-max of all ranks' logits, on every rank
            import torch
            mine = torch.from_numpy(want[0].view(np.uint16).reshape(-1).astype(np.int32))   # gloo carries no 16-bit integers
            allv = [torch.zeros_like(mine) for _ in range(world)]
            dist.all_gather(allv, mine)
            full = torch.cat(allv).numpy().astype(np.uint16).view(np.float16).astype(np.float32)
            best = int(np.flatnonzero(full == full.max())[0])
            toks = [torch.zeros(1, dtype=torch.int64) for _ in range(world)]
            dist.all_gather(toks, torch.tensor([want[1]], dtype=torch.int64))
            parity["sharded_pick_equals_argmax_of_all_logits"] = bool(all(int(t.item()) == best for t in toks))
            same = same and parity["sharded_pick_equals_argmax_of_all_logits"]
        parity["ok"] = bool(same and parity["logits_finite"])
        # the separate launches timed the same way, for comparison
        sms = max_over_ranks(timed_steps(ctx, step, n_sets, min(args.steps, 300), 5))
        parity["separate_launches_step_us"] = sms / min(args.steps, 300) * 1e3

    # ---- several ranks: the same step with the logits gathered to every rank instead ----
    gathered_step_us = None
    if keys_pick:
        step.gather_logits = True
        for pl in step.plans:
            ctx.L.nn_plan_free(pl)
        step.plans = [None] * n_sets
        step.record(with_argmax=True)
        gms = max_over_ranks(timed_steps(ctx, step, n_sets, min(args.steps, 300), 5))
        gathered_step_us = gms / min(args.steps, 300) * 1e3
        if rank == 0 or True:
            # the gathered logits must be the same vector on every rank, and its arg-max the token
            import torch
            step.launch(0)
            ctx.sync()
            g = ctx.download(step.gathered[0], (shape.vocab,), np.uint16)
            tok = step.read_token()
            h = torch.tensor([int(np.bitwise_xor.reduce(g.astype(np.int64) * (np.arange(g.size) % 65521 + 1))), tok], dtype=torch.int64)
            hs = [torch.zeros_like(h) for _ in range(world)]
            dist.all_gather(hs, h)
            parity["gathered_logits_identical_on_all_ranks"] = bool(all(torch.equal(x, hs[0]) for x in hs))
            parity["ok"] = bool(parity.get("ok", True) and parity["gathered_logits_identical_on_all_ranks"])

    # ---- the same projections with the model's data flow: QKV and gate/up read the residual stream through
    #      the (fused) layer norms, o_proj reads q (attention itself is not on the path), down reads the
    #      SwiGLU output, lm_head the final residual stream: every projection waits for the one before it,
    #      which is what the latency of a real token is made of ----
    chained = None
    if default_workload and world == 1:
        cstep = dstep.DecodeStep(ctx, shape, fmt, M=1, n_sets=min(n_sets, 3), norm=True, chained=True)
        cstep.record()
        cn = len(cstep.sets)
        cms = timed_steps(ctx, cstep, cn, min(args.steps, 500), 5)
        cstep.reset_residual()
        cstep.launch(0)
        ctx.sync()
        cgot = results_of(ctx, cstep)
        cruns, claunches = cstep.resident_runs(), cstep.kernels_per_step
        record_separate(cstep)
        cstep.reset_residual()
        cstep.launch(0)
        ctx.sync()
        cwant = results_of(ctx, cstep)
        csep = timed_steps(ctx, cstep, cn, 200, 5)
        chained = {"resident_step_us": cms / min(args.steps, 500) * 1e3, "separate_launches_step_us": csep / 200 * 1e3,
                   "launches_per_step": claunches, "resident_launches": cruns, "layer_norms_fused": 2 * shape.layers,
                   "resident_equals_separate_launches": bool(np.array_equal(cgot[0], cwant[0]) and cgot[1] == cwant[1] and np.array_equal(cgot[2], cwant[2]))}
        parity["ok"] = bool(parity.get("ok", True) and chained["resident_equals_separate_launches"])
        for st in cstep.sets:
            for w in st.values():
                w.release()

    peak, peak_src = measured_peaks()
    traffic_tbl = {}
    tp = os.path.join(REPO, "profiles", "dram_traffic.json")
    if os.path.exists(tp):
        traffic_tbl = json.load(open(tp)).get(fmt, {})
    extras = default_workload and not args.quick
    targets = roofline_targets(pkg, ctx, synth, l2_bytes) if (extras and world == 1) else None
    sharded = sharded_projections(pkg, ctx, synth, comm, rank, world, dist) if extras else None
    prefill = prefill_gemm(pkg, ctx, synth) if (extras and world == 1) else None
    probe = None
    if extras and world == 1:
        # the library's own read ceiling on this GPU (the reference's STREAM probe): both read paths, best of 5
        loads_gbs, tma_gbs = ctx.bandwidth_probe(0, 5)
        probe = {"bytes": max(1 << 30, 8 * l2_bytes), "loads_gbs": loads_gbs, "tma_bulk_gbs": tma_gbs, "trials": 5}

    cpu_base = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline and default_workload:
        cpu_base = cpu_arm(fmt, 2)

    if rank == 0:
        dominant = "decode_plan_kernel" if resident_runs else "linear_stream_kernel"
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_per_step, "decode_step_us": ms_per_step * 1e3, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None,
            "dtype": f"{fmt} weights, fp16 activations, fp32 accumulate", "data": "synthetic",
            "config": {"workload": workload_text(shape, fmt, MM),
                       "recorded_operators": recorded, "launches_per_step": kernels_per_step, "resident_launches": resident_runs,
                       "algorithmic_bytes_per_step": step_bytes_full,
                       "l2": f"{n_sets} resident weight copies rotated step to step "
                             f"({n_sets * step.weight_bytes / 1e6:.0f} MB > L2 {l2_bytes / 1e6:.0f} MB)",
                       "sharding": "none" if world == 1 else
                                   (f"lm_head rows / {world} ranks; every rank stores its rows of the logits locally and the greedy pick "
                                    "exchanges one 8-byte (value, row) key per rank over NVLink peer memory; layers replicated" if keys_pick else
                                    f"lm_head rows / {world} ranks, each rank's kernel stores into every rank's "
                                    "gather buffer over NVLink peer memory; layers replicated")},
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": MM * shape.hidden * 2,
                    "d2h_bytes_per_step": d2h_bytes, "us_per_step": e2e_s / e2e_steps * 1e6, "steps": e2e_steps},
            "gpu_launches": launches,
            "parity_checked": bool(parity.get("checked")), "parity": parity,
            # the whole step is one launch of the resident kernel: its algorithmic bytes are the step's
            "roofline": {"bound": "hbm", "kernel": dominant, "achieved": value, "peak": peak, "unit": "GB/s", "frac": value / peak,
                         "traffic": traffic_tbl.get("decode_plan_kernel"), "peak_source": peak_src,
                         "us_per_launch": ms_per_step * 1e3 / max(1, kernels_per_step), "bytes_per_launch": step_bytes_full,
                         "note": "latency-bound, not bandwidth-bound: the in-place residual adds of the step form a chain of 60 "
                                 "hand-overs through device memory, under which the step's weight stream is hidden"},
            "roofline_targets": targets,
            "chained_step": chained,
            "sharded_projections": sharded,
            "prefill_gemm": prefill,
            "read_bandwidth_probe": probe,
            "decode_step_with_gathered_logits_us": gathered_step_us,
            "clocks": clocks,
        }
        if cpu_base:
            line["cpu_baseline"] = cpu_base
        print(json.dumps(line), flush=True)
    ok = parity.get("ok", True)
    if dist:
        dist.barrier()
        dist.destroy_process_group()
    return 0 if ok else 3


if __name__ == "__main__":
    sys.exit(main())

"""Recorded decode steps whose runs of single-token operators replay as one resident launch
(the role of the reference's recordable-queue replay, src/models/smollm2-135m-instruct/src/
model.cpp:104-195,312-344): same bits as the operators called one by one, the oracle's chain
within the path's tolerance, bounded waits."""
import ctypes
import importlib

import numpy as np
import pytest

from oracle import cpu
from helpers import TOL, check_close, make_weight, make_x

pytestmark = pytest.mark.gpu


def _mods():
    return importlib.import_module("adreno_llms_b200.synth"), importlib.import_module("adreno_llms_b200.decode_step")


def _snapshot(ctx, step):
    sh = step.shape
    return {
        "logits": step.read_logits().view(np.uint16).copy(),
        "token": step.read_token(),
        "resid": ctx.download(step.resid, (1, sh.hidden), np.uint16),
        "q": ctx.download(step.q, (1, sh.q_dim), np.uint16),
        "k": ctx.download(step.k, (1, sh.kv_dim), np.uint16),
        "v": ctx.download(step.v, (1, sh.kv_dim), np.uint16),
        "act": ctx.download(step.act, (1, sh.ffn), np.uint16),
    }


def _poison(ctx, step):
    """Outputs that the step must overwrite: a stale value from an earlier run must not pass."""
    sh = step.shape
    for buf, n in ((step.q, sh.q_dim), (step.k, sh.kv_dim), (step.v, sh.kv_dim), (step.act, sh.ffn), (step.logits, step.vocab_n)):
        ctx.upload(np.full(n, 0x7E00, np.uint16), buf)
    ctx.upload(np.full(1, -7, np.int32), step.token)


SHAPES = {
    "smollm2": (576, 576, 192, 1536, 4100),       # ragged vocabulary slice
    "lfm2": (1024, 1024, 512, 4608, 4096),
    "qwen": (896, 896, 128, 4864, 8192),
}


CASES = [("lfm2", f, w) for f in ("int8", "fp16", "q4") for w in ("fixed", "fixed+norm", "chained+norm")] + \
        [(s, f, w) for s in ("smollm2", "qwen") for f in ("int8", "fp16", "q4") for w in ("fixed", "chained+norm")]


@pytest.mark.parametrize("shape_name,fmt,wiring", CASES)
def test_resident_replay_equals_separate_launches(nnb, ctx, fmt, wiring, shape_name):
    synth, dstep = _mods()
    H, Q, KV, F, V = SHAPES[shape_name]
    layers = 3
    shape = synth.ModelShape(shape_name, H, layers, Q, KV, F, V)
    step = dstep.DecodeStep(ctx, shape, fmt, M=1, n_sets=1, norm="norm" in wiring, chained="chained" in wiring)
    _poison(ctx, step)
    step.enqueue(0)
    ctx.sync()
    eager = _snapshot(ctx, step)
    lg = eager["logits"].view(np.float16).astype(np.float32).reshape(-1)
    assert np.isfinite(lg).all() and eager["token"] == int(np.argmax(lg))
    step.record()
    plan = step.plans[0]
    assert ctx.L.nn_plan_num_recorded(plan) == 4 * layers + 1
    assert step.resident_runs() >= 1
    assert step.kernels_per_step <= 2           # the first QKV may stay a launch of its own (see the wiring)
    for rep in range(3):                        # replays: every launch has its own epoch
        step.reset_residual()
        _poison(ctx, step)
        before = ctx.launch_count()
        step.launch(0)
        ctx.sync()
        assert ctx.launch_count() - before == step.kernels_per_step
        got = _snapshot(ctx, step)
        for key in eager:
            assert np.array_equal(got[key], eager[key]), f"{key} differs from the separate launches (replay {rep})"
    for st in step.sets:
        for w in st.values():
            w.release()


@pytest.mark.parametrize("fmt", ["int8", "fp16", "q4"])
def test_chained_step_follows_the_oracle_chain(nnb, ctx, fmt):
    """The data flows through the step as in the model; follow it on the CPU with the oracle's
    kernels (RMSNorm pinned to the reference's) and compare what the replay leaves behind."""
    synth, dstep = _mods()
    shape = synth.ModelShape("tiny-chain", 1024, 3, 1024, 512, 4608, 4096)
    step = dstep.DecodeStep(ctx, shape, fmt, M=1, n_sets=1, keep_host=True, norm=True, chained=True)
    step.record()
    assert step.kernels_per_step == 1 and step.resident_runs() == 1
    step.launch(0)
    ctx.sync()
    h = step.host
    r = step.resid0.copy()
    for layer in range(shape.layers):
        q = cpu.linear(fmt, cpu.rmsnorm(r, h["gamma"], step.eps), *h[f"qkv.{layer}.0"])
        r = cpu.linear_residual(fmt, q, *h[f"o_add.{layer}.0"], r)
        act = cpu.linear_swiglu(fmt, cpu.rmsnorm(r, h["gamma"], step.eps), *h[f"gate_up.{layer}.0"], *h[f"gate_up.{layer}.1"])
        r = cpu.linear_residual(fmt, act, *h[f"down_add.{layer}.0"], r)
    logits = cpu.linear(fmt, r, *h["lm_head.-1.0"])
    check_close(ctx.download(step.q, (1, shape.q_dim), np.uint16).view(np.float16), q, tol=3e-3, what=f"q {fmt}")
    check_close(ctx.download(step.act, (1, shape.ffn), np.uint16).view(np.float16), act, tol=3e-3, what=f"act {fmt}")
    check_close(ctx.download(step.resid, (1, shape.hidden), np.uint16).view(np.float16), r, tol=2e-3, what=f"residual {fmt}")
    got = step.read_logits()
    check_close(got, logits, tol=3e-3, what=f"logits {fmt}")
    assert step.read_token() == cpu.argmax_half(got)


def test_other_work_between_operators_splits_the_runs(nnb, ctx):
    """A copy enqueued by the caller between two operators stays where it was recorded; the
    operators on either side form runs of their own, and an M = 2 call stays a separate launch."""
    fmt, K, N = "int8", 576, 1536
    W1, s1 = make_weight(fmt, N, K, 501)
    W2, s2 = make_weight(fmt, K, N, 502)
    W3, s3 = make_weight(fmt, N, K, 503)
    w1, w2, w3 = (nnb.QuantWeight(ctx, fmt, W, s) for W, s in ((W1, s1), (W2, s2), (W3, s3)))
    x = make_x(1, K, 504)
    x2 = make_x(2, K, 505)
    dx, dx2 = ctx.upload(x.view(np.uint16)), ctx.upload(x2.view(np.uint16))
    a, b, b_copy, c_, d2 = ctx.alloc(N * 2), ctx.alloc(K * 2), ctx.alloc(K * 2), ctx.alloc(N * 2), ctx.alloc(2 * N * 2)

    def enqueue():
        ctx.linear(1, N, K, dx, w1.buf, a)          # run 1
        ctx.linear(1, K, N, a, w2.buf, b)
        ctx.L.nn_buf_copy(ctx.h, b_copy, b, K * 2)  # the caller's own work on the stream
        ctx.linear(1, N, K, b_copy, w3.buf, c_)     # run 2
        ctx.linear(1, K, N, c_, w2.buf, b)
        ctx.linear(2, N, K, dx2, w1.buf, d2)        # M = 2: a launch of its own
        ctx.linear(1, N, K, b, w3.buf, a)           # a single operator: stays as recorded

    def read():
        ctx.sync()
        return [ctx.download(buf, (n,), np.uint16).copy() for buf, n in ((a, N), (b, K), (b_copy, K), (c_, N), (d2, 2 * N))]

    enqueue()
    want = read()
    for buf, n in ((a, N), (b, K), (b_copy, K), (c_, N), (d2, 2 * N)):
        ctx.upload(np.full(n, 0x7E00, np.uint16), buf)
    ctx.plan_begin()
    enqueue()
    plan = ctx.plan_end()
    assert ctx.L.nn_plan_num_recorded(plan) == 7        # the M = 2 call is two launches: staging, projection
    assert ctx.L.nn_plan_num_resident_runs(plan) == 2
    assert ctx.L.nn_plan_num_kernels(plan) == 5
    for _ in range(2):
        ctx.plan_launch(plan)
        got = read()
        for g, w in zip(got, want):
            assert np.array_equal(g, w)
    # against the oracle as well
    ya = cpu.linear(fmt, x, W1, s1)
    yb = cpu.linear(fmt, ya, W2, s2)
    check_close(want[2].view(np.float16)[None, :], yb, what="copied intermediate")
    ctx.L.nn_plan_free(plan)
    for w in (w1, w2, w3):
        w.release()
    for buf in (dx, dx2, a, b, b_copy, c_, d2):
        ctx.free(buf)


def test_withheld_output_times_out_and_context_survives(nnb, ctx):
    """Fault injected on the host: one operator of a resident run never hands its output on.  The
    operators that wait for it must give up after the plan's limit, nn_sync must report
    NN_ERR_TIMEOUT, and the same plan must run correctly once the fault is taken away."""
    synth, dstep = _mods()
    shape = synth.ModelShape("tiny-fault", 576, 2, 576, 192, 1536, 2048)
    step = dstep.DecodeStep(ctx, shape, "int8", M=1, n_sets=1, norm=True, chained=True)
    step.enqueue(0)
    ctx.sync()
    want_logits, want_tok = step.read_logits().view(np.uint16).copy(), step.read_token()
    step.record()
    plan = step.plans[0]
    assert step.resident_runs() == 1
    assert ctx.L.nn_plan_set_wait_limit(plan, 50) == 0
    assert ctx.L.nn_plan_withhold_output(plan, 0, 2) == 0      # gate/up of layer 0 keeps its result to itself
    step.reset_residual()
    step.launch(0)
    with pytest.raises(nnb.NNError) as ei:
        ctx.sync()
    assert ei.value.code == nnb.NN_ERR_TIMEOUT
    # bad arguments are refused
    assert ctx.L.nn_plan_withhold_output(plan, 1, 0) == nnb.NN_ERR_ARG
    assert ctx.L.nn_plan_withhold_output(plan, 0, 99) == nnb.NN_ERR_ARG
    assert ctx.L.nn_plan_set_wait_limit(plan, 0) == nnb.NN_ERR_ARG
    # the fault removed: the plan and the context work as before
    assert ctx.L.nn_plan_withhold_output(plan, 0, -1) == 0
    for _ in range(2):
        step.reset_residual()
        step.launch(0)
        ctx.sync()
        assert np.array_equal(step.read_logits().view(np.uint16), want_logits)
        assert step.read_token() == want_tok
    W, _ = make_weight("fp16", 256, 128, 5)
    x = make_x(1, 128, 6)
    dw, dx, out = ctx.upload(W.view(np.uint16)), ctx.upload(x.view(np.uint16)), ctx.alloc(512)
    ctx.linear(1, 256, 128, dx, dw, out)
    got = ctx.download(out, (1, 256), np.uint16).view(np.float16)
    assert cpu.rel_l2(got, cpu.linear("fp16", x, W, None, order=2)) <= TOL
    for b in (dw, dx, out):
        ctx.free(b)


def test_host_copies_recorded_with_the_step(nnb, ctx):
    """The host program's own copies between nn_plan_begin and nn_plan_end are part of the plan (the
    reference records its whole token into the replayed queue): a replay copies the CURRENT contents of
    the pinned input in, runs the operators as one resident launch, and copies the results out."""
    fmt, K, N = "int8", 576, 1536
    W1, s1 = make_weight(fmt, N, K, 601)
    W2, s2 = make_weight(fmt, K, N, 602)
    w1, w2 = nnb.QuantWeight(ctx, fmt, W1, s1), nnb.QuantWeight(ctx, fmt, W2, s2)
    L = ctx.L
    hx, hy = L.nn_host_alloc(K * 2), L.nn_host_alloc(K * 2)
    dx, da, dy = ctx.alloc(K * 2), ctx.alloc(N * 2), ctx.alloc(K * 2)
    ctx.plan_begin()
    nnb._check(L.nn_buf_write(ctx.h, dx, 0, hx, K * 2))
    ctx.linear(1, N, K, dx, w1.buf, da)
    ctx.linear(1, K, N, da, w2.buf, dy)
    nnb._check(L.nn_buf_read(ctx.h, hy, dy, 0, K * 2))
    plan = ctx.plan_end()
    assert L.nn_plan_num_resident_runs(plan) == 1 and L.nn_plan_num_kernels(plan) == 1
    for rep in range(3):
        x = make_x(1, K, 610 + rep)
        ctypes.memmove(hx, x.ctypes.data, K * 2)
        ctx.plan_launch(plan)
        ctx.sync()
        got = np.ctypeslib.as_array(ctypes.cast(hy, ctypes.POINTER(ctypes.c_uint16)), (K,)).copy().view(np.float16)
        want = cpu.linear(fmt, cpu.linear(fmt, x, W1, s1), W2, s2)
        check_close(got[None, :], want, what=f"recorded copies, replay {rep}")
    L.nn_plan_free(plan)
    L.nn_host_free(hx)
    L.nn_host_free(hy)
    for w in (w1, w2):
        w.release()
    for b in (dx, da, dy):
        ctx.free(b)


@pytest.mark.parametrize("norm", [False, True])
@pytest.mark.parametrize("fmt", ["int8", "fp16", "q4"])
def test_qkv_bias_rides_in_the_resident_step(nnb, ctx, fmt, norm):
    """Qwen's q/k/v bias (bias_add_rowmajor after the fused QKV projection, src/models/qwen2-5-0-5b/src/layers/
    attention.cpp:413-469) is part of the projection's epilogue, so a Qwen-shaped step with biases still replays as
    one resident launch, with the bits of the calls made one by one, and follows the oracle's chain."""
    synth, dstep = _mods()
    shape = synth.ModelShape("qwen-bias", 896, 2, 896, 128, 4864, 4096)
    step = dstep.DecodeStep(ctx, shape, fmt, M=1, n_sets=1, keep_host=True, chained=True, qkv_bias=True, norm=norm)
    _poison(ctx, step)
    before = ctx.launch_count()
    step.enqueue(0)
    assert ctx.launch_count() - before == 4 * shape.layers + 1      # the bias costs no launch of its own
    ctx.sync()
    eager = _snapshot(ctx, step)
    step.record()
    assert step.kernels_per_step == 1 and step.resident_runs() == 1
    for rep in range(2):
        step.reset_residual()
        _poison(ctx, step)
        step.launch(0)
        ctx.sync()
        got = _snapshot(ctx, step)
        for key in eager:
            assert np.array_equal(got[key], eager[key]), f"{key} differs from the separate launches (replay {rep})"
    # the oracle's chain, with the reference's two roundings for the bias
    h = step.host
    r = step.resid0.copy()
    nrm = (lambda v: cpu.rmsnorm(v, h["gamma"], step.eps)) if norm else (lambda v: v)
    for layer in range(shape.layers):
        q = cpu.linear(fmt, nrm(r), *h[f"qkv.{layer}.0"])
        q = (q.astype(np.float32) + h[f"qkv_bias.{layer}"][0].astype(np.float32)[None, :]).astype(np.float16)
        r = cpu.linear_residual(fmt, q, *h[f"o_add.{layer}.0"], r)
        act = cpu.linear_swiglu(fmt, nrm(r), *h[f"gate_up.{layer}.0"], *h[f"gate_up.{layer}.1"])
        r = cpu.linear_residual(fmt, act, *h[f"down_add.{layer}.0"], r)
    check_close(ctx.download(step.q, (1, shape.q_dim), np.uint16).view(np.float16), q, tol=3e-3, what=f"q with bias {fmt}")
    check_close(ctx.download(step.resid, (1, shape.hidden), np.uint16).view(np.float16), r, tol=3e-3, what=f"residual with bias {fmt}")

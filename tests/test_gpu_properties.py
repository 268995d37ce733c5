"""Full-size checks through size-independent properties (the oracle is too slow to redo
every full-size product): linearity in x, unit vectors pick dequantised columns, a
row-sampled comparison against the oracle, recorded-plan replay equals eager calls."""
import os

import numpy as np
import pytest

from oracle import cpu
from helpers import check_close, make_weight, make_x

pytestmark = pytest.mark.gpu


def _run(ctx, qw, x, N, K):
    M = x.shape[0]
    xb = ctx.upload(x.view(np.uint16))
    ob = ctx.upload(np.full((M, N), 0x7E00, np.uint16))
    ctx.linear(M, N, K, xb, qw.buf, ob)
    out = ctx.download(ob, (M, N), np.uint16).view(np.float16)
    ctx.free(xb)
    ctx.free(ob)
    return out


@pytest.mark.parametrize("fmt,N,K", [("int8", 151936, 896), ("int8", 49152, 576), ("q4", 65536, 1024), ("q4", 28672, 8192),
                                     ("fp16", 151936, 896)])
def test_full_size_projection(nnb, ctx, fmt, N, K):
    W, s = make_weight(fmt, N, K, 3000 + K)
    qw = nnb.QuantWeight(ctx, fmt, W, s)
    x = make_x(1, K, 3001)
    y = _run(ctx, qw, x, N, K)
    assert np.isfinite(y.astype(np.float32)).all()
    # rows sampled across the whole range (first, last, tile edges, random) against the oracle
    rng = np.random.default_rng(5)
    rows = np.unique(np.concatenate([[0, 1, 31, 32, 127, 128, N - 129, N - 33, N - 1], rng.integers(0, N, 2000)]))
    want = cpu.linear(fmt, x, W[rows], None if s is None else s[rows], threads=8)
    check_close(y[:, rows], want, what=f"{fmt} {N}x{K} sampled rows")
    # linearity: W(2x) == 2 W x exactly wherever the output is a normal fp16 number
    # (power-of-two scaling commutes with every rounding except the subnormal one)
    y2 = _run(ctx, qw, (x.astype(np.float32) * 2).astype(np.float16), N, K)
    normal = np.abs(y.astype(np.float32)) >= 2.0 ** -13
    assert normal.mean() > 0.99
    assert np.array_equal(y2.astype(np.float32)[normal], (y.astype(np.float32) * 2)[normal])
    # batched rows are independent: row 1 of a 2-row batch equals the single call
    xb2 = np.concatenate([make_x(1, K, 3002), x])
    yb = _run(ctx, qw, xb2, N, K)
    check_close(yb[1:2], y, tol=2e-4, what="batch independence")
    ctx.L.nn_unregister_weight(ctx.h, qw.buf)
    ctx.free(qw.buf)
    if qw.scale:
        ctx.free(qw.scale)


def test_recorded_step_equals_eager(nnb, ctx):
    """A recorded plan (the reference's recorded-queue replay) gives the eager results, and
    replaying it does not re-record."""
    import importlib
    synth = importlib.import_module("adreno_llms_b200.synth")
    dstep = importlib.import_module("adreno_llms_b200.decode_step")
    shape = synth.ModelShape("tiny", 576, 2, 576, 192, 1536, 4096)
    for fmt in ("int8", "fp16", "q4"):
        if fmt == "q4":
            shape = synth.ModelShape("tiny-q4", 1024, 2, 1024, 512, 4608, 4096)
        step = dstep.DecodeStep(ctx, shape, fmt, M=1, n_sets=2, keep_host=True)
        step.enqueue(0)
        ctx.sync()
        eager_logits, eager_tok = step.read_logits(), step.read_token()
        step.reset_residual()
        n = step.record()
        assert ctx.L.nn_plan_num_recorded(step.plans[0]) == 4 * shape.layers + 1   # lm_head and the greedy pick are one launch
        if os.environ.get("NNB_PLAN_SEPARATE"):       # the plan kept as its separate launches
            assert n == 4 * shape.layers + 1 and step.resident_runs() == 0
        else:
            assert n == 1 and step.resident_runs() == 1   # ... and the whole step replays as one resident launch
        before = ctx.launch_count()
        step.launch(0)
        ctx.sync()
        assert ctx.launch_count() - before == n
        assert np.array_equal(step.read_logits().view(np.uint16), eager_logits.view(np.uint16))
        assert step.read_token() == eager_tok == cpu.argmax_half(eager_logits)
        # logits against the oracle on the same weights
        W, s = step.host["lm_head.-1.0"]
        check_close(eager_logits, cpu.linear(fmt, step.host["x_h"], W, s), what=f"step lm_head {fmt}")
        # the residual stream after 2 layers x 2 in-place adds
        r = step.resid0.copy()
        for layer in range(shape.layers):
            Wo, so = step.host[f"o_add.{layer}.0"]
            r = cpu.linear_residual(fmt, step.host["x_attn"], Wo, so, r)
            Wd, sd = step.host[f"down_add.{layer}.0"]
            r = cpu.linear_residual(fmt, step.host["x_act"], Wd, sd, r)
        got = ctx.download(step.resid, (1, shape.hidden), np.uint16).view(np.float16)
        check_close(got, r, what=f"step residual {fmt}")


@pytest.mark.parametrize("fmt", ["int8", "fp16", "q4"])
def test_step_with_fused_rmsnorm_follows_the_oracle_chain(nnb, ctx, fmt):
    """With the layer norms fused into QKV and gate/up the residual stream feeds the projections:
    follow two layers on the CPU (oracle RMSNorm -> oracle projections) and compare what the
    recorded step leaves in the q / act buffers of the last layer and in the residual stream."""
    import importlib
    synth = importlib.import_module("adreno_llms_b200.synth")
    dstep = importlib.import_module("adreno_llms_b200.decode_step")
    shape = synth.ModelShape("tiny-norm", 1024, 2, 1024, 512, 4608, 2048)
    step = dstep.DecodeStep(ctx, shape, fmt, M=1, n_sets=1, keep_host=True, norm=True)
    step.record()
    assert ctx.L.nn_plan_num_recorded(step.plans[0]) == 4 * shape.layers + 1          # the norms add no launch
    step.launch(0)
    ctx.sync()
    h = step.host
    r = step.resid0.copy()
    for layer in range(shape.layers):
        xn = cpu.rmsnorm(r, h["gamma"], step.eps)
        q = cpu.linear(fmt, xn, *h[f"qkv.{layer}.0"])
        r = cpu.linear_residual(fmt, h["x_attn"], *h[f"o_add.{layer}.0"], r)
        xn2 = cpu.rmsnorm(r, h["gamma"], step.eps)
        act = cpu.linear_swiglu(fmt, xn2, *h[f"gate_up.{layer}.0"], *h[f"gate_up.{layer}.1"])
        r = cpu.linear_residual(fmt, h["x_act"], *h[f"down_add.{layer}.0"], r)
    check_close(ctx.download(step.q, (1, shape.q_dim), np.uint16).view(np.float16), q, tol=2e-3, what=f"q after norm {fmt}")
    check_close(ctx.download(step.act, (1, shape.ffn), np.uint16).view(np.float16), act, tol=2e-3, what=f"act after norm {fmt}")
    check_close(ctx.download(step.resid, (1, shape.hidden), np.uint16).view(np.float16), r, what=f"residual {fmt}")

"""RMSNorm feeding the projections: the stand-alone kernel and the fused prologue, against the
oracle (whose RMSNorm is pinned bit for bit to the reference's rmsnorm_forward)."""
import numpy as np
import pytest

from helpers import TOL, check_close, make_weight, make_x
from oracle import cpu

pytestmark = pytest.mark.gpu
FMTS = ["fp16", "int8", "q4"]


def _gamma(K, seed):
    return (1.0 + 0.1 * np.random.default_rng(seed).standard_normal(K)).astype(np.float32).astype(np.float16)


@pytest.mark.parametrize("rows,cols,eps", [(1, 576, 1e-5), (3, 1024, 1e-5), (2, 70, 1e-6), (5, 4608, 1e-5)])
def test_rmsnorm_matches_oracle(nnb, ctx, rows, cols, eps):
    x = (make_x(rows, cols, 11).astype(np.float32) * 3.0).astype(np.float16)
    g = _gamma(cols, 12)
    dx, dg, out = ctx.upload(x.view(np.uint16)), ctx.upload(g.view(np.uint16)), ctx.alloc(rows * cols * 2)
    ctx.rmsnorm(rows, cols, dx, dg, eps, out)
    got = ctx.download(out, (rows, cols), np.uint16).view(np.float16)
    want = cpu.rmsnorm(x, g, eps)
    check_close(got, want, what="rmsnorm")
    # identical up to isolated last-place roundings (the sums are taken in a different order)
    assert (got.view(np.uint16) != want.view(np.uint16)).mean() < 0.02
    for b in (dx, dg, out):
        ctx.free(b)


@pytest.mark.parametrize("fmt", FMTS)
@pytest.mark.parametrize("M,N,K", [(1, 576, 576), (1, 1536, 1024), (5, 1056, 1024), (16, 640, 1536), (20, 512, 1024), (2, 300, 200)])
def test_rmsnorm_linear_fused_prologue(nnb, ctx, fmt, M, N, K):
    if fmt == "q4" and K % 32:
        pytest.skip("Q4 needs K % 32 == 0")
    eps = 1e-5
    W, s = make_weight(fmt, N, K, 21)
    x = (make_x(M, K, 22).astype(np.float32) * 2.5).astype(np.float16)
    g = _gamma(K, 23)
    qw = nnb.QuantWeight(ctx, fmt, W, s)
    dx, dg, out = ctx.upload(x.view(np.uint16)), ctx.upload(g.view(np.uint16)), ctx.alloc(M * N * 2)
    before = ctx.launch_count()
    ctx.rmsnorm_linear(M, N, K, dx, dg, eps, qw.buf, out)
    launches = ctx.launch_count() - before
    got = ctx.download(out, (M, N), np.uint16).view(np.float16)
    want = cpu.linear(fmt, cpu.rmsnorm(x, g, eps), W, s)
    check_close(got, want, what=f"rmsnorm->linear {fmt} M={M} K={K}")
    if M == 1 and K % 128 == 0:
        assert launches == 1            # the norm is the projection kernel's prologue
    elif M <= 16 and K % 128 == 0:
        assert launches == 2            # batched: the norm runs once, in the launch that stages the activations
    qw.release()
    for b in (dx, dg, out):
        ctx.free(b)


@pytest.mark.parametrize("fmt", FMTS)
def test_rmsnorm_qkv_and_gate_up(nnb, ctx, fmt):
    H, Q, KV, F, eps = 1024, 1024, 512, 4608, 1e-5
    x = (make_x(1, H, 31).astype(np.float32) * 4.0).astype(np.float16)
    g = _gamma(H, 32)
    xn = cpu.rmsnorm(x, g, eps)
    dx, dg = ctx.upload(x.view(np.uint16)), ctx.upload(g.view(np.uint16))
    ws = [make_weight(fmt, n, H, 33 + i) for i, n in enumerate((Q, KV, KV))]
    qws = [nnb.QuantWeight(ctx, fmt, W, s) for W, s in ws]
    outs = [ctx.alloc(n * 2) for n in (Q, KV, KV)]
    ctx.rmsnorm_linear_qkv(1, H, dx, dg, eps, qws[0].buf, Q, qws[1].buf, KV, qws[2].buf, KV, *outs)
    for (W, s), o, n in zip(ws, outs, (Q, KV, KV)):
        check_close(ctx.download(o, (1, n), np.uint16).view(np.float16), cpu.linear(fmt, xn, W, s), what=f"rmsnorm->qkv {fmt}")
    Wg, sg = make_weight(fmt, F, H, 41)
    Wu, su = make_weight(fmt, F, H, 42)
    qg, qu = nnb.QuantWeight(ctx, fmt, Wg, sg), nnb.QuantWeight(ctx, fmt, Wu, su)
    act = ctx.alloc(F * 2)
    ctx.rmsnorm_gate_up_silu(1, F, H, dx, dg, eps, qg.buf, qu.buf, act)
    check_close(ctx.download(act, (1, F), np.uint16).view(np.float16), cpu.linear_swiglu(fmt, xn, Wg, sg, Wu, su), what=f"rmsnorm->swiglu {fmt}")
    for q in qws + [qg, qu]:
        q.release()
    for b in [dx, dg, act] + outs:
        ctx.free(b)

"""Parity at the full sizes of the model configs beyond single-token calls: batched decode and
prefill row counts on the largest weights (rows sampled across the whole range against the
oracle), and the greedy token of a thousand hidden vectors per lm_head against the oracle's."""
import numpy as np
import pytest

from oracle import cpu
from helpers import check_close, make_weight, make_x, report

pytestmark = pytest.mark.gpu


def _sample_rows(N, count, seed):
    rng = np.random.default_rng(seed)
    edges = [0, 1, 31, 32, 33, 127, 128, 129, 255, 256, N // 2 - 1, N // 2, N - 257, N - 129, N - 128, N - 33, N - 32, N - 1]
    return np.unique(np.concatenate([edges, rng.integers(0, N, count)]))


FULL = [("q4", 28672, 8192, (8, 16, 32, 128)),      # the largest Q4 weight of the configs
        ("int8", 151936, 896, (4, 16, 64, 256)),    # Qwen2.5 lm_head
        ("fp16", 151936, 896, (64, 512)),
        ("q4", 65536, 1024, (8,))]                  # LFM2.5 lm_head


@pytest.mark.parametrize("fmt,N,K,Ms", FULL)
def test_full_size_batched_rows_against_the_oracle(nnb, ctx, fmt, N, K, Ms):
    W, s = make_weight(fmt, N, K, 4000 + K)
    qw = nnb.QuantWeight(ctx, fmt, W, s)
    rows = _sample_rows(N, 400, 41)
    Wr, sr = W[rows], None if s is None else s[rows]
    for M in Ms:
        x = make_x(M, K, 4001 + M)
        xb = ctx.upload(x.view(np.uint16))
        ob = ctx.upload(np.full((M, N), 0x7E00, np.uint16))
        ctx.linear(M, N, K, xb, qw.buf, ob)
        got = ctx.download(ob, (M, N), np.uint16).view(np.float16)
        assert np.isfinite(got.astype(np.float32)).all()       # every element written
        want = cpu.linear(fmt, x, Wr, sr, threads=8)
        check_close(got[:, rows], want, what=f"{fmt} {N}x{K} M={M} sampled rows")
        ctx.free(xb)
        ctx.free(ob)
    qw.release()


HEADS = [("int8", 49152, 576), ("int8", 151936, 896), ("q4", 65536, 1024), ("fp16", 49152, 576)]


@pytest.mark.parametrize("fmt,V,H", HEADS)
def test_greedy_token_of_a_thousand_vectors(nnb, ctx, fmt, V, H):
    """The fused lm_head + arg-max against the oracle's arg-max of its own fp16 logits, for 1000
    hidden vectors.  The oracle's pick is found exactly without 1000 full oracle products: an
    fp32 BLAS product of the dequantised weights (within 1e-5 of the oracle's sums) selects every
    row within four fp16 steps of the maximum, and the oracle itself is run on those rows."""
    trials = 1000
    W, s = make_weight(fmt, V, H, 5000 + H)
    Wd = cpu.dequant(fmt, W, s).astype(np.float32)
    X = make_x(trials, H, 5001)
    qw = nnb.QuantWeight(ctx, fmt, W, s)
    lb, ib = ctx.alloc(V * 2), ctx.alloc(4)
    xbuf = ctx.upload(X.view(np.uint16))
    approx = X.astype(np.float32) @ Wd.T                     # [trials, V]
    agree, flips, margins = 0, [], []
    for t in range(trials):
        a = approx[t]
        top = float(a.max())
        step = float(np.spacing(np.float16(abs(top))))
        cand = np.flatnonzero(a >= top - 4 * step)
        exact = cpu.linear(fmt, X[t:t + 1], W[cand], None if s is None else s[cand]).reshape(-1)
        best = cand[cpu.argmax_half(exact)]                  # lowest index among equal fp16 values
        srt = np.sort(exact.astype(np.float32))
        margins.append((srt[-1] - srt[-2]) / step if len(srt) > 1 else 4.0)
        ctx.L.nn_linear_argmax(ctx.h, V, H, xbuf + t * H * 2, qw.buf, lb, ib)
        tok = int(ctx.download(ib, (1,), np.int32)[0])
        if tok == best:
            agree += 1
        else:
            # a different pick is acceptable only between logits the oracle itself has within one fp16 step
            lo = cpu.linear(fmt, X[t:t + 1], W[[tok, best]], None if s is None else s[[tok, best]]).astype(np.float32).reshape(-1)
            flips.append((t, tok, int(best), float(abs(lo[0] - lo[1]) / step)))
    margins = np.asarray(margins)
    report(f"greedy token {fmt} {V}x{H}: {agree}/{trials} agree; flips (vector, ours, oracle, gap in fp16 steps): {flips}; "
           f"vectors whose top two oracle logits are within one fp16 step: {int((margins <= 1).sum())}")
    for _, _, _, gap in flips:
        assert gap <= 1.0
    assert agree >= trials - max(2, int((margins <= 1).sum()))
    qw.release()
    for b in (lb, ib, xbuf):
        ctx.free(b)

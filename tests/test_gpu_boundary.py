"""The rest of the operator surface around the projections: Qwen's q/k/v bias
(bias_add_rowmajor, src/models/qwen2-5-0-5b/kernels/bias_add.cl:18-40), the per-launch
profile (src/models/lfm2-5-350m/src/kernel_profiler.cpp:18-62), writes that stay inside the
output, and activations at the edges of fp16 on the int8 path."""
import numpy as np
import pytest

from oracle import cpu
from helpers import TOL, alloc_with_canary, check_canary, check_close, make_weight, make_x, report

pytestmark = pytest.mark.gpu


def _bias_add(y_half, bias_half):
    """The reference's two roundings: the projection's fp16 result, plus the bias in fp32, to fp16."""
    return (y_half.astype(np.float32) + bias_half.astype(np.float32)[None, :]).astype(np.float16)


@pytest.mark.parametrize("fmt", ["int8", "fp16", "q4"])
@pytest.mark.parametrize("M", [1, 5, 40])
def test_qkv_with_bias(nnb, ctx, fmt, M):
    K, Ns = 896, (896, 128, 128)           # Qwen2.5-0.5B: the one model with a q/k/v bias
    Ws = [make_weight(fmt, n, K, 160 + i) for i, n in enumerate(Ns)]
    bs = [(np.random.default_rng(170 + i).standard_normal(n) * 0.5).astype(np.float16) for i, n in enumerate(Ns)]
    x = make_x(M, K, 166)
    qs = [nnb.QuantWeight(ctx, fmt, W, s) for W, s in Ws]
    xb = ctx.upload(x.view(np.uint16))
    bb = [ctx.upload(b.view(np.uint16)) for b in bs]
    outs = [alloc_with_canary(ctx, M * n * 2) for n in Ns]
    plain = [ctx.alloc(M * n * 2) for n in Ns]
    ctx.linear_qkv(M, K, xb, qs[0].buf, Ns[0], qs[1].buf, Ns[1], qs[2].buf, Ns[2], *plain)
    ctx.linear_qkv_bias(M, K, xb, qs[0].buf, Ns[0], qs[1].buf, Ns[1], qs[2].buf, Ns[2], *bb, *outs)
    for (W, s), b, ob, pb, n in zip(Ws, bs, outs, plain, Ns):
        got = ctx.download(ob, (M, n), np.uint16).view(np.float16)
        ours = ctx.download(pb, (M, n), np.uint16).view(np.float16)
        # exactly the reference's bias kernel applied to our projection ...
        assert np.array_equal(got.view(np.uint16), _bias_add(ours, b).view(np.uint16))
        # ... and within the path's bound of the oracle's projection with the same bias kernel
        want = _bias_add(cpu.linear(fmt, x, W, s, threads=4), b)
        check_close(got, want, what=f"qkv+bias {fmt} M={M} N={n}")
        check_canary(ctx, ob, M * n * 2, f"qkv+bias {fmt} M={M} N={n}")
    # the bias kernel by itself, in place
    ctx.bias_add(M, Ns[0], plain[0], bb[0])
    again = ctx.download(plain[0], (M, Ns[0]), np.uint16)
    assert np.array_equal(again, ctx.download(outs[0], (M, Ns[0]), np.uint16))
    assert ctx.L.nn_bias_add(ctx.h, 1, 0, plain[0], bb[0]) == nnb.NN_ERR_ARG
    assert ctx.L.nn_bias_add(ctx.h, 0, 8, plain[0], bb[0]) == 0
    for q in qs:
        q.release()
    for b in [xb] + bb + outs + plain:
        ctx.free(b)


def test_profile_labels_and_counts(nnb, built_lib, monkeypatch):
    """NNOPT_KERNEL_PROFILE=1 at nn_init: every call lands under the reference's label form,
    a plan replay is one entry, and the table holds the counts."""
    monkeypatch.setenv("NNOPT_KERNEL_PROFILE", "1")
    c = nnb.Context(0)
    try:
        assert c.profile_enabled()
        N, K = 4608, 1024
        W, s = make_weight("int8", N, K, 181)
        W2, s2 = make_weight("int8", K, N, 182)
        qw, qw2 = nnb.QuantWeight(c, "int8", W, s), nnb.QuantWeight(c, "int8", W2, s2)
        x = make_x(1, K, 183)
        xb, ob, rb = c.upload(x.view(np.uint16)), c.alloc(N * 2), c.upload(make_x(1, K, 184).view(np.uint16))
        for _ in range(3):
            c.linear(1, N, K, xb, qw.buf, ob)
        c.linear_add(1, K, N, ob, qw2.buf, rb)
        c.plan_begin()
        c.linear(1, N, K, xb, qw.buf, ob)
        c.linear_add(1, K, N, ob, qw2.buf, rb)
        plan = c.plan_end()
        for _ in range(2):
            c.plan_launch(plan)
        c.sync()
        text = c.profile_report()
        rows = {ln.split()[0]: ln.split() for ln in text.splitlines() if ln and not ln.startswith("=") and not ln.startswith("label")}
        assert int(rows["gemv_m1_K1024_N4608_int8"][3]) == 3, text
        assert int(rows["gemv_m1_K4608_N1024_int8_add"][3]) == 1, text
        replay = [k for k in rows if k.startswith("plan_replay")]
        assert len(replay) == 1 and int(rows[replay[0]][3]) == 2, text
        for r in rows.values():
            assert float(r[1]) > 0 and float(r[4]) > 0 and float(r[5]) >= float(r[4]) - 1e-6
        shares = sum(float(r[2].rstrip("%")) for r in rows.values())
        assert abs(shares - 100.0) < 0.1
        # the results are the unprofiled ones
        got = c.download(ob, (1, N), np.uint16).view(np.float16)
        check_close(got, cpu.linear("int8", x, W, s), what="profiled int8 gemv")
        # reset empties the table
        c.profile_report(reset=True)
        assert "gemv_m1" not in c.profile_report()
        c.L.nn_plan_free(plan)
    finally:
        c.close()
    monkeypatch.delenv("NNOPT_KERNEL_PROFILE")
    c2 = nnb.Context(0)
    assert not c2.profile_enabled()
    c2.close()


@pytest.mark.parametrize("fmt,N,K,M", [("int8", 100, 96, 1), ("int8", 1536, 576, 1), ("fp16", 33, 64, 3), ("q4", 4608, 1024, 1), ("q4", 40, 64, 9),
                                       ("int8", 1000, 200, 2), ("fp16", 577, 70, 1), ("int8", 900, 576, 33), ("q4", 1000, 1024, 17)])
def test_nothing_is_written_past_the_output(nnb, ctx, fmt, N, K, M):
    """Every path (stream kernel, generic kernel, tensor-core GEMM; ragged row counts) leaves the
    256 patterned bytes behind its output alone and writes every element before them."""
    W, s = make_weight(fmt, N, K, 190 + N)
    x = make_x(M, K, 191)
    qw = nnb.QuantWeight(ctx, fmt, W, s)
    xb = ctx.upload(x.view(np.uint16))
    ob = alloc_with_canary(ctx, M * N * 2)
    ctx.linear(M, N, K, xb, qw.buf, ob)
    got = ctx.download(ob, (M, N), np.uint16).view(np.float16)
    check_close(got, cpu.linear(fmt, x, W, s, threads=4), what=f"canary {fmt} {N}x{K} M={M}")
    check_canary(ctx, ob, M * N * 2, f"{fmt} {N}x{K} M={M}")
    if M == 1:
        ib = alloc_with_canary(ctx, 4)
        ctx.linear_argmax(N, K, xb, qw.buf, ob, ib)
        check_canary(ctx, ib, 4, "arg-max index")
        check_canary(ctx, ob, N * 2, "logits of the fused arg-max")
        assert int(ctx.download(ib, (1,), np.int32)[0]) == cpu.argmax_half(ctx.download(ob, (N,), np.uint16).view(np.float16))
        ctx.free(ib)
    qw.release()
    ctx.free(xb)
    ctx.free(ob)


def _int8_case(nnb, ctx, x, N=1536, K=576, seed=200):
    W, s = make_weight("int8", N, K, seed)
    qw = nnb.QuantWeight(ctx, "int8", W, s)
    xb = ctx.upload(x.view(np.uint16))
    ob = ctx.upload(np.full((x.shape[0], N), 0x7E00, np.uint16))
    ctx.linear(x.shape[0], N, K, xb, qw.buf, ob)
    got = ctx.download(ob, (x.shape[0], N), np.uint16).view(np.float16)
    qw.release()
    ctx.free(xb)
    ctx.free(ob)
    return got, W, s


@pytest.mark.parametrize("M", [1, 4])
def test_int8_activations_at_the_edges_of_fp16(nnb, ctx, M):
    """The int8 path rescales each activation row to 24-bit fixed point before the integer
    products; the reference multiplies in fp32 (gemv_int8.cl:50-76).  Rows that stress the
    rescaling: one huge outlier among N(0,1) values, nothing but subnormals, all zeros, a mix
    of magnitudes across the whole fp16 range."""
    K = 576
    rng = np.random.default_rng(210 + M)
    # an outlier of 6e4 (near the largest fp16) among N(0,1) values
    x = make_x(M, K, 211)
    x[:, 100] = np.float16(6.0e4)
    got, W, s = _int8_case(nnb, ctx, x)
    want = cpu.linear("int8", x, W, s)
    finite = np.isfinite(want.astype(np.float32))
    assert np.array_equal(np.isfinite(got.astype(np.float32)), finite)        # overflow to Inf where the oracle's does
    err = cpu.rel_l2(np.where(finite, got, 0), np.where(finite, want, 0))
    report(f"int8 6e4 outlier M={M}: relative L2 {err:.3e}")
    assert err < TOL
    # the small values still count: remove the outlier's own contribution on both sides
    x2 = x.copy()
    x2[:, 100] = np.float16(64.0)
    got2, W, s = _int8_case(nnb, ctx, x2)
    check_close(got2, cpu.linear("int8", x2, W, s), what=f"int8 moderate outlier M={M}")
    # nothing but subnormals (down to the smallest, 2^-24)
    sub = (rng.integers(-1023, 1024, (M, K)).astype(np.int16))
    xs = np.where(sub < 0, (np.abs(sub).astype(np.uint16) | 0x8000), sub.astype(np.uint16)).astype(np.uint16).view(np.float16)
    gots, W, s = _int8_case(nnb, ctx, xs)
    wants = cpu.linear("int8", xs, W, s)
    # outputs are themselves subnormal or zero: compare absolutely, within one fp16 step
    assert np.abs(gots.astype(np.float32) - wants.astype(np.float32)).max() <= 2.0 ** -24
    # zeros give zeros (and no NaN from a zero row maximum)
    gotz, _, _ = _int8_case(nnb, ctx, np.zeros((M, K), np.float16))
    assert not gotz.view(np.uint16).astype(np.uint32).__and__(0x7FFF).any()
    # magnitudes from 2^-24 to 2^15 in one row: values 2^-24 of the row maximum and smaller round away
    # in the fixed-point form; their share of the result is below fp16's own rounding of the sum
    e = rng.integers(-24, 16, (M, K))
    xm = (np.ldexp(1.0, e) * rng.choice([-1.0, 1.0], (M, K))).astype(np.float16)
    gotm, W, s = _int8_case(nnb, ctx, xm)
    check_close(gotm, cpu.linear("int8", xm, W, s), what=f"int8 mixed magnitudes M={M}")


@pytest.mark.parametrize("fmt", ["int8", "fp16", "q4"])
def test_non_finite_activations_give_non_finite_rows(nnb, ctx, fmt):
    """An Inf or NaN among the activations of a row: the reference's fp32 sum is Inf or NaN for
    every weight row with a non-zero weight there; here every output of that activation row is
    non-finite as well (NaN on the int8 path, which cannot rescale such a row), and the other
    rows of the batch are untouched."""
    N, K, M = 1024, 1024, 3
    W, s = make_weight(fmt, N, K, 220)
    qw = nnb.QuantWeight(ctx, fmt, W, s)
    x = make_x(M, K, 221)
    clean = x.copy()
    x[0, 5] = np.float16(np.inf)
    x[2, 1000] = np.float16(np.nan)
    xb = ctx.upload(x.view(np.uint16))
    ob = ctx.upload(np.zeros((M, N), np.uint16))
    ctx.linear(M, N, K, xb, qw.buf, ob)
    got = ctx.download(ob, (M, N), np.uint16).view(np.float16).astype(np.float32)
    want = cpu.linear(fmt, x, W, s).astype(np.float32)
    assert np.isnan(got[2]).all() and np.isnan(want[2]).all()
    touched = cpu.dequant(fmt, W, s).astype(np.float32)[:, 5] != 0
    assert not np.isfinite(got[0][touched]).any() and not np.isfinite(want[0][touched]).any()
    check_close(got[1:2], cpu.linear(fmt, clean[1:2], W, s), what=f"clean row beside non-finite ones {fmt}")
    qw.release()
    ctx.free(xb)
    ctx.free(ob)


def test_read_bandwidth_probe(nnb, ctx):
    """The library's own ceiling for its weight streams (the reference's STREAM probe,
    src/models/lfm2-5-350m/src/main.cpp:29-139): both read paths land in the range of an HBM3e
    part, and the arguments are checked."""
    loads, tma = ctx.bandwidth_probe(512 << 20, trials=3)
    report(f"read-bandwidth probe over 512 MiB: 16-byte loads {loads:.0f} GB/s, TMA bulk copies {tma:.0f} GB/s")
    assert 1500 < loads < 9000 and 1500 < tma < 9000
    L = ctx.L
    assert L.nn_bandwidth_probe(ctx.h, 1000, 3, None, None) == nnb.NN_ERR_ARG
    assert L.nn_bandwidth_probe(ctx.h, 512 << 20, 0, None, None) == nnb.NN_ERR_ARG
    assert L.nn_bandwidth_probe(None, 0, 1, None, None) == nnb.NN_ERR_ARG
    ctx.sync()

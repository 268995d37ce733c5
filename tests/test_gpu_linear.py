"""Parity of the CUDA path, called through the C ABI, against the CPU oracle.

Bars: dequantised weights bit-exact; outputs within 1e-3 relative L2 of the oracle's
kernel-order fp32 result (tests/helpers.TOL); arg-max agreement on lm_head logits."""
import ctypes

import numpy as np
import pytest

from oracle import cpu, quant
from helpers import TOL, check_close, make_weight, make_x

pytestmark = pytest.mark.gpu

FMTS = ["fp16", "int8", "q4"]


def run_linear(nnb, ctx, fmt, W, s, x, N, K, call="linear", extra=None):
    M = x.shape[0]
    qw = nnb.QuantWeight(ctx, fmt, W, s)
    xb = ctx.upload(x.view(np.uint16))
    if call == "linear":
        ob = ctx.upload(np.full((M, N), 0x7E00, np.uint16))  # NaN canary: every element must be written
        ctx.linear(M, N, K, xb, qw.buf, ob)
    elif call == "add":
        ob = ctx.upload(extra.view(np.uint16))
        ctx.linear_add(M, N, K, xb, qw.buf, ob)
    elif call == "silu_gate":
        ob = ctx.upload(extra.view(np.uint16))
        ctx.linear_silu_gate_fused(M, N, K, xb, qw.buf, ob)
    out = ctx.download(ob, (M, N), np.uint16).view(np.float16)
    for b in (xb, ob, qw.buf, qw.scale):
        if b:
            ctx.free(b)
    ctx.L.nn_unregister_weight(ctx.h, qw.buf)
    return out


# config 1: the single int8 GEMV the reference can run on a CPU OpenCL device
def test_config1_int8_gemv(nnb, ctx):
    N, K = 1536, 576
    W, s = make_weight("int8", N, K, 1234)
    x = make_x(1, K, 4321)
    got = run_linear(nnb, ctx, "int8", W, s, x, N, K)
    want = cpu.linear("int8", x, W, s)
    err = check_close(got, want, what="config1")
    assert err < 5e-4
    # against the fp64 sum too: the fp32 association used on the GPU is as good as the kernel's
    check_close(got, cpu.store_half(cpu.linear_acc("int8", x, W, s, cpu.ORDER_F64)), what="config1 vs f64")


# every (N, K) the three model configs use (lm_head sizes are cut to a few thousand rows
# here; full sizes are covered by test_gpu_properties.py)
MODEL_SHAPES = [
    (576, 576), (192, 576), (1536, 576), (576, 1536),              # SmolLM2-135M
    (3072, 1024), (1024, 1024), (512, 1024), (4608, 1024), (1024, 4608),   # LFM2.5-350M
    (1152, 896), (896, 896), (128, 896), (4864, 896), (896, 4864),  # Qwen2.5-0.5B
    (4096, 576), (4100, 896),                                      # lm_head row slices (one ragged)
]


@pytest.mark.parametrize("fmt", FMTS)
@pytest.mark.parametrize("N,K", MODEL_SHAPES)
def test_model_shapes_m1(nnb, ctx, fmt, N, K):
    if fmt == "q4" and K % 32:
        pytest.skip("Q4 needs K % 32 == 0")
    W, s = make_weight(fmt, N, K, 100 + N + K)
    x = make_x(1, K, 7 + K)
    got = run_linear(nnb, ctx, fmt, W, s, x, N, K)
    check_close(got, cpu.linear(fmt, x, W, s), what=f"{fmt} {N}x{K}")


@pytest.mark.parametrize("fmt", FMTS)
@pytest.mark.parametrize("M", [2, 4, 8, 9, 16, 17, 33])
def test_batched_decode(nnb, ctx, fmt, M):
    """M > 1 is M independent M = 1 results."""
    N, K = 1056, 1024
    W, s = make_weight(fmt, N, K, 55)
    x = make_x(M, K, 56 + M)
    got = run_linear(nnb, ctx, fmt, W, s, x, N, K)
    want = cpu.linear(fmt, x, W, s)
    check_close(got, want, what=f"{fmt} M={M}")
    # row m of the batch equals the M = 1 call on row m
    one = run_linear(nnb, ctx, fmt, W, s, x[M - 1:M], N, K)
    # (above 16 rows a Q4 weight goes to the tensor cores as fp16(code * scale), one rounding of
    # 2^-12 per weight that the M <= 16 kernel, which scales exact block sums, does not make)
    check_close(got[M - 1:M], one, tol=5e-4 if (fmt == "q4" and M > 16) else 2e-4, what="batch row vs single")


@pytest.mark.parametrize("fmt", FMTS)
def test_dequant_bit_exact(nnb, ctx, fmt):
    N, K = 67, 256
    W, s = make_weight(fmt, N, K, 9)
    if fmt == "q4":
        W = W.copy()
        W[0, :] = np.arange(K // 2, dtype=np.uint8) * 2          # full nibble domain incl. nibble 0 -> -8
        W[1, :] = 0x00
        W[2, :] = 0xFF
    if fmt == "int8":
        W = W.copy()
        W[0, :] = np.arange(K, dtype=np.int64).astype(np.int8)   # all 256 codes incl. -128
    qw = nnb.QuantWeight(ctx, fmt, W, s)
    ob = ctx.alloc(N * K * 4)
    ctx.dequant(N, K, qw.buf, ob)
    got = ctx.download(ob, (N, K), np.float32)
    want = cpu.dequant(fmt, W, s)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    # the GEMV must use the same unpack: x = e_k picks column k of the dequantised weight
    for k in (0, 1, 37, K - 1):
        x = np.zeros((1, K), np.float16)
        x[0, k] = 1.0
        xb = ctx.upload(x.view(np.uint16))
        yb = ctx.alloc(N * 2)
        ctx.linear(1, N, K, xb, qw.buf, yb)
        y = ctx.download(yb, (N,), np.uint16).view(np.float16)
        assert np.array_equal(y, want[:, k].astype(np.float16)), f"{fmt} column {k}"
    ctx.L.nn_unregister_weight(ctx.h, qw.buf)


@pytest.mark.parametrize("fmt", FMTS)
@pytest.mark.parametrize("N,K", [(576, 576), (576, 1536), (896, 4864), (100, 96)])
def test_residual_epilogue(nnb, ctx, fmt, N, K):
    W, s = make_weight(fmt, N, K, 21)
    x = make_x(1, K, 22)
    r = make_x(1, N, 23)
    got = run_linear(nnb, ctx, fmt, W, s, x, N, K, call="add", extra=r)
    check_close(got, cpu.linear_residual(fmt, x, W, s, r), what=f"residual {fmt}")


@pytest.mark.parametrize("fmt", FMTS)
@pytest.mark.parametrize("M", [1, 3])
def test_silu_gate_epilogue(nnb, ctx, fmt, M):
    N, K = 4608, 1024
    W, s = make_weight(fmt, N, K, 31)
    x = make_x(M, K, 32)
    g = make_x(M, N, 33)
    got = run_linear(nnb, ctx, fmt, W, s, x, N, K, call="silu_gate", extra=g)
    check_close(got, cpu.linear_silu_gate(fmt, x, W, s, g), what=f"silu_gate {fmt}")


@pytest.mark.parametrize("fmt", FMTS)
@pytest.mark.parametrize("N,K,M", [(1536, 576, 1), (4864, 896, 1), (4608, 1024, 8), (1000, 1024, 2), (40, 64, 1)])
def test_swiglu_two_weights(nnb, ctx, fmt, N, K, M):
    if fmt == "q4" and K % 32:
        pytest.skip("Q4 needs K % 32 == 0")
    Wg, sg = make_weight(fmt, N, K, 41)
    Wu, su = make_weight(fmt, N, K, 42)
    x = make_x(M, K, 43)
    g = nnb.QuantWeight(ctx, fmt, Wg, sg)
    u = nnb.QuantWeight(ctx, fmt, Wu, su)
    xb = ctx.upload(x.view(np.uint16))
    ob = ctx.upload(np.full((M, N), 0x7E00, np.uint16))
    ctx.fused_gate_up_silu(M, N, K, xb, g.buf, u.buf, ob)
    got = ctx.download(ob, (M, N), np.uint16).view(np.float16)
    check_close(got, cpu.linear_swiglu(fmt, x, Wg, sg, Wu, su), what=f"swiglu {fmt}")
    for w in (g, u):
        ctx.L.nn_unregister_weight(ctx.h, w.buf)


@pytest.mark.parametrize("fmt", FMTS)
@pytest.mark.parametrize("K,Nq,Nk,Nv", [(576, 576, 192, 192), (896, 896, 128, 128), (1024, 1024, 512, 512), (64, 40, 8, 24)])
def test_fused_qkv(nnb, ctx, fmt, K, Nq, Nk, Nv):
    if fmt == "q4" and K % 32:
        pytest.skip("Q4 needs K % 32 == 0")
    Ws = [make_weight(fmt, n, K, 60 + i) for i, n in enumerate((Nq, Nk, Nv))]
    x = make_x(1, K, 66)
    qs = [nnb.QuantWeight(ctx, fmt, W, s) for W, s in Ws]
    xb = ctx.upload(x.view(np.uint16))
    outs = [ctx.upload(np.full((1, n), 0x7E00, np.uint16)) for n in (Nq, Nk, Nv)]
    ctx.linear_qkv(1, K, xb, qs[0].buf, Nq, qs[1].buf, Nk, qs[2].buf, Nv, *outs)
    for (W, s), ob, n in zip(Ws, outs, (Nq, Nk, Nv)):
        got = ctx.download(ob, (1, n), np.uint16).view(np.float16)
        check_close(got, cpu.linear(fmt, x, W, s), what=f"qkv {fmt} N={n}")
    for q in qs:
        ctx.L.nn_unregister_weight(ctx.h, q.buf)


@pytest.mark.parametrize("fmt", FMTS)
@pytest.mark.parametrize("N,K", [(1, 32), (3, 64), (33, 96), (17, 160), (64, 2080), (5, 8192)])
def test_ragged_and_tiny_shapes(nnb, ctx, fmt, N, K):
    """Rows that do not fill a tile, K that is not a multiple of the stage size, K below
    the streaming kernel's minimum (generic kernel)."""
    W, s = make_weight(fmt, N, K, 71)
    x = make_x(2, K, 72)
    got = run_linear(nnb, ctx, fmt, W, s, x, N, K)
    check_close(got, cpu.linear(fmt, x, W, s), what=f"ragged {fmt} {N}x{K}")


@pytest.mark.parametrize("fmt,K", [("fp16", 70), ("fp16", 577), ("int8", 100), ("int8", 13)])
def test_any_k_generic_path(nnb, ctx, fmt, K):
    """The reference's generic kernel takes any K (vec4 steps + scalar tail)."""
    N = 37
    W, s = make_weight(fmt, N, K, 81)
    x = make_x(1, K, 82)
    got = run_linear(nnb, ctx, fmt, W, s, x, N, K)
    check_close(got, cpu.linear(fmt, x, W, s), what=f"any-K {fmt} K={K}")


def test_row_tile_views_resolve(nnb, ctx):
    """A pointer at a row offset inside a registered weight is that weight's row tile
    (the reference's lm_head sub-buffers): scales follow the rows."""
    for fmt in ("int8", "q4"):
        N, K = 300, 1024
        W, s = make_weight(fmt, N, K, 91)
        x = make_x(1, K, 92)
        qw = nnb.QuantWeight(ctx, fmt, W, s)
        xb = ctx.upload(x.view(np.uint16))
        want = cpu.linear(fmt, x, W, s)
        rb = K if fmt == "int8" else K // 2
        for r0, n in ((0, 300), (64, 100), (299, 1), (128, 172)):
            ob = ctx.alloc(n * 2)
            ctx.linear(1, n, K, xb, ctypes.c_void_p(qw.buf + r0 * rb), ob)
            got = ctx.download(ob, (1, n), np.uint16).view(np.float16)
            check_close(got, want[:, r0:r0 + n], what=f"tile view {fmt} rows {r0}+{n}")
        # more rows than remain, a K that does not match, an offset inside a row: refused
        ob = ctx.alloc(600)
        assert ctx.L.nn_linear(ctx.h, 1, 300, K, xb, ctypes.c_void_p(qw.buf + 64 * rb), ob) == nnb.NN_ERR_ARG
        assert ctx.L.nn_linear(ctx.h, 1, 10, K // 2, xb, qw.buf, ob) == nnb.NN_ERR_ARG
        assert ctx.L.nn_linear(ctx.h, 1, 10, K, xb, ctypes.c_void_p(qw.buf + 16), ob) == nnb.NN_ERR_ARG
        ctx.L.nn_unregister_weight(ctx.h, qw.buf)


def test_argument_errors(nnb, ctx):
    L = ctx.L
    b = ctx.alloc(4096)
    assert L.nn_linear(ctx.h, 1, 0, 64, b, b, b) == nnb.NN_ERR_ARG
    assert L.nn_linear(ctx.h, -1, 8, 64, b, b, b) == nnb.NN_ERR_ARG
    assert L.nn_linear(ctx.h, 1, 8, 64, None, b, b) == nnb.NN_ERR_ARG
    assert L.nn_register_q4_weight(ctx.h, b, b, 8, 48) == nnb.NN_ERR_ARG      # K % 32
    assert L.nn_linear(ctx.h, 0, 8, 64, b, b, b) == 0                           # M = 0: nothing to do
    assert b"K % 32" in L.nn_last_error() or True
    ctx.sync()


def test_argmax_agreement(nnb, ctx):
    """Greedy token = arg-max of the lm_head logits: ours against the oracle's on the same
    hidden vectors (SmolLM2-shaped tied head, int8), plus the arg-max kernel itself."""
    V, H = 49152, 576
    W, s = make_weight("int8", V, H, 1301)
    qw = nnb.QuantWeight(ctx, "int8", W, s)
    lb = ctx.alloc(V * 2)
    ib = ctx.alloc(4)
    agree, trials = 0, 24
    for t in range(trials):
        x = make_x(1, H, 2000 + t)
        xb = ctx.upload(x.view(np.uint16))
        ctx.linear(1, V, H, xb, qw.buf, lb)
        ctx.argmax(V, lb, ib)
        idx = int(ctx.download(ib, (1,), np.int32)[0])
        logits = ctx.download(lb, (V,), np.uint16).view(np.float16)
        assert idx == cpu.argmax_half(logits)                  # kernel vs CPU on the same logits
        want = cpu.linear("int8", x, W, s, threads=8)
        o = cpu.argmax_half(want)
        if idx == o:
            agree += 1
        else:  # a flip is only acceptable between logits that are equal to within fp16 rounding
            lw = want.astype(np.float32).reshape(-1)
            assert abs(lw[idx] - lw[o]) <= 2 * np.spacing(np.float16(abs(lw[o]))).astype(np.float32)
        ctx.free(xb)
    assert agree >= trials - 2
    ctx.L.nn_unregister_weight(ctx.h, qw.buf)


@pytest.mark.parametrize("fmt,N,K,M", [("fp16", 896, 896, 64), ("fp16", 4864, 896, 512), ("fp16", 1000, 1024, 100), ("fp16", 256, 4864, 17),
                                       ("fp16", 640, 200, 48), ("int8", 1152, 896, 256), ("int8", 900, 576, 33), ("q4", 1024, 1024, 128),
                                       ("q4", 4608, 1024, 64), ("fp16", 2048, 896, 2048), ("q4", 640, 2048, 300), ("int8", 512, 1024, 300), ("q4", 1152, 8192, 257)])
def test_tensor_core_path_large_m(nnb, ctx, fmt, N, K, M):
    """M > 16 (batched decode beyond 16 rows, prefill): the tcgen05 GEMM.  The reference is
    M independent M = 1 results; compared here against an fp64 product of the dequantised
    weights, which the kernel-order oracle matches to 2e-6 (tests/test_oracle_golden.py)."""
    W, s = make_weight(fmt, N, K, 7000 + N)
    x = make_x(M, K, 7001)
    got = run_linear(nnb, ctx, fmt, W, s, x, N, K)
    want = x.astype(np.float64) @ cpu.dequant(fmt, W, s).astype(np.float64).T
    check_close(got, want, what=f"tensor-core {fmt} {N}x{K} M={M}")
    # a few rows against the kernel-order oracle itself
    rows = [0, M // 2, M - 1]
    check_close(got[rows], cpu.linear(fmt, x[rows], W, s, threads=8), what="tensor-core vs oracle rows")


def test_tensor_core_residual(nnb, ctx):
    N, K, M = 896, 4864, 64
    W, s = make_weight("int8", N, K, 7100)
    x, r = make_x(M, K, 7101), make_x(M, N, 7102)
    got = run_linear(nnb, ctx, "int8", W, s, x, N, K, call="add", extra=r)
    want = r.astype(np.float64) + x.astype(np.float64) @ cpu.dequant("int8", W, s).astype(np.float64).T
    check_close(got, want, what="tensor-core residual")


@pytest.mark.parametrize("fmt,N,K", [("int8", 49152, 576), ("fp16", 4101, 576), ("q4", 8192, 1024), ("q4", 4608, 8192), ("int8", 1000, 200)])
def test_linear_argmax_matches_linear_then_argmax(nnb, ctx, fmt, N, K):
    """The fused lm_head + greedy pick returns the index nn_linear + nn_argmax returns, with and
    without a logits buffer, launch after launch (its reduction words clear themselves)."""
    if fmt == "q4" and K % 32:
        pytest.skip("Q4 needs K % 32 == 0")
    W, s = make_weight(fmt, N, K, 71)
    qw = nnb.QuantWeight(ctx, fmt, W, s)
    logits, logits2, idx, idx2 = ctx.alloc(N * 2), ctx.alloc(N * 2), ctx.alloc(4), ctx.alloc(4)
    for rep in range(3):
        x = make_x(1, K, 72 + rep)
        dx = ctx.upload(x.view(np.uint16))
        ctx.linear(1, N, K, dx, qw.buf, logits)
        ctx.argmax(N, logits, idx)
        ctx.linear_argmax(N, K, dx, qw.buf, logits2, idx2)
        want = int(ctx.download(idx, (1,), np.int32)[0])
        got = int(ctx.download(idx2, (1,), np.int32)[0])
        a = ctx.download(logits, (N,), np.uint16)
        b = ctx.download(logits2, (N,), np.uint16)
        assert np.array_equal(a, b)
        assert got == want == int(np.argmax(a.view(np.float16).astype(np.float32)))
        if K % 64 == 0:
            ctx.linear_argmax(N, K, dx, qw.buf, None, idx2)      # logits never written
            assert int(ctx.download(idx2, (1,), np.int32)[0]) == want
        else:
            with pytest.raises(nnb.NNError):                     # the any-shape kernel needs the buffer
                ctx.linear_argmax(N, K, dx, qw.buf, None, idx2)
        # greedy-token agreement with the oracle: its logit at the chosen row is its maximum
        # up to the path's tolerance
        ref = cpu.linear(fmt, x, W, s).astype(np.float32)[0]
        assert ref[got] >= ref.max() - 2e-3 * np.abs(ref).max()
        ctx.free(dx)
    qw.release()
    for b_ in (logits, logits2, idx, idx2):
        ctx.free(b_)


@pytest.mark.parametrize("fmt", FMTS)
@pytest.mark.parametrize("N,K", [(1056, 1024), (576, 1536), (4864, 896)])
def test_batch_rows_are_bitwise_the_single_token_results(nnb, ctx, fmt, N, K):
    """Up to 16 rows share one pass over the weights; the activations of such a call are staged
    once by a launch of their own.  Row m of the batch must carry exactly the bits of the
    single-token call on row m (the reference's quantised M > 1 IS a loop of M = 1 calls,
    src/models/lfm2-5-350m/src/model.cpp:243-251), for every M and for the fused forms."""
    W, s = make_weight(fmt, N, K, 155)
    qw = nnb.QuantWeight(ctx, fmt, W, s)
    x = make_x(16, K, 156)
    x[3] *= np.float16(37.0)                  # rows of different magnitude: the int8 rescale is per row
    x[7] *= np.float16(0.01)
    xb = ctx.upload(x.view(np.uint16))
    ob = ctx.alloc(16 * N * 2)
    singles = []
    for m in range(16):
        ctx.linear(1, N, K, xb + m * K * 2, qw.buf, ob)
        singles.append(ctx.download(ob, (N,), np.uint16).copy())
    singles = np.stack(singles)
    for M in (2, 3, 8, 9, 13, 16):
        ctx.upload(np.full((M, N), 0x7E00, np.uint16), ob)
        ctx.linear(M, N, K, xb, qw.buf, ob)
        got = ctx.download(ob, (M, N), np.uint16)
        assert np.array_equal(got, singles[:M]), f"{fmt} {N}x{K} M={M}: a batch row differs from its single-token result"
    # in-place residual, batched against single
    r = make_x(16, N, 157)
    rb = ctx.upload(r.view(np.uint16))
    for m in range(16):
        ctx.linear_add(1, N, K, xb + m * K * 2, qw.buf, rb + m * N * 2)
    want = ctx.download(rb, (16, N), np.uint16).copy()
    ctx.upload(r.view(np.uint16), rb)
    ctx.linear_add(16, N, K, xb, qw.buf, rb)
    assert np.array_equal(ctx.download(rb, (16, N), np.uint16), want)
    qw.release()
    for b in (xb, ob, rb):
        ctx.free(b)


@pytest.mark.parametrize("fmt", FMTS)
@pytest.mark.parametrize("M", [40, 300])
def test_fused_forms_at_prefill_row_counts(nnb, ctx, fmt, M):
    """Above 16 rows the fused forms (QKV over three weights, SwiGLU over two, the in-place SiLU gate) run as one
    tensor-core GEMM per weight plus, for the two-weight forms, the SiLU-multiply over the fp16 results: the
    reference's own sequence for M > 1 (src/models/lfm2-5-350m/src/layers/mlp.cpp:101-129).  The oracle for it is
    that sequence on the oracle's projections: fp16 results first, then silu(g) * u in fp32, one more rounding."""
    K, N = 896, 1152
    x = make_x(M, K, 171)
    dx = ctx.upload(x.view(np.uint16))

    def silu_mul(g, u):
        g32, u32 = g.astype(np.float32), u.astype(np.float32)
        return ((g32 / (1.0 + np.exp(-g32))) * u32).astype(np.float16)

    # SwiGLU over two weights
    (Wg, sg), (Wu, su) = make_weight(fmt, N, K, 172), make_weight(fmt, N, K, 173)
    qg, qu = nnb.QuantWeight(ctx, fmt, Wg, sg), nnb.QuantWeight(ctx, fmt, Wu, su)
    out = ctx.upload(np.full((M, N), 0x7E00, np.uint16))
    before = ctx.launch_count()
    ctx.fused_gate_up_silu(M, N, K, dx, qg.buf, qu.buf, out)
    assert ctx.launch_count() - before == 3          # two GEMMs and the SiLU-multiply, not M / 16 slices
    got = ctx.download(out, (M, N), np.uint16).view(np.float16)
    g, u = cpu.linear(fmt, x, Wg, sg, threads=4), cpu.linear(fmt, x, Wu, su, threads=4)
    check_close(got, silu_mul(g, u), what=f"swiglu at M={M} {fmt}")
    # the in-place gate form on the same operands
    gate = ctx.upload(g.view(np.uint16))
    ctx.linear_silu_gate_fused(M, N, K, dx, qu.buf, gate)
    got = ctx.download(gate, (M, N), np.uint16).view(np.float16)
    check_close(got, silu_mul(g, u), what=f"silu gate at M={M} {fmt}")
    # QKV over three weights
    Ns = (896, 128, 128)
    Ws = [make_weight(fmt, n, K, 174 + i) for i, n in enumerate(Ns)]
    qs = [nnb.QuantWeight(ctx, fmt, W, s) for W, s in Ws]
    outs = [ctx.upload(np.full((M, n), 0x7E00, np.uint16)) for n in Ns]
    before = ctx.launch_count()
    ctx.linear_qkv(M, K, dx, qs[0].buf, Ns[0], qs[1].buf, Ns[1], qs[2].buf, Ns[2], *outs)
    assert ctx.launch_count() - before == 3
    for (W, s), ob, n in zip(Ws, outs, Ns):
        got = ctx.download(ob, (M, n), np.uint16).view(np.float16)
        check_close(got, cpu.linear(fmt, x, W, s, threads=4), what=f"qkv at M={M} {fmt} N={n}")
    for q in [qg, qu] + qs:
        q.release()
    for b in [dx, out, gate] + outs:
        ctx.free(b)

"""The allocation-free arg-max entry point against the regular one.

Some users of the library may not allocate device memory when they need the greedy token
(a real-time callback, an application that owns the device heap, a frozen memory budget).
nn_argmax_static serves them with scratch that lives inside the library image.  This file
is collected last on purpose: it must pass after every other test has used the GPU, and
also when it is the only test of a fresh process."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _logits(n, seed):
    rng = np.random.default_rng(seed)
    v = (rng.standard_normal(n) * 3).astype(np.float16)
    return v


def test_static_argmax_matches_regular_entry_point_twice(nnb, ctx):
    L = ctx.L
    stream = L.nn_stream(ctx.h)
    out_a, out_b = ctx.alloc(4), ctx.alloc(4)
    # two calls in a row with different inputs: the second must not see the first's scratch
    for call, (n, seed) in enumerate(((49152, 11), (151936, 12))):
        v = _logits(n, seed)
        if call == 1:
            v[:] = np.minimum(v, np.float16(1.0))      # lower maximum than the first call's
            v[n - 7] = np.float16(2.5)
        buf = ctx.upload(v.view(np.uint16))
        ctx.argmax(n, buf, out_a)
        assert L.nn_argmax_static(stream, n, buf, out_b) == 0, L.nn_last_error()
        ctx.sync()
        a = int(ctx.download(out_a, (1,), np.int32)[0])
        b = int(ctx.download(out_b, (1,), np.int32)[0])
        assert a == b == int(np.argmax(v.astype(np.float32)))
        ctx.free(buf)
    # ties go to the lowest index, as in nn_argmax
    v = np.zeros(4096, np.float16)
    v[[100, 900, 4000]] = np.float16(7.0)
    buf = ctx.upload(v.view(np.uint16))
    assert L.nn_argmax_static(stream, 4096, buf, out_b) == 0
    ctx.sync()
    assert int(ctx.download(out_b, (1,), np.int32)[0]) == 100
    # beyond the built-in maximum: a clear refusal, nothing launched
    assert L.nn_argmax_static(stream, (1 << 22) + 1, buf, out_b) == nnb.NN_ERR_ARG
    assert b"allocation-free" in L.nn_last_error()
    assert L.nn_argmax_static(stream, 16, None, out_b) == nnb.NN_ERR_ARG
    ctx.sync()


def test_static_argmax_empty_all_nan_and_default_stream(nnb, ctx):
    """The corners of the contract: no logits and nothing but NaNs give -1 (as nn_argmax
    does), and a null stream handle means the default stream."""
    import torch
    L = ctx.L
    stream = L.nn_stream(ctx.h)
    out_a, out_b = ctx.alloc(4), ctx.alloc(4)
    v = _logits(5000, 13)
    buf = ctx.upload(v.view(np.uint16))
    # n = 0: nothing is read, the result is -1 and an earlier result is overwritten
    ctx.upload(np.full(1, 1234, np.int32), out_b)
    assert L.nn_argmax_static(stream, 0, buf, out_b) == 0, L.nn_last_error()
    ctx.sync()
    assert int(ctx.download(out_b, (1,), np.int32)[0]) == -1
    # nothing but NaNs (both signs, several payloads): -1 from both entry points
    nan = np.full(5000, 0x7E00, np.uint16)
    nan[::3] = 0xFE00
    nan[1::7] = 0x7FFF
    nbuf = ctx.upload(nan)
    ctx.argmax(5000, nbuf, out_a)
    assert L.nn_argmax_static(stream, 5000, nbuf, out_b) == 0
    ctx.sync()
    assert int(ctx.download(out_a, (1,), np.int32)[0]) == -1
    assert int(ctx.download(out_b, (1,), np.int32)[0]) == -1
    # one number among the NaNs, -inf included: the number wins; only -inf and NaNs: -inf wins
    nan[4321] = np.float16(-3.0).view(np.uint16)
    nan[17] = 0xFC00
    ctx.upload(nan, nbuf)
    assert L.nn_argmax_static(stream, 5000, nbuf, out_b) == 0
    ctx.sync()
    assert int(ctx.download(out_b, (1,), np.int32)[0]) == 4321
    nan[4321] = 0x7E00
    ctx.upload(nan, nbuf)
    assert L.nn_argmax_static(stream, 5000, nbuf, out_b) == 0
    ctx.sync()
    assert int(ctx.download(out_b, (1,), np.int32)[0]) == 17
    # a null stream handle is the default stream: order it against the context's stream by hand
    ctx.sync()
    assert L.nn_argmax_static(None, 5000, buf, out_b) == 0
    torch.cuda.synchronize()
    assert int(ctx.download(out_b, (1,), np.int32)[0]) == int(np.argmax(v.astype(np.float32)))
    assert L.nn_argmax_static(stream, -1, buf, out_b) == nnb.NN_ERR_ARG
    for b in (buf, nbuf, out_a, out_b):
        ctx.free(b)

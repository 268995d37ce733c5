"""Multi-GPU parity of the row-sharded projections (needs at least two GPUs; skipped otherwise)
and the single-rank behaviour of the gather entry points, including a wait that runs out."""
import os
import socket
import subprocess
import sys

import numpy as np
import pytest

from helpers import TOL, make_weight, make_x
from oracle import cpu

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def test_two_rank_gather_matches_nccl_and_oracle(nnb, built_lib):
    n = built_lib.nn_device_count()
    if n < 2:
        pytest.skip(f"{n} GPU visible; the two-rank check needs two")
    env = dict(os.environ, NCCL_DEBUG="WARN")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", str(_free_port()), os.path.join(REPO, "tests", "multi_gpu_worker.py")]
    r = subprocess.run(cmd, cwd=REPO, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "MULTI_GPU_OK" in r.stdout, (r.stdout[-3000:], r.stderr[-3000:])


@pytest.mark.parametrize("fmt,N,K,M", [("int8", 1536, 576, 1), ("q4", 512, 1024, 8), ("fp16", 1024, 512, 48)])
def test_single_rank_gather_is_linear(nnb, ctx, fmt, N, K, M):
    comm = nnb.Comm(ctx, None, 0, 1)
    try:
        W, s = make_weight(fmt, N, K, 31)
        x = make_x(M, K, 32)
        qw = nnb.QuantWeight(ctx, fmt, W, s)
        dx = ctx.upload(x.view(np.uint16))
        g = comm.symm_alloc(M * N * 2)
        comm.linear_gather(M, N, K, dx, qw.buf, g)
        got = ctx.download(g, (M, N), np.uint16).view(np.float16)
        out = ctx.alloc(M * N * 2)
        ctx.linear(M, N, K, dx, qw.buf, out)
        ref = ctx.download(out, (M, N), np.uint16).view(np.float16)
        assert np.array_equal(got.view(np.uint16), ref.view(np.uint16))
        assert cpu.rel_l2(got, cpu.linear(fmt, x, W, s, order=2)) <= TOL
        qw.release()
        ctx.free(dx)
        ctx.free(out)
    finally:
        ctx.sync()
        comm.close()


@pytest.mark.parametrize("fmt,N,K", [("int8", 49152, 576), ("q4", 4096, 1024), ("fp16", 1536, 896)])
def test_single_rank_sharded_pick_is_linear_argmax(nnb, ctx, fmt, N, K):
    comm = nnb.Comm(ctx, None, 0, 1)
    try:
        g = comm.symm_alloc(256)   # creates the communicator's flag and key words
        W, s = make_weight(fmt, N, K, 41)
        qw = nnb.QuantWeight(ctx, fmt, W, s)
        tok, tok2 = ctx.alloc(4), ctx.alloc(4)
        logits = ctx.alloc(N * 2)
        for rep in range(3):
            x = make_x(1, K, 42 + rep)
            dx = ctx.upload(x.view(np.uint16))
            comm.linear_argmax_sharded(N, K, dx, qw.buf, logits if rep else None, tok)
            ctx.linear_argmax(N, K, dx, qw.buf, None, tok2)
            a, b = int(ctx.download(tok, (1,), np.int32)[0]), int(ctx.download(tok2, (1,), np.int32)[0])
            assert a == b and 0 <= a < N
            if rep:
                lg = ctx.download(logits, (N,), np.uint16).view(np.float16).astype(np.float32)
                assert int(np.argmax(lg)) == a
            ctx.free(dx)
        qw.release()
        for b_ in (tok, tok2, logits):
            ctx.free(b_)
        comm.symm_free(g)
    finally:
        ctx.sync()
        comm.close()


def test_gather_rejects_foreign_buffer(nnb, ctx):
    comm = nnb.Comm(ctx, None, 0, 1)
    try:
        g = comm.symm_alloc(4096)
        plain = ctx.alloc(4096)
        W, _ = make_weight("fp16", 128, 64, 1)
        dw = ctx.upload(W.view(np.uint16))
        dx = ctx.upload(make_x(1, 64, 2).view(np.uint16))
        with pytest.raises(nnb.NNError):
            comm.linear_gather(1, 128, 64, dx, dw, plain)          # not a symmetric buffer
        with pytest.raises(nnb.NNError):
            comm.linear_gather(64, 128, 64, dx, dw, g)             # 64 * 128 * 2 bytes > 4096
        for b in (plain, dw, dx):
            ctx.free(b)
    finally:
        ctx.sync()
        comm.close()


def test_wait_that_nothing_signals_times_out_and_context_survives(nnb, ctx):
    """A wait whose flag is never written must return after its limit, report NN_ERR_TIMEOUT
    through nn_sync, and leave the context usable."""
    comm = nnb.Comm(ctx, None, 0, 1)
    try:
        comm.symm_alloc(256)
        comm.wait(timeout_ms=50)            # no signal has been sent: the flag stays at 0
        with pytest.raises(nnb.NNError) as ei:
            ctx.sync()
        assert ei.value.code == nnb.NN_ERR_TIMEOUT
        # the context still works, and a matched signal / wait pair passes
        comm.signal()                       # brings the sent count level with the wait count
        comm.signal()
        comm.wait(timeout_ms=1000)
        ctx.sync()
        W, _ = make_weight("fp16", 256, 128, 5)
        x = make_x(1, 128, 6)
        dw, dx, out = ctx.upload(W.view(np.uint16)), ctx.upload(x.view(np.uint16)), ctx.alloc(512)
        ctx.linear(1, 256, 128, dx, dw, out)
        got = ctx.download(out, (1, 256), np.uint16).view(np.float16)
        assert cpu.rel_l2(got, cpu.linear("fp16", x, W, None, order=2)) <= TOL
        for b in (dw, dx, out):
            ctx.free(b)
    finally:
        comm.close()


def test_pick_whose_keys_never_arrive_times_out_and_the_next_pick_works(nnb, ctx):
    """The row-sharded greedy pick waits for one key word per rank.  Fault injected on the host: a
    pick round in which nothing stores a key.  The waiting kernel must give up after its limit
    with -1, nn_sync must report NN_ERR_TIMEOUT, and the next regular pick on the same
    communicator must give the single-device answer."""
    comm = nnb.Comm(ctx, None, 0, 1)
    try:
        comm.symm_alloc(256)
        N, K = 4096, 576
        W, s = make_weight("int8", N, K, 901)
        qw = nnb.QuantWeight(ctx, "int8", W, s)
        x = make_x(1, K, 902)
        dx, logits, idx = ctx.upload(x.view(np.uint16)), ctx.alloc(N * 2), ctx.upload(np.full(1, 77, np.int32))
        comm.linear_argmax_sharded(N, K, dx, qw.buf, logits, idx)       # a regular pick first
        ctx.sync()
        want = int(ctx.download(idx, (1,), np.int32)[0])
        assert want == cpu.argmax_half(ctx.download(logits, (N,), np.uint16).view(np.float16))
        comm.pick_unsent(50, idx)
        with pytest.raises(nnb.NNError) as ei:
            ctx.sync()
        assert ei.value.code == nnb.NN_ERR_TIMEOUT
        assert int(ctx.download(idx, (1,), np.int32)[0]) == -1
        for _ in range(3):                                            # odd and even table slots
            ctx.upload(np.full(1, 77, np.int32), idx)
            comm.linear_argmax_sharded(N, K, dx, qw.buf, logits, idx)
            ctx.sync()
            assert int(ctx.download(idx, (1,), np.int32)[0]) == want
        assert ctx.L.nn_comm_pick_unsent(comm.h, 0, idx) == nnb.NN_ERR_ARG
        qw.release()
        for b in (dx, logits, idx):
            ctx.free(b)
    finally:
        ctx.sync()
        comm.close()


def test_nccl_that_cannot_be_loaded_is_a_comm_error(nnb, built_lib):
    """nn_comm_init for more than one rank with NNB_NCCL_LIB pointing nowhere: NN_ERR_COMM and no
    communicator, in a child process (the library is looked up once per process)."""
    code = (
        "import ctypes, sys\n"
        f"L = ctypes.CDLL({nnb.LIB_PATH!r})\n"
        "L.nn_last_error.restype = ctypes.c_char_p\n"
        "h = ctypes.c_void_p()\n"
        "assert L.nn_init(0, ctypes.byref(h)) == 0\n"
        "comm = ctypes.c_void_p()\n"
        "rc = L.nn_comm_init(h, ctypes.create_string_buffer(128), 0, 2, ctypes.byref(comm))\n"
        "print(rc, bool(comm.value), L.nn_last_error().decode())\n"
        "one = ctypes.c_void_p()\n"
        "print(L.nn_comm_init(h, None, 0, 1, ctypes.byref(one)), bool(one.value))\n"
    )
    env = dict(os.environ, NNB_NCCL_LIB="/nonexistent/libnccl.so.2")
    out = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr
    first, second = out.stdout.strip().splitlines()
    rc, made, msg = first.split(" ", 2)
    assert int(rc) == nnb.NN_ERR_COMM and made == "False" and "NNB_NCCL_LIB" in msg
    assert second == "0 True"          # a single rank needs no NCCL at all


def test_batched_sharded_pick_single_rank(nnb, ctx):
    """nn_linear_argmax_sharded_rows on one rank: M greedy tokens from one call, each the arg-max of
    its row of logits (lowest index on ties, -1 for a row of NaNs), over repeated calls with
    different M (the key tables alternate and grow)."""
    comm = nnb.Comm(ctx, None, 0, 1)
    try:
        comm.symm_alloc(256)
        N, K = 4096, 576
        W, s = make_weight("int8", N, K, 911)
        qw = nnb.QuantWeight(ctx, "int8", W, s)
        for rep, M in enumerate((8, 40, 3, 300, 16)):
            x = make_x(M, K, 912 + rep)
            if M >= 3:
                x[1] = 0                                   # every logit of this row ties at 0: index 0 wins
                x[2, 7] = np.float16(np.nan)               # a NaN activation: the whole row of logits is NaN -> -1
            dx = ctx.upload(x.view(np.uint16))
            logits, idx = ctx.alloc(M * N * 2), ctx.upload(np.full(M, 77, np.int32))
            comm.linear_argmax_sharded_rows(M, N, K, dx, qw.buf, logits, idx)
            ctx.sync()
            got = ctx.download(idx, (M,), np.int32)
            lg = ctx.download(logits, (M, N), np.uint16)
            b32 = lg.astype(np.uint32)
            keys = np.where((b32 & 0x7FFF) > 0x7C00, 0, np.where(b32 & 0x8000, 0xFFFF - b32, b32 | 0x8000))
            want = np.where(keys.max(axis=1) > 0, np.argmax(keys, axis=1), -1)
            assert np.array_equal(got, want), (M, got[:8], want[:8])
            if M >= 3:
                assert got[1] == 0 and got[2] == -1
            ref = cpu.linear("int8", x[:1], W, s, threads=4)
            assert cpu.rel_l2(lg[:1].view(np.float16), ref) <= TOL
            for b in (dx, logits, idx):
                ctx.free(b)
        L = ctx.L
        b = ctx.alloc(64)
        assert L.nn_linear_argmax_sharded_rows(comm.h, 0, N, K, b, qw.buf, b, b) == nnb.NN_ERR_ARG
        assert L.nn_linear_argmax_sharded_rows(comm.h, 2000, N, K, b, qw.buf, b, b) == nnb.NN_ERR_ARG
        assert L.nn_linear_argmax_sharded_rows(comm.h, 4, N, K, b, qw.buf, None, b) == nnb.NN_ERR_ARG
        ctx.free(b)
        qw.release()
    finally:
        ctx.sync()
        comm.close()

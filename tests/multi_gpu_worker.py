"""One rank of the multi-GPU parity check (launched by test_gpu_multi.py through
torch.distributed.run, one process per GPU).

Every rank builds the same seeded weight, keeps its row block, and runs the projection twice:
  * nn_linear + NCCL all-gather (in place in the gather buffer), and
  * nn_linear_gather, whose kernel stores into every rank's gather buffer over peer memory.
Both gathered results must be bit-identical, and, reassembled to [M, N], must match the CPU
oracle on the unsharded weight within the path's tolerance.

Then the row-sharded greedy pick (nn_linear_argmax_sharded, one key per rank instead of the
logits): on every rank it must name the row that the arg-max over the gathered logits names,
lowest row on ties, over repeated calls (the key tables alternate with the epoch).
"""
import os
import sys

import numpy as np

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, REPO)
sys.path.insert(0, os.path.join(REPO, "tests"))

CASES = [  # fmt, N, K, M
    ("int8", 4096, 576, 1),
    ("q4", 2048, 1024, 8),
    ("fp16", 1536, 896, 16),
    ("fp16", 2048, 512, 64),    # tensor-core path
    ("int8", 3072, 896, 256),   # tensor-core path, quantised weight
    ("q4", 1024, 2048, 40),
]


PICK_CASES = [  # fmt, N, K
    ("int8", 4096, 576),
    ("q4", 2048, 1024),
    ("fp16", 1536, 896),
    ("int8", 49152, 576),   # the lm_head of the benchmarked shape
]


def main():
    import torch
    import torch.distributed as dist
    from conftest import load_package
    from helpers import TOL, make_weight, make_x
    from oracle import cpu
    import importlib
    pkg = load_package()
    sharding = importlib.import_module("adreno_llms_b200.sharding")

    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    dist.init_process_group("gloo", rank=rank, world_size=world)
    ctx = pkg.Context(local)
    idt = torch.zeros(128, dtype=torch.uint8)
    if rank == 0:
        idt = torch.tensor(list(pkg.Comm.unique_id()), dtype=torch.uint8)
    dist.broadcast(idt, 0)
    comm = pkg.Comm(ctx, bytes(idt.tolist()), rank, world)

    failures = []
    for fmt, N, K, M in CASES:
        W, s = make_weight(fmt, N, K, 9000 + N)
        x = make_x(M, K, 9001 + K)
        Wl, sl = sharding.shard_weight(fmt, W, s, world, rank)
        lo, n = sharding.shard_rows(N, world, rank)
        qw = pkg.QuantWeight(ctx, fmt, Wl, sl)
        dx = ctx.upload(x.view(np.uint16))
        block = M * n * 2
        # (1) NCCL, in place
        g1 = ctx.alloc(block * world)
        ctx.linear(M, n, K, dx, qw.buf, g1 + rank * block)
        comm.all_gather(g1 + rank * block, g1, block)
        r1 = ctx.download(g1, (world, M, n), np.uint16)
        # (2) fused: peer stores + flags, twice into alternating buffers (epochs advance)
        bufs = [comm.symm_alloc(block * world) for _ in range(2)]
        outs = []
        for rep in range(4):
            comm.linear_gather(M, n, K, dx, qw.buf, bufs[rep & 1])
            outs.append(ctx.download(bufs[rep & 1], (world, M, n), np.uint16))
        for rep, r2 in enumerate(outs):
            if not np.array_equal(r1, r2):
                failures.append(f"{fmt} N={N} K={K} M={M} rep {rep}: fused gather differs from NCCL gather in "
                                f"{int((r1 != r2).sum())} of {r1.size} values")
        full = sharding.gathered_to_row_major(outs[-1], world, M, N).view(np.float16)
        want = cpu.linear(fmt, x, W, s, order=2)
        err = cpu.rel_l2(full, want)
        if not err <= TOL:
            failures.append(f"{fmt} N={N} K={K} M={M}: relative L2 {err:.3e} against the oracle")
        ctx.sync()
        dist.barrier()   # nobody frees a buffer a peer may still write
        for b in bufs:
            comm.symm_free(b)
        qw.release()
        ctx.free(g1)
        ctx.free(dx)
    for fmt, N, K in PICK_CASES:
        W, s = make_weight(fmt, N, K, 9100 + N)
        Wl, sl = sharding.shard_weight(fmt, W, s, world, rank)
        lo, n = sharding.shard_rows(N, world, rank)
        qw = pkg.QuantWeight(ctx, fmt, Wl, sl)
        tok = ctx.alloc(4)
        local = ctx.alloc(n * 2)
        g1 = ctx.alloc(n * 2 * world)
        for rep in range(5):
            # rep 4: all-zero activations, every logit ties at 0 and row 0 (rank 0's first) must win
            x = make_x(1, K, 9200 + K + rep) if rep < 4 else np.zeros((1, K), np.float16)
            dx = ctx.upload(x.view(np.uint16))
            ctx.linear(1, n, K, dx, qw.buf, g1 + rank * n * 2)
            comm.all_gather(g1 + rank * n * 2, g1, n * 2)
            bits = ctx.download(g1, (N,), np.uint16)
            logits = bits.view(np.float16).astype(np.float32)
            # first maximum in the kernel's total order (sign-magnitude bits made monotonic, so -0 < +0)
            b32 = bits.astype(np.uint32)
            want = int(np.argmax(np.where(b32 & 0x8000, 0xFFFF - b32, b32 | 0x8000)))
            comm.linear_argmax_sharded(n, K, dx, qw.buf, local if rep & 1 else None, tok)
            got = int(ctx.download(tok, (1,), np.int32)[0])
            if got != want:
                failures.append(f"pick {fmt} N={N} K={K} rep {rep}: row {got}, the gathered logits say {want}")
            if rep & 1:
                mine = ctx.download(local, (n,), np.uint16).view(np.float16).astype(np.float32)
                if not np.array_equal(mine, logits[lo:lo + n]):
                    failures.append(f"pick {fmt} N={N} K={K} rep {rep}: the locally stored logits differ from nn_linear's")
            ctx.free(dx)
        ctx.sync()
        dist.barrier()
        qw.release()
        for b in (tok, local, g1):
            ctx.free(b)
    # stress: several hundred alternating gathers and picks on one weight, every gather bit-compared with the NCCL
    # gather of the same projection and every pick with the arg-max over it (orderings that only show up under load)
    fmt, N, K, M = "int8", 4096, 576, 1
    W, s = make_weight(fmt, N, K, 9500)
    Wl, sl = sharding.shard_weight(fmt, W, s, world, rank)
    lo, n = sharding.shard_rows(N, world, rank)
    qw = pkg.QuantWeight(ctx, fmt, Wl, sl)
    xs = [make_x(M, K, 9501 + i) for i in range(4)]
    dxs = [ctx.upload(x.view(np.uint16)) for x in xs]
    g1 = ctx.alloc(M * n * 2 * world)
    expect, expect_tok = [], []
    for dx in dxs:
        ctx.linear(M, n, K, dx, qw.buf, g1 + rank * M * n * 2)
        comm.all_gather(g1 + rank * M * n * 2, g1, M * n * 2)
        bits = ctx.download(g1, (world, M, n), np.uint16).copy()
        expect.append(bits)
        b32 = bits.reshape(-1).astype(np.uint32)
        expect_tok.append(int(np.argmax(np.where(b32 & 0x8000, 0xFFFF - b32, b32 | 0x8000))))
    bufs = [comm.symm_alloc(M * n * 2 * world) for _ in range(2)]
    tok = ctx.alloc(4)
    bad_g = bad_p = 0
    for i in range(300):
        j = i % 4
        comm.linear_gather(M, n, K, dxs[j], qw.buf, bufs[i & 1])
        comm.linear_argmax_sharded(n, K, dxs[j], qw.buf, None, tok)
        got = ctx.download(bufs[i & 1], (world, M, n), np.uint16)
        bad_g += int(not np.array_equal(got, expect[j]))
        bad_p += int(int(ctx.download(tok, (1,), np.int32)[0]) != expect_tok[j])
    if bad_g or bad_p:
        failures.append(f"stress: {bad_g} of 300 gathers and {bad_p} of 300 picks differ from the NCCL gather / its arg-max")
    ctx.sync()
    dist.barrier()
    for b in bufs:
        comm.symm_free(b)
    qw.release()
    for b in dxs + [g1, tok]:
        ctx.free(b)
    # the batched pick: M tokens per call, one key per row and rank instead of the logits
    for fmt, N, K, M in (("int8", 4096, 576, 8), ("q4", 2048, 1024, 40), ("int8", 3072, 896, 256), ("fp16", 1536, 896, 5)):
        W, s = make_weight(fmt, N, K, 9300 + N)
        Wl, sl = sharding.shard_weight(fmt, W, s, world, rank)
        lo, n = sharding.shard_rows(N, world, rank)
        qw = pkg.QuantWeight(ctx, fmt, Wl, sl)
        toks = ctx.alloc(M * 4)
        local = ctx.alloc(M * n * 2)
        g1 = ctx.alloc(M * n * 2 * world)
        for rep in range(3):
            x = make_x(M, K, 9400 + K + rep)
            if rep == 2:
                x[0] = 0                               # a row whose logits all tie at 0: row 0 of rank 0 wins
            dx = ctx.upload(x.view(np.uint16))
            ctx.linear(M, n, K, dx, qw.buf, g1 + rank * M * n * 2)
            comm.all_gather(g1 + rank * M * n * 2, g1, M * n * 2)
            bits = sharding.gathered_to_row_major(ctx.download(g1, (world, M, n), np.uint16), world, M, N)
            b32 = bits.astype(np.uint32)
            want = np.argmax(np.where(b32 & 0x8000, 0xFFFF - b32, b32 | 0x8000), axis=1)
            comm.linear_argmax_sharded_rows(M, n, K, dx, qw.buf, local, toks)
            got = ctx.download(toks, (M,), np.int32)
            if not np.array_equal(got, want):
                bad = int((got != want).sum())
                failures.append(f"batched pick {fmt} N={N} K={K} M={M} rep {rep}: {bad} of {M} rows differ from the gathered logits' arg-max")
            ctx.free(dx)
        ctx.sync()
        dist.barrier()
        qw.release()
        for b in (toks, local, g1):
            ctx.free(b)
    ctx.sync()
    dist.barrier()
    comm.close()
    ctx.close()
    ok = torch.tensor([0 if failures else 1])
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    for f in failures:
        print(f"rank {rank}: {f}", flush=True)
    if rank == 0:
        print("MULTI_GPU_OK" if int(ok.item()) == 1 else "MULTI_GPU_FAIL", flush=True)
    dist.destroy_process_group()
    return 0 if int(ok.item()) == 1 else 1


if __name__ == "__main__":
    sys.exit(main())

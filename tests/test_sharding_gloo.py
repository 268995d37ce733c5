"""World-size-2 CPU test of the row-sharding host logic (gloo): each rank computes its row
block with the oracle, the blocks are all-gathered in rank order, and the reassembled
[M, N] equals the unsharded result.  The GPU path uses the same arithmetic with NCCL.
The row-sharded greedy pick is covered the same way: every rank packs the key word of its rows,
the words are all-gathered, and every rank must name the first maximum of the unsharded logits."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, fmt, N, K, M, out_dir):
    sys.path.insert(0, REPO)
    sys.path.insert(0, os.path.join(REPO, "tests"))
    from conftest import load_package
    pkg = load_package()
    import importlib
    sharding = importlib.import_module("adreno_llms_b200.sharding")
    from oracle import cpu
    from helpers import make_weight, make_x
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    W, s = make_weight(fmt, N, K, 4242)              # same seed on every rank: replicated inputs
    x = make_x(M, K, 4243)
    Wl, sl = sharding.shard_weight(fmt, W, s, world, rank)
    lo, n = sharding.shard_rows(N, world, rank)
    assert Wl.shape[0] == n and (sl is None or sl.shape[0] == n)
    local = cpu.linear(fmt, x, Wl, sl)               # [M, N/G]
    send = torch.from_numpy(local.view(np.uint16).astype(np.int32).copy())
    recv = [torch.empty_like(send) for _ in range(world)]
    dist.all_gather(recv, send)
    gathered = np.stack([r.numpy().astype(np.uint16) for r in recv])       # [G][M][N/G]
    full = sharding.gathered_to_row_major(gathered, world, M, N).view(np.float16)
    want = cpu.linear(fmt, x, W, s)
    ok = np.array_equal(full.view(np.uint16), want.view(np.uint16))
    # a rank that never joined must surface as an error, not a hang: short timeout barrier
    dist.barrier()
    np.save(os.path.join(out_dir, f"ok{rank}.npy"), np.array([ok]))
    dist.destroy_process_group()


@pytest.mark.parametrize("fmt,N,K,M", [("int8", 256, 128, 3), ("q4", 64, 256, 1), ("fp16", 96, 64, 2)])
def test_row_sharded_linear_world2(tmp_path, fmt, N, K, M):
    port = _free_port()
    mp.spawn(_worker, args=(2, port, fmt, N, K, M, str(tmp_path)), nprocs=2, join=True)
    for r in range(2):
        assert np.load(tmp_path / f"ok{r}.npy")[0]


def test_shard_arithmetic(nnb):
    import importlib
    sharding = importlib.import_module("adreno_llms_b200.sharding")
    for N in (151936, 28672, 65536, 49152):
        for G in (1, 2, 4, 8):
            spans = [sharding.shard_rows(N, G, g) for g in range(G)]
            assert spans[0][0] == 0 and sum(n for _, n in spans) == N
            assert all(spans[i][0] + spans[i][1] == spans[i + 1][0] for i in range(G - 1))
    with pytest.raises(ValueError):
        sharding.shard_rows(10, 3, 0)
    with pytest.raises(ValueError):
        sharding.shard_rows(8, 2, 2)
    g = np.arange(2 * 3 * 4).reshape(2, 3, 4)
    rm = sharding.gathered_to_row_major(g, 2, 3, 8)
    assert rm.shape == (3, 8) and list(rm[1]) == [4, 5, 6, 7, 16, 17, 18, 19]


def _pick_worker(rank, world, port, fmt, N, K, case, out_dir):
    sys.path.insert(0, REPO)
    sys.path.insert(0, os.path.join(REPO, "tests"))
    from conftest import load_package
    load_package()
    import importlib
    sharding = importlib.import_module("adreno_llms_b200.sharding")
    from oracle import cpu
    from helpers import make_weight, make_x
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    W, s = make_weight(fmt, N, K, 5151)
    x = make_x(1, K, 5152) if case != "ties" else np.zeros((1, K), np.float16)
    full = cpu.linear(fmt, x, W, s).reshape(-1)
    if case == "nan":                                  # rank 1's rows are all NaN, rank 0 has one NaN
        full = full.copy()
        full[N // 2:] = np.float16(np.nan)
        full[3] = np.float16(np.nan)
    lo, n = sharding.shard_rows(N, world, rank)
    word = sharding.pick_key(full[lo:lo + n], lo, pick_number=7)
    send = torch.tensor([word - (1 << 64) if word >= (1 << 63) else word], dtype=torch.int64)
    recv = [torch.empty_like(send) for _ in range(world)]
    dist.all_gather(recv, send)
    words = [int(r.item()) & 0xFFFFFFFFFFFFFFFF for r in recv]
    got = sharding.pick_from_keys(words, pick_number=7)
    f32 = full.astype(np.float32)
    keys = np.where(np.isnan(f32), 0, sharding.ordered_half_bits(full.view(np.uint16)))
    want = int(np.argmax(keys)) if keys.max() > 0 else -1
    np.save(os.path.join(out_dir, f"pick{rank}.npy"), np.array([got, want]))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("fmt,N,K,case", [("int8", 256, 128, "plain"), ("q4", 128, 256, "plain"), ("fp16", 96, 64, "ties"),
                                         ("int8", 64, 128, "nan")])
def test_row_sharded_pick_world2(tmp_path, fmt, N, K, case):
    port = _free_port()
    mp.spawn(_pick_worker, args=(2, port, fmt, N, K, case, str(tmp_path)), nprocs=2, join=True)
    for r in range(2):
        got, want = np.load(tmp_path / f"pick{r}.npy")
        assert got == want and (case != "ties" or got == 0)


def test_pick_key_order_and_nan(nnb):
    import importlib
    sharding = importlib.import_module("adreno_llms_b200.sharding")
    vals = np.array([-np.inf, -3.5, -6e-8, -0.0, 0.0, 6e-8, 1.0, 65504.0, np.inf], np.float16)
    k = sharding.ordered_half_bits(vals.view(np.uint16))
    assert np.all(np.diff(k.astype(np.int64)) > 0) and k.min() > 0          # strictly increasing, never 0
    assert sharding.pick_from_keys([sharding.pick_key(np.full(4, np.nan, np.float16), 0)]) == -1
    a = sharding.pick_key(np.array([1, 5, 5, 2], np.float16), 100)           # first of the equal maxima
    b = sharding.pick_key(np.array([5, 0, 0, 0], np.float16), 104)           # equal value on a later rank
    assert sharding.pick_from_keys([a, b]) == 101 and sharding.pick_from_keys([b, a]) == 101
    with pytest.raises(ValueError):
        sharding.pick_from_keys([sharding.pick_key(np.ones(2, np.float16), 0, pick_number=3)], pick_number=4)


def _leaving_worker(rank, world, port, store_port, how, out_dir):
    """Two steps; rank 1 goes away between them (announced, or silently).  Rank 0 must learn of it
    on the host before its next launch, and a collective it starts anyway must end with an error."""
    import datetime
    import time
    sys.path.insert(0, REPO)
    sys.path.insert(0, os.path.join(REPO, "tests"))
    from conftest import load_package
    load_package()
    import importlib
    sharding = importlib.import_module("adreno_llms_b200.sharding")
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    store = dist.TCPStore("127.0.0.1", store_port, world, is_master=(rank == 0), timeout=datetime.timedelta(seconds=20))
    roll = sharding.RollCall(store, rank, world, timeout_s=1.0)
    # step 0: everybody is there
    roll.report(0)
    roll.check(0)
    t = torch.tensor([rank + 1])
    out = [torch.empty_like(t) for _ in range(world)]
    dist.all_gather(out, t)
    assert [int(o) for o in out] == [1, 2]
    if rank == 1:
        if how == "announced":
            roll.leave()
        # between steps, nothing in flight: this rank is gone (its process ends)
        if how == "announced":
            dist.destroy_process_group()
        return
    # rank 0, step 1
    roll.report(1)
    t0 = time.monotonic()
    try:
        roll.check(1)
        learned = "nothing"
    except sharding.PeerLost as e:
        learned = str(e)
    waited = time.monotonic() - t0
    # had it launched anyway: the collective ends with an error within the group's timeout, not a hang
    t1 = time.monotonic()
    try:
        dist.all_gather(out, t)
        collective = "completed"
    except Exception as e:                      # gloo reports a closed connection or a timeout
        collective = type(e).__name__
    took = time.monotonic() - t1
    with open(os.path.join(out_dir, "rank0.txt"), "w") as f:
        f.write(f"{learned}\n{waited:.3f}\n{collective}\n{took:.3f}\n")


@pytest.mark.parametrize("how", ["announced", "silent"])
def test_rank_leaving_between_steps_is_seen_on_the_host(tmp_path, how):
    port, store_port = _free_port(), _free_port()
    mp.spawn(_leaving_worker, args=(2, port, store_port, how, str(tmp_path)), nprocs=2, join=True)
    learned, waited, collective, took = open(tmp_path / "rank0.txt").read().splitlines()
    if how == "announced":
        assert "rank 1 left before step 1" in learned and float(waited) < 1.0
    else:
        assert "has not reported step 1" in learned and 0.9 <= float(waited) < 5.0
    assert collective != "completed" and float(took) < 30.0

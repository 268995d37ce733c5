"""Row sharding of the large projections across ranks (host-side arithmetic only).

The reference is single-device; it already cuts large weights into row tiles with
sub-buffers of W, scale and out (src/models/lfm2-5-350m/src/utils.cpp:427-452).  Here the
tile list becomes the rank list: rank g owns rows [g*N/G, (g+1)*N/G) of W and of its scales
(int8: N/G scales; Q4: N/G x K/32), x is replicated, every rank computes its [M, N/G] block
and an all-gather concatenates the blocks in rank order: gathered layout [G][M][N/G].
"""
import numpy as np


def shard_rows(N: int, world: int, rank: int):
    """(first row, row count) of `rank`; N must divide evenly (the configs' sizes do)."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} of {world}")
    if N % world:
        raise ValueError(f"N={N} is not divisible by {world} ranks")
    n = N // world
    return rank * n, n


def shard_weight(fmt: str, W: np.ndarray, scale, world: int, rank: int):
    """Row slice of the on-disk layout (rows are contiguous, so a slice is a view)."""
    lo, n = shard_rows(W.shape[0], world, rank)
    return W[lo:lo + n], (None if scale is None else scale[lo:lo + n])


def gathered_to_row_major(gathered: np.ndarray, world: int, M: int, N: int) -> np.ndarray:
    """[G][M][N/G] (what the all-gather produces) -> [M][N] (what pytorch_linear writes)."""
    n = N // world
    return np.ascontiguousarray(gathered.reshape(world, M, n).transpose(1, 0, 2)).reshape(M, N)

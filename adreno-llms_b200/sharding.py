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


# --- row-sharded greedy pick: host mirror of the 64-bit word the ranks exchange ------------------
# nn_linear_argmax_sharded leaves, on every rank, one word per rank:
#   pick number (16 bits) | ordered fp16 value (16 bits) | ~row (32 bits)
# "ordered" maps the sign-magnitude fp16 bits to an unsigned key that grows with the value
# (negative values complemented, the others with the top bit set; -0 sorts below +0), so the
# largest word is the largest value and, among equal values, the lowest row.  A payload of 0 means
# the rank saw only NaNs.

def ordered_half_bits(bits: np.ndarray) -> np.ndarray:
    """fp16 bit patterns -> unsigned keys that sort like the values (NaNs are the caller's to drop)."""
    b = np.asarray(bits).astype(np.uint32) & 0xFFFF
    return np.where(b & 0x8000, 0xFFFF - b, b | 0x8000).astype(np.uint32)


def pick_key(logits_fp16: np.ndarray, row_base: int, pick_number: int = 0) -> int:
    """The word a rank contributes for its rows `row_base + i` (first maximum, NaNs never win)."""
    bits = np.ascontiguousarray(logits_fp16, dtype=np.float16).view(np.uint16).reshape(-1)
    valid = (bits & 0x7FFF) <= 0x7C00
    tag = (pick_number & 0xFFFF) << 48
    if not valid.any():
        return tag
    keys = np.where(valid, ordered_half_bits(bits), 0)
    i = int(np.argmax(keys))                      # first of the largest keys = lowest row
    return tag | (int(keys[i]) << 32) | (0xFFFFFFFF - (row_base + i))


def pick_from_keys(words, pick_number: int = 0) -> int:
    """Winning global row among the ranks' words of one pick (-1: every value was NaN)."""
    best = 0
    for w in words:
        w = int(w)
        if (w >> 48) != (pick_number & 0xFFFF):
            raise ValueError(f"word {w:#018x} does not belong to pick {pick_number}")
        best = max(best, w & 0xFFFFFFFFFFFF)
    return -1 if best == 0 else 0xFFFFFFFF - (best & 0xFFFFFFFF)


class PeerLost(RuntimeError):
    """A rank of the sharded step left or stopped reporting; nothing must be launched that waits for it."""


class RollCall:
    """Host-side roll call between decode steps of a row-sharded model.

    The sharded lm_head stores into its peers' memory and waits (bounded) for their flags, so a
    rank may only launch a step when every peer is going to run it too.  Each rank reports the
    step it is about to launch into a key-value store (torch.distributed.TCPStore or anything
    with set / get / check) and reads its peers' reports before launching: a peer that announced
    its departure, or that has not reported within the timeout, raises PeerLost on the host,
    before any kernel is in flight.  A rank leaves only between steps (`leave`)."""

    def __init__(self, store, rank: int, world: int, timeout_s: float = 5.0, poll_s: float = 0.005):
        self.store, self.rank, self.world = store, rank, world
        self.timeout_s, self.poll_s = timeout_s, poll_s

    def _key(self, rank):
        return f"rollcall/{rank}"

    def report(self, step: int):
        self.store.set(self._key(self.rank), str(int(step)))

    def leave(self):
        self.store.set(self._key(self.rank), "left")

    def check(self, step: int):
        """Returns once every peer has reported `step` or a later one; raises PeerLost otherwise."""
        import time
        deadline = time.monotonic() + self.timeout_s
        for peer in range(self.world):
            if peer == self.rank:
                continue
            while True:
                seen = None
                if self.store.check([self._key(peer)]):
                    seen = self.store.get(self._key(peer)).decode()
                    if seen == "left":
                        raise PeerLost(f"rank {peer} left before step {step}")
                    if int(seen) >= step:
                        break
                if time.monotonic() > deadline:
                    raise PeerLost(f"rank {peer} has not reported step {step} within {self.timeout_s} s (last report: {seen})")
                time.sleep(self.poll_s)

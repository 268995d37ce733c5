"""Seeded synthetic operands shared by the GPU parity tests (shapes and value
distributions of the model configs: weights N(0, 0.02) cast to fp16 and then quantised
as the reference's scripts do, activations N(0, 1) fp16)."""
import os

import numpy as np

from oracle import cpu, quant

TOL = 1e-3  # relative L2 against the oracle, the bound stated for this path


def make_weight(fmt, N, K, seed, std=0.02):
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal((N, K)) * std).astype(np.float32).astype(np.float16)
    if fmt == "fp16":
        return w, None
    if fmt == "int8":
        return quant.quantize_int8(w)
    return quant.quantize_q4(w)


def make_x(M, K, seed):
    return np.random.default_rng(seed).standard_normal((M, K)).astype(np.float32).astype(np.float16)


def check_close(got, want, tol=TOL, what=""):
    got = np.asarray(got, dtype=np.float32)
    want = np.asarray(want, dtype=np.float32)
    assert got.shape == want.shape, (what, got.shape, want.shape)
    assert np.isfinite(got).all(), f"{what}: non-finite output"
    err = cpu.rel_l2(got, want)
    report(f"{what}: relative L2 {err:.3e} (bound {tol:g})")
    assert err < tol, f"{what}: relative L2 {err:.3e} >= {tol}"
    return err


def report(line):
    """Measured errors, one per line, into the file NNB_PARITY_REPORT names (nothing otherwise)."""
    path = os.environ.get("NNB_PARITY_REPORT")
    if path:
        with open(path, "a") as f:
            f.write(line + "\n")


CANARY_BYTES = 256


def alloc_with_canary(ctx, nbytes):
    """A device buffer followed by a patterned 256-byte tail that no kernel may touch."""
    buf = ctx.alloc(nbytes + CANARY_BYTES)
    tail = (np.arange(CANARY_BYTES, dtype=np.uint32) * 37 + 11).astype(np.uint8)
    host = np.concatenate([np.full(nbytes, 0x7E, np.uint8), tail])   # the body reads as fp16 NaNs
    ctx.upload(host, buf)
    return buf


def check_canary(ctx, buf, nbytes, what=""):
    got = ctx.download(buf, (nbytes + CANARY_BYTES,), np.uint8)[nbytes:]
    want = (np.arange(CANARY_BYTES, dtype=np.uint32) * 37 + 11).astype(np.uint8)
    assert np.array_equal(got, want), f"{what}: bytes past the end of the output were overwritten"

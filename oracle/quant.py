"""Vectorised numpy restatement of the reference's offline quantisers.

TEST INFRASTRUCTURE ONLY (synthetic weight generation for tests and the
benchmark, where the reference's own scripts are not available).  It is pinned
against vectors produced by the reference's own functions (tests/golden).

Follows, row for row:
  int8  src/models/lfm2-5-350m/scripts/quantize_weights.py:53-57
        (same function in src/models/smollm2-135m-instruct/scripts/quantize_weights.py:71-75)
  Q4    src/models/lfm2-5-350m/scripts/quantize_q4.py:62-82
Both read the fp16 bundle and upcast to fp32 before quantising.
"""
import numpy as np

Q4_BLOCK = 32


def quantize_int8(w_fp16: np.ndarray):
    """[N,K] fp16 -> (int8 [N,K], fp16 scale [N]).

    Per row: abs_max is an fp32 value promoted to a Python float (double);
    scale = abs_max / 127 in double (1.0 for an all-zero row); the division
    w / scale happens in fp32 with the scale rounded to fp32; the stored scale is
    the double rounded straight to fp16.
    """
    w32 = np.ascontiguousarray(w_fp16).astype(np.float32)
    absmax = np.max(np.abs(w32), axis=1).astype(np.float64)
    scale64 = np.where(absmax > 0, absmax / 127.0, 1.0)
    scale32 = scale64.astype(np.float32)
    q = np.clip(np.round(w32 / scale32[:, None]), -127, 127).astype(np.int8)
    return q, scale64.astype(np.float16)


def quantize_q4(w_fp16: np.ndarray):
    """[N,K] fp16 -> (uint8 [N,K/2] packed nibbles, fp16 scale [N,K/32]).

    Per block of 32: scale = absmax / 7 in fp32 (1.0 for an all-zero block),
    code = clip(round(w * (1/scale)), -7, 7), stored nibble = code + 8,
    byte i = nibble(2i) | nibble(2i+1) << 4.
    """
    w32 = np.ascontiguousarray(w_fp16).astype(np.float32)
    n, k = w32.shape
    if k % Q4_BLOCK:
        raise ValueError(f"Q4 requires K divisible by {Q4_BLOCK}, got {k}")
    blocks = w32.reshape(n, k // Q4_BLOCK, Q4_BLOCK)
    absmax = np.max(np.abs(blocks), axis=2)
    scales = np.where(absmax > 0, absmax / np.float32(7.0), np.float32(1.0)).astype(np.float32)
    inv = (np.float32(1.0) / scales)[:, :, None]
    q = np.clip(np.round(blocks * inv), -7.0, 7.0).astype(np.int8)
    stored = (q + 8).astype(np.uint8).reshape(n, k)
    packed = ((stored[:, 0::2] & 0x0F) | ((stored[:, 1::2] & 0x0F) << 4)).astype(np.uint8)
    return packed, scales.astype(np.float16)


def dequant_int8(q: np.ndarray, scale_fp16: np.ndarray) -> np.ndarray:
    """fp32 [N,K] = float(q) * float(scale[n])  (quantize_weights.py:136)."""
    return q.astype(np.float32) * scale_fp16.astype(np.float32)[:, None]


def unpack_q4_codes(packed: np.ndarray) -> np.ndarray:
    """uint8 [N,K/2] -> int32 [N,K] in [-8,7]: nibble - 8 (quantize_q4.py:158-163)."""
    n, kb = packed.shape
    codes = np.empty((n, kb * 2), dtype=np.int32)
    codes[:, 0::2] = packed & 0x0F
    codes[:, 1::2] = (packed >> 4) & 0x0F
    return codes - 8


def dequant_q4(packed: np.ndarray, scale_fp16: np.ndarray) -> np.ndarray:
    """fp32 [N,K] = float(nibble - 8) * float(scale[n, k/32])."""
    codes = unpack_q4_codes(packed).astype(np.float32)
    s = np.repeat(scale_fp16.astype(np.float32), Q4_BLOCK, axis=1)
    return codes * s

"""Seeded synthetic bundles shaped like the reference's model configs.

The real checkpoints are not available offline, so the benchmark and the smoke
check run on random weights of the same architecture: N(0, 0.02) fp32 cast to
fp16 (what scripts/convert_hf_to_bin.py stores), then quantised exactly as the
reference's offline tools do:
  int8  per-row symmetric, scale = absmax / 127 (1.0 for a zero row), fp16 scale
        (src/models/lfm2-5-350m/scripts/quantize_weights.py:53-57)
  Q4    per 32-weight block, scale = absmax / 7 (1.0 for a zero block), code in
        [-7, 7] stored as nibble code + 8, two per byte, low nibble first
        (src/models/lfm2-5-350m/scripts/quantize_q4.py:62-82)
Activations are N(0, 1) fp16.
"""
from dataclasses import dataclass

import numpy as np


@dataclass(frozen=True)
class ModelShape:
    name: str
    hidden: int
    layers: int
    q_dim: int
    kv_dim: int
    ffn: int
    vocab: int


# src/models/<model>/src/model_config.h of the three ports on the path
SMOLLM2_135M = ModelShape("smollm2-135m", 576, 30, 576, 192, 1536, 49152)
QWEN25_05B = ModelShape("qwen2.5-0.5b", 896, 24, 896, 128, 4864, 151936)
LFM25_350M = ModelShape("lfm2.5-350m", 1024, 16, 1024, 512, 4608, 65536)


def rows_int8(w16):
    w = np.asarray(w16, dtype=np.float32)
    amax = np.abs(w).max(axis=1).astype(np.float64)
    sc = np.where(amax > 0, amax / 127.0, 1.0)
    codes = np.rint(w / sc.astype(np.float32)[:, None])
    return np.clip(codes, -127, 127).astype(np.int8), sc.astype(np.float16)


def rows_q4(w16):
    w = np.asarray(w16, dtype=np.float32)
    n, k = w.shape
    if k % 32:
        raise ValueError("Q4 needs K % 32 == 0")
    blk = w.reshape(n, k // 32, 32)
    amax = np.abs(blk).max(axis=2)
    sc = np.where(amax > 0, amax / np.float32(7), np.float32(1)).astype(np.float32)
    codes = np.clip(np.rint(blk * (np.float32(1) / sc)[:, :, None]), -7, 7).astype(np.int8)
    nib = (codes + 8).astype(np.uint8).reshape(n, k)
    return (nib[:, 0::2] | (nib[:, 1::2] << 4)).astype(np.uint8), sc.astype(np.float16)


def weight(fmt, n, k, rng, std=0.02):
    """-> (bytes array in on-disk layout, fp16 scales or None)."""
    w16 = (rng.standard_normal((n, k), dtype=np.float32) * np.float32(std)).astype(np.float16)
    if fmt == "fp16":
        return w16, None
    if fmt == "int8":
        return rows_int8(w16)
    if fmt == "q4":
        return rows_q4(w16)
    raise ValueError(fmt)


def activations(m, k, rng):
    return rng.standard_normal((m, k), dtype=np.float32).astype(np.float16)


def linear_bytes(fmt, n, k, m=1):
    """Algorithmic bytes of one projection: weights + scales + x + y."""
    if fmt == "fp16":
        w = 2 * n * k
    elif fmt == "int8":
        w = n * k + 2 * n
    else:
        w = n * k // 2 + 2 * n * (k // 32)
    return w + 2 * m * k + 2 * m * n


def decode_step_ops(shape: ModelShape):
    """The projections of one decode step in launch order, as the SmolLM2 port fuses
    them (src/models/smollm2-135m-instruct/src/layers/attention.cpp:630-809,
    mlp.cpp:287-376, lm_head.cpp:300-448): per layer QKV (one launch, three weights),
    o_proj + residual, gate + up + SiLU, down + residual; then the tied lm_head."""
    ops = []
    for layer in range(shape.layers):
        ops.append(("qkv", layer, [(shape.q_dim, shape.hidden), (shape.kv_dim, shape.hidden), (shape.kv_dim, shape.hidden)]))
        ops.append(("o_add", layer, [(shape.hidden, shape.q_dim)]))
        ops.append(("gate_up", layer, [(shape.ffn, shape.hidden), (shape.ffn, shape.hidden)]))
        ops.append(("down_add", layer, [(shape.hidden, shape.ffn)]))
    ops.append(("lm_head", -1, [(shape.vocab, shape.hidden)]))
    return ops


def decode_step_bytes(shape: ModelShape, fmt, m=1):
    """Sum of linear_bytes over every projection of the step (the per-GEMV figure)."""
    return sum(linear_bytes(fmt, n, k, m) for _, _, ws in decode_step_ops(shape) for n, k in ws)


def decode_step_gemvs(shape: ModelShape):
    return sum(len(ws) for _, _, ws in decode_step_ops(shape))

#!/usr/bin/env python3
"""Regenerates the committed fixtures in this folder from the reference's own code.

Needs the reference checkout ($NNOPT_REFERENCE, or a directory "reference" beside this repository); the
tests themselves only read the committed outputs.  Run:  python tests/golden/make_golden.py

What it produces
  quant_int8.npz   fp16 rows -> (int8 codes, fp16 scales) by the reference's
                   quantize_row_symmetric (lfm2 and smollm2 copies, checked equal)
  quant_q4.npz     fp16 rows -> (packed nibbles, fp16 scales) by quantize_row_q4,
                   plus the block-0 reconstruction its sanity print computes
  bundle_lfm2/     model.{fp16,int8,q4}.bin + .meta.json written by the reference's
                   convert_hf_to_bin.py, quantize_weights.py and quantize_q4.py CLIs
                   from a tiny seeded safetensors file (LFM2 tensor names)
  bundle_smollm2/  model.{fp16,int8}.bin + .meta.json, same with the SmolLM2 script
  kernels_ref.npz  (only when oracle/_ref is built) outputs of the reference's
                   unmodified .cl kernels run on the CPU for seeded inputs
  rmsnorm_ref.npz  (same condition) outputs of the reference's rmsnorm_forward kernel
"""
import importlib.util
import json
import os
import shutil
import struct
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(os.path.dirname(HERE))
# the reference project's checkout: $NNOPT_REFERENCE, else a directory named "reference" beside this repository
REF = os.environ.get("NNOPT_REFERENCE") or os.path.join(os.path.dirname(REPO), "reference")
sys.path.insert(0, REPO)


def _load(path, name):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


LFM2_INT8 = os.path.join(REF, "src/models/lfm2-5-350m/scripts/quantize_weights.py")
LFM2_Q4 = os.path.join(REF, "src/models/lfm2-5-350m/scripts/quantize_q4.py")
SMOL_INT8 = os.path.join(REF, "src/models/smollm2-135m-instruct/scripts/quantize_weights.py")
CONVERT = os.path.join(REF, "scripts/convert_hf_to_bin.py")


def directed_rows(rng, n, k):
    """fp16 rows N(0, 0.02) plus directed cases: a zero row, a row with one spike,
    a row of exact ties (values at half-steps of the scale), tiny values."""
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32).astype(np.float16)
    w[1, :] = 0                                   # all-zero row / blocks -> scale 1.0
    w[2, :] = 0
    w[2, 5] = np.float16(0.75)                     # one spike: most codes round to 0
    w[3, :] = (np.arange(k) % 15 - 7).astype(np.float16) * np.float16(0.5)   # ties
    w[4, :] = np.float16(6e-8) * (np.arange(k) % 3)                           # subnormals
    w[5, : k // 2] = 0                             # a zero block inside a non-zero row
    return w


def make_quant():
    rng = np.random.default_rng(20240601)
    qi_l = _load(LFM2_INT8, "ref_lfm2_int8").quantize_row_symmetric
    qi_s = _load(SMOL_INT8, "ref_smol_int8").quantize_row_symmetric
    q4 = _load(LFM2_Q4, "ref_lfm2_q4").quantize_row_q4

    w = directed_rows(rng, 12, 96)
    q = np.empty(w.shape, np.int8)
    s = np.empty(w.shape[0], np.float16)
    for r in range(w.shape[0]):
        q[r], s[r] = qi_l(w[r])
        q2, s2 = qi_s(w[r])
        assert np.array_equal(q[r], q2) and s[r] == s2
    recon0 = q[0].astype(np.float32) * float(s[0])          # quantize_weights.py:136
    np.savez(os.path.join(HERE, "quant_int8.npz"), w=w.view(np.uint16), q=q, scale=s.view(np.uint16),
             recon_row0=recon0)

    w = directed_rows(rng, 10, 128)
    packed = np.empty((w.shape[0], w.shape[1] // 2), np.uint8)
    sc = np.empty((w.shape[0], w.shape[1] // 32), np.float16)
    for r in range(w.shape[0]):
        packed[r], sc[r] = q4(w[r].astype(np.float32))
    # block-0 reconstruction exactly as the script's sanity check (quantize_q4.py:156-163)
    q_stored = np.zeros(32, np.int32)
    for i in range(32):
        byte = packed[0, i // 2]
        q_stored[i] = (byte & 0xF) if (i % 2 == 0) else ((byte >> 4) & 0xF)
    recon = (q_stored.astype(np.float32) - 8.0) * float(sc[0, 0])
    np.savez(os.path.join(HERE, "quant_q4.npz"), w=w.view(np.uint16), packed=packed,
             scale=sc.view(np.uint16), recon_r0b0=recon)


def write_safetensors(path, tensors):
    """Minimal writer of the container convert_hf_to_bin.py parses (lines 58-63)."""
    header, blobs, off = {}, [], 0
    for name, arr in tensors.items():
        raw = arr.tobytes()
        dt = {np.dtype(np.float32): "F32", np.dtype(np.float16): "F16"}[arr.dtype]
        header[name] = {"dtype": dt, "shape": list(arr.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    hj = json.dumps(header).encode()
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)


def run(cmd):
    subprocess.run(cmd, check=True, stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL)


def make_bundle(kind):
    rng = np.random.default_rng(77 if kind == "lfm2" else 78)
    H, F, V = 32, 64, 24
    t = {"model.embed_tokens.weight": rng.standard_normal((V, H)).astype(np.float32) * 0.02,
         "model.norm.weight": np.ones(H, np.float32)}
    if kind == "lfm2":
        t["model.layers.0.conv.in_proj.weight"] = rng.standard_normal((3 * H, H)).astype(np.float32) * 0.02
        t["model.layers.0.conv.out_proj.weight"] = rng.standard_normal((H, H)).astype(np.float32) * 0.02
        t["model.layers.0.conv.conv.weight"] = rng.standard_normal((H, 1, 3)).astype(np.float32) * 0.02
        t["model.layers.1.self_attn.q_proj.weight"] = rng.standard_normal((H, H)).astype(np.float32) * 0.02
        t["model.layers.1.self_attn.k_proj.weight"] = rng.standard_normal((H // 2, H)).astype(np.float32) * 0.02
        t["model.layers.1.self_attn.v_proj.weight"] = rng.standard_normal((H // 2, H)).astype(np.float16)
        t["model.layers.1.self_attn.out_proj.weight"] = rng.standard_normal((H, H)).astype(np.float32) * 0.02
        for i in (0, 1):
            t[f"model.layers.{i}.feed_forward.w1.weight"] = rng.standard_normal((F, H)).astype(np.float32) * 0.02
            t[f"model.layers.{i}.feed_forward.w3.weight"] = rng.standard_normal((F, H)).astype(np.float32) * 0.02
            t[f"model.layers.{i}.feed_forward.w2.weight"] = rng.standard_normal((H, F)).astype(np.float32) * 0.02
    else:
        for i in (0, 1):
            p = f"model.layers.{i}."
            t[p + "self_attn.q_proj.weight"] = rng.standard_normal((H, H)).astype(np.float32) * 0.02
            t[p + "self_attn.k_proj.weight"] = rng.standard_normal((H // 4, H)).astype(np.float32) * 0.02
            t[p + "self_attn.v_proj.weight"] = rng.standard_normal((H // 4, H)).astype(np.float32) * 0.02
            t[p + "self_attn.o_proj.weight"] = rng.standard_normal((H, H)).astype(np.float32) * 0.02
            t[p + "mlp.gate_proj.weight"] = rng.standard_normal((F, H)).astype(np.float32) * 0.02
            t[p + "mlp.up_proj.weight"] = rng.standard_normal((F, H)).astype(np.float32) * 0.02
            t[p + "mlp.down_proj.weight"] = rng.standard_normal((H, F)).astype(np.float32) * 0.02
            t[p + "input_layernorm.weight"] = np.ones(H, np.float32)
    out = os.path.join(HERE, f"bundle_{kind}")
    shutil.rmtree(out, ignore_errors=True)
    os.makedirs(out)
    with tempfile.TemporaryDirectory() as tmp:
        st = os.path.join(tmp, "model.safetensors")
        write_safetensors(st, t)
        run([sys.executable, CONVERT, "--input", st, "--model-id", f"tiny-{kind}", "--output-dir", out])
    if kind == "lfm2":
        run([sys.executable, LFM2_INT8, "--weights-dir", out, "--emit-lm-head-int8"])
        run([sys.executable, LFM2_Q4, "--weights-dir", out, "--emit-lm-head-q4"])
    else:
        args = [sys.executable, SMOL_INT8, "--weights-dir", out]
        src = open(SMOL_INT8).read()
        if "--emit-lm-head-int8" in src:
            args.append("--emit-lm-head-int8")
        run(args)


def make_kernels_ref():
    try:
        from oracle import ref_cl
    except Exception as e:  # noqa: BLE001
        print("oracle/_ref not available, kernels_ref.npz not regenerated:", e)
        return
    if not ref_cl.available():
        print("oracle/_ref not built, kernels_ref.npz not regenerated")
        return
    ref_cl.write_golden(os.path.join(HERE, "kernels_ref.npz"))
    ref_cl.write_golden_rmsnorm(os.path.join(HERE, "rmsnorm_ref.npz"))


if __name__ == "__main__":
    make_quant()
    make_bundle("lfm2")
    make_bundle("smollm2")
    make_kernels_ref()
    print("golden fixtures written to", HERE)

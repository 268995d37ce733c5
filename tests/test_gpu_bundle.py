"""Bundles written by the reference's own scripts, loaded through the C ABI and through the
C++ mirror of the reference's interface, against the oracle on the same bytes."""
import ctypes
import json
import os
import subprocess

import numpy as np
import pytest

from oracle import cpu
from helpers import check_close, make_x

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _host_tensor(d, tag, name):
    meta = json.load(open(os.path.join(d, f"model.{tag}.meta.json")))["tensors"][name]
    raw = open(os.path.join(d, f"model.{tag}.bin"), "rb").read()
    dt = {"float16": np.float16, "int8": np.int8, "q4_packed": np.uint8}[meta["dtype"]]
    return np.frombuffer(raw, dtype=dt, count=meta["num_elements"], offset=meta["offset"]).reshape(meta["shape"])


@pytest.mark.parametrize("kind,tag", [("lfm2", "fp16"), ("lfm2", "int8"), ("lfm2", "q4"), ("smollm2", "int8")])
def test_every_projection_of_the_bundle(nnb, ctx, kind, tag):
    L = ctx.L
    d = os.path.join(GOLDEN, f"bundle_{kind}")
    w = ctypes.c_void_p()
    assert L.nn_weights_load(ctx.h, os.path.join(d, f"model.{tag}.bin").encode(),
                             os.path.join(d, f"model.{tag}.meta.json").encode(), ctypes.byref(w)) == 0
    nreg = L.nn_weights_register_quantized(ctx.h, w)
    meta = json.load(open(os.path.join(d, f"model.{tag}.meta.json")))["tensors"]
    quant_names = [n for n, t in meta.items() if t["dtype"] in ("int8", "q4_packed")]
    assert nreg == len(quant_names)
    done = 0
    for name, t in meta.items():
        if len(t["shape"]) != 2 or name.endswith(".scale"):
            continue
        fmt = {"float16": "fp16", "int8": "int8", "q4_packed": "q4"}[t["dtype"]]
        W = _host_tensor(d, tag, name)
        s = _host_tensor(d, tag, name + ".scale") if fmt != "fp16" else None
        N, K = W.shape[0], (W.shape[1] * 2 if fmt == "q4" else W.shape[1])
        x = make_x(1, K, 500 + done)
        xb = ctx.upload(x.view(np.uint16))
        ob = ctx.alloc(N * 2)
        Wb = L.nn_weights_get_buffer(w, name.encode(), 0)
        assert Wb and Wb == L.nn_weights_get_buffer(w, name.encode(), 0)      # created once, then cached
        ctx.linear(1, N, K, xb, Wb, ob)
        got = ctx.download(ob, (1, N), np.uint16).view(np.float16)
        check_close(got, cpu.linear(fmt, x, W, s), what=f"{kind}/{tag}/{name}")
        done += 1
    assert done >= 8
    assert L.nn_weights_free(w) == 0


def _build_host_mirror(tmp_path):
    exe = str(tmp_path / "host_mirror")
    lib_dir = os.path.join(REPO, "adreno-llms_b200", "lib")
    subprocess.check_call(["g++", "-std=c++17", "-O1", os.path.join(REPO, "tests", "host_mirror.cpp"), "-o", exe,
                           f"-L{lib_dir}", "-lnnopt_b200", f"-Wl,-rpath,{lib_dir}"])
    return exe


@pytest.mark.parametrize("tag,key,M", [("q4", "model.layers.0.feed_forward.w1.weight", 1), ("int8", "lm_head.weight", 3),
                                       ("fp16", "model.layers.1.self_attn.q_proj.weight", 1)])
def test_cpp_mirror_of_reference_interface(built_lib, tmp_path, tag, key, M):
    """nnopt::Weights + nnopt::pytorch_linear from C++ (the names the reference's layers call)."""
    exe = _build_host_mirror(tmp_path)
    d = os.path.join(GOLDEN, "bundle_lfm2")
    W = _host_tensor(d, tag, key)
    fmt = {"fp16": "fp16", "int8": "int8", "q4": "q4"}[tag]
    s = _host_tensor(d, tag, key + ".scale") if fmt != "fp16" else None
    K = W.shape[1] * 2 if fmt == "q4" else W.shape[1]
    x = make_x(M, K, 77)
    xf, of = tmp_path / "x.f16", tmp_path / "out.f16"
    x.view(np.uint16).tofile(xf)
    r = subprocess.run([exe, os.path.join(d, f"model.{tag}.bin"), os.path.join(d, f"model.{tag}.meta.json"), key, str(xf), str(of), str(M)],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    got = np.fromfile(of, dtype=np.uint16).view(np.float16).reshape(M, W.shape[0])
    check_close(got, cpu.linear(fmt, x, W, s), what=f"C++ mirror {tag} {key}")

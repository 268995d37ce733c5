"""CPU-side checks of the C-ABI library: it loads, exports every symbol the header
declares, fails loudly without a GPU, and its host-only parts (bundle loader) work."""
import ctypes
import json
import os

import numpy as np
import pytest

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _has_gpu(L):
    h = ctypes.c_void_p()
    rc = L.nn_init(0, ctypes.byref(h))
    if rc == 0:
        L.nn_shutdown(h)
    return rc == 0


def test_library_exports_every_declared_symbol(nnb, built_lib):
    names = nnb.declared_symbols()
    assert len(names) >= 45
    missing = [n for n in names if not hasattr(built_lib, n)]
    assert not missing, f"declared in include/nnopt_b200.h but not exported: {missing}"
    assert b"sm_100a" in built_lib.nn_version()


def test_no_cpu_fallback(nnb, built_lib):
    """Without a CUDA device nn_init fails with a clear message; nothing computes on the CPU."""
    if _has_gpu(built_lib):
        pytest.skip("a GPU is present")
    h = ctypes.c_void_p()
    rc = built_lib.nn_init(0, ctypes.byref(h))
    assert rc == nnb.NN_ERR_CUDA and not h.value
    assert b"no CPU path" in built_lib.nn_last_error()
    with pytest.raises(nnb.NNError):
        nnb.Context(0)


def test_null_arguments_are_rejected(nnb, built_lib):
    L = built_lib
    assert L.nn_linear(None, 1, 8, 8, None, None, None) == nnb.NN_ERR_ARG
    assert b"null context" in L.nn_last_error()
    assert L.nn_register_int8_weight(None, None, None, 4, 4) == nnb.NN_ERR_ARG
    assert L.nn_sync(None) == nnb.NN_ERR_ARG
    assert L.nn_plan_begin(None) == nnb.NN_ERR_ARG
    assert L.nn_shutdown(None) == 0 and L.nn_weights_free(None) == 0 and L.nn_plan_free(None) == 0


@pytest.mark.parametrize("kind,tag", [("lfm2", "fp16"), ("lfm2", "int8"), ("lfm2", "q4"), ("smollm2", "int8")])
def test_bundle_loader_matches_meta(nnb, built_lib, kind, tag):
    """Weights::load / has_tensor / get_dtype / get_shape / all_keys / get_host_vec on
    bundles written by the reference's own scripts."""
    L = built_lib
    d = os.path.join(GOLDEN, f"bundle_{kind}")
    binp, metap = os.path.join(d, f"model.{tag}.bin"), os.path.join(d, f"model.{tag}.meta.json")
    w = ctypes.c_void_p()
    assert L.nn_weights_load(None, binp.encode(), metap.encode(), ctypes.byref(w)) == 0
    meta = json.load(open(metap))["tensors"]
    raw = open(binp, "rb").read()
    n = L.nn_weights_num_keys(w)
    keys = [L.nn_weights_key_at(w, i).decode() for i in range(n)]
    assert keys == sorted(meta)
    for name, t in meta.items():
        assert L.nn_weights_has_tensor(w, name.encode()) == 1
        assert L.nn_weights_get_dtype(w, name.encode()).decode() == t["dtype"]
        dims = (ctypes.c_int * 4)()
        rank = L.nn_weights_get_shape(w, name.encode(), dims, 4)
        assert list(dims[:rank]) == t["shape"]
        assert L.nn_weights_get_size_bytes(w, name.encode()) == t["size_bytes"]
        assert L.nn_weights_get_num_elements(w, name.encode()) == t["num_elements"]
        out = np.empty(t["num_elements"], np.float32)
        assert L.nn_weights_get_host_f32(w, name.encode(), out.ctypes.data_as(ctypes.c_void_p), out.size) == 0
        dt = {"float16": np.float16, "int8": np.int8, "q4_packed": np.uint8}[t["dtype"]]
        want = np.frombuffer(raw, dtype=dt, count=t["num_elements"], offset=t["offset"]).astype(np.float32)
        assert np.array_equal(out, want)
    assert L.nn_weights_has_tensor(w, b"no.such.tensor") == 0
    assert L.nn_weights_get_dtype(w, b"no.such.tensor") == b""
    assert not L.nn_weights_get_buffer(w, b"no.such.tensor", 1)          # optional: silent
    assert not L.nn_weights_get_buffer(w, b"no.such.tensor", 0)          # loud
    assert b"weight key not found" in L.nn_last_error()
    assert L.nn_weights_free(w) == 0


def test_bundle_loader_errors(nnb, built_lib, tmp_path):
    L = built_lib
    w = ctypes.c_void_p()
    assert L.nn_weights_load(None, b"/nonexistent.bin", b"/nonexistent.json", ctypes.byref(w)) == nnb.NN_ERR_IO
    binp = tmp_path / "m.bin"
    binp.write_bytes(b"\0" * 64)
    bad = tmp_path / "bad.json"
    bad.write_text("{ not json")
    assert L.nn_weights_load(None, str(binp).encode(), str(bad).encode(), ctypes.byref(w)) == nnb.NN_ERR_IO
    # flat form (no "tensors" wrapper) and the older "size" key, both accepted by the reference parser
    flat = tmp_path / "flat.json"
    flat.write_text(json.dumps({"a.weight": {"offset": 0, "size": 32, "shape": [4, 4], "dtype": "float16"},
                                "format": "binary"}))
    assert L.nn_weights_load(None, str(binp).encode(), str(flat).encode(), ctypes.byref(w)) == 0
    assert L.nn_weights_num_keys(w) == 1 and L.nn_weights_get_num_elements(w, b"a.weight") == 16
    L.nn_weights_free(w)


def test_profile_aggregation_table(nnb, built_lib):
    """The per-launch profile's aggregation and table (the reference's exit-time table:
    src/models/lfm2-5-350m/src/kernel_profiler.cpp:18-62): totals per label, largest first,
    share of the whole, calls, average and maximum."""
    L = built_lib
    samples = [("gemv_m1_K1024_N4608_int8", 10.0), ("gemv_m1_K1024_N1024_int8_add", 4.0), ("gemv_m1_K1024_N4608_int8", 30.0),
               ("plan_replay", 100.0), ("gemv_m1_K1024_N1024_int8_add", 6.0), ("gemv_m1_K1024_N4608_int8", 20.0)]
    labels = (ctypes.c_char_p * len(samples))(*[s[0].encode() for s in samples])
    us = (ctypes.c_double * len(samples))(*[s[1] for s in samples])
    buf = ctypes.create_string_buffer(4096)
    n = L.nn_profile_aggregate(len(samples), labels, us, buf, len(buf))
    text = buf.value.decode()
    assert n == len(text)
    rows = [ln.split() for ln in text.splitlines() if ln and (ln.startswith("gemv") or ln.startswith("plan"))]
    assert [r[0] for r in rows] == ["plan_replay", "gemv_m1_K1024_N4608_int8", "gemv_m1_K1024_N1024_int8_add"]
    by = {r[0]: [float(v.rstrip("%")) for v in r[1:]] for r in rows}
    total_ms, share, calls, avg_us, max_us = by["gemv_m1_K1024_N4608_int8"]
    assert abs(total_ms - 0.060) < 1e-6 and calls == 3 and abs(avg_us - 20.0) < 1e-6 and abs(max_us - 30.0) < 1e-6
    assert abs(share - 100.0 * 60.0 / 170.0) < 0.06
    assert abs(by["plan_replay"][1] - 100.0 * 100.0 / 170.0) < 0.06
    # a short buffer is cut, never overrun; the length returned is the full table's
    small = ctypes.create_string_buffer(16)
    assert L.nn_profile_aggregate(len(samples), labels, us, small, len(small)) == n
    assert len(small.value) == 15
    assert L.nn_profile_aggregate(2, None, None, buf, len(buf)) == nnb.NN_ERR_ARG
    assert L.nn_profile_enabled(None) == 0


def test_named_nccl_library_is_the_only_one_tried(nnb, built_lib):
    """NNB_NCCL_LIB names the library to load: a wrong path is NN_ERR_COMM, not a silent
    switch to the libnccl the loader would find (checked in a child process: the library
    is loaded once per process)."""
    import subprocess
    import sys
    code = (
        "import ctypes, sys\n"
        f"L = ctypes.CDLL({nnb.LIB_PATH!r})\n"
        "L.nn_last_error.restype = ctypes.c_char_p\n"
        "buf = ctypes.create_string_buffer(128)\n"
        "rc = L.nn_comm_unique_id(buf)\n"
        "print(rc, L.nn_last_error().decode())\n"
    )
    env = dict(os.environ, NNB_NCCL_LIB="/nonexistent/libnccl.so.2")
    out = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=120)
    assert out.returncode == 0, out.stderr
    rc, msg = out.stdout.strip().split(" ", 1)
    assert int(rc) == nnb.NN_ERR_COMM
    assert "NNB_NCCL_LIB" in msg and "/nonexistent/libnccl.so.2" in msg

"""Runs the reference's own .cl kernels on the CPU (TEST INFRASTRUCTURE ONLY).

The shared libraries under oracle/_ref/ are built by oracle/build_ref.py from the
reference checkout.  This module calls a kernel by name with the kernel's own
argument list, with the launch geometry the reference's host code uses
(global size = N / outputs_per_group * 64, local size 64; utils.cpp:461-535, 676-740,
867-932 of the lfm2 port), and produces the committed fixture
tests/golden/kernels_ref.npz.
"""
import ctypes
import json
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_REF = os.path.join(_HERE, "_ref")
_libs = {}


def available() -> bool:
    return os.path.exists(os.path.join(_REF, "liblfm2_gemv_m1_int8.so"))


def _lib(tag):
    if tag not in _libs:
        L = ctypes.CDLL(os.path.join(_REF, f"lib{tag}.so"))
        L.refcl_run.argtypes = [ctypes.c_char_p, ctypes.c_ulong, ctypes.POINTER(ctypes.c_void_p), ctypes.c_int]
        L.refcl_run.restype = ctypes.c_int
        L.refcl_kernels.restype = ctypes.c_char_p
        _libs[tag] = L
    return _libs[tag]


class _Image(ctypes.Structure):
    _fields_ = [("data", ctypes.c_void_p), ("pitch", ctypes.c_size_t)]


def run(tag, kernel, args, n_groups, threads=1):
    """args: list of ("ptr", ndarray) | ("img", ndarray 2-D, row-major weight) | ("int", value) | ("float", value).
    Arrays are used in place (outputs are written into them)."""
    keep, argv = [], (ctypes.c_void_p * len(args))()
    for i, a in enumerate(args):
        if a[0] == "ptr":
            assert a[1].flags["C_CONTIGUOUS"]
            argv[i] = a[1].ctypes.data
        elif a[0] == "img":
            w = a[1]
            assert w.flags["C_CONTIGUOUS"] and w.ndim == 2
            im = _Image(w.ctypes.data, w.strides[0])
            keep.append(im)
            argv[i] = ctypes.addressof(im)
        elif a[0] == "float":
            v = ctypes.c_float(float(a[1]))
            keep.append(v)
            argv[i] = ctypes.addressof(v)
        else:
            v = ctypes.c_int(int(a[1]))
            keep.append(v)
            argv[i] = ctypes.addressof(v)
    rc = _lib(tag).refcl_run(kernel.encode(), n_groups, argv, threads)
    if rc != 0:
        raise KeyError(f"{kernel} not found in lib{tag}.so")


def _h(a):
    return np.ascontiguousarray(a).view(np.uint16).copy()


# ---- one entry per kernel family: (tag, kernel, rows per work-group) -----------------------
def gemv_scaled(tag, kernel, per_group, x, W, scale, threads=1):
    """int8 / Q4 kernels: (x, W_img, scales, out, N)."""
    N = W.shape[0]
    out = np.zeros(N, np.uint16)
    run(tag, kernel, [("ptr", _h(x)), ("img", np.ascontiguousarray(W)), ("ptr", _h(scale)), ("ptr", out), ("int", N)],
        N // per_group, threads)
    return out.view(np.float16)


def gemv_fp16_img(tag, kernel, per_group, x, W, threads=1):
    """fp16 image kernels: (x, W_img, out, N)."""
    N = W.shape[0]
    out = np.zeros(N, np.uint16)
    run(tag, kernel, [("ptr", _h(x)), ("img", _h(W)), ("ptr", out), ("int", N)], N // per_group, threads)
    return out.view(np.float16)


def residual_scaled(tag, kernel, x, W, scale, r, threads=1):
    """(x, W_img, scales, residual_inout, H), 4 rows per group."""
    N = W.shape[0]
    out = _h(r).reshape(-1)
    run(tag, kernel, [("ptr", _h(x)), ("img", np.ascontiguousarray(W)), ("ptr", _h(scale)), ("ptr", out), ("int", N)], N // 4, threads)
    return out.view(np.float16)


def residual_fp16_img(tag, kernel, x, W, r, threads=1):
    N = W.shape[0]
    out = _h(r).reshape(-1)
    run(tag, kernel, [("ptr", _h(x)), ("img", _h(W)), ("ptr", out), ("int", N)], N // 4, threads)
    return out.view(np.float16)


def swiglu_int8(x, Wg, sg, Wu, su, threads=1):
    N = Wg.shape[0]
    out = np.zeros(N, np.uint16)
    run("smollm2_block_fused_int8", "fused_gate_up_silu_m1_v4_img_int8",
        [("ptr", _h(x)), ("img", np.ascontiguousarray(Wg)), ("img", np.ascontiguousarray(Wu)), ("ptr", _h(sg)), ("ptr", _h(su)),
         ("ptr", out), ("int", N)], N, threads)
    return out.view(np.float16)


def swiglu_fp16(x, Wg, Wu, threads=1):
    N, K = Wg.shape
    out = np.zeros(N, np.uint16)
    run("smollm2_block_fused", "fused_gate_up_silu_m1_v4",
        [("ptr", _h(x)), ("ptr", _h(Wg)), ("ptr", _h(Wu)), ("ptr", out), ("int", K), ("int", N)], N, threads)
    return out.view(np.float16)


def silu_gate_fp16(x, W3, gate, threads=1):
    N = W3.shape[0]
    out = _h(gate).reshape(-1)
    run("lfm2_mlp_fused", "gemv_m1_k1024_no8_silufused_img", [("ptr", _h(x)), ("img", _h(W3)), ("ptr", out), ("int", N)], N // 8, threads)
    return out.view(np.float16)


def generic_fp16(x, W, threads=1):
    """lfm2 gemv_m1_generic(x, W, out, K, N): any K, one row per group."""
    N, K = W.shape
    out = np.zeros(N, np.uint16)
    run("lfm2_gemv_m1", "gemv_m1_generic", [("ptr", _h(x)), ("ptr", _h(W)), ("ptr", out), ("int", K), ("int", N)], N, threads)
    return out.view(np.float16)


def rmsnorm_fp16(x, weight, eps, threads=1):
    """rmsnorm_forward of the SmolLM2 port: one work-group per row."""
    xx, ww = _h(x), _h(weight)
    rows, cols = xx.shape
    out = np.zeros((rows, cols), np.uint16)
    run("smollm2_rmsnorm", "rmsnorm_forward", [("ptr", xx), ("ptr", ww), ("ptr", out), ("int", rows), ("int", cols), ("float", eps)], rows, threads)
    return out.view(np.float16)


def write_golden_rmsnorm(path):
    rng = np.random.default_rng(515151)
    data, cases = {}, []
    for i, (rows, cols, eps) in enumerate(((1, 576, 1e-5), (3, 1024, 1e-5), (2, 896, 1e-6), (1, 70, 1e-5), (4, 1536, 1e-5))):
        x = (rng.standard_normal((rows, cols)) * (0.3 + i)).astype(np.float32).astype(np.float16)
        w = (1.0 + 0.1 * rng.standard_normal(cols)).astype(np.float32).astype(np.float16)
        tag = f"rms{i}"
        data[tag + "_x"], data[tag + "_w"], data[tag + "_y"] = _h(x), _h(w), _h(rmsnorm_fp16(x, w, eps))
        cases.append({"tag": tag, "rows": rows, "cols": cols, "eps": eps})
    import json
    data["cases"] = np.frombuffer(json.dumps(cases).encode(), dtype=np.uint8)
    np.savez_compressed(path, **data)
    return cases


# ---- fixture generation ------------------------------------------------------------------
def write_golden(path):
    from oracle import quant
    rng = np.random.default_rng(424242)
    data, cases = {}, []

    def wfp16(n, k):
        return (rng.standard_normal((n, k)) * 0.02).astype(np.float32).astype(np.float16)

    def xv(k):
        return rng.standard_normal((1, k)).astype(np.float32).astype(np.float16)

    def add(tag, fmt, epi, kernel, x, W, s, y, **extra):
        data[tag + "_x"] = _h(x)
        data[tag + "_W"] = np.ascontiguousarray(W).view(np.uint16) if fmt == "fp16" else np.ascontiguousarray(W)
        if s is not None:
            data[tag + "_s"] = _h(s)
        data[tag + "_y"] = _h(y)
        for k, v in extra.items():
            data[tag + "_" + k] = v
        cases.append({"tag": tag, "fmt": fmt, "epi": epi, "kernel": kernel})

    # int8, lfm2 port
    for kern, K, per in (("gemv_m1_k1024_no4_img_int8", 1024, 4), ("gemv_m1_k1024_no8_img_int8", 1024, 8),
                         ("gemv_m1_k4608_no4_img_int8", 4608, 4), ("gemv_m1_k4608_no8_img_int8", 4608, 8),
                         ("gemv_m1_k2560_no4_img_int8", 2560, 4)):
        W, s = quant.quantize_int8(wfp16(8, K))
        x = xv(K)
        add(kern, "int8", "store", kern, x, W, s, gemv_scaled("lfm2_gemv_m1_int8", kern, per, x, W, s))
    # Q4, lfm2 port
    for kern, K, per in (("gemv_m1_k1024_q4_no4_img", 1024, 4), ("gemv_m1_k1024_q4_no8_img", 1024, 8),
                         ("gemv_m1_k4608_q4_no4_img", 4608, 4), ("gemv_m1_k2560_q4_no4_img", 2560, 4)):
        W, s = quant.quantize_q4(wfp16(8, K))
        x = xv(K)
        add(kern, "q4", "store", kern, x, W, s, gemv_scaled("lfm2_gemv_m1_q4", kern, per, x, W, s))
    # fp16 image kernels of the three ports
    for tag, kern, K, per in (("lfm2_gemv_m1", "gemv_m1_k1024_no4_img", 1024, 4), ("lfm2_gemv_m1", "gemv_m1_k1024_no2_img", 1024, 2),
                              ("lfm2_gemv_m1", "gemv_m1_k1024_no8_img", 1024, 8), ("lfm2_gemv_m1", "gemv_m1_k4608_no4_img", 4608, 4),
                              ("smollm2_block_fused", "gemv_m1_k576_no4_img", 576, 4),
                              ("qwen_gemv_m1", "gemv_m1_k896_no4_img", 896, 4), ("qwen_gemv_m1", "gemv_m1_k4864_no4_img", 4864, 4)):
        W = wfp16(8, K)
        x = xv(K)
        add(tag.split("_")[0] + "_" + kern, "fp16", "store", kern, x, W, None, gemv_fp16_img(tag, kern, per, x, W))
    # any-K generic kernel (vec4 steps + scalar tail)
    for K in (72, 576, 1000):   # this kernel takes K % 4 == 0 (no scalar tail)
        W = wfp16(9, K)
        x = xv(K)
        add(f"lfm2_generic_k{K}", "fp16", "store", "gemv_m1_generic", x, W, None, generic_fp16(x, W))
    # SmolLM2 int8 fused kernels
    W, s = quant.quantize_int8(wfp16(8, 576))
    x = xv(576)
    add("smol_k576_int8", "int8", "store", "gemv_m1_k576_no4_img_int8", x, W, s,
        gemv_scaled("smollm2_block_fused_int8", "gemv_m1_k576_no4_img_int8", 4, x, W, s))
    r = xv(8)
    add("smol_oproj_int8", "int8", "residual", "fused_oproj_residual_m1_no4_img_int8", x, W, s,
        residual_scaled("smollm2_block_fused_int8", "fused_oproj_residual_m1_no4_img_int8", x, W, s, r), r=_h(r))
    Wd, sd = quant.quantize_int8(wfp16(8, 1536))
    xd = xv(1536)
    add("smol_down_int8", "int8", "residual", "fused_down_residual_m1_no4_img_int8", xd, Wd, sd,
        residual_scaled("smollm2_block_fused_int8", "fused_down_residual_m1_no4_img_int8", xd, Wd, sd, r), r=_h(r))
    Wu, su = quant.quantize_int8(wfp16(8, 576))
    add("smol_swiglu_int8", "int8", "swiglu", "fused_gate_up_silu_m1_v4_img_int8", x, W, s, swiglu_int8(x, W, s, Wu, su),
        W2=Wu, s2=_h(su))
    # SmolLM2 fp16 fused kernels
    Wf, Wf2 = wfp16(8, 576), wfp16(8, 576)
    add("smol_oproj_fp16", "fp16", "residual", "fused_oproj_residual_m1_no4_img", x, Wf, None,
        residual_fp16_img("smollm2_block_fused", "fused_oproj_residual_m1_no4_img", x, Wf, r), r=_h(r))
    Wdf = wfp16(8, 1536)
    add("smol_down_fp16", "fp16", "residual", "fused_down_residual_m1_no4_img", xd, Wdf, None,
        residual_fp16_img("smollm2_block_fused", "fused_down_residual_m1_no4_img", xd, Wdf, r), r=_h(r))
    add("smol_swiglu_fp16", "fp16", "swiglu", "fused_gate_up_silu_m1_v4", x, Wf, None, swiglu_fp16(x, Wf, Wf2), W2=Wf2.view(np.uint16))
    # LFM2 silu(gate) * W3 x
    W3 = wfp16(8, 1024)
    x3, g3 = xv(1024), xv(8)
    add("lfm2_silufused", "fp16", "silu_gate", "gemv_m1_k1024_no8_silufused_img", x3, W3, None, silu_gate_fp16(x3, W3, g3), r=_h(g3))

    np.savez_compressed(path, cases=np.array(json.dumps(cases)), **data)
    return len(cases)

"""ctypes binding to the C oracle (oracle/oracle.c).  TEST INFRASTRUCTURE ONLY.

Only tests, the smoke check and the benchmark's CPU-baseline leg import this.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")

FMT_FP16, FMT_INT8, FMT_Q4 = 0, 1, 2
FMT = {"fp16": FMT_FP16, "int8": FMT_INT8, "q4": FMT_Q4}
ORDER_KERNEL, ORDER_FMA, ORDER_F64 = 0, 1, 2


def build(force: bool = False) -> str:
    src = os.path.join(_HERE, "oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-s", "-B", "liboracle.so"])
    return _LIB_PATH


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(_LIB_PATH)
        vp, i, sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t
        L.oracle_f16_to_f32.argtypes = [ctypes.c_uint16]
        L.oracle_f16_to_f32.restype = ctypes.c_float
        L.oracle_f32_to_f16.argtypes = [ctypes.c_float]
        L.oracle_f32_to_f16.restype = ctypes.c_uint16
        L.oracle_dequant.argtypes = [i, i, i, vp, vp, vp]
        L.oracle_dequant.restype = None
        L.oracle_linear_acc.argtypes = [i, i, i, i, vp, vp, vp, vp, i, i]
        L.oracle_linear_acc.restype = i
        L.oracle_store_half.argtypes = [sz, vp, vp]
        L.oracle_store_residual.argtypes = [sz, vp, vp]
        L.oracle_store_swiglu.argtypes = [sz, vp, vp, vp]
        L.oracle_store_silu_gate.argtypes = [sz, vp, vp]
        L.oracle_argmax_half.argtypes = [sz, vp]
        L.oracle_argmax_half.restype = i
        _lib = L
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _c(a, dt=None):
    if a is None:
        return None
    a = np.ascontiguousarray(a)
    return a if dt is None else a.view(dt) if a.dtype.itemsize == np.dtype(dt).itemsize else a.astype(dt)


def true_k(fmt: str, W: np.ndarray) -> int:
    return W.shape[1] * 2 if fmt == "q4" else W.shape[1]


def dequant(fmt: str, W, scale=None) -> np.ndarray:
    W = _c(W)
    N, K = W.shape[0], true_k(fmt, W)
    out = np.empty((N, K), dtype=np.float32)
    s = _c(scale, np.uint16)
    lib().oracle_dequant(FMT[fmt], N, K, _p(W), _p(s), _p(out))
    return out


def linear_acc(fmt: str, x, W, scale=None, order=ORDER_KERNEL, threads=1) -> np.ndarray:
    """fp32 [M,N]: the value held before the final half store."""
    W = _c(W)
    x = _c(x, np.uint16)
    if x.ndim == 1:
        x = x[None, :]
    M, K = x.shape
    N = W.shape[0]
    assert true_k(fmt, W) == K, (fmt, W.shape, K)
    acc = np.empty((M, N), dtype=np.float32)
    s = _c(scale, np.uint16)
    rc = lib().oracle_linear_acc(FMT[fmt], M, N, K, _p(W), _p(s), _p(x), _p(acc), order, threads)
    if rc != 0:
        raise ValueError("oracle_linear_acc rejected the arguments")
    return acc


def store_half(acc) -> np.ndarray:
    acc = _c(acc, np.float32)
    out = np.empty(acc.shape, dtype=np.uint16)
    lib().oracle_store_half(acc.size, _p(acc), _p(out))
    return out.view(np.float16)


def linear(fmt, x, W, scale=None, order=ORDER_KERNEL, threads=1) -> np.ndarray:
    """fp16 [M,N] = pytorch_linear(M,N,K,x,W) as the GEMV kernels compute it."""
    return store_half(linear_acc(fmt, x, W, scale, order, threads))


def linear_residual(fmt, x, W, scale, residual, order=ORDER_KERNEL) -> np.ndarray:
    acc = linear_acc(fmt, x, W, scale, order)
    r = _c(residual, np.uint16).copy().reshape(acc.shape)
    lib().oracle_store_residual(acc.size, _p(acc), _p(r))
    return r.view(np.float16)


def linear_swiglu(fmt, x, Wg, sg, Wu, su, order=ORDER_KERNEL) -> np.ndarray:
    g = linear_acc(fmt, x, Wg, sg, order)
    u = linear_acc(fmt, x, Wu, su, order)
    out = np.empty(g.shape, dtype=np.uint16)
    lib().oracle_store_swiglu(g.size, _p(g), _p(u), _p(out))
    return out.view(np.float16)


def linear_silu_gate(fmt, x, W3, s3, gate, order=ORDER_KERNEL) -> np.ndarray:
    acc = linear_acc(fmt, x, W3, s3, order)
    g = _c(gate, np.uint16).copy().reshape(acc.shape)
    lib().oracle_store_silu_gate(acc.size, _p(acc), _p(g))
    return g.view(np.float16)


def rmsnorm(x, weight, eps) -> np.ndarray:
    """fp16 [rows, cols] = the reference's rmsnorm_forward on fp16 storage."""
    x = _c(x, np.uint16)
    if x.ndim == 1:
        x = x[None, :]
    w = _c(weight, np.uint16)
    out = np.empty(x.shape, dtype=np.uint16)
    L = lib()
    L.oracle_rmsnorm_half.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_float, ctypes.c_void_p]
    L.oracle_rmsnorm_half(x.shape[0], x.shape[1], _p(x), _p(w), float(eps), _p(out))
    return out.view(np.float16)


def argmax_half(v) -> int:
    v = _c(v, np.uint16).reshape(-1)
    return int(lib().oracle_argmax_half(v.size, _p(v)))


def rel_l2(a, b) -> float:
    a = np.asarray(a, dtype=np.float64).reshape(-1)
    b = np.asarray(b, dtype=np.float64).reshape(-1)
    den = np.linalg.norm(b)
    return float(np.linalg.norm(a - b) / den) if den > 0 else float(np.linalg.norm(a - b))

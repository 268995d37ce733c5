"""ctypes view of libnnopt_b200.so for tests, the smoke check and the benchmark.

The product is the C-ABI shared library (include/nnopt_b200.h) and the C++ mirror
of the reference's operator interface (host/nnopt_linear.hpp); this module only
loads that library and moves numpy arrays in and out of device buffers.  The
directory name is not a Python identifier, so load it by path:

    import importlib.util, sys
    spec = importlib.util.spec_from_file_location("adreno_llms_b200", "adreno-llms_b200/__init__.py")
    mod = importlib.util.module_from_spec(spec); sys.modules[spec.name] = mod; spec.loader.exec_module(mod)

There is no fallback: if the library is missing or no GPU is present the calls fail.
"""
import ctypes
import os
import re

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libnnopt_b200.so")
HEADER_PATH = os.path.join(os.path.dirname(_HERE), "include", "nnopt_b200.h")

NN_OK, NN_ERR_ARG, NN_ERR_CUDA, NN_ERR_UNSUPPORTED, NN_ERR_IO, NN_ERR_NOTFOUND, NN_ERR_COMM, NN_ERR_TIMEOUT = 0, -1, -2, -3, -4, -5, -6, -7


class NNError(RuntimeError):
    def __init__(self, code, msg):
        super().__init__(f"nnopt_b200 error {code}: {msg}")
        self.code = code


def declared_symbols():
    """Every function name include/nnopt_b200.h declares."""
    text = open(HEADER_PATH).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(nn_[a-z0-9_]+)\s*\(", text)))


_lib = None


def load():
    """dlopen the library and declare argument types (no GPU needed for this)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise FileNotFoundError(f"{LIB_PATH} not built; run python adreno-llms_b200/build.py")
    L = ctypes.CDLL(LIB_PATH)
    vp, i, sz, cp = ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t, ctypes.c_char_p
    pvp = ctypes.POINTER(ctypes.c_void_p)
    sig = {
        "nn_last_error": ([], cp), "nn_version": ([], cp),
        "nn_init": ([i, pvp], i), "nn_shutdown": ([vp], i), "nn_stream": ([vp], vp), "nn_sync": ([vp], i),
        "nn_device_info": ([vp, ctypes.POINTER(i), ctypes.POINTER(sz), ctypes.POINTER(sz)], i),
        "nn_buf_alloc": ([vp, sz], vp), "nn_buf_free": ([vp, vp], i),
        "nn_buf_write": ([vp, vp, sz, vp, sz], i), "nn_buf_read": ([vp, vp, vp, sz, sz], i),
        "nn_buf_copy": ([vp, vp, vp, sz], i), "nn_buf_fill": ([vp, vp, i, sz], i),
        "nn_host_alloc": ([sz], vp), "nn_host_free": ([vp], i),
        "nn_register_int8_weight": ([vp, vp, vp, i, i], i), "nn_register_q4_weight": ([vp, vp, vp, i, i], i),
        "nn_unregister_weight": ([vp, vp], i),
        "nn_linear": ([vp, i, i, i, vp, vp, vp], i), "nn_linear_add": ([vp, i, i, i, vp, vp, vp], i),
        "nn_linear_silu_gate_fused": ([vp, i, i, i, vp, vp, vp], i),
        "nn_fused_gate_up_silu": ([vp, i, i, i, vp, vp, vp, vp], i),
        "nn_linear_qkv": ([vp, i, i, vp, vp, i, vp, i, vp, i, vp, vp, vp], i),
        "nn_linear_qkv_bias": ([vp, i, i, vp, vp, i, vp, i, vp, i, vp, vp, vp, vp, vp, vp], i),
        "nn_bias_add": ([vp, i, i, vp, vp], i),
        "nn_bandwidth_probe": ([vp, sz, i, ctypes.POINTER(ctypes.c_double), ctypes.POINTER(ctypes.c_double)], i),
        "nn_profile_enabled": ([vp], i), "nn_profile_report": ([vp, cp, sz, i], i),
        "nn_profile_aggregate": ([i, ctypes.POINTER(cp), ctypes.POINTER(ctypes.c_double), cp, sz], i),
        "nn_dequant": ([vp, i, i, vp, vp], i), "nn_argmax": ([vp, i, vp, vp], i),
        "nn_argmax_static": ([vp, i, vp, vp], i),
        "nn_linear_argmax": ([vp, i, i, vp, vp, vp, vp], i),
        "nn_rmsnorm": ([vp, i, i, vp, vp, ctypes.c_float, vp], i),
        "nn_rmsnorm_linear": ([vp, i, i, i, vp, vp, ctypes.c_float, vp, vp], i),
        "nn_rmsnorm_linear_qkv": ([vp, i, i, vp, vp, ctypes.c_float, vp, i, vp, i, vp, i, vp, vp, vp], i),
        "nn_rmsnorm_linear_qkv_bias": ([vp, i, i, vp, vp, ctypes.c_float, vp, i, vp, i, vp, i, vp, vp, vp, vp, vp, vp], i),
        "nn_rmsnorm_gate_up_silu": ([vp, i, i, i, vp, vp, ctypes.c_float, vp, vp, vp], i),
        "nn_plan_begin": ([vp], i), "nn_plan_end": ([vp, pvp], i), "nn_plan_launch": ([vp, vp], i),
        "nn_plan_num_kernels": ([vp], i), "nn_plan_free": ([vp], i),
        "nn_plan_num_recorded": ([vp], i), "nn_plan_num_resident_runs": ([vp], i),
        "nn_plan_set_wait_limit": ([vp, ctypes.c_uint], i), "nn_plan_withhold_output": ([vp, i, i], i),
        "nn_plan_analyze": ([i, vp, vp, vp, vp, vp, vp, i, vp, vp, vp, vp], i),
        "nn_weights_load": ([vp, cp, cp, pvp], i), "nn_weights_free": ([vp], i),
        "nn_weights_has_tensor": ([vp, cp], i), "nn_weights_get_buffer": ([vp, cp, i], vp),
        "nn_weights_get_dtype": ([vp, cp], cp), "nn_weights_get_shape": ([vp, cp, ctypes.POINTER(i), i], i),
        "nn_weights_get_size_bytes": ([vp, cp], sz), "nn_weights_get_num_elements": ([vp, cp], sz),
        "nn_weights_num_keys": ([vp], i), "nn_weights_key_at": ([vp, i], cp),
        "nn_weights_get_host_f32": ([vp, cp, vp, sz], i), "nn_weights_register_quantized": ([vp, vp], i),
        "nn_event_create": ([pvp], i), "nn_event_record": ([vp, vp], i),
        "nn_event_elapsed_ms": ([vp, vp, ctypes.POINTER(ctypes.c_float)], i), "nn_event_destroy": ([vp], i),
        "nn_l2_flush": ([vp], i), "nn_launch_count": ([vp], ctypes.c_longlong),
        "nn_comm_unique_id": ([vp], i), "nn_comm_init": ([vp, vp, i, i, pvp], i),
        "nn_comm_all_gather": ([vp, vp, vp, sz], i), "nn_comm_free": ([vp], i),
        "nn_comm_symm_alloc": ([vp, sz, pvp], i), "nn_comm_symm_free": ([vp, vp], i),
        "nn_linear_gather": ([vp, i, i, i, vp, vp, vp], i),
        "nn_linear_argmax_sharded": ([vp, i, i, vp, vp, vp, vp], i),
        "nn_comm_signal": ([vp], i), "nn_comm_wait": ([vp, ctypes.c_uint], i),
        "nn_comm_pick_unsent": ([vp, ctypes.c_uint, vp], i),
        "nn_linear_argmax_sharded_rows": ([vp, i, i, i, vp, vp, vp, vp], i),
        "nn_device_count": ([], i),
    }
    for name, (args, res) in sig.items():
        if hasattr(L, name):
            fn = getattr(L, name)
            fn.argtypes = args
            fn.restype = res
    _lib = L
    return L


def _check(rc):
    if rc != 0:
        raise NNError(rc, load().nn_last_error().decode())
    return rc


class Context:
    """One GPU, one stream: nn_init / nn_shutdown plus numpy conveniences."""

    def __init__(self, device=0):
        self.L = load()
        h = ctypes.c_void_p()
        _check(self.L.nn_init(device, ctypes.byref(h)))
        self.h = h
        self._bufs = []

    def close(self):
        if self.h:
            for b in self._bufs:
                self.L.nn_buf_free(self.h, b)
            self._bufs = []
            self.L.nn_shutdown(self.h)
            self.h = None

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    # -- buffers --
    def alloc(self, nbytes):
        p = self.L.nn_buf_alloc(self.h, nbytes)
        if not p:
            raise NNError(NN_ERR_CUDA, self.L.nn_last_error().decode())
        self._bufs.append(p)
        return p

    def free(self, p):
        if p in self._bufs:
            self._bufs.remove(p)
        _check(self.L.nn_buf_free(self.h, p))

    def upload(self, arr, buf=None):
        arr = np.ascontiguousarray(arr)
        if buf is None:
            buf = self.alloc(max(arr.nbytes, 16))
        _check(self.L.nn_buf_write(self.h, buf, 0, arr.ctypes.data_as(ctypes.c_void_p), arr.nbytes))
        _check(self.L.nn_sync(self.h))  # the source array may be a temporary
        return buf

    def download(self, buf, shape, dtype, offset=0):
        out = np.empty(shape, dtype=dtype)
        _check(self.L.nn_buf_read(self.h, out.ctypes.data_as(ctypes.c_void_p), buf, offset, out.nbytes))
        self.sync()
        return out

    def sync(self):
        _check(self.L.nn_sync(self.h))

    def device_info(self):
        sm, l2, hbm = ctypes.c_int(), ctypes.c_size_t(), ctypes.c_size_t()
        _check(self.L.nn_device_info(self.h, ctypes.byref(sm), ctypes.byref(l2), ctypes.byref(hbm)))
        return sm.value, l2.value, hbm.value

    # -- registry / operators (thin, same argument order as the C ABI) --
    def register_int8(self, W, scale, N, K):
        _check(self.L.nn_register_int8_weight(self.h, W, scale, N, K))

    def register_q4(self, W, scale, N, K):
        _check(self.L.nn_register_q4_weight(self.h, W, scale, N, K))

    def linear(self, M, N, K, x, W, out):
        _check(self.L.nn_linear(self.h, M, N, K, x, W, out))

    def linear_add(self, M, N, K, x, W, r):
        _check(self.L.nn_linear_add(self.h, M, N, K, x, W, r))

    def linear_silu_gate_fused(self, M, N, K, x, W3, g):
        _check(self.L.nn_linear_silu_gate_fused(self.h, M, N, K, x, W3, g))

    def fused_gate_up_silu(self, M, N, K, x, Wg, Wu, out):
        _check(self.L.nn_fused_gate_up_silu(self.h, M, N, K, x, Wg, Wu, out))

    def linear_qkv(self, M, K, x, Wq, Nq, Wk, Nk, Wv, Nv, q, k, v):
        _check(self.L.nn_linear_qkv(self.h, M, K, x, Wq, Nq, Wk, Nk, Wv, Nv, q, k, v))

    def linear_qkv_bias(self, M, K, x, Wq, Nq, Wk, Nk, Wv, Nv, bq, bk, bv, q, k, v):
        _check(self.L.nn_linear_qkv_bias(self.h, M, K, x, Wq, Nq, Wk, Nk, Wv, Nv, bq, bk, bv, q, k, v))

    def bias_add(self, rows, cols, out, bias):
        _check(self.L.nn_bias_add(self.h, rows, cols, out, bias))

    def bandwidth_probe(self, nbytes=0, trials=5):
        """Best-of-trials read bandwidth in GB/s: (plain 16-byte loads, TMA bulk copies)."""
        a, b = ctypes.c_double(), ctypes.c_double()
        _check(self.L.nn_bandwidth_probe(self.h, nbytes, trials, ctypes.byref(a), ctypes.byref(b)))
        return a.value, b.value

    def profile_enabled(self):
        return bool(self.L.nn_profile_enabled(self.h))

    def profile_report(self, reset=False):
        """The per-launch profile so far as the table nn_shutdown prints."""
        buf = ctypes.create_string_buffer(1 << 16)
        n = self.L.nn_profile_report(self.h, buf, len(buf), 1 if reset else 0)
        if n < 0:
            _check(n)
        return buf.value.decode()

    def dequant(self, N, K, W, out):
        _check(self.L.nn_dequant(self.h, N, K, W, out))

    def argmax(self, n, logits, out_idx):
        _check(self.L.nn_argmax(self.h, n, logits, out_idx))

    def linear_argmax(self, N, K, x, W, logits, out_idx):
        _check(self.L.nn_linear_argmax(self.h, N, K, x, W, logits, out_idx))

    def rmsnorm(self, rows, cols, x, weight, eps, out):
        _check(self.L.nn_rmsnorm(self.h, rows, cols, x, weight, eps, out))

    def rmsnorm_linear(self, M, N, K, x, gamma, eps, W, out):
        _check(self.L.nn_rmsnorm_linear(self.h, M, N, K, x, gamma, eps, W, out))

    def rmsnorm_linear_qkv(self, M, K, x, gamma, eps, Wq, Nq, Wk, Nk, Wv, Nv, q, k, v):
        _check(self.L.nn_rmsnorm_linear_qkv(self.h, M, K, x, gamma, eps, Wq, Nq, Wk, Nk, Wv, Nv, q, k, v))

    def rmsnorm_linear_qkv_bias(self, M, K, x, gamma, eps, Wq, Nq, Wk, Nk, Wv, Nv, bq, bk, bv, q, k, v):
        _check(self.L.nn_rmsnorm_linear_qkv_bias(self.h, M, K, x, gamma, eps, Wq, Nq, Wk, Nk, Wv, Nv, bq, bk, bv, q, k, v))

    def rmsnorm_gate_up_silu(self, M, N, K, x, gamma, eps, Wg, Wu, out):
        _check(self.L.nn_rmsnorm_gate_up_silu(self.h, M, N, K, x, gamma, eps, Wg, Wu, out))

    def l2_flush(self):
        _check(self.L.nn_l2_flush(self.h))

    def launch_count(self):
        return int(self.L.nn_launch_count(self.h))

    # -- recorded step --
    def plan_begin(self):
        _check(self.L.nn_plan_begin(self.h))

    def plan_end(self):
        p = ctypes.c_void_p()
        _check(self.L.nn_plan_end(self.h, ctypes.byref(p)))
        return p

    def plan_launch(self, plan):
        _check(self.L.nn_plan_launch(self.h, plan))

    # -- timing --
    def event(self):
        e = ctypes.c_void_p()
        _check(self.L.nn_event_create(ctypes.byref(e)))
        return e

    def record(self, ev):
        _check(self.L.nn_event_record(self.h, ev))

    def elapsed_ms(self, a, b):
        ms = ctypes.c_float()
        _check(self.L.nn_event_elapsed_ms(a, b, ctypes.byref(ms)))
        return ms.value


class QuantWeight:
    """A weight uploaded in its on-disk layout and registered like main.cpp does."""

    def __init__(self, ctx: Context, fmt: str, W: np.ndarray, scale=None):
        self.fmt = fmt
        self.N = W.shape[0]
        self.K = W.shape[1] * 2 if fmt == "q4" else W.shape[1]
        self.buf = ctx.upload(W)
        self.scale = None
        if fmt == "int8":
            self.scale = ctx.upload(np.ascontiguousarray(scale).view(np.uint16))
            ctx.register_int8(self.buf, self.scale, self.N, self.K)
        elif fmt == "q4":
            self.scale = ctx.upload(np.ascontiguousarray(scale).view(np.uint16))
            ctx.register_q4(self.buf, self.scale, self.N, self.K)
        self.nbytes = W.nbytes + (0 if scale is None else np.asarray(scale).nbytes)
        self.ctx = ctx

    def release(self):
        """Drop the registry entry and free the device copies."""
        if self.buf:
            if self.scale:
                _check(self.ctx.L.nn_unregister_weight(self.ctx.h, self.buf))
                self.ctx.free(self.scale)
            self.ctx.free(self.buf)
            self.buf = self.scale = None


class Comm:
    """Row-sharding communicator of one rank (nn_comm_*).  `unique_id()` is called on rank 0 and
    its 128 bytes are handed to the other ranks by whatever channel the host program has."""

    @staticmethod
    def unique_id():
        raw = (ctypes.c_ubyte * 128)()
        _check(load().nn_comm_unique_id(raw))
        return bytes(raw)

    def __init__(self, ctx: Context, id_bytes, rank: int, world: int):
        self.ctx, self.rank, self.world = ctx, rank, world
        raw = (ctypes.c_ubyte * 128)(*id_bytes) if id_bytes else None
        h = ctypes.c_void_p()
        _check(ctx.L.nn_comm_init(ctx.h, raw, rank, world, ctypes.byref(h)))
        self.h = h

    def all_gather(self, send, recv, bytes_per_rank):
        _check(self.ctx.L.nn_comm_all_gather(self.h, send, recv, bytes_per_rank))

    def symm_alloc(self, nbytes):
        p = ctypes.c_void_p()
        _check(self.ctx.L.nn_comm_symm_alloc(self.h, nbytes, ctypes.byref(p)))
        return p.value

    def symm_free(self, buf):
        _check(self.ctx.L.nn_comm_symm_free(self.h, buf))

    def linear_gather(self, M, n_local, K, x, W, gathered):
        _check(self.ctx.L.nn_linear_gather(self.h, M, n_local, K, x, W, gathered))

    def linear_argmax_sharded(self, n_local, K, x, W, logits_local, out_idx):
        _check(self.ctx.L.nn_linear_argmax_sharded(self.h, n_local, K, x, W, logits_local, out_idx))

    def linear_argmax_sharded_rows(self, M, n_local, K, x, W, logits_local, out_idx):
        _check(self.ctx.L.nn_linear_argmax_sharded_rows(self.h, M, n_local, K, x, W, logits_local, out_idx))

    def pick_unsent(self, timeout_ms, out_idx):
        _check(self.ctx.L.nn_comm_pick_unsent(self.h, timeout_ms, out_idx))

    def signal(self):
        _check(self.ctx.L.nn_comm_signal(self.h))

    def wait(self, timeout_ms=2000):
        _check(self.ctx.L.nn_comm_wait(self.h, timeout_ms))

    def close(self):
        if self.h:
            self.ctx.L.nn_comm_free(self.h)
            self.h = None

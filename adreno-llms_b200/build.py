"""Builds libnnopt_b200.so (C++ host layer + sm_100a CUDA kernels) in-tree with nvcc.

    python adreno-llms_b200/build.py [--force] [--verbose]

nvcc cross-compiles for sm_100a without a GPU.  The library links cudart
statically and dlopens NCCL at run time, so it has no dependency beyond the driver.
"""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB_DIR = os.path.join(HERE, "lib")
LIB = os.path.join(LIB_DIR, "libnnopt_b200.so")
SOURCES = ["api.cpp", "weights.cpp", "comm.cpp", "comm_kernels.cu", "gemv_stream.cu", "stage_image.cu", "decode_plan.cu", "plan.cpp", "gemv_generic.cu", "misc.cu", "gemm_tc.cu", "noalloc.cu"]
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _nvcc():
    return shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"


def sources():
    return [os.path.join(CSRC, s) for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]


def _stale():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [os.path.join(HERE, "..", "include", "nnopt_b200.h")]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False):
    if not force and not _stale():
        return LIB
    os.makedirs(LIB_DIR, exist_ok=True)
    objs = []
    for src in sources():
        obj = os.path.join(LIB_DIR, os.path.basename(src) + ".o")
        cmd = [_nvcc(), *ARCH, "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC,-Wall", "-x", "cu", "-c", src, "-o", obj]
        if verbose:
            cmd += ["-Xptxas", "-v"]
        if not force and os.path.exists(obj) and all(
                os.path.getmtime(obj) > os.path.getmtime(os.path.join(CSRC, f)) for f in os.listdir(CSRC)
                if f.endswith((".h", ".cuh")) or os.path.join(CSRC, f) == src):
            objs.append(obj)
            continue
        r = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or r.returncode:
            sys.stderr.write(r.stdout + r.stderr)
        if r.returncode:
            raise RuntimeError(f"nvcc failed on {src}")
        objs.append(obj)
    cmd = [_nvcc(), *ARCH, "-shared", "-o", LIB, *objs, "-cudart", "static", "-ldl", "-lpthread"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("link failed")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))

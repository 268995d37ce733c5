"""Compiles the reference's own OpenCL kernel sources for the CPU (TEST INFRASTRUCTURE ONLY).

    python oracle/build_ref.py            # needs the reference checkout ($NNOPT_REFERENCE, or a directory "reference" beside this repository)

For each .cl file on the decode GEMV path, g++ reads from a pipe:
    oracle/cl_shim.h  +  #define USE_FP16  +  the .cl file exactly where it lies in the
    reference checkout (one textual fix-up: a `__local` pointer PARAMETER loses its
    qualifier, which the shim cannot express)  +  a generated name -> call dispatcher.
Nothing from the reference is written into this repository; the outputs are shared
libraries under oracle/_ref/ (git-ignored).  Each kernel is then callable through
`refcl_run(name, n_groups, argv)` with the kernel's own argument list
(see oracle/ref_cl.py).

Built with -O2 -ffp-contract=off: multiply and add stay separate, and the shim's dot()
is evaluated left to right, so the outputs do not depend on FMA contraction.
"""
import os
import re
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
# the reference project's checkout: $NNOPT_REFERENCE, else a directory named "reference" beside this repository
REF = os.environ.get("NNOPT_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")

# (library tag, path inside the reference project)
CL_FILES = [
    ("lfm2_gemv_m1", "src/models/lfm2-5-350m/kernels/gemv_m1.cl"),
    ("lfm2_gemv_m1_int8", "src/models/lfm2-5-350m/kernels/gemv_m1_int8.cl"),
    ("lfm2_gemv_m1_q4", "src/models/lfm2-5-350m/kernels/gemv_m1_q4.cl"),
    ("lfm2_mlp_fused", "src/models/lfm2-5-350m/kernels/mlp_fused.cl"),
    ("smollm2_block_fused", "src/models/smollm2-135m-instruct/kernels/block_fused.cl"),
    ("smollm2_block_fused_int8", "src/models/smollm2-135m-instruct/kernels/block_fused_int8.cl"),
    ("qwen_gemv_m1", "src/models/qwen2-5-0-5b/kernels/gemv_m1.cl"),
    ("smollm2_rmsnorm", "src/models/smollm2-135m-instruct/kernels/rmsnorm.cl"),
]

_KERNEL_RE = re.compile(r"__kernel\b(?P<attrs>(?:\s*__attribute__\s*\(\((?:[^()]|\([^()]*\))*\)\))*)\s*void\s+(?P<name>\w+)\s*\((?P<params>[^{]*?)\)\s*\{", re.S)


def strip_comments(text):
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return re.sub(r"//[^\n]*", "", text)


def parse_kernels(text):
    """-> [(name, work_group_size_token, [(kind, ctype)])], kind in ptr/image/int/float/local."""
    out = []
    for m in _KERNEL_RE.finditer(strip_comments(text)):
        wg = re.search(r"reqd_work_group_size\s*\(\s*([\w]+)", m.group("attrs") or "")
        params = []
        for raw in m.group("params").split(","):
            p = " ".join(re.sub(r"__attribute__\s*\(\(.*?\)\)", "", raw).split())
            if not p:
                continue
            if "image2d_t" in p:
                params.append(("image", "image2d_t"))
            elif "*" in p:
                is_local = "__local" in p
                base = re.sub(r"\b(__global|__constant|__local|const|restrict)\b", "", p)
                base = base[: base.index("*")].strip()
                params.append(("local" if is_local else "ptr", base))
            elif re.search(r"\bfloat\b", p):
                params.append(("float", "float"))
            else:
                params.append(("int", "int"))
        out.append((m.group("name"), wg.group(1) if wg else "64", params))
    return out


def dispatcher(kernels):
    lines = ["\n#include <string.h>\n#include <thread>\n",
             'extern "C" int refcl_run(const char* name, unsigned long n_groups, void** argv, int n_threads) {']
    for name, wg, params in kernels:
        if any(k == "local" for k, _ in params):
            continue  # kernels taking a __local pointer are not on the projection path
        args = []
        for i, (kind, ctype) in enumerate(params):
            if kind == "image":
                args.append(f"*(image2d_t*)argv[{i}]")
            elif kind == "ptr":
                args.append(f"({ctype}*)argv[{i}]")
            elif kind == "float":
                args.append(f"*(float*)argv[{i}]")
            else:
                args.append(f"*(int*)argv[{i}]")
        call = f"{name}({', '.join(args)});"
        lines.append(f'  if (!strcmp(name, "{name}")) {{')
        lines.append(f"    const std::function<void()> body = [&]() {{ {call} }};")
        lines.append("    if (n_threads < 1) n_threads = 1;")
        lines.append("    if ((unsigned long)n_threads > n_groups) n_threads = n_groups ? (int)n_groups : 1;")
        lines.append("    std::vector<std::thread> th;")
        lines.append("    for (int t = 0; t < n_threads; ++t) {")
        lines.append("      const unsigned long g0 = n_groups * t / n_threads, g1 = n_groups * (t + 1) / n_threads;")
        lines.append(f"      th.emplace_back([&, g0, g1]() {{ clshim::run_groups(g0, g1, n_groups, {wg}, body); }});")
        lines.append("    }")
        lines.append("    for (auto& t : th) t.join();")
        lines.append("    return 0;")
        lines.append("  }")
    lines.append("  return -1;\n}")
    names = [k[0] for k in kernels if not any(kind == "local" for kind, _ in k[2])]
    lines.append('extern "C" const char* refcl_kernels() { return "' + " ".join(names) + '"; }')
    return "\n".join(lines) + "\n"


def build(verbose=False):
    if not os.path.isdir(REF):
        print(f"oracle/_ref: reference checkout not found at {REF}; skipped")
        return []
    os.makedirs(OUT, exist_ok=True)
    built = []
    for tag, rel in CL_FILES:
        src = os.path.join(REF, rel)
        if not os.path.exists(src):
            continue
        text = open(src, encoding="utf-8").read()
        kernels = parse_kernels(text)
        body = re.sub(r"__local(\s+\w+\s*\*)", r"\1", text)  # __local pointer parameters only
        unit = f'#include "{os.path.join(HERE, "cl_shim.h")}"\n#define USE_FP16 1\n#line 1 "{rel}"\n' + body + dispatcher(kernels)
        lib = os.path.join(OUT, f"lib{tag}.so")
        cmd = ["g++", "-x", "c++", "-std=c++17", "-O2", "-ffp-contract=off", "-fno-fast-math", "-fPIC", "-shared", "-w",
               "-o", lib, "-", "-lpthread", "-lm"]
        r = subprocess.run(cmd, input=unit, text=True, capture_output=True)
        if r.returncode:
            print(f"oracle/_ref: {rel} did not compile under the shim:\n{r.stderr[:2000]}")
            continue
        built.append((tag, [k[0] for k in kernels]))
        if verbose:
            print(f"oracle/_ref: built {lib}: {len(kernels)} kernels")
    with open(os.path.join(OUT, "MANIFEST"), "w") as f:
        for tag, names in built:
            f.write(f"{tag}: {' '.join(names)}\n")
    return built


if __name__ == "__main__":
    b = build(verbose=True)
    sys.exit(0 if b or not os.path.isdir(REF) else 1)

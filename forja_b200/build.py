"""Builds libforja_cuda.so (the sm_100a backend library) in-tree with nvcc.

The library has no Python, PyTorch or CPU-fallback dependency: CUDA runtime (linked statically)
and the C++ standard library only.
"""
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")
OUTPUT = os.path.join(HERE, "libforja_cuda.so")
SOURCES = ["fj_backend.cu", "fj_model.cu", "fj_elementwise.cu", "fj_paged.cu", "fj_gemm.cu", "fj_gemm_tma.cu", "fj_attn_tc5.cu", "fj_quant.cu", "fj_pack.cu", "fj_moe.cu", "fj_grouped.cu", "fj_grouped_tc5.cu", "fj_sample.cu", "fj_dense_ops.cu", "fj_sched.cpp", "fj_weights.cpp"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
              "--expt-relaxed-constexpr", "-I", INCLUDE, "-I", CSRC]


def _deps():
    files = [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [os.path.join(INCLUDE, "forja_cuda.h")]
    return [f for f in files if f.endswith((".cu", ".cuh", ".h", ".cpp"))]


def needs_build() -> bool:
    if not os.path.exists(OUTPUT):
        return True
    built = os.path.getmtime(OUTPUT)
    return any(os.path.getmtime(f) > built for f in _deps())


def _compile(src: str, verbose: bool) -> str:
    obj = os.path.join(CSRC, os.path.splitext(src)[0] + ".o")
    deps_newer = not os.path.exists(obj) or any(os.path.getmtime(f) > os.path.getmtime(obj) for f in _deps() if f.endswith((".cuh", ".h")) or f.endswith(src))
    if deps_newer:
        cmd = ["nvcc", *NVCC_FLAGS, "-c", os.path.join(CSRC, src), "-o", obj]
        if verbose:
            cmd += ["-Xptxas", "-v"]
        out = subprocess.run(cmd, capture_output=True, text=True)
        if verbose:
            sys.stderr.write(out.stderr)
        if out.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src}:\n{out.stdout}\n{out.stderr}")
    return obj


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not needs_build():
        return OUTPUT
    if force:
        for s in SOURCES:
            obj = os.path.join(CSRC, os.path.splitext(s)[0] + ".o")
            if os.path.exists(obj):
                os.remove(obj)
    with ThreadPoolExecutor(max_workers=8) as pool:
        objs = list(pool.map(lambda s: _compile(s, verbose), SOURCES))
    cmd = ["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-Xcompiler", "-fPIC", "-cudart", "static", "-o", OUTPUT, *objs, "-ldl"]
    subprocess.check_call(cmd)
    return OUTPUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))

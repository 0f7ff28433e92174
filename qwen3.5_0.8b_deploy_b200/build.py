"""Builds libb200attn.so in-tree with nvcc for sm_100a (cross-compiles without a GPU).

    python qwen3.5_0.8b_deploy_b200/build.py [--force] [--verbose]

One translation unit per .cu under csrc/, compiled in parallel, linked against cudart and cuBLAS.
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import shlex
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "libb200attn.so")
OBJ = os.path.join(HERE, "build")
SOURCES = ["gemm.cu", "kv_cache.cu", "fa_decode.cu", "fa_prefill.cu", "fa_ops.cu", "la_kernels.cu", "la_chunk.cu",
           "la_ops.cu", "stack.cu", "fa_decode_static.cu", "gemm_tc.cu"]
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
         "--expt-relaxed-constexpr", "-Xptxas", "-v"]
FLAGS += shlex.split(os.environ.get("B200ATTN_NVCC_EXTRA", ""))      # e.g. "-DNAME" to try a compile-time variant


def _newest_header() -> float:
    hs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    hs.append(os.path.join(HERE, "..", "include", "b200attn.h"))
    return max(os.path.getmtime(h) for h in hs)


def _compile(src: str, force: bool, verbose: bool) -> str:
    obj = os.path.join(OBJ, src.replace(".cu", ".o"))
    path = os.path.join(CSRC, src)
    if (not force and os.path.exists(obj) and os.path.getmtime(obj) > os.path.getmtime(path)
            and os.path.getmtime(obj) > _newest_header()):
        return obj
    cmd = [NVCC, *FLAGS, "-c", path, "-o", obj]
    p = subprocess.run(cmd, capture_output=True, text=True)
    log = os.path.join(OBJ, src.replace(".cu", ".ptxas.log"))
    with open(log, "w") as f:
        f.write(p.stdout + p.stderr)
    if p.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src}:\n{p.stderr[-6000:]}")
    if verbose:
        print(p.stderr)
    return obj


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    srcs = [s for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]
    with cf.ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        objs = list(ex.map(lambda s: _compile(s, force, verbose), srcs))
    if force or not os.path.exists(OUT) or any(os.path.getmtime(o) > os.path.getmtime(OUT) for o in objs):
        cmd = [NVCC, "-shared", "-o", OUT, *objs, "-lcublas", "-Xlinker", "-rpath,/usr/local/cuda/lib64"]
        p = subprocess.run(cmd, capture_output=True, text=True)
        if p.returncode != 0:
            raise RuntimeError(f"link failed:\n{p.stderr[-4000:]}")
    build_compat(force)
    return OUT


def build_compat(force: bool = False) -> None:
    """libb200attn_compat.so (the reference's operator classes on top of the C ABI) and the compat_check program."""
    comp = os.path.join(HERE, "compat")
    lib = os.path.join(HERE, "libb200attn_compat.so")
    exe = os.path.join(comp, "compat_check")
    srcs = [os.path.join(comp, f) for f in ("qwen_cuda_compat.cpp", "qwen_cuda_compat.hpp", "compat_check.cpp", "qwen_cuda_compat_free.cu")]
    newest = max(os.path.getmtime(f) for f in srcs + [OUT])
    if not force and os.path.exists(lib) and os.path.exists(exe) and min(os.path.getmtime(lib), os.path.getmtime(exe)) > newest:
        return
    cxx = os.environ.get("CXX", "g++")
    common = ["-std=c++17", "-O2", "-I/usr/local/cuda/include", "-L/usr/local/cuda/lib64", f"-L{HERE}"]
    free_obj = os.path.join(OBJ, "qwen_cuda_compat_free.o")     # the free launchers carry small conversion kernels
    for cmd in (
        [NVCC, "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O2", "-std=c++17", "-Xcompiler", "-fPIC", "-c", srcs[3], "-o", free_obj],
        [cxx, *common, "-fPIC", "-shared", "-o", lib, srcs[0], free_obj, "-lb200attn", "-lcudart", "-Wl,-rpath,$ORIGIN", "-Wl,-rpath,/usr/local/cuda/lib64"],
        [cxx, *common, "-o", exe, srcs[2], "-lb200attn_compat", "-lb200attn", "-lcudart", "-Wl,-rpath,$ORIGIN/..",
         "-Wl,-rpath,/usr/local/cuda/lib64"],
    ):
        p = subprocess.run(cmd, capture_output=True, text=True)
        if p.returncode != 0:
            raise RuntimeError(f"compat build failed: {' '.join(cmd)}\n{p.stderr[-4000:]}")


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))

"""Compiles the CUDA sources of this package into one shared library, in-tree.

    python llm-infer_b200/build.py            # build if sources are newer than the library
    python llm-infer_b200/build.py --force
    python llm-infer_b200/build.py --check    # checking build (libllm_infer_attn_check.so, -DATTN_BOUNDS_CHECK): the
                                              # decode passes verify their workspace indices and report instead of
                                              # accessing; loaded when LLM_INFER_ATTN_LIB names it
    python llm-infer_b200/build.py --trace    # profiling build (libllm_infer_attn_trace.so): the decode kernels
                                              # record time stamps per CTA; loaded when LLM_INFER_ATTN_LIB names it

Only sm_100a code is generated. nvcc cross-compiles, so no GPU is needed to build.
"""
from __future__ import annotations

import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")
LIB = os.path.join(HERE, "libllm_infer_attn.so")
TRACE_LIB = os.path.join(HERE, "libllm_infer_attn_trace.so")
CHECK_LIB = os.path.join(HERE, "libllm_infer_attn_check.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def sources() -> list[str]:
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def _deps() -> list[str]:
    return sources() + glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(INCLUDE, "*.h")) + \
        glob.glob(os.path.join(INCLUDE, "*.cuh"))


def needs_build(lib: str = LIB) -> bool:
    if not os.path.exists(lib):
        return True
    t = os.path.getmtime(lib)
    return any(os.path.getmtime(f) > t for f in _deps())


def build_library(force: bool = False, verbose: bool = False, trace: bool = False, check: bool = False) -> str:
    """Compile every .cu under csrc/ (one object per file, in parallel) and link the library. ``trace`` builds the
    profiling variant (-DATTN_TRACE), ``check`` the index-checking variant (-DATTN_BOUNDS_CHECK), each next to the
    product library, which they never replace."""
    lib = TRACE_LIB if trace else CHECK_LIB if check else LIB
    if not force and not needs_build(lib):
        return lib
    nvcc = os.environ.get("NVCC", "nvcc")
    objdir = os.path.join(HERE, "build_trace" if trace else "build_check" if check else "build")
    os.makedirs(objdir, exist_ok=True)
    procs = []
    objs = []
    for src in sources():
        obj = os.path.join(objdir, os.path.basename(src)[:-3] + ".o")
        objs.append(obj)
        defines = ["-DATTN_TRACE"] if trace else ["-DATTN_BOUNDS_CHECK"] if check else []
        cmd = [nvcc, *NVCC_FLAGS, *defines, "-I", INCLUDE, "-c", src, "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for src, pr in procs:
        out, _ = pr.communicate()
        if pr.returncode != 0 or verbose:
            sys.stderr.write(f"--- {os.path.basename(src)} ---\n{out}\n")
        failed |= pr.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    subprocess.check_call([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-o", lib, *objs])
    return lib


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose="-v" in sys.argv, trace="--trace" in sys.argv,
                        check="--check" in sys.argv))

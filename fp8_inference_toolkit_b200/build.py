"""Build the CUDA library in-tree with nvcc for sm_100a.

    python fp8_inference_toolkit_b200/build.py [--force] [--verbose]

Produces ``fp8_inference_toolkit_b200/csrc/libint4tc_b200.so`` (a plain C-ABI shared library with
no PyTorch dependency).  nvcc cross-compiles without a GPU.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(CSRC, "libint4tc_b200.so")
SOURCES = ["runtime.cu", "quant.cu", "quant_ext.cu", "gemm_kernel.cu", "gemm_host.cu", "gemv.cu", "skinny.cu", "moe.cu"]
HEADERS = ["common.cuh", "gemm.cuh", "ptx.cuh", os.path.join("..", "..", "include", "int4tc_b200.h")]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; the int4tc_b200 library cannot be built")
    return cand


def _stale() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, s) for s in SOURCES + HEADERS] + [os.path.abspath(__file__)]
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile every .cu file for sm_100a and link the shared library.  Returns its path."""
    if not force and not _stale():
        return LIB
    nvcc = _nvcc()
    flags = [
        "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
        "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
    ]
    if verbose:
        flags += ["-Xptxas", "-v"]
    objs = []
    procs = []
    for s in SOURCES:
        o = os.path.join(CSRC, s.replace(".cu", ".o"))
        objs.append(o)
        cmd = [nvcc, *flags, "-c", os.path.join(CSRC, s), "-o", o]
        procs.append((cmd, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for cmd, p in procs:
        out, _ = p.communicate()
        if verbose or p.returncode != 0:
            sys.stderr.write(" ".join(cmd) + "\n" + out)
        failed |= p.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed; see the output above")
    link = [nvcc, "-shared", "-o", LIB, *objs, "-gencode", "arch=compute_100a,code=sm_100a"]
    r = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout)
        raise RuntimeError("link failed")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))

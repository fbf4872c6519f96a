"""In-tree build of the C-ABI library ``lib/libgraphcuda_b200.so`` with nvcc.

Every translation unit is compiled for sm_100a only (``-gencode
arch=compute_100a,code=sm_100a``), without fast-math (the adjacency
normalisation must round like IEEE/torch-CPU), and linked into one shared
object with the static CUDA runtime.  The driver API is reached through
``cudaGetDriverEntryPoint`` at run time, so the library has no link-time
dependency on libcuda and builds on a machine without a GPU.

Usage:  python -m graphcuda_b200.build [-v] [--force]
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
LIBDIR = os.path.join(PKG, "lib")
OBJDIR = os.path.join(LIBDIR, "obj")
LIBNAME = "libgraphcuda_b200.so"

SOURCES = [
    "abi.cu",
    "spmm_csr.cu",
    "gather_probe.cu",
    "gemm.cu",
    "gemm_simt.cu",
    "gemm_tcgen05.cu",
    "elementwise.cu",
    "gcn_layer.cu",
    "graph_build.cu",
    "loss.cu", "optim.cu",
]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def lib_path() -> str:
    return os.path.join(LIBDIR, LIBNAME)


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; set NVCC or install the CUDA toolkit")
    return cand


def _deps_mtime() -> float:
    t = 0.0
    for root in (CSRC, os.path.join(os.path.dirname(PKG), "include")):
        for f in os.listdir(root):
            if f.endswith((".cu", ".cuh", ".h")):
                t = max(t, os.path.getmtime(os.path.join(root, f)))
    return t


def _sources() -> list[str]:
    return [s for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]


def build(verbose: bool = False, force: bool = False, ptxas_verbose: bool = False) -> str:
    """Compile what is out of date and link; returns the library path."""
    os.makedirs(OBJDIR, exist_ok=True)
    nvcc = _nvcc()
    newest = _deps_mtime()
    headers_newest = max(
        [os.path.getmtime(os.path.join(CSRC, f)) for f in os.listdir(CSRC) if f.endswith(".cuh")]
        + [os.path.getmtime(os.path.join(os.path.dirname(PKG), "include", "graphcuda_b200.h"))]
    )
    jobs = []
    objs = []
    for src in _sources():
        sp = os.path.join(CSRC, src)
        op = os.path.join(OBJDIR, src[:-3] + ".o")
        objs.append(op)
        stale = force or not os.path.exists(op) or os.path.getmtime(op) < max(os.path.getmtime(sp), headers_newest)
        if stale:
            cmd = [nvcc, *NVCC_FLAGS, "-c", sp, "-o", op]
            if ptxas_verbose:
                cmd[1:1] = ["-Xptxas", "-v"]
            jobs.append((src, cmd))

    def run(job):
        src, cmd = job
        r = subprocess.run(cmd, capture_output=True, text=True)
        return src, r.returncode, r.stdout + r.stderr

    if jobs:
        with cf.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for src, rc, out in ex.map(run, jobs):
                if verbose or rc != 0 or ptxas_verbose:
                    sys.stderr.write(f"[nvcc {src}] rc={rc}\n{out}\n")
                if rc != 0:
                    raise RuntimeError(f"nvcc failed on {src}:\n{out}")
    lp = lib_path()
    if jobs or not os.path.exists(lp) or os.path.getmtime(lp) < newest:
        cmd = [nvcc, "-shared", "-o", lp, *objs, "-gencode", "arch=compute_100a,code=sm_100a"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("link failed:\n" + r.stdout + r.stderr)
    return lp


if __name__ == "__main__":
    p = build(verbose="-v" in sys.argv, force="--force" in sys.argv, ptxas_verbose="--ptxas" in sys.argv)
    print(p)

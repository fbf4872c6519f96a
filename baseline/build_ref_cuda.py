"""Builds the reference's own CUDA extension, unmodified, for the same-box GPU comparison.

The sources are compiled where they lie in the mounted reference tree
(src/graphcuda/cuda/{pybind,gcn,spmm_cusparse,gemm_cublas,matmul1..4}.cu) with
the reference's own flags (setup.py:24-36) except the architecture, which its
setup.py pins to sm_75: here ``compute_100 / sm_100`` so that the module loads
on a B200.  The result goes to ``baseline/_ref/`` (kept out of the history; it
travels to the GPU machine like every other built file).  Nothing of this
repository is linked into it, and the package never imports it: only
``bench.py``'s auxiliary "reference_cuda_same_box" block does, to time the
reference's library wrappers (cuSPARSE COO SpMM, cuBLAS SGEMM, GCNConv) beside
this library on the same inputs.

Usage:  python baseline/build_ref_cuda.py
"""
from __future__ import annotations

import glob
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
NAME = "graphcuda_ref_cuda"


def reference_root() -> str:
    """The mounted reference tree: $GRAPHCUDA_REFERENCE_ROOT, else the directory ``reference`` beside this
    repository."""
    default = os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
    return os.environ.get("GRAPHCUDA_REFERENCE_ROOT", default)


def built_path():
    hits = glob.glob(os.path.join(OUT, NAME + "*.so"))
    return hits[0] if hits else None


def build(verbose: bool = False):
    """Returns the path of the built module, or None when the reference tree is not mounted."""
    src_dir = os.path.join(reference_root(), "src", "graphcuda", "cuda")
    if not os.path.isdir(src_dir):
        return built_path()
    have = built_path()
    sources = sorted(glob.glob(os.path.join(src_dir, "*.cu")))
    if have and all(os.path.getmtime(have) >= os.path.getmtime(s) for s in sources):
        return have
    os.makedirs(OUT, exist_ok=True)
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0")  # no GPU is needed (or queried) to compile
    from torch.utils import cpp_extension
    cpp_extension.load(
        name=NAME, sources=sources, build_directory=OUT, verbose=verbose, is_python_module=False,
        extra_cflags=["-O3"],
        extra_cuda_cflags=["-O3", "--use_fast_math", "-gencode=arch=compute_100,code=sm_100"],
        extra_ldflags=["-lcublas", "-lcusparse"])
    return built_path()


def load():
    """The built module (exports gcn_conv_forward/backward, spmm_cusparse, gemm_cublas, matmul1..4 as the
    reference's pybind.cu:7-23 declares them)."""
    import importlib.machinery
    import importlib.util

    import torch  # noqa: F401
    path = built_path()
    if not path:
        raise ImportError("reference CUDA extension not built (python baseline/build_ref_cuda.py)")
    loader = importlib.machinery.ExtensionFileLoader(NAME, path)
    spec = importlib.util.spec_from_file_location(NAME, path, loader=loader)
    mod = importlib.util.module_from_spec(spec)
    loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    p = build(verbose="-v" in sys.argv)
    print(p or "reference tree not mounted and no prebuilt module")

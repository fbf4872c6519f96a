"""Build recipe for the reference's own CPU implementation of the GCN layer.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package may import this.

The reference project carries a device-agnostic ATen restatement of its layer,
``src/graphcuda/cpp/gcn.cpp`` (``gcn_conv_forward`` lines 4-20,
``gcn_conv_backward`` lines 22-41, its own PYBIND11_MODULE lines 43-46).  That
one file compiles for CPU against the installed libtorch without the
reference's build system.  This script compiles it *where it lies* in the
mounted reference tree and writes only the resulting extension module into
``oracle/_ref/`` (git-ignored).  No reference source is copied.

The built module is used
  * to validate the restatement in ``oracle/gcn_oracle.py``,
  * to generate the fixtures under ``tests/golden/``,
  * as the timed CPU baseline (``cpu_baseline.kind == "reference"``).

Where the reference tree is not mounted (the GPU box) the prebuilt module is
loaded as is; see ``oracle/ref_loader.py``.
"""
from __future__ import annotations

import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
NAME = "graphcuda_ref_cpu"


def reference_root() -> str:
    """The mounted reference tree: $GRAPHCUDA_REFERENCE_ROOT, else the directory
    ``reference`` beside this repository."""
    default = os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
    return os.environ.get("GRAPHCUDA_REFERENCE_ROOT", default)


def built_path() -> str:
    return os.path.join(OUT, NAME + ".so")


def build(verbose: bool = False) -> str | None:
    """Compile the reference file; returns the path of the module or None when
    the reference tree is absent and nothing was prebuilt."""
    src = os.path.join(reference_root(), "src", "graphcuda", "cpp", "gcn.cpp")
    if not os.path.exists(src):
        return built_path() if os.path.exists(built_path()) else None
    if os.path.exists(built_path()) and os.path.getmtime(built_path()) >= os.path.getmtime(src):
        return built_path()
    os.makedirs(OUT, exist_ok=True)
    from torch.utils.cpp_extension import load

    build_dir = os.path.join(OUT, "build")
    os.makedirs(build_dir, exist_ok=True)
    load(
        name=NAME,
        sources=[src],
        extra_cflags=["-O3"],
        build_directory=build_dir,
        verbose=verbose,
        is_python_module=True,
    )
    shutil.copyfile(os.path.join(build_dir, NAME + ".so"), built_path())
    return built_path()


if __name__ == "__main__":
    p = build(verbose="-v" in sys.argv)
    print(p if p else "reference tree not mounted and no prebuilt module")

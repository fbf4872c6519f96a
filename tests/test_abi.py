"""The C-ABI library loads and exports every symbol the header declares, the
ctypes table mirrors the header, and argument validation answers without
touching a GPU."""
import ctypes
import os
import re

import pytest

from graphcuda_b200 import _lib, build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "graphcuda_b200.h")


def declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(gc_[a-z0-9_]+)\s*\(", text)))


def test_library_is_built():
    assert os.path.exists(build.lib_path()), "run python -m graphcuda_b200.build"


def test_every_declared_symbol_is_exported():
    handle = ctypes.CDLL(build.lib_path())
    names = declared_symbols()
    assert len(names) >= 20
    for n in names:
        assert hasattr(handle, n), f"{n} declared in the header but not exported"


def test_ctypes_table_matches_header():
    assert sorted(_lib.SIGNATURES) == declared_symbols()


def test_header_cites_the_reference():
    text = open(HEADER).read()
    for needle in ("spmm_cusparse.cu", "gemm_cublas.cu", "matmul1.cu", "gcn.cu", "graphcuda_impl.py"):
        assert needle in text


def test_status_strings_and_version():
    L = _lib.lib()
    assert L.gc_abi_version() >= 3
    assert L.gc_status_string(0) == b"ok"
    assert b"workspace" in L.gc_status_string(-4)


def test_argument_validation_without_gpu():
    L = _lib.lib()
    # negative size
    assert L.gc_gemm_f32(0, 0, -1, 4, 4, None, 4, None, 4, None, 4, None, 0, None, None, 0, None, 0, None) == -1
    assert b"negative" in L.gc_last_error()
    # leading dimension too small
    assert L.gc_gemm_f32(0, 0, 8, 8, 8, 16, 4, 16, 8, 16, 8, None, 0, None, None, 0, None, 0, None) == -1
    # unknown epilogue bit
    assert L.gc_spmm_csr_f32(16, 16, 16, 4, 4, 4, 16, 4, None, 64, 16, 4, None, None, None, 0, 0, 0, None, 0, None) == -1
    # empty problems succeed without launching anything
    assert L.gc_gemm_f32(0, 0, 0, 4, 4, None, 4, None, 4, None, 4, None, 0, None, None, 0, None, 0, None) == 0
    assert L.gc_spmm_csr_f32(None, None, None, 0, 0, 8, None, 8, None, 0, None, 8, None, None, None, 0, 0, 0, None, 0, None) == 0
    # a plan that cuts rows needs gc_spmm_scratch_bytes(n_slots, F) of scratch: less is refused before any launch
    assert L.gc_spmm_csr_f32(16, 16, 16, 4, 4, 8, 16, 8, None, 0, 16, 8, None, None, 16, 6, 3, 1, 16, 64, None) == -4
    assert b"partial-sum rows" in L.gc_last_error()
    # counts that cannot belong to one plan (a cut row has at least two pieces)
    assert L.gc_spmm_csr_f32(16, 16, 16, 4, 4, 8, 16, 8, None, 0, 16, 8, None, None, 16, 6, 1, 1, 16, 4096, None) == -1
    assert L.gc_gather_sum_f32(16, 6, 4, 6, 16, 4, 4, 16, 8, 0, None) == -1  # rows must be multiples of four floats
    assert L.gc_gather_sum_f32(None, 8, 4, 8, None, 0, 4, None, 8, 0, None) == 0
    # evaluation tail and optimizer step: bad arguments are refused before any launch
    assert L.gc_argmax_accuracy_f32(16, 2, 4, 3, None, None, 0, None, None, None) == -1  # ld < C
    assert L.gc_argmax_accuracy_f32(16, 4, 4, 3, None, 16, 9, None, None, None) == -1  # more than 8 selections
    assert L.gc_argmax_accuracy_f32(None, 4, 0, 3, None, None, 0, None, None, None) == 0  # no rows
    assert L.gc_adam_step_f32(33, 16, 16, 16, 16, 16, 0.01, 0.9, 0.999, 1e-8, 0.0, 16, None) == -1
    assert b"tensors" in L.gc_last_error()
    assert L.gc_adam_step_f32(1, 16, 16, 16, 16, 16, 0.01, 0.9, 0.999, 1e-8, 0.0, None, None) == -1  # null state
    assert L.gc_sgd_step_f32(0, None, None, None, 0.1, 0.0, None) == 0
    with pytest.raises(RuntimeError):
        _lib.check(-1, "probe")


def test_plan_and_workspace_sizes():
    L = _lib.lib()
    assert L.gc_spmm_plan_bytes(0, 0) >= 32
    assert L.gc_spmm_plan_bytes(1000, 10) >= 32 + 3 * 4 * 1000 + 3 * 4 * 10
    assert L.gc_spmm_plan_workspace_bytes(1000, 0) >= 6 * 4 * 1000
    assert L.gc_spmm_plan_workspace_bytes(1000, 5000) >= 6 * 4 * 1000 + 36 * 5000
    assert L.gc_spmm_scratch_bytes(10_000, 256) == 10_000 * 256 * 4
    assert L.gc_spmm_scratch_bytes(10, 47) == 10 * 48 * 4  # rows padded to 16 bytes
    # panel width: a power of two whose rows of H take about 128 MiB, at most 262144 and never more than K
    assert L.gc_spmm_default_panel_cols(2_449_029, 256) == 131072
    assert L.gc_spmm_default_panel_cols(2_449_029, 48) == 262144
    assert L.gc_spmm_default_panel_cols(2708, 16) == 2708
    # segment length: a power of two near nnz / 8192 within [128, 2048]
    assert L.gc_spmm_default_segment(13_566) == 128
    assert L.gc_spmm_default_segment(2_501_829) == 512
    assert L.gc_spmm_default_segment(126_167_309) == 2048
    assert L.gc_gemm_workspace_bytes(0, 0, 4096, 256, 256, _lib.PREC_TF32X3) >= 256 + 2 * 256 * 256 * 4


def test_precision_resolution_is_host_logic():
    L = _lib.lib()
    P = _lib
    # small problem -> CUDA cores; large aligned problem -> split-TF32 tensor cores
    assert L.gc_gemm_resolve_precision(0, 0, 2708, 16, 1433, 1433, 16, 16, P.PREC_AUTO) == P.PREC_FP32_SIMT
    assert L.gc_gemm_resolve_precision(0, 0, 169343, 256, 128, 128, 256, 256, P.PREC_AUTO) == P.PREC_TF32X3
    # unaligned row pitch of an operand read in place -> CUDA cores under AUTO, error when forced
    assert L.gc_gemm_resolve_precision(0, 0, 169343, 256, 127, 127, 256, 256, P.PREC_AUTO) == P.PREC_FP32_SIMT
    assert L.gc_gemm_resolve_precision(0, 0, 169343, 256, 127, 127, 256, 256, P.PREC_TF32) == -2
    # weight-gradient shape (few tiles, huge K): tensor cores with split-K, operands read in place
    assert L.gc_gemm_resolve_precision(1, 0, 256, 256, 2449029, 256, 256, 256, P.PREC_AUTO) == P.PREC_TF32X3
    assert L.gc_gemm_resolve_precision(1, 0, 256, 47, 2449029, 256, 47, 47, P.PREC_AUTO) == P.PREC_FP32_SIMT
    assert L.gc_gemm_resolve_precision(0, 0, 8192, 8192, 8192, 8192, 8192, 8192, P.PREC_FP32_SIMT) == P.PREC_FP32_SIMT


def test_header_is_plain_c_and_links_from_a_c_program(tmp_path):
    """The boundary is a C ABI: the header must compile as C99 and a C program must link and call it."""
    import shutil
    import subprocess
    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("no C compiler")
    src = tmp_path / "probe.c"
    src.write_text(
        '#include "graphcuda_b200.h"\n#include <stdio.h>\n'
        "int main(void) {\n"
        "  /* argument errors are reported without touching a device */\n"
        "  int rc = gc_gemm_f32(0, 0, -1, 4, 4, 0, 4, 0, 4, 0, 4, 0, 0, 0, 0, GC_PREC_AUTO, 0, 0, 0);\n"
        '  printf("%d %d %s\\n", gc_abi_version(), rc, gc_status_string(rc));\n'
        "  return rc == GC_ERR_INVALID ? 0 : 1;\n}\n")
    exe = tmp_path / "probe"
    libdir = os.path.dirname(build.lib_path())
    r = subprocess.run([gcc, "-std=c99", "-Wall", "-Werror", "-I", os.path.dirname(HEADER), str(src), "-o", str(exe),
                        "-L", libdir, "-lgraphcuda_b200", f"-Wl,-rpath,{libdir}"], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    run = subprocess.run([str(exe)], capture_output=True, text=True)
    assert run.returncode == 0, run.stdout + run.stderr
    assert run.stdout.split()[0] == str(_lib.lib().gc_abi_version())

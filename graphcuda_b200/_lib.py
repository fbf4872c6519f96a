"""ctypes binding of the C-ABI library (``include/graphcuda_b200.h``).

The library is the product: there is no PyTorch or CPU fallback behind these
calls.  If ``lib/libgraphcuda_b200.so`` is missing, importing the operators
raises with the build command instead of degrading silently.
"""
from __future__ import annotations

import ctypes as C
import os

from . import build as _build

_i32p = C.c_void_p
_i64p = C.c_void_p
_f32p = C.c_void_p
_void = C.c_void_p
_i64 = C.c_int64
_int = C.c_int
_size = C.c_size_t

# name -> (restype, argtypes); mirrors include/graphcuda_b200.h one to one
SIGNATURES = {
    "gc_abi_version": (_int, []),
    "gc_launch_count": (C.c_longlong, []),
    "gc_last_error": (C.c_char_p, []),
    "gc_status_string": (C.c_char_p, [_int]),
    "gc_spmm_default_panel_cols": (_i64, [_i64, _i64]),
    "gc_spmm_plan_workspace_bytes": (_size, [_i64, _i64]),
    "gc_spmm_default_segment": (_i64, [_i64]),
    "gc_spmm_plan_count": (_int, [_i32p, _i32p, _i64, _i64, _i64, _i64, _i64p, _void, _size, _void]),
    "gc_spmm_plan_bytes": (_size, [_i64, _i64]),
    "gc_spmm_plan_build": (_int, [_i32p, _i32p, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _void, _size, _void, _size,
                                  _void]),
    "gc_spmm_scratch_bytes": (_size, [_i64, _i64]),
    "gc_spmm_plan_check": (_int, [_void, _i64, _i64, _i64, _void]),
    "gc_spmm_csr_f32": (_int, [_i32p, _i32p, _f32p, _i64, _i64, _i64, _f32p, _i64, _f32p, _int, _f32p, _i64,
                               _f32p, _f32p, _void, _i64, _i64, _i64, _void, _size, _void]),
    "gc_spmm_csr_bf16h_f32": (_int, [_i32p, _i32p, _f32p, _i64, _i64, _i64, _void, _i64, _f32p, _int, _f32p, _i64,
                                     _f32p, _f32p, _void, _i64, _i64, _i64, _void, _size, _void]),
    "gc_spmm_csr_f32_blocks": (_int, [_i32p, _i32p, _f32p, _i64, _i64, _i64, _f32p, _i64, _f32p, _int, _void, _int,
                                      _i64, _i64, _void, _i64, _i64, _i64, _void, _size, _void]),
    "gc_scatter_column_slabs_f32": (_int, [_f32p, _i64, _i64, _i64, _i64, _void, _int, _i64, _void]),
    "gc_gather_sum_f32": (_int, [_f32p, _i64, _i64, _i64, _i32p, _i64, _i64, _f32p, _i64, _int, _void]),
    "gc_spmm_csr_f32_noalloc": (_int, [_i32p, _i32p, _f32p, _i64, _i64, _i64, _f32p, _i64, _f32p, _int, _f32p,
                                       _i64, _f32p, _f32p, _void, _i64, _i64, _i64, _void]),
    "gc_gemm_workspace_bytes": (_size, [_int, _int, _i64, _i64, _i64, _int]),
    "gc_gemm_f32": (_int, [_int, _int, _i64, _i64, _i64, _f32p, _i64, _f32p, _i64, _f32p, _i64, _f32p, _int,
                           _f32p, _f32p, _int, _void, _size, _void]),
    "gc_convert_f32_bf16": (_int, [_f32p, _i64, _i64, _i64, _void, _i64, _int, _void]),
    "gc_gemm_bf16_workspace_bytes": (_size, [_i64, _i64, _i64]),
    "gc_gemm_bf16_f32": (_int, [_i64, _i64, _i64, _void, _i64, _void, _i64, _f32p, _i64, _f32p, _int, _f32p, _f32p,
                                _void, _size, _void]),
    "gc_gemm_resolve_precision": (_int, [_int, _int, _i64, _i64, _i64, _i64, _i64, _i64, _int]),
    "gc_gemm_check_flag": (_int, [_void, _void]),
    "gc_gcn_layer_workspace_bytes": (_size, [_i64, _i64, _i64, _i64, _int, _int]),
    "gc_gcn_conv_forward_csr_f32": (_int, [_i32p, _i32p, _f32p, _i64, _i64, _i64, _f32p, _i64, _f32p, _i64, _f32p,
                                           _int, _f32p, _i64, _f32p, _f32p, _i64, _void, _i64, _i64, _i64, _int,
                                           _void, _size, _void]),
    "gc_gcn_conv_backward_csr_f32": (_int, [_i32p, _i32p, _f32p, _i64, _i64, _i64, _f32p, _i64, _f32p, _i64, _f32p,
                                            _i64, _int, _f32p, _i64, _f32p, _i64, _f32p, _i64, _f32p, _i64, _void,
                                            _i64, _i64, _i64, _int, _void, _size, _void]),
    "gc_relu_backward_f32": (_int, [_f32p, _i64, _f32p, _i64, _f32p, _i64, _i64, _i64, _void]),
    "gc_mask_mul_f32": (_int, [_f32p, _i64, _f32p, _i64, _f32p, _i64, _i64, _i64, _void]),
    "gc_transpose_f32": (_int, [_f32p, _i64, _f32p, _i64, _i64, _i64, _void]),
    "gc_nll_workspace_bytes": (_size, [_i64]),
    "gc_logsoftmax_nll_forward_f32": (_int, [_f32p, _i64, _i64p, _void, _i64, _i64, C.c_float, _f32p, _void, _size,
                                             _void]),
    "gc_logsoftmax_nll_backward_f32": (_int, [_f32p, _i64, _i64p, _void, _i64, _i64, C.c_float, _f32p, _f32p, _i64,
                                              _void, _void]),
    "gc_argmax_accuracy_f32": (_int, [_f32p, _i64, _i64, _i64, _i64p, _void, _int, _i64p, _i64p, _void]),
    "gc_adam_step_f32": (_int, [_int, _void, _void, _void, _void, _void, C.c_double, C.c_double, C.c_double,
                                C.c_double, C.c_double, _void, _void]),
    "gc_sgd_step_f32": (_int, [_int, _void, _void, _void, C.c_double, C.c_double, _void]),
    "gc_coo_rows_to_rowptr": (_int, [_i64p, _i64, _i64, _i32p, _void]),
    "gc_narrow_i64_i32": (_int, [_i64p, _i32p, _i64, _void]),
    "gc_gcn_norm_f32": (_int, [_i64p, _i64p, _i64, _i64, _f32p, _f32p, _void]),
    "gc_csr_build_workspace_bytes": (_size, [_i64]),
    "gc_csr_count_unique": (_int, [_i64p, _i64p, _i64, _i32p, _i64p, _void, _size, _void]),
    "gc_csr_fill": (_int, [_i64p, _i64p, _f32p, _i64, _i64, _i32p, _i32p, _i32p, _f32p, _void]),
    "gc_csr_is_symmetric": (_int, [_i32p, _i32p, _f32p, _i64, _i32p, _void]),
}

# epilogue / precision constants of the header
SPMM_STATIC_SCRATCH_BYTES = 8 << 20
SPMM_MAX_BLOCKS = 16
EPI_RELU = 1
EPI_ACCUMULATE = 2
EPI_TRANSPOSED_OUT = 4
LAYER_RELU = 1
LAYER_TRANSFORM_FIRST = 2
PREC_AUTO = -1
PREC_FP32_SIMT = 0
PREC_TF32X3 = 1
PREC_TF32 = 2
PREC_BF16 = 3

_lib = None


class LibraryMissing(ImportError):
    pass


def lib() -> C.CDLL:
    """The loaded C-ABI library.  Raises LibraryMissing when it was not built."""
    global _lib
    if _lib is not None:
        return _lib
    path = os.environ.get("GRAPHCUDA_B200_LIB", _build.lib_path())
    if not os.path.exists(path):
        raise LibraryMissing(
            f"{path} not found: the CUDA library has not been built. "
            "Run `python -m graphcuda_b200.build` (needs nvcc). There is no CPU or PyTorch fallback."
        )
    handle = C.CDLL(path)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(handle, name)  # AttributeError here means header and library disagree
        fn.restype = res
        fn.argtypes = args
    _lib = handle
    return handle


def check(status: int, what: str) -> None:
    """Maps a non-zero status to RuntimeError (what TORCH_CHECK raises in the
    reference: src/graphcuda/cuda/gemm_cublas.cu:4-7)."""
    if status != 0:
        l = lib()
        msg = l.gc_last_error().decode() or l.gc_status_string(status).decode()
        raise RuntimeError(f"{what}: {msg} (status {status})")

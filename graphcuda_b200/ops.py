"""Tensor-level wrappers over the C ABI: shape checks, output allocation from
torch's caching allocator, the current stream, the device guard.

This is the layer the reference implements in C++ with ``torch::Tensor``
arguments (src/graphcuda/cuda/gemm_cublas.cu:3-31, spmm_cusparse.cu:3-31,
matmul1.cu:27-43): it owns allocation and error mapping; the C ABI below it
sees raw pointers only.  CPU tensors are rejected like the reference does
(``is_cuda`` checks) -- there is no CPU path.
"""
from __future__ import annotations

import threading
from typing import Optional

import torch

from . import _lib
from ._lib import (EPI_ACCUMULATE, EPI_RELU, EPI_TRANSPOSED_OUT, PREC_AUTO, PREC_BF16, PREC_FP32_SIMT, PREC_TF32,
                   PREC_TF32X3)

PRECISIONS = {
    "fp32": PREC_AUTO,          # fp32 semantics; tensor cores in split-TF32 mode when the shape qualifies
    "fp32_simt": PREC_FP32_SIMT,  # IEEE fp32 FMA on CUDA cores, bit-stable
    "tf32x3": PREC_TF32X3,
    "tf32": PREC_TF32,          # opt-in, 1e-2 tolerance tier
    "bf16": PREC_BF16,          # opt-in, 1e-2 tolerance tier: bf16 operands, fp32 accumulation
}

_default_precision = "fp32"


def set_default_precision(name: str) -> None:
    if name not in PRECISIONS:
        raise ValueError(f"precision must be one of {sorted(PRECISIONS)}")
    global _default_precision
    _default_precision = name


def get_default_precision() -> str:
    return _default_precision


def _prec(precision: Optional[str]) -> int:
    name = precision or _default_precision
    try:
        return PRECISIONS[name]
    except KeyError:
        raise ValueError(f"precision must be one of {sorted(PRECISIONS)}, got {name!r}") from None


# ---------------------------------------------------------------- workspaces
class _Arena:
    """Grow-only scratch buffers, one set per (device, stream, tag).  Kernels
    enqueued on one stream run in order, so a buffer is never in use by two
    launches at once.  New buffers are zero-filled (the tensor-core GEMM keeps
    a sticky error word at the start of its workspace)."""

    def __init__(self):
        self._bufs = {}
        self._lock = threading.Lock()

    def get(self, tag: str, nbytes: int, device: torch.device) -> torch.Tensor:
        stream = torch.cuda.current_stream(device).cuda_stream
        key = (device.index, stream, tag)
        with self._lock:
            buf = self._bufs.get(key)
            if buf is None or buf.numel() < nbytes:
                # round up so growth is rare
                size = max(256, int(nbytes * 1.25) + 255 & ~255)
                new = torch.zeros(size, dtype=torch.uint8, device=device)
                if buf is not None:
                    # the first 256 bytes carry sticky state (the GEMM's error word): it moves with the buffer,
                    # in stream order, so a flag raised before the growth is still there to be read afterwards
                    new[:256].copy_(buf[:256])
                buf = new
                self._bufs[key] = buf
            return buf

    def clear(self):
        with self._lock:
            self._bufs.clear()


arena = _Arena()


def _stream(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _require(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError(msg)


def _row_major(t: torch.Tensor) -> torch.Tensor:
    """A view usable with a leading dimension: unit stride along columns."""
    if t.stride(1) == 1 and t.stride(0) >= max(1, t.size(1)):
        return t
    if t.size(1) == 1 and t.stride(0) >= 1:
        return t
    return t.contiguous()


def _ld(t: torch.Tensor) -> int:
    return t.stride(0) if t.size(0) > 1 else max(t.size(1), t.stride(0), 1)


def _as_operand(t: torch.Tensor):
    """(storage tensor, trans flag, ld): a transposed view of a row-major matrix
    is passed as such instead of being copied (the reference copies:
    gemm_cublas.cu:11-16)."""
    if t.stride(1) == 1 and (t.size(0) <= 1 or t.stride(0) >= t.size(1)):
        return t, 0, _ld(t)
    if t.stride(0) == 1 and (t.size(1) <= 1 or t.stride(1) >= t.size(0)):
        tt = t.t()
        return tt, 1, _ld(tt)
    c = t.contiguous()
    return c, 0, _ld(c)


# ---------------------------------------------------------------- GEMM
def gemm(A: torch.Tensor, B: torch.Tensor, *, bias: Optional[torch.Tensor] = None, relu: bool = False,
         want_mask: bool = False, precision: Optional[str] = None, transposed_out: bool = False,
         out: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None):
    """C = A @ B (+bias)(ReLU) in fp32.  A and B may be transposed views.
    Returns C, or (C, mask) when want_mask.  With transposed_out the result
    tensor holds C^T (shape N x M).  gate (contiguous, shape of the result):
    the result is multiplied by (gate > 0) in the store."""
    _require(A.dim() == 2 and B.dim() == 2, "Inputs must be 2D")
    _require(A.size(1) == B.size(0), "A.cols must match B.rows")
    _require(A.is_cuda and B.is_cuda, "Inputs must be CUDA tensors")
    _require(A.dtype == torch.float32 and B.dtype == torch.float32, "Only float32 is supported here")
    _require(A.device == B.device, "Inputs must be on the same device")
    M, K = A.shape
    N = B.size(1)
    dev = A.device
    with torch.cuda.device(dev):
        a, ta, lda = _as_operand(A)
        b, tb, ldb = _as_operand(B)
        shape = (N, M) if transposed_out else (M, N)
        if out is None:
            out = torch.empty(shape, dtype=torch.float32, device=dev)
        else:
            _require(tuple(out.shape) == shape and out.dtype == torch.float32 and out.is_contiguous(),
                     "out has the wrong shape, dtype or layout")
        mask = torch.empty(shape, dtype=torch.float32, device=dev) if want_mask else None
        if bias is not None:
            _require(bias.is_cuda and bias.dtype == torch.float32 and bias.numel() == N, "bias must be float32 [N]")
            bias = bias.contiguous()
        if gate is not None:
            _require(gate.is_cuda and gate.dtype == torch.float32 and tuple(gate.shape) == shape
                     and gate.is_contiguous() and out.is_contiguous(), "gate must be a contiguous float32 tensor "
                     "of the result's shape")
        if M and N:
            L = _lib.lib()
            prec = _prec(precision)
            ws_bytes = L.gc_gemm_workspace_bytes(ta, tb, M, N, K, prec)
            ws = arena.get("gemm", ws_bytes, dev)
            epi = (EPI_RELU if relu else 0) | (EPI_TRANSPOSED_OUT if transposed_out else 0)
            st = L.gc_gemm_f32(ta, tb, M, N, K, a.data_ptr(), lda, b.data_ptr(), ldb, out.data_ptr(),
                               max(out.stride(0), 1) if out.size(0) > 1 else max(out.size(1), 1),
                               bias.data_ptr() if bias is not None else None, epi,
                               mask.data_ptr() if mask is not None else None,
                               gate.data_ptr() if gate is not None else None, prec, ws.data_ptr(), ws.numel(),
                               _stream(dev))
            _lib.check(st, "gc_gemm_f32")
    return (out, mask) if want_mask else out


def to_bf16(X: torch.Tensor, *, transpose: bool = False) -> torch.Tensor:
    """bf16 copy of a float32 matrix for the bf16 tier (round to nearest even), laid out for the tensor cores:
    rows x cols with the row pitch rounded up to 8 elements and the pad zero-filled; ``transpose=True`` gives the
    copy of X^T.  The result is a view [rows, cols] of the padded buffer."""
    _require(X.dim() == 2 and X.is_cuda and X.dtype == torch.float32, "to_bf16: float32 CUDA matrix expected")
    X = _row_major(X)
    rows, cols = (X.size(1), X.size(0)) if transpose else (X.size(0), X.size(1))
    ld = (cols + 7) // 8 * 8
    out = torch.empty((rows, ld), dtype=torch.bfloat16, device=X.device)
    with torch.cuda.device(X.device):
        st = _lib.lib().gc_convert_f32_bf16(X.data_ptr(), _ld(X), rows, cols, out.data_ptr(), ld, 1 if transpose else 0,
                                            _stream(X.device))
    _lib.check(st, "gc_convert_f32_bf16")
    return out[:, :cols]


def gemm_bf16_operands(A16: torch.Tensor, Bt16: torch.Tensor, *, bias: Optional[torch.Tensor] = None,
                       relu: bool = False, out: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None):
    """C (float32) = A16 @ Bt16^T for operands already in bf16 (as to_bf16 lays them out: K contiguous, pitch a
    multiple of 8).  What gemm(precision="bf16") runs after converting its operands; calling it directly lets a
    constant operand (a dense adjacency, a weight) be converted once."""
    _require(A16.dtype == torch.bfloat16 and Bt16.dtype == torch.bfloat16 and A16.is_cuda and Bt16.is_cuda,
             "bf16 CUDA operands expected")
    _require(A16.size(1) == Bt16.size(1), "A16 and Bt16 must share K")
    _require(A16.stride(1) == 1 and Bt16.stride(1) == 1, "operands must have unit stride along K")
    M, K = A16.shape
    N = Bt16.size(0)
    dev = A16.device
    with torch.cuda.device(dev):
        if out is None:
            out = torch.empty((M, N), dtype=torch.float32, device=dev)
        else:
            _require(tuple(out.shape) == (M, N) and out.dtype == torch.float32 and out.is_contiguous(),
                     "out has the wrong shape, dtype or layout")
        if bias is not None:
            _require(bias.is_cuda and bias.dtype == torch.float32 and bias.numel() == N, "bias must be float32 [N]")
            bias = bias.contiguous()
        if gate is not None:
            _require(gate.is_cuda and gate.dtype == torch.float32 and tuple(gate.shape) == (M, N)
                     and gate.is_contiguous(), "gate must be a contiguous float32 tensor of the result's shape")
        if M and N:
            L = _lib.lib()
            ws = arena.get("gemm", L.gc_gemm_bf16_workspace_bytes(M, N, K), dev)
            st = L.gc_gemm_bf16_f32(M, N, K, A16.data_ptr(), A16.stride(0) if M > 1 else (K + 7) // 8 * 8,
                                    Bt16.data_ptr(), Bt16.stride(0) if N > 1 else (K + 7) // 8 * 8, out.data_ptr(), N,
                                    bias.data_ptr() if bias is not None else None, EPI_RELU if relu else 0, None,
                                    gate.data_ptr() if gate is not None else None, ws.data_ptr(), ws.numel(),
                                    _stream(dev))
            _lib.check(st, "gc_gemm_bf16_f32")
    return out


def gemm_path(A: torch.Tensor, B: torch.Tensor, precision: Optional[str] = None) -> str:
    """Which back end gemm(A, B) takes: 'fp32_simt', 'tf32x3' or 'tf32'."""
    a, ta, lda = _as_operand(A)
    b, tb, ldb = _as_operand(B)
    M, K = A.shape
    N = B.size(1)
    r = _lib.lib().gc_gemm_resolve_precision(ta, tb, M, N, K, lda, ldb, N, _prec(precision))
    _lib.check(min(r, 0), "gc_gemm_resolve_precision")
    return {PREC_FP32_SIMT: "fp32_simt", PREC_TF32X3: "tf32x3", PREC_TF32: "tf32", PREC_BF16: "bf16"}[r]


def check_gemm_flag(device: torch.device) -> None:
    """Raises if a tensor-core GEMM on this device/stream gave up a bounded wait."""
    ws = arena.get("gemm", 256, device)
    _lib.check(_lib.lib().gc_gemm_check_flag(ws.data_ptr(), _stream(device)), "gc_gemm_check_flag")


# ---------------------------------------------------------------- element-wise
def relu_backward(dY: torch.Tensor, Y: torch.Tensor) -> torch.Tensor:
    """dY * (Y > 0)."""
    _require(dY.shape == Y.shape and dY.is_cuda and Y.is_cuda, "relu_backward: shape/device mismatch")
    dY = _row_major(dY)
    Y = _row_major(Y)
    M, N = dY.shape
    G = torch.empty((M, N), dtype=torch.float32, device=dY.device)
    with torch.cuda.device(dY.device):
        st = _lib.lib().gc_relu_backward_f32(dY.data_ptr(), _ld(dY), Y.data_ptr(), _ld(Y), G.data_ptr(), max(N, 1),
                                             M, N, _stream(dY.device))
    _lib.check(st, "gc_relu_backward_f32")
    return G


def mask_mul(dY: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    """dY * mask for a stored fp32 mask (reference gcn.cu:36)."""
    _require(dY.shape == mask.shape and dY.is_cuda and mask.is_cuda, "mask_mul: shape/device mismatch")
    dY = _row_major(dY)
    mask = _row_major(mask)
    M, N = dY.shape
    G = torch.empty((M, N), dtype=torch.float32, device=dY.device)
    with torch.cuda.device(dY.device):
        st = _lib.lib().gc_mask_mul_f32(dY.data_ptr(), _ld(dY), mask.data_ptr(), _ld(mask), G.data_ptr(), max(N, 1),
                                        M, N, _stream(dY.device))
    _lib.check(st, "gc_mask_mul_f32")
    return G


def scatter_column_slabs(src: torch.Tensor, dsts, w: int) -> None:
    """dsts[q][r, c] = src[r, q * w + c]: the column slabs of a row-major float32 matrix, each written to its own
    destination (float32 views of at least src.size(0) rows with one common row stride; other GPUs' peer-mapped
    buffers are fine).  One kernel; every element of src is read once."""
    import ctypes
    _require(src.dim() == 2 and src.is_cuda and src.dtype == torch.float32, "float32 CUDA matrix expected")
    src = _row_major(src)
    rows, F = src.shape
    _require(1 <= len(dsts) <= _lib.SPMM_MAX_BLOCKS and len(dsts) * w >= F, "slabs must cover the columns")
    ld = dsts[0].stride(0)
    for q, d in enumerate(dsts):
        need = min(w, F - q * w)
        _require(d.dtype == torch.float32 and d.dim() == 2 and d.stride(1) == 1 and d.stride(0) == ld
                 and d.size(0) >= rows and (need <= 0 or d.size(1) >= need), "bad slab destination")
    if rows == 0 or F == 0:
        return
    ptrs = (ctypes.c_void_p * len(dsts))(*[d.data_ptr() for d in dsts])
    with torch.cuda.device(src.device):
        st = _lib.lib().gc_scatter_column_slabs_f32(src.data_ptr(), _ld(src), rows, F, w, ptrs, len(dsts), ld,
                                                    _stream(src.device))
    _lib.check(st, "gc_scatter_column_slabs_f32")


def transpose(X: torch.Tensor) -> torch.Tensor:
    _require(X.dim() == 2 and X.is_cuda and X.dtype == torch.float32, "transpose: float32 CUDA matrix expected")
    X = _row_major(X)
    M, N = X.shape
    out = torch.empty((N, M), dtype=torch.float32, device=X.device)
    with torch.cuda.device(X.device):
        st = _lib.lib().gc_transpose_f32(X.data_ptr(), _ld(X), out.data_ptr(), max(M, 1), M, N, _stream(X.device))
    _lib.check(st, "gc_transpose_f32")
    return out

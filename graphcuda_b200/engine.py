"""Layer-level composition of the kernels: one GCN layer forward and backward.

Reference math (src/graphcuda/cuda/gcn.cu:5-52, twin src/graphcuda/cpp/gcn.cpp:4-41):
    forward   Y  = relu((A X) W)
    backward  G  = dY * mask;  dW = (A X)^T G;  dX = A (G W^T)
The reference always aggregates first and recomputes A X in the backward pass.
Here the aggregation runs on the narrower side -- (A X) W when in <= out,
A (X W) when out < in and A is symmetric -- the intermediate is kept for the
backward pass, ReLU/bias/mask are fused into the producing kernel, transposed
operands are read in place, and dX is skipped when nobody needs it.  For a
non-symmetric A the aggregate-first order is always used, so the results are
the reference's (including its use of A rather than A^T for dX, gcn.cu:49).
"""
from __future__ import annotations

import weakref
from typing import Optional

import torch

from . import ops
from .ops import _require


def _check_layer_args(X, adj, W):
    _require(X.dim() == 2 and W.dim() == 2, "Inputs must be 2D")
    _require(X.is_cuda and W.is_cuda, "Inputs must be CUDA tensors")
    _require(X.dtype == torch.float32 and W.dtype == torch.float32, "Only float32 is supported here")
    _require(adj.shape[1] == X.size(0), "A.cols must match B.rows")
    _require(X.size(1) == W.size(0), "A.cols must match B.rows")


def choose_order(in_dim: int, out_dim: int, symmetric: bool) -> str:
    return "transform_first" if (out_dim < in_dim and symmetric) else "aggregate_first"


# Transform-first layers with an output width that is not a multiple of 4
# (47 classes) run on a zero-padded width so every row pitch is 16-byte aligned
# (vector gathers in the aggregation, TMA in the tensor-core GEMMs).  Small
# problems are not worth the copies.
_PAD_MIN_WORK = 1 << 27


def _padded_width(n_rows: int, in_dim: int, out_dim: int) -> int:
    if out_dim % 4 == 0 or n_rows * in_dim * out_dim < _PAD_MIN_WORK:
        return out_dim
    return (out_dim + 3) // 4 * 4


# Buffers this library produced with zero-filled pad columns, by the address of their first element: the loss
# backward writes the gradient of a padded logits matrix straight into such a buffer and hands out the unpadded
# view; the layer below recognises the view here and uses the buffer instead of zero-filling and copying a new one.
_zero_padded = weakref.WeakValueDictionary()


def register_zero_padded(buf: torch.Tensor) -> None:
    _zero_padded[buf.data_ptr()] = buf


def _pad_cols(t: torch.Tensor, width: int) -> torch.Tensor:
    if t.size(-1) == width:
        return t
    if t.dim() == 2 and t.stride(1) == 1 and t.stride(0) == width:
        base = _zero_padded.get(t.data_ptr())
        if base is not None and tuple(base.shape) == (t.size(0), width) and base.is_contiguous():
            return base
    out = t.new_zeros(t.shape[:-1] + (width,))
    out[..., :t.size(-1)] = t
    return out


def _adj_matmul(adj, H, precision, **kw):
    from .adjacency import DenseAdjacency
    if isinstance(adj, DenseAdjacency):
        return adj.matmul(H, precision=precision, **kw)
    if ((precision or ops.get_default_precision()) == "bf16" and H.size(1) >= 128 and H.size(1) % 8 == 0
            and adj.nnz >= 16 * H.size(0)):
        # bf16 tier, wide H on a graph with enough non-zeros per row: the aggregation gathers a bf16 copy (half the
        # bytes through the SM fill path, fp32 sums).  126 M non-zeros, F = 256: 6.9 ms + 0.6 ms for the copy against
        # 8.8 ms; narrower or sparser products do not repay the conversion pass.
        return adj.matmul(ops.to_bf16(H), **kw)
    return adj.matmul(H, **kw)


def layer_forward(X, adj, W, bias: Optional[torch.Tensor], relu: bool, *, want_mask: bool = False,
                  precision: Optional[str] = None, order: Optional[str] = None):
    """Returns (Y, mask or None, saved) where saved = (order, intermediate):
    the intermediate is A X (aggregate_first) or None (transform_first)."""
    _check_layer_args(X, adj, W)
    if order is None:
        order = choose_order(W.size(0), W.size(1), adj.symmetric if W.size(1) < W.size(0) else False)
    if order == "aggregate_first":
        AX = _adj_matmul(adj, X, precision)
        r = ops.gemm(AX, W, bias=bias, relu=relu, want_mask=want_mask, precision=precision)
        Y, mask = r if want_mask else (r, None)
        return Y, mask, (order, AX)
    out_dim = W.size(1)
    width = _padded_width(X.size(0), W.size(0), out_dim)
    Wp = _pad_cols(W, width)
    bp = _pad_cols(bias, width) if bias is not None else None
    H = ops.gemm(X, Wp, precision=precision)
    r = _adj_matmul(adj, H, precision, bias=bp, relu=relu, want_mask=want_mask)
    Y, mask = r if want_mask else (r, None)
    if width != out_dim:  # views on the padded buffers; the pad columns hold zeros
        Y = Y[:, :out_dim]
        mask = mask[:, :out_dim] if mask is not None else None
    return Y, mask, (order, None)


def layer_backward(dY, X, adj, W, relu: bool, Y, saved, *, need_dX: bool = True, need_dW: bool = True,
                   need_db: bool = False, precision: Optional[str] = None, grad_is_gated: bool = False,
                   gate_dx_by_input: bool = False):
    """Gradients (dX, dW, db) of layer_forward; Y is the saved activation (the
    ReLU mask is re-derived from it as Y > 0).

    Cross-layer fusion of the ReLU backward (reference gcn.cu:36): when this
    layer's input X is itself the ReLU output of the layer below
    (gate_dx_by_input), dX is multiplied by (X > 0) in the store of the kernel
    that produces it -- which is exactly the masking the layer below would do
    on its incoming gradient; that layer is then told its gradient arrives
    gated (grad_is_gated) and skips the separate pass."""
    order, AX = saved
    G = ops.relu_backward(dY, Y) if (relu and not grad_is_gated) else dY
    gate = X if (gate_dx_by_input and need_dX and X.is_contiguous()) else None
    if G.stride(1) != 1:
        G = G.contiguous()
    dX = dW = db = None
    if need_db:
        db = G.sum(0)
    out_dim = W.size(1)
    width = _padded_width(X.size(0), W.size(0), out_dim) if order == "transform_first" else out_dim
    if width != out_dim:
        Gp = _pad_cols(G, width)
        Wp = _pad_cols(W, width)
        S = _adj_matmul(adj, Gp, precision)
        if need_dW:
            dW = ops.gemm(X.t(), S, precision=precision)[:, :out_dim]
        if need_dX:
            dX = ops.gemm(S, Wp.t(), precision=precision, gate=gate)
        return dX, dW, db
    if order == "aggregate_first":
        if need_dW:
            dW = ops.gemm(AX.t(), G, precision=precision)
        if need_dX:
            T = ops.gemm(G, W.t(), precision=precision)
            dX = _adj_matmul(adj, T, precision, gate=gate)  # A, not A^T: reference gcn.cu:49
    else:
        # Y = A (X W), A symmetric: S = A^T G = A G
        S = _adj_matmul(adj, G, precision)
        if need_dW:
            dW = ops.gemm(X.t(), S, precision=precision)
        if need_dX:
            dX = ops.gemm(S, W.t(), precision=precision, gate=gate)
    if gate_dx_by_input and need_dX and gate is None:  # non-contiguous input: separate pass
        dX = ops.relu_backward(dX, X)
    return dX, dW, db


def layer_backward_reference_form(dY, X, adj, W, relu: bool, mask, *, precision: Optional[str] = None):
    """(dX, dW) from exactly what the reference's backward entry point receives
    (no saved intermediate): src/graphcuda/cuda/gcn.cu:27-52."""
    _check_layer_args(X, adj, W)
    _require(dY.is_cuda and dY.dtype == torch.float32, "Y_grad must be a float32 CUDA tensor")
    G = ops.mask_mul(dY, mask) if relu else (dY if dY.stride(1) == 1 else dY.contiguous())
    AX = _adj_matmul(adj, X, precision)
    dW = ops.gemm(AX.t(), G, precision=precision)
    T = ops.gemm(G, W.t(), precision=precision)
    dX = _adj_matmul(adj, T, precision)
    return dX, dW

"""Fused ``log_softmax`` + ``nll_loss`` for the classification tail of the
reference's training script (tests/gcn/graphcuda_impl.py:24,55)."""
from __future__ import annotations

from typing import Optional

import torch

from . import _lib
from .ops import _require, _stream


class _LogSoftmaxNLL(torch.autograd.Function):
    @staticmethod
    def forward(ctx, Z, labels, row_mask, scale):
        _require(Z.dim() == 2 and Z.is_cuda and Z.dtype == torch.float32, "logits must be a float32 CUDA matrix")
        _require(labels.is_cuda and labels.dtype == torch.int64 and labels.numel() == Z.size(0),
                 "labels must be a CUDA int64 vector with one entry per row")
        if Z.stride(1) != 1:
            Z = Z.contiguous()
        labels = labels.contiguous()
        mask8 = None
        if row_mask is not None:
            _require(row_mask.is_cuda and row_mask.numel() == Z.size(0), "row_mask must have one entry per row")
            mask8 = row_mask.to(torch.uint8).contiguous()
        M, C = Z.shape
        L = _lib.lib()
        dev = Z.device
        wsb = L.gc_nll_workspace_bytes(M)
        ws = torch.empty(max(wsb, 4), dtype=torch.uint8, device=dev)
        loss = torch.empty((), dtype=torch.float32, device=dev)
        ldz = Z.stride(0) if M > 1 else max(C, 1)
        with torch.cuda.device(dev):
            st = L.gc_logsoftmax_nll_forward_f32(Z.data_ptr(), ldz, labels.data_ptr(),
                                                 mask8.data_ptr() if mask8 is not None else None, M, C,
                                                 float(scale), loss.data_ptr(), ws.data_ptr(), ws.numel(),
                                                 _stream(dev))
        _lib.check(st, "gc_logsoftmax_nll_forward_f32")
        ctx.save_for_backward(Z, labels, ws)
        ctx.mask8 = mask8
        ctx.scale = float(scale)
        return loss

    @staticmethod
    def backward(ctx, grad_loss):
        Z, labels, ws = ctx.saved_tensors
        M, C = Z.shape
        dev = Z.device
        dZ = torch.empty((M, C), dtype=torch.float32, device=dev)
        g = grad_loss.to(torch.float32).contiguous()
        ldz = Z.stride(0) if M > 1 else max(C, 1)
        with torch.cuda.device(dev):
            st = _lib.lib().gc_logsoftmax_nll_backward_f32(
                Z.data_ptr(), ldz, labels.data_ptr(), ctx.mask8.data_ptr() if ctx.mask8 is not None else None, M, C,
                ctx.scale, g.data_ptr(), dZ.data_ptr(), max(C, 1), ws.data_ptr(), _stream(dev))
        _lib.check(st, "gc_logsoftmax_nll_backward_f32")
        return dZ, None, None, None


def log_softmax_nll_loss(logits: torch.Tensor, labels: torch.Tensor, row_mask: Optional[torch.Tensor] = None,
                         scale: Optional[float] = None) -> torch.Tensor:
    """``F.nll_loss(torch.log_softmax(logits, 1)[row_mask], labels[row_mask])`` in one
    kernel per direction.  ``scale`` defaults to 1 / (number of selected rows)
    (reduction='mean'); pass it explicitly to avoid the host read of the mask
    count, or for a different normalisation (e.g. 1 / global rows in the
    row-partitioned model)."""
    if scale is None:
        cnt = int(row_mask.sum().item()) if row_mask is not None else logits.size(0)
        scale = 1.0 / max(cnt, 1)
    return _LogSoftmaxNLL.apply(logits, labels, row_mask, scale)

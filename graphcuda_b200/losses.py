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
        ldz = Z.stride(0) if M > 1 else max(C, 1)
        lddz = max(C, 1)
        if M > 1 and C < ldz <= C + 3 and ldz % 4 == 0:
            # The logits are a view of a matrix padded to 16-byte rows (an odd class count): give the gradient the
            # same pitch with zero pad columns, so the layer below can aggregate it without re-padding a copy.
            from .engine import register_zero_padded
            buf = torch.empty((M, ldz), dtype=torch.float32, device=dev)
            buf[:, C:].zero_()
            register_zero_padded(buf)
            dZ = buf[:, :C]
            lddz = ldz
        else:
            dZ = torch.empty((M, C), dtype=torch.float32, device=dev)
        g = grad_loss.to(torch.float32).contiguous()
        with torch.cuda.device(dev):
            st = _lib.lib().gc_logsoftmax_nll_backward_f32(
                Z.data_ptr(), ldz, labels.data_ptr(), ctx.mask8.data_ptr() if ctx.mask8 is not None else None, M, C,
                ctx.scale, g.data_ptr(), dZ.data_ptr(), lddz, ws.data_ptr(), _stream(dev))
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


def argmax_accuracy(logits: torch.Tensor, labels: Optional[torch.Tensor] = None, masks=None, *,
                    want_pred: bool = True):
    """The evaluation tail of the reference's script (tests/gcn/graphcuda_impl.py:63-68) in one kernel.

    Returns ``(pred, counts)``: ``pred`` = ``logits.argmax(dim=1)`` (int64; lowest index among equal
    maxima; None when want_pred is False), ``counts`` = int64 tensor ``[n, 2]`` on the device with, per
    row selection, the number of selected rows predicted right and the number selected (None without
    labels).  ``masks``: None (all rows), one bool / uint8 vector, or a sequence of up to 8 of them.
    Nothing is read back to the host: ``counts[:, 0] / counts[:, 1]`` are the accuracies."""
    if not (logits.is_cuda and logits.dim() == 2 and logits.dtype == torch.float32):
        raise RuntimeError("argmax_accuracy: float32 CUDA matrix expected")
    Z = logits if logits.stride(1) == 1 or logits.size(1) == 1 else logits.contiguous()
    M, C = Z.shape
    dev = Z.device
    mask_mat = None
    n_masks = 0
    if masks is not None:
        if labels is None:
            raise RuntimeError("argmax_accuracy: masks need labels")
        rows = [masks] if isinstance(masks, torch.Tensor) and masks.dim() == 1 else list(masks)
        if not 1 <= len(rows) <= 8:
            raise RuntimeError("argmax_accuracy: between 1 and 8 row selections")
        for m in rows:
            if m.numel() != M or m.device != dev:
                raise RuntimeError("argmax_accuracy: every selection needs one entry per row, on the logits' device")
        mask_mat = torch.stack([m.reshape(M).ne(0) for m in rows]).to(torch.uint8).contiguous()
        n_masks = len(rows)
    if labels is not None:
        if not (labels.dtype == torch.int64 and labels.numel() == M and labels.device == dev):
            raise RuntimeError("argmax_accuracy: labels must be int64 [M] on the logits' device")
        labels = labels.contiguous()
    with torch.cuda.device(dev):
        pred = torch.empty(M, dtype=torch.int64, device=dev) if want_pred else None
        counts = torch.empty((max(n_masks, 1), 2), dtype=torch.int64, device=dev) if labels is not None else None
        st = _lib.lib().gc_argmax_accuracy_f32(
            Z.data_ptr(), Z.stride(0) if M > 1 else max(C, 1), M, C,
            labels.data_ptr() if labels is not None else None,
            mask_mat.data_ptr() if mask_mat is not None else None, n_masks,
            pred.data_ptr() if pred is not None else None,
            counts.data_ptr() if counts is not None else None, _stream(dev))
        _lib.check(st, "gc_argmax_accuracy_f32")
    return pred, counts

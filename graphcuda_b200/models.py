"""The stacked model of the reference's training script
(tests/gcn/graphcuda_impl.py:15-24), generalised to any depth: GCNConv layers
with ReLU on all but the last, ``log_softmax`` on top."""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from .gcn import GCNConv
from .losses import argmax_accuracy


class GCN(torch.nn.Module):
    def __init__(self, dims: Sequence[int], *, precision: Optional[str] = None, fuse_relu_backward: bool = True):
        super().__init__()
        self.convs = torch.nn.ModuleList(
            [GCNConv(dims[i], dims[i + 1], apply_relu=(i < len(dims) - 2), precision=precision)
             for i in range(len(dims) - 1)])
        if fuse_relu_backward:
            # Layer i's ReLU output has exactly one consumer here (layer i + 1), so the ReLU backward of layer i
            # is applied where layer i + 1 produces its input gradient (reference gcn.cu:36 as a fused store).
            for lower, upper in zip(self.convs[:-1], self.convs[1:]):
                if lower.apply_relu:
                    lower.fuse_relu_backward |= 1
                    upper.fuse_relu_backward |= 2

    def forward(self, x, adj, log_softmax: bool = True, return_hidden: bool = False):
        """log_softmax=False returns the last layer's raw output, for
        losses.log_softmax_nll_loss which fuses the normalisation with the loss.
        return_hidden=True returns (output, [x, h1, ..., logits]): every layer's
        input and output, for checks that compare layer by layer."""
        hidden = [x]
        for conv in self.convs:
            x = conv(x, adj)
            hidden.append(x)
        out = torch.log_softmax(x, dim=1) if log_softmax else x
        return (out, hidden) if return_hidden else out

    @torch.no_grad()
    def evaluate(self, x, adj, labels, masks=None):
        """The reference script's ``test()`` (tests/gcn/graphcuda_impl.py:60-69): a forward pass without
        autograd state (nothing is saved, no mask is written, log_softmax is skipped because it does not
        move the argmax) followed by the fused argmax / count kernel.  Returns ``(pred, counts)`` as
        losses.argmax_accuracy does; ``(counts[:, 0] / counts[:, 1]).tolist()`` gives the accuracies with
        one host read."""
        return argmax_accuracy(self.forward(x, adj, log_softmax=False), labels, masks)

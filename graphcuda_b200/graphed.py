"""Whole-step CUDA-graph capture for launch-bound problems.

On a Cora-sized graph one training step is a few dozen kernels of a few
microseconds each, so the step time is launch latency and Python dispatch (the
reference's 9-13 ms epochs on that graph are the same effect:
tests/gcn/graphcuda_impl.py:77-85).  ``GraphedTrainStep`` records forward,
fused loss, backward and the optimizer update once and replays them as one
graph launch.  Every kernel of this library is enqueued on the stream it is
given, allocates nothing itself and needs no host synchronisation, so it
captures as is; the plan / symmetry checks that read a value back to the host
run during the warm-up steps, before the capture.
"""
from __future__ import annotations

from typing import Optional

import torch

from .losses import log_softmax_nll_loss


class GraphedTrainStep:
    """step() = zero_grad; loss = log_softmax_nll(model(X, adj)[, mask]); backward; optimizer.step().

    X, labels and mask are static buffers: refresh them in place
    (``step.X.copy_(new_X)``) between replays.
    Build it before the model is trained eagerly on another stream: autograd
    ties a parameter's gradient accumulation to the stream of its first use for
    as long as that step's graph is referenced, and a launch on the default
    stream is illegal during capture.  The optimizer must be
    capturable: ``graphcuda_b200.FusedAdam`` (one launch, step count on the
    device) or e.g. ``torch.optim.Adam(..., capturable=True)``."""

    def __init__(self, model, adj, X: torch.Tensor, labels: torch.Tensor, optimizer,
                 row_mask: Optional[torch.Tensor] = None, warmup: int = 3):
        self.model, self.adj, self.optimizer = model, adj, optimizer
        self.X, self.labels, self.row_mask = X, labels, row_mask
        self.scale = 1.0 / max(int(row_mask.sum().item()) if row_mask is not None else X.size(0), 1)
        side = torch.cuda.Stream(device=X.device)
        side.wait_stream(torch.cuda.current_stream(X.device))
        with torch.cuda.stream(side):
            for _ in range(max(warmup, 1)):
                self.warmup_loss = self._eager_step()  # loss of the last eager step, for callers that log it
        torch.cuda.current_stream(X.device).wait_stream(side)
        torch.cuda.synchronize(X.device)
        self.graph = torch.cuda.CUDAGraph()
        optimizer.zero_grad(set_to_none=True)
        with torch.cuda.graph(self.graph):
            self.loss = self._forward_backward_update()

    def _forward_backward_update(self):
        out = self.model(self.X, self.adj, log_softmax=False)
        loss = log_softmax_nll_loss(out, self.labels, self.row_mask, scale=self.scale)
        loss.backward()
        self.optimizer.step()
        return loss

    def _eager_step(self):
        self.optimizer.zero_grad(set_to_none=True)
        return self._forward_backward_update()

    def step(self) -> torch.Tensor:
        """Replays the recorded step; returns the (static) loss tensor."""
        self.graph.replay()
        return self.loss

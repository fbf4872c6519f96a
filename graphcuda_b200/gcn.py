"""``GCNConv`` -- the module the reference exposes as ``graphcuda.GCNConv``
(src/graphcuda/python/gcn.py:36-48) with its autograd function
(src/graphcuda/python/gcn.py:14-34).

Same constructor, same parameter (one tensor ``weights`` of shape in x out,
initialised ``uniform(-s, s)``, ``s = sqrt(2 / (in + out))`` with the same RNG
consumption), same ``forward(X, adjm)``.  Additive keyword arguments: an
optional ``bias`` (absent by default, so ``state_dict()`` keys are unchanged)
and a ``precision`` switch.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn
from torch.nn.parameter import Parameter

from .adjacency import as_adjacency
from .engine import layer_backward, layer_forward


class GCNConvFunction(torch.autograd.Function):
    """Y = relu((adjm @ X) @ weights [+ bias]).

    Unlike the reference (python/gcn.py:18) the fp32 mask is not materialised:
    the activation itself is saved and the mask re-derived as Y > 0; the
    aggregated features are saved instead of being recomputed (gcn.cu:40)."""

    @staticmethod
    def forward(ctx, X, adjm, weights, apply_relu, bias=None, precision=None, fuse=0):
        # fuse: bit 0 = the incoming gradient is already multiplied by this layer's ReLU mask;
        #       bit 1 = X is the ReLU output of the layer below: gate dX by (X > 0) where it is produced
        adj = as_adjacency(adjm)
        Y, _, saved = layer_forward(X, adj, weights, bias, bool(apply_relu), precision=precision)
        order, inter = saved
        ctx.adj = adj
        ctx.order = order
        ctx.apply_relu = bool(apply_relu)
        ctx.precision = precision
        ctx.has_bias = bias is not None
        ctx.has_inter = inter is not None
        ctx.fuse = int(fuse)
        tensors = [X, weights, Y]
        if inter is not None:
            tensors.append(inter)
        ctx.save_for_backward(*tensors)
        return Y

    @staticmethod
    def backward(ctx, grad_Y):
        saved = ctx.saved_tensors
        X, weights, Y = saved[:3]
        inter = saved[3] if ctx.has_inter else None
        need_dX, _, need_dW = ctx.needs_input_grad[:3]
        need_db = ctx.has_bias and ctx.needs_input_grad[4]
        if grad_Y.stride(-1) != 1:  # rows may keep a larger pitch (a padded gradient from the fused loss)
            grad_Y = grad_Y.contiguous()
        dX, dW, db = layer_backward(grad_Y, X, ctx.adj, weights, ctx.apply_relu, Y,
                                    (ctx.order, inter), need_dX=need_dX, need_dW=need_dW, need_db=need_db,
                                    precision=ctx.precision, grad_is_gated=bool(ctx.fuse & 1),
                                    gate_dx_by_input=bool(ctx.fuse & 2))
        return dX, None, dW, None, db, None, None


class GCNConv(nn.Module):
    def __init__(self, in_dim: int, out_dim: int, apply_relu: bool = True, *, bias: bool = False,
                 precision: Optional[str] = None):
        super().__init__()
        self.in_dim = in_dim
        self.out_dim = out_dim
        self.apply_relu = apply_relu
        self.precision = precision
        # Set by a container that knows the layer's neighbours (models.GCN): see GCNConvFunction.forward.
        # Only valid when this layer's output feeds exactly one consumer that gates its input gradient.
        self.fuse_relu_backward = 0

        stdv = math.sqrt(2.0 / (in_dim + out_dim))
        self.weights = Parameter(torch.Tensor(in_dim, out_dim))
        self.weights.data.uniform_(-stdv, stdv)
        if bias:
            self.bias = Parameter(torch.zeros(out_dim))
        else:
            self.register_parameter("bias", None)

    def forward(self, X: torch.Tensor, adjm) -> torch.Tensor:
        return GCNConvFunction.apply(X, adjm, self.weights, self.apply_relu, self.bias, self.precision,
                                     self.fuse_relu_backward)

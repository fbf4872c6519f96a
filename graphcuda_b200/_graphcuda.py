"""The eight operators the reference exports from its pybind module
(src/graphcuda/cuda/pybind.cu:7-23), same names and positional signatures,
backed by this package's sm_100a kernels.

Differences a caller can observe, all additive:
  * ``adjm`` / ``sparseA`` may be a sparse COO tensor (the reference's only
    accepted layout, spmm_cusparse.cu:5-6), a sparse CSR tensor, a dense matrix
    (what the README and src/graphcuda/cpp/gcn.cpp:10 use), a
    ``(rowptr, col, val)`` int32 CSR tuple or a ``CSRAdjacency``;
  * ``matmul3``/``matmul4`` are correct for every shape (the reference's are
    not when the tile shapes differ or N % 4 != 0: matmul3.cu:215-232,
    matmul4.cu:185-201);
  * everything runs on the current stream of the input's device.
CPU tensors raise RuntimeError as in the reference; there is no CPU path.
"""
from __future__ import annotations

import torch

from . import ops
from .adjacency import as_adjacency
from .engine import layer_backward_reference_form, layer_forward


def gcn_conv_forward(X, adjm, weights, apply_relu):
    """(Y, mask) with Y = relu((adjm @ X) @ weights) and mask = (pre-activation
    > 0) as float32; without ReLU the mask is an uninitialised 0-dim CPU tensor
    (src/graphcuda/cuda/gcn.cu:5-25)."""
    adj = as_adjacency(adjm)
    Y, mask, _ = layer_forward(X, adj, weights, None, bool(apply_relu), want_mask=bool(apply_relu))
    if not apply_relu:
        mask = torch.empty(())
    return Y, mask


def gcn_conv_backward(Y_grad, X_cached, adjm, weights, apply_relu, mask_cached):
    """(dX, dW) as src/graphcuda/cuda/gcn.cu:27-52 computes them:
    G = Y_grad * mask; dW = (adjm @ X)^T @ G; dX = adjm @ (G @ weights^T)."""
    adj = as_adjacency(adjm)
    return layer_backward_reference_form(Y_grad, X_cached, adj, weights, bool(apply_relu), mask_cached)


def _matmul(A, B):
    return ops.gemm(A, B)


def matmul1(A, B):
    """C = A @ B (src/graphcuda/cuda/matmul1.cu:27-61)."""
    return _matmul(A, B)


def matmul2(A, B):
    """C = A @ B (src/graphcuda/cuda/matmul2.cu:65-100)."""
    return _matmul(A, B)


def matmul3(A, B):
    """C = A @ B (src/graphcuda/cuda/matmul3.cu:194-243)."""
    return _matmul(A, B)


def matmul4(A, B):
    """C = A @ B (src/graphcuda/cuda/matmul4.cu:209-265)."""
    return _matmul(A, B)


def gemm_cublas(A, B):
    """C = A @ B in fp32 (src/graphcuda/cuda/gemm_cublas.cu:3-55)."""
    return _matmul(A, B)


def spmm_cusparse(sparseA, B):
    """C = sparseA @ B (src/graphcuda/cuda/spmm_cusparse.cu:3-126)."""
    if isinstance(sparseA, torch.Tensor):
        if not (sparseA.layout in (torch.sparse_coo, torch.sparse_csr)):
            raise RuntimeError("A must be a sparse COO tensor")
    adj = as_adjacency(sparseA)
    return adj.matmul(B)

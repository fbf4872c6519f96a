"""CPU oracle for the GCN layer path -- TEST INFRASTRUCTURE ONLY.

Only ``tests/``, ``__graft_entry__.smoke()`` and the ``cpu_baseline`` /
``--impl reference`` legs of ``bench.py`` may import this module, and only as
the checker or the timed CPU baseline; the shipped package never does.

It restates, with torch CPU ops, the reference's own algorithm:

  * layer forward / backward: src/graphcuda/cpp/gcn.cpp:4-20 and :22-41 (the
    ATen twin of src/graphcuda/cuda/gcn.cu:5-52; same math as
    tests/gcn/pytorch_impl.py:14-38);
  * the autograd wrapper and module: src/graphcuda/python/gcn.py:14-48;
  * the stand-alone operators: ``A @ B`` for matmul1..4 / gemm_cublas
    (src/graphcuda/cuda/gemm_cublas.cu:37-48) and ``torch.sparse.mm`` for
    spmm_cusparse (src/graphcuda/cuda/spmm_cusparse.cu:105-116), which is what
    the reference's own check compares against
    (tests/matmul/graphcuda_impl.py:68-79,99-100);
  * adjacency construction as the reference's scripts do it
    (tests/gcn/graphcuda_impl.py:27-38): add_self_loops -> gcn_norm ->
    sparse_coo_tensor(...).coalesce().

Pinning.  The layer math is pinned against the reference's own gcn.cpp compiled
for CPU (``oracle/build_ref.py`` -> ``oracle/_ref``; tests/test_oracle_pin.py)
and against fixtures that code produced (``tests/golden``).  The
normalisation comes from a third-party dependency that is NOT in the reference
tree and not installed here: torch_geometric, pinned ``torch-geometric==2.6.1``
(requirements.txt:5).  ``gcn_norm`` below restates that library's published
algorithm (degree by scatter-add over the target index, ``deg.pow(-0.5)``,
inf -> 0, ``dinv[row] * w * dinv[col]``); the reference holds no golden vector
for it, so at that boundary parity is UNPINNED (a hand-computed known-answer
case and structural properties are all that anchor it).
"""
from __future__ import annotations

import math

import torch


# ---------------------------------------------------------------- layer math
def gcn_conv_forward(X, adjm, weights, apply_relu):
    """src/graphcuda/cpp/gcn.cpp:4-20."""
    y = adjm.mm(X).mm(weights)
    if apply_relu:
        mask = y.gt(0).to(torch.float32)
        return y * mask, mask
    return y, torch.empty(())


def gcn_conv_backward(Y_grad, X_cached, adjm, weights, apply_relu, mask_cached):
    """src/graphcuda/cpp/gcn.cpp:22-41 (A, not A^T, multiplies the input gradient)."""
    if apply_relu:
        Y_grad = Y_grad * mask_cached
    A_X = adjm.mm(X_cached)
    dW = A_X.transpose(0, 1).mm(Y_grad)
    dX = adjm.mm(Y_grad.mm(weights.transpose(0, 1)))
    return dX, dW


class _Ops:
    """Stand-in for the extension module the autograd function calls into."""
    gcn_conv_forward = staticmethod(gcn_conv_forward)
    gcn_conv_backward = staticmethod(gcn_conv_backward)


class GCNConvFunction(torch.autograd.Function):
    """src/graphcuda/python/gcn.py:14-34; ``ops`` selects the restatement above
    or the reference's compiled module."""

    ops = _Ops

    @staticmethod
    def forward(ctx, X, adjm, weights, apply_relu, ops=None):
        ops = ops or GCNConvFunction.ops
        Y, mask = ops.gcn_conv_forward(X, adjm, weights, apply_relu)
        ctx.save_for_backward(X, adjm, weights, mask)
        ctx.apply_relu = apply_relu
        ctx.ops = ops
        return Y

    @staticmethod
    def backward(ctx, grad_Y):
        X_cached, adjm, weights, mask_cached = ctx.saved_tensors
        dX, dW = ctx.ops.gcn_conv_backward(grad_Y.contiguous(), X_cached, adjm, weights, ctx.apply_relu, mask_cached)
        return dX, None, dW, None, None


class GCNConv(torch.nn.Module):
    """src/graphcuda/python/gcn.py:36-48 (same initialiser, same RNG use)."""

    def __init__(self, in_dim, out_dim, apply_relu=True, ops=None):
        super().__init__()
        self.in_dim, self.out_dim, self.apply_relu = in_dim, out_dim, apply_relu
        self.ops = ops
        stdv = math.sqrt(2.0 / (in_dim + out_dim))
        self.weights = torch.nn.Parameter(torch.Tensor(in_dim, out_dim))
        self.weights.data.uniform_(-stdv, stdv)

    def forward(self, X, adjm):
        return GCNConvFunction.apply(X, adjm, self.weights, self.apply_relu, self.ops)


class GCN(torch.nn.Module):
    """The stacked model of the reference's training script
    (tests/gcn/graphcuda_impl.py:15-24): ReLU on every layer but the last,
    log_softmax on top; ``dims`` = [in, hidden..., classes]."""

    def __init__(self, dims, ops=None):
        super().__init__()
        self.convs = torch.nn.ModuleList(
            [GCNConv(dims[i], dims[i + 1], apply_relu=(i < len(dims) - 2), ops=ops) for i in range(len(dims) - 1)])

    def forward(self, x, adj):
        for conv in self.convs:
            x = conv(x, adj)
        return torch.log_softmax(x, dim=1)


def layer_with_bias(X, adjm, weights, bias, apply_relu):
    """relu((A X) W + b): the reference pre-activation with a bias added, the
    definition used for the bias+ReLU configuration."""
    y = adjm.mm(X).mm(weights) + bias
    if apply_relu:
        mask = y.gt(0).to(torch.float32)
        return y * mask, mask
    return y, None


# ---------------------------------------------------------------- operators
def matmul(A, B):
    """What matmul1..4 / gemm_cublas compute (gemm_cublas.cu:37-48)."""
    return A @ B


def spmm(A_sparse, B):
    """What spmm_cusparse computes (spmm_cusparse.cu:105-116)."""
    return torch.sparse.mm(A_sparse, B)


# ---------------------------------------------------------------- adjacency
def add_self_loops(edge_index, num_nodes):
    """One (i, i) edge per node appended (tests/gcn/graphcuda_impl.py:27)."""
    loops = torch.arange(num_nodes, dtype=torch.int64)
    return torch.cat([edge_index, torch.stack([loops, loops])], dim=1)


def gcn_norm(edge_index, num_nodes):
    """Published algorithm of torch_geometric 2.6.1 ``gcn_norm`` for unit edge
    weights on an edge list that already holds every self-loop (so its
    add_remaining_self_loops step changes nothing but the edge order):
    deg = scatter_add(1, col); dinv = deg ** -0.5 with inf -> 0;
    w = dinv[row] * 1 * dinv[col].  Call site: tests/gcn/graphcuda_impl.py:28."""
    row, col = edge_index[0], edge_index[1]
    ones = torch.ones(edge_index.size(1), dtype=torch.float32)
    deg = torch.zeros(num_nodes, dtype=torch.float32).scatter_add_(0, col, ones)
    dinv = deg.pow(-0.5)
    dinv.masked_fill_(dinv == float("inf"), 0)
    return dinv[row] * ones * dinv[col]


def normalized_adjacency_coo(edge_index, num_nodes):
    """tests/gcn/graphcuda_impl.py:27-38: self-loops, gcn_norm, coalesced COO."""
    ei = add_self_loops(edge_index, num_nodes)
    w = gcn_norm(ei, num_nodes)
    return torch.sparse_coo_tensor(ei, w, (num_nodes, num_nodes)).coalesce()


def coo_to_csr_int32(A_coo):
    """(rowptr int32, col int32, val fp32) of a coalesced COO matrix."""
    csr = A_coo.to_sparse_csr()
    return csr.crow_indices().to(torch.int32), csr.col_indices().to(torch.int32), csr.values().clone()


# ---------------------------------------------------------------- metrics
def rel_fro(out, ref):
    """||out - ref||_F / ||ref||_F in float64 (0 when both are zero)."""
    out = out.detach().double().cpu()
    ref = ref.detach().double().cpu()
    d = (out - ref).norm().item()
    n = ref.norm().item()
    return d / n if n > 0 else d


def rel_max(out, ref):
    """max|out - ref| / max|ref|."""
    out = out.detach().double().cpu()
    ref = ref.detach().double().cpu()
    d = (out - ref).abs().max().item() if out.numel() else 0.0
    n = ref.abs().max().item() if ref.numel() else 0.0
    return d / n if n > 0 else d

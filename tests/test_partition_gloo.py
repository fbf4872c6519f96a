"""Row-partitioned layer on 2 and 3 gloo ranks (CPU): partition arithmetic, the
all-gather / all-reduce orchestration and the autograd wiring, with torch CPU
ops standing in for the CUDA kernels.  The single-process oracle model is the
reference for outputs and gradients."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from graphcuda_b200.partition import (DistGCN, FeatureShardedGraph, PartitionedGraph, RowPartition,
                                      slice_csr_rows, split_csr_columns)
from oracle import gcn_oracle as O


class TorchCPUBackend:
    """Same interface as partition.CudaBackend, on torch CPU ops."""

    def make_adj(self, rowptr, col, val, shape):
        return torch.sparse_csr_tensor(rowptr.long(), col.long(), val, size=tuple(shape))

    def spmm(self, adj, H, *, bias=None, relu=False, accumulate_into=None, out=None, gate=None):
        y = adj @ H if adj.shape[0] and adj.shape[1] else torch.zeros(adj.shape[0], H.size(1))
        if accumulate_into is not None:
            y = accumulate_into + y
        if bias is not None:
            y = y + bias
        if relu:
            y = y * (y > 0)
        if gate is not None:
            y = y * (gate > 0)
        if accumulate_into is not None:  # in place, like the CUDA kernel
            accumulate_into.copy_(y)
            return accumulate_into
        if out is not None:
            out.copy_(y)
            return out
        return y

    def gemm(self, A, B, *, bias=None, relu=False, precision=None, gate=None):
        y = A @ B
        if bias is not None:
            y = y + bias
        if relu:
            y = y * (y > 0)
        if gate is not None:
            y = y * (gate > 0)
        return y

    def relu_backward(self, dY, Y):
        return dY * (Y > 0)


def test_row_partition_bounds():
    p = RowPartition(10, 4)
    assert p.block == 3 and p.padded == 12
    assert [p.bounds(r) for r in range(4)] == [(0, 3), (3, 6), (6, 9), (9, 10)]
    assert p.owner(9) == 3 and p.owner(2) == 0
    q = RowPartition(5, 8)  # more ranks than rows per block boundary: some ranks own nothing
    assert q.bounds(7) == (5, 5)
    assert RowPartition(2449029, 8).block == 306129
    with pytest.raises(ValueError):
        RowPartition(10, 0)


def test_nnz_balanced_partition():
    """Block boundaries placed on the prefix sums of the row lengths: every block carries about nnz / world
    non-zeros even when the rows are ordered by degree, and padded space round-trips."""
    deg = torch.tensor([50, 30, 10, 4, 2, 1, 1, 1, 1, 0, 0, 0])
    rowptr = torch.cat([torch.zeros(1, dtype=torch.int64), torch.cumsum(deg, 0)]).to(torch.int32)
    p = RowPartition(12, 3, rowptr=rowptr)
    assert not p.uniform and p.starts[0] == 0 and p.starts[-1] == 12
    sizes = [int(rowptr[b] - rowptr[a]) for a, b in zip(p.starts[:-1], p.starts[1:])]
    assert sum(sizes) == 100 and max(sizes) <= 50  # no block holds more than the heaviest single row forces
    assert p.block == max(b - a for a, b in zip(p.starts[:-1], p.starts[1:])) and p.padded == 3 * p.block
    ids = torch.arange(12)
    pos = p.to_padded(ids)
    for r in range(3):
        lo, hi = p.bounds(r)
        assert torch.equal(pos[lo:hi], torch.arange(hi - lo) + r * p.block)
        assert all(p.owner(i) == r for i in range(lo, hi))
    full = torch.full((p.padded, 2), -1.0)
    full[pos] = torch.arange(24.0).view(12, 2)
    assert torch.equal(p.unpad(full), torch.arange(24.0).view(12, 2))
    u = RowPartition(10, 4)
    assert u.uniform and torch.equal(u.to_padded(ids[:10]), ids[:10])
    assert torch.equal(u.unpad(torch.arange(24.0).view(12, 2)), torch.arange(20.0).view(10, 2))


def _graph(n, seed):
    from graphcuda_b200 import synth
    e = synth.rmat_edges(max(4, (n - 1).bit_length()), n, n * 4, seed)
    A = O.normalized_adjacency_coo(synth.symmetrize(e), n)
    return A, O.coo_to_csr_int32(A)


def test_csr_slicing_and_column_split():
    n = 101
    A, (rowptr, col, val) = _graph(n, 1)
    D = A.to_dense()
    lo, hi = 30, 64
    rp, c, v = slice_csr_rows(rowptr, col, val, lo, hi)
    sub = torch.sparse_csr_tensor(rp.long(), c.long(), v, size=(hi - lo, n)).to_dense()
    assert torch.equal(sub, D[lo:hi])
    (rp_i, c_i, v_i), (rp_o, c_o, v_o) = split_csr_columns(rp, c, v, lo, hi)
    inside = torch.sparse_csr_tensor(rp_i.long(), c_i.long(), v_i, size=(hi - lo, hi - lo)).to_dense()
    outside = torch.sparse_csr_tensor(rp_o.long(), c_o.long(), v_o, size=(hi - lo, n)).to_dense()
    assert torch.equal(inside, D[lo:hi, lo:hi])
    ref_out = D[lo:hi].clone()
    ref_out[:, lo:hi] = 0
    assert torch.equal(outside, ref_out)
    assert rp_i.dtype == torch.int32 and c_i.dtype == torch.int32


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, n, dims, q, mode="rows", fuse=True, balance="rows"):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.set_num_threads(1)
        A, (rowptr, col, val) = _graph(n, 3)
        g = torch.Generator().manual_seed(0)
        X = torch.randn(n, dims[0], generator=g)
        y = torch.randint(0, dims[-1], (n,), generator=g)
        be = TorchCPUBackend()
        if mode == "rows":
            graph = PartitionedGraph(rowptr, col, val, n, backend=be, balance=balance)
        elif mode == "hybrid":
            from graphcuda_b200.partition import HybridGraph
            graph = HybridGraph(rowptr, col, val, be.make_adj(rowptr, col, val, (n, n)), n, backend=be,
                                wide_from=10)
        else:
            graph = FeatureShardedGraph(be.make_adj(rowptr, col, val, (n, n)), n, backend=be)
        lo, hi = graph.lo, graph.hi
        torch.manual_seed(5)
        model = DistGCN(dims, fuse_relu_backward=fuse)
        Xl = X[lo:hi].clone().requires_grad_()
        # constant input features: exchanged once, outside the step
        Xg = graph.prepare_constant(X[lo:hi])
        out = model(Xl, graph, X_gathered=Xg)
        loss = torch.nn.functional.nll_loss(out, y[lo:hi], reduction="sum") / n
        loss.backward()
        total = graph.all_reduce_sum(loss.detach().clone())
        q.put((rank, lo, hi, out.detach(), Xl.grad, [w.grad for w in model.weights], float(total)))
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,n,dims", [(2, 64, [12, 20, 20, 5]), (3, 50, [9, 16, 4]), (2, 33, [20, 8, 6])])
@pytest.mark.parametrize("mode,fuse", [("rows", True), ("features", True), ("rows", False), ("rows-nnz", True),
                                       ("hybrid", True)])
def test_partitioned_model_matches_single_process(world, n, dims, mode, fuse):
    """fuse: the ReLU backward of a hidden layer applied where the layer above produces its input gradient
    (in the GEMM's store, or in a pass after the aggregation's exchange), or as the reference places it."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    balance = "nnz" if mode == "rows-nnz" else "rows"
    mode = "rows" if mode == "rows-nnz" else mode
    procs = [ctx.Process(target=_worker, args=(r, world, port, n, dims, q, mode, fuse, balance)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    # single-process reference
    A, _ = _graph(n, 3)
    g = torch.Generator().manual_seed(0)
    X = torch.randn(n, dims[0], generator=g)
    y = torch.randint(0, dims[-1], (n,), generator=g)
    torch.manual_seed(5)
    ref = O.GCN(dims)
    Xr = X.clone().requires_grad_()
    out = ref(Xr, A)
    loss = torch.nn.functional.nll_loss(out, y, reduction="sum") / n
    loss.backward()
    for rank, lo, hi, o, dx, dws, total in sorted(results, key=lambda r: r[0]):
        assert O.rel_fro(o, out[lo:hi]) < 1e-5
        assert O.rel_fro(dx, Xr.grad[lo:hi]) < 1e-5
        for dw, conv in zip(dws, ref.convs):
            assert O.rel_fro(dw, conv.weights.grad) < 1e-5  # already summed over ranks
        assert abs(total - loss.item()) < 1e-5


def test_width_padding_helpers():
    from graphcuda_b200 import engine
    assert engine._padded_width(2_449_029, 256, 47) == 48
    assert engine._padded_width(2708, 16, 7) == 7          # small problems are not padded
    assert engine._padded_width(2_449_029, 256, 256) == 256
    W = torch.arange(6.0).reshape(2, 3)
    P = engine._pad_cols(W, 4)
    assert P.shape == (2, 4) and torch.equal(P[:, :3], W) and float(P[:, 3].abs().sum()) == 0.0
    assert engine._pad_cols(W, 3) is W

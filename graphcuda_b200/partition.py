"""Row-partitioned GCN layer for graphs spread over several GPUs (one process
per GPU, ``torch.distributed``; NCCL over NVLink on the GPUs, gloo in the CPU
tests).  The reference has no distributed code; this extends its layer
(src/graphcuda/cuda/gcn.cu:5-52) to the 1-D row partition:

  * rank r owns rows [r*B, (r+1)*B) of the normalised adjacency (all columns,
    global column ids), the matching rows of every feature matrix, and a
    replica of every weight;
  * the one exchange per aggregation is an all-gather of the row blocks of
    the matrix being aggregated (X, H = X W, or the backward counterparts);
  * the local rows' adjacency is split by column into the diagonal block
    (columns owned by this rank) and the rest, so the diagonal-block SpMM runs
    on the compute stream while the all-gather is in flight, and the
    off-diagonal SpMM accumulates on top once the gathered matrix has landed
    in local memory (remote rows are never read through peer pointers);
  * weight gradients are summed with an all-reduce (tiny: in x out).

The numerical work goes through a small backend object so that the same
orchestration runs on CUDA (this library's kernels) and, in the CPU tests,
on torch CPU ops under gloo.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from .engine import _pad_cols, _padded_width


# ---------------------------------------------------------------- partition arithmetic
class RowPartition:
    """Contiguous row blocks, one per rank.

    Without ``rowptr``: uniform blocks of ceil(n / world) rows; the last block
    may be short (or empty).  With ``rowptr`` (the CSR row pointer of the matrix
    being partitioned): block boundaries are placed so that every block carries
    about nnz / world non-zeros -- what balances the aggregation when the vertex
    labels are ordered by degree (adjacency.normalized_adjacency(reorder=
    "degree")) and equal row counts would give the first rank most of the work.

    Collectives move equal-sized blocks, so every block is padded to ``block``
    rows (the largest block): "padded space" is the row numbering of the
    gathered matrix, rank r's rows at [r * block, r * block + rows_r)."""

    def __init__(self, n: int, world: int, *, rowptr: Optional[torch.Tensor] = None):
        if n < 0 or world < 1:
            raise ValueError("RowPartition: n >= 0 and world >= 1 required")
        self.n = n
        self.world = world
        if rowptr is None or n == 0:
            self.block = -(-n // world) if n else 0
            self.starts = [min(r * self.block, n) for r in range(world + 1)]
            self.uniform = True
        else:
            if rowptr.numel() != n + 1:
                raise ValueError("RowPartition: rowptr must have n + 1 entries")
            rp = rowptr.detach().to("cpu", torch.int64)
            nnz = int(rp[-1])
            # first row whose prefix of non-zeros reaches r/world of the total
            targets = torch.tensor([(nnz * r + world - 1) // world for r in range(1, world)], dtype=torch.int64)
            cuts = torch.searchsorted(rp, targets, right=False).clamp_(0, n).tolist() if world > 1 else []
            starts = [0] + cuts + [n]
            for i in range(1, len(starts)):  # keep the boundaries monotone
                starts[i] = max(starts[i], starts[i - 1])
            self.starts = starts
            self.block = max(b - a for a, b in zip(starts[:-1], starts[1:]))
            self.uniform = False
        self.padded = self.block * world

    def bounds(self, rank: int):
        if not 0 <= rank < self.world:
            raise ValueError("rank out of range")
        return self.starts[rank], self.starts[rank + 1]

    def owner(self, row: int) -> int:
        if self.uniform:
            return row // self.block if self.block else 0
        import bisect
        return min(bisect.bisect_right(self.starts, row) - 1, self.world - 1)

    def to_padded(self, ids: torch.Tensor) -> torch.Tensor:
        """Global row / column ids -> positions in padded space (the identity for uniform blocks)."""
        if self.uniform:
            return ids
        starts = torch.tensor(self.starts, dtype=torch.int64, device=ids.device)
        own = torch.bucketize(ids.to(torch.int64), starts[1:-1].contiguous(), right=True)
        return (own * self.block + (ids.to(torch.int64) - starts[own])).to(ids.dtype)

    def unpad(self, full: torch.Tensor) -> torch.Tensor:
        """Rows of a gathered matrix ([padded, F]) back in global order ([n, F])."""
        if self.uniform:
            return full[:self.n]
        return torch.cat([full[r * self.block: r * self.block + (self.starts[r + 1] - self.starts[r])]
                          for r in range(self.world)])


def slice_csr_rows(rowptr: torch.Tensor, col: torch.Tensor, val: torch.Tensor, lo: int, hi: int):
    """Rows [lo, hi) of a CSR matrix as a CSR matrix (column ids untouched)."""
    s = int(rowptr[lo])
    e = int(rowptr[hi])
    rp = (rowptr[lo:hi + 1] - rowptr[lo]).to(rowptr.dtype)
    return rp, col[s:e], val[s:e]


def split_csr_columns(rowptr: torch.Tensor, col: torch.Tensor, val: torch.Tensor, lo: int, hi: int):
    """Splits a CSR matrix into the entries with lo <= col < hi (column ids
    rebased to col - lo) and the rest (column ids untouched).  Order within a
    row is preserved in both parts."""
    inside = (col >= lo) & (col < hi)
    csum = torch.zeros(col.numel() + 1, dtype=torch.int64, device=col.device)
    torch.cumsum(inside.to(torch.int64), 0, out=csum[1:])
    rp64 = rowptr.to(torch.int64)
    rp_in = csum[rp64]
    rp_out = rp64 - rp_in
    part_in = (rp_in.to(rowptr.dtype), (col[inside] - lo).to(col.dtype), val[inside])
    part_out = (rp_out.to(rowptr.dtype), col[~inside], val[~inside])
    return part_in, part_out


# ---------------------------------------------------------------- backends
class CudaBackend:
    """This library's kernels."""

    def make_adj(self, rowptr, col, val, shape):
        from .adjacency import CSRAdjacency
        return CSRAdjacency(rowptr.contiguous(), col.contiguous(), val.contiguous(), shape, symmetric=False)

    def spmm(self, adj, H, *, bias=None, relu=False, accumulate_into=None, out=None):
        return adj.matmul(H, bias=bias, relu=relu, accumulate_into=accumulate_into, out=out)

    def gemm(self, A, B, *, bias=None, relu=False, precision=None, gate=None):
        from . import ops
        return ops.gemm(A, B, bias=bias, relu=relu, precision=precision, gate=gate)

    def relu_backward(self, dY, Y):
        from . import ops
        return ops.relu_backward(dY, Y)


# ---------------------------------------------------------------- partitioned graph
class PartitionedGraph:
    """This rank's rows of a (symmetric) normalised adjacency, split into the
    diagonal block and the remainder, plus the gather buffers."""

    def __init__(self, rowptr, col, val, n_nodes: int, *, rank: Optional[int] = None,
                 world: Optional[int] = None, group=None, backend=None, rows_are_local: bool = False,
                 balance: str = "rows", partition: Optional[RowPartition] = None):
        """rowptr/col/val: the GLOBAL CSR (every rank passes the same), or with
        rows_are_local=True this rank's row block only (global column ids; pass
        the `partition` it was cut with).  balance: "rows" = equal row counts,
        "nnz" = equal non-zeros per rank (needs the global rowptr)."""
        self.group = group
        self.rank = dist.get_rank(group) if rank is None else rank
        self.world = dist.get_world_size(group) if world is None else world
        if balance not in ("rows", "nnz"):
            raise ValueError("balance must be 'rows' or 'nnz'")
        if partition is not None:
            self.part = partition
        elif balance == "nnz":
            if rows_are_local:
                raise ValueError("balance='nnz' needs the global row pointer (or pass partition=)")
            self.part = RowPartition(n_nodes, self.world, rowptr=rowptr)
        else:
            self.part = RowPartition(n_nodes, self.world)
        self.lo, self.hi = self.part.bounds(self.rank)
        self.n = n_nodes
        self.rows = self.hi - self.lo
        self.backend = backend or CudaBackend()
        if not rows_are_local:
            rowptr, col, val = slice_csr_rows(rowptr, col, val, self.lo, self.hi)
        self.nnz_local_rows = int(col.numel())
        (rp_d, c_d, v_d), (rp_o, c_o, v_o) = split_csr_columns(rowptr, col, val, self.lo, self.hi)
        c_o = self.part.to_padded(c_o)  # the remainder gathers from the all-gathered matrix (padded space)
        self.diag = self.backend.make_adj(rp_d, c_d, v_d, (self.rows, max(self.rows, 0)))
        self.offd = self.backend.make_adj(rp_o, c_o, v_o, (self.rows, self.part.padded))
        self.nnz_diag = int(c_d.numel())
        self.nnz_offd = int(c_o.numel())
        self.device = val.device
        self._gather_bufs = {}
        self._stage_bufs = {}

    # -- collectives ----------------------------------------------------------
    def _gather_buffer(self, F: int, tag: str):
        key = (F, tag)
        buf = self._gather_bufs.get(key)
        if buf is None:
            buf = torch.zeros((self.part.padded, F), dtype=torch.float32, device=self.device)
            self._gather_bufs[key] = buf
        return buf

    def all_gather_rows_async(self, H_local: torch.Tensor, tag: str = "a"):
        """Starts the all-gather of the row blocks; returns (gathered, work).
        `gathered` is indexable by global row id once work.wait() returned."""
        F = H_local.size(1)
        out = self._gather_buffer(F, tag)
        src = H_local
        if self.rows != self.part.block or not H_local.is_contiguous():
            key = (F, tag)
            st = self._stage_bufs.get(key)
            if st is None:
                st = torch.zeros((self.part.block, F), dtype=torch.float32, device=self.device)
                self._stage_bufs[key] = st
            st[:self.rows].copy_(H_local)
            src = st
        if self.world == 1:
            out[:self.part.block].copy_(src)
            return out, None
        work = dist.all_gather_into_tensor(out, src, group=self.group, async_op=True)
        return out, work

    def all_reduce_sum(self, t: torch.Tensor) -> torch.Tensor:
        if self.world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.SUM, group=self.group)
        return t

    def prepare_constant(self, X_local: torch.Tensor) -> torch.Tensor:
        """All rows of a matrix that does not change between steps (the input
        features): gathered once, reused by every step."""
        buf, work = self.all_gather_rows_async(X_local, tag="x")
        if work is not None:
            work.wait()
        return buf.clone()

    # -- aggregation ----------------------------------------------------------
    def aggregate(self, H_local: torch.Tensor, *, gathered=None, bias=None, relu=False, tag="a"):
        """rows_r of A @ H for H given by its local row block: diagonal block
        first (overlapping the all-gather), then the off-diagonal remainder with
        the fused bias/ReLU.  `gathered` short-circuits the exchange when the
        full matrix is already resident (constant input features)."""
        work = None
        if gathered is None:
            gathered, work = self.all_gather_rows_async(H_local, tag)
        Y = self.backend.spmm(self.diag, H_local)
        if work is not None:
            work.wait()
        return self.backend.spmm(self.offd, gathered, bias=bias, relu=relu, accumulate_into=Y)


class FeatureShardedGraph:
    """The aggregation sharded over FEATURE columns instead of adjacency rows.

    Every rank keeps the whole normalised adjacency (int32 CSR: 8 bytes per
    non-zero) and aggregates a slab of F/P feature columns for ALL nodes, so the
    aggregation itself needs no exchange and gathers from a slab of H that is P
    times narrower (and so far friendlier to the L2).  Dense layers stay
    row-sharded (rank r owns rows [r*B, (r+1)*B)), which makes the exchange two
    all-to-all transposes around each aggregation:

        rows -> columns : rank r sends Y_r[:, slab_q] to rank q
        columns -> rows : rank r sends Z[rows of q, slab_r] to rank q

    An all-to-all moves every element once ((P-1)/P^2 of N*F*4 bytes per rank),
    where the all-gather of the row-partitioned scheme delivers (P-1)/P of it to
    every rank -- P times less traffic over NVLink.

    Same interface as PartitionedGraph (aggregate / prepare_constant /
    all_reduce_sum), so DistGCNConvFunction and DistGCN run on either.
    """

    def __init__(self, adj, n_nodes: int, *, rank: Optional[int] = None, world: Optional[int] = None, group=None,
                 backend=None, device=None):
        """adj: the whole adjacency as the backend's matrix object (CSRAdjacency
        on CUDA), identical on every rank."""
        self.group = group
        self.rank = dist.get_rank(group) if rank is None else rank
        self.world = dist.get_world_size(group) if world is None else world
        self.part = RowPartition(n_nodes, self.world)
        self.lo, self.hi = self.part.bounds(self.rank)
        self.n = n_nodes
        self.rows = self.hi - self.lo
        self.backend = backend or CudaBackend()
        self.adj = adj
        self.device = device if device is not None else getattr(adj, "device", torch.device("cpu"))
        self._bufs = {}

    # -- helpers ----------------------------------------------------------------
    def slab_width(self, F: int) -> int:
        """Columns per rank: F padded to a multiple of 4*P (16-byte rows in every slab)."""
        q = 4 * self.world
        return (F + q - 1) // q * q // self.world

    def _buf(self, key, shape):
        b = self._bufs.get(key)
        if b is None or tuple(b.shape) != tuple(shape):
            b = torch.zeros(shape, dtype=torch.float32, device=self.device)
            self._bufs[key] = b
        return b

    def all_reduce_sum(self, t: torch.Tensor) -> torch.Tensor:
        if self.world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.SUM, group=self.group)
        return t

    def _all_to_all(self, out: torch.Tensor, inp: torch.Tensor) -> None:
        if self.world == 1:
            out.copy_(inp)
        else:
            dist.all_to_all_single(out, inp, group=self.group)

    # -- the two transposes -------------------------------------------------------
    def rows_to_columns(self, Y_rows: torch.Tensor, tag: str = "a") -> torch.Tensor:
        """[rows_r, F] (this rank's rows, all columns) -> [P*B, slab] (all rows,
        this rank's column slab; row index = global node id, tail rows zero)."""
        P, B = self.world, self.part.block
        F = Y_rows.size(1)
        w = self.slab_width(F)
        send = self._buf(("s", w, tag), (P, B, w))
        if F == P * w and self.rows == B:
            send.copy_(Y_rows.reshape(B, P, w).permute(1, 0, 2))
        else:
            flat = self._buf(("p", w, tag), (B, P * w))  # pad rows and columns with zeros
            flat[:self.rows, :F].copy_(Y_rows)
            send.copy_(flat.view(B, P, w).permute(1, 0, 2))
        recv = self._buf(("r", w, tag), (P, B, w))
        self._all_to_all(recv, send)
        return recv.view(P * B, w)

    def columns_to_rows(self, Z_cols: torch.Tensor, F: int, tag: str = "a") -> torch.Tensor:
        """[P*B, slab] -> [rows_r, F]: the inverse transpose (a fresh tensor)."""
        P, B = self.world, self.part.block
        w = Z_cols.size(1)
        recv = self._buf(("r2", w, tag), (P, B, w))
        self._all_to_all(recv, Z_cols.view(P, B, w))
        out = recv.permute(1, 0, 2).reshape(B, P * w)[:self.rows, :F]
        # never hand out memory of the reusable receive buffer: the next exchange with this tag overwrites it
        return out.clone() if out.untyped_storage().data_ptr() == recv.untyped_storage().data_ptr() else out.contiguous()

    def prepare_constant(self, X_local: torch.Tensor) -> torch.Tensor:
        """Column slab of a matrix that does not change between steps (the input
        features): transposed once, reused by every step."""
        return self.rows_to_columns(X_local, tag="x").clone()

    # -- aggregation --------------------------------------------------------------
    def aggregate(self, H_local: torch.Tensor, *, gathered=None, bias=None, relu=False, tag="a"):
        """rows_r of A @ H (+bias)(ReLU) for H given by its local row block.
        `gathered` is a column slab from prepare_constant()."""
        F = H_local.size(1)
        w = self.slab_width(F)
        cols = gathered if gathered is not None else self.rows_to_columns(H_local, tag)
        b_slab = None
        if bias is not None:
            bp = self._buf(("bias", w, tag), (self.world * w,))  # zero-filled once; the tail beyond F stays zero
            bp[:F].copy_(bias)
            b_slab = bp[self.rank * w:(self.rank + 1) * w]
        out = self._buf(("o", w, tag), (self.part.padded, w))
        self.backend.spmm(self.adj, cols[:self.n], bias=b_slab, relu=relu, out=out[:self.n])  # tail rows stay zero
        return self.columns_to_rows(out, F, tag)


class HybridGraph:
    """Both schemes behind one interface, chosen per aggregation by the width of
    the matrix being aggregated.

    The all-gather of the row partition delivers (P-1)/P of the matrix to every
    rank, the two transposes of feature sharding move 2 (P-1)/P^2 of it but the
    aggregation then walks ALL non-zeros on a slab of width F/P.  Narrow
    matrices (the class logits and their gradients) are cheap to gather and
    degenerate to a few columns per rank when sharded, wide ones (the hidden
    width) are the other way round; constant inputs are gathered once and cost
    no exchange at all in the row partition.  So: rows for F < wide_from and for
    pre-gathered inputs, feature slabs for F >= wide_from.  Dense layers are
    row-sharded in both, so the two can be mixed freely inside one model.
    """

    def __init__(self, rowptr, col, val, adj, n_nodes: int, *, rank: Optional[int] = None,
                 world: Optional[int] = None, group=None, backend=None, device=None, wide_from: int = 128):
        """rowptr/col/val: the global CSR (sliced into this rank's rows here);
        adj: the same matrix as the backend's object (every rank holds it whole)."""
        self.rows_graph = PartitionedGraph(rowptr, col, val, n_nodes, rank=rank, world=world, group=group,
                                           backend=backend)
        self.cols_graph = FeatureShardedGraph(adj, n_nodes, rank=rank, world=world, group=group, backend=backend,
                                              device=device if device is not None else val.device)
        g = self.rows_graph
        self.group, self.rank, self.world, self.part = g.group, g.rank, g.world, g.part
        self.lo, self.hi, self.rows, self.n = g.lo, g.hi, g.rows, g.n
        self.backend = g.backend
        self.device = g.device
        self.wide_from = int(wide_from)

    def all_reduce_sum(self, t: torch.Tensor) -> torch.Tensor:
        return self.rows_graph.all_reduce_sum(t)

    def prepare_constant(self, X_local: torch.Tensor) -> torch.Tensor:
        return self.rows_graph.prepare_constant(X_local)

    def scheme_for(self, F: int, pre_gathered: bool) -> str:
        return "rows" if (pre_gathered or F < self.wide_from or self.world == 1) else "features"

    def aggregate(self, H_local: torch.Tensor, *, gathered=None, bias=None, relu=False, tag="a"):
        if self.scheme_for(H_local.size(1), gathered is not None) == "rows":
            return self.rows_graph.aggregate(H_local, gathered=gathered, bias=bias, relu=relu, tag=tag)
        return self.cols_graph.aggregate(H_local, bias=bias, relu=relu, tag=tag)


class DistGCNConvFunction(torch.autograd.Function):
    """One layer on the local row block; collectives inside forward/backward.
    The returned weight gradient is already summed over ranks."""

    @staticmethod
    def forward(ctx, X, graph, W, apply_relu, bias, precision, X_gathered, fuse=0):
        # fuse: bit 0 = the incoming gradient is already multiplied by this layer's ReLU mask;
        #       bit 1 = X is the ReLU output of the layer below: hand dX over multiplied by (X > 0)
        be = graph.backend
        fin, fout = W.shape
        transform_first = fout < fin  # the partitioned adjacency is symmetric by contract
        width = fout
        if transform_first:
            # odd output widths run zero-padded to a multiple of 4 (see engine._padded_width)
            width = _padded_width(graph.n, fin, fout)
            H = be.gemm(X, _pad_cols(W, width), precision=precision)
            Y = graph.aggregate(H, bias=_pad_cols(bias, width) if bias is not None else None,
                                relu=bool(apply_relu), tag="f")
            if width != fout:
                Y = Y[:, :fout]
            inter = None
        else:
            AX = graph.aggregate(X, gathered=X_gathered, tag="f")
            Y = be.gemm(AX, W, bias=bias, relu=bool(apply_relu), precision=precision)
            inter = AX
        ctx.graph = graph
        ctx.width = width
        ctx.transform_first = transform_first
        ctx.apply_relu = bool(apply_relu)
        ctx.precision = precision
        ctx.has_bias = bias is not None
        ctx.has_inter = inter is not None
        ctx.fuse = int(fuse)
        ctx.save_for_backward(*([X, W, Y] + ([inter] if inter is not None else [])))
        return Y

    @staticmethod
    def backward(ctx, dY):
        graph = ctx.graph
        be = graph.backend
        saved = ctx.saved_tensors
        X, W, Y = saved[:3]
        need_dX = ctx.needs_input_grad[0]
        need_dW = ctx.needs_input_grad[2]
        dY = dY.contiguous()
        G = be.relu_backward(dY, Y) if (ctx.apply_relu and not ctx.fuse & 1) else dY
        gate_dx = bool(ctx.fuse & 2)
        dX = dW = db = None
        if ctx.has_bias and ctx.needs_input_grad[4]:
            db = graph.all_reduce_sum(G.sum(0))
        if ctx.transform_first:
            fout = W.size(1)
            S = graph.aggregate(_pad_cols(G, ctx.width), tag="b")  # A^T G = A G (symmetric)
            if need_dW:
                dW = be.gemm(X.t(), S, precision=ctx.precision)[:, :fout].contiguous()
                dW = graph.all_reduce_sum(dW)
            if need_dX:  # the gate rides in the GEMM's store (a non-contiguous input gets a pass of its own)
                fused_gate = gate_dx and X.is_contiguous()
                dX = be.gemm(S, _pad_cols(W, ctx.width).t(), precision=ctx.precision, gate=X if fused_gate else None)
                if gate_dx and not fused_gate:
                    dX = be.relu_backward(dX, X)
        else:
            AX = saved[3]
            if need_dW:
                dW = graph.all_reduce_sum(be.gemm(AX.t(), G, precision=ctx.precision))
            if need_dX:
                T = be.gemm(G, W.t(), precision=ctx.precision)
                dX = graph.aggregate(T, tag="b")
                if gate_dx:  # the aggregation ends in an exchange or an accumulate: gate in a pass of its own
                    dX = be.relu_backward(dX, X)
        return dX, None, dW, None, db, None, None, None


class DistGCN(torch.nn.Module):
    """Stack of layers as in the reference's training script
    (tests/gcn/graphcuda_impl.py:15-24) over a PartitionedGraph: ReLU on all
    layers but the last, log_softmax on top.  Every rank must construct it with
    the same RNG state so the weight replicas agree."""

    def __init__(self, dims, *, precision: Optional[str] = None, fuse_relu_backward: bool = True):
        super().__init__()
        import math
        self.precision = precision
        # as in models.GCN: a hidden layer's ReLU backward is applied where the layer above produces its input gradient
        self.fuse_relu_backward = fuse_relu_backward
        self.weights = torch.nn.ParameterList()
        for i in range(len(dims) - 1):
            s = math.sqrt(2.0 / (dims[i] + dims[i + 1]))
            w = torch.Tensor(dims[i], dims[i + 1])
            w.uniform_(-s, s)  # same initialiser as src/graphcuda/python/gcn.py:43-45
            self.weights.append(torch.nn.Parameter(w))

    def forward(self, X_local, graph, X_gathered=None, log_softmax: bool = True, return_hidden: bool = False):
        h = X_local
        hidden = [h]
        last = len(self.weights) - 1
        for i, W in enumerate(self.weights):
            fuse = 0
            if self.fuse_relu_backward:
                fuse = (1 if i < last else 0) | (2 if i > 0 else 0)  # every layer but the last has a ReLU
            h = DistGCNConvFunction.apply(h, graph, W, i < last, None, self.precision,
                                          X_gathered if i == 0 else None, fuse)
            hidden.append(h)
        out = torch.log_softmax(h, dim=1) if log_softmax else h
        return (out, hidden) if return_hidden else out

"""Adjacency handling: CSR (int32) device storage, its SpMM plan, conversion
from the layouts the reference API is called with, and GCN normalisation.

The reference's layer takes the normalised adjacency as a torch tensor: sparse
COO with int64 indices in the shipped extension
(src/graphcuda/cuda/spmm_cusparse.cu:5-6,33-41), dense in its ATen twin and in
the README (src/graphcuda/cpp/gcn.cpp:10).  Here every sparse form is turned
once into an int32 CSR plus a long-row plan and cached on the tensor's
identity, so a training loop that passes the same ``adj`` every step pays the
conversion once.
"""
from __future__ import annotations

import threading
import weakref
from typing import Optional

import torch

from . import _lib
from .ops import _require, _stream, arena, EPI_RELU, EPI_ACCUMULATE


class SpmmPlan:
    """A built processing plan: device buffer and the counts it was built with."""

    __slots__ = ("buf", "n_pieces", "n_slots", "n_cut", "panel_cols")

    def __init__(self, buf, n_pieces, n_slots, n_cut, panel_cols):
        self.buf, self.n_pieces, self.n_slots, self.n_cut, self.panel_cols = buf, n_pieces, n_slots, n_cut, panel_cols


class CSRAdjacency:
    """int32 CSR on one device, with the SpMM plan and the symmetry verdict."""

    def __init__(self, rowptr: torch.Tensor, col: torch.Tensor, val: torch.Tensor, shape, *,
                 symmetric: Optional[bool] = None, build_plan: bool = True):
        _require(rowptr.is_cuda and col.is_cuda and val.is_cuda, "CSR arrays must be CUDA tensors")
        _require(rowptr.dtype == torch.int32 and col.dtype == torch.int32, "rowptr/col must be int32")
        _require(val.dtype == torch.float32, "CSR values must be float32")
        _require(rowptr.numel() == shape[0] + 1, "rowptr must have M+1 entries")
        _require(col.numel() == val.numel(), "col and val must have the same length")
        self.rowptr = rowptr.contiguous()
        self.col = col.contiguous()
        self.val = val.contiguous()
        self.shape = (int(shape[0]), int(shape[1]))
        self.nnz = int(col.numel())
        self.device = rowptr.device
        self._symmetric = symmetric
        self.use_plan = bool(build_plan)
        self.segment = None  # longest piece in non-zeros; None: gc_spmm_default_segment(nnz)
        self.perm = None  # set by normalized_adjacency(reorder=...): perm[new] = old vertex id
        self.inv_perm = None
        self._plans = {}  # panel_cols -> SpmmPlan

    def plan_for(self, F: int, panel_cols: Optional[int] = None):
        """The processing plan for feature width F (built on first use and kept):
        (plan buffer, n_pieces, n_slots, n_cut)."""
        L = _lib.lib()
        M, K = self.shape
        if panel_cols is None:
            panel_cols = int(L.gc_spmm_default_panel_cols(K, max(F, 1)))
        hit = self._plans.get(panel_cols)
        if hit is not None:
            return hit
        seg = int(L.gc_spmm_default_segment(self.nnz)) if self.segment is None else int(self.segment)
        dev = self.device
        with torch.cuda.device(dev):
            s = _stream(dev)
            counts = torch.zeros(3, dtype=torch.int64, device=dev)
            wsb = L.gc_spmm_plan_workspace_bytes(M, 0)
            ws = torch.empty(wsb, dtype=torch.uint8, device=dev)
            _lib.check(L.gc_spmm_plan_count(self.rowptr.data_ptr(), self.col.data_ptr(), M, K, panel_cols, seg,
                                            counts.data_ptr(), ws.data_ptr(), wsb, s), "gc_spmm_plan_count")
            n_pieces, n_slots, n_cut = (int(x) for x in counts.tolist())  # the one host read of plan building
            del ws
            pbytes = L.gc_spmm_plan_bytes(n_pieces, n_cut)
            plan = torch.empty(pbytes, dtype=torch.uint8, device=dev)
            wsb = L.gc_spmm_plan_workspace_bytes(M, n_pieces)
            ws = torch.empty(wsb, dtype=torch.uint8, device=dev)
            _lib.check(L.gc_spmm_plan_build(self.rowptr.data_ptr(), self.col.data_ptr(), M, K, panel_cols, seg,
                                            n_pieces, n_slots, n_cut, plan.data_ptr(), pbytes, ws.data_ptr(), wsb,
                                            s), "gc_spmm_plan_build")
            torch.cuda.current_stream(dev).synchronize()  # ws is released below
        entry = SpmmPlan(plan, n_pieces, n_slots, n_cut, panel_cols)
        self._plans[panel_cols] = entry
        return entry

    @property
    def symmetric(self) -> bool:
        """Whether A == A^T bit for bit (decides if the layer may aggregate on
        the output side; the reference multiplies by A in the backward pass,
        never A^T: src/graphcuda/cuda/gcn.cu:49)."""
        if self._symmetric is None:
            if self.shape[0] != self.shape[1]:
                self._symmetric = False
            else:
                out = torch.empty(1, dtype=torch.int32, device=self.device)
                with torch.cuda.device(self.device):
                    st = _lib.lib().gc_csr_is_symmetric(self.rowptr.data_ptr(), self.col.data_ptr(),
                                                        self.val.data_ptr(), self.shape[0], out.data_ptr(),
                                                        _stream(self.device))
                _lib.check(st, "gc_csr_is_symmetric")
                self._symmetric = bool(out.item())
        return self._symmetric

    def plan_counts(self, F: int = 256, panel_cols: Optional[int] = None):
        """(pieces, scratch slots, cut rows) of the plan for width F -- for tests and reports."""
        p = self.plan_for(F, panel_cols)
        return p.n_pieces, p.n_slots, p.n_cut

    # -- products -----------------------------------------------------------
    def matmul(self, H: torch.Tensor, *, bias: Optional[torch.Tensor] = None, relu: bool = False,
               want_mask: bool = False, accumulate_into: Optional[torch.Tensor] = None,
               out: Optional[torch.Tensor] = None, panel_cols: Optional[int] = None,
               gate: Optional[torch.Tensor] = None):
        """Y = A @ H (+bias)(ReLU).  Returns Y or (Y, mask).  gate (contiguous,
        shape of Y): Y is multiplied by (gate > 0) in the store.  H may be a bfloat16 matrix as ops.to_bf16 lays
        it out (the reduced-precision tier: half the gathered bytes, fp32 sums and output)."""
        _require(H.dim() == 2, "B must be 2D")
        _require(H.size(0) == self.shape[1], "A.cols must match B.rows")
        _require(H.is_cuda and H.device == self.device, "A and B must be CUDA tensors on the same device")
        h16 = H.dtype == torch.bfloat16
        _require(H.dtype == torch.float32 or h16, "B must be float32 (or bfloat16 for the reduced-precision tier)")
        if h16:
            _require(H.stride(1) == 1 and H.size(1) % 8 == 0 and (H.size(0) <= 1 or H.stride(0) % 8 == 0)
                     and H.data_ptr() % 16 == 0, "a bfloat16 B needs a width and row pitch that are multiples of 8")
        elif H.stride(1) != 1 or (H.size(0) > 1 and H.stride(0) < H.size(1)):
            H = H.contiguous()
        M, K = self.shape
        F = H.size(1)
        dev = self.device
        epi = EPI_RELU if relu else 0
        if accumulate_into is not None:
            out = accumulate_into
            epi |= EPI_ACCUMULATE
        if out is None:
            out = torch.empty((M, F), dtype=torch.float32, device=dev)
        # `out` may be a column slice of a wider row-major matrix (unit column stride)
        _require(tuple(out.shape) == (M, F) and out.dtype == torch.float32 and out.stride(1) == 1
                 and (M <= 1 or out.stride(0) >= F), "out has the wrong shape, dtype or layout")
        ldy = out.stride(0) if M > 1 else max(F, 1)
        _require(not want_mask or ldy == F, "a mask needs a contiguous output")
        mask = torch.empty((M, F), dtype=torch.float32, device=dev) if want_mask else None
        if bias is not None:
            _require(bias.is_cuda and bias.dtype == torch.float32 and bias.numel() == F, "bias must be float32 [F]")
            bias = bias.contiguous()
        if gate is not None:
            _require(gate.is_cuda and gate.dtype == torch.float32 and tuple(gate.shape) == (M, F)
                     and gate.is_contiguous() and ldy == F, "gate must be a contiguous float32 tensor of Y's shape")
        if M == 0 or F == 0:
            return (out, mask) if want_mask else out
        L = _lib.lib()
        with torch.cuda.device(dev):
            plan = self.plan_for(F, panel_cols) if self.use_plan else None
            scratch = None
            if plan is not None and plan.n_cut > 0:
                scratch = arena.get("spmm", L.gc_spmm_scratch_bytes(plan.n_slots, F), dev)
            ldh = H.stride(0) if H.size(0) > 1 else max(F, 1)
            fn = L.gc_spmm_csr_bf16h_f32 if h16 else L.gc_spmm_csr_f32
            st = fn(self.rowptr.data_ptr(), self.col.data_ptr(), self.val.data_ptr(), M, K, F,
                                   H.data_ptr(), ldh, bias.data_ptr() if bias is not None else None, epi,
                                   out.data_ptr(), ldy, mask.data_ptr() if mask is not None else None,
                                   gate.data_ptr() if gate is not None else None,
                                   plan.buf.data_ptr() if plan is not None else None,
                                   plan.n_pieces if plan is not None else 0, plan.n_slots if plan is not None else 0,
                                   plan.n_cut if plan is not None else 0,
                                   scratch.data_ptr() if scratch is not None else None,
                                   scratch.numel() if scratch is not None else 0, _stream(dev))
        _lib.check(st, "gc_spmm_csr_f32")
        return (out, mask) if want_mask else out

    def matmul_into_blocks(self, H: torch.Tensor, blocks, block_rows: int, *, bias: Optional[torch.Tensor] = None,
                           relu: bool = False, panel_cols: Optional[int] = None) -> None:
        """A @ H (+bias)(ReLU) with row i stored in blocks[i // block_rows] at row i % block_rows.

        blocks: float32 matrices of F columns, unit column stride and one common row stride; they may be views
        of other GPUs' buffers (peer-mapped memory): the aggregation's stores then deliver every owner's rows
        (gc_spmm_csr_f32_blocks).  The caller orders the use of those buffers across GPUs."""
        import ctypes
        _require(H.dim() == 2 and H.size(0) == self.shape[1] and H.is_cuda and H.device == self.device
                 and H.dtype == torch.float32, "B must be a float32 CUDA matrix with A.cols rows")
        if H.stride(1) != 1 or (H.size(0) > 1 and H.stride(0) < H.size(1)):
            H = H.contiguous()
        M, K = self.shape
        F = H.size(1)
        L = _lib.lib()
        _require(1 <= len(blocks) <= _lib.SPMM_MAX_BLOCKS and len(blocks) * block_rows >= M,
                 "blocks must cover the rows of A")
        ld = blocks[0].stride(0)
        for b in blocks:
            _require(b.dtype == torch.float32 and b.dim() == 2 and b.size(1) == F and b.stride(1) == 1
                     and b.stride(0) == ld and ld >= F, "blocks must be float32 [rows, F] views with one row stride")
        for i, b in enumerate(blocks):
            _require(b.size(0) >= min(block_rows, M - i * block_rows), "a block is shorter than its rows")
        if bias is not None:
            _require(bias.is_cuda and bias.dtype == torch.float32 and bias.numel() == F, "bias must be float32 [F]")
            bias = bias.contiguous()
        if M == 0 or F == 0:
            return
        ptrs = (ctypes.c_void_p * len(blocks))(*[b.data_ptr() for b in blocks])
        dev = self.device
        with torch.cuda.device(dev):
            plan = self.plan_for(F, panel_cols) if self.use_plan else None
            scratch = None
            if plan is not None and plan.n_cut > 0:
                scratch = arena.get("spmm", L.gc_spmm_scratch_bytes(plan.n_slots, F), dev)
            ldh = H.stride(0) if H.size(0) > 1 else max(F, 1)
            st = L.gc_spmm_csr_f32_blocks(self.rowptr.data_ptr(), self.col.data_ptr(), self.val.data_ptr(), M, K, F,
                                          H.data_ptr(), ldh, bias.data_ptr() if bias is not None else None,
                                          EPI_RELU if relu else 0, ptrs, len(blocks), block_rows, ld,
                                          plan.buf.data_ptr() if plan is not None else None,
                                          plan.n_pieces if plan is not None else 0,
                                          plan.n_slots if plan is not None else 0,
                                          plan.n_cut if plan is not None else 0,
                                          scratch.data_ptr() if scratch is not None else None,
                                          scratch.numel() if scratch is not None else 0, _stream(dev))
        _lib.check(st, "gc_spmm_csr_f32_blocks")

    def to_sparse_coo(self) -> torch.Tensor:
        counts = (self.rowptr[1:] - self.rowptr[:-1]).long()
        rows = torch.repeat_interleave(torch.arange(self.shape[0], device=self.device), counts)
        idx = torch.stack([rows, self.col.long()])
        return torch.sparse_coo_tensor(idx, self.val, self.shape, device=self.device, is_coalesced=True)


class DenseAdjacency:
    """A dense normalised adjacency (the README / ATen-twin calling convention,
    src/graphcuda/cpp/gcn.cpp:10).  Products run on the dense GEMM path."""

    def __init__(self, A: torch.Tensor, symmetric: Optional[bool] = None):
        _require(A.dim() == 2 and A.is_cuda and A.dtype == torch.float32, "dense adjacency must be a float32 CUDA matrix")
        self.A = A
        self.shape = tuple(A.shape)
        self.device = A.device
        self._symmetric = symmetric

    @property
    def symmetric(self) -> bool:
        """A == A^T bit for bit.  The verdict is remembered on the tensor itself (with the version it was taken
        at), so wrapping the same matrix again -- every layer call does -- does not repeat the comparison."""
        if self._symmetric is None:
            memo = getattr(self.A, "_gc_symmetric", None)
            if memo is not None and memo[0] == self.A._version:
                self._symmetric = memo[1]
            else:
                self._symmetric = self.shape[0] == self.shape[1] and bool(torch.equal(self.A, self.A.t()))
                try:
                    self.A._gc_symmetric = (self.A._version, self._symmetric)
                except Exception:
                    pass
        return self._symmetric

    def matmul(self, H: torch.Tensor, *, bias=None, relu=False, want_mask=False, accumulate_into=None, out=None,
               precision=None, gate=None):
        from .ops import gemm, gemm_bf16_operands, get_default_precision, to_bf16
        _require(accumulate_into is None, "accumulate is not available on the dense path")
        if (precision or get_default_precision()) == "bf16" and not want_mask:
            # the adjacency does not change between calls: its bf16 copy is made once (per version of the tensor)
            # (remembered on the tensor itself, like the symmetry verdict, so that it lives exactly as long as A)
            memo = getattr(self.A, "_gc_bf16", None)
            if memo is None or memo[0] != self.A._version:
                memo = (self.A._version, to_bf16(self.A))
                try:
                    self.A._gc_bf16 = memo
                except Exception:
                    pass
            return gemm_bf16_operands(memo[1], to_bf16(H, transpose=True), bias=bias, relu=relu, out=out, gate=gate)
        return gemm(self.A, H, bias=bias, relu=relu, want_mask=want_mask, precision=precision, out=out, gate=gate)


# ---------------------------------------------------------------- conversion
def csr_from_sorted_coo(rows: torch.Tensor, cols: torch.Tensor, vals: torch.Tensor, shape, *,
                        symmetric: Optional[bool] = None) -> CSRAdjacency:
    """CSR from a *coalesced* COO triple (rows ascending, then cols; int64)."""
    dev = rows.device
    M = int(shape[0])
    nnz = int(rows.numel())
    _require(nnz < 2**31 - 1 and M < 2**31 - 1 and int(shape[1]) < 2**31 - 1, "matrix too large for int32 CSR")
    L = _lib.lib()
    rowptr = torch.empty(M + 1, dtype=torch.int32, device=dev)
    col32 = torch.empty(nnz, dtype=torch.int32, device=dev)
    rows = rows.contiguous()
    cols = cols.contiguous()
    with torch.cuda.device(dev):
        s = _stream(dev)
        _lib.check(L.gc_coo_rows_to_rowptr(rows.data_ptr(), nnz, M, rowptr.data_ptr(), s), "gc_coo_rows_to_rowptr")
        _lib.check(L.gc_narrow_i64_i32(cols.data_ptr(), col32.data_ptr(), nnz, s), "gc_narrow_i64_i32")
    return CSRAdjacency(rowptr, col32, vals.contiguous(), shape, symmetric=symmetric)


_cache_lock = threading.Lock()
_cache: dict = {}


def _cache_key(t: torch.Tensor):
    if t.layout == torch.sparse_coo:
        v = t._values()
        i = t._indices()
        return ("coo", v.data_ptr(), i.data_ptr(), v._version, i._version, tuple(t.shape), t._nnz(), t.is_coalesced())
    if t.layout == torch.sparse_csr:
        v = t.values()
        return ("csr", v.data_ptr(), t.crow_indices().data_ptr(), t.col_indices().data_ptr(), v._version,
                tuple(t.shape))
    raise RuntimeError(f"unsupported adjacency layout {t.layout}")


def as_adjacency(adjm, *, symmetric: Optional[bool] = None):
    """CSRAdjacency / DenseAdjacency for whatever the caller passed as ``adjm``.

    Accepts a CSRAdjacency, a (rowptr, col, val[, shape]) tuple, or a torch
    tensor with strided, sparse_coo or sparse_csr layout.  Results for tensors
    are cached on (storage pointer, version counter, shape); the cache holds a
    weak reference to the tensor and drops the entry when the tensor dies.
    """
    if isinstance(adjm, (CSRAdjacency, DenseAdjacency)):
        return adjm
    if isinstance(adjm, (tuple, list)):
        rowptr, col, val = adjm[:3]
        shape = adjm[3] if len(adjm) > 3 else (rowptr.numel() - 1, rowptr.numel() - 1)
        return CSRAdjacency(rowptr, col, val, shape, symmetric=symmetric)
    _require(isinstance(adjm, torch.Tensor), "adjacency must be a tensor, a CSR tuple or a CSRAdjacency")
    _require(adjm.dim() == 2, "A must be 2D")
    _require(adjm.is_cuda, "A and B must be CUDA tensors")
    _require(adjm.dtype == torch.float32, "A values must be float32")
    if adjm.layout == torch.strided:
        # not cached: the wrapper holds the matrix itself, so a cache entry would pin an N x N buffer for good
        return DenseAdjacency(adjm, symmetric=symmetric)
    key = _cache_key(adjm)
    with _cache_lock:
        hit = _cache.get(key)
        if hit is not None and hit[0]() is not None:
            return hit[1]
    if adjm.layout == torch.sparse_coo:
        t = adjm if adjm.is_coalesced() else adjm.coalesce()
        idx = t._indices()
        _require(idx.dtype == torch.int64, "A indices must be int64")
        adj = csr_from_sorted_coo(idx[0], idx[1], t._values(), t.shape, symmetric=symmetric)
    elif adjm.layout == torch.sparse_csr:
        adj = CSRAdjacency(adjm.crow_indices().to(torch.int32), adjm.col_indices().to(torch.int32), adjm.values(),
                           adjm.shape, symmetric=symmetric)
    else:
        raise RuntimeError(f"unsupported adjacency layout {adjm.layout}")
    with _cache_lock:
        if len(_cache) > 64:
            for k in [k for k, v in _cache.items() if v[0]() is None]:
                _cache.pop(k, None)
        try:
            _cache[key] = (weakref.ref(adjm), adj)
        except TypeError:
            pass
    return adj


def clear_cache() -> None:
    with _cache_lock:
        _cache.clear()


# ---------------------------------------------------------------- normalisation
def gcn_norm(edge_index: torch.Tensor, num_nodes: int) -> torch.Tensor:
    """Symmetric GCN edge weights deg^-1/2[row] * deg^-1/2[col] for an edge list
    that already holds the self-loops (deg counted on the target index), as
    torch_geometric's gcn_norm computes them for unit weights at the
    reference's call site tests/gcn/graphcuda_impl.py:28.  Bit-exact against
    the torch CPU formula."""
    _require(edge_index.is_cuda and edge_index.dtype == torch.int64 and edge_index.dim() == 2
             and edge_index.size(0) == 2, "edge_index must be a CUDA int64 [2, E] tensor")
    dev = edge_index.device
    E = edge_index.size(1)
    row = edge_index[0].contiguous()
    col = edge_index[1].contiguous()
    w = torch.empty(E, dtype=torch.float32, device=dev)
    deg = torch.empty(max(num_nodes, 1), dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        st = _lib.lib().gc_gcn_norm_f32(row.data_ptr(), col.data_ptr(), E, num_nodes, deg.data_ptr(), w.data_ptr(),
                                        _stream(dev))
    _lib.check(st, "gc_gcn_norm_f32")
    return w


def degree_order(edge_index: torch.Tensor, num_nodes: int):
    """Vertex relabelling by decreasing degree (ties: lower old id first).

    Returns (perm, inv): perm[new] = old, inv[old] = new.  The degree is the
    number of edges whose target (edge_index[1]) is the vertex, as gcn_norm
    counts it.  In the relabelled graph the heavy vertices are the low ids, so
    the rows of a feature matrix that most gathers hit are contiguous."""
    _require(edge_index.dtype == torch.int64 and edge_index.dim() == 2 and edge_index.size(0) == 2,
             "edge_index must be an int64 [2, E] tensor")
    deg = torch.bincount(edge_index[1], minlength=num_nodes)
    perm = torch.argsort(deg, descending=True, stable=True)
    inv = torch.empty_like(perm)
    inv[perm] = torch.arange(num_nodes, device=perm.device, dtype=perm.dtype)
    return perm, inv


def normalized_adjacency(edge_index: torch.Tensor, num_nodes: int, *, add_self_loops: bool = True,
                         symmetric: Optional[bool] = None, reorder: Optional[str] = None) -> CSRAdjacency:
    """Edge list -> (+self-loops) -> symmetric normalisation -> coalesced int32
    CSR, the whole preprocessing of tests/gcn/graphcuda_impl.py:27-38 on the
    GPU.  The (row, col) ordering uses torch.sort on the device; degree,
    normalisation, de-duplication and CSR assembly are this library's kernels.

    reorder="degree": the vertices are first relabelled by decreasing degree
    (degree_order); the result is the adjacency of the relabelled graph and
    carries ``perm`` (perm[new] = old) and ``inv_perm``.  Feature and label
    rows must be permuted the same way (``X[adj.perm]``); outputs come back in
    the new order (``Y_old = Y[adj.inv_perm]``).
    """
    _require(edge_index.is_cuda and edge_index.dtype == torch.int64, "edge_index must be a CUDA int64 tensor")
    _require(reorder in (None, "degree"), "reorder must be None or 'degree'")
    if reorder == "degree":
        perm, inv = degree_order(edge_index, num_nodes)  # self-loops add one to every degree: same order
        adj = normalized_adjacency(inv[edge_index], num_nodes, add_self_loops=add_self_loops, symmetric=symmetric)
        adj.perm, adj.inv_perm = perm, inv
        return adj
    dev = edge_index.device
    if add_self_loops:
        loops = torch.arange(num_nodes, device=dev, dtype=torch.int64)
        edge_index = torch.cat([edge_index, torch.stack([loops, loops])], dim=1)
    w = gcn_norm(edge_index, num_nodes)
    key = edge_index[0] * num_nodes + edge_index[1]
    key, order = torch.sort(key, stable=True)
    row = edge_index[0][order].contiguous()
    col = edge_index[1][order].contiguous()
    w = w[order].contiguous()
    E = row.numel()
    L = _lib.lib()
    head = torch.empty(max(E, 1), dtype=torch.int32, device=dev)
    nnz_dev = torch.empty(1, dtype=torch.int64, device=dev)
    wsb = L.gc_csr_build_workspace_bytes(E)
    ws = torch.empty(wsb, dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        s = _stream(dev)
        _lib.check(L.gc_csr_count_unique(row.data_ptr(), col.data_ptr(), E, head.data_ptr(), nnz_dev.data_ptr(),
                                         ws.data_ptr(), wsb, s), "gc_csr_count_unique")
        nnz = int(nnz_dev.item())
        rowptr = torch.empty(num_nodes + 1, dtype=torch.int32, device=dev)
        ccol = torch.empty(nnz, dtype=torch.int32, device=dev)
        cval = torch.empty(nnz, dtype=torch.float32, device=dev)
        _lib.check(L.gc_csr_fill(row.data_ptr(), col.data_ptr(), w.data_ptr(), E, num_nodes, head.data_ptr(),
                                 rowptr.data_ptr(), ccol.data_ptr(), cval.data_ptr(), s), "gc_csr_fill")
    return CSRAdjacency(rowptr, ccol, cval, (num_nodes, num_nodes), symmetric=symmetric)

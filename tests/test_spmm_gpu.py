"""CSR aggregation kernel vs the oracle (torch.sparse.mm on CPU), through the
C ABI (graphcuda_b200.adjacency -> gc_spmm_csr_f32)."""
import os

import numpy as np
import pytest
import torch

from oracle import gcn_oracle as O
from tests.helpers import random_csr, to_gpu_csr

pytestmark = pytest.mark.gpu

TOL = 1e-4  # relative Frobenius / max, fp32 path


@pytest.mark.parametrize("F", [1, 3, 4, 7, 8, 12, 16, 20, 28, 32, 36, 47, 48, 64, 100, 128, 200, 256, 260, 700])
def test_feature_widths(cuda, F):
    A = random_csr(500, 400, 9.0, seed=F, empty_rows=(0, 13, 499))
    H = torch.randn(400, F, generator=torch.Generator().manual_seed(F + 1))
    ref = O.spmm(A, H)
    adj = to_gpu_csr(A, cuda)
    out = adj.matmul(H.to(cuda))
    assert O.rel_fro(out, ref) < TOL and O.rel_max(out, ref) < TOL
    assert float(out[0].abs().max()) == 0.0 and float(out[499].abs().max()) == 0.0


@pytest.mark.parametrize("F", [16, 100, 256])
def test_long_rows_are_cut_into_pieces(cuda, F):
    # rows of about 1500, 2048, 2049 and 9000 non-zeros, cut every `seg` non-zeros (one panel: H fits the L2)
    A = random_csr(3000, 12000, 4.0, seed=3, long_rows=((7, 1500), (100, 2048), (101, 2049), (2999, 9000)))
    H = torch.randn(12000, F, generator=torch.Generator().manual_seed(9))
    ref = O.spmm(A, H)
    adj = to_gpu_csr(A, cuda)
    from graphcuda_b200 import _lib
    seg = int(_lib.lib().gc_spmm_default_segment(adj.nnz))
    assert seg == 128  # a small matrix gets short pieces
    deg = (adj.rowptr[1:] - adj.rowptr[:-1]).cpu()
    pieces_per_row = torch.clamp((deg + seg - 1) // seg, min=1)
    n_pieces, n_slots, n_cut = adj.plan_counts(F)
    assert n_pieces == int(pieces_per_row.sum())
    assert n_cut == int((pieces_per_row > 1).sum()) and n_cut >= 4
    assert n_slots == int(pieces_per_row[pieces_per_row > 1].sum())
    out = adj.matmul(H.to(cuda))
    assert O.rel_fro(out, ref) < TOL and O.rel_max(out, ref) < TOL
    # the longest allowed pieces give the same product
    long_seg = to_gpu_csr(A, cuda)
    long_seg.segment = 2048
    assert long_seg.plan_counts(F)[0] < n_pieces
    assert O.rel_fro(long_seg.matmul(H.to(cuda)), ref) < TOL
    # same result without a plan (every row one piece, natural order)
    from graphcuda_b200 import CSRAdjacency
    plain = CSRAdjacency(adj.rowptr, adj.col, adj.val, adj.shape, build_plan=False)
    out2 = plain.matmul(H.to(cuda))
    assert O.rel_fro(out2, ref) < TOL


@pytest.mark.parametrize("F,panel", [(64, 1024), (256, 4096), (100, 2048), (7, 1024)])
def test_column_panels(cuda, F, panel):
    """Rows above the panel threshold are cut at column-panel boundaries; narrow
    panels force many pieces per row, empty panels and the length cut inside a panel."""
    A = random_csr(5000, 20000, 8.0, seed=12, long_rows=((0, 129), (9, 500), (77, 6000), (4999, 15000)),
                   empty_rows=(3, 4))
    H = torch.randn(20000, F, generator=torch.Generator().manual_seed(2))
    ref = O.spmm(A, H)
    adj = to_gpu_csr(A, cuda)
    n_pieces, n_slots, n_cut = adj.plan_counts(F, panel_cols=panel)
    deg = (adj.rowptr[1:] - adj.rowptr[:-1]).cpu()
    assert n_cut >= int((deg > 128).sum())  # every row above the threshold spans several panels here
    assert n_pieces > 5000 and n_slots >= 2 * n_cut
    b = torch.randn(F, generator=torch.Generator().manual_seed(3))
    pre = ref + b
    out = adj.matmul(H.to(cuda), bias=b.to(cuda), relu=True, panel_cols=panel)
    assert O.rel_fro(out, pre * (pre > 0)) < TOL
    again = adj.matmul(H.to(cuda), bias=b.to(cuda), relu=True, panel_cols=panel)
    assert torch.equal(out, again)
    # an empty row yields relu(bias)
    assert torch.allclose(out[3].cpu(), torch.relu(b))


def test_bias_relu_mask_accumulate(cuda):
    A = random_csr(800, 800, 12.0, seed=5, long_rows=((3, 3000),))
    g = torch.Generator().manual_seed(6)
    H = torch.randn(800, 64, generator=g)
    b = torch.randn(64, generator=g)
    pre = O.spmm(A, H) + b
    adj = to_gpu_csr(A, cuda)
    Y, mask = adj.matmul(H.to(cuda), bias=b.to(cuda), relu=True, want_mask=True)
    assert O.rel_fro(Y, pre * (pre > 0)) < TOL
    # the mask may differ only where the pre-activation is within rounding of zero
    diff = (mask.cpu() != (pre > 0).float())
    assert float(pre[diff].abs().max() if diff.any() else 0.0) < 1e-5
    base = torch.randn(800, 64, generator=g)
    acc = base.to(cuda).clone()
    adj.matmul(H.to(cuda), accumulate_into=acc)
    assert O.rel_fro(acc, base + O.spmm(A, H)) < TOL


def test_empty_matrix_and_zero_nnz(cuda):
    from graphcuda_b200 import CSRAdjacency
    rowptr = torch.zeros(11, dtype=torch.int32, device=cuda)
    col = torch.empty(0, dtype=torch.int32, device=cuda)
    val = torch.empty(0, dtype=torch.float32, device=cuda)
    adj = CSRAdjacency(rowptr, col, val, (10, 6))
    out = adj.matmul(torch.randn(6, 5, device=cuda))
    assert out.shape == (10, 5) and float(out.abs().max()) == 0.0


def test_deterministic_run_to_run(cuda):
    A = random_csr(4000, 4000, 20.0, seed=8, long_rows=((1, 5000), (2, 2500)))
    H = torch.randn(4000, 128, generator=torch.Generator().manual_seed(1)).to(cuda)
    adj = to_gpu_csr(A, cuda)
    a = adj.matmul(H)
    b = adj.matmul(H)
    assert torch.equal(a, b)


def test_inf_in_unrelated_row_does_not_leak(cuda):
    A = random_csr(64, 64, 3.0, seed=2)
    dense = A.to_dense()
    dense[:, 0] = 0  # nobody references row 0 of H
    A = dense.to_sparse().coalesce()
    H = torch.randn(64, 32)
    H[0] = float("inf")
    out = to_gpu_csr(A, cuda).matmul(H.to(cuda))
    assert torch.isfinite(out).all()


def test_spmm_cusparse_api(cuda):
    """graphcuda.spmm_cusparse(sparseA, B): COO int64 input like the reference
    (spmm_cusparse.cu:5-12,33-41) and the same error behaviour."""
    import graphcuda
    A = random_csr(300, 200, 6.0, seed=11)
    B = torch.randn(200, 33, generator=torch.Generator().manual_seed(2))
    out = graphcuda.spmm_cusparse(A.to(cuda), B.to(cuda))
    assert O.rel_fro(out, O.spmm(A, B)) < TOL
    # uncoalesced input is coalesced first (spmm_cusparse.cu:18)
    idx = torch.cat([A.indices(), A.indices()[:, :50]], dim=1)
    val = torch.cat([A.values(), A.values()[:50]])
    dup = torch.sparse_coo_tensor(idx, val, A.shape).to(cuda)
    out2 = graphcuda.spmm_cusparse(dup, B.to(cuda))
    assert O.rel_fro(out2, O.spmm(dup.cpu().coalesce(), B)) < TOL
    with pytest.raises(RuntimeError):
        graphcuda.spmm_cusparse(A, B)  # CPU tensors are rejected
    with pytest.raises(RuntimeError):
        graphcuda.spmm_cusparse(A.to_dense().to(cuda), B.to(cuda))  # dense A is rejected by this operator
    with pytest.raises(RuntimeError):
        graphcuda.spmm_cusparse(A.to(cuda), torch.randn(201, 4, device=cuda))
    # CSR overloads
    out3 = graphcuda.spmm_cusparse(A.to_sparse_csr().to(cuda), B.to(cuda))
    assert O.rel_fro(out3, O.spmm(A, B)) < TOL


def test_golden_sparse_layer_aggregation(cuda, golden_dir):
    g = np.load(os.path.join(golden_dir, "layer_sparse.npz"))
    n = int(g["n"])
    A = torch.sparse_coo_tensor(torch.stack([torch.from_numpy(g["rows"]), torch.from_numpy(g["cols"])]),
                                torch.from_numpy(g["vals"]), (n, n)).coalesce()
    X, W = torch.from_numpy(g["X"]), torch.from_numpy(g["W"])
    adj = to_gpu_csr(A, cuda)
    AX = adj.matmul(X.to(cuda))
    assert O.rel_fro(AX.cpu() @ W, torch.from_numpy(g["Y0"])) < TOL


def test_full_size_arxiv_like_graph(cuda):
    """169,343 nodes / 1,166,243 undirected R-MAT edges, F = 128 and 256: direct
    comparison with the CPU oracle plus the row-sum identity A 1 = rowsum(A)."""
    from graphcuda_b200 import synth
    from tests.helpers import sym_norm_graph
    cfg = synth.CONFIGS["rmat_arxiv"]
    n = cfg["nodes"]
    e = synth.rmat_edges(cfg["scale"], n, cfg["edges"], cfg["seed"])
    A = sym_norm_graph(e, n)
    assert A._nnz() == 2 * cfg["edges"] + n
    adj = to_gpu_csr(A, cuda)
    assert adj.plan_counts(128)[2] > 0  # the heavy tail exists: some rows are cut
    for F in (128, 256):
        H = synth.normal_features(n, F, seed=F)
        out = adj.matmul(H.to(cuda))
        ref = O.spmm(A, H)
        assert O.rel_fro(out, ref) < TOL
        assert O.rel_max(out, ref) < TOL
    ones = torch.ones(n, 4, device=cuda)
    rs = adj.matmul(ones)[:, 0].cpu()
    ref_rs = torch.sparse.sum(A, dim=1).to_dense()
    assert O.rel_max(rs, ref_rs) < 1e-4


def test_understated_scratch_is_refused_or_flagged_never_truncated_silently(cuda):
    """C callers pass the plan's counts themselves.  Too little scratch for the slots they declare is refused
    before any launch; slots they did not declare are skipped by the kernels and leave a sticky error word in
    the plan that gc_spmm_plan_check reports.  Neither case writes outside the caller's buffers."""
    from graphcuda_b200 import _lib
    L = _lib.lib()
    A = random_csr(400, 6000, 3.0, seed=21, long_rows=((2, 5000), (9, 3000)))
    adj = to_gpu_csr(A, cuda)
    F = 32
    plan = adj.plan_for(F)
    assert plan.n_cut >= 2 and plan.n_slots >= 4
    H = torch.randn(6000, F, device=cuda)
    Y = torch.zeros(400, F, device=cuda)
    s = torch.cuda.current_stream().cuda_stream
    need = L.gc_spmm_scratch_bytes(plan.n_slots, F)
    scratch = torch.zeros(need, dtype=torch.uint8, device=cuda)

    def call(n_slots, nbytes):
        return L.gc_spmm_csr_f32(adj.rowptr.data_ptr(), adj.col.data_ptr(), adj.val.data_ptr(), 400, 6000, F,
                                 H.data_ptr(), F, None, 0, Y.data_ptr(), F, None, None, plan.buf.data_ptr(),
                                 plan.n_pieces, n_slots, plan.n_cut, scratch.data_ptr(), nbytes, s)

    assert call(plan.n_slots, need - 16) == -4 and b"partial-sum rows" in L.gc_last_error()
    assert L.gc_spmm_plan_check(plan.buf.data_ptr(), plan.n_pieces, plan.n_slots, plan.n_cut, s) == 0
    # the right counts: the product, and the plan stays clean
    assert call(plan.n_slots, need) == 0
    assert O.rel_fro(Y, O.spmm(A, H.cpu())) < TOL
    assert L.gc_spmm_plan_check(plan.buf.data_ptr(), plan.n_pieces, plan.n_slots, plan.n_cut, s) == 0
    # counts that are not the plan's own are reported by the check ...
    assert L.gc_spmm_plan_check(plan.buf.data_ptr(), plan.n_pieces, plan.n_slots - 1, plan.n_cut, s) == -1
    # ... and a launch that understates the slots raises the sticky word instead of returning wrong sums unnoticed
    assert call(plan.n_slots - 1, need) == 0
    assert L.gc_spmm_plan_check(plan.buf.data_ptr(), plan.n_pieces, plan.n_slots, plan.n_cut, s) == -5
    assert b"skipped" in L.gc_last_error()


@pytest.mark.parametrize("F,deg,in_flight", [(256, 64, 4), (256, 7, 8), (100, 33, 4), (32, 64, 8), (8, 5, 4), (512, 3, 4)])
def test_gather_sum_probe_is_a_real_sum(cuda, F, deg, in_flight):
    """The measurement aid behind the gather ceiling computes what it says: Y[i] = sum_k H[idx[i, k]]."""
    from graphcuda_b200 import _lib
    L = _lib.lib()
    g = torch.Generator().manual_seed(F + deg)
    K, n_rows = 5000, 777
    H = torch.randn(K, F, generator=g)
    idx = torch.randint(0, K, (n_rows, deg), generator=g, dtype=torch.int32)
    ref = H[idx.long()].double().sum(1)
    Hd, idxd = H.to(cuda), idx.to(cuda)
    Y = torch.full((n_rows, F), float("nan"), device=cuda)
    st = L.gc_gather_sum_f32(Hd.data_ptr(), F, K, F, idxd.data_ptr(), n_rows, deg, Y.data_ptr(), F, in_flight,
                             torch.cuda.current_stream().cuda_stream)
    assert st == 0, L.gc_last_error()
    assert O.rel_fro(Y, ref) < 1e-5


@pytest.mark.parametrize("F,n_blocks", [(32, 4), (8, 8), (100, 3), (256, 2), (7, 5)])
def test_rows_stored_into_per_owner_blocks(cuda, F, n_blocks):
    """gc_spmm_csr_f32_blocks: row i goes to block i // block_rows, row i % block_rows -- here the blocks are
    column slices of local matrices (as the owners' buffers are in the multi-GPU scheme), long rows included."""
    M, K = 1003, 4000
    A = random_csr(M, K, 7.0, seed=F, long_rows=((5, 3000), (1002, 2500)), empty_rows=(0,))
    H = torch.randn(K, F, generator=torch.Generator().manual_seed(1))
    b = torch.randn(F, generator=torch.Generator().manual_seed(2))
    pre = O.spmm(A, H) + b
    ref = pre * (pre > 0)
    adj = to_gpu_csr(A, cuda)
    B = -(-M // n_blocks)
    wide = [torch.full((B, F + 12), float("nan"), device=cuda) for _ in range(n_blocks)]
    blocks = [w[:, 4:4 + F] for w in wide]  # views with a larger row stride and a column offset
    adj.matmul_into_blocks(H.to(cuda), blocks, B, bias=b.to(cuda), relu=True)
    out = torch.cat([blk for blk in blocks])[:M]
    assert O.rel_fro(out, ref) < TOL and O.rel_max(out, ref) < TOL
    for w in wide:  # nothing outside the slices was touched
        assert bool(torch.isnan(w[:, :4]).all()) and bool(torch.isnan(w[:, 4 + F:]).all())
    assert bool(torch.isnan(torch.cat(blocks)[M:]).all())  # rows past M of the last block too


@pytest.mark.parametrize("F", [8, 16, 48, 64, 104, 128, 256, 520])
def test_bf16_gathers_sum_in_fp32(cuda, F):
    """H held in bf16 (reduced-precision tier, 1e-2): against the float64 product the error is that of rounding
    H; against the product of the rounded H only the fp32 summation order differs."""
    from graphcuda_b200 import ops
    A = random_csr(3000, 5000, 9.0, seed=F, long_rows=((7, 3000), (100, 2049)), empty_rows=(0, 13))
    H = torch.randn(5000, F, generator=torch.Generator().manual_seed(F + 1))
    b = torch.randn(F, generator=torch.Generator().manual_seed(3))
    adj = to_gpu_csr(A, cuda)
    H16 = ops.to_bf16(H.to(cuda))
    out = adj.matmul(H16)
    assert out.dtype == torch.float32
    assert O.rel_fro(out, O.spmm(A, H)) < 1e-2
    assert O.rel_fro(out, O.spmm(A.double(), H.bfloat16().double())) < 1e-5
    pre = O.spmm(A.double(), H.bfloat16().double()) + b.double()
    out2 = adj.matmul(H16, bias=b.to(cuda), relu=True)
    assert O.rel_fro(out2, pre * (pre > 0)) < 1e-5
    assert torch.equal(out, adj.matmul(H16))
    with pytest.raises(RuntimeError):
        adj.matmul(H.to(cuda).bfloat16()[:, :F - 1])  # widths must be multiples of 8


@pytest.mark.parametrize("rows,F,w", [(1000, 256, 32), (777, 100, 16), (50, 47, 12), (3, 8, 8), (1200, 96, 96)])
def test_column_slabs_scattered_to_their_destinations(cuda, rows, F, w):
    """gc_scatter_column_slabs_f32: the rows -> columns transpose of the feature-sharded scheme in one kernel."""
    from graphcuda_b200 import ops
    P = -(-F // w)
    src = torch.randn(rows, F, generator=torch.Generator().manual_seed(F)).to(cuda)
    bufs = [torch.full((rows + 5, w + 4), float("nan"), device=cuda) for _ in range(P)]
    ops.scatter_column_slabs(src, [b[:rows, :w] for b in bufs], w)
    for q, b in enumerate(bufs):
        c0, c1 = q * w, min((q + 1) * w, F)
        assert torch.equal(b[:rows, :c1 - c0], src[:, c0:c1])
        assert bool(torch.isnan(b[rows:]).all()) and bool(torch.isnan(b[:, w:]).all())
        assert bool(torch.isnan(b[:rows, c1 - c0:w]).all())  # a short last slab leaves its pad alone

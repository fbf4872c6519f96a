"""Parity at the sizes the benchmark times, against CPU float64 references.

The smaller parity tests compare whole outputs with the oracle; at these sizes
a whole-output CPU reference would take minutes, so each case checks a fixed
sample of output rows / entries whose reference is computed on the CPU in
float64 from the same inputs, with the oracle's formulas:

  * aggregation  Y = A H           (oracle.spmm; src/graphcuda/cuda/spmm_cusparse.cu:105-116)
    on the 2,449,029-node / 126 M-non-zero R-MAT graph: 19 column panels at
    F = 256, 2048-entry segments, hub rows above 100,000 non-zeros;
  * operator GEMMs C = A B         (oracle.matmul; src/graphcuda/cuda/gemm_cublas.cu:37-48)
    at 4096^3, 8192^3, 2^20 x 64 x 128 and 2^20 x 256 x 256 (split-K, in-place
    transposed operands, 64-bit row offsets);
  * dense-adjacency layer relu(A (X W) + b) at N = 32,768
    (src/graphcuda/cpp/gcn.cpp:10-15 with the bias added to the pre-activation).

Tolerances: 1e-4 relative for the fp32-semantics paths, 1e-2 for single-pass
TF32 and bf16.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu

TOL = 1e-4
TOL_LOW = 1e-2


def _rel(out, ref):
    out = out.double().cpu()
    ref = ref.double().cpu()
    fro = float((out - ref).norm() / ref.norm())
    mx = float((out - ref).abs().max() / ref.abs().max())
    return fro, mx


# ---------------------------------------------------------------- the 126 M-non-zero graph
@pytest.fixture(scope="module")
def products_graph(cuda):
    import graphcuda_b200 as gc
    from graphcuda_b200 import synth
    cfg = synth.CONFIGS["rmat_products"]
    n = cfg["nodes"]
    e = synth.rmat_edges(cfg["scale"], n, cfg["edges"], cfg["seed"], device=cuda)
    adj = gc.normalized_adjacency(synth.symmetrize(e), n, symmetric=True)
    del e
    assert adj.nnz == 2 * cfg["edges"] + n
    rowptr = adj.rowptr.cpu().long()
    deg = rowptr[1:] - rowptr[:-1]
    order = torch.argsort(deg, descending=True, stable=True)
    g = torch.Generator().manual_seed(77)
    rows = torch.cat([order[:64], order[-64:], torch.randint(0, n, (1872,), generator=g)]).unique()
    # CSR slices of the sampled rows, on the CPU
    col = adj.col.cpu()
    val = adj.val.cpu()
    slices = [(int(r), col[rowptr[r]:rowptr[r + 1]].long(), val[rowptr[r]:rowptr[r + 1]].double()) for r in rows]
    yield adj, n, rows, slices, deg
    torch.cuda.empty_cache()


def _reference_rows(slices, H_cpu):
    """sum_j A[r, j] H[j, :] in float64 for the sampled rows."""
    out = torch.empty(len(slices), H_cpu.size(1), dtype=torch.float64)
    for i, (_, c, v) in enumerate(slices):
        out[i] = v @ H_cpu[c].double() if c.numel() else 0.0
    return out


def test_products_graph_has_the_shape_the_plan_is_tuned_for(products_graph):
    adj, n, rows, slices, deg = products_graph
    assert int(deg.max()) > 100_000 and int(deg.min()) >= 1  # hub rows and the self-loop floor
    n_pieces, n_slots, n_cut = adj.plan_counts(256)
    from graphcuda_b200 import _lib
    assert int(_lib.lib().gc_spmm_default_panel_cols(n, 256)) == 131072  # 19 column panels
    assert n_cut > 10_000 and n_slots > 2 * n_cut and n_pieces > n
    # the normalisation at this size: val(i, j) = d_i^-1/2 d_j^-1/2 bit for bit on the sampled rows
    dinv = deg.float().pow(-0.5)
    for r, c, v in slices[:200]:
        assert torch.equal(v.float(), dinv[r] * 1.0 * dinv[c])


@pytest.mark.parametrize("F", [100, 256, 48])
def test_aggregation_on_the_products_graph(products_graph, cuda, F):
    from graphcuda_b200 import synth
    adj, n, rows, slices, _ = products_graph
    H = synth.normal_features(n, F, seed=F, device=cuda)
    H_cpu = H.cpu()
    ref = _reference_rows(slices, H_cpu)
    idx = rows.to(cuda)
    Y = adj.matmul(H)
    fro, mx = _rel(Y[idx], ref)
    assert fro < TOL and mx < TOL, (F, fro, mx)
    # fused epilogues as the training step uses them: bias + ReLU in the forward store,
    # the previous layer's ReLU mask ("gate") in the backward store
    b = synth.normal_features(1, F, seed=F + 1, device=cuda)[0]
    pre = ref + b.double().cpu()
    Yb = adj.matmul(H, bias=b, relu=True)
    fro, mx = _rel(Yb[idx], pre * (pre > 0))
    assert fro < TOL and mx < TOL, (F, fro, mx)
    gate = synth.normal_features(n, F, seed=F + 2, device=cuda)
    Yg = adj.matmul(H, gate=gate)
    fro, mx = _rel(Yg[idx], ref * (gate[idx].double().cpu() > 0))
    assert fro < TOL and mx < TOL, (F, fro, mx)
    # bit-reproducible run to run at this size too
    assert torch.equal(Y, adj.matmul(H))
    del H, Y, Yb, Yg, gate


def test_row_sums_over_the_whole_products_graph(products_graph, cuda):
    """A 1 = rowsum(A): a size-independent identity over every row (not a sample)."""
    adj, n, _, _, _ = products_graph
    ones = torch.ones(n, 4, device=cuda)
    rs = adj.matmul(ones)[:, 0]
    cs = torch.cat([torch.zeros(1, dtype=torch.float64, device=cuda), torch.cumsum(adj.val.double(), 0)])
    seg = cs[adj.rowptr[1:].long()] - cs[adj.rowptr[:-1].long()]
    assert float((rs.double() - seg).abs().max() / seg.abs().max()) < TOL


# ---------------------------------------------------------------- operator GEMMs at the timed sizes
GEMM_SHAPES = [(4096, 4096, 4096), (8192, 8192, 8192), (1 << 20, 64, 128), (1 << 20, 256, 256),
               (1 << 20, 64, 256), (1 << 20, 256, 128)]


@pytest.mark.parametrize("M,N,K", GEMM_SHAPES)
@pytest.mark.parametrize("prec,tol", [("tf32x3", TOL), ("tf32", TOL_LOW), ("bf16", TOL_LOW)])
def test_operator_gemm_at_the_timed_sizes(cuda, M, N, K, prec, tol):
    import graphcuda_b200 as gc
    from graphcuda_b200 import ops
    g = torch.Generator(device=cuda)
    g.manual_seed(1)
    A = torch.rand(M, K, generator=g, device=cuda) * 2 - 1
    B = torch.rand(K, N, generator=g, device=cuda) * 2 - 1
    C = gc.gemm(A, B, precision=prec)
    torch.cuda.synchronize()
    ops.check_gemm_flag(cuda)
    gs = torch.Generator().manual_seed(2)
    ii = torch.randint(0, M, (4096,), generator=gs)
    jj = torch.randint(0, N, (4096,), generator=gs)
    ii[:4] = torch.tensor([0, M - 1, 0, M - 1])
    jj[:4] = torch.tensor([0, 0, N - 1, N - 1])
    a = A[ii.to(cuda)].double().cpu()
    b = B[:, jj.to(cuda)].double().cpu()
    ref = (a * b.t()).sum(1)
    out = C[ii.to(cuda), jj.to(cuda)]
    fro, mx = _rel(out, ref)
    assert fro < tol and mx < tol, (prec, M, N, K, fro, mx)


def test_matmul_names_at_a_timed_size(cuda):
    """The reference's operator names on a 2^20-row skinny shape (matmul3 is wrong there in the reference:
    src/graphcuda/cuda/matmul3.cu:215-232)."""
    import graphcuda
    g = torch.Generator(device=cuda)
    g.manual_seed(3)
    A = torch.rand(1 << 20, 128, generator=g, device=cuda) * 2 - 1
    B = torch.rand(128, 64, generator=g, device=cuda) * 2 - 1
    rows = torch.arange(0, 1 << 20, 4099, device=cuda)
    ref = A[rows].double().cpu() @ B.double().cpu()
    for fn in (graphcuda.matmul3, graphcuda.matmul4, graphcuda.gemm_cublas):
        fro, mx = _rel(fn(A, B)[rows], ref)
        assert fro < TOL and mx < TOL


# ---------------------------------------------------------------- dense adjacency, N = 32,768
@pytest.mark.parametrize("prec,tol", [("tf32x3", TOL), ("tf32", TOL_LOW), ("bf16", TOL_LOW)])
def test_dense_adjacency_layer_at_32768(cuda, prec, tol):
    import graphcuda_b200 as gc
    from graphcuda_b200 import ops, synth
    n = 32768
    e = synth.erdos_renyi_edges(n, 0.01, seed=3, device=cuda)
    a = gc.normalized_adjacency(synth.symmetrize(e), n, symmetric=True)
    dense = torch.zeros(n, n, device=cuda)
    r = torch.repeat_interleave(torch.arange(n, device=cuda), (a.rowptr[1:] - a.rowptr[:-1]).long())
    dense[r, a.col.long()] = a.val
    X = synth.normal_features(n, 512, seed=5, device=cuda)
    W = synth.reference_init(512, 256, seed=6, device=cuda)
    b = synth.normal_features(1, 256, seed=7, device=cuda)[0] * 0.1
    dadj = gc.DenseAdjacency(dense, symmetric=True)
    Y = dadj.matmul(gc.gemm(X, W, precision=prec), bias=b, relu=True, precision=prec)
    torch.cuda.synchronize()
    ops.check_gemm_flag(cuda)
    rows = torch.arange(0, n, 128, device=cuda)  # 256 rows
    H = X.double().cpu() @ W.double().cpu()
    pre = dense[rows].double().cpu() @ H + b.double().cpu()
    fro, mx = _rel(Y[rows], pre * (pre > 0))
    assert fro < tol and mx < tol, (prec, fro, mx)
    # the same layer through the CSR path agrees with the dense path
    Yc = a.matmul(gc.gemm(X, W, precision="tf32x3"), bias=b, relu=True)
    fro, mx = _rel(Yc[rows], pre * (pre > 0))
    assert fro < TOL and mx < TOL

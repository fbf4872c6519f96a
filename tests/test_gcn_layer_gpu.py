"""GCNConv forward/backward vs the oracle (the reference's ATen composition,
src/graphcuda/cpp/gcn.cpp, on CPU) and vs the fixtures its code produced."""
import os

import numpy as np
import pytest
import torch

from oracle import gcn_oracle as O
from tests.helpers import untie

pytestmark = pytest.mark.gpu

TOL = 1e-4
TOL_TF32 = 1e-2


def _t(a):
    return torch.from_numpy(np.asarray(a))


def _graph(n, avg_deg, seed):
    from graphcuda_b200 import synth
    scale = max(4, (n - 1).bit_length())
    e = synth.rmat_edges(scale, n, int(n * avg_deg / 2), seed)
    return O.normalized_adjacency_coo(synth.symmetrize(e), n)


def _adj_variant(A, kind, dev):
    if kind == "dense":
        return A.to_dense().to(dev)
    if kind == "coo":
        return A.to(dev)
    if kind == "csr":
        return A.to_sparse_csr().to(dev)
    rowptr, col, val = O.coo_to_csr_int32(A)
    return (rowptr.to(dev), col.to(dev), val.to(dev))


@pytest.mark.parametrize("kind", ["dense", "coo", "csr", "tuple"])
@pytest.mark.parametrize("dims", [(40, 12), (12, 40), (33, 33), (100, 7)])
@pytest.mark.parametrize("relu", [True, False])
def test_layer_forward_backward(cuda, kind, dims, relu):
    """Both aggregation orders (in <= out and out < in), all adjacency layouts."""
    import graphcuda
    fin, fout = dims
    n = 600
    A = _graph(n, 8, seed=fin)
    g = torch.Generator().manual_seed(fin * 100 + fout)
    X = torch.randn(n, fin, generator=g)
    dY = torch.randn(n, fout, generator=g)
    torch.manual_seed(3)
    conv = graphcuda.GCNConv(fin, fout, apply_relu=relu)
    torch.manual_seed(3)
    ref = O.GCNConv(fin, fout, apply_relu=relu)
    assert torch.equal(conv.weights.detach(), ref.weights.detach())  # same initialiser, same RNG use
    assert list(conv.state_dict().keys()) == ["weights"]
    conv = conv.to(cuda)

    Xr = X.clone().requires_grad_()
    Yr = ref(Xr, A)
    if relu:  # gradients are compared away from ReLU ties
        dY = untie(dY, A.mm(X).mm(ref.weights.detach()))
    Yr.backward(dY)
    Xg = X.to(cuda).requires_grad_()
    Y = conv(Xg, _adj_variant(A, kind, cuda))
    Y.backward(dY.to(cuda))
    assert O.rel_fro(Y, Yr) < TOL and O.rel_max(Y, Yr) < TOL * 10
    assert O.rel_fro(Xg.grad, Xr.grad) < TOL
    assert O.rel_fro(conv.weights.grad, ref.weights.grad) < TOL


def test_extension_level_functions(cuda):
    """graphcuda._graphcuda.gcn_conv_forward / gcn_conv_backward keep the
    reference's signatures and return conventions (gcn.cuh:6-18)."""
    import graphcuda
    n, fin, fout = 500, 24, 16
    A = _graph(n, 6, seed=1)
    g = torch.Generator().manual_seed(0)
    X, W, dY = torch.randn(n, fin, generator=g), torch.randn(fin, fout, generator=g), torch.randn(n, fout, generator=g)
    Yr, mr = O.gcn_conv_forward(X, A, W, True)
    dY = untie(dY, A.mm(X).mm(W))
    dXr, dWr = O.gcn_conv_backward(dY, X, A, W, True, mr)
    Ag = A.to(cuda)
    Y, m = graphcuda._graphcuda.gcn_conv_forward(X.to(cuda), Ag, W.to(cuda), True)
    assert m.shape == (n, fout) and m.dtype == torch.float32 and m.is_cuda
    assert O.rel_fro(Y, Yr) < TOL
    dX, dW = graphcuda._graphcuda.gcn_conv_backward(dY.to(cuda), X.to(cuda), Ag, W.to(cuda), True, m)
    assert O.rel_fro(dX, dXr) < TOL and O.rel_fro(dW, dWr) < TOL
    Y0, m0 = graphcuda._graphcuda.gcn_conv_forward(X.to(cuda), Ag, W.to(cuda), False)
    assert m0.dim() == 0 and not m0.is_cuda  # 0-dim CPU tensor, gcn.cu:22
    dX0, dW0 = graphcuda._graphcuda.gcn_conv_backward(dY.to(cuda), X.to(cuda), Ag, W.to(cuda), False, m0)
    dXr0, dWr0 = O.gcn_conv_backward(dY, X, A, W, False, torch.empty(()))
    assert O.rel_fro(dX0, dXr0) < TOL and O.rel_fro(dW0, dWr0) < TOL
    with pytest.raises(RuntimeError):
        graphcuda._graphcuda.gcn_conv_forward(X, A, W, True)  # CPU tensors: no CPU path


def test_non_symmetric_adjacency_follows_the_reference(cuda):
    """The reference multiplies by A (not A^T) in the backward pass
    (gcn.cu:49); for a non-symmetric A that is what must come out."""
    import graphcuda
    from tests.helpers import random_csr
    n, fin, fout = 300, 30, 10  # out < in: would pick transform-first if A were symmetric
    A = random_csr(n, n, 5.0, seed=4)
    g = torch.Generator().manual_seed(1)
    X, dY = torch.randn(n, fin, generator=g), torch.randn(n, fout, generator=g)
    torch.manual_seed(5)
    conv = graphcuda.GCNConv(fin, fout).to(cuda)
    torch.manual_seed(5)
    ref = O.GCNConv(fin, fout)
    Xr = X.clone().requires_grad_()
    dY = untie(dY, A.mm(X).mm(ref.weights.detach()))
    ref(Xr, A).backward(dY)
    Xg = X.to(cuda).requires_grad_()
    conv(Xg, A.to(cuda)).backward(dY.to(cuda))
    assert O.rel_fro(Xg.grad, Xr.grad) < TOL
    assert O.rel_fro(conv.weights.grad, ref.weights.grad) < TOL


def test_golden_layers(cuda, golden_dir):
    import graphcuda
    g = np.load(os.path.join(golden_dir, "layer_dense.npz"))
    A, X, W, dY = (_t(g[k]).to(cuda) for k in ("A", "X", "W", "dY"))
    Y, m = graphcuda._graphcuda.gcn_conv_forward(X, A, W, True)
    # the backward entry point takes the mask as an argument: feed it the reference's
    dX, dW = graphcuda._graphcuda.gcn_conv_backward(dY, X, A, W, True, _t(g["mask"]).to(cuda))
    assert float((m.cpu() != _t(g["mask"])).float().mean()) < 1e-3
    for name, got in (("Y", Y), ("dX", dX), ("dW", dW)):
        assert O.rel_fro(got, _t(g[name])) < TOL, name
    s = np.load(os.path.join(golden_dir, "layer_sparse.npz"))
    n = int(s["n"])
    As = torch.sparse_coo_tensor(torch.stack([_t(s["rows"]), _t(s["cols"])]), _t(s["vals"]), (n, n)).coalesce().to(cuda)
    X, W, dY = (_t(s[k]).to(cuda) for k in ("X", "W", "dY"))
    Y1, m1 = graphcuda._graphcuda.gcn_conv_forward(X, As, W, True)
    dX1, dW1 = graphcuda._graphcuda.gcn_conv_backward(dY, X, As, W, True, _t(s["mask1"]).to(cuda))
    for name, got in (("Y1", Y1), ("dX1", dX1), ("dW1", dW1)):
        assert O.rel_fro(got, _t(s[name])) < TOL, name


def test_golden_module_training(cuda, golden_dir):
    """5 Adam steps of the 2-layer model: losses, weights and argmax of the
    reference module's run."""
    import graphcuda
    g = np.load(os.path.join(golden_dir, "module_train.npz"))
    A, X, y = _t(g["A"]).to(cuda), _t(g["X"]).to(cuda), _t(g["y"]).to(cuda)
    torch.manual_seed(int(g["seed"]))
    c1 = graphcuda.GCNConv(X.size(1), g["W1_0"].shape[1], apply_relu=True)
    c2 = graphcuda.GCNConv(g["W2_0"].shape[0], g["W2_0"].shape[1], apply_relu=False)
    assert torch.equal(c1.weights.detach(), _t(g["W1_0"])) and torch.equal(c2.weights.detach(), _t(g["W2_0"]))
    c1, c2 = c1.to(cuda), c2.to(cuda)
    opt = torch.optim.Adam(list(c1.parameters()) + list(c2.parameters()), lr=0.01)
    losses = []
    for _ in range(5):
        opt.zero_grad()
        out = torch.log_softmax(c2(c1(X, A), A), dim=1)
        loss = torch.nn.functional.nll_loss(out[:20], y[:20])
        loss.backward()
        opt.step()
        losses.append(loss.item())
    assert np.allclose(losses, g["losses"], rtol=1e-4)
    assert O.rel_fro(c1.weights, _t(g["W1"])) < TOL and O.rel_fro(c2.weights, _t(g["W2"])) < TOL
    with torch.no_grad():
        logits = torch.log_softmax(c2(c1(X, A), A), dim=1)
    assert O.rel_fro(logits, _t(g["logits"])) < TOL
    assert torch.equal(logits.argmax(1).cpu(), _t(g["logits"]).argmax(1))


@pytest.mark.parametrize("kind", ["dense", "coo"])
def test_cora_like_training_logits_and_argmax(cuda, kind):
    """2-layer GCN, N=2708, 1433 -> 16 -> 7, 20 Adam epochs on the synthetic
    Cora-shaped input: logits within 1e-4 and identical argmax."""
    import graphcuda
    from graphcuda_b200 import synth
    cfg = synth.CONFIGS["cora_like"]
    n = cfg["nodes"]
    e = synth.preferential_attachment_edges(n, cfg["edges"], cfg["seed"])
    A = O.normalized_adjacency_coo(synth.symmetrize(e), n)
    X = synth.bow_features(n, cfg["features"], 0.0127, seed=1)
    y = synth.uniform_labels(n, cfg["classes"], seed=2)
    train, _, _ = synth.planetoid_split(n)
    torch.manual_seed(0)
    ref = O.GCN([cfg["features"], cfg["hidden"], cfg["classes"]])
    torch.manual_seed(0)
    c1 = graphcuda.GCNConv(cfg["features"], cfg["hidden"], apply_relu=True)
    c2 = graphcuda.GCNConv(cfg["hidden"], cfg["classes"], apply_relu=False)
    c1, c2 = c1.to(cuda), c2.to(cuda)
    Aref = A.to_dense() if kind == "dense" else A
    Ag = Aref.to(cuda)
    Xg, yg, tg = X.to(cuda), y.to(cuda), train.to(cuda)
    opt_r = torch.optim.Adam(ref.parameters(), lr=0.01)
    opt_g = torch.optim.Adam(list(c1.parameters()) + list(c2.parameters()), lr=0.01)
    for _ in range(20):
        opt_r.zero_grad()
        lr_ = torch.nn.functional.nll_loss(ref(X, Aref)[train], y[train])
        lr_.backward()
        opt_r.step()
        opt_g.zero_grad()
        out = torch.log_softmax(c2(c1(Xg, Ag), Ag), dim=1)
        lg = torch.nn.functional.nll_loss(out[tg], yg[tg])
        lg.backward()
        opt_g.step()
    assert abs(lr_.item() - lg.item()) < 1e-4 * max(1.0, abs(lr_.item()))
    with torch.no_grad():
        logits_r = ref(X, Aref)
        logits_g = torch.log_softmax(c2(c1(Xg, Ag), Ag), dim=1).cpu()
    assert O.rel_fro(logits_g, logits_r) < TOL
    # identical argmax; a disagreement is only tolerable on a numerical tie
    pr, pg = logits_r.argmax(1), logits_g.argmax(1)
    if not torch.equal(pr, pg):
        bad = (pr != pg).nonzero().flatten()
        top2 = logits_r[bad].double().topk(2, dim=1).values
        assert float((top2[:, 0] - top2[:, 1]).max()) < 1e-6, "argmax differs away from ties"


def test_bias_relu_layer_arxiv_like_shape(cuda):
    """Single layer with bias + ReLU on a reduced R-MAT graph, 128 -> 256 (the
    tensor-core path): relu((A X) W + b) against the oracle, fp32 and the two
    reduced-precision tiers (single-pass TF32, bf16) at 1e-2."""
    import graphcuda
    from graphcuda_b200 import synth
    n = 20_000
    A = _graph(n, 14, seed=2)
    X = synth.normal_features(n, 128, seed=5)
    b = synth.normal_features(1, 256, seed=6)[0] * 0.1
    dY = synth.normal_features(n, 256, seed=7)
    torch.manual_seed(11)
    conv = graphcuda.GCNConv(128, 256, apply_relu=True, bias=True)
    W = conv.weights.detach().clone()
    with torch.no_grad():
        conv.bias.copy_(b)
    conv = conv.to(cuda)
    Xr = X.clone().requires_grad_()
    Wr = W.clone().requires_grad_()
    br = b.clone().requires_grad_()
    pre = A.mm(Xr).mm(Wr) + br
    Yr = pre * (pre > 0)
    # one reference gradient per tolerance tier: ties are excluded at the tier's own resolution
    # "bf16": bf16 operands in the dense products and a bf16 copy of the matrix being aggregated, fp32 sums
    for prec, tol in ((None, TOL), ("tf32", TOL_TF32), ("bf16", TOL_TF32)):
        for t in (Xr, Wr, br):
            t.grad = None
        dYt = untie(dY, pre.detach(), rel=tol)
        Yr.backward(dYt, retain_graph=True)
        conv.precision = prec
        conv.zero_grad()
        Xg = X.to(cuda).requires_grad_()
        Y = conv(Xg, A.to(cuda))
        Y.backward(dYt.to(cuda))
        assert O.rel_fro(Y, Yr) < tol, prec
        assert O.rel_fro(Xg.grad, Xr.grad) < tol, prec
        assert O.rel_fro(conv.weights.grad, Wr.grad) < tol, prec
        assert O.rel_fro(conv.bias.grad, br.grad) < tol, prec
    from graphcuda_b200 import ops
    ops.check_gemm_flag(cuda)


def test_input_layer_skips_dx(cuda):
    import graphcuda
    A = _graph(400, 6, seed=9)
    X = torch.randn(400, 20).to(cuda)  # requires_grad False
    conv = graphcuda.GCNConv(20, 8).to(cuda)
    conv(X, A.to(cuda)).sum().backward()
    assert conv.weights.grad is not None and X.grad is None


def test_odd_output_width_runs_padded(cuda):
    """256 -> 47 on enough rows to take the zero-padded transform-first path
    (aligned row pitches for the vector gathers and the tensor-core GEMMs)."""
    import graphcuda
    from graphcuda_b200 import engine, synth
    n = 20_000
    assert engine._padded_width(n, 256, 47) == 48
    A = _graph(n, 10, seed=6)
    X = synth.normal_features(n, 256, seed=8)
    dY = synth.normal_features(n, 47, seed=9)
    torch.manual_seed(21)
    conv = graphcuda.GCNConv(256, 47, apply_relu=False).to(cuda)
    W = conv.weights.detach().cpu()
    Xr = X.clone().requires_grad_()
    Wr = W.clone().requires_grad_()
    Yr = A.mm(Xr).mm(Wr)
    Yr.backward(dY)
    Xg = X.to(cuda).requires_grad_()
    Y = conv(Xg, A.to(cuda))
    assert Y.shape == (n, 47)
    Y.backward(dY.to(cuda))
    assert O.rel_fro(Y, Yr) < TOL
    assert O.rel_fro(Xg.grad, Xr.grad) < TOL
    assert O.rel_fro(conv.weights.grad, Wr.grad) < TOL


def test_cuda_graph_replay_matches_eager_training(cuda):
    """The recorded step (forward, fused loss, backward, Adam) replays to the same
    weights as the eager loop, bit for bit (same kernels, same order)."""
    import graphcuda_b200 as gc
    from graphcuda_b200 import synth
    from graphcuda_b200.models import GCN
    n = 2708
    e = synth.preferential_attachment_edges(n, 5429, 0).to(cuda)
    adj = gc.normalized_adjacency(synth.symmetrize(e), n, symmetric=True)
    X = synth.bow_features(n, 1433, 0.0127, seed=1, device=cuda)
    y = synth.uniform_labels(n, 7, seed=2, device=cuda)
    train = synth.planetoid_split(n)[0].to(cuda)

    def make():
        torch.manual_seed(0)
        m = GCN([1433, 16, 7]).to(cuda)
        return m, torch.optim.Adam(m.parameters(), lr=0.01, capturable=True)

    m1, o1 = make()
    for _ in range(3 + 5):  # GraphedTrainStep runs 3 eager warm-up steps before recording
        o1.zero_grad(set_to_none=True)
        loss = gc.log_softmax_nll_loss(m1(X, adj, log_softmax=False), y, train, scale=1.0 / 140)
        loss.backward()
        o1.step()
    m2, o2 = make()
    g = gc.GraphedTrainStep(m2, adj, X, y, o2, row_mask=train, warmup=3)
    for _ in range(5):
        lg = g.step()
    torch.cuda.synchronize()
    assert torch.equal(lg, loss)
    for a, b in zip(m1.parameters(), m2.parameters()):
        assert torch.equal(a, b)


@pytest.mark.parametrize("dims", [[24, 32, 40, 7], [64, 32, 16, 7], [100, 256, 256, 47]])
def test_fused_relu_backward_equals_separate_pass(cuda, dims):
    """models.GCN applies a layer's ReLU backward in the store of the kernel that
    produces the upper layer's input gradient (SpMM or GEMM).  Multiplying by the
    same 0/1 mask in another place changes no bit of any gradient."""
    import graphcuda_b200 as gc
    from graphcuda_b200 import synth
    from graphcuda_b200.models import GCN
    n = 6000 if dims[1] < 256 else 20000
    A = _graph(n, 12, seed=3)
    adj = gc.as_adjacency(A.to(cuda), symmetric=True)
    X = synth.normal_features(n, dims[0], seed=4, device=cuda)
    y = synth.uniform_labels(n, dims[-1], seed=5, device=cuda)
    grads = []
    for fuse in (True, False):
        torch.manual_seed(1)
        m = GCN(dims, fuse_relu_backward=fuse).to(cuda)
        assert [c.fuse_relu_backward for c in m.convs] == ([1, 3, 2] if fuse else [0, 0, 0])
        Xg = X.clone().requires_grad_()
        loss = gc.log_softmax_nll_loss(m(Xg, adj, log_softmax=False), y)
        loss.backward()
        grads.append([Xg.grad.clone()] + [c.weights.grad.clone() for c in m.convs])
    for a, b in zip(*grads):
        assert torch.equal(a, b)
    # and against the oracle model (ties excluded by the tolerance: two ReLUs, rare mask flips)
    torch.manual_seed(1)
    ref = O.GCN(dims)
    Xr = X.cpu().clone().requires_grad_()
    lr = torch.nn.functional.nll_loss(ref(Xr, A), y.cpu())
    lr.backward()
    assert O.rel_fro(grads[0][0], Xr.grad) < 2e-3
    for gw, conv in zip(grads[0][1:], ref.convs):
        assert O.rel_fro(gw, conv.weights.grad) < 2e-3


def test_evaluate_matches_the_scripts_test_function(cuda):
    """GCN.evaluate = the reference script's test() (tests/gcn/graphcuda_impl.py:60-69): no-grad forward,
    argmax, per-split accuracy; compared with the oracle model carrying the same weights."""
    from graphcuda_b200 import synth
    from graphcuda_b200.models import GCN
    cfg = synth.CONFIGS["cora_like"]
    n = cfg["nodes"]
    e = synth.preferential_attachment_edges(n, cfg["edges"], cfg["seed"])
    A = O.normalized_adjacency_coo(synth.symmetrize(e), n)
    X = synth.bow_features(n, cfg["features"], 0.0127, seed=1)
    y = synth.uniform_labels(n, cfg["classes"], seed=2)
    splits = synth.planetoid_split(n)
    dims = [cfg["features"], cfg["hidden"], cfg["classes"]]
    torch.manual_seed(3)
    ref = O.GCN(dims)
    torch.manual_seed(3)
    model = GCN(dims).to(cuda)
    with torch.no_grad():
        out = ref(X, A)
    pr = out.argmax(1)
    want = [[int(((pr == y) & m).sum()), int(m.sum())] for m in splits]
    pred, counts = model.evaluate(X.to(cuda), A.to(cuda), y.to(cuda), [m.to(cuda) for m in splits])
    got = counts.cpu().tolist()
    flips = int((pred.cpu() != pr).sum())
    if flips == 0:
        assert got == want
    else:  # only numerical ties may flip
        bad = (pred.cpu() != pr).nonzero().flatten()
        top2 = out[bad].double().topk(2, dim=1).values
        assert float((top2[:, 0] - top2[:, 1]).max()) < 1e-6
    assert [c[1] for c in got] == [140, 500, 1000]
    # no autograd state is kept by the evaluation pass
    assert all(p.grad is None for p in model.parameters())


@pytest.mark.parametrize("order", ["aggregate_first", "transform_first"])
@pytest.mark.parametrize("relu,recompute", [(True, False), (False, False), (True, True)])
def test_layer_entry_points_of_the_c_abi(cuda, order, relu, recompute):
    """gc_gcn_conv_forward_csr_f32 / gc_gcn_conv_backward_csr_f32 called with raw pointers, as a C++ binding of the
    ABI would: the reference's two layer functions (gcn.cu:5-52) against the oracle, in both product orders, with
    and without ReLU, with A X kept from the forward call or recomputed like the reference does."""
    from graphcuda_b200 import _lib
    from tests.helpers import to_gpu_csr, untie
    L = _lib.lib()
    n, fin, fout = 3000, 40, 24
    A = _graph(n, 10, seed=4)
    g = torch.Generator().manual_seed(8)
    X = torch.randn(n, fin, generator=g)
    W = (torch.rand(fin, fout, generator=g) * 2 - 1) * 0.3
    dY = torch.randn(n, fout, generator=g)
    Yr, mask_r = O.gcn_conv_forward(X, A, W, relu)
    if relu:
        dY = untie(dY, A.mm(X).mm(W))
    dXr, dWr = O.gcn_conv_backward(dY, X, A, W, relu, mask_r)
    adj = to_gpu_csr(A, cuda)
    plan = adj.plan_for(max(fin, fout))
    flags = (_lib.LAYER_RELU if relu else 0) | (_lib.LAYER_TRANSFORM_FIRST if order == "transform_first" else 0)
    Xg, Wg, dYg = X.to(cuda), W.to(cuda), dY.to(cuda)
    Y = torch.empty(n, fout, device=cuda)
    mask = torch.empty(n, fout, device=cuda)
    AX = torch.empty(n, fin, device=cuda)
    s = torch.cuda.current_stream().cuda_stream
    P = _lib.PREC_FP32_SIMT
    wsf = torch.zeros(L.gc_gcn_layer_workspace_bytes(n, fin, fout, plan.n_slots, P, 0), dtype=torch.uint8, device=cuda)
    st = L.gc_gcn_conv_forward_csr_f32(adj.rowptr.data_ptr(), adj.col.data_ptr(), adj.val.data_ptr(), n, fin, fout,
                                       Xg.data_ptr(), fin, Wg.data_ptr(), fout, None, flags, Y.data_ptr(), fout,
                                       mask.data_ptr(), AX.data_ptr(), fin, plan.buf.data_ptr(), plan.n_pieces,
                                       plan.n_slots, plan.n_cut, P, wsf.data_ptr(), wsf.numel(), s)
    assert st == 0, L.gc_last_error()
    assert O.rel_fro(Y, Yr) < TOL
    if order == "aggregate_first":
        assert O.rel_fro(AX, A.mm(X)) < TOL
    dX = torch.empty(n, fin, device=cuda)
    dW = torch.empty(fin, fout, device=cuda)
    wsb = torch.zeros(L.gc_gcn_layer_workspace_bytes(n, fin, fout, plan.n_slots, P, 1), dtype=torch.uint8, device=cuda)
    keep_ax = order == "aggregate_first" and not recompute
    st = L.gc_gcn_conv_backward_csr_f32(adj.rowptr.data_ptr(), adj.col.data_ptr(), adj.val.data_ptr(), n, fin, fout,
                                        dYg.data_ptr(), fout, Xg.data_ptr(), fin, Wg.data_ptr(), fout, flags,
                                        mask.data_ptr() if relu else None, fout,
                                        AX.data_ptr() if keep_ax else None, fin, dX.data_ptr(), fin, dW.data_ptr(),
                                        fout, plan.buf.data_ptr(), plan.n_pieces, plan.n_slots, plan.n_cut, P,
                                        wsb.data_ptr(), wsb.numel(), s)
    assert st == 0, L.gc_last_error()
    assert O.rel_fro(dX, dXr) < TOL and O.rel_fro(dW, dWr) < TOL
    # a workspace that is too small is refused before anything is launched
    assert L.gc_gcn_conv_forward_csr_f32(adj.rowptr.data_ptr(), adj.col.data_ptr(), adj.val.data_ptr(), n, fin, fout,
                                         Xg.data_ptr(), fin, Wg.data_ptr(), fout, None, flags, Y.data_ptr(), fout,
                                         None, AX.data_ptr(), fin, plan.buf.data_ptr(), plan.n_pieces, plan.n_slots,
                                         plan.n_cut, P, wsf.data_ptr(), 1024, s) == -4


def test_padded_logits_gradient_flows_without_a_repadding_copy(cuda):
    """256 -> 47 on enough rows to run padded to 48 columns, trained through the fused loss: the loss backward
    writes its gradient with the logits' 48-float pitch and zero pad, the layer picks that buffer up as it is.
    Gradients against the oracle model with torch's log_softmax + nll_loss."""
    import graphcuda_b200 as gc
    from graphcuda_b200 import engine, synth
    from graphcuda_b200.models import GCN
    n = 20_000
    assert engine._padded_width(n, 256, 47) == 48
    A = _graph(n, 12, seed=21)
    X = synth.normal_features(n, 64, seed=22)
    y = synth.uniform_labels(n, 47, seed=23)
    dims = [64, 256, 47]
    torch.manual_seed(4)
    ref = O.GCN(dims)
    torch.manual_seed(4)
    model = GCN(dims).to(cuda)
    out = ref(X, A)
    torch.nn.functional.nll_loss(out, y).backward()
    adj = gc.as_adjacency(A.to(cuda), symmetric=True)
    logits = model(X.to(cuda), adj, log_softmax=False)
    assert logits.shape == (n, 47) and logits.stride(0) == 48
    loss = gc.log_softmax_nll_loss(logits, y.to(cuda))
    seen = {}
    def note(g):
        seen["stride"] = g.stride()

    logits.register_hook(note)
    loss.backward()
    assert seen["stride"] == (48, 1)  # the gradient arrived with the padded pitch
    assert abs(float(loss) - float(torch.nn.functional.nll_loss(out, y))) < 1e-5
    for conv, rconv in zip(model.convs, ref.convs):
        assert O.rel_fro(conv.weights.grad, rconv.weights.grad) < 1e-3  # through a ReLU: rare tie flips
    assert len(engine._zero_padded) <= 1  # the registry holds no buffer beyond the live gradient

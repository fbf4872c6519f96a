"""Pins the CPU oracle (oracle/gcn_oracle.py) against the reference's own code:
the compiled src/graphcuda/cpp/gcn.cpp (oracle/_ref) and the golden fixtures
that code produced (tests/golden, made by tests/golden/make_golden.py)."""
import os

import numpy as np
import pytest
import torch

from oracle import gcn_oracle as O
from oracle import ref_loader


def _t(a):
    return torch.from_numpy(np.asarray(a))


def test_golden_layer_dense_bit_exact(golden_dir):
    torch.set_num_threads(1)
    g = np.load(os.path.join(golden_dir, "layer_dense.npz"))
    A, X, W, dY = _t(g["A"]), _t(g["X"]), _t(g["W"]), _t(g["dY"])
    Y, mask = O.gcn_conv_forward(X, A, W, True)
    dX, dW = O.gcn_conv_backward(dY, X, A, W, True, mask)
    assert torch.equal(mask, _t(g["mask"]))
    for name, got in (("Y", Y), ("dX", dX), ("dW", dW)):
        assert O.rel_fro(got, _t(g[name])) < 1e-6, name


def test_golden_layer_sparse(golden_dir):
    torch.set_num_threads(1)
    g = np.load(os.path.join(golden_dir, "layer_sparse.npz"))
    n = int(g["n"])
    A = torch.sparse_coo_tensor(torch.stack([_t(g["rows"]), _t(g["cols"])]), _t(g["vals"]), (n, n)).coalesce()
    X, W, dY = _t(g["X"]), _t(g["W"]), _t(g["dY"])
    Y0, _ = O.gcn_conv_forward(X, A, W, False)
    dX0, dW0 = O.gcn_conv_backward(dY, X, A, W, False, torch.empty(()))
    Y1, mask1 = O.gcn_conv_forward(X, A, W, True)
    dX1, dW1 = O.gcn_conv_backward(dY, X, A, W, True, mask1)
    assert torch.equal(mask1, _t(g["mask1"]))
    for name, got in (("Y0", Y0), ("dX0", dX0), ("dW0", dW0), ("Y1", Y1), ("dX1", dX1), ("dW1", dW1)):
        assert O.rel_fro(got, _t(g[name])) < 1e-6, name
    # empty rows of the adjacency give zero output rows
    for r in (5, 17, 63):
        assert float(Y0[r].abs().max()) == 0.0


def test_golden_module_training(golden_dir):
    """The oracle's GCNConv/GCN restatement reproduces the reference module's
    initial weights (same RNG use) and its 5-step Adam trajectory."""
    torch.set_num_threads(1)
    g = np.load(os.path.join(golden_dir, "module_train.npz"))
    A, X, y = _t(g["A"]), _t(g["X"]), _t(g["y"])
    torch.manual_seed(int(g["seed"]))
    c1 = O.GCNConv(X.size(1), g["W1_0"].shape[1], apply_relu=True)
    c2 = O.GCNConv(g["W2_0"].shape[0], g["W2_0"].shape[1], apply_relu=False)
    assert torch.equal(c1.weights.detach(), _t(g["W1_0"]))
    assert torch.equal(c2.weights.detach(), _t(g["W2_0"]))
    opt = torch.optim.Adam(list(c1.parameters()) + list(c2.parameters()), lr=0.01)
    losses = []
    for _ in range(5):
        opt.zero_grad()
        out = torch.log_softmax(c2(c1(X, A), A), dim=1)
        loss = torch.nn.functional.nll_loss(out[:20], y[:20])
        loss.backward()
        opt.step()
        losses.append(loss.item())
    assert np.allclose(losses, g["losses"], rtol=1e-6, atol=0)
    assert O.rel_fro(c1.weights, _t(g["W1"])) < 1e-6
    assert O.rel_fro(c2.weights, _t(g["W2"])) < 1e-6
    with torch.no_grad():
        logits = torch.log_softmax(c2(c1(X, A), A), dim=1)
    assert torch.equal(logits.argmax(1), _t(g["logits"]).argmax(1))


needs_ref = pytest.mark.skipif(not ref_loader.ref_ext_available(), reason="oracle/_ref not built")


@needs_ref
@pytest.mark.parametrize("sparse", [False, True])
@pytest.mark.parametrize("relu", [False, True])
def test_oracle_equals_compiled_reference(sparse, relu):
    ext = ref_loader.load_ref_ext()
    g = torch.Generator().manual_seed(5 + 2 * sparse + relu)
    n, fin, fout = 97, 31, 13
    A = (torch.rand(n, n, generator=g) < 0.1).float() * torch.rand(n, n, generator=g)
    A = A + A.t()
    if sparse:
        A = A.to_sparse().coalesce()
    X = torch.randn(n, fin, generator=g)
    W = torch.randn(fin, fout, generator=g)
    dY = torch.randn(n, fout, generator=g)
    Y, m = O.gcn_conv_forward(X, A, W, relu)
    Yr, mr = ext.gcn_conv_forward(X, A, W, relu)
    assert torch.equal(Y, Yr)
    if relu:
        assert torch.equal(m, mr)
    else:
        assert m.dim() == 0 and mr.dim() == 0 and not mr.is_cuda
    dX, dW = O.gcn_conv_backward(dY, X, A, W, relu, m)
    dXr, dWr = ext.gcn_conv_backward(dY, X, A, W, relu, mr)
    assert torch.equal(dX, dXr) and torch.equal(dW, dWr)


def test_gcn_norm_known_answer():
    """Path graph 0-1-2 with self-loops: degrees (2, 3, 2)."""
    ei = torch.tensor([[0, 1, 1, 2], [1, 0, 2, 1]])
    A = O.normalized_adjacency_coo(ei, 3).to_dense()
    d = torch.tensor([2.0, 3.0, 2.0])
    expect = torch.tensor([[1, 1, 0], [1, 1, 1], [0, 1, 1]], dtype=torch.float32) / torch.sqrt(d[:, None] * d[None, :])
    assert torch.allclose(A, expect, rtol=1e-6, atol=0)
    assert torch.equal(A, A.t())


def test_gcn_norm_isolated_node_and_duplicates():
    # node 3 isolated (only its self-loop); edge (0,1) given twice
    ei = torch.tensor([[0, 1, 0, 1], [1, 0, 1, 0]])
    A = O.normalized_adjacency_coo(ei, 4)
    D = A.to_dense()
    assert float(D[3, 3]) == 1.0
    assert A._nnz() == 6  # (0,0) (0,1) (1,0) (1,1) (2,2) (3,3)
    rowptr, col, val = O.coo_to_csr_int32(A)
    assert rowptr.tolist() == [0, 2, 4, 5, 6]
    assert col.dtype == torch.int32 and rowptr.dtype == torch.int32

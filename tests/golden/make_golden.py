"""Generates the golden fixtures of this directory by running the reference's
OWN code on the CPU: src/graphcuda/cpp/gcn.cpp compiled by oracle/build_ref.py
and the unmodified src/graphcuda/python/gcn.py on top of it (see
oracle/ref_loader.py).  Needs the reference tree mounted; the resulting .npz
files are committed so the tests can run where it is not.

    python tests/golden/make_golden.py

Cases (all seeded, all small):
  layer_dense.npz    one layer fwd+bwd, dense adjacency, ReLU on
  layer_sparse.npz   one layer fwd+bwd, sparse COO adjacency with empty rows, ReLU off and on
  module_train.npz   2-layer model (python/gcn.py GCNConv), 5 Adam steps: weights, logits, losses
"""
from __future__ import annotations

import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle import ref_loader  # noqa: E402


def sym_norm_dense(n, density, gen):
    a = (torch.rand(n, n, generator=gen) < density).float()
    a = ((a + a.t()) > 0).float()
    a.fill_diagonal_(1.0)
    d = a.sum(1)
    dinv = d.pow(-0.5)
    return dinv[:, None] * a * dinv[None, :]


def main():
    ext = ref_loader.load_ref_ext()
    refpy = ref_loader.load_ref_python()
    torch.set_num_threads(1)

    g = torch.Generator().manual_seed(1234)
    n, fin, fout = 48, 20, 12
    A = sym_norm_dense(n, 0.15, g)
    X = torch.randn(n, fin, generator=g)
    W = torch.randn(fin, fout, generator=g) * 0.3
    dY = torch.randn(n, fout, generator=g)
    Y, mask = ext.gcn_conv_forward(X, A, W, True)
    dX, dW = ext.gcn_conv_backward(dY, X, A, W, True, mask)
    np.savez(os.path.join(HERE, "layer_dense.npz"), A=A.numpy(), X=X.numpy(), W=W.numpy(), dY=dY.numpy(),
             Y=Y.numpy(), mask=mask.numpy(), dX=dX.numpy(), dW=dW.numpy())

    g = torch.Generator().manual_seed(4321)
    n, fin, fout = 64, 9, 33
    A = sym_norm_dense(n, 0.08, g)
    A[5, :] = 0; A[:, 5] = 0; A[17, :] = 0; A[:, 17] = 0; A[63, :] = 0; A[:, 63] = 0  # empty rows
    Asp = A.to_sparse().coalesce()
    X = torch.randn(n, fin, generator=g)
    W = torch.randn(fin, fout, generator=g) * 0.3
    dY = torch.randn(n, fout, generator=g)
    Y0, _ = ext.gcn_conv_forward(X, Asp, W, False)
    dX0, dW0 = ext.gcn_conv_backward(dY, X, Asp, W, False, torch.empty(()))
    Y1, mask1 = ext.gcn_conv_forward(X, Asp, W, True)
    dX1, dW1 = ext.gcn_conv_backward(dY, X, Asp, W, True, mask1)
    np.savez(os.path.join(HERE, "layer_sparse.npz"), rows=Asp.indices()[0].numpy(), cols=Asp.indices()[1].numpy(),
             vals=Asp.values().numpy(), n=n, X=X.numpy(), W=W.numpy(), dY=dY.numpy(), Y0=Y0.numpy(),
             dX0=dX0.numpy(), dW0=dW0.numpy(), Y1=Y1.numpy(), mask1=mask1.numpy(), dX1=dX1.numpy(),
             dW1=dW1.numpy())

    # the reference's module and autograd function, trained like its script
    # (tests/gcn/graphcuda_impl.py:15-24,51-58) but seeded and with Adam lr=0.01
    g = torch.Generator().manual_seed(99)
    n, fin, hid, ncls = 40, 24, 8, 5
    A = sym_norm_dense(n, 0.12, g)
    X = (torch.rand(n, fin, generator=g) < 0.2).float()
    X = X / X.sum(1, keepdim=True).clamp_min(1)
    y = torch.randint(0, ncls, (n,), generator=g)
    torch.manual_seed(7)
    c1 = refpy.GCNConv(fin, hid, apply_relu=True)
    c2 = refpy.GCNConv(hid, ncls, apply_relu=False)
    W1_0, W2_0 = c1.weights.detach().clone(), c2.weights.detach().clone()
    opt = torch.optim.Adam(list(c1.parameters()) + list(c2.parameters()), lr=0.01)
    losses = []
    for _ in range(5):
        opt.zero_grad()
        out = torch.log_softmax(c2(c1(X, A), A), dim=1)
        loss = torch.nn.functional.nll_loss(out[:20], y[:20])
        loss.backward()
        opt.step()
        losses.append(loss.item())
    with torch.no_grad():
        logits = torch.log_softmax(c2(c1(X, A), A), dim=1)
    np.savez(os.path.join(HERE, "module_train.npz"), A=A.numpy(), X=X.numpy(), y=y.numpy(), W1_0=W1_0.numpy(),
             W2_0=W2_0.numpy(), W1=c1.weights.detach().numpy(), W2=c2.weights.detach().numpy(),
             logits=logits.numpy(), losses=np.array(losses, dtype=np.float64), seed=7)
    for f in sorted(os.listdir(HERE)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(os.path.join(HERE, f)), "bytes")


if __name__ == "__main__":
    main()

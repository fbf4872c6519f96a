"""Fused log_softmax + NLL against torch's own ops (the ones the reference's
script calls: tests/gcn/graphcuda_impl.py:24,55) on the CPU."""
import pytest
import torch

from oracle import gcn_oracle as O

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("M,C", [(1, 1), (5, 3), (1000, 7), (4097, 47), (300, 200)])
@pytest.mark.parametrize("masked", [False, True])
def test_loss_and_gradient(cuda, M, C, masked):
    from graphcuda_b200 import log_softmax_nll_loss
    g = torch.Generator().manual_seed(M * 31 + C)
    Z = torch.randn(M, C, generator=g) * 3
    y = torch.randint(0, C, (M,), generator=g)
    mask = (torch.rand(M, generator=g) < 0.3) if masked else None
    if masked and not mask.any():
        mask[0] = True
    Zr = Z.clone().requires_grad_()
    lp = torch.log_softmax(Zr, dim=1)
    ref = torch.nn.functional.nll_loss(lp[mask], y[mask]) if masked else torch.nn.functional.nll_loss(lp, y)
    (ref * 1.7).backward()
    Zg = Z.to(cuda).requires_grad_()
    loss = log_softmax_nll_loss(Zg, y.to(cuda), mask.to(cuda) if masked else None)
    (loss * 1.7).backward()
    assert abs(loss.item() - ref.item()) < 1e-5 * max(1.0, abs(ref.item()))
    assert O.rel_fro(Zg.grad, Zr.grad) < 1e-5
    if masked and bool((~mask).any()):
        assert float(Zg.grad[~mask.to(cuda)].abs().max()) == 0.0


def test_strided_logits_and_explicit_scale(cuda):
    from graphcuda_b200 import log_softmax_nll_loss
    Zp = torch.randn(500, 48)
    Z = Zp[:, :47]  # a view on a padded buffer, as the padded 47-class layer produces
    y = torch.randint(0, 47, (500,))
    ref = torch.nn.functional.nll_loss(torch.log_softmax(Z, 1), y, reduction="sum") / 12345.0
    Zg = Zp.to(cuda)[:, :47].requires_grad_()
    loss = log_softmax_nll_loss(Zg, y.to(cuda), scale=1.0 / 12345.0)
    loss.backward()
    assert abs(loss.item() - ref.item()) < 1e-6 * max(1.0, abs(ref.item())) + 1e-7
    a = log_softmax_nll_loss(Zg.detach(), y.to(cuda), scale=1.0).item()
    b = log_softmax_nll_loss(Zg.detach(), y.to(cuda), scale=1.0).item()
    assert a == b  # fixed reduction order


@pytest.mark.parametrize("M,C", [(1, 1), (5, 3), (1000, 7), (4097, 47), (300, 200)])
def test_argmax_and_accuracy_counts(cuda, M, C):
    """The script's test() tail (tests/gcn/graphcuda_impl.py:63-68): exact integers."""
    from graphcuda_b200 import argmax_accuracy
    g = torch.Generator().manual_seed(M * 17 + C)
    Z = torch.randn(M, C, generator=g)
    Z[::3] = torch.round(Z[::3])  # ties: the lowest index wins
    y = torch.randint(0, C, (M,), generator=g)
    masks = [torch.rand(M, generator=g) < p for p in (0.1, 0.5, 1.1)]
    want_pred = torch.stack([(Z[r] == Z[r].max()).nonzero()[0, 0] for r in range(M)]) if M <= 1000 else Z.argmax(1)
    pred, counts = argmax_accuracy(Z.to(cuda), y.to(cuda), [m.to(cuda) for m in masks])
    if M <= 1000:
        assert torch.equal(pred.cpu(), want_pred)
    else:  # torch does not promise which of several equal maxima it returns
        assert torch.equal(Z.gather(1, pred.cpu()[:, None])[:, 0], Z.max(1).values)
    hit = pred.cpu() == y
    want = torch.tensor([[int((hit & m).sum()), int(m.sum())] for m in masks])
    assert torch.equal(counts.cpu(), want)
    # all rows, no masks; prediction only
    _, c_all = argmax_accuracy(Z.to(cuda), y.to(cuda), want_pred=False)
    assert c_all.cpu().tolist() == [[int(hit.sum()), M]]
    p_only, none = argmax_accuracy(Z.to(cuda))
    assert none is None and torch.equal(p_only, pred)


def test_argmax_on_a_padded_view_and_errors(cuda):
    from graphcuda_b200 import argmax_accuracy
    Zp = torch.randn(64, 48)
    Zp[:, 47] = 100.0  # the padding column must not be seen
    pred, _ = argmax_accuracy(Zp.to(cuda)[:, :47])
    assert torch.equal(pred.cpu(), Zp[:, :47].argmax(1))
    with pytest.raises(RuntimeError):
        argmax_accuracy(torch.randn(4, 3))  # CPU tensors are rejected
    with pytest.raises(RuntimeError):
        argmax_accuracy(Zp.to(cuda), masks=torch.ones(64, dtype=torch.bool, device=cuda))  # masks without labels

"""Single-launch Adam / SGD against torch's own optimizers on the CPU (the
``optimizer.step()`` of the reference's script, tests/gcn/graphcuda_impl.py:45,56)."""
import pytest
import torch

pytestmark = pytest.mark.gpu

SHAPES = [(1433, 16), (16, 7), (5,), (1024,), (1025,), (300, 257)]


def _params(seed, device):
    g = torch.Generator().manual_seed(seed)
    return [torch.nn.Parameter(torch.randn(*s, generator=g).to(device)) for s in SHAPES]


def _grads(step, device):
    g = torch.Generator().manual_seed(1000 + step)
    return [torch.randn(*s, generator=g).to(device) for s in SHAPES]


@pytest.mark.parametrize("wd", [0.0, 0.05])
def test_fused_adam_follows_torch_adam(cuda, wd):
    from graphcuda_b200 import FusedAdam
    ref_p = _params(0, "cpu")
    our_p = _params(0, cuda)
    ref = torch.optim.Adam(ref_p, lr=0.01, betas=(0.9, 0.999), eps=1e-8, weight_decay=wd)
    ours = FusedAdam(our_p, lr=0.01, betas=(0.9, 0.999), eps=1e-8, weight_decay=wd)
    for step in range(6):
        for p, q, g in zip(ref_p, our_p, _grads(step, "cpu")):
            p.grad = g.clone()
            q.grad = g.to(cuda)
        ref.step()
        ours.step()
    assert ours.steps_taken() == 6
    for p, q in zip(ref_p, our_p):
        assert torch.allclose(q.detach().cpu(), p.detach(), rtol=2e-6, atol=2e-7)
        assert torch.allclose(ours.state[q]["exp_avg"].cpu(), ref.state[p]["exp_avg"], rtol=2e-6, atol=1e-6)
        assert torch.allclose(ours.state[q]["exp_avg_sq"].cpu(), ref.state[p]["exp_avg_sq"], rtol=1e-5, atol=1e-8)


def test_fused_adam_skips_parameters_without_gradient_and_many_tensors(cuda):
    from graphcuda_b200 import FusedAdam
    ps = [torch.nn.Parameter(torch.full((3,), float(i), device=cuda)) for i in range(70)]  # three launches
    ref = [torch.nn.Parameter(p.detach().cpu().clone()) for p in ps]
    ours, theirs = FusedAdam(ps, lr=0.1), torch.optim.Adam(ref, lr=0.1)
    for i, (p, r) in enumerate(zip(ps, ref)):
        if i % 7:
            p.grad = torch.full((3,), 0.5 + i, device=cuda)
            r.grad = torch.full((3,), 0.5 + i)
    ours.step()
    theirs.step()
    for p, r in zip(ps, ref):
        assert torch.allclose(p.detach().cpu(), r.detach(), rtol=2e-6, atol=1e-7)


def test_fused_sgd_is_the_scripts_optimizer(cuda):
    from graphcuda_b200 import FusedSGD
    ref_p, our_p = _params(2, "cpu"), _params(2, cuda)
    ref, ours = torch.optim.SGD(ref_p, lr=1.0, weight_decay=0.01), FusedSGD(our_p, lr=1.0, weight_decay=0.01)
    for step in range(3):
        for p, q, g in zip(ref_p, our_p, _grads(step, "cpu")):
            p.grad, q.grad = g.clone(), g.to(cuda)
        ref.step()
        ours.step()
    for p, q in zip(ref_p, our_p):
        assert torch.allclose(q.detach().cpu(), p.detach(), rtol=1e-6, atol=1e-6)


def test_rejects_cpu_parameters():
    from graphcuda_b200 import FusedAdam
    p = torch.nn.Parameter(torch.zeros(4))
    p.grad = torch.ones(4)
    with pytest.raises(RuntimeError):
        FusedAdam([p]).step()


def test_graph_replay_with_fused_adam_matches_eager_torch_adam(cuda):
    """The whole step -- layers, fused loss, backward, one-launch Adam -- as one CUDA graph."""
    from graphcuda_b200 import FusedAdam, GraphedTrainStep, log_softmax_nll_loss, normalized_adjacency, synth
    from graphcuda_b200.models import GCN
    cfg = synth.CONFIGS["cora_like"]
    n = cfg["nodes"]
    e = synth.preferential_attachment_edges(n, cfg["edges"], cfg["seed"]).to(cuda)
    adj = normalized_adjacency(synth.symmetrize(e), n, symmetric=True)
    X = synth.bow_features(n, cfg["features"], 0.0127, seed=1).to(cuda)
    y = synth.uniform_labels(n, cfg["classes"], seed=2).to(cuda)
    train = synth.planetoid_split(n)[0].to(cuda)
    dims = [cfg["features"], cfg["hidden"], cfg["classes"]]
    torch.manual_seed(5)
    eager = GCN(dims).to(cuda)
    torch.manual_seed(5)
    graphed = GCN(dims).to(cuda)
    opt_e = torch.optim.Adam(eager.parameters(), lr=0.01)
    warm = 3
    step = GraphedTrainStep(graphed, adj, X, y, FusedAdam(graphed.parameters(), lr=0.01), row_mask=train, warmup=warm)
    replays = 7
    for _ in range(replays):
        loss_g = step.step()
    # the capture records but does not execute: weights saw `warm` eager steps + `replays` replays
    for _ in range(warm + replays):
        opt_e.zero_grad(set_to_none=True)
        loss_e = log_softmax_nll_loss(eager(X, adj, log_softmax=False), y, train)
        loss_e.backward()
        opt_e.step()
    assert abs(loss_g.item() - loss_e.item()) < 1e-4 * max(1.0, abs(loss_e.item()))
    for a, b in zip(graphed.parameters(), eager.parameters()):
        assert torch.allclose(a, b, rtol=1e-3, atol=1e-5)

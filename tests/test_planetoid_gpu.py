"""The reference's training script flow (tests/gcn/graphcuda_impl.py) through
graphcuda_b200.train_planetoid on a synthetic data set in the Planetoid layout."""
import numpy as np
import pytest
import torch

from tests.test_planetoid import _write

pytestmark = pytest.mark.gpu


def _toy(tmp_path):
    ids = list(range(200, 260))
    np.random.default_rng(5).shuffle(ids)
    _write(str(tmp_path), "toy", n_train=20, n_other=180, test_ids=ids, n_feat=50, n_cls=4, seed=7)
    return str(tmp_path)


@pytest.mark.parametrize("optimizer", ["sgd", "adam"])
def test_script_flow_eager_and_graph_agree(cuda, tmp_path, optimizer, capsys):
    from graphcuda_b200.train_planetoid import main
    raw = _toy(tmp_path)
    common = ["--raw", raw, "--name", "toy", "--epochs", "6", "--optimizer", optimizer, "--seed", "11"]
    eager = main(common)
    graph = main(common + ["--graph"])
    out = capsys.readouterr().out
    assert out.count("Epoch 006 | Time:") == 2 and "Epoch 000 | Train Acc:" in out
    he, hg = eager["history"], graph["history"]
    assert len(he) == 7 and he[0]["epoch"] == 0
    assert he[-1]["loss"] < he[1]["loss"]  # it trains
    for a, b in zip(he[1:], hg[1:]):  # same kernels in the same order: same numbers
        assert a["loss"] == b["loss"]
        assert (a["train"], a["val"], a["test"]) == (b["train"], b["val"], b["test"])


def test_accuracy_lines_match_a_plain_torch_evaluation(cuda, tmp_path):
    import graphcuda_b200 as gc
    from graphcuda_b200.models import GCN
    from graphcuda_b200.planetoid import load_planetoid_raw
    d = load_planetoid_raw(_toy(tmp_path), "toy", n_val=30).to(cuda)
    adj = gc.normalized_adjacency(d.edge_index, d.num_nodes, symmetric=True)
    torch.manual_seed(1)
    model = GCN([d.num_node_features, 16, d.num_classes]).to(cuda)
    pred, counts = model.evaluate(d.x, adj, d.y, [d.train_mask, d.val_mask, d.test_mask])
    with torch.no_grad():
        ref_pred = model(d.x, adj).argmax(dim=1)
    assert torch.equal(pred, ref_pred)
    for i, m in enumerate([d.train_mask, d.val_mask, d.test_mask]):
        assert int(counts[i, 0]) == int((ref_pred[m] == d.y[m]).sum()) and int(counts[i, 1]) == int(m.sum())

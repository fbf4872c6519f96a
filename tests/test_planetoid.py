"""Planetoid raw-file reader (graphcuda_b200/planetoid.py): the data step of the
reference's script (tests/gcn/graphcuda_impl.py:12-13) without torch_geometric."""
import collections
import os
import pickle

import numpy as np
import pytest
import scipy.sparse as sp
import torch

from graphcuda_b200.planetoid import load_planetoid_raw
from oracle.build_ref import reference_root


def _write(dirpath, name, n_train, n_other, test_ids, n_feat, n_cls, seed, extra_edges=()):
    """A synthetic data set in the published layout; returns the expected (x, y, undirected edge set)."""
    rng = np.random.default_rng(seed)
    n_all = n_train + n_other
    lo, hi = min(test_ids), max(test_ids)
    n = hi + 1
    assert lo == n_all
    X = (rng.random((n, n_feat)) < 0.3).astype(np.float32)
    Y = rng.integers(0, n_cls, n)
    present = np.zeros(n, dtype=bool)
    present[:n_all] = True
    present[list(test_ids)] = True
    X[~present] = 0
    onehot = np.eye(n_cls, dtype=np.int32)[Y]
    onehot[~present] = 0
    graph = collections.defaultdict(list)
    edges = set()
    for _ in range(3 * n):
        u, v = (int(t) for t in rng.integers(0, n, 2))
        if present[u] and present[v]:
            graph[u].append(v)  # one direction only, with repeats and self-edges: the reader must clean up
            if u != v:
                edges.add((min(u, v), max(u, v)))
    for u, v in extra_edges:
        graph[u].append(v)
        edges.add((min(u, v), max(u, v)))
    t = list(test_ids)
    files = {"x": sp.csr_matrix(X[:n_train]), "allx": sp.csr_matrix(X[:n_all]), "tx": sp.csr_matrix(X[t]),
             "y": onehot[:n_train], "ally": onehot[:n_all], "ty": onehot[t], "graph": graph}
    for k, v in files.items():
        with open(os.path.join(dirpath, f"ind.{name}.{k}"), "wb") as f:
            pickle.dump(v, f, protocol=2)
    with open(os.path.join(dirpath, f"ind.{name}.test.index"), "w") as f:
        f.write("\n".join(str(i) for i in t) + "\n")
    Yexp = Y.copy()
    Yexp[~present] = 0
    return X, Yexp, edges, present


def test_reads_the_published_layout(tmp_path):
    test_ids = [37, 31, 39, 30, 33, 38, 32, 35, 34, 36]  # unsorted, as in the real files
    X, Y, edges, _ = _write(str(tmp_path), "toy", n_train=6, n_other=24, test_ids=test_ids, n_feat=11, n_cls=4, seed=0)
    d = load_planetoid_raw(str(tmp_path), "toy", n_val=8)
    assert d.num_nodes == 40 and d.num_node_features == 11 and d.num_classes == 4
    assert np.array_equal(d.x.numpy(), X) and np.array_equal(d.y.numpy(), Y)
    assert d.train_mask.nonzero().flatten().tolist() == list(range(6))
    assert d.val_mask.nonzero().flatten().tolist() == list(range(6, 14))
    assert d.test_mask.nonzero().flatten().tolist() == sorted(test_ids)
    r, c = d.edge_index
    assert int((r == c).sum()) == 0
    got = {(int(a), int(b)) for a, b in zip(r.tolist(), c.tolist())}
    assert got == {(u, v) for u, v in edges} | {(v, u) for u, v in edges}
    assert len(got) == d.edge_index.size(1)  # no duplicates
    key = r * 40 + c
    assert bool((key[1:] > key[:-1]).all())  # sorted by (row, col)


def test_gapped_test_range_leaves_isolated_zero_nodes(tmp_path):
    test_ids = [20, 23, 21, 25]  # 22 and 24 never appear (the citeseer case)
    X, Y, _, present = _write(str(tmp_path), "gap", n_train=4, n_other=16, test_ids=test_ids, n_feat=5, n_cls=3, seed=1)
    d = load_planetoid_raw(str(tmp_path), "gap", n_val=3)
    assert d.num_nodes == 26
    assert float(d.x[22].abs().sum()) == 0.0 and float(d.x[24].abs().sum()) == 0.0
    assert np.array_equal(d.x.numpy(), X)
    assert not bool(d.test_mask[22]) and int(d.test_mask.sum()) == 4
    touched = set(d.edge_index.flatten().tolist())
    assert 22 not in touched and 24 not in touched


def test_refuses_pickles_that_name_other_code(tmp_path):
    _write(str(tmp_path), "bad", n_train=2, n_other=4, test_ids=[6, 7], n_feat=3, n_cls=2, seed=2)
    with open(os.path.join(str(tmp_path), "ind.bad.ty"), "wb") as f:
        pickle.dump(os.path.join, f, protocol=2)  # a harmless stand-in for "some other callable"
    with pytest.raises(pickle.UnpicklingError):
        load_planetoid_raw(str(tmp_path), "bad")


@pytest.mark.skipif(not os.path.isdir(os.path.join(reference_root(), "data", "Cora", "raw")),
                    reason="reference tree not mounted")
def test_cora_files_of_the_reference_tree_have_the_known_shape():
    """Shape statistics only (the counts torch_geometric reports for Cora)."""
    d = load_planetoid_raw(os.path.join(reference_root(), "data", "Cora", "raw"), "cora")
    assert (d.num_nodes, d.num_node_features, d.num_classes) == (2708, 1433, 7)
    assert d.edge_index.size(1) == 10556
    assert (int(d.train_mask.sum()), int(d.val_mask.sum()), int(d.test_mask.sum())) == (140, 500, 1000)
    assert torch.equal(d.edge_index, d.edge_index.flip(0)[:, torch.argsort(d.edge_index[1] * 2708 + d.edge_index[0])])

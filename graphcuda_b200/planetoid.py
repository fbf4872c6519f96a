"""Reader for the Planetoid raw files (``ind.<name>.{x,tx,allx,y,ty,ally,graph,test.index}``)
that the reference's training script gets through ``torch_geometric.datasets.Planetoid``
(tests/gcn/graphcuda_impl.py:12-13; the files sit under ``data/Cora/raw`` of the reference tree).

With it the script's data step needs neither torch_geometric nor a download::

    d = load_planetoid_raw("<root>/data/Cora/raw", "cora")
    adj = graphcuda_b200.normalized_adjacency(d.edge_index.cuda(), d.num_nodes)   # lines 27-38 of the script
    out = model(d.x.cuda(), adj)

The layout is the published one of the Planetoid / GCN data release:
``x`` / ``tx`` / ``allx`` are pickled scipy CSR feature matrices of the labelled training nodes, the test
nodes and all non-test nodes, ``y`` / ``ty`` / ``ally`` the matching one-hot label arrays, ``graph`` a dict
``node -> [neighbours]`` and ``test.index`` the (unsorted) ids of the test nodes as text.  Node ids are: the
rows of ``allx`` first, then the test nodes in sorted order of ``test.index``; ids missing from a gapped test
range (citeseer) become isolated all-zero nodes.  Splits follow the standard setting: the ``len(y)`` labelled
nodes train, the next 500 validate, ``test.index`` tests.

The pickles are read with an unpickler that only resolves the numpy / scipy / collections names these
files need, so a tampered file cannot run other code.
"""
from __future__ import annotations

import io
import os
import pickle
from dataclasses import dataclass

import numpy as np
import torch

_ALLOWED = {
    ("numpy", "ndarray"), ("numpy", "dtype"),
    ("numpy.core.multiarray", "_reconstruct"), ("numpy._core.multiarray", "_reconstruct"),
    ("numpy.core.multiarray", "scalar"), ("numpy._core.multiarray", "scalar"),
    ("scipy.sparse.csr", "csr_matrix"), ("scipy.sparse._csr", "csr_matrix"),
    ("collections", "defaultdict"), ("collections", "OrderedDict"),
    ("_codecs", "encode"),  # how protocol-2 pickles written by Python 3 carry the bytes of an array
    ("builtins", "list"), ("__builtin__", "list"), ("builtins", "dict"), ("__builtin__", "dict"),
}


class _NamesOnly(pickle.Unpickler):
    def find_class(self, module, name):
        if (module, name) not in _ALLOWED:
            raise pickle.UnpicklingError(f"refusing to resolve {module}.{name} from a data file")
        if module == "__builtin__":
            module = "builtins"
        if module == "scipy.sparse.csr":  # where old files place the class; same class, current home
            module = "scipy.sparse"
        return super().find_class(module, name)


def _read_pickle(path: str):
    with open(path, "rb") as f:
        return _NamesOnly(io.BytesIO(f.read()), encoding="latin1").load()


@dataclass
class PlanetoidData:
    x: torch.Tensor            # [N, F] float32
    y: torch.Tensor            # [N] int64
    edge_index: torch.Tensor   # [2, E] int64: both directions, no self-edges, sorted by (row, col), no duplicates
    train_mask: torch.Tensor   # [N] bool
    val_mask: torch.Tensor
    test_mask: torch.Tensor
    num_classes: int

    @property
    def num_nodes(self) -> int:
        return int(self.x.size(0))

    @property
    def num_node_features(self) -> int:
        return int(self.x.size(1))

    def to(self, device) -> "PlanetoidData":
        return PlanetoidData(self.x.to(device), self.y.to(device), self.edge_index.to(device),
                             self.train_mask.to(device), self.val_mask.to(device), self.test_mask.to(device),
                             self.num_classes)


def _dense(m) -> np.ndarray:
    return np.asarray(m.todense() if hasattr(m, "todense") else m, dtype=np.float32)


def load_planetoid_raw(raw_dir: str, name: str = "cora", *, n_val: int = 500) -> PlanetoidData:
    name = name.lower()
    part = {k: _read_pickle(os.path.join(raw_dir, f"ind.{name}.{k}")) for k in ("x", "tx", "allx", "y", "ty", "ally",
                                                                                   "graph")}
    with open(os.path.join(raw_dir, f"ind.{name}.test.index")) as f:
        test_idx = np.array([int(line) for line in f.read().split()], dtype=np.int64)
    allx, tx = _dense(part["allx"]), _dense(part["tx"])
    ally, ty = np.asarray(part["ally"]), np.asarray(part["ty"])
    n_train = int(np.asarray(part["y"]).shape[0])
    order = np.sort(test_idx)
    lo, hi = int(order[0]), int(order[-1])
    if lo != allx.shape[0]:
        raise ValueError(f"{name}: test ids start at {lo}, expected {allx.shape[0]} (rows of allx)")
    if tx.shape[0] != test_idx.shape[0] or ty.shape[0] != test_idx.shape[0]:
        raise ValueError(f"{name}: tx / ty rows do not match test.index")
    # rows of tx / ty are in the order of test.index; ids absent from a gapped range stay zero
    span = hi - lo + 1
    tx_full = np.zeros((span, tx.shape[1]), dtype=np.float32)
    ty_full = np.zeros((span, ty.shape[1]), dtype=ty.dtype)
    tx_full[test_idx - lo] = tx
    ty_full[test_idx - lo] = ty
    x = np.vstack([allx, tx_full])
    onehot = np.vstack([ally, ty_full])
    y = onehot.argmax(axis=1).astype(np.int64)
    n = x.shape[0]

    rows, cols = [], []
    for u, nbrs in part["graph"].items():
        for v in nbrs:
            rows.append(int(u))
            cols.append(int(v))
    r = np.asarray(rows, dtype=np.int64)
    c = np.asarray(cols, dtype=np.int64)
    if r.size and (min(r.min(), c.min()) < 0 or max(r.max(), c.max()) >= n):
        raise ValueError(f"{name}: graph refers to a node outside 0..{n - 1}")
    keep = r != c
    r, c = r[keep], c[keep]
    key = np.unique(np.concatenate([r * n + c, c * n + r]))  # both directions, sorted, duplicates dropped
    edge_index = torch.from_numpy(np.stack([key // n, key % n]))

    train_mask = torch.zeros(n, dtype=torch.bool)
    val_mask = torch.zeros(n, dtype=torch.bool)
    test_mask = torch.zeros(n, dtype=torch.bool)
    train_mask[:n_train] = True
    val_mask[n_train:n_train + n_val] = True
    test_mask[torch.from_numpy(test_idx)] = True
    return PlanetoidData(torch.from_numpy(x), torch.from_numpy(y), edge_index, train_mask, val_mask, test_mask,
                         int(onehot.shape[1]))

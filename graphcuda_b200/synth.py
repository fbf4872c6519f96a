"""Seeded synthetic inputs with the shapes and value distributions of the
benchmark configurations (no datasets are needed or read):

  cora_like      N=2708, 5429 undirected preferential-attachment edges,
                 1433 Bernoulli(0.0127) bag-of-words features, row-normalised,
                 7 uniform classes, 140/500/1000 split
  rmat           R-MAT (a,b,c,d = .57,.19,.19,.05) undirected graphs
                 (169,343 nodes / 1,166,243 edges; 2,449,029 / 61,859,140)
  erdos_renyi    G(n, p) undirected (32,768 nodes, p = 0.01)

Edge generators return *undirected, distinct, non-self* edges as an int64
[2, E] tensor with u < v; ``symmetrize`` yields both directions.  They run on
whatever device they are given (CPU for the small parity cases, the GPU for
the 62 M-edge graph); the stream of random numbers differs between devices, so
parity tests generate on the CPU and copy.
"""
from __future__ import annotations

import math

import numpy as np
import torch


def symmetrize(edges: torch.Tensor) -> torch.Tensor:
    """[2, E] undirected (u < v) -> [2, 2E] directed, both directions."""
    return torch.cat([edges, edges.flip(0)], dim=1)


def preferential_attachment_edges(n: int, n_edges: int, seed: int) -> torch.Tensor:
    """Grow node by node, each newcomer attaching to existing nodes with
    probability proportional to degree, then add degree-proportional edges
    between existing nodes until exactly n_edges distinct undirected edges."""
    rng = np.random.default_rng(seed)
    per_node = max(1, n_edges // max(n - 1, 1))
    ends = [0, 1]  # every edge contributes both endpoints: sampling from it is degree-proportional
    seen = {(0, 1)}
    for v in range(2, n):
        want = min(per_node, v)
        picked = set()
        while len(picked) < want and len(seen) + len(picked) < n_edges:
            u = ends[rng.integers(len(ends))]
            if u != v:
                picked.add(u)
        for u in picked:
            seen.add((min(u, v), max(u, v)))
            ends.extend((u, v))
        if not picked:  # edge budget exhausted: keep the node connected anyway
            u = ends[rng.integers(len(ends))]
            seen.add((min(u, v), max(u, v)))
            ends.extend((u, v))
    while len(seen) < n_edges:
        u = ends[rng.integers(len(ends))]
        v = ends[rng.integers(len(ends))]
        if u != v and (min(u, v), max(u, v)) not in seen:
            seen.add((min(u, v), max(u, v)))
            ends.extend((u, v))
    e = np.array(sorted(seen)[:n_edges] if len(seen) > n_edges else sorted(seen), dtype=np.int64).T
    return torch.from_numpy(np.ascontiguousarray(e))


def _unique_undirected(u: torch.Tensor, v: torch.Tensor, n: int) -> torch.Tensor:
    keep = (u != v) & (u < n) & (v < n)
    u, v = u[keep], v[keep]
    lo, hi = torch.minimum(u, v), torch.maximum(u, v)
    return torch.unique(lo * n + hi)


def rmat_edges(scale: int, n_nodes: int, n_edges: int, seed: int, device="cpu",
               abcd=(0.57, 0.19, 0.19, 0.05), scramble: bool = True) -> torch.Tensor:
    """R-MAT on 2**scale ids; ids >= n_nodes, self-edges and duplicates are
    dropped; draws until n_edges distinct undirected edges exist and keeps a
    seeded random subset of exactly that many.  With `scramble` the vertex
    labels are then permuted at random (as the Graph500 generator does), so
    that the heavy vertices are not the low ids and contiguous row blocks of
    the adjacency carry similar numbers of edges."""
    a, b, c, _ = abcd
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    keys = torch.empty(0, dtype=torch.int64, device=device)
    batch = int(n_edges * 1.15) + 1024
    chunk = 1 << 24
    for _ in range(64):
        parts = []
        for s in range(0, batch, chunk):
            m = min(chunk, batch - s)
            u = torch.zeros(m, dtype=torch.int64, device=device)
            v = torch.zeros(m, dtype=torch.int64, device=device)
            for _level in range(scale):
                r = torch.rand(m, generator=g, device=device)
                # quadrants: a -> (0,0), b -> (0,1), c -> (1,0), d -> (1,1)
                ubit = (r >= a + b).to(torch.int64)
                vbit = (((r >= a) & (r < a + b)) | (r >= a + b + c)).to(torch.int64)
                u = (u << 1) | ubit
                v = (v << 1) | vbit
            parts.append(_unique_undirected(u, v, n_nodes))
        keys = torch.unique(torch.cat([keys] + parts))
        if keys.numel() >= n_edges:
            break
        batch = int((n_edges - keys.numel()) * 1.5) + 1024
    if keys.numel() < n_edges:
        raise RuntimeError("R-MAT generator could not reach the requested number of distinct edges")
    if keys.numel() > n_edges:
        perm = torch.randperm(keys.numel(), generator=g, device=device)[:n_edges]
        keys = keys[perm.sort().values]
    u, v = keys // n_nodes, keys % n_nodes
    if scramble:
        relabel = torch.randperm(n_nodes, generator=g, device=device)
        u, v = relabel[u], relabel[v]
        keys = torch.sort(torch.minimum(u, v) * n_nodes + torch.maximum(u, v)).values
        u, v = keys // n_nodes, keys % n_nodes
    return torch.stack([u, v])


def erdos_renyi_edges(n: int, p: float, seed: int, device="cpu") -> torch.Tensor:
    """G(n, m) with m = round(p * n(n-1)/2) distinct undirected edges drawn
    uniformly (the fixed-size twin of G(n, p))."""
    m = int(round(p * n * (n - 1) / 2))
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    keys = torch.empty(0, dtype=torch.int64, device=device)
    need = m
    for _ in range(64):
        k = int(need * 1.1) + 1024
        u = torch.randint(0, n, (k,), generator=g, device=device)
        v = torch.randint(0, n, (k,), generator=g, device=device)
        keys = torch.unique(torch.cat([keys, _unique_undirected(u, v, n)]))
        if keys.numel() >= m:
            break
        need = m - keys.numel()
    if keys.numel() > m:
        perm = torch.randperm(keys.numel(), generator=g, device=device)[:m]
        keys = keys[perm.sort().values]
    return torch.stack([keys // n, keys % n])


def bow_features(n: int, f: int, p: float, seed: int, device="cpu") -> torch.Tensor:
    """Binary bag-of-words (Bernoulli p) with each row scaled to sum 1; empty
    rows stay zero."""
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    x = (torch.rand(n, f, generator=g, device=device) < p).to(torch.float32)
    s = x.sum(1, keepdim=True)
    return x / s.clamp_min(1.0)


def normal_features(n: int, f: int, seed: int, device="cpu") -> torch.Tensor:
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return torch.randn(n, f, generator=g, device=device)


def uniform_labels(n: int, classes: int, seed: int, device="cpu") -> torch.Tensor:
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return torch.randint(0, classes, (n,), generator=g, device=device)


def reference_init(in_dim: int, out_dim: int, seed: int, device="cpu") -> torch.Tensor:
    """uniform(-s, s), s = sqrt(2 / (in + out)): the reference's initialiser
    (src/graphcuda/python/gcn.py:43-45)."""
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    s = math.sqrt(2.0 / (in_dim + out_dim))
    return (torch.rand(in_dim, out_dim, generator=g, device=device) * 2 - 1) * s


def planetoid_split(n: int, n_train=140, n_val=500, n_test=1000):
    """First n_train / next n_val / last n_test nodes."""
    train = torch.zeros(n, dtype=torch.bool)
    val = torch.zeros(n, dtype=torch.bool)
    test = torch.zeros(n, dtype=torch.bool)
    train[:n_train] = True
    val[n_train:n_train + n_val] = True
    test[n - n_test:] = True
    return train, val, test


CONFIGS = {
    # name: nodes, undirected edges, R-MAT scale (None: other generator)
    "cora_like": dict(nodes=2708, edges=5429, features=1433, hidden=16, classes=7, seed=0),
    "rmat_arxiv": dict(nodes=169_343, edges=1_166_243, scale=18, features=128, out=256, seed=2),
    "er_dense": dict(nodes=32_768, p=0.01, features=512, out=256, seed=3),
    "rmat_products": dict(nodes=2_449_029, edges=61_859_140, scale=22, features=100, hidden=256, classes=47, seed=4),
}

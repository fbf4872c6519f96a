"""Shared builders for the GPU parity tests (CPU side = the oracle)."""
import torch

from oracle import gcn_oracle as O


def random_csr(n_rows, n_cols, avg_deg, seed, long_rows=(), empty_rows=()):
    """Random coalesced COO (CPU) with chosen long and empty rows."""
    g = torch.Generator().manual_seed(seed)
    nnz = int(n_rows * avg_deg)
    r = torch.randint(0, n_rows, (nnz,), generator=g)
    c = torch.randint(0, n_cols, (nnz,), generator=g)
    parts_r, parts_c = [r], [c]
    for row, deg in long_rows:
        cc = torch.randperm(n_cols, generator=g)[:deg]
        parts_r.append(torch.full((cc.numel(),), row, dtype=torch.int64))
        parts_c.append(cc)
    r = torch.cat(parts_r)
    c = torch.cat(parts_c)
    if len(empty_rows):
        keep = ~torch.isin(r, torch.tensor(list(empty_rows)))
        r, c = r[keep], c[keep]
    v = torch.randn(r.numel(), generator=g)
    return torch.sparse_coo_tensor(torch.stack([r, c]), v, (n_rows, n_cols)).coalesce()


def to_gpu_csr(A_coo, device):
    from graphcuda_b200 import CSRAdjacency
    rowptr, col, val = O.coo_to_csr_int32(A_coo)
    return CSRAdjacency(rowptr.to(device), col.to(device), val.to(device), A_coo.shape)


def sym_norm_graph(edges_undirected, n):
    """Oracle-side normalised adjacency (coalesced COO, CPU) of an undirected edge list."""
    from graphcuda_b200 import synth
    return O.normalized_adjacency_coo(synth.symmetrize(edges_undirected), n)


def untie(dY, pre_ref, rel=1e-4):
    """Zeroes the upstream gradient where the reference pre-activation is within
    `rel` of zero (relative to its largest magnitude).  The ReLU mask of such an
    element is decided by rounding, so two correct implementations may disagree
    on it; everywhere else the gradient comparison is unaffected."""
    dY = dY.clone()
    dY[pre_ref.abs() < rel * pre_ref.abs().max()] = 0
    return dY

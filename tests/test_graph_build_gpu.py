"""GPU adjacency construction vs the oracle: CSR structure identical, values
bit-identical (integer / IEEE-rounded work: no tolerance)."""
import pytest
import torch

from oracle import gcn_oracle as O

pytestmark = pytest.mark.gpu


def _bits(t):
    return t.cpu().contiguous().view(torch.int32)


def _check_bit_exact(adj, A_ref):
    rowptr, col, val = O.coo_to_csr_int32(A_ref)
    assert torch.equal(adj.rowptr.cpu(), rowptr)
    assert torch.equal(adj.col.cpu(), col)
    assert torch.equal(_bits(adj.val), _bits(val))


def test_normalized_adjacency_cora_like(cuda):
    from graphcuda_b200 import normalized_adjacency, synth
    e = synth.preferential_attachment_edges(2708, 5429, 0)
    ei = synth.symmetrize(e)
    adj = normalized_adjacency(ei.to(cuda), 2708)
    A_ref = O.normalized_adjacency_coo(ei, 2708)
    assert adj.nnz == 2 * 5429 + 2708
    _check_bit_exact(adj, A_ref)
    assert adj.symmetric


def test_normalized_adjacency_rmat_with_isolated_nodes_and_hubs(cuda):
    from graphcuda_b200 import normalized_adjacency, synth
    n = 20000
    e = synth.rmat_edges(15, n, 150_000, 7)
    ei = synth.symmetrize(e)
    adj = normalized_adjacency(ei.to(cuda), n)
    _check_bit_exact(adj, O.normalized_adjacency_coo(ei, n))
    assert adj.symmetric


def test_duplicate_edges_are_summed_like_coalesce(cuda):
    from graphcuda_b200 import normalized_adjacency
    ei = torch.tensor([[0, 1, 0, 1, 2, 0, 1], [1, 0, 1, 0, 0, 2, 0]])
    adj = normalized_adjacency(ei.to(cuda), 5)
    _check_bit_exact(adj, O.normalized_adjacency_coo(ei, 5))


def test_gcn_norm_weights_bit_exact_for_many_degrees(cuda):
    """A star per degree value: deg^-1/2 products for degrees 1..3000."""
    from graphcuda_b200 import gcn_norm
    rows, cols = [], []
    base = 0
    hubs = list(range(1, 60)) + [100, 255, 256, 257, 999, 1000, 2047, 2048, 3000]
    for d in hubs:
        leaves = torch.arange(base + 1, base + 1 + d)
        rows += [torch.full((d,), base), leaves]
        cols += [leaves, torch.full((d,), base)]
        base += d + 1
    ei = O.add_self_loops(torch.stack([torch.cat(rows), torch.cat(cols)]), base)
    w = gcn_norm(ei.to(cuda), base)
    assert torch.equal(_bits(w), _bits(O.gcn_norm(ei, base)))


def test_coo_and_csr_tensor_inputs(cuda):
    from graphcuda_b200 import as_adjacency, synth
    e = synth.rmat_edges(12, 3000, 20000, 3)
    A = O.normalized_adjacency_coo(synth.symmetrize(e), 3000)
    a1 = as_adjacency(A.to(cuda))
    _check_bit_exact(a1, A)
    a2 = as_adjacency(A.to_sparse_csr().to(cuda))
    _check_bit_exact(a2, A)
    rowptr, col, val = O.coo_to_csr_int32(A)
    a3 = as_adjacency((rowptr.to(cuda), col.to(cuda), val.to(cuda)))
    _check_bit_exact(a3, A)
    # cached on the tensor's identity
    Ag = A.to(cuda)
    assert as_adjacency(Ag) is as_adjacency(Ag)


def test_symmetry_verdict(cuda):
    from graphcuda_b200 import as_adjacency
    from tests.helpers import random_csr
    A = random_csr(200, 200, 5.0, seed=1)
    assert not as_adjacency(A.to(cuda)).symmetric
    S = (A + A.t()).coalesce()
    assert as_adjacency(S.to(cuda)).symmetric
    D = S.to_dense()
    assert as_adjacency(D.to(cuda)).symmetric
    D[3, 4] += 1.0
    assert not as_adjacency(D.to(cuda)).symmetric


def test_degree_reordering_is_the_oracle_adjacency_of_the_relabelled_graph(cuda):
    """reorder="degree": the CSR equals, bit for bit, what the oracle builds from the relabelled edge list;
    the permutation is by decreasing degree (ties by old id) and products commute with it."""
    from graphcuda_b200 import degree_order, normalized_adjacency, synth
    n = 20000
    e = synth.rmat_edges(15, n, 150_000, 7)
    ei = synth.symmetrize(e)
    adj = normalized_adjacency(ei.to(cuda), n, reorder="degree")
    perm, inv = adj.perm.cpu(), adj.inv_perm.cpu()
    deg = torch.bincount(ei[1], minlength=n)
    assert torch.equal(perm, torch.argsort(deg, descending=True, stable=True))
    assert torch.equal(inv[perm], torch.arange(n))
    p2, i2 = degree_order(ei, n)  # the same helper on the CPU
    assert torch.equal(p2, perm) and torch.equal(i2, inv)
    _check_bit_exact(adj, O.normalized_adjacency_coo(inv[ei], n))
    new_deg = (adj.rowptr[1:] - adj.rowptr[:-1]).cpu()
    assert bool((new_deg[:-1] >= new_deg[1:]).all())  # heavy vertices first
    # (P A P^T)(P H) = P (A H): aggregate in the new order, read the result back in the old one
    plain = normalized_adjacency(ei.to(cuda), n)
    H = torch.randn(n, 64, generator=torch.Generator().manual_seed(1)).to(cuda)
    Y_old = plain.matmul(H)
    Y_new = adj.matmul(H[adj.perm])
    assert O.rel_fro(Y_new[adj.inv_perm], Y_old) < 1e-5

"""The no-allocation aggregation entry point, called through the C ABI.

Some users of this library cannot allocate device memory where they need the
product (a host application that owns all GPU memory, a serving loop with a
frozen budget), so ``gc_spmm_csr_f32_noalloc`` keeps its long-row
scratch in a fixed buffer inside the library.  It must give exactly what the
ordinary entry point gives with caller-provided scratch, on repeated calls
(the buffer keeps the previous call's contents), and refuse problems whose
scratch bound exceeds the built-in buffer.

Collected last on purpose: a failure here does not hide any other test.
"""
import pytest
import torch

from oracle import gcn_oracle as O
from tests.helpers import random_csr, to_gpu_csr

pytestmark = pytest.mark.gpu


def _call_noalloc(L, adj, H, Y, bias=None, epilogue=0, n_slots=None):
    M, K = adj.shape
    F = H.size(1)
    plan = adj.plan_for(F)
    return L.gc_spmm_csr_f32_noalloc(
        adj.rowptr.data_ptr(), adj.col.data_ptr(), adj.val.data_ptr(), M, K, F,
        H.data_ptr(), F, bias.data_ptr() if bias is not None else None, epilogue, Y.data_ptr(), F, None, None,
        plan.buf.data_ptr(), plan.n_pieces, plan.n_slots if n_slots is None else n_slots, plan.n_cut,
        torch.cuda.current_stream().cuda_stream)


def test_noalloc_matches_the_ordinary_entry_point_twice_in_a_row(cuda):
    from graphcuda_b200 import _lib
    L = _lib.lib()
    # long rows of several segments so the scratch is really used
    A = random_csr(6000, 9000, 6.0, seed=31, long_rows=((5, 1500), (77, 5000), (5999, 8000)))
    adj = to_gpu_csr(A, cuda)
    assert adj.plan_counts(64)[1] >= 3 + 4  # partial-sum slots of the two rows above 2048 non-zeros
    g = torch.Generator().manual_seed(3)
    for F, relu in ((64, False), (256, True)):
        H1 = torch.randn(9000, F, generator=g).to(cuda)
        H2 = torch.randn(9000, F, generator=g).to(cuda)
        b = torch.randn(F, generator=g).to(cuda)
        for H in (H1, H2):  # two calls in a row share the built-in buffer
            expect = adj.matmul(H, bias=b, relu=relu)  # gc_spmm_csr_f32 with caller scratch
            Y = torch.full_like(expect, float("nan"))
            before = torch.cuda.memory_allocated()
            st = _call_noalloc(L, adj, H, Y, bias=b, epilogue=_lib.EPI_RELU if relu else 0)
            assert st == 0, L.gc_last_error()
            assert torch.cuda.memory_allocated() == before
            torch.cuda.synchronize()
            assert torch.equal(Y, expect)  # same kernels, same order of additions: bit-identical
            assert torch.allclose(Y, expect, rtol=1e-4, atol=1e-6)
            # and against the CPU oracle directly, not only through the ordinary entry point
            pre = O.spmm(A, H.cpu()) + b.cpu()
            assert O.rel_fro(Y, pre * (pre > 0) if relu else pre) < 1e-4


def test_noalloc_refuses_what_does_not_fit(cuda):
    from graphcuda_b200 import _lib
    L = _lib.lib()
    Y = torch.empty(500, 32, device=cuda)
    A = random_csr(500, 5000, 4.0, seed=1, long_rows=((1, 4500),))
    adj = to_gpu_csr(A, cuda)
    H = torch.randn(5000, 32, device=cuda)
    # claim more partial-sum rows than the built-in scratch can hold
    too_many = _lib.SPMM_STATIC_SCRATCH_BYTES // (32 * 4) + 8
    st = _call_noalloc(L, adj, H, Y, n_slots=too_many)
    assert st == -4 and b"built-in" in L.gc_last_error()
    assert L.gc_spmm_scratch_bytes(too_many, 32) > _lib.SPMM_STATIC_SCRATCH_BYTES

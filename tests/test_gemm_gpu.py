"""Dense GEMM back ends vs the oracle (A @ B on CPU), through the C ABI."""
import pytest
import torch

from oracle import gcn_oracle as O

pytestmark = pytest.mark.gpu

TOL_FP32 = 1e-4
TOL_TF32 = 1e-2


def _rand(m, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.rand(m, n, generator=g) * 2 - 1  # uniform(-1, 1)


@pytest.mark.parametrize("shape", [(1, 1, 1), (5, 7, 3), (64, 64, 64), (65, 63, 17), (130, 200, 33),
                                   (2708, 16, 1433), (2708, 7, 16), (300, 47, 256), (257, 129, 1000)])
@pytest.mark.parametrize("ta,tb", [(0, 0), (0, 1), (1, 0), (1, 1)])
def test_simt_all_layouts(cuda, shape, ta, tb):
    from graphcuda_b200 import gemm
    M, N, K = shape
    A = _rand(M, K, 1)
    B = _rand(K, N, 2)
    ref = O.matmul(A, B)
    Ag = (A.t().contiguous().to(cuda).t() if ta else A.to(cuda))
    Bg = (B.t().contiguous().to(cuda).t() if tb else B.to(cuda))
    out = gemm(Ag, Bg, precision="fp32_simt")
    assert out.shape == (M, N)
    assert O.rel_fro(out, ref) < TOL_FP32 and O.rel_max(out, ref) < TOL_FP32


def test_simt_split_k_weight_gradient_shape(cuda):
    from graphcuda_b200 import gemm
    A = _rand(200_000, 40, 3)   # (A X): N_nodes x in
    G = _rand(200_000, 24, 4)   # N_nodes x out
    ref = O.matmul(A.t().double(), G.double()).float()
    out = gemm(A.to(cuda).t(), G.to(cuda), precision="fp32_simt")
    assert O.rel_fro(out, ref) < TOL_FP32
    out2 = gemm(A.to(cuda).t(), G.to(cuda), precision="fp32_simt")
    assert torch.equal(out, out2)  # fixed summation order


def test_simt_epilogue(cuda):
    from graphcuda_b200 import gemm
    A, B, b = _rand(300, 50, 5), _rand(50, 70, 6), _rand(1, 70, 7)[0]
    pre = O.matmul(A, B) + b
    Y, mask = gemm(A.to(cuda), B.to(cuda), bias=b.to(cuda), relu=True, want_mask=True, precision="fp32_simt")
    assert O.rel_fro(Y, pre * (pre > 0)) < TOL_FP32
    diff = mask.cpu() != (pre > 0).float()
    assert float(pre[diff].abs().max() if diff.any() else 0.0) < 1e-5
    Yt = gemm(A.to(cuda), B.to(cuda), transposed_out=True, precision="fp32_simt")
    assert Yt.shape == (70, 300) and O.rel_fro(Yt.t(), O.matmul(A, B)) < TOL_FP32


TC_SHAPES = [(128, 64, 32), (128, 256, 64), (256, 128, 96), (1000, 256, 100), (4096, 256, 256),
             (777, 47, 256), (3000, 300, 130), (512, 512, 512), (129, 65, 33), (20000, 256, 128)]


@pytest.mark.parametrize("shape", TC_SHAPES)
@pytest.mark.parametrize("prec,tol", [("tf32x3", TOL_FP32), ("tf32", TOL_TF32)])
def test_tensor_core_nt_form(cuda, shape, prec, tol):
    """A row-major, B given as its transpose (N x K): both operands K-major, no
    pre-pass except the low-part split."""
    from graphcuda_b200 import gemm, ops
    M, N, K = shape
    K4 = (K + 3) // 4 * 4  # the tensor-core path needs 16-byte row pitches
    A = _rand(M, K4, 11)[:, :K]
    Bt = _rand(N, K4, 12)[:, :K]
    ref = O.matmul(A.double(), Bt.t().double()).float()
    Ag = _rand(M, K4, 11).to(cuda)[:, :K]
    Btg = _rand(N, K4, 12).to(cuda)[:, :K]
    out = gemm(Ag, Btg.t(), precision=prec)
    ops.check_gemm_flag(cuda)
    assert O.rel_fro(out, ref) < tol, (O.rel_fro(out, ref), O.rel_max(out, ref))
    assert O.rel_max(out, ref) < tol * 4


@pytest.mark.parametrize("ta,tb", [(0, 0), (1, 0), (1, 1)])
def test_tensor_core_other_layouts(cuda, ta, tb):
    from graphcuda_b200 import gemm, ops
    M, N, K = 1500, 200, 260
    A, B = _rand(M, K, 21), _rand(K, N, 22)
    ref = O.matmul(A.double(), B.double()).float()
    Ag = (A.t().contiguous().to(cuda).t() if ta else A.to(cuda))
    Bg = (B.t().contiguous().to(cuda).t() if tb else B.to(cuda))
    out = gemm(Ag, Bg, precision="tf32x3")
    ops.check_gemm_flag(cuda)
    assert O.rel_fro(out, ref) < TOL_FP32


@pytest.mark.parametrize("prec,tol", [("tf32x3", TOL_FP32), ("tf32", TOL_TF32)])
@pytest.mark.parametrize("shape", [(256, 256, 100_000), (100, 256, 70_001), (256, 48, 50_000), (128, 64, 4096),
                                   (300, 200, 20_000)])
def test_tensor_core_weight_gradient_form(cuda, shape, prec, tol):
    """C = A^T B with A stored K x M and B stored K x N (both read in place,
    MN-major in shared memory), K split across CTAs, partials reduced in order."""
    from graphcuda_b200 import gemm, ops
    M, N, K = shape
    A = _rand(K, M, 41)
    B = _rand(K, N, 42)
    ref = O.matmul(A.t().double(), B.double()).float()
    Ag, Bg = A.to(cuda), B.to(cuda)
    out = gemm(Ag.t(), Bg, precision=prec)
    ops.check_gemm_flag(cuda)
    assert O.rel_fro(out, ref) < tol, (O.rel_fro(out, ref), O.rel_max(out, ref))
    out2 = gemm(Ag.t(), Bg, precision=prec)
    assert torch.equal(out, out2)  # split-K partials are added in a fixed order


@pytest.mark.parametrize("prec,tol", [("tf32x3", TOL_FP32), ("tf32", TOL_TF32)])
def test_tensor_core_large_b_operands(cuda, prec, tol):
    """B too large to be re-laid: consumed in place, MN-major (A @ B with B
    stored K x N, e.g. a dense adjacency times features) or K-major (A @ Bt^T),
    its low part made in shared memory."""
    from graphcuda_b200 import gemm, ops
    A, B = _rand(1024, 6000, 51), _rand(6000, 512, 52)          # N*K = 3.07 M elements
    ref = O.matmul(A.double(), B.double()).float()
    out = gemm(A.to(cuda), B.to(cuda), precision=prec)
    ops.check_gemm_flag(cuda)
    assert O.rel_fro(out, ref) < tol, O.rel_fro(out, ref)
    Bt = _rand(1100, 2100, 53)                                    # N x K, 2.31 M elements
    A2 = _rand(3000, 2100, 54)
    ref2 = O.matmul(A2.double(), Bt.t().double()).float()
    out2 = gemm(A2.to(cuda), Bt.to(cuda).t(), precision=prec)
    ops.check_gemm_flag(cuda)
    assert O.rel_fro(out2, ref2) < tol, O.rel_fro(out2, ref2)


def test_tensor_core_epilogue(cuda):
    from graphcuda_b200 import gemm, ops
    A, B, b = _rand(1000, 128, 31), _rand(128, 256, 32), _rand(1, 256, 33)[0]
    pre = O.matmul(A, B) + b
    Y, mask = gemm(A.to(cuda), B.to(cuda), bias=b.to(cuda), relu=True, want_mask=True, precision="tf32x3")
    ops.check_gemm_flag(cuda)
    assert O.rel_fro(Y, pre * (pre > 0)) < TOL_FP32
    diff = mask.cpu() != (pre > 0).float()
    assert float(pre[diff].abs().max() if diff.any() else 0.0) < 1e-3
    Yt = gemm(A.to(cuda), B.to(cuda), transposed_out=True, precision="tf32x3")
    assert Yt.shape == (256, 1000) and O.rel_fro(Yt.t(), O.matmul(A, B)) < TOL_FP32


def test_tensor_core_matches_simt_on_device(cuda):
    """Large persistent case (more tiles than SMs, both TMEM buffers cycling):
    split-TF32 vs the fp32 CUDA-core kernel, on device."""
    from graphcuda_b200 import gemm, ops
    g = torch.Generator(device=cuda).manual_seed(0)
    A = torch.rand(40_000, 256, generator=g, device=cuda) * 2 - 1
    B = torch.rand(256, 256, generator=g, device=cuda) * 2 - 1
    ref = gemm(A, B, precision="fp32_simt")
    out = gemm(A, B, precision="tf32x3")
    ops.check_gemm_flag(cuda)
    assert O.rel_fro(out, ref) < TOL_FP32
    out1 = gemm(A, B, precision="tf32")
    assert O.rel_fro(out1, ref) < TOL_TF32


def test_auto_precision_dispatch(cuda):
    from graphcuda_b200 import ops
    small = torch.empty(2708, 1433, device=cuda), torch.empty(1433, 16, device=cuda)
    big = torch.empty(169_343, 128, device=cuda), torch.empty(128, 256, device=cuda)
    assert ops.gemm_path(*small) == "fp32_simt"
    assert ops.gemm_path(*big) == "tf32x3"
    assert ops.gemm_path(*big, precision="tf32") == "tf32"


@pytest.mark.parametrize("name", ["matmul1", "matmul2", "matmul3", "matmul4", "gemm_cublas"])
def test_reference_operator_names(cuda, name):
    """Same names, shapes and error behaviour as the reference operators
    (matmul1.cu:27-31, gemm_cublas.cu:3-7); matmul3's mixed tile shapes (M >= 128 > N)
    and matmul4's N % 4 != 0 are correct here."""
    import graphcuda
    fn = getattr(graphcuda, name)
    for (M, N, K) in [(512, 512, 512), (300, 64, 128), (130, 7, 50), (1024, 1024, 256)]:
        A, B = _rand(M, K, M + N), _rand(K, N, K)
        out = fn(A.to(cuda), B.to(cuda))
        assert O.rel_fro(out, O.matmul(A, B)) < TOL_FP32
    with pytest.raises(RuntimeError):
        fn(torch.randn(4, 5, device=cuda), torch.randn(6, 4, device=cuda))
    with pytest.raises(RuntimeError):
        fn(torch.randn(4, 5), torch.randn(5, 4))
    with pytest.raises(RuntimeError):
        fn(torch.randn(4, 5, 2, device=cuda), torch.randn(5, 4, device=cuda))
    # non-contiguous inputs are accepted (the reference copies them: gemm_cublas.cu:11-16)
    A, B = _rand(40, 30, 1), _rand(50, 30, 2)
    out = fn(A.to(cuda), B.to(cuda).t())
    assert O.rel_fro(out, O.matmul(A, B.t())) < TOL_FP32


@pytest.mark.parametrize("S", [512, 1024, 2048])
def test_square_sweep(cuda, S):
    import graphcuda
    A, B = _rand(S, S, S), _rand(S, S, S + 1)
    ref = O.matmul(A, B)
    assert O.rel_fro(graphcuda.gemm_cublas(A.to(cuda), B.to(cuda)), ref) < TOL_FP32


# ---------------------------------------------------------------- bf16 tier (opt-in, 1e-2)
TOL_BF16 = 1e-2


@pytest.mark.parametrize("shape", TC_SHAPES + [(300, 200, 7), (1, 1, 1), (2048, 2048, 2048)])
@pytest.mark.parametrize("ta,tb", [(0, 0), (0, 1), (1, 0), (1, 1)])
def test_bf16_tier_all_layouts(cuda, shape, ta, tb):
    """precision="bf16": both operands are converted to bf16 (round to nearest even) into the workspace, in any of
    the four storage layouts and with odd sizes / pitches, then multiplied with kind::f16 MMAs and fp32
    accumulation.  Reference: the same product in float64; tolerance of the reduced-precision tier."""
    from graphcuda_b200 import gemm, ops
    M, N, K = shape
    A, B = _rand(M, K, 61), _rand(K, N, 62)
    ref = O.matmul(A.double(), B.double()).float()
    Ag = (A.t().contiguous().to(cuda).t() if ta else A.to(cuda))
    Bg = (B.t().contiguous().to(cuda).t() if tb else B.to(cuda))
    # gemm(precision="bf16") takes the bf16 engine for compute-bound products only; here the engine itself is
    # exercised on every shape: operands converted (and re-laid K-major) exactly as gc_gemm_f32 does, then multiplied
    out = ops.gemm_bf16_operands(ops.to_bf16(Ag), ops.to_bf16(Bg, transpose=True))
    ops.check_gemm_flag(cuda)
    assert O.rel_fro(out, ref) < TOL_BF16, (O.rel_fro(out, ref), O.rel_max(out, ref))
    # against the product of the rounded operands the error is only the fp32 accumulation
    ref16 = O.matmul(A.bfloat16().double(), B.bfloat16().double()).float()
    assert O.rel_fro(out, ref16) < 1e-5, O.rel_fro(out, ref16)


def test_bf16_conversion_rounds_to_nearest_even(cuda):
    from graphcuda_b200 import ops
    g = torch.Generator().manual_seed(5)
    X = torch.randn(257, 131, generator=g) * torch.logspace(-20, 20, 131)
    X[0, :4] = torch.tensor([float("inf"), -float("inf"), 0.0, -0.0])
    X[1, 0] = 1.00390625  # exactly between two bf16 values: ties to even
    Y = ops.to_bf16(X.to(cuda))
    assert Y.dtype == torch.bfloat16 and Y.shape == X.shape and Y.stride(0) == 136
    assert torch.equal(Y.cpu(), X.bfloat16())
    Yt = ops.to_bf16(X.to(cuda), transpose=True)
    assert Yt.shape == (131, 257) and torch.equal(Yt.cpu(), X.t().bfloat16())


def test_bf16_weight_gradient_and_epilogue(cuda):
    from graphcuda_b200 import ops
    A, G = _rand(100_000, 96, 71), _rand(100_000, 256, 72)  # (A X)^T G: few tiles, K split across CTAs
    ref = O.matmul(A.t().double(), G.double()).float()
    A16, G16 = ops.to_bf16(A.to(cuda), transpose=True), ops.to_bf16(G.to(cuda), transpose=True)
    out = ops.gemm_bf16_operands(A16, G16)
    ops.check_gemm_flag(cuda)
    assert O.rel_fro(out, ref) < TOL_BF16
    assert torch.equal(out, ops.gemm_bf16_operands(A16, G16))
    X, W, b = _rand(5000, 128, 73), _rand(128, 256, 74), _rand(1, 256, 75)[0]
    pre = O.matmul(X.double(), W.double()).float() + b
    gate = _rand(5000, 256, 76)
    Y = ops.gemm_bf16_operands(ops.to_bf16(X.to(cuda)), ops.to_bf16(W.to(cuda), transpose=True), bias=b.to(cuda),
                               relu=True, gate=gate.to(cuda))
    assert O.rel_fro(Y, pre * (pre > 0) * (gate > 0)) < 2 * TOL_BF16  # ReLU flips near zero add a little


def test_bf16_tier_picks_its_engine_by_arithmetic_intensity(cuda):
    """precision="bf16" is the reduced-precision tier: bf16 MMAs where the product is compute-bound, single-pass
    TF32 (fp32 operands read in place) where converting the operands would cost more than the faster MMAs save."""
    from graphcuda_b200 import gemm, ops
    sq = torch.empty(4096, 4096, device=cuda)
    assert ops.gemm_path(sq, sq, precision="bf16") == "bf16"
    tall = torch.empty(1 << 18, 256, device=cuda), torch.empty(256, 256, device=cuda)
    assert ops.gemm_path(*tall, precision="bf16") == "tf32"
    odd = torch.empty(3000, 4099, device=cuda), torch.empty(4099, 3000, device=cuda)  # pitches TF32 cannot read in place
    assert ops.gemm_path(*odd, precision="bf16") == "bf16"
    A, B = _rand(4096, 4096, 91).to(cuda), _rand(4096, 4096, 92).to(cuda)
    out = gemm(A, B, precision="bf16")
    ops.check_gemm_flag(cuda)
    rows = torch.arange(0, 4096, 64, device=cuda)
    ref = A[rows].double() @ B.double()
    assert O.rel_fro(out[rows], ref) < TOL_BF16


def test_bf16_dense_adjacency_keeps_one_converted_copy(cuda):
    import graphcuda_b200 as gc
    from graphcuda_b200 import ops
    n, F = 3000, 64
    A = (_rand(n, n, 81) > 0.98).float() * _rand(n, n, 82).abs()
    A = (A + A.t()).to(cuda)
    H = _rand(n, F, 83).to(cuda)
    b = _rand(1, F, 84)[0].to(cuda)
    dadj = gc.DenseAdjacency(A, symmetric=True)
    Y = dadj.matmul(H, bias=b, relu=True, precision="bf16")
    ops.check_gemm_flag(cuda)
    pre = A.double().cpu() @ H.double().cpu() + b.double().cpu()
    assert O.rel_fro(Y, pre * (pre > 0)) < 2 * TOL_BF16
    memo = A._gc_bf16
    dadj.matmul(H, precision="bf16")
    assert A._gc_bf16 is memo  # not converted again
    A[0, 1] += 1.0             # an in-place change invalidates the copy
    dadj.matmul(H, precision="bf16")
    assert A._gc_bf16 is not memo

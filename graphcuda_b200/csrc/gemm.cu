// gc_gemm_f32: argument checks and the choice between the CUDA-core and the
// tensor-core back end.  Replaces the reference's GEMM entry points
// (src/graphcuda/cuda/gemm_cublas.cu:3-55, matmul1.cu:27-61, matmul2.cu:65-100,
// matmul3.cu:194-243, matmul4.cu:209-265).
#include "common.cuh"
#include "gemm_internal.cuh"

namespace {

int resolve(bool ta, bool tb, int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb, int64_t ldc,
            int precision) {
  if (precision == GC_PREC_FP32_SIMT) return GC_PREC_FP32_SIMT;
  const bool tc_ok = gc::tc_supported(ta, tb, M, N, K, lda, ldb, ldc);
  if (precision == GC_PREC_BF16) {
    // The reduced-precision tier picks the faster of its two engines.  bf16 MMAs run at twice the TF32 rate but
    // both fp32 operands are first converted into the workspace (read 4 + write 2 + read 2 bytes per element where
    // the TF32 kernel reads 4): that pays only for compute-bound products.  Measured: 4096^3 (683 flop/byte)
    // 0.196 ms bf16 against 0.236 ms TF32, 2048^3 (341) 0.050 against 0.042, 2^20 x 256 x 256 (64) 0.77 against 0.39.
    if (M <= 0 || N <= 0 || K <= 0) return gc::fail(GC_ERR_UNSUPPORTED, "bf16 GEMM needs non-empty sizes");
    const double flops = 2.0 * double(M) * double(N) * double(K);
    const double bytes = 4.0 * (double(M) * double(K) + double(K) * double(N) + double(M) * double(N));
    if (tc_ok && flops < 512.0 * bytes) return GC_PREC_TF32;
    return GC_PREC_BF16;  // operands are converted into the workspace: no alignment demands on the inputs
  }
  if (precision == GC_PREC_TF32X3 || precision == GC_PREC_TF32) {
    if (!tc_ok)
      return gc::fail(GC_ERR_UNSUPPORTED,
                      "tensor-core GEMM needs 16-byte aligned row pitches for operands read in place "
                      "(lda %% 4 == 0 when transA == 0, ldb %% 4 == 0 when transB == 1) and non-empty sizes");
    return precision;
  }
  if (precision != GC_PREC_AUTO) return gc::fail(GC_ERR_INVALID, "unknown precision %d", precision);
  if (!tc_ok) return GC_PREC_FP32_SIMT;
  // Small problems are launch-bound and stay on the CUDA cores (bit-stable).
  // Few-tile / huge-K shapes (weight gradients) are split along K on either path.
  const double flops = 2.0 * double(M) * double(N) * double(K);
  if (flops < double(1ull << 30)) return GC_PREC_FP32_SIMT;
  return GC_PREC_TF32X3;
}

}  // namespace

extern "C" {

int gc_gemm_resolve_precision(int transA, int transB, int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb,
                              int64_t ldc, int precision) {
  return resolve(transA != 0, transB != 0, M, N, K, lda, ldb, ldc, precision);
}

size_t gc_gemm_workspace_bytes(int transA, int transB, int64_t M, int64_t N, int64_t K, int precision) {
  if (M <= 0 || N <= 0 || K < 0) return 256;
  // AUTO may resolve either way depending on leading dimensions: report the larger.
  size_t simt = gc::simt_workspace_bytes(M, N, K);
  size_t tc3 = gc::tc_workspace_bytes(transA != 0, transB != 0, M, N, K, 3);
  size_t tc1 = gc::tc_workspace_bytes(transA != 0, transB != 0, M, N, K, 1);
  switch (precision) {
    case GC_PREC_FP32_SIMT: return std::max<size_t>(simt, 256);
    case GC_PREC_TF32X3: return tc3;
    case GC_PREC_TF32: return tc1;
    case GC_PREC_BF16: return std::max(tc1, gc::bf16_workspace_bytes(M, N, std::max<int64_t>(K, 1)));
    default: return std::max(std::max(simt, tc3), size_t(256));
  }
}

int gc_gemm_f32(int transA, int transB, int64_t M, int64_t N, int64_t K, const float* A, int64_t lda,
                const float* B, int64_t ldb, float* C, int64_t ldc, const float* bias, int epilogue, float* mask,
                const float* gate, int precision, void* workspace, size_t workspace_bytes, void* stream) {
  GC_REQUIRE(M >= 0 && N >= 0 && K >= 0, "gc_gemm_f32: negative size");
  GC_REQUIRE(M < INT32_MAX && N < INT32_MAX && K < INT32_MAX, "gc_gemm_f32: size out of int32 range");
  GC_REQUIRE((epilogue & ~(GC_EPI_RELU | GC_EPI_TRANSPOSED_OUT)) == 0, "gc_gemm_f32: unknown epilogue bits");
  if (M == 0 || N == 0) return GC_OK;
  const bool ta = transA != 0, tb = transB != 0;
  const bool tr = (epilogue & GC_EPI_TRANSPOSED_OUT) != 0;
  GC_REQUIRE(C, "gc_gemm_f32: null C");
  GC_REQUIRE(K == 0 || (A && B), "gc_gemm_f32: null operand");
  GC_REQUIRE(lda >= (ta ? M : K), "gc_gemm_f32: lda too small");
  GC_REQUIRE(ldb >= (tb ? K : N), "gc_gemm_f32: ldb too small");
  GC_REQUIRE(ldc >= (tr ? M : N), "gc_gemm_f32: ldc too small");
  gc::GemmEpilogue ep{bias, mask, gate, (epilogue & GC_EPI_RELU) ? 1 : 0, tr ? 1 : 0};
  cudaStream_t st = gc::as_stream(stream);
  int prec = (K == 0) ? GC_PREC_FP32_SIMT : resolve(ta, tb, M, N, K, lda, ldb, ldc, precision);
  if (prec < 0) return prec;
  if (prec == GC_PREC_FP32_SIMT)
    return gc::gemm_simt(ta, tb, M, N, K, A, lda, B, ldb, C, ldc, ep, workspace, workspace_bytes, st);
  if (prec == GC_PREC_BF16)
    return gc::gemm_bf16(ta, tb, M, N, K, A, lda, B, ldb, C, ldc, ep, workspace, workspace_bytes, st);
  return gc::gemm_tc(ta, tb, M, N, K, A, lda, B, ldb, C, ldc, ep, prec == GC_PREC_TF32X3 ? 3 : 1, workspace,
                     workspace_bytes, st);
}

int gc_convert_f32_bf16(const float* src, int64_t ld_src, int64_t rows, int64_t cols, uint16_t* dst, int64_t ld_dst,
                        int transpose, void* stream) {
  GC_REQUIRE(rows >= 0 && cols >= 0 && rows < INT32_MAX && cols < INT32_MAX, "gc_convert_f32_bf16: bad size");
  if (rows == 0 || cols == 0) return GC_OK;
  GC_REQUIRE(src && dst, "gc_convert_f32_bf16: null pointer");
  GC_REQUIRE(ld_dst >= cols && ld_dst % 2 == 0 && (reinterpret_cast<uintptr_t>(dst) & 3u) == 0,
             "gc_convert_f32_bf16: ld_dst must be even and >= cols, dst 4-byte aligned");
  GC_REQUIRE(ld_src >= (transpose ? rows : cols), "gc_convert_f32_bf16: ld_src too small");
  return gc::convert_bf16(src, ld_src, rows, cols, dst, ld_dst, transpose != 0, gc::as_stream(stream));
}

size_t gc_gemm_bf16_workspace_bytes(int64_t M, int64_t N, int64_t K) {
  if (M <= 0 || N <= 0 || K <= 0) return 256;
  return gc::bf16_core_workspace_bytes(M, N, K);
}

int gc_gemm_bf16_f32(int64_t M, int64_t N, int64_t K, const uint16_t* A, int64_t lda, const uint16_t* Bt,
                     int64_t ldb, float* C, int64_t ldc, const float* bias, int epilogue, float* mask,
                     const float* gate, void* workspace, size_t workspace_bytes, void* stream) {
  GC_REQUIRE(M >= 0 && N >= 0 && K >= 1, "gc_gemm_bf16_f32: bad size");
  GC_REQUIRE(M < INT32_MAX && N < INT32_MAX && K < INT32_MAX, "gc_gemm_bf16_f32: size out of int32 range");
  GC_REQUIRE((epilogue & ~(GC_EPI_RELU | GC_EPI_TRANSPOSED_OUT)) == 0, "gc_gemm_bf16_f32: unknown epilogue bits");
  if (M == 0 || N == 0) return GC_OK;
  const bool tr = (epilogue & GC_EPI_TRANSPOSED_OUT) != 0;
  GC_REQUIRE(A && Bt && C, "gc_gemm_bf16_f32: null pointer");
  GC_REQUIRE(lda >= K && ldb >= K && ldc >= (tr ? M : N), "gc_gemm_bf16_f32: leading dimension too small");
  gc::GemmEpilogue ep{bias, mask, gate, (epilogue & GC_EPI_RELU) ? 1 : 0, tr ? 1 : 0};
  return gc::gemm_bf16_core(M, N, K, A, lda, Bt, ldb, C, ldc, ep, workspace, workspace_bytes, gc::as_stream(stream));
}

int gc_gemm_check_flag(const void* workspace, void* stream) {
  GC_REQUIRE(workspace, "gc_gemm_check_flag: null workspace");
  int h = 0;
  cudaError_t e = cudaMemcpyAsync(&h, workspace, sizeof(int), cudaMemcpyDeviceToHost, gc::as_stream(stream));
  if (e == cudaSuccess) e = cudaStreamSynchronize(gc::as_stream(stream));
  if (e != cudaSuccess) return gc::fail(GC_ERR_CUDA, "gc_gemm_check_flag: %s", cudaGetErrorString(e));
  if (h != 0) return gc::fail(GC_ERR_DEVICE_FLAG, "a tensor-core GEMM kernel gave up a bounded wait");
  return GC_OK;
}

}  // extern "C"

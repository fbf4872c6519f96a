// Internal interface between the GEMM dispatcher and its two back ends.
#pragma once

#include "common.cuh"

#include <algorithm>

namespace gc {

struct GemmEpilogue {
  const float* bias;  // [N] or null
  float* mask;        // same shape / leading dimension as C, or null
  const float* gate;  // same shape / leading dimension as C, or null: C *= (gate > 0) after everything else
  int relu;
  int transposed;     // store C^T (N x M, leading dimension ldc)
};

// Bias, ReLU as y * (y > 0) (reference gcn.cu:19-20), fp32 mask, one element.
__device__ __forceinline__ void epilogue_store(float v, int m, int n, float* C, int64_t ldc, const GemmEpilogue& ep) {
  if (ep.bias) v += __ldg(ep.bias + n);
  const int64_t off = ep.transposed ? int64_t(n) * ldc + m : int64_t(m) * ldc + n;
  if (ep.relu || ep.mask) {
    const float mk = v > 0.f ? 1.f : 0.f;
    if (ep.mask) ep.mask[off] = mk;
    if (ep.relu) v *= mk;
  }
  if (ep.gate) v *= (__ldg(ep.gate + off) > 0.f ? 1.f : 0.f);
  C[off] = v;
}

// CUDA-core path (gemm_simt.cu)
int simt_splits(int64_t M, int64_t N, int64_t K);
size_t simt_workspace_bytes(int64_t M, int64_t N, int64_t K);
int gemm_simt(bool ta, bool tb, int64_t M, int64_t N, int64_t K, const float* A, int64_t lda, const float* B,
              int64_t ldb, float* C, int64_t ldc, const GemmEpilogue& ep, void* workspace, size_t workspace_bytes,
              cudaStream_t st);

// Tensor-core path (gemm_tcgen05.cu)
bool tc_supported(bool ta, bool tb, int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb, int64_t ldc);
size_t tc_workspace_bytes(bool ta, bool tb, int64_t M, int64_t N, int64_t K, int passes);
int gemm_tc(bool ta, bool tb, int64_t M, int64_t N, int64_t K, const float* A, int64_t lda, const float* B,
            int64_t ldb, float* C, int64_t ldc, const GemmEpilogue& ep, int passes, void* workspace,
            size_t workspace_bytes, cudaStream_t st);

// bf16 operands, fp32 accumulation (gemm_tcgen05.cu)
size_t bf16_workspace_bytes(int64_t M, int64_t N, int64_t K);
size_t bf16_core_workspace_bytes(int64_t M, int64_t N, int64_t K);
int convert_bf16(const float* src, int64_t lds, int64_t rows, int64_t cols, uint16_t* dst, int64_t ldd, bool transpose,
                 cudaStream_t st);
int gemm_bf16_core(int64_t M, int64_t N, int64_t K, const uint16_t* A, int64_t lda, const uint16_t* Bt, int64_t ldb,
                   float* C, int64_t ldc, const GemmEpilogue& ep, void* workspace, size_t workspace_bytes,
                   cudaStream_t st);
int gemm_bf16(bool ta, bool tb, int64_t M, int64_t N, int64_t K, const float* A, int64_t lda, const float* B,
              int64_t ldb, float* C, int64_t ldc, const GemmEpilogue& ep, void* workspace, size_t workspace_bytes,
              cudaStream_t st);

}  // namespace gc

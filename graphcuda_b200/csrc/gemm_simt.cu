// IEEE fp32 GEMM on CUDA cores with a fixed summation order.
//
// The bit-stable path behind gc_gemm_f32: it serves every shape and leading
// dimension (the tensor-core path needs 16-byte aligned rows), the small
// Cora-sized products where launch latency dominates, and it is the on-device
// cross-check for the tcgen05 kernels.  Takes over matmul1..4
// (src/graphcuda/cuda/matmul1.cu:5-23, matmul2.cu:3-62, matmul3.cu:8-191,
// matmul4.cu:44-206) and cublasSgemm as wrapped by
// src/graphcuda/cuda/gemm_cublas.cu:37-48; unlike matmul3/matmul4 it is
// correct for every M, N, K (no tile-shape or N%4 preconditions).
//
// Tiling: BM x BN x 16 per CTA, 256 threads, TM x TN accumulators per thread,
// operands staged k-major in shared memory.  K can be split across
// gridDim.z; partial tiles go to the workspace and a second kernel adds them
// in split order, so results do not depend on scheduling.
#include "common.cuh"
#include "gemm_internal.cuh"

namespace {

constexpr int BK = 16;

template <int BM, int BN, int TM, int TN, bool TA, bool TB>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(int M, int N, int K, const float* __restrict__ A, int64_t lda, const float* __restrict__ B,
                 int64_t ldb, float* __restrict__ C, int64_t ldc, gc::GemmEpilogue ep, int k_per_split,
                 float* __restrict__ partial) {
  static_assert((BM / TM) * (BN / TN) == 256, "256 threads per CTA");
  __shared__ float As[BK][BM + 4];
  __shared__ float Bs[BK][BN + 4];
  const int tid = threadIdx.x;
  const int m0 = blockIdx.x * BM, n0 = blockIdx.y * BN;
  const int kb = blockIdx.z * k_per_split;
  const int ke = min(K, kb + k_per_split);
  const int tx = tid % (BN / TN), ty = tid / (BN / TN);

  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

  for (int k0 = kb; k0 < ke; k0 += BK) {
    // stage A tile: element (m, k) -> As[k][m]
    for (int i = tid; i < BM * BK; i += 256) {
      int m, k;
      if (TA) { m = i % BM; k = i / BM; } else { k = i % BK; m = i / BK; }
      const int gm = m0 + m, gk = k0 + k;
      float v = 0.f;
      if (gm < M && gk < ke) v = TA ? __ldg(A + int64_t(gk) * lda + gm) : __ldg(A + int64_t(gm) * lda + gk);
      As[k][m] = v;
    }
    // stage B tile: element (k, n) -> Bs[k][n]
    for (int i = tid; i < BN * BK; i += 256) {
      int n, k;
      if (TB) { k = i % BK; n = i / BK; } else { n = i % BN; k = i / BN; }
      const int gn = n0 + n, gk = k0 + k;
      float v = 0.f;
      if (gn < N && gk < ke) v = TB ? __ldg(B + int64_t(gn) * ldb + gk) : __ldg(B + int64_t(gk) * ldb + gn);
      Bs[k][n] = v;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float a[TM], b[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[k][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) b[j] = Bs[k][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }

#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int gm = m0 + ty * TM + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int gn = n0 + tx * TN + j;
      if (gn >= N) continue;
      if (partial) {
        partial[(int64_t(blockIdx.z) * M + gm) * N + gn] = acc[i][j];
      } else {
        gc::epilogue_store(acc[i][j], gm, gn, C, ldc, ep);
      }
    }
  }
}

__global__ void __launch_bounds__(256)
splitk_reduce_kernel(int M, int N, int splits, const float* __restrict__ partial, float* __restrict__ C,
                     int64_t ldc, gc::GemmEpilogue ep) {
  const int64_t total = int64_t(M) * N;
  for (int64_t i = int64_t(blockIdx.x) * 256 + threadIdx.x; i < total; i += int64_t(gridDim.x) * 256) {
    float s = partial[i];
    for (int z = 1; z < splits; ++z) s += partial[int64_t(z) * total + i];
    gc::epilogue_store(s, int(i / N), int(i % N), C, ldc, ep);
  }
}

template <int BM, int BN, int TM, int TN>
void launch(bool ta, bool tb, dim3 grid, cudaStream_t st, int M, int N, int K, const float* A, int64_t lda,
            const float* B, int64_t ldb, float* C, int64_t ldc, const gc::GemmEpilogue& ep, int kps,
            float* partial) {
#define GC_L(TA_, TB_) \
  gemm_simt_kernel<BM, BN, TM, TN, TA_, TB_><<<grid, 256, 0, st>>>(M, N, K, A, lda, B, ldb, C, ldc, ep, kps, partial)
  if (!ta && !tb) GC_L(false, false);
  else if (!ta && tb) GC_L(false, true);
  else if (ta && !tb) GC_L(true, false);
  else GC_L(true, true);
#undef GC_L
}

}  // namespace

namespace gc {

int simt_splits(int64_t M, int64_t N, int64_t K) {
  const bool narrow = N <= 32;
  const int64_t bm = narrow ? 128 : 64, bn = narrow ? 32 : 64;
  const int64_t tiles = ceil_div(M, bm) * ceil_div(N, bn);
  // few output tiles (narrow products of the small graphs, weight gradients): spread K over the SMs
  if (tiles >= kNumSMs || K < 256) return 1;
  int64_t splits = std::min<int64_t>(ceil_div(2 * kNumSMs, tiles), ceil_div(K, 64));
  return int(std::max<int64_t>(1, std::min<int64_t>(splits, 512)));
}

// The first 256 bytes of every GEMM workspace hold the tensor-core path's
// sticky error word; split-K partials start behind it.
constexpr size_t kFlagBytes = 256;

size_t simt_workspace_bytes(int64_t M, int64_t N, int64_t K) {
  const int s = simt_splits(M, N, K);
  return s > 1 ? kFlagBytes + size_t(s) * size_t(M) * size_t(N) * sizeof(float) : 0;
}

int gemm_simt(bool ta, bool tb, int64_t M, int64_t N, int64_t K, const float* A, int64_t lda, const float* B,
              int64_t ldb, float* C, int64_t ldc, const GemmEpilogue& ep, void* workspace, size_t workspace_bytes,
              cudaStream_t st) {
  const bool narrow = N <= 32;
  const int bm = narrow ? 128 : 64, bn = narrow ? 32 : 64;
  int splits = simt_splits(M, N, K);
  float* partial = nullptr;
  if (splits > 1) {
    if (!workspace || workspace_bytes < kFlagBytes + size_t(splits) * M * N * sizeof(float)) splits = 1;
    else partial = reinterpret_cast<float*>(static_cast<char*>(workspace) + kFlagBytes);
  }
  int kps = int(ceil_div(ceil_div(K, splits), BK) * BK);
  if (kps <= 0) kps = BK;
  splits = int(std::max<int64_t>(1, ceil_div(K, kps)));
  if (splits == 1) partial = nullptr;
  dim3 grid(unsigned(ceil_div(M, bm)), unsigned(ceil_div(N, bn)), unsigned(splits));
  if (grid.y > 65535u) return fail(GC_ERR_UNSUPPORTED, "gemm_simt: N too large for this launch shape");
  if (narrow)
    launch<128, 32, 4, 4>(ta, tb, grid, st, int(M), int(N), int(K), A, lda, B, ldb, C, ldc, ep, kps, partial);
  else
    launch<64, 64, 4, 4>(ta, tb, grid, st, int(M), int(N), int(K), A, lda, B, ldb, C, ldc, ep, kps, partial);
  int rc = check_launch("gemm_simt");
  if (rc != GC_OK) return rc;
  if (partial) {
    const int64_t total = M * N;
    const unsigned g = unsigned(std::min<int64_t>(ceil_div(total, 256), kNumSMs * 8));
    splitk_reduce_kernel<<<g, 256, 0, st>>>(int(M), int(N), splits, partial, C, ldc, ep);
    rc = check_launch("gemm_simt split-K reduce");
  }
  return rc;
}

}  // namespace gc

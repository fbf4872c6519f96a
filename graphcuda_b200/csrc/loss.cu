// Fused classification tail: log_softmax over the class dimension + negative
// log-likelihood of the labelled class, and its gradient with respect to the
// logits.  Takes over the PyTorch ops the reference's training script runs
// after the last layer (tests/gcn/graphcuda_impl.py:24 log_softmax,
// :55 F.nll_loss on the masked rows) -- four kernels and two N x C temporaries
// there, one pass here in each direction.
//
//   loss = scale * sum over selected rows r of ( logsumexp(Z[r, :]) - Z[r, y_r] )
//   dZ[r, c] = g * scale * ( exp(Z[r, c] - lse_r) - [c == y_r] )   for selected rows, 0 otherwise
//
// One warp per row, lanes across classes (coalesced), shuffles for the max /
// sum; the loss is reduced per warp, per block and by a final single block in
// a fixed order (no atomics, bit-reproducible).
#include "common.cuh"

#include <algorithm>

namespace {

constexpr int kLossBlocks = gc::kNumSMs * 8;

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__global__ void __launch_bounds__(256)
lse_nll_forward_kernel(const float* __restrict__ Z, int64_t ldz, const int64_t* __restrict__ labels,
                       const uint8_t* __restrict__ row_mask, int64_t M, int C, float* __restrict__ lse,
                       float* __restrict__ partials) {
  __shared__ float warp_loss[8];
  const int lane = threadIdx.x % 32, warp = threadIdx.x / 32;
  const int64_t warps = int64_t(gridDim.x) * 8;
  float acc = 0.f;
  for (int64_t r = int64_t(blockIdx.x) * 8 + warp; r < M; r += warps) {
    const float* z = Z + r * ldz;
    float mx = -INFINITY;
    for (int c = lane; c < C; c += 32) mx = fmaxf(mx, __ldg(z + c));
    mx = warp_max(mx);
    float s = 0.f;
    for (int c = lane; c < C; c += 32) s += expf(__ldg(z + c) - mx);
    s = warp_sum(s);
    const float l = mx + logf(s);
    if (lane == 0) {
      lse[r] = l;
      if (!row_mask || row_mask[r]) {
        const int64_t y = labels[r];
        if (y >= 0 && y < C) acc += l - __ldg(z + y);
      }
    }
  }
  if (lane == 0) warp_loss[warp] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float b = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) b += warp_loss[w];
    partials[blockIdx.x] = b;
  }
}

__global__ void __launch_bounds__(256)
loss_reduce_kernel(const float* __restrict__ partials, int n, float scale, float* __restrict__ loss) {
  __shared__ float sh[256];
  float a = 0.f;
  for (int i = threadIdx.x; i < n; i += 256) a += partials[i];
  sh[threadIdx.x] = a;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if (threadIdx.x < o) sh[threadIdx.x] += sh[threadIdx.x + o];
    __syncthreads();
  }
  if (threadIdx.x == 0) *loss = sh[0] * scale;
}

__global__ void __launch_bounds__(256)
lse_nll_backward_kernel(const float* __restrict__ Z, int64_t ldz, const int64_t* __restrict__ labels,
                        const uint8_t* __restrict__ row_mask, const float* __restrict__ lse,
                        const float* __restrict__ grad_loss, float scale, int64_t M, int C, float* __restrict__ dZ,
                        int64_t lddz) {
  const int lane = threadIdx.x % 32, warp = threadIdx.x / 32;
  const int64_t warps = int64_t(gridDim.x) * 8;
  const float g = (grad_loss ? __ldg(grad_loss) : 1.f) * scale;
  for (int64_t r = int64_t(blockIdx.x) * 8 + warp; r < M; r += warps) {
    float* d = dZ + r * lddz;
    if (row_mask && !row_mask[r]) {
      for (int c = lane; c < C; c += 32) d[c] = 0.f;
      continue;
    }
    const float* z = Z + r * ldz;
    const float l = __ldg(lse + r);
    const int64_t y = labels[r];
    for (int c = lane; c < C; c += 32) d[c] = g * (expf(__ldg(z + c) - l) - (c == y ? 1.f : 0.f));
  }
}

}  // namespace

extern "C" {

size_t gc_nll_workspace_bytes(int64_t M) {
  if (M < 0) return 0;
  return size_t(kLossBlocks) * sizeof(float) + size_t(M) * sizeof(float);
}

int gc_logsoftmax_nll_forward_f32(const float* Z, int64_t ldz, const int64_t* labels, const uint8_t* row_mask,
                                  int64_t M, int64_t C, float scale, float* loss, void* workspace,
                                  size_t workspace_bytes, void* stream) {
  GC_REQUIRE(M >= 0 && C >= 1 && C < INT32_MAX, "gc_logsoftmax_nll_forward_f32: bad size");
  GC_REQUIRE(loss && workspace, "gc_logsoftmax_nll_forward_f32: null pointer");
  GC_REQUIRE(M == 0 || (Z && labels), "gc_logsoftmax_nll_forward_f32: null pointer");
  GC_REQUIRE(ldz >= C, "gc_logsoftmax_nll_forward_f32: leading dimension smaller than C");
  if (workspace_bytes < gc_nll_workspace_bytes(M))
    return gc::fail(GC_ERR_WORKSPACE, "gc_logsoftmax_nll_forward_f32: workspace too small");
  cudaStream_t st = gc::as_stream(stream);
  float* partials = static_cast<float*>(workspace);
  float* lse = partials + kLossBlocks;
  const int blocks = int(std::max<int64_t>(1, std::min<int64_t>((M + 7) / 8, kLossBlocks)));
  lse_nll_forward_kernel<<<blocks, 256, 0, st>>>(Z, ldz, labels, row_mask, M, int(C), lse, partials);
  loss_reduce_kernel<<<1, 256, 0, st>>>(partials, blocks, scale, loss);
  return gc::check_launch("gc_logsoftmax_nll_forward_f32", 2);
}

int gc_logsoftmax_nll_backward_f32(const float* Z, int64_t ldz, const int64_t* labels, const uint8_t* row_mask,
                                   int64_t M, int64_t C, float scale, const float* grad_loss, float* dZ,
                                   int64_t lddz, const void* workspace, void* stream) {
  GC_REQUIRE(M >= 0 && C >= 1 && C < INT32_MAX, "gc_logsoftmax_nll_backward_f32: bad size");
  if (M == 0) return GC_OK;
  GC_REQUIRE(Z && labels && dZ && workspace, "gc_logsoftmax_nll_backward_f32: null pointer");
  GC_REQUIRE(ldz >= C && lddz >= C, "gc_logsoftmax_nll_backward_f32: leading dimension smaller than C");
  const float* lse = static_cast<const float*>(workspace) + kLossBlocks;
  const int blocks = int(std::max<int64_t>(1, std::min<int64_t>((M + 7) / 8, kLossBlocks)));
  lse_nll_backward_kernel<<<blocks, 256, 0, gc::as_stream(stream)>>>(Z, ldz, labels, row_mask, lse, grad_loss, scale,
                                                                    M, int(C), dZ, lddz);
  return gc::check_launch("gc_logsoftmax_nll_backward_f32");
}

}  // extern "C"

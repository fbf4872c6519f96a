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
// A group of lanes per row (8 lanes up to 64 classes, else the warp), lanes across classes, shuffles for the
// max / sum; the loss is reduced per warp, per block and by a final single block in
// a fixed order (no atomics, bit-reproducible).
#include "common.cuh"

#include <algorithm>

namespace {

constexpr int kLossBlocks = gc::kNumSMs * 8;

// G lanes per row (8 for up to 64 classes, else the whole warp): 32 / G rows are in flight per warp, so the
// per-row chain of two reductions and a logf is overlapped within the warp as well as across warps.
template <int G>
__global__ void __launch_bounds__(256)
lse_nll_forward_kernel(const float* __restrict__ Z, int64_t ldz, const int64_t* __restrict__ labels,
                       const uint8_t* __restrict__ row_mask, int64_t M, int C, float* __restrict__ lse,
                       float* __restrict__ partials) {
  __shared__ float warp_loss[8];
  constexpr int R = 32 / G;  // rows per warp pass
  const int lane = threadIdx.x % 32, warp = threadIdx.x / 32;
  const int lg = lane % G, sub = lane / G;
  const int64_t stride = int64_t(gridDim.x) * 8 * R;
  float acc = 0.f;
  for (int64_t r0 = (int64_t(blockIdx.x) * 8 + warp) * R; r0 < M; r0 += stride) {  // uniform across the warp
    const int64_t r = r0 + sub;
    const bool valid = r < M;
    const float* z = Z + (valid ? r : 0) * ldz;
    float mx = -INFINITY;
    if (valid)
      for (int c = lg; c < C; c += G) mx = fmaxf(mx, __ldg(z + c));
#pragma unroll
    for (int o = G / 2; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float s = 0.f;
    if (valid)
      for (int c = lg; c < C; c += G) s += expf(__ldg(z + c) - mx);
#pragma unroll
    for (int o = G / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (valid && lg == 0) {
      const float l = mx + logf(s);
      lse[r] = l;
      if (!row_mask || row_mask[r]) {
        const int64_t y = labels[r];
        if (y >= 0 && y < C) acc += l - __ldg(z + y);
      }
    }
  }
  // the R row-slots of the warp, then the 8 warps, in a fixed order
#pragma unroll
  for (int o = 16; o >= G; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
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

template <int G>
__global__ void __launch_bounds__(256)
lse_nll_backward_kernel(const float* __restrict__ Z, int64_t ldz, const int64_t* __restrict__ labels,
                        const uint8_t* __restrict__ row_mask, const float* __restrict__ lse,
                        const float* __restrict__ grad_loss, float scale, int64_t M, int C, float* __restrict__ dZ,
                        int64_t lddz) {
  constexpr int R = 32 / G;
  const int lane = threadIdx.x % 32, warp = threadIdx.x / 32;
  const int lg = lane % G, sub = lane / G;
  const int64_t stride = int64_t(gridDim.x) * 8 * R;
  const float g = (grad_loss ? __ldg(grad_loss) : 1.f) * scale;
  for (int64_t r = (int64_t(blockIdx.x) * 8 + warp) * R + sub; r < M; r += stride) {
    float* d = dZ + r * lddz;
    if (row_mask && !row_mask[r]) {
      for (int c = lg; c < C; c += G) d[c] = 0.f;
      continue;
    }
    const float* z = Z + r * ldz;
    const float l = __ldg(lse + r);
    const int64_t y = labels[r];
    for (int c = lg; c < C; c += G) d[c] = g * (expf(__ldg(z + c) - l) - (c == y ? 1.f : 0.f));
  }
}

// Evaluation tail (reference tests/gcn/graphcuda_impl.py:63-68): row-wise
// argmax (lowest index among equal maxima) and, for each of n_masks row
// selections, how many selected rows were predicted right and how many were
// selected.  Integer atomics: the counts do not depend on the order.
template <int G>
__global__ void __launch_bounds__(256)
argmax_count_kernel(const float* __restrict__ Z, int64_t ldz, int64_t M, int C, const int64_t* __restrict__ labels,
                    const uint8_t* __restrict__ masks, int n_masks, int64_t* __restrict__ pred,
                    unsigned long long* __restrict__ counts) {
  __shared__ unsigned int sh[8][2 * 8];
  constexpr int R = 32 / G;  // rows per warp pass, G lanes each
  const int lane = threadIdx.x % 32, warp = threadIdx.x / 32;
  const int lg = lane % G, sub = lane / G;
  const int64_t stride = int64_t(gridDim.x) * 8 * R;
  unsigned int right[8], chosen[8];
#pragma unroll
  for (int m = 0; m < 8; ++m) right[m] = chosen[m] = 0;
  for (int64_t r0 = (int64_t(blockIdx.x) * 8 + warp) * R; r0 < M; r0 += stride) {  // uniform across the warp
    const int64_t r = r0 + sub;
    const bool valid = r < M;
    const float* z = Z + (valid ? r : 0) * ldz;
    float best = -INFINITY;
    int arg = C;  // no candidate seen yet
    if (valid)
      for (int c = lg; c < C; c += G) {
        const float v = __ldg(z + c);
        if (v > best || arg == C) {
          best = v;
          arg = c;
        }
      }
#pragma unroll
    for (int o = G / 2; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
      if (oa < C && (arg == C || ob > best || (ob == best && oa < arg))) {
        best = ob;
        arg = oa;
      }
    }
    if (valid && lg == 0) {
      if (pred) pred[r] = arg;
      if (labels) {
        const bool hit = labels[r] == int64_t(arg);
        if (masks) {
#pragma unroll
          for (int m = 0; m < 8; ++m)  // fixed trip count: the counters stay in registers
            if (m < n_masks && masks[int64_t(m) * M + r]) {
              chosen[m]++;
              right[m] += hit ? 1u : 0u;
            }
        } else {
          chosen[0]++;
          right[0] += hit ? 1u : 0u;
        }
      }
    }
  }
  if (!labels) return;
  const int nm = masks ? n_masks : 1;
  // the R row-slots of a warp (their leaders are lanes 0, G, 2G, ...), then the 8 warps
#pragma unroll
  for (int m = 0; m < 8; ++m) {
    if (m < nm) {  // uniform
#pragma unroll
      for (int o = 16; o >= G; o >>= 1) {
        right[m] += __shfl_xor_sync(0xffffffffu, right[m], o);
        chosen[m] += __shfl_xor_sync(0xffffffffu, chosen[m], o);
      }
      if (lane == 0) {
        sh[warp][2 * m] = right[m];
        sh[warp][2 * m + 1] = chosen[m];
      }
    }
  }
  __syncthreads();
  if (threadIdx.x < 2 * nm) {
    unsigned long long t = 0;
#pragma unroll
    for (int w = 0; w < 8; ++w) t += sh[w][threadIdx.x];
    if (t) atomicAdd(counts + threadIdx.x, t);
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
  const int rows_per_block = C <= 64 ? 32 : 8;
  const int blocks = int(std::max<int64_t>(1, std::min<int64_t>((M + rows_per_block - 1) / rows_per_block, kLossBlocks)));
  if (C <= 64)
    lse_nll_forward_kernel<8><<<blocks, 256, 0, st>>>(Z, ldz, labels, row_mask, M, int(C), lse, partials);
  else
    lse_nll_forward_kernel<32><<<blocks, 256, 0, st>>>(Z, ldz, labels, row_mask, M, int(C), lse, partials);
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
  const int rows_per_block = C <= 64 ? 32 : 8;
  const int blocks = int(std::max<int64_t>(1, std::min<int64_t>((M + rows_per_block - 1) / rows_per_block, kLossBlocks)));
  if (C <= 64)
    lse_nll_backward_kernel<8><<<blocks, 256, 0, gc::as_stream(stream)>>>(Z, ldz, labels, row_mask, lse, grad_loss,
                                                                         scale, M, int(C), dZ, lddz);
  else
    lse_nll_backward_kernel<32><<<blocks, 256, 0, gc::as_stream(stream)>>>(Z, ldz, labels, row_mask, lse, grad_loss,
                                                                          scale, M, int(C), dZ, lddz);
  return gc::check_launch("gc_logsoftmax_nll_backward_f32");
}

int gc_argmax_accuracy_f32(const float* Z, int64_t ldz, int64_t M, int64_t C, const int64_t* labels,
                           const uint8_t* masks, int n_masks, int64_t* pred, int64_t* counts, void* stream) {
  GC_REQUIRE(M >= 0 && C >= 1 && C < INT32_MAX, "gc_argmax_accuracy_f32: bad size");
  GC_REQUIRE(ldz >= C, "gc_argmax_accuracy_f32: leading dimension smaller than C");
  GC_REQUIRE(n_masks >= 0 && n_masks <= 8, "gc_argmax_accuracy_f32: at most 8 row selections");
  GC_REQUIRE(!masks || n_masks >= 1, "gc_argmax_accuracy_f32: masks given with n_masks = 0");
  GC_REQUIRE(!labels || counts, "gc_argmax_accuracy_f32: labels given without counts");
  GC_REQUIRE(M == 0 || Z, "gc_argmax_accuracy_f32: null Z");
  cudaStream_t st = gc::as_stream(stream);
  if (labels) {
    const int nm = masks ? n_masks : 1;
    if (cudaMemsetAsync(counts, 0, size_t(2 * nm) * sizeof(int64_t), st) != cudaSuccess)
      return gc::fail(GC_ERR_CUDA, "gc_argmax_accuracy_f32: clearing the counts failed");
  }
  if (M == 0 || (!pred && !labels)) return GC_OK;
  const int rows_per_block = C <= 64 ? 32 : 8;
  const int blocks = int(std::max<int64_t>(1, std::min<int64_t>((M + rows_per_block - 1) / rows_per_block, kLossBlocks)));
  if (C <= 64)
    argmax_count_kernel<8><<<blocks, 256, 0, st>>>(Z, ldz, M, int(C), labels, masks, n_masks, pred,
                                                   reinterpret_cast<unsigned long long*>(counts));
  else
    argmax_count_kernel<32><<<blocks, 256, 0, st>>>(Z, ldz, M, int(C), labels, masks, n_masks, pred,
                                                    reinterpret_cast<unsigned long long*>(counts));
  return gc::check_launch("gc_argmax_accuracy_f32");
}

}  // extern "C"

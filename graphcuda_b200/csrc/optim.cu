// Adam update of every parameter tensor of a model in ONE launch.
//
// The reference's training scripts step a stock torch optimizer after the
// backward pass (tests/gcn/graphcuda_impl.py:45,56 -- SGD there, Adam in the
// configurations this library is measured on).  On a Cora-sized model that
// tail is a dozen tiny kernels; here it is one, and because the step count
// lives on the device the launch can be recorded in a CUDA graph and replayed.
//
// Arithmetic follows torch.optim.Adam (amsgrad = False, maximize = False):
//   t    = step + 1
//   g    = grad + weight_decay * p
//   m    = m + (g - m) * (1 - beta1)
//   v    = v * beta2 + g * g * (1 - beta2)
//   p    = p - (lr / (1 - beta1^t)) * m / (sqrt(v) / sqrt(1 - beta2^t) + eps)
// and, like SGD (dampening 0, no momentum) for the reference's own script:
//   p    = p - lr * (grad + weight_decay * p)
#include "common.cuh"

#include <algorithm>

namespace {

constexpr int kMaxTensors = 32;
constexpr int kChunk = 1024;  // elements per CTA pass: 256 threads x 4

struct TensorList {
  float* p[kMaxTensors];
  const float* g[kMaxTensors];
  float* m[kMaxTensors];
  float* v[kMaxTensors];
  int64_t first_chunk[kMaxTensors + 1];  // prefix sum of ceil(n / kChunk)
  int64_t n[kMaxTensors];
  int count;
};

// state[0] = steps taken so far (read by every CTA before it counts itself in
// state[1]); the CTA that arrives last writes the new step count and clears
// the arrival counter, so no CTA can observe the incremented value.
__global__ void __launch_bounds__(256)
adam_kernel(TensorList tl, double lr, double beta1, double beta2, float eps, float weight_decay,
            unsigned long long* __restrict__ state) {
  __shared__ unsigned long long step_s;
  __shared__ float consts_s[2];
  if (threadIdx.x == 0) {
    step_s = *reinterpret_cast<volatile unsigned long long*>(state);
    // scalar part in double, as the Python arithmetic of torch.optim.Adam does it
    const double t = double(step_s + 1ull);
    consts_s[0] = float(lr / (1.0 - pow(beta1, t)));
    consts_s[1] = float(sqrt(1.0 - pow(beta2, t)));
  }
  __syncthreads();
  const float step_size = consts_s[0];
  const float bc2_sqrt = consts_s[1];
  const float w1 = float(1.0 - beta1), w2 = float(1.0 - beta2), b2 = float(beta2);
  const int64_t total = tl.first_chunk[tl.count];
  for (int64_t vc = blockIdx.x; vc < total; vc += gridDim.x) {
    int k = 0;
    while (k + 1 < tl.count && vc >= tl.first_chunk[k + 1]) ++k;
    const int64_t base = (vc - tl.first_chunk[k]) * kChunk;
    float* __restrict__ p = tl.p[k];
    const float* __restrict__ g = tl.g[k];
    float* __restrict__ m = tl.m[k];
    float* __restrict__ v = tl.v[k];
    const int64_t n = tl.n[k];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int64_t i = base + u * 256 + threadIdx.x;
      if (i < n) {
        const float pi = p[i];
        const float gi = g[i] + weight_decay * pi;
        const float mi = m[i] + (gi - m[i]) * w1;
        const float vi = v[i] * b2 + gi * gi * w2;
        m[i] = mi;
        v[i] = vi;
        p[i] = pi - step_size * (mi / (sqrtf(vi) / bc2_sqrt + eps));
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned long long arrived = atomicAdd(state + 1, 1ull);
    if (arrived == gridDim.x - 1) {
      state[1] = 0ull;
      state[0] = step_s + 1ull;
    }
  }
}

__global__ void __launch_bounds__(256)
sgd_kernel(TensorList tl, float lr, float weight_decay) {  // lr, weight_decay: rounded once from the doubles
  const int64_t total = tl.first_chunk[tl.count];
  for (int64_t vc = blockIdx.x; vc < total; vc += gridDim.x) {
    int k = 0;
    while (k + 1 < tl.count && vc >= tl.first_chunk[k + 1]) ++k;
    const int64_t base = (vc - tl.first_chunk[k]) * kChunk;
    float* __restrict__ p = tl.p[k];
    const float* __restrict__ g = tl.g[k];
    const int64_t n = tl.n[k];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int64_t i = base + u * 256 + threadIdx.x;
      if (i < n) p[i] = p[i] - lr * (g[i] + weight_decay * p[i]);
    }
  }
}

int fill_list(TensorList& tl, int n_tensors, float* const* params, const float* const* grads, float* const* exp_avg,
              float* const* exp_avg_sq, const int64_t* sizes, bool adam, const char* who) {
  if (n_tensors < 0 || n_tensors > kMaxTensors)
    return gc::fail(GC_ERR_INVALID, "%s: between 0 and %d tensors per call", who, kMaxTensors);
  tl.count = n_tensors;
  tl.first_chunk[0] = 0;
  for (int k = 0; k < n_tensors; ++k) {
    if (sizes[k] < 0) return gc::fail(GC_ERR_INVALID, "%s: negative size", who);
    if (sizes[k] > 0 && (!params[k] || !grads[k] || (adam && (!exp_avg[k] || !exp_avg_sq[k]))))
      return gc::fail(GC_ERR_INVALID, "%s: null pointer in tensor %d", who, k);
    tl.p[k] = params[k];
    tl.g[k] = grads[k];
    tl.m[k] = adam ? exp_avg[k] : nullptr;
    tl.v[k] = adam ? exp_avg_sq[k] : nullptr;
    tl.n[k] = sizes[k];
    tl.first_chunk[k + 1] = tl.first_chunk[k] + (sizes[k] + kChunk - 1) / kChunk;
  }
  return GC_OK;
}

}  // namespace

extern "C" {

int gc_adam_step_f32(int n_tensors, float* const* params, const float* const* grads, float* const* exp_avg,
                     float* const* exp_avg_sq, const int64_t* sizes, double lr, double beta1, double beta2, double eps,
                     double weight_decay, void* state, void* stream) {
  GC_REQUIRE(state, "gc_adam_step_f32: null state");
  GC_REQUIRE(n_tensors == 0 || (params && grads && exp_avg && exp_avg_sq && sizes), "gc_adam_step_f32: null list");
  TensorList tl;
  int rc = fill_list(tl, n_tensors, params, grads, exp_avg, exp_avg_sq, sizes, true, "gc_adam_step_f32");
  if (rc != GC_OK) return rc;
  const int64_t total = tl.first_chunk[tl.count];
  // an empty model still counts the step
  const int blocks = int(std::max<int64_t>(1, std::min<int64_t>(total, gc::kNumSMs * 8)));
  adam_kernel<<<blocks, 256, 0, gc::as_stream(stream)>>>(tl, lr, beta1, beta2, float(eps), float(weight_decay),
                                                         static_cast<unsigned long long*>(state));
  return gc::check_launch("gc_adam_step_f32");
}

int gc_sgd_step_f32(int n_tensors, float* const* params, const float* const* grads, const int64_t* sizes, double lr,
                    double weight_decay, void* stream) {
  GC_REQUIRE(n_tensors == 0 || (params && grads && sizes), "gc_sgd_step_f32: null list");
  TensorList tl;
  int rc = fill_list(tl, n_tensors, params, grads, nullptr, nullptr, sizes, false, "gc_sgd_step_f32");
  if (rc != GC_OK) return rc;
  const int64_t total = tl.first_chunk[tl.count];
  if (total == 0) return GC_OK;
  const int blocks = int(std::min<int64_t>(total, gc::kNumSMs * 8));
  sgd_kernel<<<blocks, 256, 0, gc::as_stream(stream)>>>(tl, float(lr), float(weight_decay));
  return gc::check_launch("gc_sgd_step_f32");
}

}  // extern "C"

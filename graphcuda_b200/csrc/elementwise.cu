// Element-wise helpers of the GCN layer: the ReLU-mask products of the
// backward pass (src/graphcuda/cuda/gcn.cu:36) and an out-of-place transpose.
#include "common.cuh"

#include <algorithm>

namespace {

template <bool FROM_ACT>
__global__ void __launch_bounds__(256)
mask_mul_kernel(const float* __restrict__ dY, int64_t lddy, const float* __restrict__ S, int64_t lds,
                float* __restrict__ G, int64_t ldg, int64_t M, int N) {
  const int64_t total = M * N;
  for (int64_t i = int64_t(blockIdx.x) * 256 + threadIdx.x; i < total; i += int64_t(gridDim.x) * 256) {
    const int64_t r = i / N;
    const int c = int(i % N);
    const float s = __ldg(S + r * lds + c);
    const float m = FROM_ACT ? (s > 0.f ? 1.f : 0.f) : s;
    G[r * ldg + c] = __ldg(dY + r * lddy + c) * m;
  }
}

// Rows are contiguous and 16-byte aligned on all three operands.
template <bool FROM_ACT>
__global__ void __launch_bounds__(256)
mask_mul_vec4_kernel(const float4* __restrict__ dY, const float4* __restrict__ S, float4* __restrict__ G,
                     int64_t n4) {
  for (int64_t i = int64_t(blockIdx.x) * 256 + threadIdx.x; i < n4; i += int64_t(gridDim.x) * 256) {
    const float4 d = __ldg(dY + i), s = __ldg(S + i);
    float4 g;
    if (FROM_ACT) {
      g.x = d.x * (s.x > 0.f ? 1.f : 0.f);
      g.y = d.y * (s.y > 0.f ? 1.f : 0.f);
      g.z = d.z * (s.z > 0.f ? 1.f : 0.f);
      g.w = d.w * (s.w > 0.f ? 1.f : 0.f);
    } else {
      g.x = d.x * s.x; g.y = d.y * s.y; g.z = d.z * s.z; g.w = d.w * s.w;
    }
    G[i] = g;
  }
}

__global__ void __launch_bounds__(256)
transpose_kernel(const float* __restrict__ in, int64_t ldin, float* __restrict__ out, int64_t ldout, int R, int Cc) {
  __shared__ float t[32][33];
  const int tx = threadIdx.x % 32, ty = threadIdx.x / 32;
  const int64_t tiles_c = (Cc + 31) / 32;
  const int64_t tiles = int64_t((R + 31) / 32) * tiles_c;
  for (int64_t tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
    const int r0 = int(tile / tiles_c) * 32, c0 = int(tile % tiles_c) * 32;
    for (int i = ty; i < 32; i += 8)
      t[i][tx] = (r0 + i < R && c0 + tx < Cc) ? __ldg(in + int64_t(r0 + i) * ldin + c0 + tx) : 0.f;
    __syncthreads();
    for (int i = ty; i < 32; i += 8)
      if (c0 + i < Cc && r0 + tx < R) out[int64_t(c0 + i) * ldout + r0 + tx] = t[tx][i];
    __syncthreads();
  }
}

template <bool FROM_ACT>
int mask_mul(const float* dY, int64_t lddy, const float* S, int64_t lds, float* G, int64_t ldg, int64_t M, int64_t N,
             void* stream, const char* who) {
  GC_REQUIRE(M >= 0 && N >= 0 && N < INT32_MAX, "%s: bad size", who);
  if (M == 0 || N == 0) return GC_OK;
  GC_REQUIRE(dY && S && G, "%s: null pointer", who);
  GC_REQUIRE(lddy >= N && lds >= N && ldg >= N, "%s: leading dimension smaller than N", who);
  cudaStream_t st = gc::as_stream(stream);
  const bool dense = lddy == N && lds == N && ldg == N && (M * N) % 4 == 0 && gc::aligned16(dY) &&
                     gc::aligned16(S) && gc::aligned16(G);
  if (dense) {
    const int64_t n4 = M * N / 4;
    const unsigned grid = unsigned(std::min<int64_t>(gc::ceil_div(n4, 256), gc::kNumSMs * 16));
    mask_mul_vec4_kernel<FROM_ACT><<<grid, 256, 0, st>>>(reinterpret_cast<const float4*>(dY),
                                                         reinterpret_cast<const float4*>(S),
                                                         reinterpret_cast<float4*>(G), n4);
  } else {
    const unsigned grid = unsigned(std::min<int64_t>(gc::ceil_div(M * N, 256), gc::kNumSMs * 16));
    mask_mul_kernel<FROM_ACT><<<grid, 256, 0, st>>>(dY, lddy, S, lds, G, ldg, M, int(N));
  }
  return gc::check_launch(who);
}

// Column slabs of a row-major matrix, each to its own destination matrix: dst[q][r, c] = src[r, q * w + c].
// The destinations may be other GPUs' buffers (peer-mapped memory): the rows -> columns transpose of the
// feature-sharded multi-GPU scheme as ONE kernel of ordinary loads and stores, every element read once.
struct SlabDests {
  float* base[GC_SPMM_MAX_BLOCKS];
};

template <int VW>
__global__ void __launch_bounds__(256)
scatter_slabs_kernel(const float* __restrict__ src, int64_t ld, int64_t rows, int F, int w, int64_t dst_ld,
                     const __grid_constant__ SlabDests d) {
  const int per_row = (F + VW - 1) / VW;
  const int64_t total = rows * per_row;
  for (int64_t i = int64_t(blockIdx.x) * 256 + threadIdx.x; i < total; i += int64_t(gridDim.x) * 256) {
    const int64_t r = i / per_row;
    const int c = int(i % per_row) * VW;
    const int q = c / w;
    float* out = d.base[q] + r * dst_ld + (c - q * w);
    if (VW == 4) {
      *reinterpret_cast<float4*>(out) = __ldcs(reinterpret_cast<const float4*>(src + r * ld + c));
    } else {
      *out = __ldcs(src + r * ld + c);
    }
  }
}

}  // namespace

extern "C" {

int gc_scatter_column_slabs_f32(const float* src, int64_t ld, int64_t rows, int64_t F, int64_t w, float* const* dst,
                                int n_dst, int64_t dst_ld, void* stream) {
  GC_REQUIRE(rows >= 0 && F >= 0 && F < INT32_MAX && w >= 1 && w < INT32_MAX, "gc_scatter_column_slabs_f32: bad size");
  GC_REQUIRE(n_dst >= 1 && n_dst <= GC_SPMM_MAX_BLOCKS && int64_t(n_dst) * w >= F,
             "gc_scatter_column_slabs_f32: n_dst slabs of w columns must cover F (at most %d slabs)", GC_SPMM_MAX_BLOCKS);
  if (rows == 0 || F == 0) return GC_OK;
  GC_REQUIRE(src && dst && ld >= F && dst_ld >= w, "gc_scatter_column_slabs_f32: null pointer or leading dimension");
  SlabDests d{};
  bool vec = (w % 4 == 0) && (F % 4 == 0) && (ld % 4 == 0) && (dst_ld % 4 == 0) && gc::aligned16(src);
  for (int q = 0; q < n_dst; ++q) {
    GC_REQUIRE(dst[q] || int64_t(q) * w >= F, "gc_scatter_column_slabs_f32: null destination");
    d.base[q] = dst[q];
    vec = vec && gc::aligned16(dst[q]);
  }
  const int64_t items = rows * (vec ? (F + 3) / 4 : F);
  const unsigned grid = unsigned(std::min<int64_t>(gc::ceil_div(items, 256), gc::kNumSMs * 16));
  if (vec) scatter_slabs_kernel<4><<<grid, 256, 0, gc::as_stream(stream)>>>(src, ld, rows, int(F), int(w), dst_ld, d);
  else scatter_slabs_kernel<1><<<grid, 256, 0, gc::as_stream(stream)>>>(src, ld, rows, int(F), int(w), dst_ld, d);
  return gc::check_launch("gc_scatter_column_slabs_f32");
}

int gc_relu_backward_f32(const float* dY, int64_t lddy, const float* Y, int64_t ldy, float* G, int64_t ldg,
                         int64_t M, int64_t N, void* stream) {
  return mask_mul<true>(dY, lddy, Y, ldy, G, ldg, M, N, stream, "gc_relu_backward_f32");
}

int gc_mask_mul_f32(const float* dY, int64_t lddy, const float* mask, int64_t ldm, float* G, int64_t ldg,
                    int64_t M, int64_t N, void* stream) {
  return mask_mul<false>(dY, lddy, mask, ldm, G, ldg, M, N, stream, "gc_mask_mul_f32");
}

int gc_transpose_f32(const float* in, int64_t ldin, float* out, int64_t ldout, int64_t M, int64_t N, void* stream) {
  GC_REQUIRE(M >= 0 && N >= 0 && M < INT32_MAX && N < INT32_MAX, "gc_transpose_f32: bad size");
  if (M == 0 || N == 0) return GC_OK;
  GC_REQUIRE(in && out, "gc_transpose_f32: null pointer");
  GC_REQUIRE(ldin >= N && ldout >= M, "gc_transpose_f32: leading dimension too small");
  const int64_t tiles = gc::ceil_div(M, 32) * gc::ceil_div(N, 32);
  const unsigned grid = unsigned(std::min<int64_t>(tiles, gc::kNumSMs * 16));
  transpose_kernel<<<grid, 256, 0, gc::as_stream(stream)>>>(in, ldin, out, ldout, int(M), int(N));
  return gc::check_launch("gc_transpose_f32");
}

}  // extern "C"

// Adjacency construction on the GPU: GCN normalisation, COO -> CSR, symmetry
// test.  Takes over what the reference's scripts do with torch_geometric and
// torch sparse tensors before the layer is called
// (tests/gcn/graphcuda_impl.py:27-38: add_self_loops -> gcn_norm ->
// sparse_coo_tensor(...).coalesce()).
//
// Built WITHOUT fast-math: the normalisation must round exactly like torch's
// CPU kernels (1.0f / sqrtf(d), then two IEEE multiplications).
#include "common.cuh"

#include <algorithm>
#include <cub/device/device_scan.cuh>

namespace {

__global__ void __launch_bounds__(256)
rows_to_rowptr_kernel(const int64_t* __restrict__ rows, int64_t nnz, int64_t M, int32_t* __restrict__ rowptr) {
  const int64_t stride = int64_t(gridDim.x) * 256;
  for (int64_t e = int64_t(blockIdx.x) * 256 + threadIdx.x; e <= nnz; e += stride) {
    // entry e opens every row in (rows[e-1], rows[e]]; e == nnz closes the tail
    const int64_t prev = e > 0 ? rows[e - 1] : -1;
    const int64_t cur = e < nnz ? rows[e] : M;
    for (int64_t r = prev + 1; r <= cur && r <= M; ++r) rowptr[r] = int32_t(e);
  }
}

__global__ void __launch_bounds__(256)
narrow_kernel(const int64_t* __restrict__ src, int32_t* __restrict__ dst, int64_t n) {
  for (int64_t i = int64_t(blockIdx.x) * 256 + threadIdx.x; i < n; i += int64_t(gridDim.x) * 256)
    dst[i] = int32_t(src[i]);
}

__global__ void __launch_bounds__(256)
degree_kernel(const int64_t* __restrict__ col, int64_t E, int32_t* __restrict__ deg) {
  for (int64_t e = int64_t(blockIdx.x) * 256 + threadIdx.x; e < E; e += int64_t(gridDim.x) * 256)
    atomicAdd(deg + col[e], 1);  // integer counts: exact and order-independent
}

__global__ void __launch_bounds__(256)
dinv_kernel(int32_t* __restrict__ deg_then_dinv, int64_t N) {
  for (int64_t i = int64_t(blockIdx.x) * 256 + threadIdx.x; i < N; i += int64_t(gridDim.x) * 256) {
    const float d = float(deg_then_dinv[i]);
    // pow(d, -0.5) on torch CPU == 1.0f / sqrtf(d); isolated nodes: inf -> 0
    const float r = d > 0.f ? __fdiv_rn(1.0f, __fsqrt_rn(d)) : 0.f;
    reinterpret_cast<float*>(deg_then_dinv)[i] = r;
  }
}

__global__ void __launch_bounds__(256)
norm_weight_kernel(const int64_t* __restrict__ row, const int64_t* __restrict__ col, int64_t E,
                   const float* __restrict__ dinv, float* __restrict__ w) {
  for (int64_t e = int64_t(blockIdx.x) * 256 + threadIdx.x; e < E; e += int64_t(gridDim.x) * 256) {
    // dinv[row] * 1.0f * dinv[col], left to right
    const float a = __fmul_rn(dinv[row[e]], 1.0f);
    w[e] = __fmul_rn(a, dinv[col[e]]);
  }
}

__global__ void __launch_bounds__(256)
head_flag_kernel(const int64_t* __restrict__ row, const int64_t* __restrict__ col, int64_t E,
                 int32_t* __restrict__ head) {
  for (int64_t e = int64_t(blockIdx.x) * 256 + threadIdx.x; e < E; e += int64_t(gridDim.x) * 256)
    head[e] = (e == 0 || row[e] != row[e - 1] || col[e] != col[e - 1]) ? 1 : 0;
}

__global__ void total_kernel(const int64_t* __restrict__ row, const int64_t* __restrict__ col, int64_t E,
                             const int32_t* __restrict__ head_excl, int64_t* __restrict__ nnz_out) {
  if (E == 0) { *nnz_out = 0; return; }
  const int64_t e = E - 1;
  const int last = (e == 0 || row[e] != row[e - 1] || col[e] != col[e - 1]) ? 1 : 0;
  *nnz_out = int64_t(head_excl[e]) + last;
}

__global__ void __launch_bounds__(256)
csr_fill_kernel(const int64_t* __restrict__ row, const int64_t* __restrict__ col, const float* __restrict__ w,
                int64_t E, int64_t M, const int32_t* __restrict__ head_excl, int32_t* __restrict__ rowptr,
                int32_t* __restrict__ csr_col, float* __restrict__ csr_val) {
  const int64_t stride = int64_t(gridDim.x) * 256;
  for (int64_t e = int64_t(blockIdx.x) * 256 + threadIdx.x; e <= E; e += stride) {
    if (e == E) {
      // close the tail rows
      const int64_t prev = E > 0 ? row[E - 1] : -1;
      int32_t nnz = 0;
      if (E > 0) {
        const int64_t l = E - 1;
        nnz = head_excl[l] + ((l == 0 || row[l] != row[l - 1] || col[l] != col[l - 1]) ? 1 : 0);
      }
      for (int64_t r = prev + 1; r <= M; ++r) rowptr[r] = nnz;
      continue;
    }
    const bool new_row = (e == 0) || row[e] != row[e - 1];
    const bool is_head = new_row || col[e] != col[e - 1];
    if (!is_head) continue;
    const int32_t j = head_excl[e];
    if (new_row) {
      const int64_t prev = e > 0 ? row[e - 1] : -1;
      for (int64_t r = prev + 1; r <= row[e]; ++r) rowptr[r] = j;
    }
    // duplicates are added in input order
    float s = w[e];
    for (int64_t d = e + 1; d < E && row[d] == row[e] && col[d] == col[e]; ++d) s += w[d];
    csr_col[j] = int32_t(col[e]);
    csr_val[j] = s;
  }
}

__global__ void set_one_kernel(int32_t* out) { *out = 1; }

// One warp per row; every entry (i, j, v) looks for (j, i) by bisection of
// row j (columns sorted) and compares the value bits.
__global__ void __launch_bounds__(256)
symmetric_kernel(const int32_t* __restrict__ rowptr, const int32_t* __restrict__ col,
                 const float* __restrict__ val, int M, int32_t* __restrict__ out) {
  const int lane = threadIdx.x % 32;
  const int64_t warps = int64_t(gridDim.x) * 8;
  for (int64_t i = int64_t(blockIdx.x) * 8 + threadIdx.x / 32; i < M; i += warps) {
    const int s = rowptr[i], e = rowptr[i + 1];
    for (int p = s + lane; p < e; p += 32) {
      const int j = col[p];
      bool found = false;
      if (j >= 0 && j < M) {
        int lo = rowptr[j], hi = rowptr[j + 1];
        while (lo < hi) {
          const int mid = (lo + hi) >> 1;
          const int c = col[mid];
          if (c < int(i)) lo = mid + 1; else hi = mid;
        }
        if (lo < rowptr[j + 1] && col[lo] == int(i))
          found = __float_as_uint(val[lo]) == __float_as_uint(val[p]);
      }
      if (!found) *out = 0;
    }
  }
}

inline unsigned grid_for(int64_t n) {
  return unsigned(std::max<int64_t>(1, std::min<int64_t>(gc::ceil_div(n, 256), gc::kNumSMs * 16)));
}

}  // namespace

extern "C" {

int gc_coo_rows_to_rowptr(const int64_t* rows, int64_t nnz, int64_t M, int32_t* rowptr, void* stream) {
  GC_REQUIRE(nnz >= 0 && M >= 0 && nnz < INT32_MAX && M < INT32_MAX, "gc_coo_rows_to_rowptr: size out of range");
  GC_REQUIRE(rowptr && (nnz == 0 || rows), "gc_coo_rows_to_rowptr: null pointer");
  rows_to_rowptr_kernel<<<grid_for(nnz + 1), 256, 0, gc::as_stream(stream)>>>(rows, nnz, M, rowptr);
  return gc::check_launch("gc_coo_rows_to_rowptr");
}

int gc_narrow_i64_i32(const int64_t* src, int32_t* dst, int64_t n, void* stream) {
  GC_REQUIRE(n >= 0, "gc_narrow_i64_i32: negative size");
  if (n == 0) return GC_OK;
  GC_REQUIRE(src && dst, "gc_narrow_i64_i32: null pointer");
  narrow_kernel<<<grid_for(n), 256, 0, gc::as_stream(stream)>>>(src, dst, n);
  return gc::check_launch("gc_narrow_i64_i32");
}

int gc_gcn_norm_f32(const int64_t* row, const int64_t* col, int64_t E, int64_t N, float* deg_scratch, float* w,
                    void* stream) {
  GC_REQUIRE(E >= 0 && N >= 0 && N < INT32_MAX, "gc_gcn_norm_f32: size out of range");
  if (E == 0 || N == 0) return GC_OK;
  GC_REQUIRE(row && col && deg_scratch && w, "gc_gcn_norm_f32: null pointer");
  cudaStream_t st = gc::as_stream(stream);
  cudaError_t e = cudaMemsetAsync(deg_scratch, 0, size_t(N) * 4, st);
  if (e != cudaSuccess) return gc::fail(GC_ERR_CUDA, "gc_gcn_norm_f32: %s", cudaGetErrorString(e));
  int32_t* deg = reinterpret_cast<int32_t*>(deg_scratch);
  degree_kernel<<<grid_for(E), 256, 0, st>>>(col, E, deg);
  dinv_kernel<<<grid_for(N), 256, 0, st>>>(deg, N);
  norm_weight_kernel<<<grid_for(E), 256, 0, st>>>(row, col, E, deg_scratch, w);
  return gc::check_launch("gc_gcn_norm_f32", 3);
}

size_t gc_csr_build_workspace_bytes(int64_t E) {
  if (E <= 0) return 256;
  size_t bytes = 0;
  cub::DeviceScan::ExclusiveSum(nullptr, bytes, static_cast<int32_t*>(nullptr), static_cast<int32_t*>(nullptr),
                                int(std::min<int64_t>(E, INT32_MAX)));
  return std::max<size_t>(bytes, 256);
}

int gc_csr_count_unique(const int64_t* row, const int64_t* col, int64_t E, int32_t* head, int64_t* nnz_out,
                        void* workspace, size_t workspace_bytes, void* stream) {
  GC_REQUIRE(E >= 0 && E < INT32_MAX, "gc_csr_count_unique: E out of int32 range");
  GC_REQUIRE(nnz_out, "gc_csr_count_unique: null nnz_out");
  cudaStream_t st = gc::as_stream(stream);
  if (E > 0) {
    GC_REQUIRE(row && col && head, "gc_csr_count_unique: null pointer");
    if (!workspace || workspace_bytes < gc_csr_build_workspace_bytes(E))
      return gc::fail(GC_ERR_WORKSPACE, "gc_csr_count_unique: workspace too small");
    head_flag_kernel<<<grid_for(E), 256, 0, st>>>(row, col, E, head);
    size_t bytes = workspace_bytes;
    cudaError_t e = cub::DeviceScan::ExclusiveSum(workspace, bytes, head, head, int(E), st);
    if (e != cudaSuccess) return gc::fail(GC_ERR_CUDA, "gc_csr_count_unique: scan: %s", cudaGetErrorString(e));
  }
  total_kernel<<<1, 1, 0, st>>>(row, col, E, head, nnz_out);
  return gc::check_launch("gc_csr_count_unique", E > 0 ? 2 : 1);
}

int gc_csr_fill(const int64_t* row, const int64_t* col, const float* w, int64_t E, int64_t M, const int32_t* head,
                int32_t* rowptr, int32_t* csr_col, float* csr_val, void* stream) {
  GC_REQUIRE(E >= 0 && E < INT32_MAX && M >= 0 && M < INT32_MAX, "gc_csr_fill: size out of int32 range");
  GC_REQUIRE(rowptr, "gc_csr_fill: null rowptr");
  GC_REQUIRE(E == 0 || (row && col && w && head && csr_col && csr_val), "gc_csr_fill: null pointer");
  csr_fill_kernel<<<grid_for(E + 1), 256, 0, gc::as_stream(stream)>>>(row, col, w, E, M, head, rowptr, csr_col,
                                                                       csr_val);
  return gc::check_launch("gc_csr_fill");
}

int gc_csr_is_symmetric(const int32_t* rowptr, const int32_t* col, const float* val, int64_t M, int32_t* out,
                        void* stream) {
  GC_REQUIRE(M >= 0 && M < INT32_MAX, "gc_csr_is_symmetric: M out of range");
  GC_REQUIRE(out, "gc_csr_is_symmetric: null out");
  cudaStream_t st = gc::as_stream(stream);
  set_one_kernel<<<1, 1, 0, st>>>(out);
  if (M > 0) {
    GC_REQUIRE(rowptr, "gc_csr_is_symmetric: null rowptr");
    const unsigned grid = unsigned(std::min<int64_t>(gc::ceil_div(M, 8), gc::kNumSMs * 16));
    symmetric_kernel<<<grid, 256, 0, st>>>(rowptr, col, val, int(M), out);
  }
  return gc::check_launch("gc_csr_is_symmetric", M > 0 ? 2 : 1);
}

}  // extern "C"

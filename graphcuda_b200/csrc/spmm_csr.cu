// CSR (int32) x dense fp32 aggregation  Y = A * H (+bias)(ReLU)(mask).
//
// Takes over the reference's cuSPARSE COO SpMM wrapper
// (src/graphcuda/cuda/spmm_cusparse.cu:3-126) on the GCN path
// (src/graphcuda/cuda/gcn.cu:12,40,49).
//
// HBM/L2-bound gather.  Layout and schedule:
//   * a row of Y is produced by a "group" of GROUP lanes (GROUP = 2..32, the
//     smallest power of two that covers the feature width with 128-bit
//     loads), so narrow feature widths keep all 32 lanes of a warp busy on
//     several rows at once;
//   * the group's lanes fetch GROUP (col,val) pairs with one coalesced load
//     and broadcast them with shuffles; the H row of each non-zero is read
//     with 128-bit loads, four non-zeros in flight per lane;
//   * rows longer than GC_SPMM_LONG_ROW are cut into GC_SPMM_SEGMENT-sized
//     segments, one CTA per segment, partial sums to scratch, then a
//     finalize pass adds the segments in order -- no atomics anywhere, so the
//     result is bit-reproducible run to run;
//   * bias, ReLU (as y * (y > 0), the reference's formula, gcn.cu:19-20), the
//     fp32 mask and an optional accumulate are fused into the store.
#include "common.cuh"

#include <mutex>

namespace {

struct PlanHeader {
  int32_t n_long;
  int32_t n_seg;
  int32_t pad[2];
};

__host__ __device__ inline size_t plan_long_rows_offset() { return sizeof(PlanHeader); }
__host__ __device__ inline size_t plan_seg_off_offset(int64_t M) {
  return sizeof(PlanHeader) + ((size_t(M) * 4 + 15) & ~size_t(15));
}

// ---------------------------------------------------------------- epilogue
struct Epilogue {
  const float* bias;
  float* mask;
  int relu;
  int accumulate;
};

template <int VW>
struct Vec;
template <>
struct Vec<4> {
  using T = float4;
  static __device__ __forceinline__ T zero() { return make_float4(0.f, 0.f, 0.f, 0.f); }
  static __device__ __forceinline__ T load(const float* p) { return __ldg(reinterpret_cast<const float4*>(p)); }
  static __device__ __forceinline__ T load_plain(const float* p) { return *reinterpret_cast<const float4*>(p); }
  static __device__ __forceinline__ void store(float* p, T v) { *reinterpret_cast<float4*>(p) = v; }
  static __device__ __forceinline__ void fma(T& a, float s, const T& h) {
    a.x = fmaf(s, h.x, a.x);
    a.y = fmaf(s, h.y, a.y);
    a.z = fmaf(s, h.z, a.z);
    a.w = fmaf(s, h.w, a.w);
  }
  static __device__ __forceinline__ T add(const T& a, const T& b) {
    return make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w);
  }
  static __device__ __forceinline__ T gt0(const T& a) {
    return make_float4(a.x > 0.f ? 1.f : 0.f, a.y > 0.f ? 1.f : 0.f, a.z > 0.f ? 1.f : 0.f, a.w > 0.f ? 1.f : 0.f);
  }
  static __device__ __forceinline__ T mul(const T& a, const T& b) {
    return make_float4(a.x * b.x, a.y * b.y, a.z * b.z, a.w * b.w);
  }
};
template <>
struct Vec<1> {
  using T = float;
  static __device__ __forceinline__ T zero() { return 0.f; }
  static __device__ __forceinline__ T load(const float* p) { return __ldg(p); }
  static __device__ __forceinline__ T load_plain(const float* p) { return *p; }
  static __device__ __forceinline__ void store(float* p, T v) { *p = v; }
  static __device__ __forceinline__ void fma(T& a, float s, const T& h) { a = fmaf(s, h, a); }
  static __device__ __forceinline__ T add(const T& a, const T& b) { return a + b; }
  static __device__ __forceinline__ T gt0(const T& a) { return a > 0.f ? 1.f : 0.f; }
  static __device__ __forceinline__ T mul(const T& a, const T& b) { return a * b; }
};

// Applies accumulate / bias / mask / ReLU to one vector and stores it.
template <int VW>
__device__ __forceinline__ void finish_store(typename Vec<VW>::T acc, float* yrow, float* mrow, int f,
                                             const Epilogue& ep) {
  using V = Vec<VW>;
  if (ep.accumulate) acc = V::add(acc, V::load_plain(yrow + f));
  if (ep.bias) acc = V::add(acc, V::load(ep.bias + f));
  if (ep.relu || mrow) {
    typename V::T m = V::gt0(acc);
    if (mrow) V::store(mrow + f, m);
    if (ep.relu) acc = V::mul(acc, m);
  }
  V::store(yrow + f, acc);
}

// ---------------------------------------------------------------- row kernel
// One group of GROUP lanes per row; NACC vectors of VW floats per lane cover
// GROUP*NACC*VW feature columns per pass; wider F loops over passes.
template <int GROUP, int NACC, int VW>
__global__ void __launch_bounds__(256)
spmm_rows_kernel(const int32_t* __restrict__ rowptr, const int32_t* __restrict__ col,
                 const float* __restrict__ val, int M, int F, const float* __restrict__ H, int64_t ldH,
                 float* __restrict__ Y, int64_t ldY, Epilogue ep, int skip_long) {
  using V = Vec<VW>;
  constexpr int ROWS_PER_CTA = 256 / GROUP;
  constexpr int PASS = GROUP * NACC * VW;
  constexpr int U = GROUP < 4 ? GROUP : 4;
  const int lane_g = threadIdx.x % GROUP;
  const int row = blockIdx.x * ROWS_PER_CTA + threadIdx.x / GROUP;
  if (row >= M) return;
  const unsigned gmask = (GROUP == 32) ? 0xffffffffu
                                       : (((1u << GROUP) - 1u) << ((threadIdx.x % 32) / GROUP * GROUP));
  const int start = __ldg(rowptr + row);
  const int end = __ldg(rowptr + row + 1);
  if (skip_long && (end - start) > GC_SPMM_LONG_ROW) return;
  float* yrow = Y + int64_t(row) * ldY;
  float* mrow = ep.mask ? ep.mask + int64_t(row) * ldY : nullptr;

  for (int f0 = 0; f0 < F; f0 += PASS) {
    typename V::T acc[NACC];
#pragma unroll
    for (int a = 0; a < NACC; ++a) acc[a] = V::zero();
    bool live[NACC];
#pragma unroll
    for (int a = 0; a < NACC; ++a) live[a] = (f0 + (a * GROUP + lane_g) * VW) < F;

    for (int base = start; base < end; base += GROUP) {
      const int e = base + lane_g;
      int c = 0;
      float v = 0.f;
      if (e < end) {
        c = __ldg(col + e);
        v = __ldg(val + e);
      }
      const int cnt = min(GROUP, end - base);
      // U gathers in flight per lane; entries past the end of the row are
      // never loaded (a 0 * Inf would poison the sum).
      for (int j = 0; j < cnt; j += U) {
        int cj[U];
        float vj[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          cj[u] = __shfl_sync(gmask, c, j + u, GROUP);
          vj[u] = __shfl_sync(gmask, v, j + u, GROUP);
        }
        typename V::T h[U][NACC];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const float* hp = H + int64_t(cj[u]) * ldH + f0;
          const bool valid = (j + u) < cnt;
#pragma unroll
          for (int a = 0; a < NACC; ++a)
            h[u][a] = (live[a] && valid) ? V::load(hp + (a * GROUP + lane_g) * VW) : V::zero();
        }
#pragma unroll
        for (int u = 0; u < U; ++u)
#pragma unroll
          for (int a = 0; a < NACC; ++a) V::fma(acc[a], (j + u) < cnt ? vj[u] : 0.f, h[u][a]);
      }
    }
#pragma unroll
    for (int a = 0; a < NACC; ++a)
      if (live[a]) finish_store<VW>(acc[a], yrow, mrow, f0 + (a * GROUP + lane_g) * VW, ep);
  }
}

// ---------------------------------------------------------------- long rows
// One CTA (8 warps) per segment of a long row; warps interleave 32-entry
// batches, then their partial vectors are added in warp order through shared
// memory and written to scratch[segment][F].
template <int NACC, int VW>
__global__ void __launch_bounds__(256)
spmm_segments_kernel(const int32_t* __restrict__ rowptr, const int32_t* __restrict__ col,
                     const float* __restrict__ val, int F, const float* __restrict__ H, int64_t ldH,
                     const PlanHeader* __restrict__ hdr, const int32_t* __restrict__ long_rows,
                     const int32_t* __restrict__ seg_off, float* __restrict__ scratch, int64_t ldS,
                     int seg_capacity) {
  using V = Vec<VW>;
  constexpr int PASS = 32 * NACC * VW;
  __shared__ __align__(16) float red[8][PASS];
  const int lane = threadIdx.x % 32, warp = threadIdx.x / 32;
  // never write past the caller's scratch, whatever the plan says
  const int n_seg = min(hdr->n_seg, seg_capacity), n_long = hdr->n_long;
  for (int seg = blockIdx.x; seg < n_seg; seg += gridDim.x) {
    // largest i with seg_off[i] <= seg
    int lo = 0, hi = n_long;
    while (hi - lo > 1) {
      int mid = (lo + hi) >> 1;
      if (__ldg(seg_off + mid) <= seg) lo = mid; else hi = mid;
    }
    const int row = __ldg(long_rows + lo);
    const int rstart = __ldg(rowptr + row), rend = __ldg(rowptr + row + 1);
    const int start = rstart + (seg - __ldg(seg_off + lo)) * GC_SPMM_SEGMENT;
    const int end = min(start + GC_SPMM_SEGMENT, rend);
    for (int f0 = 0; f0 < F; f0 += PASS) {
      typename V::T acc[NACC];
      bool live[NACC];
#pragma unroll
      for (int a = 0; a < NACC; ++a) {
        acc[a] = V::zero();
        live[a] = (f0 + (a * 32 + lane) * VW) < F;
      }
      for (int base = start + warp * 32; base < end; base += 256) {
        const int e = base + lane;
        int c = 0;
        float v = 0.f;
        if (e < end) {
          c = __ldg(col + e);
          v = __ldg(val + e);
        }
        const int cnt = min(32, end - base);
        for (int j = 0; j < cnt; j += 4) {
          int cj[4];
          float vj[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            cj[u] = __shfl_sync(0xffffffffu, c, (j + u) & 31);
            vj[u] = __shfl_sync(0xffffffffu, v, (j + u) & 31);
          }
          typename V::T h[4][NACC];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const float* hp = H + int64_t(cj[u]) * ldH + f0;
            const bool valid = (j + u) < cnt;
#pragma unroll
            for (int a = 0; a < NACC; ++a)
              h[u][a] = (live[a] && valid) ? V::load(hp + (a * 32 + lane) * VW) : V::zero();
          }
#pragma unroll
          for (int u = 0; u < 4; ++u)
#pragma unroll
            for (int a = 0; a < NACC; ++a) V::fma(acc[a], (j + u) < cnt ? vj[u] : 0.f, h[u][a]);
        }
      }
#pragma unroll
      for (int a = 0; a < NACC; ++a) V::store(&red[warp][(a * 32 + lane) * VW], acc[a]);
      __syncthreads();
      for (int i = threadIdx.x; i < PASS; i += 256) {
        if (f0 + i < F) {
          float s = red[0][i];
#pragma unroll
          for (int w = 1; w < 8; ++w) s += red[w][i];
          scratch[int64_t(seg) * ldS + f0 + i] = s;
        }
      }
      __syncthreads();
    }
  }
}

// One warp per long row: adds that row's segments in order, then the fused store.
__global__ void __launch_bounds__(256)
spmm_finalize_kernel(int F, const PlanHeader* __restrict__ hdr, const int32_t* __restrict__ long_rows,
                     const int32_t* __restrict__ seg_off, const float* __restrict__ scratch, int64_t ldS,
                     float* __restrict__ Y, int64_t ldY, Epilogue ep) {
  const int lane = threadIdx.x % 32;
  const int n_long = hdr->n_long;
  const int warps = gridDim.x * 8;
  for (int i = blockIdx.x * 8 + threadIdx.x / 32; i < n_long; i += warps) {
    const int row = __ldg(long_rows + i);
    const int s0 = __ldg(seg_off + i), s1 = __ldg(seg_off + i + 1);
    float* yrow = Y + int64_t(row) * ldY;
    float* mrow = ep.mask ? ep.mask + int64_t(row) * ldY : nullptr;
    for (int f = lane; f < F; f += 32) {
      float s = 0.f;
      for (int sgi = s0; sgi < s1; ++sgi) s += scratch[int64_t(sgi) * ldS + f];
      finish_store<1>(s, yrow, mrow, f, ep);
    }
  }
}

// ---------------------------------------------------------------- plan
__global__ void plan_collect_kernel(const int32_t* __restrict__ rowptr, int M, PlanHeader* hdr,
                                    int32_t* __restrict__ flags) {
  int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row < M) flags[row] = (__ldg(rowptr + row + 1) - __ldg(rowptr + row)) > GC_SPMM_LONG_ROW ? 1 : 0;
}

// Single CTA: ordered compaction of the long rows (ascending row id) and the
// running segment count.  The per-row flags live in the seg_off area of the
// plan (M+1 ints); pass 1 consumes all of them before pass 2 overwrites the
// first n_long+1 entries with the segment offsets.
__global__ void __launch_bounds__(1024)
plan_scan_kernel(const int32_t* __restrict__ rowptr, int M, PlanHeader* hdr, int32_t* long_rows,
                 int32_t* flags_then_seg_off) {
  __shared__ int warp_sums[32];
  __shared__ int carry_s;
  const int tid = threadIdx.x, lane = tid % 32, warp = tid / 32;
  if (tid == 0) carry_s = 0;
  __syncthreads();
  // pass 1: compact long rows in ascending order
  for (int base = 0; base < M; base += 1024) {
    const int row = base + tid;
    const int f = (row < M) ? flags_then_seg_off[row] : 0;
    int x = f;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      int y = __shfl_up_sync(0xffffffffu, x, o);
      if (lane >= o) x += y;
    }
    if (lane == 31) warp_sums[warp] = x;
    __syncthreads();
    if (warp == 0) {
      int w = warp_sums[lane];
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        int y = __shfl_up_sync(0xffffffffu, w, o);
        if (lane >= o) w += y;
      }
      warp_sums[lane] = w;
    }
    __syncthreads();
    const int carry = carry_s;
    const int incl = x + (warp ? warp_sums[warp - 1] : 0);
    if (f) long_rows[carry + incl - 1] = row;
    __syncthreads();
    if (tid == 1023) carry_s = carry + incl;
    __syncthreads();
  }
  const int n_long = carry_s;
  __syncthreads();
  // pass 2: exclusive scan of segments per long row
  if (tid == 0) carry_s = 0;
  __syncthreads();
  for (int base = 0; base < n_long; base += 1024) {
    const int i = base + tid;
    int nseg = 0;
    if (i < n_long) {
      const int r = long_rows[i];
      const int deg = __ldg(rowptr + r + 1) - __ldg(rowptr + r);
      nseg = (deg + GC_SPMM_SEGMENT - 1) / GC_SPMM_SEGMENT;
    }
    int x = nseg;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      int y = __shfl_up_sync(0xffffffffu, x, o);
      if (lane >= o) x += y;
    }
    if (lane == 31) warp_sums[warp] = x;
    __syncthreads();
    if (warp == 0) {
      int w = warp_sums[lane];
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        int y = __shfl_up_sync(0xffffffffu, w, o);
        if (lane >= o) w += y;
      }
      warp_sums[lane] = w;
    }
    __syncthreads();
    const int carry = carry_s;
    const int incl = x + (warp ? warp_sums[warp - 1] : 0);
    if (i < n_long) flags_then_seg_off[i] = carry + incl - nseg;
    __syncthreads();
    if (tid == 1023) carry_s = carry + incl;
    __syncthreads();
  }
  if (tid == 0) {
    flags_then_seg_off[n_long] = carry_s;
    hdr->n_long = n_long;
    hdr->n_seg = carry_s;
    hdr->pad[0] = hdr->pad[1] = 0;
  }
}

// ---------------------------------------------------------------- dispatch
template <int GROUP, int NACC, int VW>
void launch_rows(const int32_t* rowptr, const int32_t* col, const float* val, int M, int F, const float* H,
                 int64_t ldH, float* Y, int64_t ldY, const Epilogue& ep, int skip_long, cudaStream_t st) {
  constexpr int ROWS_PER_CTA = 256 / GROUP;
  const unsigned grid = unsigned((M + ROWS_PER_CTA - 1) / ROWS_PER_CTA);
  spmm_rows_kernel<GROUP, NACC, VW><<<grid, 256, 0, st>>>(rowptr, col, val, M, F, H, ldH, Y, ldY, ep, skip_long);
}

template <int VW>
void dispatch_rows(const int32_t* rowptr, const int32_t* col, const float* val, int M, int F, const float* H,
                   int64_t ldH, float* Y, int64_t ldY, const Epilogue& ep, int skip_long, cudaStream_t st) {
  const int units = (F + VW - 1) / VW;  // vectors per row
#define GC_ROWS(G, A) launch_rows<G, A, VW>(rowptr, col, val, M, F, H, ldH, Y, ldY, ep, skip_long, st)
  if (units <= 2) GC_ROWS(2, 1);
  else if (units <= 4) GC_ROWS(4, 1);
  else if (units <= 8) GC_ROWS(8, 1);
  else if (units <= 16) GC_ROWS(16, 1);
  else if (units <= 32) GC_ROWS(32, 1);
  else if (units <= 64) GC_ROWS(32, 2);
  else GC_ROWS(32, 4);
#undef GC_ROWS
}

template <int VW>
void dispatch_segments(const int32_t* rowptr, const int32_t* col, const float* val, int F, const float* H,
                       int64_t ldH, const PlanHeader* hdr, const int32_t* long_rows, const int32_t* seg_off,
                       float* scratch, int64_t ldS, int cap, cudaStream_t st) {
  const int units = (F + VW - 1) / VW;
  const unsigned grid = gc::kNumSMs * 8;
  if (units <= 32)
    spmm_segments_kernel<1, VW><<<grid, 256, 0, st>>>(rowptr, col, val, F, H, ldH, hdr, long_rows, seg_off, scratch, ldS, cap);
  else if (units <= 64)
    spmm_segments_kernel<2, VW><<<grid, 256, 0, st>>>(rowptr, col, val, F, H, ldH, hdr, long_rows, seg_off, scratch, ldS, cap);
  else
    spmm_segments_kernel<4, VW><<<grid, 256, 0, st>>>(rowptr, col, val, F, H, ldH, hdr, long_rows, seg_off, scratch, ldS, cap);
}

inline int64_t scratch_ld(int64_t F) { return (F + 3) & ~int64_t(3); }

}  // namespace

extern "C" {

size_t gc_spmm_plan_bytes(int64_t M) {
  if (M < 0) return 0;
  return plan_seg_off_offset(M) + ((size_t(M + 1) * 4 + 15) & ~size_t(15));
}

int gc_spmm_plan_build(const int32_t* rowptr, int64_t M, void* plan, size_t plan_bytes, void* stream) {
  GC_REQUIRE(rowptr && plan, "gc_spmm_plan_build: null pointer");
  GC_REQUIRE(M >= 0 && M < INT32_MAX, "gc_spmm_plan_build: M=%lld out of int32 range", (long long)M);
  GC_REQUIRE(gc::aligned16(plan), "gc_spmm_plan_build: plan must be 16-byte aligned");
  if (plan_bytes < gc_spmm_plan_bytes(M)) return gc::fail(GC_ERR_WORKSPACE, "gc_spmm_plan_build: plan buffer too small");
  cudaStream_t st = gc::as_stream(stream);
  auto* hdr = reinterpret_cast<PlanHeader*>(plan);
  auto* long_rows = reinterpret_cast<int32_t*>(static_cast<char*>(plan) + plan_long_rows_offset());
  auto* seg_off = reinterpret_cast<int32_t*>(static_cast<char*>(plan) + plan_seg_off_offset(M));
  if (M > 0) plan_collect_kernel<<<unsigned((M + 255) / 256), 256, 0, st>>>(rowptr, int(M), hdr, seg_off);
  plan_scan_kernel<<<1, 1024, 0, st>>>(rowptr, int(M), hdr, long_rows, seg_off);
  return gc::check_launch("gc_spmm_plan_build", M > 0 ? 2 : 1);
}

size_t gc_spmm_scratch_bytes(int64_t nnz, int64_t F) {
  if (nnz < 0 || F <= 0) return 0;
  // every segment belongs to a row with more than GC_SPMM_LONG_ROW entries and
  // ceil(d / SEGMENT) <= d / LONG_ROW for d > LONG_ROW (SEGMENT = 2 * LONG_ROW)
  return size_t(nnz / GC_SPMM_LONG_ROW + 1) * size_t(scratch_ld(F)) * sizeof(float);
}

int gc_spmm_csr_f32(const int32_t* rowptr, const int32_t* col, const float* val, int64_t M, int64_t K, int64_t F,
                    const float* H, int64_t ldH, const float* bias, int epilogue, float* Y, int64_t ldY,
                    float* mask, const void* plan, void* scratch, size_t scratch_bytes, void* stream) {
  GC_REQUIRE(M >= 0 && K >= 0 && F >= 0, "gc_spmm_csr_f32: negative size");
  GC_REQUIRE(M < INT32_MAX && K < INT32_MAX && F < INT32_MAX, "gc_spmm_csr_f32: size out of int32 range");
  if (M == 0 || F == 0) return GC_OK;
  GC_REQUIRE(rowptr && Y, "gc_spmm_csr_f32: null rowptr/Y");
  GC_REQUIRE(ldY >= F && (K == 0 || ldH >= F), "gc_spmm_csr_f32: leading dimension smaller than F");
  GC_REQUIRE(K == 0 || H, "gc_spmm_csr_f32: null H");
  GC_REQUIRE((epilogue & ~(GC_EPI_RELU | GC_EPI_ACCUMULATE)) == 0, "gc_spmm_csr_f32: unknown epilogue bits");
  cudaStream_t st = gc::as_stream(stream);
  Epilogue ep{bias, mask, (epilogue & GC_EPI_RELU) ? 1 : 0, (epilogue & GC_EPI_ACCUMULATE) ? 1 : 0};

  const bool vec4 = (F % 4 == 0) && (ldH % 4 == 0) && (ldY % 4 == 0) && gc::aligned16(H) && gc::aligned16(Y) &&
                    (!bias || gc::aligned16(bias)) && (!mask || gc::aligned16(mask));
  const int skip_long = plan ? 1 : 0;
  if (plan) {
    GC_REQUIRE(gc::aligned16(plan), "gc_spmm_csr_f32: plan must be 16-byte aligned");
    if (!scratch) return gc::fail(GC_ERR_WORKSPACE, "gc_spmm_csr_f32: plan given but scratch is null");
    GC_REQUIRE(gc::aligned16(scratch), "gc_spmm_csr_f32: scratch must be 16-byte aligned");
  }
  if (vec4)
    dispatch_rows<4>(rowptr, col, val, int(M), int(F), H, ldH, Y, ldY, ep, skip_long, st);
  else
    dispatch_rows<1>(rowptr, col, val, int(M), int(F), H, ldH, Y, ldY, ep, skip_long, st);
  int rc = gc::check_launch("gc_spmm_csr_f32 (rows)");
  if (rc != GC_OK) return rc;

  if (plan) {
    const auto* hdr = reinterpret_cast<const PlanHeader*>(plan);
    const auto* long_rows = reinterpret_cast<const int32_t*>(static_cast<const char*>(plan) + plan_long_rows_offset());
    const auto* seg_off = reinterpret_cast<const int32_t*>(static_cast<const char*>(plan) + plan_seg_off_offset(M));
    const int64_t ldS = scratch_ld(F);
    // The segment count lives on the device; the scratch must hold the bound
    // gc_spmm_scratch_bytes() gives for this structure's nnz, which the caller
    // knows.  A scratch smaller than one segment row is certainly wrong.
    if (scratch_bytes < size_t(ldS) * sizeof(float))
      return gc::fail(GC_ERR_WORKSPACE, "gc_spmm_csr_f32: scratch too small");
    float* sc = static_cast<float*>(scratch);
    const size_t cap_rows = scratch_bytes / (size_t(ldS) * sizeof(float));
    const int cap = cap_rows > size_t(INT32_MAX) ? INT32_MAX : int(cap_rows);
    if (vec4)
      dispatch_segments<4>(rowptr, col, val, int(F), H, ldH, hdr, long_rows, seg_off, sc, ldS, cap, st);
    else
      dispatch_segments<1>(rowptr, col, val, int(F), H, ldH, hdr, long_rows, seg_off, sc, ldS, cap, st);
    rc = gc::check_launch("gc_spmm_csr_f32 (segments)");
    if (rc != GC_OK) return rc;
    spmm_finalize_kernel<<<gc::kNumSMs * 2, 256, 0, st>>>(int(F), hdr, long_rows, seg_off, sc, ldS, Y, ldY, ep);
    rc = gc::check_launch("gc_spmm_csr_f32 (finalize)");
  }
  return rc;
}

// ---------------------------------------------------------------- no-allocation variant
// Scratch for gc_spmm_csr_f32_noalloc: part of the library image, so every
// GPU that loads the library carries these bytes until the process exits.
#define GC_SPMM_STATIC_SCRATCH_FLOATS (size_t(GC_SPMM_STATIC_SCRATCH_BYTES) / sizeof(float))
static __device__ __align__(256) float g_static_scratch[GC_SPMM_STATIC_SCRATCH_FLOATS];

namespace {
constexpr int kMaxDevices = 64;
std::mutex g_static_mutex;
float* g_static_ptr[kMaxDevices] = {nullptr};

// Device address of g_static_scratch on the CURRENT device.  In host code the
// symbol's name is only a handle for the runtime, not a device address, so it
// is translated with cudaGetSymbolAddress -- once per device, with that device
// current -- and the translated pointer is what the kernels receive.
int static_scratch_for_current_device(float** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return gc::fail(GC_ERR_CUDA, "cudaGetDevice: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices) return gc::fail(GC_ERR_UNSUPPORTED, "device ordinal %d not supported", dev);
  std::lock_guard<std::mutex> lock(g_static_mutex);
  if (!g_static_ptr[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess || !p)
      return gc::fail(GC_ERR_CUDA, "cudaGetSymbolAddress(static scratch): %s", cudaGetErrorString(e));
    g_static_ptr[dev] = static_cast<float*>(p);
  }
  *out = g_static_ptr[dev];
  return GC_OK;
}
}  // namespace

int gc_spmm_csr_f32_noalloc(const int32_t* rowptr, const int32_t* col, const float* val, int64_t M, int64_t K,
                            int64_t F, int64_t nnz, const float* H, int64_t ldH, const float* bias, int epilogue,
                            float* Y, int64_t ldY, float* mask, const void* plan, void* stream) {
  GC_REQUIRE(nnz >= 0, "gc_spmm_csr_f32_noalloc: negative nnz");
  if (!plan)  // no long-row segments, hence no scratch at all
    return gc_spmm_csr_f32(rowptr, col, val, M, K, F, H, ldH, bias, epilogue, Y, ldY, mask, nullptr, nullptr, 0,
                           stream);
  const size_t need = gc_spmm_scratch_bytes(nnz, F);
  if (need > size_t(GC_SPMM_STATIC_SCRATCH_BYTES))
    return gc::fail(GC_ERR_WORKSPACE,
                    "gc_spmm_csr_f32_noalloc: nnz=%lld, F=%lld needs up to %zu bytes of scratch, the built-in "
                    "buffer holds %zu; use gc_spmm_csr_f32 with caller-provided scratch",
                    (long long)nnz, (long long)F, need, size_t(GC_SPMM_STATIC_SCRATCH_BYTES));
  float* scratch = nullptr;
  const int rc = static_scratch_for_current_device(&scratch);
  if (rc != GC_OK) return rc;
  // Every partial-sum row the finalize pass reads is fully written by the
  // segment pass of the same call, so stale contents of the shared buffer are
  // never observed and nothing has to be cleared.
  return gc_spmm_csr_f32(rowptr, col, val, M, K, F, H, ldH, bias, epilogue, Y, ldY, mask, plan, scratch,
                         size_t(GC_SPMM_STATIC_SCRATCH_BYTES), stream);
}

}  // extern "C"

// CSR (int32) x dense fp32 aggregation  Y = A * H (+bias)(ReLU)(mask).
//
// Takes over the reference's cuSPARSE COO SpMM wrapper
// (src/graphcuda/cuda/spmm_cusparse.cu:3-126) on the GCN path
// (src/graphcuda/cuda/gcn.cu:12,40,49).
//
// The product is a gather: every non-zero (i, j) reads row j of H.  On
// power-law graphs most of that traffic is not compulsory -- H is far larger
// than the 126 MB L2 and the heavy rows pull in rows of H from everywhere.
// The schedule therefore works on "pieces" (a contiguous run of non-zeros of
// one row) listed by a plan that is built once per CSR structure:
//   * rows with more than GC_SPMM_PANEL_MIN_ROW non-zeros are cut at column
//     panel boundaries (panel = a range of columns whose rows of H fit the
//     L2 together); pieces are processed panel by panel, so the whole GPU
//     gathers from one L2-resident slab of H at a time;
//   * any piece longer than the plan's segment length (128..2048 non-zeros,
//     growing with the size of the matrix) is cut further, so a hub row is
//     spread over many warps and no single piece dominates the launch;
//   * pieces of cut rows write partial sums to scratch; a finalize pass adds
//     a row's partials in piece order and applies the epilogue -- no atomics
//     anywhere, results are bit-reproducible run to run;
//   * uncut rows are processed after the panels, longest first, and write Y
//     directly with the fused epilogue;
//   * within a phase pieces are sorted by length, so the sub-warp groups of a
//     warp carry similar work.
// A piece is handled by a group of GROUP lanes (2..32): the lanes fetch GROUP
// (col, val) pairs with one coalesced load (the next batch is prefetched),
// broadcast them with shuffles and gather the H rows with 128-bit loads,
// U non-zeros x NACC vectors in flight per lane.
// Bias, ReLU (as y * (y > 0), the reference's formula, gcn.cu:19-20), the fp32
// mask and an optional accumulate are fused into the store.
#include "common.cuh"

#include <algorithm>
#include <cub/device/device_radix_sort.cuh>
#include <cub/device/device_scan.cuh>
#include <mutex>

namespace {

struct PlanHeader {
  int32_t magic;
  int32_t M;
  int32_t n_pieces;  // entries of the piece list
  int32_t n_slots;   // partial-sum rows in scratch (pieces of cut rows)
  int32_t n_cut;     // rows that were cut
  int32_t panel_cols;
  int32_t overflow;  // sticky: a launch found less scratch than the plan's partial sums need and skipped some
  int32_t pad;
};
constexpr int32_t kPlanMagic = 0x47435032;  // "GCP2"

inline size_t align16(size_t x) { return (x + 15) & ~size_t(15); }

// Plan memory: header | piece_start[n] | piece_len[n] | piece_target[n] |
//              cut_row[c] | cut_slot0[c] | cut_nslots[c]
struct PlanView {
  PlanHeader* hdr;
  int32_t *start, *len, *target, *cut_row, *cut_slot0, *cut_nslots;
};
inline PlanView plan_view(void* plan, int64_t n_pieces, int64_t n_cut) {
  char* p = static_cast<char*>(plan);
  PlanView v;
  v.hdr = reinterpret_cast<PlanHeader*>(p);
  size_t off = sizeof(PlanHeader);
  const size_t np = align16(size_t(n_pieces) * 4), nc = align16(size_t(n_cut) * 4);
  v.start = reinterpret_cast<int32_t*>(p + off); off += np;
  v.len = reinterpret_cast<int32_t*>(p + off); off += np;
  v.target = reinterpret_cast<int32_t*>(p + off); off += np;
  v.cut_row = reinterpret_cast<int32_t*>(p + off); off += nc;
  v.cut_slot0 = reinterpret_cast<int32_t*>(p + off); off += nc;
  v.cut_nslots = reinterpret_cast<int32_t*>(p + off);
  return v;
}

// ---------------------------------------------------------------- epilogue
struct Epilogue {
  const float* bias;
  float* mask;
  const float* gate;  // same shape / leading dimension as Y, or null: Y *= (gate > 0) after everything else
  int relu;
  int accumulate;
};

// Output rows may be spread over several matrices of the same leading
// dimension: row i lives in base[i / block_rows] at row i % block_rows.  That
// is how a rank of the feature-sharded multi-GPU scheme stores its slab of the
// product straight into every owner's buffer (peer-mapped memory, ordinary
// stores): the aggregation's epilogue is the exchange.  block_rows == 0: one
// matrix, the Y argument.
struct RowBlocks {
  float* base[GC_SPMM_MAX_BLOCKS];
  int block_rows;
};

__device__ __forceinline__ float* out_row(const RowBlocks& rb, float* Y, int64_t ldY, int row) {
  if (rb.block_rows == 0) return Y + int64_t(row) * ldY;
  const int q = row / rb.block_rows;
  return rb.base[q] + int64_t(row - q * rb.block_rows) * ldY;
}

template <int VW>
struct Vec;
template <>
struct Vec<4> {
  using T = float4;   // accumulator / output vector
  using HT = float;   // element type of H
  using G = float4;   // one gathered vector of H
  static __device__ __forceinline__ T zero() { return make_float4(0.f, 0.f, 0.f, 0.f); }
  static __device__ __forceinline__ G gzero() { return make_float4(0.f, 0.f, 0.f, 0.f); }
  static __device__ __forceinline__ G gather(const HT* p) { return __ldg(reinterpret_cast<const float4*>(p)); }
  static __device__ __forceinline__ T load(const float* p) { return __ldg(reinterpret_cast<const float4*>(p)); }
  static __device__ __forceinline__ T load_plain(const float* p) { return *reinterpret_cast<const float4*>(p); }
  static __device__ __forceinline__ T load_stream(const float* p) { return __ldcs(reinterpret_cast<const float4*>(p)); }
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
  using HT = float;
  using G = float;
  static __device__ __forceinline__ T zero() { return 0.f; }
  static __device__ __forceinline__ G gzero() { return 0.f; }
  static __device__ __forceinline__ G gather(const HT* p) { return __ldg(p); }
  static __device__ __forceinline__ T load(const float* p) { return __ldg(p); }
  static __device__ __forceinline__ T load_plain(const float* p) { return *p; }
  static __device__ __forceinline__ T load_stream(const float* p) { return __ldcs(p); }
  static __device__ __forceinline__ void store(float* p, T v) { *p = v; }
  static __device__ __forceinline__ void fma(T& a, float s, const T& h) { a = fmaf(s, h, a); }
  static __device__ __forceinline__ T add(const T& a, const T& b) { return a + b; }
  static __device__ __forceinline__ T gt0(const T& a) { return a > 0.f ? 1.f : 0.f; }
  static __device__ __forceinline__ T mul(const T& a, const T& b) { return a * b; }
};

// H held in bf16 (the reduced-precision tier): a lane gathers 8 elements (16 bytes) at a time and accumulates
// them in fp32; everything on the output side stays fp32.  Element 2i sits in the low half of word i.
struct Float8 {
  float4 a, b;
};
template <>
struct Vec<8> {
  using T = Float8;
  using HT = uint16_t;
  using G = uint4;
  using V4 = Vec<4>;
  static __device__ __forceinline__ T zero() { return Float8{V4::zero(), V4::zero()}; }
  static __device__ __forceinline__ G gzero() { return make_uint4(0u, 0u, 0u, 0u); }
  static __device__ __forceinline__ G gather(const HT* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }
  static __device__ __forceinline__ T load(const float* p) { return Float8{V4::load(p), V4::load(p + 4)}; }
  static __device__ __forceinline__ T load_plain(const float* p) { return Float8{V4::load_plain(p), V4::load_plain(p + 4)}; }
  static __device__ __forceinline__ T load_stream(const float* p) { return Float8{V4::load_stream(p), V4::load_stream(p + 4)}; }
  static __device__ __forceinline__ void store(float* p, const T& v) {
    V4::store(p, v.a);
    V4::store(p + 4, v.b);
  }
  static __device__ __forceinline__ float lo(uint32_t u) { return __uint_as_float(u << 16); }
  static __device__ __forceinline__ float hi(uint32_t u) { return __uint_as_float(u & 0xFFFF0000u); }
  // (c0, c1) += s * (low half, high half of u) as ONE packed fp32 FMA (fma.rn.f32x2: same rounding as two fmaf).
  // The unpacking costs two integer operations per word; with scalar FMAs on top the bf16 kernel issued 1.7 times
  // the instructions of the fp32 one for half the bytes and gained nothing at F = 256.
  static __device__ __forceinline__ void fma2(float& c0, float& c1, unsigned long long ss, uint32_t u) {
    unsigned long long c, h, r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(c) : "f"(c0), "f"(c1));
    asm("mov.b64 %0, {%1, %2};" : "=l"(h) : "r"(u << 16), "r"(u & 0xFFFF0000u));
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(ss), "l"(h), "l"(c));
    asm("mov.b64 {%0, %1}, %2;" : "=f"(c0), "=f"(c1) : "l"(r));
  }
  static __device__ __forceinline__ void fma(T& acc, float s, const G& h) {
    unsigned long long ss;
    asm("mov.b64 %0, {%1, %1};" : "=l"(ss) : "f"(s));
    fma2(acc.a.x, acc.a.y, ss, h.x);
    fma2(acc.a.z, acc.a.w, ss, h.y);
    fma2(acc.b.x, acc.b.y, ss, h.z);
    fma2(acc.b.z, acc.b.w, ss, h.w);
  }
  static __device__ __forceinline__ T add(const T& x, const T& y) { return Float8{V4::add(x.a, y.a), V4::add(x.b, y.b)}; }
  static __device__ __forceinline__ T gt0(const T& x) { return Float8{V4::gt0(x.a), V4::gt0(x.b)}; }
  static __device__ __forceinline__ T mul(const T& x, const T& y) { return Float8{V4::mul(x.a, y.a), V4::mul(x.b, y.b)}; }
};

// Applies accumulate / bias / mask / ReLU to one vector and stores it.
template <int VW>
__device__ __forceinline__ void finish_store(typename Vec<VW>::T acc, float* yrow, float* mrow, int f,
                                             const Epilogue& ep, const float* grow = nullptr) {
  using V = Vec<VW>;
  if (ep.accumulate) acc = V::add(acc, V::load_plain(yrow + f));
  if (ep.bias) acc = V::add(acc, V::load(ep.bias + f));
  if (ep.relu || mrow) {
    typename V::T m = V::gt0(acc);
    if (mrow) V::store(mrow + f, m);
    if (ep.relu) acc = V::mul(acc, m);
  }
  if (grow) acc = V::mul(acc, V::gt0(V::load_stream(grow + f)));  // read once: keep it out of the caches
  V::store(yrow + f, acc);
}

// ---------------------------------------------------------------- piece kernel
// One group of GROUP lanes per piece; NACC vectors of VW floats per lane cover
// GROUP*NACC*VW feature columns per pass; wider F loops over passes.
// PLANNED: pieces come from the plan (target >= 0: row of Y with the
// epilogue; target < 0: scratch row ~target, raw sums); otherwise piece v is
// row v of the matrix.
// MIN_CTAS (resident CTAs per SM the register allocation must allow) is part
// of the tuning: left to itself the compiler settles near 78 registers and
// serialises the gathers; told its budget (80 registers at 3 CTAs, 128 at 2)
// it keeps a whole round of U x NACC loads in flight.  Measured on the
// 126 M-non-zero graph, F = 256: 12.6 ms unconstrained, 8.7 ms at 2, 8.4 ms
// at 3; F = 100: 6.3 / 4.4 / 4.4 ms.
template <int GROUP, int NACC, int VW, int U, bool PLANNED, int MIN_CTAS>
__global__ void __launch_bounds__(256, MIN_CTAS)
spmm_pieces_kernel(const int32_t* __restrict__ rowptr, const int32_t* __restrict__ col,
                   const float* __restrict__ val, int n_pieces, const int32_t* __restrict__ p_start,
                   const int32_t* __restrict__ p_len, const int32_t* __restrict__ p_target, int F,
                   const typename Vec<VW>::HT* __restrict__ H, int64_t ldH, float* __restrict__ Y, int64_t ldY,
                   float* __restrict__ scratch, int64_t ldS, int slot_capacity, int32_t* __restrict__ overflow,
                   Epilogue ep, const __grid_constant__ RowBlocks rb) {
  using V = Vec<VW>;
  constexpr int PIECES_PER_CTA = 256 / GROUP;
  constexpr int PASS = GROUP * NACC * VW;
  static_assert(U <= GROUP, "a round cannot be wider than a batch");
  const int lane_g = threadIdx.x % GROUP;
  const int v = blockIdx.x * PIECES_PER_CTA + threadIdx.x / GROUP;
  if (v >= n_pieces) return;
  const unsigned gmask = (GROUP == 32) ? 0xffffffffu
                                       : (((1u << GROUP) - 1u) << ((threadIdx.x % 32) / GROUP * GROUP));
  int start, end, target;
  if (PLANNED) {
    start = __ldg(p_start + v);
    end = start + __ldg(p_len + v);
    target = __ldg(p_target + v);
  } else {
    start = __ldg(rowptr + v);
    end = __ldg(rowptr + v + 1);
    target = v;
  }
  const bool direct = target >= 0;
  if (!direct && (~target) >= slot_capacity) {  // never write past the caller's scratch; leave a trace instead
    if (lane_g == 0) *overflow = 1;
    return;
  }
  float* yrow = direct ? out_row(rb, Y, ldY, target) : scratch + int64_t(~target) * ldS;
  float* mrow = (direct && ep.mask) ? ep.mask + int64_t(target) * ldY : nullptr;
  const float* grow = (direct && ep.gate) ? ep.gate + int64_t(target) * ldY : nullptr;
  Epilogue my_ep = ep;
  if (!direct) my_ep = Epilogue{nullptr, nullptr, nullptr, 0, 0};

  // Feature columns beyond one pass are walked in turn -- or, when the matrix has too few pieces to fill the
  // GPU (a Cora-sized graph with a 1433-wide H), spread over gridDim.y so that the passes run side by side.
  for (int f0 = blockIdx.y * PASS; f0 < F; f0 += gridDim.y * PASS) {
    typename V::T acc[NACC];
    bool live[NACC];
#pragma unroll
    for (int a = 0; a < NACC; ++a) {
      acc[a] = V::zero();
      live[a] = (f0 + (a * GROUP + lane_g) * VW) < F;
    }
    int c_next = 0;
    float w_next = 0.f;
    if (start + lane_g < end) {
      c_next = __ldg(col + start + lane_g);
      w_next = __ldg(val + start + lane_g);
    }
    for (int base = start; base < end; base += GROUP) {
      const int c = c_next;
      const float w = w_next;
      const int e2 = base + GROUP + lane_g;  // prefetch the next batch of (col, val)
      if (e2 < end) {
        c_next = __ldg(col + e2);
        w_next = __ldg(val + e2);
      }
      const int cnt = min(GROUP, end - base);
      // U gathers in flight per lane and accumulator; entries past the end of
      // the piece are never loaded (a 0 * Inf would poison the sum).
      for (int j = 0; j < cnt; j += U) {
        int cj[U];
        float wj[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          cj[u] = __shfl_sync(gmask, c, (j + u) % GROUP, GROUP);
          wj[u] = __shfl_sync(gmask, w, (j + u) % GROUP, GROUP);
        }
        typename V::G h[U][NACC];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const typename V::HT* hp = H + int64_t(cj[u]) * ldH + f0;
          const bool valid = (j + u) < cnt;
#pragma unroll
          for (int a = 0; a < NACC; ++a)
            h[u][a] = (live[a] && valid) ? V::gather(hp + (a * GROUP + lane_g) * VW) : V::gzero();
        }
#pragma unroll
        for (int u = 0; u < U; ++u)
#pragma unroll
          for (int a = 0; a < NACC; ++a) V::fma(acc[a], (j + u) < cnt ? wj[u] : 0.f, h[u][a]);
      }
    }
#pragma unroll
    for (int a = 0; a < NACC; ++a)
      if (live[a]) finish_store<VW>(acc[a], yrow, mrow, f0 + (a * GROUP + lane_g) * VW, my_ep, grow);
  }
}

// Very narrow feature widths (F <= 8): the lanes of a group walk the NON-ZEROS of a
// piece instead of its feature columns.  Each lane gathers whole (short) rows
// of H for its own entries -- U entries in flight -- and keeps a private sum;
// the 8 lanes' sums are combined by a butterfly of shuffles in a fixed order.
// With 16..32-byte rows this keeps several times as many gathers in flight per
// warp as the column-parallel mapping and needs no (col, val) broadcast.
template <int NV, int U, bool PLANNED>
__global__ void __launch_bounds__(256)
spmm_pieces_narrow_kernel(const int32_t* __restrict__ rowptr, const int32_t* __restrict__ col,
                          const float* __restrict__ val, int n_pieces, const int32_t* __restrict__ p_start,
                          const int32_t* __restrict__ p_len, const int32_t* __restrict__ p_target, int F,
                          const float* __restrict__ H, int64_t ldH, float* __restrict__ Y, int64_t ldY,
                          float* __restrict__ scratch, int64_t ldS, int slot_capacity,
                          int32_t* __restrict__ overflow, Epilogue ep, const __grid_constant__ RowBlocks rb) {
  constexpr int G = 8;
  const int lane_g = threadIdx.x % G;
  const int v = blockIdx.x * (256 / G) + threadIdx.x / G;
  if (v >= n_pieces) return;
  const unsigned gmask = 0xFFu << ((threadIdx.x % 32) / G * G);
  int start, end, target;
  if (PLANNED) {
    start = __ldg(p_start + v);
    end = start + __ldg(p_len + v);
    target = __ldg(p_target + v);
  } else {
    start = __ldg(rowptr + v);
    end = __ldg(rowptr + v + 1);
    target = v;
  }
  const bool direct = target >= 0;
  if (!direct && (~target) >= slot_capacity) {
    if (lane_g == 0) *overflow = 1;
    return;
  }
  const int units = F / 4;
  float4 acc[NV];
#pragma unroll
  for (int a = 0; a < NV; ++a) acc[a] = make_float4(0.f, 0.f, 0.f, 0.f);
  // lane l takes entries start + l, start + l + G, ...; U of them per round
  for (int base = start + lane_g; base < end; base += G * U) {
    int c[U];
    float w[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int e = base + u * G;
      const bool ok = e < end;
      c[u] = ok ? __ldg(col + e) : -1;
      w[u] = ok ? __ldg(val + e) : 0.f;
    }
    float4 h[U][NV];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const float4* hp = reinterpret_cast<const float4*>(H + int64_t(c[u] < 0 ? 0 : c[u]) * ldH);
#pragma unroll
      for (int a = 0; a < NV; ++a)
        h[u][a] = (c[u] >= 0 && a < units) ? __ldg(hp + a) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int u = 0; u < U; ++u)
#pragma unroll
      for (int a = 0; a < NV; ++a) Vec<4>::fma(acc[a], w[u], h[u][a]);
  }
  // butterfly over the 8 lanes: every lane ends with the total, added in a fixed order
#pragma unroll
  for (int o = 1; o < G; o <<= 1) {
#pragma unroll
    for (int a = 0; a < NV; ++a) {
      acc[a].x += __shfl_xor_sync(gmask, acc[a].x, o, G);
      acc[a].y += __shfl_xor_sync(gmask, acc[a].y, o, G);
      acc[a].z += __shfl_xor_sync(gmask, acc[a].z, o, G);
      acc[a].w += __shfl_xor_sync(gmask, acc[a].w, o, G);
    }
  }
  float* yrow = direct ? out_row(rb, Y, ldY, target) : scratch + int64_t(~target) * ldS;
  float* mrow = (direct && ep.mask) ? ep.mask + int64_t(target) * ldY : nullptr;
  const float* grow = (direct && ep.gate) ? ep.gate + int64_t(target) * ldY : nullptr;
  Epilogue my_ep = ep;
  if (!direct) my_ep = Epilogue{nullptr, nullptr, nullptr, 0, 0};
  // lane a stores vector a
#pragma unroll
  for (int a = 0; a < NV; ++a)
    if (lane_g == a && a < units) finish_store<4>(acc[a], yrow, mrow, a * 4, my_ep, grow);
}

// One warp per cut row: adds that row's partial sums in slot order, then the
// fused store.  Lanes cover the feature columns (128-bit vectors when the rows
// are aligned); four slots are loaded ahead of the ordered additions.
template <int VW>
__global__ void __launch_bounds__(256)
spmm_finalize_kernel(int F, int n_cut, const int32_t* __restrict__ cut_row, const int32_t* __restrict__ cut_slot0,
                     const int32_t* __restrict__ cut_nslots, const float* __restrict__ scratch, int64_t ldS,
                     int slot_capacity, int32_t* __restrict__ overflow, float* __restrict__ Y, int64_t ldY,
                     Epilogue ep, const __grid_constant__ RowBlocks rb) {
  using V = Vec<VW>;
  const int lane = threadIdx.x % 32;
  const int warps = gridDim.x * 8;
  for (int i = blockIdx.x * 8 + threadIdx.x / 32; i < n_cut; i += warps) {
    const int row = __ldg(cut_row + i);
    const int s0 = __ldg(cut_slot0 + i);
    const int s_end = s0 + __ldg(cut_nslots + i);
    const int s1 = min(s_end, slot_capacity);
    if (s_end > slot_capacity && lane == 0) *overflow = 1;
    float* yrow = out_row(rb, Y, ldY, row);
    float* mrow = ep.mask ? ep.mask + int64_t(row) * ldY : nullptr;
    const float* grow = ep.gate ? ep.gate + int64_t(row) * ldY : nullptr;
    for (int f = lane * VW; f < F; f += 32 * VW) {
      typename V::T s = V::zero();
      int sl = s0;
      for (; sl + 4 <= s1; sl += 4) {
        const float* p = scratch + int64_t(sl) * ldS + f;
        const typename V::T a = V::load_plain(p), b = V::load_plain(p + ldS), c = V::load_plain(p + 2 * ldS),
                            d = V::load_plain(p + 3 * ldS);
        s = V::add(V::add(V::add(V::add(s, a), b), c), d);
      }
      for (; sl < s1; ++sl) s = V::add(s, V::load_plain(scratch + int64_t(sl) * ldS + f));
      finish_store<VW>(s, yrow, mrow, f, ep, grow);
    }
  }
}

// ---------------------------------------------------------------- plan construction
__device__ __forceinline__ int lower_bound_col(const int32_t* __restrict__ col, int lo, int hi, int key) {
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if (__ldg(col + mid) < key) lo = mid + 1; else hi = mid;
  }
  return lo;
}

__device__ __forceinline__ int pieces_of(int cnt, int seg) { return (cnt + seg - 1) / seg; }

// Per row: how many pieces it contributes and whether it is cut.
__global__ void __launch_bounds__(256)
plan_count_kernel(const int32_t* __restrict__ rowptr, const int32_t* __restrict__ col, int M, int K, int panel_cols,
                  int seg, int32_t* __restrict__ rows_pieces, int32_t* __restrict__ rows_cut,
                  int32_t* __restrict__ rows_slots) {
  const int r = blockIdx.x * 256 + threadIdx.x;
  if (r >= M) return;
  const int s = __ldg(rowptr + r), e = __ldg(rowptr + r + 1), d = e - s;
  const int n_panels = (K + panel_cols - 1) / panel_cols;
  int pieces;
  if (d > GC_SPMM_PANEL_MIN_ROW && n_panels > 1) {
    pieces = 0;
    int lo = s;
    for (int p = 0; p < n_panels && lo < e; ++p) {
      const int hi = (p + 1 == n_panels) ? e : lower_bound_col(col, lo, e, (p + 1) * panel_cols);
      pieces += pieces_of(hi - lo, seg);
      lo = hi;
    }
  } else {
    pieces = max(1, pieces_of(d, seg));
  }
  rows_pieces[r] = pieces;
  rows_cut[r] = pieces > 1 ? 1 : 0;
  rows_slots[r] = pieces > 1 ? pieces : 0;
}

__global__ void plan_totals_kernel(const int32_t* __restrict__ rows_pieces, const int32_t* __restrict__ rows_cut,
                                   const int32_t* __restrict__ rows_slots, const int32_t* __restrict__ piece_base,
                                   const int32_t* __restrict__ cut_base, const int32_t* __restrict__ slot_base,
                                   int M, int64_t* __restrict__ counts) {
  if (M == 0) { counts[0] = counts[1] = counts[2] = 0; return; }
  const int l = M - 1;
  counts[0] = int64_t(piece_base[l]) + rows_pieces[l];  // pieces
  counts[1] = int64_t(slot_base[l]) + rows_slots[l];    // scratch slots
  counts[2] = int64_t(cut_base[l]) + rows_cut[l];       // cut rows
}

// Emits the pieces of every row with a sort key (phase << 32 | ~length):
// phase = panel index for pieces of panel-cut rows, 0 for rows cut by length
// only, n_panels for uncut rows (they run after all panels).
__global__ void __launch_bounds__(256)
plan_emit_kernel(const int32_t* __restrict__ rowptr, const int32_t* __restrict__ col, int M, int K, int panel_cols,
                 int seg, const int32_t* __restrict__ rows_cut, const int32_t* __restrict__ piece_base,
                 const int32_t* __restrict__ cut_base, const int32_t* __restrict__ slot_base,
                 const int32_t* __restrict__ rows_pieces, uint64_t* __restrict__ keys, int32_t* __restrict__ ids,
                 int32_t* __restrict__ u_start, int32_t* __restrict__ u_len, int32_t* __restrict__ u_target,
                 int32_t* __restrict__ cut_row, int32_t* __restrict__ cut_slot0, int32_t* __restrict__ cut_nslots) {
  const int r = blockIdx.x * 256 + threadIdx.x;
  if (r >= M) return;
  const int s = __ldg(rowptr + r), e = __ldg(rowptr + r + 1), d = e - s;
  const int n_panels = (K + panel_cols - 1) / panel_cols;
  int out = piece_base[r];
  if (!rows_cut[r]) {
    u_start[out] = s;
    u_len[out] = d;
    u_target[out] = r;
    keys[out] = (uint64_t(uint32_t(n_panels)) << 32) | uint64_t(0xFFFFFFFFu - uint32_t(d));
    ids[out] = out;
    return;
  }
  int slot = slot_base[r];
  const int ci = cut_base[r];
  cut_row[ci] = r;
  cut_slot0[ci] = slot;
  cut_nslots[ci] = rows_pieces[r];
  const bool by_panel = d > GC_SPMM_PANEL_MIN_ROW && n_panels > 1;
  int lo = s;
  for (int p = 0; p < (by_panel ? n_panels : 1) && lo < e; ++p) {
    const int hi = (!by_panel || p + 1 == n_panels) ? e : lower_bound_col(col, lo, e, (p + 1) * panel_cols);
    for (int q = lo; q < hi; q += seg) {
      const int len = min(seg, hi - q);
      u_start[out] = q;
      u_len[out] = len;
      u_target[out] = ~slot;
      keys[out] = (uint64_t(uint32_t(by_panel ? p : 0)) << 32) | uint64_t(0xFFFFFFFFu - uint32_t(len));
      ids[out] = out;
      ++out;
      ++slot;
    }
    lo = hi;
  }
}

__global__ void __launch_bounds__(256)
plan_gather_kernel(const int32_t* __restrict__ ids_sorted, int n, const int32_t* __restrict__ u_start,
                   const int32_t* __restrict__ u_len, const int32_t* __restrict__ u_target,
                   int32_t* __restrict__ start, int32_t* __restrict__ len, int32_t* __restrict__ target) {
  const int i = blockIdx.x * 256 + threadIdx.x;
  if (i >= n) return;
  const int j = ids_sorted[i];
  start[i] = u_start[j];
  len[i] = u_len[j];
  target[i] = u_target[j];
}

__global__ void plan_header_kernel(PlanHeader* hdr, int M, int n_pieces, int n_slots, int n_cut, int panel_cols) {
  hdr->magic = kPlanMagic;
  hdr->M = M;
  hdr->n_pieces = n_pieces;
  hdr->n_slots = n_slots;
  hdr->n_cut = n_cut;
  hdr->panel_cols = panel_cols;
  hdr->overflow = 0;
  hdr->pad = 0;
}

// Workspace carve-up shared by the count and build steps.
struct PlanWs {
  int32_t *rows_pieces, *rows_cut, *rows_slots, *piece_base, *cut_base, *slot_base;
  uint64_t *keys, *keys_alt;
  int32_t *ids, *ids_alt, *u_start, *u_len, *u_target;
  void* cub;
  size_t cub_bytes;
  size_t total;
};

// Temporary storage for the CUB scan / sort.  Sized by formula rather than by
// querying CUB, so the answer is the same on a machine without a GPU: the
// one-sweep radix sort and the decoupled look-back scan need a few bytes per
// 1000 items plus fixed histograms.
size_t cub_temp_bytes(int64_t M, int64_t n_pieces) {
  return (size_t(4) << 20) + size_t(std::max<int64_t>(M, n_pieces)) / 4;
}

PlanWs carve(void* ws, int64_t M, int64_t n_pieces) {
  PlanWs w{};
  char* p = static_cast<char*>(ws);
  size_t off = 0;
  auto take = [&](size_t bytes) {
    char* q = p ? p + off : nullptr;
    off += (bytes + 255) & ~size_t(255);
    return q;
  };
  const size_t m4 = size_t(std::max<int64_t>(M, 1)) * 4, n4 = size_t(std::max<int64_t>(n_pieces, 1)) * 4;
  w.rows_pieces = reinterpret_cast<int32_t*>(take(m4));
  w.rows_cut = reinterpret_cast<int32_t*>(take(m4));
  w.rows_slots = reinterpret_cast<int32_t*>(take(m4));
  w.piece_base = reinterpret_cast<int32_t*>(take(m4));
  w.cut_base = reinterpret_cast<int32_t*>(take(m4));
  w.slot_base = reinterpret_cast<int32_t*>(take(m4));
  w.keys = reinterpret_cast<uint64_t*>(take(n4 * 2));
  w.keys_alt = reinterpret_cast<uint64_t*>(take(n4 * 2));
  w.ids = reinterpret_cast<int32_t*>(take(n4));
  w.ids_alt = reinterpret_cast<int32_t*>(take(n4));
  w.u_start = reinterpret_cast<int32_t*>(take(n4));
  w.u_len = reinterpret_cast<int32_t*>(take(n4));
  w.u_target = reinterpret_cast<int32_t*>(take(n4));
  w.cub_bytes = cub_temp_bytes(M, n_pieces);
  w.cub = take(w.cub_bytes);
  w.total = off;
  return w;
}

int exclusive_scan(const PlanWs& w, const int32_t* in, int32_t* out, int n, cudaStream_t st) {
  size_t need = 0;
  cudaError_t e = cub::DeviceScan::ExclusiveSum(nullptr, need, in, out, n, st);
  if (e == cudaSuccess && need > w.cub_bytes)
    return gc::fail(GC_ERR_WORKSPACE, "spmm plan: scan needs %zu bytes of temporary storage, have %zu", need,
                    w.cub_bytes);
  size_t b = w.cub_bytes;
  if (e == cudaSuccess) e = cub::DeviceScan::ExclusiveSum(w.cub, b, in, out, n, st);
  if (e != cudaSuccess) return gc::fail(GC_ERR_CUDA, "spmm plan: scan: %s", cudaGetErrorString(e));
  gc::count_launches(1);
  return GC_OK;
}

int count_rows(const int32_t* rowptr, const int32_t* col, int M, int K, int panel_cols, int seg, const PlanWs& w,
               cudaStream_t st) {
  const unsigned g = unsigned((M + 255) / 256);
  plan_count_kernel<<<g, 256, 0, st>>>(rowptr, col, M, K, panel_cols, seg, w.rows_pieces, w.rows_cut, w.rows_slots);
  int rc = gc::check_launch("spmm plan: count");
  if (rc == GC_OK) rc = exclusive_scan(w, w.rows_pieces, w.piece_base, M, st);
  if (rc == GC_OK) rc = exclusive_scan(w, w.rows_cut, w.cut_base, M, st);
  if (rc == GC_OK) rc = exclusive_scan(w, w.rows_slots, w.slot_base, M, st);
  return rc;
}

// ---------------------------------------------------------------- dispatch
// Two resident CTAs (128 registers) for the 3- and 4-accumulator mappings on groups
// of up to 8 lanes: on a 2.3 M-non-zero graph they run F = 48..128 in
// 0.11-0.13 ms against 0.15-0.22 ms at three; everything else is as fast or
// faster at three (F = 512 on 126 M non-zeros: 17.9 against 20.5 ms).
constexpr int pieces_min_ctas(int group, int nacc, int vw) {
  return ((vw == 4 && nacc >= 3 && group <= 8) || (vw == 8 && nacc >= 2 && group <= 8)) ? 2 : 3;
}

template <int GROUP, int NACC, int VW, int U>
void launch_pieces(bool planned, const int32_t* rowptr, const int32_t* col, const float* val, int n_pieces,
                   const int32_t* ps, const int32_t* pl, const int32_t* pt, int F, const typename Vec<VW>::HT* H,
                   int64_t ldH,
                   float* Y, int64_t ldY, float* scratch, int64_t ldS, int cap, int32_t* ovf, const Epilogue& ep,
                   const RowBlocks& rb, cudaStream_t st) {
  constexpr int PER_CTA = 256 / GROUP;
  const unsigned gx = unsigned((n_pieces + PER_CTA - 1) / PER_CTA);
  const int passes = (F + GROUP * NACC * VW - 1) / (GROUP * NACC * VW);
  // few pieces and several passes: one CTA row per pass (up to about eight CTAs per SM in total)
  const unsigned gy = unsigned(std::max(1, std::min<int>(passes, int(gc::kNumSMs * 8 / std::max(gx, 1u)))));
  const dim3 grid(gx, gy);
  constexpr int MINB = pieces_min_ctas(GROUP, NACC, VW);
  if (planned)
    spmm_pieces_kernel<GROUP, NACC, VW, U, true, MINB>
        <<<grid, 256, 0, st>>>(rowptr, col, val, n_pieces, ps, pl, pt, F, H, ldH, Y, ldY, scratch, ldS, cap, ovf, ep, rb);
  else
    spmm_pieces_kernel<GROUP, NACC, VW, U, false, MINB>
        <<<grid, 256, 0, st>>>(rowptr, col, val, n_pieces, ps, pl, pt, F, H, ldH, Y, ldY, scratch, ldS, cap, ovf, ep, rb);
}

#define GC_PIECES(G, A, VWID, UU)                                                                                 \
  launch_pieces<G, A, VWID, UU>(planned, rowptr, col, val, n_pieces, ps, pl, pt, F, H, ldH, Y, ldY, scratch, ldS, \
                                cap, ovf, ep, rb, st)

// GROUP x NACC 128-bit vectors cover a row of H; small groups keep several
// pieces in flight per warp and four accumulators per lane amortise the
// (col, val) broadcast.
void dispatch_vec4(bool planned, const int32_t* rowptr, const int32_t* col, const float* val, int n_pieces,
                   const int32_t* ps, const int32_t* pl, const int32_t* pt, int F, const float* H, int64_t ldH,
                   float* Y, int64_t ldY, float* scratch, int64_t ldS, int cap, int32_t* ovf, const Epilogue& ep,
                   const RowBlocks& rb, cudaStream_t st) {
  const int units = F / 4;  // 128-bit vectors per row
  // Measured on the 126 M-non-zero graph: up to 8 floats the lane-per-non-zero kernel wins (F = 8: 0.99 ms
  // against 2.0 ms); from 12 to 32 floats groups of 4 lanes with one or two 128-bit vectors per lane and 4
  // non-zeros in flight do (F = 32: 1.5 ms against 1.7 ms for 8 lanes x 1 vector, 3.4 ms for 2 lanes x 4
  // vectors and 4.2 ms for lane-per-non-zero).
  if (units <= 2) {
    const unsigned grid = unsigned((n_pieces + 31) / 32);
#define GC_NARROW(NV, UU)                                                                                       \
  do {                                                                                                          \
    if (planned)                                                                                                \
      spmm_pieces_narrow_kernel<NV, UU, true><<<grid, 256, 0, st>>>(rowptr, col, val, n_pieces, ps, pl, pt, F, H, \
                                                                   ldH, Y, ldY, scratch, ldS, cap, ovf, ep, rb);    \
    else                                                                                                        \
      spmm_pieces_narrow_kernel<NV, UU, false><<<grid, 256, 0, st>>>(rowptr, col, val, n_pieces, ps, pl, pt, F,  \
                                                                    H, ldH, Y, ldY, scratch, ldS, cap, ovf, ep, rb); \
  } while (0)
    if (units <= 1) GC_NARROW(1, 4);
    else GC_NARROW(2, 4);
#undef GC_NARROW
    return;
  }
  if (units <= 4) GC_PIECES(4, 1, 4, 4);
  else if (units <= 8) GC_PIECES(4, 2, 4, 4);  // F = 32: 1.54 ms; 8 lanes x 1 vector x 8 in flight: 1.73 ms
  else if (units <= 12) GC_PIECES(4, 3, 4, 4);  // F = 48 on 126 M non-zeros: 2.24 ms against 2.35 ms with a fourth, idle vector
  else if (units <= 16) GC_PIECES(4, 4, 4, 4);
  else if (units <= 32) GC_PIECES(8, 4, 4, 4);
  else if (units <= 64) GC_PIECES(16, 4, 4, 4);
  else GC_PIECES(32, 4, 4, 2);
}

void dispatch_scalar(bool planned, const int32_t* rowptr, const int32_t* col, const float* val, int n_pieces,
                     const int32_t* ps, const int32_t* pl, const int32_t* pt, int F, const float* H, int64_t ldH,
                     float* Y, int64_t ldY, float* scratch, int64_t ldS, int cap, int32_t* ovf, const Epilogue& ep,
                     const RowBlocks& rb, cudaStream_t st) {
  if (F <= 8) GC_PIECES(8, 1, 1, 4);
  else if (F <= 16) GC_PIECES(16, 1, 1, 4);
  else if (F <= 32) GC_PIECES(32, 1, 1, 4);
  else if (F <= 64) GC_PIECES(32, 2, 1, 4);
  else GC_PIECES(32, 4, 1, 4);
}
// H in bf16: 8 elements per 16-byte vector; the same bytes in flight per lane as the fp32 mappings
// (two accumulator vectors of 8 floats, up to 8 rows of H per round).
void dispatch_bf16(bool planned, const int32_t* rowptr, const int32_t* col, const float* val, int n_pieces,
                   const int32_t* ps, const int32_t* pl, const int32_t* pt, int F, const uint16_t* H, int64_t ldH,
                   float* Y, int64_t ldY, float* scratch, int64_t ldS, int cap, int32_t* ovf, const Epilogue& ep,
                   const RowBlocks& rb, cudaStream_t st) {
  const int units = F / 8;
  if (units <= 4) GC_PIECES(4, 1, 8, 4);
  else if (units <= 8) GC_PIECES(4, 2, 8, 4);
  else if (units <= 16) GC_PIECES(8, 2, 8, 8);
  else if (units <= 32) GC_PIECES(16, 2, 8, 8);
  else GC_PIECES(32, 2, 8, 4);
}
#undef GC_PIECES

inline int64_t scratch_ld(int64_t F) { return (F + 3) & ~int64_t(3); }

}  // namespace

extern "C" {

int64_t gc_spmm_default_panel_cols(int64_t K, int64_t F) {
  if (K <= 0 || F <= 0) return 1;
  // Measured on a 2.4 M-node power-law graph (B200, 126 MB L2): the time falls
  // with the panel width until a panel's rows of H take about 128 MB -- every
  // cut costs a partial-sum row and shortens the pieces -- and rises again when
  // the matrix is not cut by column at all.
  const int64_t target_bytes = int64_t(128) << 20;
  const int64_t cols = target_bytes / (F * 4);
  int64_t p2 = 1024;
  while (p2 * 2 <= cols && p2 < 262144) p2 *= 2;
  return std::min<int64_t>(p2, std::max<int64_t>(K, 1));
}

int64_t gc_spmm_default_segment(int64_t nnz) {
  // A piece is walked by one group of lanes, a few gathers per memory round
  // trip, so its length bounds the critical path of the launch.  Aim at about
  // twice the average load of the ~16 K groups a B200 keeps resident.
  int64_t want = nnz / 8192;
  int64_t p2 = 128;
  while (p2 < want && p2 < GC_SPMM_SEGMENT_MAX) p2 *= 2;
  return p2;
}

size_t gc_spmm_plan_workspace_bytes(int64_t M, int64_t n_pieces) {
  if (M < 0 || n_pieces < 0) return 0;
  return carve(nullptr, M, n_pieces).total;
}

int gc_spmm_plan_count(const int32_t* rowptr, const int32_t* col, int64_t M, int64_t K, int64_t panel_cols,
                       int64_t segment, int64_t* counts, void* workspace, size_t workspace_bytes, void* stream) {
  GC_REQUIRE(M >= 0 && K >= 0 && M < INT32_MAX && K < INT32_MAX, "gc_spmm_plan_count: size out of int32 range");
  GC_REQUIRE(panel_cols >= 1 && panel_cols < INT32_MAX, "gc_spmm_plan_count: panel_cols must be positive");
  GC_REQUIRE(segment >= 32 && segment <= GC_SPMM_SEGMENT_MAX, "gc_spmm_plan_count: segment out of range");
  GC_REQUIRE(counts && workspace, "gc_spmm_plan_count: null pointer");
  GC_REQUIRE(M == 0 || rowptr, "gc_spmm_plan_count: null rowptr");
  if (workspace_bytes < gc_spmm_plan_workspace_bytes(M, 0))
    return gc::fail(GC_ERR_WORKSPACE, "gc_spmm_plan_count: workspace too small");
  cudaStream_t st = gc::as_stream(stream);
  const PlanWs w = carve(workspace, M, 0);
  if (M > 0) {
    int rc = count_rows(rowptr, col, int(M), int(K), int(panel_cols), int(segment), w, st);
    if (rc != GC_OK) return rc;
  }
  plan_totals_kernel<<<1, 1, 0, st>>>(w.rows_pieces, w.rows_cut, w.rows_slots, w.piece_base, w.cut_base,
                                      w.slot_base, int(M), counts);
  return gc::check_launch("gc_spmm_plan_count");
}

size_t gc_spmm_plan_bytes(int64_t n_pieces, int64_t n_cut) {
  if (n_pieces < 0 || n_cut < 0) return 0;
  return sizeof(PlanHeader) + 3 * align16(size_t(n_pieces) * 4) + 3 * align16(size_t(n_cut) * 4);
}

int gc_spmm_plan_build(const int32_t* rowptr, const int32_t* col, int64_t M, int64_t K, int64_t panel_cols,
                       int64_t segment, int64_t n_pieces, int64_t n_slots, int64_t n_cut, void* plan, size_t plan_bytes,
                       void* workspace, size_t workspace_bytes, void* stream) {
  GC_REQUIRE(M >= 0 && K >= 0 && M < INT32_MAX && K < INT32_MAX, "gc_spmm_plan_build: size out of int32 range");
  GC_REQUIRE(panel_cols >= 1 && panel_cols < INT32_MAX, "gc_spmm_plan_build: panel_cols must be positive");
  GC_REQUIRE(segment >= 32 && segment <= GC_SPMM_SEGMENT_MAX, "gc_spmm_plan_build: segment out of range");
  GC_REQUIRE(n_pieces >= M && n_pieces < INT32_MAX && n_slots >= 0 && n_slots < INT32_MAX && n_cut >= 0 && n_cut <= M,
             "gc_spmm_plan_build: counts are not those gc_spmm_plan_count reported");
  GC_REQUIRE(plan && workspace, "gc_spmm_plan_build: null pointer");
  GC_REQUIRE(gc::aligned16(plan), "gc_spmm_plan_build: plan must be 16-byte aligned");
  if (plan_bytes < gc_spmm_plan_bytes(n_pieces, n_cut))
    return gc::fail(GC_ERR_WORKSPACE, "gc_spmm_plan_build: plan buffer too small");
  if (workspace_bytes < gc_spmm_plan_workspace_bytes(M, n_pieces))
    return gc::fail(GC_ERR_WORKSPACE, "gc_spmm_plan_build: workspace too small");
  cudaStream_t st = gc::as_stream(stream);
  const PlanWs w = carve(workspace, M, n_pieces);
  PlanView pv = plan_view(plan, n_pieces, n_cut);
  plan_header_kernel<<<1, 1, 0, st>>>(pv.hdr, int(M), int(n_pieces), int(n_slots), int(n_cut), int(panel_cols));
  int rc = gc::check_launch("spmm plan: header");
  if (rc != GC_OK || M == 0) return rc;
  if ((rc = count_rows(rowptr, col, int(M), int(K), int(panel_cols), int(segment), w, st)) != GC_OK) return rc;
  const unsigned gm = unsigned((M + 255) / 256), gp = unsigned((n_pieces + 255) / 256);
  plan_emit_kernel<<<gm, 256, 0, st>>>(rowptr, col, int(M), int(K), int(panel_cols), int(segment), w.rows_cut, w.piece_base,
                                       w.cut_base, w.slot_base, w.rows_pieces, w.keys, w.ids, w.u_start, w.u_len,
                                       w.u_target, pv.cut_row, pv.cut_slot0, pv.cut_nslots);
  if ((rc = gc::check_launch("spmm plan: emit")) != GC_OK) return rc;
  cub::DoubleBuffer<uint64_t> dk(w.keys, w.keys_alt);
  cub::DoubleBuffer<int32_t> dv(w.ids, w.ids_alt);
  const int n_panels = int((K + panel_cols - 1) / panel_cols);
  int phase_bits = 1;
  while ((1 << phase_bits) <= n_panels) ++phase_bits;
  size_t need = 0;
  cudaError_t e = cub::DeviceRadixSort::SortPairs(nullptr, need, dk, dv, int(n_pieces), 0, 32 + phase_bits, st);
  if (e == cudaSuccess && need > w.cub_bytes)
    return gc::fail(GC_ERR_WORKSPACE, "spmm plan: sort needs %zu bytes of temporary storage, have %zu", need,
                    w.cub_bytes);
  size_t b = w.cub_bytes;
  if (e == cudaSuccess) e = cub::DeviceRadixSort::SortPairs(w.cub, b, dk, dv, int(n_pieces), 0, 32 + phase_bits, st);
  if (e != cudaSuccess) return gc::fail(GC_ERR_CUDA, "spmm plan: sort: %s", cudaGetErrorString(e));
  gc::count_launches(4);
  plan_gather_kernel<<<gp, 256, 0, st>>>(dv.Current(), int(n_pieces), w.u_start, w.u_len, w.u_target, pv.start,
                                         pv.len, pv.target);
  return gc::check_launch("spmm plan: gather");
}

size_t gc_spmm_scratch_bytes(int64_t n_slots, int64_t F) {
  if (n_slots < 0 || F <= 0) return 0;
  return std::max<size_t>(size_t(n_slots) * size_t(scratch_ld(F)) * sizeof(float), 256);
}

int gc_spmm_plan_check(const void* plan, int64_t n_pieces, int64_t n_slots, int64_t n_cut, void* stream) {
  GC_REQUIRE(plan, "gc_spmm_plan_check: null plan");
  cudaStream_t st = gc::as_stream(stream);
  PlanHeader h{};
  cudaError_t e = cudaMemcpyAsync(&h, plan, sizeof(h), cudaMemcpyDeviceToHost, st);
  if (e == cudaSuccess) e = cudaStreamSynchronize(st);
  if (e != cudaSuccess) return gc::fail(GC_ERR_CUDA, "gc_spmm_plan_check: %s", cudaGetErrorString(e));
  if (h.magic != kPlanMagic) return gc::fail(GC_ERR_INVALID, "gc_spmm_plan_check: not a plan built by this library");
  if (h.n_pieces != n_pieces || h.n_slots != n_slots || h.n_cut != n_cut)
    return gc::fail(GC_ERR_INVALID,
                    "gc_spmm_plan_check: the plan holds %d pieces / %d slots / %d cut rows, the caller passed "
                    "%lld / %lld / %lld",
                    h.n_pieces, h.n_slots, h.n_cut, (long long)n_pieces, (long long)n_slots, (long long)n_cut);
  if (h.overflow)
    return gc::fail(GC_ERR_DEVICE_FLAG,
                    "gc_spmm_plan_check: a launch on this plan skipped partial sums (counts or scratch too small)");
  return GC_OK;
}

}  // extern "C"

namespace {
// The product behind gc_spmm_csr_f32 (rb.block_rows == 0, rows go to Y) and gc_spmm_csr_f32_blocks.
// H16 non-null: H is read from that bf16 copy instead (H ignored).
int spmm_run(const int32_t* rowptr, const int32_t* col, const float* val, int64_t M, int64_t K, int64_t F,
             const float* H, const uint16_t* H16, int64_t ldH, const float* bias, int epilogue, float* Y,
             const RowBlocks& rb, int64_t ldY,
             float* mask, const float* gate, const void* plan, int64_t n_pieces, int64_t n_slots, int64_t n_cut,
             void* scratch, size_t scratch_bytes, void* stream) {
  GC_REQUIRE(M >= 0 && K >= 0 && F >= 0, "gc_spmm_csr_f32: negative size");
  GC_REQUIRE(M < INT32_MAX && K < INT32_MAX && F < INT32_MAX, "gc_spmm_csr_f32: size out of int32 range");
  GC_REQUIRE((epilogue & ~(GC_EPI_RELU | GC_EPI_ACCUMULATE)) == 0, "gc_spmm_csr_f32: unknown epilogue bits");
  if (M == 0 || F == 0) return GC_OK;
  GC_REQUIRE(rowptr && Y, "gc_spmm_csr_f32: null rowptr/Y");
  GC_REQUIRE(ldY >= F && (K == 0 || ldH >= F), "gc_spmm_csr_f32: leading dimension smaller than F");
  GC_REQUIRE(K == 0 || H || H16, "gc_spmm_csr_f32: null H");
  cudaStream_t st = gc::as_stream(stream);
  Epilogue ep{bias, mask, gate, (epilogue & GC_EPI_RELU) ? 1 : 0, (epilogue & GC_EPI_ACCUMULATE) ? 1 : 0};

  bool blocks_aligned = true;
  if (rb.block_rows)
    for (int64_t b = 0; b * rb.block_rows < M; ++b) blocks_aligned = blocks_aligned && gc::aligned16(rb.base[b]);
  const bool out_vec4 = (ldY % 4 == 0) && gc::aligned16(Y) && blocks_aligned && (!bias || gc::aligned16(bias)) &&
                        (!mask || gc::aligned16(mask)) && (!gate || gc::aligned16(gate));
  const bool vec4 = (F % 4 == 0) && (ldH % 4 == 0) && gc::aligned16(H) && out_vec4;
  if (H16 && !((F % 8 == 0) && (ldH % 8 == 0) && gc::aligned16(H16) && out_vec4))
    return gc::fail(GC_ERR_UNSUPPORTED,
                    "gc_spmm_csr_bf16h_f32: F and ldH must be multiples of 8, H16 / Y / bias / mask / gate 16-byte "
                    "aligned, ldY a multiple of 4");
  const bool planned = plan != nullptr;
  const int32_t *ps = nullptr, *pl = nullptr, *pt = nullptr;
  PlanView pv{};
  int np = int(M), cap = 0;
  int32_t* ovf = nullptr;
  const int64_t ldS = scratch_ld(F);
  if (planned) {
    GC_REQUIRE(gc::aligned16(plan), "gc_spmm_csr_f32: plan must be 16-byte aligned");
    GC_REQUIRE(n_pieces >= M && n_pieces < INT32_MAX && n_cut >= 0 && n_cut <= M && n_slots >= 0 &&
                   n_slots <= n_pieces && (n_cut == 0) == (n_slots == 0) && n_slots >= 2 * n_cut,
               "gc_spmm_csr_f32: n_pieces / n_slots / n_cut do not describe a plan of this matrix");
    pv = plan_view(const_cast<void*>(plan), n_pieces, n_cut);
    ovf = &pv.hdr->overflow;  // the one word of the plan a launch may write
    ps = pv.start;
    pl = pv.len;
    pt = pv.target;
    np = int(n_pieces);
    if (n_cut > 0) {
      if (!scratch) return gc::fail(GC_ERR_WORKSPACE, "gc_spmm_csr_f32: the plan cuts rows but scratch is null");
      GC_REQUIRE(gc::aligned16(scratch), "gc_spmm_csr_f32: scratch must be 16-byte aligned");
      const size_t need = gc_spmm_scratch_bytes(n_slots, F);
      if (scratch_bytes < need)
        return gc::fail(GC_ERR_WORKSPACE,
                        "gc_spmm_csr_f32: %lld partial-sum rows of F=%lld need %zu bytes of scratch, got %zu",
                        (long long)n_slots, (long long)F, need, scratch_bytes);
      cap = int(n_slots);  // slots beyond what the caller declared are skipped and flagged, never written
    }
  }
  float* sc = static_cast<float*>(scratch);
  if (H16)
    dispatch_bf16(planned, rowptr, col, val, np, ps, pl, pt, int(F), H16, ldH, Y, ldY, sc, ldS, cap, ovf, ep, rb, st);
  else if (vec4)
    dispatch_vec4(planned, rowptr, col, val, np, ps, pl, pt, int(F), H, ldH, Y, ldY, sc, ldS, cap, ovf, ep, rb, st);
  else
    dispatch_scalar(planned, rowptr, col, val, np, ps, pl, pt, int(F), H, ldH, Y, ldY, sc, ldS, cap, ovf, ep, rb, st);
  int rc = gc::check_launch("gc_spmm_csr_f32 (pieces)");
  if (rc != GC_OK) return rc;
  if (planned && n_cut > 0) {
    const unsigned g = unsigned(std::min<int64_t>((n_cut + 7) / 8, gc::kNumSMs * 8));
    if (vec4 || H16)
      spmm_finalize_kernel<4><<<g, 256, 0, st>>>(int(F), int(n_cut), pv.cut_row, pv.cut_slot0, pv.cut_nslots, sc, ldS,
                                                 cap, ovf, Y, ldY, ep, rb);
    else
      spmm_finalize_kernel<1><<<g, 256, 0, st>>>(int(F), int(n_cut), pv.cut_row, pv.cut_slot0, pv.cut_nslots, sc, ldS,
                                                 cap, ovf, Y, ldY, ep, rb);
    rc = gc::check_launch("gc_spmm_csr_f32 (finalize)");
  }
  return rc;
}
}  // namespace

extern "C" {

int gc_spmm_csr_f32(const int32_t* rowptr, const int32_t* col, const float* val, int64_t M, int64_t K, int64_t F,
                    const float* H, int64_t ldH, const float* bias, int epilogue, float* Y, int64_t ldY,
                    float* mask, const float* gate, const void* plan, int64_t n_pieces, int64_t n_slots, int64_t n_cut,
                    void* scratch, size_t scratch_bytes, void* stream) {
  RowBlocks rb{};
  return spmm_run(rowptr, col, val, M, K, F, H, nullptr, ldH, bias, epilogue, Y, rb, ldY, mask, gate, plan, n_pieces,
                  n_slots, n_cut, scratch, scratch_bytes, stream);
}

int gc_spmm_csr_bf16h_f32(const int32_t* rowptr, const int32_t* col, const float* val, int64_t M, int64_t K, int64_t F,
                          const uint16_t* H16, int64_t ldH, const float* bias, int epilogue, float* Y, int64_t ldY,
                          float* mask, const float* gate, const void* plan, int64_t n_pieces, int64_t n_slots,
                          int64_t n_cut, void* scratch, size_t scratch_bytes, void* stream) {
  RowBlocks rb{};
  GC_REQUIRE(K == 0 || M == 0 || F == 0 || H16, "gc_spmm_csr_bf16h_f32: null H16");
  return spmm_run(rowptr, col, val, M, K, F, nullptr, H16, ldH, bias, epilogue, Y, rb, ldY, mask, gate, plan, n_pieces,
                  n_slots, n_cut, scratch, scratch_bytes, stream);
}

int gc_spmm_csr_f32_blocks(const int32_t* rowptr, const int32_t* col, const float* val, int64_t M, int64_t K,
                           int64_t F, const float* H, int64_t ldH, const float* bias, int epilogue,
                           float* const* Y_blocks, int n_blocks, int64_t block_rows, int64_t ldY, const void* plan,
                           int64_t n_pieces, int64_t n_slots, int64_t n_cut, void* scratch, size_t scratch_bytes,
                           void* stream) {
  GC_REQUIRE(n_blocks >= 1 && n_blocks <= GC_SPMM_MAX_BLOCKS, "gc_spmm_csr_f32_blocks: between 1 and %d blocks",
             GC_SPMM_MAX_BLOCKS);
  GC_REQUIRE(block_rows >= 1 && block_rows < INT32_MAX && M >= 0 && int64_t(n_blocks) * block_rows >= M,
             "gc_spmm_csr_f32_blocks: n_blocks * block_rows must cover the M rows");
  GC_REQUIRE((epilogue & ~GC_EPI_RELU) == 0, "gc_spmm_csr_f32_blocks: only bias and ReLU can be fused here");
  GC_REQUIRE(Y_blocks, "gc_spmm_csr_f32_blocks: null block list");
  RowBlocks rb{};
  for (int b = 0; b < n_blocks; ++b) {
    GC_REQUIRE(Y_blocks[b] || int64_t(b) * block_rows >= M, "gc_spmm_csr_f32_blocks: null block pointer");
    rb.base[b] = Y_blocks[b];
  }
  rb.block_rows = int(block_rows);
  return spmm_run(rowptr, col, val, M, K, F, H, nullptr, ldH, bias, epilogue, Y_blocks[0], rb, ldY, nullptr, nullptr,
                  plan, n_pieces, n_slots, n_cut, scratch, scratch_bytes, stream);
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
                            int64_t F, const float* H, int64_t ldH, const float* bias, int epilogue, float* Y,
                            int64_t ldY, float* mask, const float* gate, const void* plan, int64_t n_pieces,
                            int64_t n_slots, int64_t n_cut, void* stream) {
  GC_REQUIRE(n_slots >= 0, "gc_spmm_csr_f32_noalloc: negative n_slots");
  if (!plan || n_cut == 0)  // no cut rows, hence no scratch at all
    return gc_spmm_csr_f32(rowptr, col, val, M, K, F, H, ldH, bias, epilogue, Y, ldY, mask, gate, plan, n_pieces,
                           n_slots, n_cut, nullptr, 0, stream);
  const size_t need = gc_spmm_scratch_bytes(n_slots, F);
  if (need > size_t(GC_SPMM_STATIC_SCRATCH_BYTES))
    return gc::fail(GC_ERR_WORKSPACE,
                    "gc_spmm_csr_f32_noalloc: %lld partial-sum rows of F=%lld need %zu bytes of scratch, the "
                    "built-in buffer holds %zu; use gc_spmm_csr_f32 with caller-provided scratch",
                    (long long)n_slots, (long long)F, need, size_t(GC_SPMM_STATIC_SCRATCH_BYTES));
  float* scratch = nullptr;
  const int rc = static_scratch_for_current_device(&scratch);
  if (rc != GC_OK) return rc;
  // Every partial-sum row the finalize pass reads is fully written by the
  // piece pass of the same call, so stale contents of the shared buffer are
  // never observed and nothing has to be cleared.
  return gc_spmm_csr_f32(rowptr, col, val, M, K, F, H, ldH, bias, epilogue, Y, ldY, mask, gate, plan, n_pieces,
                         n_slots, n_cut, scratch, size_t(GC_SPMM_STATIC_SCRATCH_BYTES), stream);
}

}  // extern "C"

// Fixed-degree, unit-weight row gather:  Y[i, :] = sum_{k < deg} H[idx[i * deg + k], :].
//
// A measurement aid for the CSR aggregation (spmm_csr.cu, which takes over
// src/graphcuda/cuda/spmm_cusparse.cu:3-126): the same access pattern -- a
// group of lanes reads whole rows of H with 128-bit loads, U rows x NACC
// vectors in flight per lane -- with everything else removed (no values, no
// plan, no epilogue, no ragged rows).  Timed on index lists with a chosen
// locality it gives the rate at which the memory system delivers gathered rows
// to the SMs, i.e. the ceiling the aggregation kernel can be compared with
// when H is far larger than the L2.  The result is a real sum, so the kernel
// is checked like any other (tests/test_spmm_gpu.py).
#include "common.cuh"

namespace {

template <int GROUP, int NACC, int U, int MIN_CTAS>
__global__ void __launch_bounds__(256, MIN_CTAS)
gather_sum_kernel(const float* __restrict__ H, int64_t ldH, const int32_t* __restrict__ idx, int n_rows, int deg,
                  int F, float* __restrict__ Y, int64_t ldY) {
  constexpr int ROWS_PER_CTA = 256 / GROUP;
  constexpr int PASS = GROUP * NACC * 4;
  const int lane_g = threadIdx.x % GROUP;
  const int r = blockIdx.x * ROWS_PER_CTA + threadIdx.x / GROUP;
  if (r >= n_rows) return;
  const unsigned gmask = (GROUP == 32) ? 0xffffffffu
                                       : (((1u << GROUP) - 1u) << ((threadIdx.x % 32) / GROUP * GROUP));
  const int32_t* my = idx + int64_t(r) * deg;
  for (int f0 = 0; f0 < F; f0 += PASS) {
    float4 acc[NACC];
    bool live[NACC];
#pragma unroll
    for (int a = 0; a < NACC; ++a) {
      acc[a] = make_float4(0.f, 0.f, 0.f, 0.f);
      live[a] = (f0 + (a * GROUP + lane_g) * 4) < F;
    }
    int c_next = lane_g < deg ? __ldcs(my + lane_g) : 0;
    for (int base = 0; base < deg; base += GROUP) {
      const int c = c_next;
      const int e2 = base + GROUP + lane_g;
      if (e2 < deg) c_next = __ldcs(my + e2);
      const int cnt = min(GROUP, deg - base);
      for (int j = 0; j < cnt; j += U) {
        float4 h[U][NACC];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int cj = __shfl_sync(gmask, c, (j + u) % GROUP, GROUP);
          const float* hp = H + int64_t(cj) * ldH + f0;
          const bool valid = (j + u) < cnt;
#pragma unroll
          for (int a = 0; a < NACC; ++a)
            h[u][a] = (live[a] && valid) ? __ldg(reinterpret_cast<const float4*>(hp + (a * GROUP + lane_g) * 4))
                                         : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int u = 0; u < U; ++u)
#pragma unroll
          for (int a = 0; a < NACC; ++a) {
            acc[a].x += h[u][a].x;
            acc[a].y += h[u][a].y;
            acc[a].z += h[u][a].z;
            acc[a].w += h[u][a].w;
          }
      }
    }
    float* yrow = Y + int64_t(r) * ldY + f0;
#pragma unroll
    for (int a = 0; a < NACC; ++a)
      if (live[a]) *reinterpret_cast<float4*>(yrow + (a * GROUP + lane_g) * 4) = acc[a];
  }
}

template <int GROUP, int NACC, int U, int MIN_CTAS>
void launch(const float* H, int64_t ldH, const int32_t* idx, int n_rows, int deg, int F, float* Y, int64_t ldY,
            cudaStream_t st) {
  constexpr int PER = 256 / GROUP;
  gather_sum_kernel<GROUP, NACC, U, MIN_CTAS>
      <<<unsigned((n_rows + PER - 1) / PER), 256, 0, st>>>(H, ldH, idx, n_rows, deg, F, Y, ldY);
}

}  // namespace

extern "C" int gc_gather_sum_f32(const float* H, int64_t ldH, int64_t K, int64_t F, const int32_t* idx,
                                 int64_t n_rows, int64_t deg, float* Y, int64_t ldY, int in_flight, void* stream) {
  GC_REQUIRE(n_rows >= 0 && deg >= 0 && K >= 0 && F >= 0, "gc_gather_sum_f32: negative size");
  GC_REQUIRE(n_rows < INT32_MAX && deg < INT32_MAX && K < INT32_MAX && F < INT32_MAX,
             "gc_gather_sum_f32: size out of int32 range");
  GC_REQUIRE(in_flight == 0 || in_flight == 4 || in_flight == 8, "gc_gather_sum_f32: in_flight must be 0, 4 or 8");
  if (n_rows == 0 || F == 0) return GC_OK;
  GC_REQUIRE(H && Y && (deg == 0 || idx), "gc_gather_sum_f32: null pointer");
  GC_REQUIRE(F % 4 == 0 && ldH % 4 == 0 && ldY % 4 == 0 && ldH >= F && ldY >= F && gc::aligned16(H) &&
                 gc::aligned16(Y),
             "gc_gather_sum_f32: rows must be 16-byte aligned multiples of four floats");
  cudaStream_t st = gc::as_stream(stream);
  const int units = int(F / 4);
  const bool deep = in_flight == 8;
#define GC_GATHER(G, A)                                                                    \
  do {                                                                                     \
    if (deep) launch<G, A, (G < 8 ? G : 8), 2>(H, ldH, idx, int(n_rows), int(deg), int(F), Y, ldY, st); \
    else launch<G, A, 4, 3>(H, ldH, idx, int(n_rows), int(deg), int(F), Y, ldY, st);        \
  } while (0)
  // the lane mappings of the aggregation kernel for the same widths
  if (units <= 4) GC_GATHER(4, 1);
  else if (units <= 8) GC_GATHER(4, 2);
  else if (units <= 16) GC_GATHER(4, 4);
  else if (units <= 32) GC_GATHER(8, 4);
  else if (units <= 64) GC_GATHER(16, 4);
  else GC_GATHER(32, 4);
#undef GC_GATHER
  return gc::check_launch("gc_gather_sum_f32");
}

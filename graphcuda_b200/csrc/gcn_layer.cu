// One GCN layer, forward and backward, as two C entry points: the composition
// the reference does in its gcn_conv_forward / gcn_conv_backward
// (src/graphcuda/cuda/gcn.cu:5-25 and :27-52; ATen twin src/graphcuda/cpp/gcn.cpp:4-41)
// out of spmm_cusparse, gemm_cublas and element-wise ATen calls, done here out
// of this library's aggregation and GEMM with the ReLU / mask / bias work fused
// into their stores.  A host that binds the C ABI gets the whole layer -- the
// order of the two products, the fused epilogues, the saved intermediate --
// without re-deriving it from the single-kernel entry points.
//
//   forward   Y  = relu((A X) W + b)                         gcn.cu:12-20
//   backward  G  = dY * mask;  dW = (A X)^T G;  dX = A (G W^T)   gcn.cu:36-49
//
// GC_LAYER_TRANSFORM_FIRST computes A (X W) instead (and S = A G, dW = X^T S,
// dX = S W^T in the backward pass): the aggregation then runs on the output
// width.  Only valid for a symmetric A (the reference multiplies by A, never
// A^T, in its backward pass: gcn.cu:49) -- the caller asserts that.
#include "common.cuh"

#include <algorithm>

namespace {

inline size_t up256(size_t x) { return (x + 255) & ~size_t(255); }

struct LayerWs {
  char* spmm_scratch;
  size_t spmm_bytes;
  char* gemm_ws;
  size_t gemm_bytes;
  float* inter;   // n x max(in, out): H = X W (forward, transform first), G / T / S (backward)
  float* inter2;  // n x max(in, out): second intermediate of the backward pass
  size_t total;
};

LayerWs carve(void* ws, int64_t n, int64_t in_dim, int64_t out_dim, int64_t n_slots, int precision, bool backward) {
  LayerWs w{};
  char* p = static_cast<char*>(ws);
  size_t off = 0;
  const int64_t wide = std::max(in_dim, out_dim);
  w.spmm_bytes = up256(gc_spmm_scratch_bytes(n_slots, wide));
  w.spmm_scratch = p ? p + off : nullptr;
  off += w.spmm_bytes;
  size_t g = 256;
  // every product of the layer: (n x in) (in x out), (in x n) (n x out), (n x out) (out x in)
  g = std::max(g, gc_gemm_workspace_bytes(0, 0, n, out_dim, in_dim, precision));
  if (backward) {
    g = std::max(g, gc_gemm_workspace_bytes(1, 0, in_dim, out_dim, n, precision));
    g = std::max(g, gc_gemm_workspace_bytes(0, 1, n, in_dim, out_dim, precision));
  }
  w.gemm_bytes = up256(g);
  w.gemm_ws = p ? p + off : nullptr;
  off += w.gemm_bytes;
  const size_t inter_bytes = up256(size_t(n) * size_t(wide) * sizeof(float));
  w.inter = reinterpret_cast<float*>(p ? p + off : nullptr);
  off += inter_bytes;
  if (backward) {
    w.inter2 = reinterpret_cast<float*>(p ? p + off : nullptr);
    off += inter_bytes;
  }
  w.total = off;
  return w;
}

}  // namespace

extern "C" {

size_t gc_gcn_layer_workspace_bytes(int64_t n, int64_t in_dim, int64_t out_dim, int64_t n_slots, int precision,
                                    int backward) {
  if (n < 0 || in_dim < 0 || out_dim < 0 || n_slots < 0) return 0;
  return carve(nullptr, std::max<int64_t>(n, 1), std::max<int64_t>(in_dim, 1), std::max<int64_t>(out_dim, 1), n_slots,
               precision, backward != 0)
      .total;
}

int gc_gcn_conv_forward_csr_f32(const int32_t* rowptr, const int32_t* col, const float* val, int64_t n, int64_t in_dim,
                                int64_t out_dim, const float* X, int64_t ldx, const float* W, int64_t ldw,
                                const float* bias, int flags, float* Y, int64_t ldy, float* mask, float* AX,
                                int64_t ldax, const void* plan, int64_t n_pieces, int64_t n_slots, int64_t n_cut,
                                int precision, void* workspace, size_t workspace_bytes, void* stream) {
  GC_REQUIRE(n >= 0 && in_dim >= 0 && out_dim >= 0, "gc_gcn_conv_forward_csr_f32: negative size");
  GC_REQUIRE((flags & ~(GC_LAYER_RELU | GC_LAYER_TRANSFORM_FIRST)) == 0, "gc_gcn_conv_forward_csr_f32: unknown flags");
  if (n == 0 || out_dim == 0) return GC_OK;
  GC_REQUIRE(X && W && Y && rowptr, "gc_gcn_conv_forward_csr_f32: null pointer");
  const bool tf = (flags & GC_LAYER_TRANSFORM_FIRST) != 0;
  GC_REQUIRE(tf || AX, "gc_gcn_conv_forward_csr_f32: AX (n x in) receives A X in the aggregate-first order");
  GC_REQUIRE(workspace && (reinterpret_cast<uintptr_t>(workspace) & 255u) == 0,
             "gc_gcn_conv_forward_csr_f32: workspace must be 256-byte aligned");
  const LayerWs w = carve(workspace, n, std::max<int64_t>(in_dim, 1), out_dim, n_slots, precision, false);
  if (workspace_bytes < w.total)
    return gc::fail(GC_ERR_WORKSPACE, "gc_gcn_conv_forward_csr_f32: workspace of %zu bytes, need %zu", workspace_bytes,
                    w.total);
  const int epi = (flags & GC_LAYER_RELU) ? GC_EPI_RELU : 0;
  int rc;
  if (!tf) {
    // AX = A X (kept by the caller for the backward pass), Y = relu(AX W + b) with the mask from the GEMM's store
    rc = gc_spmm_csr_f32(rowptr, col, val, n, n, in_dim, X, ldx, nullptr, 0, AX, ldax, nullptr, nullptr, plan, n_pieces,
                         n_slots, n_cut, w.spmm_scratch, w.spmm_bytes, stream);
    if (rc != GC_OK) return rc;
    return gc_gemm_f32(0, 0, n, out_dim, in_dim, AX, ldax, W, ldw, Y, ldy, bias, epi, mask, nullptr, precision,
                       w.gemm_ws, w.gemm_bytes, stream);
  }
  // H = X W, Y = relu(A H + b) with the mask from the aggregation's store
  rc = gc_gemm_f32(0, 0, n, out_dim, in_dim, X, ldx, W, ldw, w.inter, out_dim, nullptr, 0, nullptr, nullptr, precision,
                   w.gemm_ws, w.gemm_bytes, stream);
  if (rc != GC_OK) return rc;
  return gc_spmm_csr_f32(rowptr, col, val, n, n, out_dim, w.inter, out_dim, bias, epi, Y, ldy, mask, nullptr, plan,
                         n_pieces, n_slots, n_cut, w.spmm_scratch, w.spmm_bytes, stream);
}

int gc_gcn_conv_backward_csr_f32(const int32_t* rowptr, const int32_t* col, const float* val, int64_t n, int64_t in_dim,
                                 int64_t out_dim, const float* dY, int64_t lddy, const float* X, int64_t ldx,
                                 const float* W, int64_t ldw, int flags, const float* mask, int64_t ldmask,
                                 const float* AX, int64_t ldax, float* dX, int64_t lddx, float* dW, int64_t lddw,
                                 const void* plan, int64_t n_pieces, int64_t n_slots, int64_t n_cut, int precision,
                                 void* workspace, size_t workspace_bytes, void* stream) {
  GC_REQUIRE(n >= 0 && in_dim >= 0 && out_dim >= 0, "gc_gcn_conv_backward_csr_f32: negative size");
  GC_REQUIRE((flags & ~(GC_LAYER_RELU | GC_LAYER_TRANSFORM_FIRST)) == 0, "gc_gcn_conv_backward_csr_f32: unknown flags");
  if (n == 0 || in_dim == 0 || out_dim == 0) return GC_OK;
  GC_REQUIRE(dY && X && W && rowptr, "gc_gcn_conv_backward_csr_f32: null pointer");
  const bool relu = (flags & GC_LAYER_RELU) != 0;
  const bool tf = (flags & GC_LAYER_TRANSFORM_FIRST) != 0;
  GC_REQUIRE(!relu || mask, "gc_gcn_conv_backward_csr_f32: the ReLU layer's backward needs the forward's mask");
  GC_REQUIRE(dX || dW, "gc_gcn_conv_backward_csr_f32: nothing to compute");
  GC_REQUIRE(workspace && (reinterpret_cast<uintptr_t>(workspace) & 255u) == 0,
             "gc_gcn_conv_backward_csr_f32: workspace must be 256-byte aligned");
  const LayerWs w = carve(workspace, n, in_dim, out_dim, n_slots, precision, true);
  if (workspace_bytes < w.total)
    return gc::fail(GC_ERR_WORKSPACE, "gc_gcn_conv_backward_csr_f32: workspace of %zu bytes, need %zu", workspace_bytes,
                    w.total);
  int rc;
  // G = dY * mask (gcn.cu:36)
  const float* G = dY;
  int64_t ldg = lddy;
  if (relu) {
    rc = gc_mask_mul_f32(dY, lddy, mask, ldmask, w.inter, out_dim, n, out_dim, stream);
    if (rc != GC_OK) return rc;
    G = w.inter;
    ldg = out_dim;
  }
  if (!tf) {
    // dW = (A X)^T G (gcn.cu:40-43; A X recomputed like the reference when the caller did not keep it)
    if (dW) {
      const float* ax = AX;
      int64_t ld = ldax;
      if (!ax) {
        rc = gc_spmm_csr_f32(rowptr, col, val, n, n, in_dim, X, ldx, nullptr, 0, w.inter2, in_dim, nullptr, nullptr, plan,
                             n_pieces, n_slots, n_cut, w.spmm_scratch, w.spmm_bytes, stream);
        if (rc != GC_OK) return rc;
        ax = w.inter2;
        ld = in_dim;
      }
      rc = gc_gemm_f32(1, 0, in_dim, out_dim, n, ax, ld, G, ldg, dW, lddw, nullptr, 0, nullptr, nullptr, precision,
                       w.gemm_ws, w.gemm_bytes, stream);
      if (rc != GC_OK) return rc;
    }
    // dX = A (G W^T) (gcn.cu:46-49: A, not A^T)
    if (dX) {
      rc = gc_gemm_f32(0, 1, n, in_dim, out_dim, G, ldg, W, ldw, w.inter2, in_dim, nullptr, 0, nullptr, nullptr, precision,
                       w.gemm_ws, w.gemm_bytes, stream);
      if (rc != GC_OK) return rc;
      rc = gc_spmm_csr_f32(rowptr, col, val, n, n, in_dim, w.inter2, in_dim, nullptr, 0, dX, lddx, nullptr, nullptr, plan,
                           n_pieces, n_slots, n_cut, w.spmm_scratch, w.spmm_bytes, stream);
      if (rc != GC_OK) return rc;
    }
    return GC_OK;
  }
  // Y = A (X W), A symmetric: S = A^T G = A G, dW = X^T S, dX = S W^T
  rc = gc_spmm_csr_f32(rowptr, col, val, n, n, out_dim, G, ldg, nullptr, 0, w.inter2, out_dim, nullptr, nullptr, plan,
                       n_pieces, n_slots, n_cut, w.spmm_scratch, w.spmm_bytes, stream);
  if (rc != GC_OK) return rc;
  if (dW) {
    rc = gc_gemm_f32(1, 0, in_dim, out_dim, n, X, ldx, w.inter2, out_dim, dW, lddw, nullptr, 0, nullptr, nullptr, precision,
                     w.gemm_ws, w.gemm_bytes, stream);
    if (rc != GC_OK) return rc;
  }
  if (dX) {
    rc = gc_gemm_f32(0, 1, n, in_dim, out_dim, w.inter2, out_dim, W, ldw, dX, lddx, nullptr, 0, nullptr, nullptr, precision,
                     w.gemm_ws, w.gemm_bytes, stream);
    if (rc != GC_OK) return rc;
  }
  return GC_OK;
}

}  // extern "C"

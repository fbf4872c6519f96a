/*
 * graphcuda_b200 -- C ABI of the B200 (sm_100a) GCN layer engine.
 *
 * Every entry point takes plain device pointers, 64-bit sizes / leading
 * dimensions (in elements) and the CUDA stream to enqueue on (a cudaStream_t
 * passed as void*).  Entry points enqueue work and return; they never
 * allocate device memory, never synchronise the device and never throw.
 * Callers own every buffer, including the scratch ("workspace") buffers whose
 * sizes the *_bytes queries report.  Return value: GC_OK (0) or a negative
 * GC_ERR_* code; gc_last_error() gives a thread-local message for the last
 * failure on the calling thread.
 *
 * All matrices are row-major fp32.  "ld" is the distance in elements between
 * consecutive rows.
 *
 * Each declaration cites the reference interface (path within the GraphCUDA
 * project : lines) whose work it takes over.
 */
#ifndef GRAPHCUDA_B200_H
#define GRAPHCUDA_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define GC_OK 0
#define GC_ERR_INVALID (-1)      /* bad argument (null pointer, negative size, misaligned, overflow) */
#define GC_ERR_UNSUPPORTED (-2)  /* valid request this build cannot serve (e.g. tensor-core path on an odd ld) */
#define GC_ERR_CUDA (-3)         /* a CUDA runtime / driver call or kernel launch failed */
#define GC_ERR_WORKSPACE (-4)    /* workspace pointer null or too small */
#define GC_ERR_DEVICE_FLAG (-5)  /* a kernel reported a bounded wait that ran out (read back by gc_gemm_check_flag) */

/* ---- library ---------------------------------------------------------- */

/* ABI version, bumped when a signature changes. */
int gc_abi_version(void);
/* Kernels this library has launched in this process so far (all threads). */
long long gc_launch_count(void);
/* Message for the last failure on this thread ("" if none). */
const char* gc_last_error(void);
/* Static text for a GC_* code. */
const char* gc_status_string(int status);

/* ---- CSR sparse x dense (aggregation) ---------------------------------- */

/*
 * Replaces: src/graphcuda/cuda/spmm_cusparse.cu:3-126 (cusparseSpMM on a COO
 * adjacency) as used by gcn_conv_forward / gcn_conv_backward
 * (src/graphcuda/cuda/gcn.cu:12,40,49).
 *
 * A "plan" is derived once per CSR structure (and column-panel width).  It
 * lists the matrix as pieces -- contiguous runs of non-zeros of one row --
 * in the order they are processed:
 *   - rows with more than GC_SPMM_PANEL_MIN_ROW non-zeros are cut at column
 *     panel boundaries (panel_cols columns per panel) and the pieces are
 *     processed panel by panel, so the gathers of a phase hit one slab of H
 *     that stays in the L2;
 *   - pieces longer than `segment` non-zeros are cut further, so heavy rows are
 *     spread over many warps and no piece dominates the launch;
 *   - within a phase pieces are ordered by decreasing length.
 * Pieces of cut rows write partial sums ("slots") to scratch; a second pass
 * adds them in a fixed order.  Building is two calls because the sizes depend
 * on the data: gc_spmm_plan_count -> read the three counts -> allocate ->
 * gc_spmm_plan_build.
 */
#define GC_SPMM_PANEL_MIN_ROW 128 /* rows with more non-zeros than this are cut at panel boundaries */
#define GC_SPMM_SEGMENT_MAX 2048  /* upper limit of the segment length, in non-zeros */

/* Default panel width (columns): a power of two for which panel_cols rows of H
 * (F fp32 each) take about 128 MB, at most 262144 and at most K. */
int64_t gc_spmm_default_panel_cols(int64_t K, int64_t F);
/* Default segment length for a matrix of nnz non-zeros: a power of two in
 * [128, GC_SPMM_SEGMENT_MAX], about nnz / 8192. */
int64_t gc_spmm_default_segment(int64_t nnz);
/* Scratch for plan construction; pass n_pieces = 0 for gc_spmm_plan_count. */
size_t gc_spmm_plan_workspace_bytes(int64_t M, int64_t n_pieces);
/* counts (device, int64[3]) <- {n_pieces, n_slots, n_cut}. */
int gc_spmm_plan_count(const int32_t* rowptr, const int32_t* col, int64_t M, int64_t K, int64_t panel_cols,
                       int64_t segment, int64_t* counts, void* workspace, size_t workspace_bytes, void* stream);
size_t gc_spmm_plan_bytes(int64_t n_pieces, int64_t n_cut);
/* plan: 16-byte aligned device memory of gc_spmm_plan_bytes(n_pieces, n_cut). */
int gc_spmm_plan_build(const int32_t* rowptr, const int32_t* col, int64_t M, int64_t K, int64_t panel_cols,
                       int64_t segment, int64_t n_pieces, int64_t n_slots, int64_t n_cut, void* plan, size_t plan_bytes,
                       void* workspace, size_t workspace_bytes, void* stream);
/* Scratch gc_spmm_csr_f32 needs with a plan of n_slots slots and F feature columns. */
size_t gc_spmm_scratch_bytes(int64_t n_slots, int64_t F);
/* Synchronises `stream` and checks a built plan against the counts the caller
 * holds: GC_OK, GC_ERR_INVALID when n_pieces / n_slots / n_cut are not the
 * plan's own, GC_ERR_DEVICE_FLAG when an earlier gc_spmm_csr_f32 on this plan
 * had to skip partial sums because its counts or scratch were too small
 * (debug / test use: it reads the plan header back to the host). */
int gc_spmm_plan_check(const void* plan, int64_t n_pieces, int64_t n_slots, int64_t n_cut, void* stream);

#define GC_EPI_RELU 1        /* out = max(out, 0) computed as out * (out > 0), reference gcn.cu:19-20 */
#define GC_EPI_ACCUMULATE 2  /* out += result instead of out = result (bias/relu applied after the add) */

/*
 * Y[M,F] = A_csr[M,K] * H[K,F] (+ bias[F]) (ReLU).  mask, when non-null,
 * receives (pre-activation > 0) as 0.0f/1.0f with leading dimension ldY
 * (the fp32 mask of reference gcn.cu:19).  plan may be null: then every row is
 * one piece in natural order (n_pieces, n_cut ignored, no scratch needed).
 * With a plan, n_pieces, n_slots and n_cut are the counts it was built with;
 * scratch_bytes must be at least gc_spmm_scratch_bytes(n_slots, F), else the
 * call is refused with GC_ERR_WORKSPACE (nothing is launched, nothing truncated).
 * Should the counts understate what the plan holds, the pieces that find no
 * room are skipped and a sticky error word is raised in the plan header
 * (read it back with gc_spmm_plan_check).
 * gate, when non-null, is a matrix of Y's shape and leading dimension: the
 * result is multiplied by (gate > 0) last of all -- the ReLU mask of the
 * PREVIOUS layer (reference gcn.cu:36) applied where this layer's input
 * gradient is produced, instead of in a separate pass.
 * No atomics: results are deterministic run to run.
 */
int gc_spmm_csr_f32(const int32_t* rowptr, const int32_t* col, const float* val,
                    int64_t M, int64_t K, int64_t F,
                    const float* H, int64_t ldH,
                    const float* bias, int epilogue,
                    float* Y, int64_t ldY, float* mask, const float* gate,
                    const void* plan, int64_t n_pieces, int64_t n_slots, int64_t n_cut,
                    void* scratch, size_t scratch_bytes,
                    void* stream);

/*
 * The same product with H held in bf16 (bit patterns, K x F, leading dimension ldH in elements; F and ldH
 * multiples of 8, H16 16-byte aligned): the gathers move half the bytes, sums and the output stay fp32.
 * Part of the opt-in reduced-precision tier (1e-2 relative), like GC_PREC_BF16 for the dense products; stands
 * in for the same reference call (spmm_cusparse.cu:105-116).  gc_convert_f32_bf16 makes the copy.
 */
int gc_spmm_csr_bf16h_f32(const int32_t* rowptr, const int32_t* col, const float* val,
                          int64_t M, int64_t K, int64_t F,
                          const uint16_t* H16, int64_t ldH,
                          const float* bias, int epilogue,
                          float* Y, int64_t ldY, float* mask, const float* gate,
                          const void* plan, int64_t n_pieces, int64_t n_slots, int64_t n_cut,
                          void* scratch, size_t scratch_bytes,
                          void* stream);

/*
 * The same product with its rows spread over several output matrices: row i is
 * written to Y_blocks[i / block_rows] at row i % block_rows (leading dimension
 * ldY in all of them).  Y_blocks is a HOST array of n_blocks (<= GC_SPMM_MAX_BLOCKS)
 * device pointers, read during the call.  No counterpart in the reference
 * (it is single-GPU): in the feature-sharded multi-GPU scheme every rank
 * aggregates a slab of columns for ALL nodes and the rows belong to different
 * ranks, so the blocks are the owners' buffers, peer-mapped over NVLink, and the
 * aggregation's own stores deliver the result -- the exchange that would follow
 * the kernel happens inside it (ordinary stores; the caller orders the use of
 * the buffers with its own cross-GPU barrier).  Only bias and ReLU can be
 * fused here (mask, gate and accumulate read or write matrices of Y's shape).
 */
#define GC_SPMM_MAX_BLOCKS 16
int gc_spmm_csr_f32_blocks(const int32_t* rowptr, const int32_t* col, const float* val,
                           int64_t M, int64_t K, int64_t F,
                           const float* H, int64_t ldH,
                           const float* bias, int epilogue,
                           float* const* Y_blocks, int n_blocks, int64_t block_rows, int64_t ldY,
                           const void* plan, int64_t n_pieces, int64_t n_slots, int64_t n_cut,
                           void* scratch, size_t scratch_bytes,
                           void* stream);

/*
 * dst[q][r, c] = src[r, q * w + c] for the n_dst column slabs of width w of a rows x F matrix (the last slab may be
 * narrower).  dst is a HOST array of device pointers, each a matrix of leading dimension dst_ld; they may be other
 * GPUs' peer-mapped buffers.  No counterpart in the reference: it is the rows -> columns transpose that precedes
 * gc_spmm_csr_f32_blocks in the feature-sharded multi-GPU scheme, as one kernel that reads every element once and
 * stores it where the rank that aggregates its slab will gather from.
 */
int gc_scatter_column_slabs_f32(const float* src, int64_t ld, int64_t rows, int64_t F, int64_t w,
                                float* const* dst, int n_dst, int64_t dst_ld, void* stream);

/*
 * Measurement aid, no counterpart in the reference: the access pattern of the
 * aggregation above with everything else removed.
 *   Y[i, :] = sum over k < deg of H[idx[i * deg + k], :]      (i < n_rows)
 * H is K x F (ldH), idx holds n_rows * deg row numbers in [0, K).  F, ldH, ldY
 * multiples of 4, H and Y 16-byte aligned.  in_flight: 0 or 4 = four rows of H
 * in flight per lane as the aggregation keeps, 8 = eight.  Timed on index
 * lists of chosen locality it gives the rate at which gathered rows reach the
 * SMs -- the practical ceiling of gc_spmm_csr_f32 when H is far larger than
 * the L2 (bench.py reports it beside the HBM fraction).
 */
int gc_gather_sum_f32(const float* H, int64_t ldH, int64_t K, int64_t F,
                      const int32_t* idx, int64_t n_rows, int64_t deg,
                      float* Y, int64_t ldY, int in_flight, void* stream);

/*
 * The same aggregation for callers that must not allocate device memory.
 *
 * No counterpart in the reference (its SpMM wrapper cudaMallocs a workspace on
 * every call, spmm_cusparse.cu:100-103).  Some hosts of this library cannot
 * call cudaMalloc at the point where they need the product: a real-time or
 * serving loop with a frozen memory budget, a plugin whose host application
 * owns all device memory and hands out only the input and output buffers.
 * For them the partial-sum scratch lives in a fixed buffer inside the library
 * image: GC_SPMM_STATIC_SCRATCH_BYTES bytes of device memory on every GPU that
 * loads the library, held until the process exits.  The caller still passes
 * the CSR arrays, H, Y (and the plan, which it built once into memory it owns).
 *
 *  - Limit: gc_spmm_scratch_bytes(n_slots, F) must not exceed
 *    GC_SPMM_STATIC_SCRATCH_BYTES; larger problems are refused with
 *    GC_ERR_WORKSPACE and a message, never truncated.
 *  - The first call on a device looks up the buffer's device address
 *    (cudaGetSymbolAddress) with that device current; make that first call
 *    outside any stream capture.  The device that owns `stream` must be the
 *    current device.
 *  - All calls on a device share the one buffer: two calls whose kernels can
 *    overlap on the GPU (different streams, no dependency) race on it.
 *    Serialise them or use gc_spmm_csr_f32 with separate scratch buffers.
 *  - Nothing in the buffer has to be cleared between calls.
 *  - Calls cudaMalloc / cudaFree / any allocating routine: never.
 */
#define GC_SPMM_STATIC_SCRATCH_BYTES (8u << 20)
int gc_spmm_csr_f32_noalloc(const int32_t* rowptr, const int32_t* col, const float* val,
                            int64_t M, int64_t K, int64_t F,
                            const float* H, int64_t ldH,
                            const float* bias, int epilogue,
                            float* Y, int64_t ldY, float* mask, const float* gate,
                            const void* plan, int64_t n_pieces, int64_t n_slots, int64_t n_cut,
                            void* stream);

/* ---- dense GEMM --------------------------------------------------------- */

/*
 * Replaces: gemm_cublas (src/graphcuda/cuda/gemm_cublas.cu:3-55) and the four
 * hand-written SGEMMs matmul1..4 (src/graphcuda/cuda/matmul1.cu:27-61,
 * matmul2.cu:65-100, matmul3.cu:194-243, matmul4.cu:209-265); also the
 * transpose copies the reference makes before its backward GEMMs
 * (gemm_cublas.cu:11-16 called from gcn.cu:43,46): op(A)/op(B) are read in
 * place.
 *
 * C[M,N] = op(A)[M,K] * op(B)[K,N] (+ bias[N]) (ReLU), optional fp32 mask and
 * optional gate input as above (leading dimension ldc).  transA=0: A is stored M x K; transA=1: A is
 * stored K x M.  transB likewise (transB=0: K x N; transB=1: N x K).
 */
#define GC_PREC_AUTO (-1)      /* fp32 semantics: TF32X3 on tensor cores when the shape qualifies, else FP32_SIMT */
#define GC_PREC_FP32_SIMT 0    /* IEEE fp32 FMA on CUDA cores, fixed summation order */
#define GC_PREC_TF32X3 1       /* tcgen05 kind::tf32, split operands, three MMA passes, fp32 accumulate in TMEM */
#define GC_PREC_TF32 2         /* tcgen05 kind::tf32, one pass (opt-in, 1e-2 tolerance tier) */
#define GC_PREC_BF16 3         /* opt-in, 1e-2 tolerance tier: tcgen05 kind::f16 on bf16 copies of both operands made
                                  in the workspace, fp32 accumulate (twice the TF32 tensor rate) when the product is
                                  compute-bound (>= 512 flop per operand byte); memory-bound products run as
                                  GC_PREC_TF32, which reads the fp32 operands in place
                                  (gc_gemm_resolve_precision tells which) */

#define GC_EPI_TRANSPOSED_OUT 4 /* store C transposed: C is N x M with leading dimension ldc (mask likewise) */

size_t gc_gemm_workspace_bytes(int transA, int transB, int64_t M, int64_t N, int64_t K, int precision);
int gc_gemm_f32(int transA, int transB, int64_t M, int64_t N, int64_t K,
                const float* A, int64_t lda, const float* B, int64_t ldb,
                float* C, int64_t ldc,
                const float* bias, int epilogue, float* mask, const float* gate,
                int precision, void* workspace, size_t workspace_bytes,
                void* stream);
/* Which path gc_gemm_f32 would take for these arguments: one of GC_PREC_*
 * (never AUTO), or a negative error. */
int gc_gemm_resolve_precision(int transA, int transB, int64_t M, int64_t N, int64_t K,
                              int64_t lda, int64_t ldb, int64_t ldc, int precision);
/*
 * The bf16 tier with operands the caller keeps in bf16 (a constant matrix -- a dense adjacency, weights --
 * is converted once instead of on every call).  Same role as above: cublasSgemm at
 * src/graphcuda/cuda/gemm_cublas.cu:37-48 and the dense adjm.mm(X) of src/graphcuda/cpp/gcn.cpp:10,
 * under the 1e-2 tolerance tier.
 * gc_convert_f32_bf16: dst (bf16 bit patterns, rows x cols, pitch ld_dst) = src rounded to nearest even; src is
 *   rows x cols (transpose = 0) or cols x rows (transpose = 1); columns [cols, ld_dst) of dst are zero-filled.
 * gc_gemm_bf16_f32: C[M,N] (fp32) = A[M,K] * Bt[N,K]^T, both operands bf16 with K contiguous, pitches multiples
 *   of 8 elements, bases 16-byte aligned; fp32 accumulation; epilogue arguments as gc_gemm_f32.
 */
int gc_convert_f32_bf16(const float* src, int64_t ld_src, int64_t rows, int64_t cols,
                        uint16_t* dst, int64_t ld_dst, int transpose, void* stream);
size_t gc_gemm_bf16_workspace_bytes(int64_t M, int64_t N, int64_t K);
int gc_gemm_bf16_f32(int64_t M, int64_t N, int64_t K,
                     const uint16_t* A, int64_t lda, const uint16_t* Bt, int64_t ldb,
                     float* C, int64_t ldc,
                     const float* bias, int epilogue, float* mask, const float* gate,
                     void* workspace, size_t workspace_bytes, void* stream);

/* Tensor-core kernels bound every wait; a wait that ran out sets a flag word
 * at the start of the workspace.  Synchronises `stream`, reads it back and
 * returns GC_OK or GC_ERR_DEVICE_FLAG (debug / test use). */
int gc_gemm_check_flag(const void* workspace, void* stream);

/* ---- the layer as one call (reference gcn.cu:5-52) ------------------------ */

/*
 * Replaces: gcn_conv_forward (src/graphcuda/cuda/gcn.cu:5-25; signature gcn.cuh:6-10) and gcn_conv_backward
 * (gcn.cu:27-52; gcn.cuh:12-18), ATen twins src/graphcuda/cpp/gcn.cpp:4-41, for a CSR adjacency.
 *
 *   forward   Y[n,out] = relu((A X) W + bias);  mask[n,out] = (pre-activation > 0) as 0/1 floats (may be null)
 *   backward  G = dY * mask;  dW[in,out] = (A X)^T G;  dX[n,in] = A (G W^T)       (A, not A^T: gcn.cu:49)
 *
 * flags: GC_LAYER_RELU = the reference's apply_relu.  GC_LAYER_TRANSFORM_FIRST = compute A (X W) (and
 * S = A G, dW = X^T S, dX = S W^T backward) so that the aggregation runs on the output width; the caller
 * asserts that A is symmetric (gc_csr_is_symmetric), for which the two orders agree up to rounding.
 * AX (n x in, leading dimension ldax): in the aggregate-first order the forward call writes A X there and the
 * backward call reads it; backward accepts null and then recomputes A X as the reference does (gcn.cu:40).
 * dX or dW may be null (not computed; the reference always computes both).  bias may be null (the reference has
 * none).  plan / n_pieces / n_slots / n_cut: as for gc_spmm_csr_f32 (plan may be null).
 * workspace: gc_gcn_layer_workspace_bytes(n, in, out, n_slots, precision, backward) bytes, 256-byte aligned,
 * zero-filled once before its first use (the GEMM keeps a sticky error word in it).
 */
#define GC_LAYER_RELU 1
#define GC_LAYER_TRANSFORM_FIRST 2
size_t gc_gcn_layer_workspace_bytes(int64_t n, int64_t in_dim, int64_t out_dim, int64_t n_slots, int precision,
                                    int backward);
int gc_gcn_conv_forward_csr_f32(const int32_t* rowptr, const int32_t* col, const float* val,
                                int64_t n, int64_t in_dim, int64_t out_dim,
                                const float* X, int64_t ldx, const float* W, int64_t ldw, const float* bias,
                                int flags, float* Y, int64_t ldy, float* mask, float* AX, int64_t ldax,
                                const void* plan, int64_t n_pieces, int64_t n_slots, int64_t n_cut,
                                int precision, void* workspace, size_t workspace_bytes, void* stream);
int gc_gcn_conv_backward_csr_f32(const int32_t* rowptr, const int32_t* col, const float* val,
                                 int64_t n, int64_t in_dim, int64_t out_dim,
                                 const float* dY, int64_t lddy, const float* X, int64_t ldx,
                                 const float* W, int64_t ldw, int flags,
                                 const float* mask, int64_t ldmask, const float* AX, int64_t ldax,
                                 float* dX, int64_t lddx, float* dW, int64_t lddw,
                                 const void* plan, int64_t n_pieces, int64_t n_slots, int64_t n_cut,
                                 int precision, void* workspace, size_t workspace_bytes, void* stream);

/* ---- ReLU mask helpers (reference gcn.cu:19-20,36) ----------------------- */

/* G = dY * (Y > 0), element-wise over an M x N view (reference gcn.cu:36 with
 * the mask re-derived from the saved activation instead of a stored fp32 mask). */
int gc_relu_backward_f32(const float* dY, int64_t lddy, const float* Y, int64_t ldy,
                         float* G, int64_t ldg, int64_t M, int64_t N, void* stream);
/* G = dY * mask for a stored fp32 mask (reference gcn.cu:36 verbatim). */
int gc_mask_mul_f32(const float* dY, int64_t lddy, const float* mask, int64_t ldm,
                    float* G, int64_t ldg, int64_t M, int64_t N, void* stream);
/* out = in^T : in is M x N (ldin), out is N x M (ldout). */
int gc_transpose_f32(const float* in, int64_t ldin, float* out, int64_t ldout,
                     int64_t M, int64_t N, void* stream);

/* ---- classification tail (reference tests/gcn/graphcuda_impl.py:24,55) ---- */

/*
 * loss = scale * sum over rows r with row_mask[r] != 0 (all rows when row_mask
 * is null) of -log_softmax(Z[r, :])[labels[r]]: torch.log_softmax followed by
 * F.nll_loss on the masked rows as the reference's script computes them
 * (scale = 1 / number of selected rows gives reduction='mean').  The
 * workspace (gc_nll_workspace_bytes(M)) keeps the per-row logsumexp for the
 * backward call.  loss: one device float.
 */
size_t gc_nll_workspace_bytes(int64_t M);
int gc_logsoftmax_nll_forward_f32(const float* Z, int64_t ldz, const int64_t* labels, const uint8_t* row_mask,
                                  int64_t M, int64_t C, float scale, float* loss,
                                  void* workspace, size_t workspace_bytes, void* stream);
/* dZ = grad_loss * scale * (softmax(Z) - onehot(labels)) on selected rows, 0
 * elsewhere; grad_loss is one device float (null: 1). */
int gc_logsoftmax_nll_backward_f32(const float* Z, int64_t ldz, const int64_t* labels, const uint8_t* row_mask,
                                   int64_t M, int64_t C, float scale, const float* grad_loss,
                                   float* dZ, int64_t lddz, const void* workspace, void* stream);

/*
 * Evaluation tail of the reference's script (tests/gcn/graphcuda_impl.py:63-68:
 * out.argmax(dim=1), then (pred[mask] == y[mask]).sum() / mask.sum() for the
 * train / validation / test selections) in one pass over Z.
 * pred (int64[M], may be null): index of the row maximum, the lowest index
 * among equal maxima (argmax of log_softmax(Z) and of Z coincide, so the
 * logits can be passed as they are).
 * With labels: counts[2 m] = selected rows of selection m predicted right,
 * counts[2 m + 1] = rows selection m holds; masks is n_masks x M bytes
 * (row-major, non-zero = selected), n_masks <= 8; masks null = one selection
 * of all rows.  counts (int64[2 * max(n_masks, 1)]) is cleared by the call.
 */
int gc_argmax_accuracy_f32(const float* Z, int64_t ldz, int64_t M, int64_t C, const int64_t* labels,
                           const uint8_t* masks, int n_masks, int64_t* pred, int64_t* counts, void* stream);

/* ---- optimizer step (reference tests/gcn/graphcuda_impl.py:45,56) --------- */

/*
 * The optimizer.step() of the reference's training script for every parameter
 * tensor in one launch.  params / grads / exp_avg / exp_avg_sq and sizes are
 * HOST arrays of n_tensors (<= 32) device pointers / element counts, read
 * during the call; all tensors contiguous fp32.
 * gc_adam_step_f32: torch.optim.Adam's update (amsgrad and maximize off,
 * weight_decay added to the gradient; hyper-parameters are doubles as in
 * Python, 1 - beta and the bias corrections are formed in double and rounded
 * once).  `state` is 16 bytes of device memory,
 * zero before the first step: the step count (uint64) lives there and is
 * advanced by the kernel, so a recorded launch can be replayed.
 * gc_sgd_step_f32: p -= lr * (g + weight_decay * p), the SGD the reference's
 * script constructs (no momentum).
 */
int gc_adam_step_f32(int n_tensors, float* const* params, const float* const* grads,
                     float* const* exp_avg, float* const* exp_avg_sq, const int64_t* sizes,
                     double lr, double beta1, double beta2, double eps, double weight_decay,
                     void* state, void* stream);
int gc_sgd_step_f32(int n_tensors, float* const* params, const float* const* grads, const int64_t* sizes,
                    double lr, double weight_decay, void* stream);

/* ---- adjacency construction (reference tests/gcn/graphcuda_impl.py:27-38) - */

/*
 * Row pointer of a coalesced COO matrix: rows[nnz] sorted ascending (int64, as
 * torch's coalesce() leaves them; spmm_cusparse.cu:18,33-41) -> rowptr[M+1].
 */
int gc_coo_rows_to_rowptr(const int64_t* rows, int64_t nnz, int64_t M, int32_t* rowptr, void* stream);
/* int64 -> int32 narrowing of column indices. */
int gc_narrow_i64_i32(const int64_t* src, int32_t* dst, int64_t n, void* stream);

/*
 * Symmetric GCN normalisation of an edge list that already contains the
 * self-loops: deg[i] = number of edges whose *target* (col) is i, weights
 * w_e = deg[row]^-1/2 * deg[col]^-1/2 with IEEE-rounded 1/sqrt and products
 * (bit-identical to torch CPU pow(-0.5) and left-to-right multiplication),
 * inf -> 0 for isolated nodes.  Takes over torch_geometric's gcn_norm as
 * called at tests/gcn/graphcuda_impl.py:28.
 *   deg_scratch: N floats.  w: E floats out.
 */
int gc_gcn_norm_f32(const int64_t* row, const int64_t* col, int64_t E, int64_t N,
                    float* deg_scratch, float* w, void* stream);

/*
 * CSR from an edge list sorted by (row, col) with duplicates allowed:
 * duplicates are summed in input order (what coalesce() does,
 * tests/gcn/graphcuda_impl.py:33-38).  Two steps so the caller can size the
 * outputs: gc_csr_count_unique writes the number of distinct (row,col) pairs
 * to *nnz_out (device int64) and a head flag per edge into head[E] (int32
 * scratch holding the exclusive running count afterwards); gc_csr_fill then
 * writes rowptr[M+1], col[nnz], val[nnz].
 */
size_t gc_csr_build_workspace_bytes(int64_t E);
int gc_csr_count_unique(const int64_t* row, const int64_t* col, int64_t E,
                        int32_t* head, int64_t* nnz_out,
                        void* workspace, size_t workspace_bytes, void* stream);
int gc_csr_fill(const int64_t* row, const int64_t* col, const float* w, int64_t E, int64_t M,
                const int32_t* head, int32_t* rowptr, int32_t* csr_col, float* csr_val,
                void* stream);

/* 1 written to *out (device int32) when the CSR matrix with sorted columns
 * equals its transpose bit for bit, else 0.  Decides whether the engine may
 * aggregate on the output side (the reference multiplies by A, never A^T:
 * gcn.cu:49). */
int gc_csr_is_symmetric(const int32_t* rowptr, const int32_t* col, const float* val,
                        int64_t M, int32_t* out, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* GRAPHCUDA_B200_H */

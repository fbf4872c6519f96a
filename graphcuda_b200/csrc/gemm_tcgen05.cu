// fp32-in / fp32-out GEMM on the 5th-generation tensor cores (sm_100a).
//
// C[M,N] = A[M,K] * Bt[N,K]^T with both operands K-major in shared memory,
// kind::tf32 MMAs issued by one thread per CTA, fp32 accumulators in TMEM.
// Takes over cublasSgemm as the reference wraps it
// (src/graphcuda/cuda/gemm_cublas.cu:37-48) for the large products of the GCN
// layer (src/graphcuda/cuda/gcn.cu:15,43,46).
//
// fp32 semantics on a TF32 pipe ("three-pass" mode): the tensor core reads the
// upper 19 bits of each fp32 word, so x_hi = trunc19(x) comes for free and
// x_lo = x - x_hi is exact in fp32.  D = A_lo*B_hi + A_hi*B_lo + A_hi*B_hi
// restores ~21 bits of operand precision.  B_lo (weights: small, reused by
// every tile) is produced once by a pre-pass into the workspace; A_lo is made
// on the fly by four converter warps from the tile TMA just landed, so A is
// read from HBM exactly once.
//
// CTA = 16 warps, persistent over 128 x BN output tiles:
//   warp 0        TMA producer (one lane)           full[s]  <- bytes landed
//   warp 1        MMA issuer (one lane)             empty[s] <- tcgen05.commit
//   warp 2        TMEM allocator / idle;  warp 3 idle
//   warps 4-7     epilogue group 0: tcgen05.ld -> bias/ReLU/mask/gate -> global, even 32-column chunks
//   warps 8-11    converter (three-pass mode): A tile -> A_lo tile (and B -> B_lo)    conv[s]
//   warps 12-15   epilogue group 1: the odd 32-column chunks
// Two TMEM accumulators (2 x BN columns) let the epilogue of tile i overlap
// the main loop of tile i+1.
//
// Every wait is bounded: a wait that runs out raises a CTA-wide abort flag and
// a word in global memory, all roles leave their loops, outstanding TMA
// copies are drained (bounded) and TMEM is released before the CTA exits.
#include "common.cuh"
#include "gemm_internal.cuh"

#include <cuda.h>

namespace {

constexpr int BM = 128;
// K extent of a stage: 32 fp32 (128-byte rows, 128-byte swizzle) or, where
// that leaves only two stages of shared memory, 16 fp32 (64-byte rows,
// 64-byte swizzle) for twice as many stages in flight.
template <int BN, int PASSES>
constexpr int block_k() { return (PASSES == 3 && BN == 256) ? 16 : 32; }
constexpr int UMMA_K = 8;   // K of one kind::tf32 instruction
constexpr int kThreads = 512;  // 16 warps: producer, MMA issuer, TMEM allocator, idle | 4 epilogue | 4 converter | 4 epilogue
constexpr uint32_t kWaitLimit = 1u << 24;

// ------------------------------------------------------------------ PTX
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait.  Returns false when the CTA is aborting (this wait or another
// ran out).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_s) {
  for (uint32_t i = 0; i < kWaitLimit; ++i) {
    if (mbar_test(bar, parity)) return true;
    if (i > 128) {
      __nanosleep(64);
      if (*abort_s) return false;
    }
  }
  *abort_s = 1;
  return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void umma_tf32(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// kind::f16 with bf16 operands (K = 16 per instruction: the same 32 bytes of every row as one kind::tf32 step)
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Shared-memory matrix descriptors (version 1 = sm_100).  Tiles are rows of
// 128 bytes as TMA writes them:
//  * K-major operand (layout type 2, SWIZZLE_128B, 16-byte atoms): a row is 32
//    consecutive K values of one M/N index; 8-row groups follow each other
//    every 1024 bytes (stride byte offset); one MMA (K = 8) reads 32 bytes of
//    every row, so successive k-steps advance the start address by 32 bytes.
//  * MN-major operand (layout type 1, SWIZZLE_128B with 32-byte atoms -- the
//    only swizzle kind::tf32 accepts for transposed 32-bit operands; with the
//    16-byte-atom swizzle or no swizzle the MMA returns zeros): a row is 32
//    consecutive M/N values at one k; the 32-byte unit index is XORed with
//    k % 4; groups of 4 k-rows are 512 bytes apart (stride byte offset) and
//    32-column chunks `mn_chunk` bytes apart (leading byte offset); one MMA
//    reads 8 k-rows = 1024 bytes, the advance per k-step.
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes,
                                              uint32_t layout_type) {
  uint64_t d = 0;
  d |= uint64_t((saddr & 0x3FFFFu) >> 4);
  d |= uint64_t((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= uint64_t((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= uint64_t(1) << 46;
  d |= uint64_t(layout_type) << 61;
  return d;
}
// K-major tiles with 16 fp32 per row use the 64-byte swizzle (layout type 4):
// 8-row groups are 512 bytes apart.
template <int BK>
__device__ __forceinline__ uint64_t smem_desc_operand(uint32_t saddr, bool mn_major, uint32_t mn_chunk) {
  if (mn_major) return smem_desc(saddr, mn_chunk, 512u, 1u);
  return BK == 32 ? smem_desc(saddr, 0u, 1024u, 2u) : smem_desc(saddr, 0u, 512u, 4u);
}

// Instruction descriptor for kind::tf32 with fp32 accumulation.
__host__ __device__ constexpr uint32_t make_idesc(int bn, bool a_mn, bool b_mn) {
  return (1u << 4)                      // D format: F32
         | (2u << 7)                    // A format: TF32
         | (2u << 10)                   // B format: TF32
         | (uint32_t(a_mn ? 1 : 0) << 15)  // A major: 0 = K, 1 = MN
         | (uint32_t(b_mn ? 1 : 0) << 16)  // B major
         | (uint32_t(bn >> 3) << 17)    // N / 8
         | (uint32_t(BM >> 4) << 24);   // M / 16
}

// Instruction descriptor for kind::f16 with bf16 operands (both K-major) and fp32 accumulation.
__host__ __device__ constexpr uint32_t make_idesc_bf16(int bn) {
  return (1u << 4)                     // D format: F32
         | (1u << 7)                   // A format: BF16
         | (1u << 10)                  // B format: BF16
         | (uint32_t(bn >> 3) << 17)   // N / 8
         | (uint32_t(BM >> 4) << 24);  // M / 16
}

struct TcParams {
  int M, N, K;
  float* C;
  int64_t ldc;
  gc::GemmEpilogue ep;
  int* flag;       // global word set when a wait ran out
  int vec_store;   // rows of C are 16-byte aligned
  int splits;      // > 1: K is cut into `splits` ranges of kb_per_split k-blocks,
  int kb_per_split;  //    raw partial tiles go to partial[split][M][N]
  float* partial;
};

template <int BN, int PASSES>
struct Cfg {
  static constexpr int BK = block_k<BN, PASSES>();
  static constexpr int kABytes = BM * BK * 4;
  static constexpr int kBBytes = BN * BK * 4;
  static constexpr int kStageBytes = (PASSES == 3 ? 2 : 1) * (kABytes + kBBytes);
  static constexpr int kStages = (200 * 1024 / kStageBytes) > 8 ? 8 : (200 * 1024 / kStageBytes);
  static constexpr int kStagingBytes = 8 * 32 * 32 * 4;  // one 32 x 32 fp32 tile per epilogue warp
  static constexpr int kSmemBytes =
      kStages * kStageBytes + 1024 /*alignment slack*/ + 256 /*barriers*/ + kStagingBytes;
  static_assert(kSmemBytes <= 227 * 1024, "shared memory budget");
  static constexpr uint32_t kTmemCols = 2 * BN < 32 ? 32 : 2 * BN;
  static_assert(kStages >= 2, "need at least two stages");
};

// A_MN / B_MN: the operand is MN-major in global memory (A stored K x M,
// B stored K x N) and is staged MN-major, 32 columns per TMA box.
// CONV_B: B_lo is produced in shared memory by the converter warps like A_lo
// (large B operands: activations, gradients); otherwise it is loaded from a
// pre-split copy (weights).
// BF16: the operands are bf16 matrices (K-major, 64 elements = 128 bytes per row of a stage), one kind::f16
// MMA per 32-byte step; everything else -- pipeline, TMEM, epilogue -- is the single-pass fp32 kernel.
template <int BN, int PASSES, bool A_MN, bool B_MN, bool CONV_B, bool BF16 = false>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tf32_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
                 const __grid_constant__ CUtensorMap mapBlo, TcParams p) {
  using C_ = Cfg<BN, PASSES>;
  constexpr int S = C_::kStages;
  constexpr int BK = C_::BK;
  constexpr int KE = BF16 ? 2 * BK : BK;  // K elements per stage (a stage row is BK * 4 bytes either way)
  static_assert(!BF16 || (PASSES == 1 && !A_MN && !B_MN), "bf16 operands are K-major, one pass");
  constexpr bool kConvB = CONV_B && PASSES == 3;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw);
  // stage layout: [A | B | A_lo | B_lo]
  auto sA = [&](int s) { return base + s * C_::kStageBytes; };
  auto sB = [&](int s) { return base + s * C_::kStageBytes + C_::kABytes; };
  auto sAlo = [&](int s) { return base + s * C_::kStageBytes + C_::kABytes + C_::kBBytes; };
  auto sBlo = [&](int s) { return base + s * C_::kStageBytes + 2 * C_::kABytes + C_::kBBytes; };
  const uint32_t bars = base + S * C_::kStageBytes;
  auto bar_full = [&](int s) { return bars + 8 * s; };
  auto bar_empty = [&](int s) { return bars + 8 * (S + s); };
  auto bar_conv = [&](int s) { return bars + 8 * (2 * S + s); };
  auto bar_tfull = [&](int b) { return bars + 8 * (3 * S + b); };
  auto bar_tempty = [&](int b) { return bars + 8 * (3 * S + 2 + b); };
  float* stage_tiles = reinterpret_cast<float*>(smem + S * C_::kStageBytes + 256);
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_s;

  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int tiles_n = (p.N + BN - 1) / BN;
  const int tiles_m = (p.M + BM - 1) / BM;
  const int nkb_total = (p.K + KE - 1) / KE;
  const int splits = p.splits > 1 ? p.splits : 1;
  const int kb_per = splits > 1 ? p.kb_per_split : nkb_total;
  // work item = (split, m tile, n tile), n fastest
  const int num_items = tiles_m * tiles_n * splits;
  auto item_coords = [&](int item, int& m0, int& n0, int& kb0, int& kb1, int& split) {
    const int t = item % (tiles_m * tiles_n);
    split = item / (tiles_m * tiles_n);
    m0 = (t / tiles_n) * BM;
    n0 = (t % tiles_n) * BN;
    kb0 = split * kb_per;
    kb1 = min(nkb_total, kb0 + kb_per);
  };

  if (threadIdx.x == 0) {
    abort_s = 0;
    for (int s = 0; s < S; ++s) {
      mbar_init(bar_full(s), 1);
      mbar_init(bar_empty(s), 1);
      mbar_init(bar_conv(s), 4);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_tfull(b), 1);
      mbar_init(bar_tempty(b), 8);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_async_smem();
  }
  if (warp == 2) tmem_alloc(smem_u32(&tmem_base_s), C_::kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_s;
  volatile int* abort_p = &abort_s;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      constexpr uint32_t kTx = C_::kABytes + ((PASSES == 3 && !kConvB) ? 2 : 1) * C_::kBBytes;
      for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x) {
        int m0, n0, kb0, kb1, split;
        item_coords(item, m0, n0, kb0, kb1, split);
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % S;
          const uint32_t ph = (it / S) & 1u;
          if (!mbar_wait(bar_empty(s), ph ^ 1u, abort_p)) { ok = false; break; }
          mbar_expect_tx(bar_full(s), kTx);
          if (A_MN) {
#pragma unroll
            for (int c = 0; c < BM / 32; ++c)
              tma_load_2d(sA(s) + c * (BK * 128), &mapA, m0 + c * 32, kb * BK, bar_full(s));
          } else {
            tma_load_2d(sA(s), &mapA, kb * KE, m0, bar_full(s));
          }
          if (B_MN) {
#pragma unroll
            for (int c = 0; c < BN / 32; ++c)
              tma_load_2d(sB(s) + c * (BK * 128), &mapB, n0 + c * 32, kb * BK, bar_full(s));
          } else {
            tma_load_2d(sB(s), &mapB, kb * KE, n0, bar_full(s));
            if (PASSES == 3 && !kConvB) tma_load_2d(sBlo(s), &mapBlo, kb * BK, n0, bar_full(s));
          }
        }
      }
      // Drain: every copy issued must have landed before the CTA may exit.
      // `it` stages were issued; the last min(S, it) of them may be in flight.
      const uint32_t pending = it < uint32_t(S) ? it : uint32_t(S);
      for (uint32_t j = 0; j < pending; ++j) {
        const uint32_t q = it - 1 - j;
        const uint32_t bar = bar_full(q % S), par = (q / S) & 1u;
        for (uint32_t i = 0; i < kWaitLimit; ++i) {
          if (mbar_test(bar, par)) break;
          __nanosleep(64);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = BF16 ? make_idesc_bf16(BN) : make_idesc(BN, A_MN, B_MN);
      constexpr uint32_t kMnLbo = BK * 128;  // bytes between 32-column chunks of an MN-major tile
      constexpr uint32_t kAStep = A_MN ? 1024u : uint32_t(UMMA_K * 4);  // start-address advance per k-step
      constexpr uint32_t kBStep = B_MN ? 1024u : uint32_t(UMMA_K * 4);
      uint32_t it = 0, tcount = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x, ++tcount) {
        int m0, n0, kb0, kb1, split;
        item_coords(item, m0, n0, kb0, kb1, split);
        const int b = tcount & 1;
        const uint32_t bph = (tcount >> 1) & 1u;
        if (!mbar_wait(bar_tempty(b), bph ^ 1u, abort_p)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + uint32_t(b * BN);
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % S;
          const uint32_t ph = (it / S) & 1u;
          if (!mbar_wait(bar_full(s), ph, abort_p)) { ok = false; break; }
          if (PASSES == 3 && !mbar_wait(bar_conv(s), ph, abort_p)) { ok = false; break; }
          tc_fence_after();
          const uint64_t da = smem_desc_operand<BK>(sA(s), A_MN, kMnLbo);
          const uint64_t db = smem_desc_operand<BK>(sB(s), B_MN, kMnLbo);
          const uint64_t dal = smem_desc_operand<BK>(sAlo(s), A_MN, kMnLbo);
          const uint64_t dbl = smem_desc_operand<BK>(sBlo(s), B_MN, kMnLbo);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t aa = uint64_t((k * kAStep) >> 4);  // byte offset >> 4 into the address field
            const uint64_t ab = uint64_t((k * kBStep) >> 4);
            const uint32_t acc = (kb > kb0 || k > 0) ? 1u : 0u;
            if (PASSES == 3) {
              umma_tf32(d_tmem, dal + aa, db + ab, idesc, acc);
              umma_tf32(d_tmem, da + aa, dbl + ab, idesc, 1u);
              umma_tf32(d_tmem, da + aa, db + ab, idesc, 1u);
            } else if (BF16) {
              umma_bf16(d_tmem, da + aa, db + ab, idesc, acc);
            } else {
              umma_tf32(d_tmem, da + aa, db + ab, idesc, acc);
            }
          }
          umma_commit(bar_empty(s));  // frees the stage once these MMAs have read it
        }
        if (ok) umma_commit(bar_tfull(b));
      }
    }
  } else if ((warp >= 4 && warp < 8) || warp >= 12) {
    // ------------------------------------------------------------ epilogue
    // Two warps per TMEM lane quarter (a warp may only read lanes 32 * (warp % 4) ...): group 0 takes the even
    // 32-column chunks of a tile, group 1 the odd ones.  A single warp per scheduler left the epilogue bound by
    // the latency of its own dependent instructions (about 0.8 us per chunk whatever the chunk did).
    const int q = warp % 4;             // TMEM lane quarter
    const int grp = warp >= 12 ? 1 : 0;  // chunk parity
    uint32_t tcount = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x, ++tcount) {
      int m0, n0, kb0, kb1, split;
      item_coords(item, m0, n0, kb0, kb1, split);
      const int b = tcount & 1;
      const uint32_t bph = (tcount >> 1) & 1u;
      if (!mbar_wait(bar_tfull(b), bph, abort_p)) { ok = false; break; }
      tc_fence_after();
      const int gm = m0 + q * 32 + lane;
      const uint32_t taddr = tmem_base + (uint32_t(q * 32) << 16) + uint32_t(b * BN);
      // split-K: raw partial tile, row-major M x N, no epilogue
      const bool raw_out = splits > 1;
      float* Cb = raw_out ? p.partial + int64_t(split) * p.M * p.N : p.C;
      const int64_t ldc = raw_out ? int64_t(p.N) : p.ldc;
      gc::GemmEpilogue ep = p.ep;
      if (raw_out) ep = gc::GemmEpilogue{nullptr, nullptr, nullptr, 0, 0};
      const bool vec = raw_out ? (p.N % 4 == 0) : (p.vec_store != 0);
      // Gate values of the NEXT tile of this CTA are requested into the L2 now, a whole tile time before the
      // epilogue reads them (they come from DRAM: 128 KB per tile, read once).
      if (ep.gate && item + int(gridDim.x) < num_items) {
        int nm0, nn0, nk0, nk1, nsplit;
        item_coords(item + int(gridDim.x), nm0, nn0, nk0, nk1, nsplit);
        const int prow = nm0 + q * 32 + lane;
        if (prow < p.M) {
          const char* g = reinterpret_cast<const char*>(ep.gate + int64_t(prow) * ldc + nn0);
          const int bytes = min(BN, p.N - nn0) * 4;
          for (int off = grp * 128; off < bytes; off += 256) asm volatile("prefetch.global.L2 [%0];" ::"l"(g + off));
        }
      }
      // Row r of the 32 x 32 block a warp stores in one pass: lanes 8k..8k+7 cover the 128 bytes of row 4*pass + k.
      const int c4 = (lane % 8) * 4;
      const int row_in_quarter = lane / 8;
      const int64_t row0_off = int64_t(m0 + q * 32 + row_in_quarter) * ldc + c4;  // element offset of pass 0
      const int rows_left = p.M - (m0 + q * 32 + row_in_quarter);                // pass valid iff 4 * pass < rows_left
      float4* tile4 = reinterpret_cast<float4*>(stage_tiles + (grp * 4 + q) * (32 * 32));
      uint32_t r[32];
      tmem_ld32(taddr + uint32_t(grp * 32), r);
      tmem_ld_wait();
#pragma unroll 1
      for (int c = grp; c < BN / 32; c += 2) {
        const int gn0 = n0 + c * 32;
        if (gn0 >= p.N) break;  // uniform across the warp; nothing is in flight here
        const bool have_next = c + 2 < BN / 32;
        if (ep.transposed) {
          // lanes hold consecutive m: a column of C is a contiguous run of C^T
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int gn = gn0 + j;
            if (gn < p.N && gm < p.M) gc::epilogue_store(__uint_as_float(r[j]), gm, gn, Cb, ldc, ep);
          }
          if (have_next) tmem_ld32(taddr + uint32_t((c + 2) * 32), r);
        } else if (vec && gn0 + 32 <= p.N) {
          // The accumulator arrives one row per lane.  Stored like that, every 128-bit store of the warp would
          // touch 32 different lines.  The 32 x 32 block is turned through shared memory -- 128-bit accesses both
          // ways, the 16-byte chunk index XORed with the row so that neither direction has bank conflicts -- and
          // every store instruction covers four complete 128-byte row segments.  The TMEM load of the next 32
          // columns and the gate values of this block are in flight while the block is turned.
          float4 gv[8];
          if (ep.gate) {
#pragma unroll
            for (int pass = 0; pass < 8; ++pass)
              gv[pass] = 4 * pass < rows_left
                             ? __ldcs(reinterpret_cast<const float4*>(ep.gate + row0_off + int64_t(4 * pass) * ldc + gn0))
                             : make_float4(0.f, 0.f, 0.f, 0.f);
          }
#pragma unroll
          for (int j4 = 0; j4 < 8; ++j4)
            tile4[lane * 8 + (j4 ^ (lane & 7))] =
                make_float4(__uint_as_float(r[4 * j4]), __uint_as_float(r[4 * j4 + 1]), __uint_as_float(r[4 * j4 + 2]),
                            __uint_as_float(r[4 * j4 + 3]));
          if (have_next) tmem_ld32(taddr + uint32_t((c + 2) * 32), r);
          __syncwarp();
          float4 bv = make_float4(0.f, 0.f, 0.f, 0.f);
          if (ep.bias) bv = __ldg(reinterpret_cast<const float4*>(ep.bias + gn0 + c4));
#pragma unroll
          for (int pass = 0; pass < 8; ++pass) {
            const int row = pass * 4 + row_in_quarter;
            float4 v = tile4[row * 8 + ((lane & 7) ^ (row & 7))];
            if (4 * pass < rows_left) {
              const int64_t off = row0_off + int64_t(4 * pass) * ldc + gn0;
              v.x += bv.x; v.y += bv.y; v.z += bv.z; v.w += bv.w;
              if (ep.relu || ep.mask) {
                const float4 mk = make_float4(v.x > 0.f ? 1.f : 0.f, v.y > 0.f ? 1.f : 0.f, v.z > 0.f ? 1.f : 0.f,
                                              v.w > 0.f ? 1.f : 0.f);
                if (ep.mask) *reinterpret_cast<float4*>(ep.mask + off) = mk;
                if (ep.relu) { v.x *= mk.x; v.y *= mk.y; v.z *= mk.z; v.w *= mk.w; }
              }
              if (ep.gate) {
                v.x *= gv[pass].x > 0.f ? 1.f : 0.f; v.y *= gv[pass].y > 0.f ? 1.f : 0.f;
                v.z *= gv[pass].z > 0.f ? 1.f : 0.f; v.w *= gv[pass].w > 0.f ? 1.f : 0.f;
              }
              *reinterpret_cast<float4*>(Cb + off) = v;
            }
          }
          __syncwarp();
        } else {
          if (gm < p.M) {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const int gn = gn0 + j;
              if (gn < p.N) gc::epilogue_store(__uint_as_float(r[j]), gm, gn, Cb, ldc, ep);
            }
          }
          if (have_next) tmem_ld32(taddr + uint32_t((c + 2) * 32), r);
        }
        if (have_next) tmem_ld_wait();
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_tempty(b));
    }
  } else if (warp >= 8 && PASSES == 3) {
    // ------------------------------------------------------------ converter
    const int ct = threadIdx.x - 256;  // 0..127
    constexpr int kVecs = (C_::kABytes + (kConvB ? C_::kBBytes : 0)) / 16;  // A (and B) are contiguous in a stage
    uint32_t it = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x) {
      int m0, n0, kb0, kb1, split;
      item_coords(item, m0, n0, kb0, kb1, split);
      for (int kb = kb0; kb < kb1; ++kb, ++it) {
        const int s = it % S;
        const uint32_t ph = (it / S) & 1u;
        if (!mbar_wait(bar_full(s), ph, abort_p)) { ok = false; break; }
        const float4* src = reinterpret_cast<const float4*>(smem + s * C_::kStageBytes);
        float4* dst = reinterpret_cast<float4*>(smem + s * C_::kStageBytes + C_::kABytes + C_::kBBytes);
#pragma unroll 8
        for (int i = ct; i < kVecs; i += 128) {
          const float4 v = src[i];
          float4 lo;
          lo.x = v.x - __uint_as_float(__float_as_uint(v.x) & 0xFFFFE000u);
          lo.y = v.y - __uint_as_float(__float_as_uint(v.y) & 0xFFFFE000u);
          lo.z = v.z - __uint_as_float(__float_as_uint(v.z) & 0xFFFFE000u);
          lo.w = v.w - __uint_as_float(__float_as_uint(v.w) & 0xFFFFE000u);
          dst[i] = lo;
        }
        fence_async_smem();  // generic-proxy writes -> visible to the tensor core's async-proxy reads
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_conv(s));
      }
    }
  }

  // ---------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 2) tmem_dealloc(tmem_base, C_::kTmemCols);
  if (threadIdx.x == 0 && abort_s && p.flag) atomicExch(p.flag, 1);
}

// B_lo = B - trunc19(B) over an R x Kc view.
__global__ void __launch_bounds__(256)
split_lo_kernel(const float* __restrict__ src, int64_t lds, float* __restrict__ dst, int64_t ldd, int R, int Kc) {
  const int64_t total = int64_t(R) * Kc;
  for (int64_t i = int64_t(blockIdx.x) * 256 + threadIdx.x; i < total; i += int64_t(gridDim.x) * 256) {
    const int r = int(i / Kc), k = int(i % Kc);
    const float v = __ldg(src + int64_t(r) * lds + k);
    dst[int64_t(r) * ldd + k] = v - __uint_as_float(__float_as_uint(v) & 0xFFFFE000u);
  }
}

// out[c][r] = in[r][c] through a 32 x 33 shared tile.
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

// C = sum over splits of partial[split], then the epilogue.  The order of the additions is fixed (eight
// contiguous groups of splits summed in split order by eight warps, the eight group sums added in group order), so
// the result is the same run to run; the groups run side by side because a capped-chain product has a thousand
// partial tiles and one thread per element walking them all was latency-bound (0.22 ms for a 100 x 256 result).
__global__ void __launch_bounds__(256)
tc_splitk_reduce_kernel(int M, int N, int splits, const float* __restrict__ partial, float* __restrict__ C,
                        int64_t ldc, gc::GemmEpilogue ep) {
  __shared__ float sm[8][32];
  const int e = threadIdx.x % 32, g = threadIdx.x / 32;
  const int64_t total = int64_t(M) * N;
  const int per = (splits + 7) / 8;
  const int z0 = g * per, z1 = min(splits, z0 + per);
  for (int64_t base = int64_t(blockIdx.x) * 32; base < total; base += int64_t(gridDim.x) * 32) {
    const int64_t i = base + e;
    float s = 0.f;
    if (i < total) {
      int z = z0;
      for (; z + 4 <= z1; z += 4) {
        const float a = partial[int64_t(z) * total + i], b = partial[int64_t(z + 1) * total + i],
                    c = partial[int64_t(z + 2) * total + i], d = partial[int64_t(z + 3) * total + i];
        s = (((s + a) + b) + c) + d;
      }
      for (; z < z1; ++z) s += partial[int64_t(z) * total + i];
    }
    sm[g][e] = s;
    __syncthreads();
    if (g == 0 && i < total) {
      float t = sm[0][e];
#pragma unroll
      for (int k = 1; k < 8; ++k) t += sm[k][e];
      gc::epilogue_store(t, int(i / N), int(i % N), C, ldc, ep);
    }
    __syncthreads();
  }
}

// dst (bf16, R x Cc, pitch ldd) = src (fp32): as stored (transpose == 0: src is R x Cc) or transposed
// (src is Cc x R).  Round to nearest even, as __float2bfloat16_rn does.
__device__ __forceinline__ uint16_t to_bf16(float v) {
  uint32_t u = __float_as_uint(v);
  if ((u & 0x7F800000u) == 0x7F800000u) return uint16_t((u >> 16) | ((u & 0xFFFFu) ? 0x40u : 0u));  // inf / nan
  return uint16_t((u + 0x7FFFu + ((u >> 16) & 1u)) >> 16);
}
__global__ void __launch_bounds__(256)
cvt_bf16_kernel(const float* __restrict__ src, int64_t lds, uint16_t* __restrict__ dst, int64_t ldd, int R, int Cc) {
  // pairs of columns per thread; the pad columns [Cc, ldd) are zero-filled so that a K pitch rounded up to 8 holds zeros
  const int64_t pairs_per_row = ldd / 2;
  const int64_t total = int64_t(R) * pairs_per_row;
  for (int64_t i = int64_t(blockIdx.x) * 256 + threadIdx.x; i < total; i += int64_t(gridDim.x) * 256) {
    const int r = int(i / pairs_per_row), c = int(i % pairs_per_row) * 2;
    const float a = c < Cc ? __ldg(src + int64_t(r) * lds + c) : 0.f;
    const float b = c + 1 < Cc ? __ldg(src + int64_t(r) * lds + c + 1) : 0.f;
    reinterpret_cast<uint32_t*>(dst + int64_t(r) * ldd)[c / 2] = uint32_t(to_bf16(a)) | (uint32_t(to_bf16(b)) << 16);
  }
}
// The same for 16-byte aligned rows: eight elements per thread (two 128-bit loads, one 128-bit store).
__global__ void __launch_bounds__(256)
cvt_bf16_vec8_kernel(const float* __restrict__ src, int64_t lds, uint16_t* __restrict__ dst, int64_t ldd, int R, int Cc) {
  const int64_t oct_per_row = ldd / 8;
  const int64_t total = int64_t(R) * oct_per_row;
  for (int64_t i = int64_t(blockIdx.x) * 256 + threadIdx.x; i < total; i += int64_t(gridDim.x) * 256) {
    const int r = int(i / oct_per_row), c = int(i % oct_per_row) * 8;
    const float* p = src + int64_t(r) * lds + c;
    float v[8];
    if (c + 8 <= Cc) {
      const float4 a = __ldcs(reinterpret_cast<const float4*>(p)), b = __ldcs(reinterpret_cast<const float4*>(p + 4));
      v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    } else {
#pragma unroll
      for (int k = 0; k < 8; ++k) v[k] = c + k < Cc ? __ldg(p + k) : 0.f;
    }
    uint4 o;
    o.x = uint32_t(to_bf16(v[0])) | (uint32_t(to_bf16(v[1])) << 16);
    o.y = uint32_t(to_bf16(v[2])) | (uint32_t(to_bf16(v[3])) << 16);
    o.z = uint32_t(to_bf16(v[4])) | (uint32_t(to_bf16(v[5])) << 16);
    o.w = uint32_t(to_bf16(v[6])) | (uint32_t(to_bf16(v[7])) << 16);
    *reinterpret_cast<uint4*>(dst + int64_t(r) * ldd + c) = o;
  }
}
__global__ void __launch_bounds__(256)
cvt_transpose_bf16_kernel(const float* __restrict__ in, int64_t ldin, uint16_t* __restrict__ out, int64_t ldout, int R,
                          int Cc) {
  // in is R x Cc (fp32), out is Cc x R (bf16, pitch ldout >= R, pad columns zero-filled), 32 x 32 tiles
  __shared__ float t[32][33];
  const int tx = threadIdx.x % 32, ty = threadIdx.x / 32;
  const int64_t tiles_r = (ldout + 31) / 32;  // cover the padded pitch so the pad is written
  const int64_t tiles_c = (Cc + 31) / 32;
  const int64_t tiles = tiles_r * tiles_c;
  for (int64_t tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
    const int r0 = int(tile / tiles_c) * 32, c0 = int(tile % tiles_c) * 32;
    for (int i = ty; i < 32; i += 8)
      t[i][tx] = (r0 + i < R && c0 + tx < Cc) ? __ldg(in + int64_t(r0 + i) * ldin + c0 + tx) : 0.f;
    __syncthreads();
    for (int i = ty; i < 32; i += 8)
      if (c0 + i < Cc && r0 + tx < ldout) out[int64_t(c0 + i) * ldout + r0 + tx] = to_bf16(t[tx][i]);
    __syncthreads();
  }
}

// ------------------------------------------------------------------ host
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn get_encode() {
  static EncodeFn fn = [] {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      f = nullptr;
    return reinterpret_cast<EncodeFn>(f);
  }();
  return fn;
}

// Tensor map over a row-major fp32 matrix of `rows` rows and `cols` columns
// (row pitch ld): box = 32 columns (128 bytes, the swizzle span) x box_rows.
// K-major operands pass (rows = M or N, cols = K) and take the 16-byte-atom
// 128-byte swizzle; MN-major operands pass (rows = K, cols = M or N) and take
// the 32-byte-atom one.
int make_map(CUtensorMap* map, const float* ptr, int64_t rows, int64_t cols, int64_t ld, int box_rows,
             bool mn_major, int bk) {
  EncodeFn enc = get_encode();
  if (!enc) return gc::fail(GC_ERR_CUDA, "cuTensorMapEncodeTiled entry point not available");
  cuuint64_t dims[2] = {cuuint64_t(cols), cuuint64_t(rows)};
  cuuint64_t strides[1] = {cuuint64_t(ld) * 4};
  // MN-major: 32 columns (128 bytes) x bk rows; K-major: bk columns x box_rows rows
  cuuint32_t box[2] = {mn_major ? 32u : cuuint32_t(bk), cuuint32_t(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(ptr), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE,
                   mn_major ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B
                            : (bk == 32 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B),
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return gc::fail(GC_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", int(r));
  return GC_OK;
}

// Tensor map over a row-major bf16 matrix (rows x cols, pitch ld elements): box = 64 columns (128 bytes) x box_rows.
int make_map_bf16(CUtensorMap* map, const uint16_t* ptr, int64_t rows, int64_t cols, int64_t ld, int box_rows) {
  EncodeFn enc = get_encode();
  if (!enc) return gc::fail(GC_ERR_CUDA, "cuTensorMapEncodeTiled entry point not available");
  cuuint64_t dims[2] = {cuuint64_t(cols), cuuint64_t(rows)};
  cuuint64_t strides[1] = {cuuint64_t(ld) * 2};
  cuuint32_t box[2] = {64u, cuuint32_t(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<uint16_t*>(ptr), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return gc::fail(GC_ERR_CUDA, "cuTensorMapEncodeTiled (bf16) failed with CUresult %d", int(r));
  return GC_OK;
}

inline int64_t round4(int64_t x) { return (x + 3) & ~int64_t(3); }
inline int64_t round8(int64_t x) { return (x + 7) & ~int64_t(7); }
inline size_t align256(size_t x) { return (x + 255) & ~size_t(255); }

int pick_bn(int64_t N) {
  if (N <= 64) return 64;
  if (N <= 128) return 128;
  const int64_t rem = N % 256;
  return (rem == 0 || rem > 128) ? 256 : 128;
}

// B operands up to this many elements (weights) are re-laid K-major and
// pre-split once per call; larger ones are consumed in place.
constexpr int64_t kSmallB = int64_t(1) << 21;
constexpr int64_t kMaxChainK = 2048;  // longest fp32-semantics accumulation chain where K is split (see make_plan)

struct Plan {
  bool transpose_a;  // A given K x M, re-laid M x K in the workspace
  bool a_mn;         // A consumed MN-major in place
  bool transpose_b;  // B given K x N, re-laid N x K in the workspace
  bool b_mn;         // B consumed MN-major in place
  bool conv_b;       // B_lo made in shared memory (else pre-split into the workspace)
  int bn;
  int splits, kb_per_split;
};

Plan make_plan(bool ta, bool tb, int64_t M, int64_t N, int64_t K, int passes) {
  Plan pl{};
  pl.bn = pick_bn(N);
  const bool small_b = N * K <= kSmallB;
  if (ta) {
    // weight-gradient form: consume A in place; B in place too unless it is a small N x K matrix
    pl.a_mn = true;
  }
  if (!tb) {
    if (small_b && !ta) pl.transpose_b = true;
    else pl.b_mn = true;
  }
  // the MN-major kernel variant is instantiated for (A_MN, B_MN) = (1,1) and (0,1); (1,0) re-lays A
  if (pl.a_mn && !pl.b_mn) {
    pl.a_mn = false;
    pl.transpose_a = true;
  }
  // Pre-splitting B (weights) costs a second tile load per stage; making B_lo in shared memory costs converter
  // time.  In-kernel wins while the tile's MMA work is small.  Measured on 1.2 M-row operands, in shared memory
  // against pre-split: K x BN = 100 x 256 0.48 / 0.63 ms, 128 x 256 0.50 / 0.48 ms, 256 x 128 0.58 / 0.48 ms,
  // 256 x 256 0.80 / 0.81 ms, 256 x 64 and 48 x 256 equal.
  pl.conv_b = pl.b_mn || !(small_b) || (K * pl.bn < 128 * 256);
  if (passes != 3) pl.conv_b = pl.b_mn;  // selects the template only
  const int64_t tiles = gc::ceil_div(M, BM) * gc::ceil_div(N, pl.bn);
  const int bk = (passes == 3 && pl.bn == 256) ? 16 : 32;
  const int64_t nkb = gc::ceil_div(K, bk);
  int64_t splits = 1;
  if (tiles * 2 <= gc::kNumSMs && nkb >= 64) splits = std::min<int64_t>(gc::kNumSMs / tiles, nkb / 16);
  splits = std::max<int64_t>(1, splits);
  pl.kb_per_split = int(gc::ceil_div(nkb, splits));
  // The tensor core adds into its fp32 accumulator by truncation, not rounding: the error of a sum grows in
  // proportion to the length of the accumulation chain (measured against float64 on a 2.4 M-long weight-gradient
  // sum, three-pass mode: 1.2e-4 relative at 16.5 K elements per chain, 2.9e-5 at 4096, 1.5e-5 at 2048, 7.5e-6 at
  // 1024).  Where K is split anyway, fp32-semantics chains are therefore kept to kMaxChainK elements; the partial
  // tiles are then added by CUDA cores in a fixed order (+0.27 ms on that product).  The 1e-2 tiers keep long chains.
  if (passes == 3 && splits > 1)
    pl.kb_per_split = int(std::max<int64_t>(1, std::min<int64_t>(pl.kb_per_split, kMaxChainK / bk)));
  pl.splits = int(gc::ceil_div(nkb, pl.kb_per_split));
  return pl;
}

template <int BN, int PASSES, bool A_MN, bool B_MN, bool CONV_B>
int launch_tc(const CUtensorMap& mA, const CUtensorMap& mB, const CUtensorMap& mBlo, const TcParams& p,
              cudaStream_t st) {
  using C_ = Cfg<BN, PASSES>;
  auto kern = gemm_tf32_kernel<BN, PASSES, A_MN, B_MN, CONV_B>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C_::kSmemBytes);
  if (e != cudaSuccess) return gc::fail(GC_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
  const int64_t items = gc::ceil_div(p.M, BM) * gc::ceil_div(p.N, BN) * (p.splits > 1 ? p.splits : 1);
  const unsigned grid = unsigned(std::min<int64_t>(items, gc::kNumSMs));
  kern<<<grid, kThreads, C_::kSmemBytes, st>>>(mA, mB, mBlo, p);
  return gc::check_launch("gemm_tf32_kernel");
}

template <int BN, int PASSES>
int launch_layout(const Plan& pl, const CUtensorMap& mA, const CUtensorMap& mB, const CUtensorMap& mBlo,
                  const TcParams& p, cudaStream_t st) {
  if (pl.a_mn && pl.b_mn) return launch_tc<BN, PASSES, true, true, true>(mA, mB, mBlo, p, st);
  if (pl.b_mn) return launch_tc<BN, PASSES, false, true, true>(mA, mB, mBlo, p, st);
  if (pl.conv_b && PASSES == 3) return launch_tc<BN, PASSES, false, false, true>(mA, mB, mBlo, p, st);
  return launch_tc<BN, PASSES, false, false, false>(mA, mB, mBlo, p, st);
}

}  // namespace

namespace gc {

bool tc_supported(bool ta, bool tb, int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb, int64_t ldc) {
  (void)ldc;
  if (M <= 0 || N <= 0 || K <= 0) return false;
  if (M >= (int64_t(1) << 31) || N >= (int64_t(1) << 31) || K >= (int64_t(1) << 31)) return false;
  // operands consumed in place need 16-byte aligned row pitches; operands that
  // are re-laid into the workspace get a padded pitch there
  const Plan pl = make_plan(ta, tb, M, N, K, 3);
  if (!pl.transpose_a && lda % 4 != 0) return false;
  if (!pl.transpose_b && ldb % 4 != 0) return false;
  return true;
}

// Workspace layout: [flag: 256 B][A^T][B^T][B_lo][split-K partials]
size_t tc_workspace_bytes(bool ta, bool tb, int64_t M, int64_t N, int64_t K, int passes) {
  const Plan pl = make_plan(ta, tb, M, N, K, passes);
  size_t b = 256;
  const size_t kp = size_t(round4(K));
  if (pl.transpose_a) b += align256(size_t(M) * kp * 4);
  if (pl.transpose_b) b += align256(size_t(N) * kp * 4);
  if (passes == 3 && !pl.conv_b) b += align256(size_t(N) * kp * 4);
  if (pl.splits > 1) b += align256(size_t(pl.splits) * size_t(M) * size_t(N) * 4);
  return b;
}

int gemm_tc(bool ta, bool tb, int64_t M, int64_t N, int64_t K, const float* A, int64_t lda, const float* B,
            int64_t ldb, float* C, int64_t ldc, const GemmEpilogue& ep, int passes, void* workspace,
            size_t workspace_bytes, cudaStream_t st) {
  if (!workspace || workspace_bytes < tc_workspace_bytes(ta, tb, M, N, K, passes))
    return fail(GC_ERR_WORKSPACE, "gemm_tc: workspace missing or smaller than gc_gemm_workspace_bytes()");
  if (!aligned16(workspace)) return fail(GC_ERR_INVALID, "gemm_tc: workspace must be 16-byte aligned");
  const Plan pl = make_plan(ta, tb, M, N, K, passes);
  char* ws = static_cast<char*>(workspace);
  int* flag = reinterpret_cast<int*>(ws);
  ws += 256;
  const int64_t kp = round4(K);
  const unsigned tgrid = kNumSMs * 8;
  int rc;

  const float* Aop = A;
  int64_t lda_op = lda;
  if (pl.transpose_a) {
    float* At = reinterpret_cast<float*>(ws);
    ws += align256(size_t(M) * kp * 4);
    transpose_kernel<<<tgrid, 256, 0, st>>>(A, lda, At, kp, int(K), int(M));
    if ((rc = check_launch("transpose A")) != GC_OK) return rc;
    Aop = At;
    lda_op = kp;
  }
  const float* Bop = B;
  int64_t ldb_op = ldb;
  if (pl.transpose_b) {
    float* Bt = reinterpret_cast<float*>(ws);
    ws += align256(size_t(N) * kp * 4);
    transpose_kernel<<<tgrid, 256, 0, st>>>(B, ldb, Bt, kp, int(K), int(N));
    if ((rc = check_launch("transpose B")) != GC_OK) return rc;
    Bop = Bt;
    ldb_op = kp;
  }
  const float* Blo = Bop;
  int64_t ldblo = ldb_op;
  if (passes == 3 && !pl.conv_b) {
    float* bl = reinterpret_cast<float*>(ws);
    ws += align256(size_t(N) * kp * 4);
    split_lo_kernel<<<tgrid, 256, 0, st>>>(Bop, ldb_op, bl, kp, int(N), int(K));
    if ((rc = check_launch("split B")) != GC_OK) return rc;
    Blo = bl;
    ldblo = kp;
  }
  float* partial = nullptr;
  if (pl.splits > 1) {
    partial = reinterpret_cast<float*>(ws);
    ws += align256(size_t(pl.splits) * size_t(M) * size_t(N) * 4);
  }
  if (!aligned16(Aop) || !aligned16(Bop)) return fail(GC_ERR_UNSUPPORTED, "gemm_tc: operand base not 16-byte aligned");

  CUtensorMap mA, mB, mBlo;
  const int bk = (passes == 3 && pl.bn == 256) ? 16 : 32;
  if (pl.a_mn) rc = make_map(&mA, Aop, K, M, lda_op, bk, true, bk);
  else rc = make_map(&mA, Aop, M, K, lda_op, BM, false, bk);
  if (rc != GC_OK) return rc;
  if (pl.b_mn) rc = make_map(&mB, Bop, K, N, ldb_op, bk, true, bk);
  else rc = make_map(&mB, Bop, N, K, ldb_op, pl.bn, false, bk);
  if (rc != GC_OK) return rc;
  if (pl.b_mn) mBlo = mB;
  else if ((rc = make_map(&mBlo, Blo, N, K, ldblo, pl.bn, false, bk)) != GC_OK) return rc;

  TcParams p;
  p.M = int(M);
  p.N = int(N);
  p.K = int(K);
  p.C = C;
  p.ldc = ldc;
  p.ep = ep;
  p.flag = flag;
  p.vec_store = (!ep.transposed && ldc % 4 == 0 && aligned16(C) && (!ep.mask || aligned16(ep.mask)) && (!ep.gate || aligned16(ep.gate)) &&
                 (!ep.bias || aligned16(ep.bias)))
                    ? 1
                    : 0;
  p.splits = pl.splits;
  p.kb_per_split = pl.kb_per_split;
  p.partial = partial;
  if (passes == 3) {
    if (pl.bn == 64) rc = launch_layout<64, 3>(pl, mA, mB, mBlo, p, st);
    else if (pl.bn == 128) rc = launch_layout<128, 3>(pl, mA, mB, mBlo, p, st);
    else rc = launch_layout<256, 3>(pl, mA, mB, mBlo, p, st);
  } else {
    if (pl.bn == 64) rc = launch_layout<64, 1>(pl, mA, mB, mBlo, p, st);
    else if (pl.bn == 128) rc = launch_layout<128, 1>(pl, mA, mB, mBlo, p, st);
    else rc = launch_layout<256, 1>(pl, mA, mB, mBlo, p, st);
  }
  if (rc != GC_OK) return rc;
  if (pl.splits > 1) {
    const int64_t total = M * N;
    const unsigned g = unsigned(std::min<int64_t>(ceil_div(total, 32), kNumSMs * 8));
    tc_splitk_reduce_kernel<<<g, 256, 0, st>>>(int(M), int(N), pl.splits, partial, C, ldc, ep);
    rc = check_launch("gemm_tc split-K reduce");
  }
  return rc;
}

// ---- bf16 operands -------------------------------------------------------------------------------------------
namespace {
void bf16_splits(int64_t M, int64_t N, int64_t K, int bn, int& splits, int& kb_per_split) {
  const int64_t tiles = ceil_div(M, BM) * ceil_div(N, bn);
  const int64_t nkb = ceil_div(K, 64);
  int64_t s = 1;
  if (tiles * 2 <= kNumSMs && nkb >= 64) s = std::min<int64_t>(kNumSMs / tiles, nkb / 16);
  s = std::max<int64_t>(1, s);
  kb_per_split = int(ceil_div(nkb, s));
  splits = int(ceil_div(nkb, kb_per_split));
}
}  // namespace

size_t bf16_core_workspace_bytes(int64_t M, int64_t N, int64_t K) {
  int splits, kbs;
  bf16_splits(M, N, K, pick_bn(N), splits, kbs);
  return 256 + (splits > 1 ? align256(size_t(splits) * size_t(M) * size_t(N) * 4) : 0);
}

size_t bf16_workspace_bytes(int64_t M, int64_t N, int64_t K) {
  const size_t kp = size_t(round8(K));
  return bf16_core_workspace_bytes(M, N, K) + align256(size_t(M) * kp * 2) + align256(size_t(N) * kp * 2);
}

int convert_bf16(const float* src, int64_t lds, int64_t rows, int64_t cols, uint16_t* dst, int64_t ldd, bool transpose,
                 cudaStream_t st) {
  // dst is rows x cols (pitch ldd, even); src is rows x cols, or cols x rows when transpose
  const unsigned grid = kNumSMs * 8;
  if (transpose) cvt_transpose_bf16_kernel<<<grid, 256, 0, st>>>(src, lds, dst, ldd, int(cols), int(rows));
  else if (lds % 4 == 0 && ldd % 8 == 0 && aligned16(src) && aligned16(dst))
    cvt_bf16_vec8_kernel<<<grid, 256, 0, st>>>(src, lds, dst, ldd, int(rows), int(cols));
  else cvt_bf16_kernel<<<grid, 256, 0, st>>>(src, lds, dst, ldd, int(rows), int(cols));
  return check_launch("convert to bf16");
}

// C = A * Bt^T with A (M x K) and Bt (N x K) bf16, K-major, pitches multiples of 8 elements, bases 16-byte aligned.
int gemm_bf16_core(int64_t M, int64_t N, int64_t K, const uint16_t* A, int64_t lda, const uint16_t* Bt, int64_t ldb,
                   float* C, int64_t ldc, const GemmEpilogue& ep, void* workspace, size_t workspace_bytes,
                   cudaStream_t st) {
  if (!workspace || workspace_bytes < bf16_core_workspace_bytes(M, N, K))
    return fail(GC_ERR_WORKSPACE, "bf16 GEMM: workspace missing or too small");
  if (!aligned16(workspace) || !aligned16(A) || !aligned16(Bt) || lda % 8 != 0 || ldb % 8 != 0)
    return fail(GC_ERR_INVALID, "bf16 GEMM: operands and workspace must be 16-byte aligned, pitches multiples of 8");
  char* ws = static_cast<char*>(workspace);
  int* flag = reinterpret_cast<int*>(ws);
  ws += 256;
  const int bn = pick_bn(N);
  TcParams p;
  p.M = int(M); p.N = int(N); p.K = int(K);
  p.C = C; p.ldc = ldc; p.ep = ep; p.flag = flag;
  p.vec_store = (!ep.transposed && ldc % 4 == 0 && aligned16(C) && (!ep.mask || aligned16(ep.mask)) &&
                 (!ep.gate || aligned16(ep.gate)) && (!ep.bias || aligned16(ep.bias))) ? 1 : 0;
  bf16_splits(M, N, K, bn, p.splits, p.kb_per_split);
  p.partial = p.splits > 1 ? reinterpret_cast<float*>(ws) : nullptr;
  CUtensorMap mA, mB;
  int rc = make_map_bf16(&mA, A, M, K, lda, BM);
  if (rc == GC_OK) rc = make_map_bf16(&mB, Bt, N, K, ldb, bn);
  if (rc != GC_OK) return rc;
  auto run = [&](auto kern, int smem, int bn_) -> int {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return fail(GC_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    const int64_t items = ceil_div(M, BM) * ceil_div(N, bn_) * (p.splits > 1 ? p.splits : 1);
    kern<<<unsigned(std::min<int64_t>(items, kNumSMs)), kThreads, smem, st>>>(mA, mB, mB, p);
    return check_launch("gemm_tf32_kernel (bf16 operands)");
  };
  if (bn == 64) rc = run(gemm_tf32_kernel<64, 1, false, false, false, true>, Cfg<64, 1>::kSmemBytes, 64);
  else if (bn == 128) rc = run(gemm_tf32_kernel<128, 1, false, false, false, true>, Cfg<128, 1>::kSmemBytes, 128);
  else rc = run(gemm_tf32_kernel<256, 1, false, false, false, true>, Cfg<256, 1>::kSmemBytes, 256);
  if (rc != GC_OK) return rc;
  if (p.splits > 1) {
    const int64_t total = M * N;
    const unsigned g = unsigned(std::min<int64_t>(ceil_div(total, 32), kNumSMs * 8));
    tc_splitk_reduce_kernel<<<g, 256, 0, st>>>(int(M), int(N), p.splits, p.partial, C, ldc, ep);
    rc = check_launch("bf16 GEMM split-K reduce");
  }
  return rc;
}

// fp32 operands in any of the four layouts: both are converted (and re-laid K-major) into the workspace first.
int gemm_bf16(bool ta, bool tb, int64_t M, int64_t N, int64_t K, const float* A, int64_t lda, const float* B,
              int64_t ldb, float* C, int64_t ldc, const GemmEpilogue& ep, void* workspace, size_t workspace_bytes,
              cudaStream_t st) {
  if (!workspace || workspace_bytes < bf16_workspace_bytes(M, N, K))
    return fail(GC_ERR_WORKSPACE, "gemm_bf16: workspace missing or smaller than gc_gemm_workspace_bytes()");
  if (!aligned16(workspace)) return fail(GC_ERR_INVALID, "gemm_bf16: workspace must be 16-byte aligned");
  const int64_t kp = round8(K);
  const size_t core = bf16_core_workspace_bytes(M, N, K);
  char* ws = static_cast<char*>(workspace);
  uint16_t* Ab = reinterpret_cast<uint16_t*>(ws + core);
  uint16_t* Bb = reinterpret_cast<uint16_t*>(ws + core + align256(size_t(M) * kp * 2));
  int rc = convert_bf16(A, lda, M, K, Ab, kp, ta, st);                // A given M x K, or K x M when ta
  if (rc == GC_OK) rc = convert_bf16(B, ldb, N, K, Bb, kp, !tb, st);  // B given N x K when tb, else K x N
  if (rc != GC_OK) return rc;
  return gemm_bf16_core(M, N, K, Ab, kp, Bb, kp, C, ldc, ep, workspace, core, st);
}

}  // namespace gc

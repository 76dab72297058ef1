// bf16 matrix product on the Blackwell tensor cores (tcgen05 + TMEM + TMA).
//
//   D[M, N] = (beta ? D : 0) + sum_s A_s[M, k_s] . B_s[k_s, N] + bias, optional residual
//
// Persistent kernel, one CTA per SM, 192 threads in three roles:
//   warp 0      TMA producer: one lane streams 128x64 A tiles and 256x64 B tiles
//               (bf16, 128-byte swizzle) into a 4-stage shared-memory ring;
//   warp 1      MMA issuer: one lane issues tcgen05.mma (M=128, N=256, K=16) from
//               shared-memory descriptors into one of two fp32 accumulators in
//               TMEM (2 x 256 columns), releasing ring stages with tcgen05.commit;
//   warps 2-5   epilogue: tcgen05.ld the finished accumulator (each warp owns the 32
//               TMEM lanes of its lane quarter), add bias / previous value /
//               residual, round, and store 64-byte row segments to global memory
//               while the MMA warp already works on the next tile in the other
//               accumulator.
// The contraction may be a concatenation of up to six (A_s, B_s) segments, each
// with its own pair of tensor maps: the LoRA term x.A^T.B^T rides in the same
// accumulator as the base product as [x | xa] . [W | B]^T, and dX sums
// dY.W + low.A the same way. Each operand may be K-major (contraction index
// contiguous) or MN-major (row/column index contiguous); MN-major tiles arrive as
// 64x64 TMA boxes and are described to the tensor core with the MN-major
// canonical layout, so W[N, K] serves both the forward and the dX product and
// the token-contracted dA/dB products need no transposed copies.
// A contraction can also be split into `splits` slices whose fp32 partial tiles
// go to separate planes (summed afterwards in a fixed order).
//
// Two variants share one body. gemm_tcgen05_kernel: one CTA per 128 x 256 tile, 4 stages of
// 48 KB. gemm_tcgen05_pair_kernel: a cluster of two CTAs per 256 x 256 tile; each CTA stages
// its 128 rows of A and its 128 columns of B (3 stages of two 32 KB k-blocks), the even CTA issues
// tcgen05.mma.cta_group::2 (M = 256) for both, the tensor cores fetch the other half of B from
// the peer's shared memory, TMA completions of both CTAs are counted on the leader's barrier
// and tcgen05.commit releases stages / publishes accumulators in both CTAs. That halves the
// B bytes each SM has to stage per MMA.
//
// Every mbarrier wait is bounded by a wall-clock limit; on expiry the CTA
// raises the device error flag, stops issuing work, frees its TMEM and exits.
// No TMA load in this file uses cluster multicast.
#include <cuda.h>
#include <cudaTypedefs.h>

#include <cstdlib>
#include <cstring>
#include <mutex>

#include "common.cuh"

namespace ct {
namespace {

// BM rows of A per CTA; a tile is (BM * CTAS) x BN where CTAS is 1, or 2 for a CTA pair that
// shares one cta_group::2 MMA (each CTA then stages BM rows of A and BN / 2 columns of B).
constexpr int BM = 128, BN = 256, BK = 64, UMMA_K = 16;
constexpr uint32_t A_HALF_BYTES = BM * BK * 2;  // 16 KB: the 128 rows of A behind one MMA
constexpr uint32_t MN_BOX_BYTES = 64 * BK * 2;  // one 64(mn) x 64(k) box of an MN-major operand
constexpr uint32_t TMEM_COLS = 2 * BN;          // all 512 columns: two accumulators, or the two row halves of one
constexpr uint32_t STORE_STAGING_BYTES = 32 * 1024;   // epilogue staging tiles for the TMA store (all warps together)
constexpr uint32_t STORE_TILE_BYTES = 32 * 128;       // one warp's tile: 32 rows x 64 bf16 columns, 128-byte swizzle

// MH = row halves per CTA. MH = 1: a CTA owns 128 rows of a tile and alternates between two accumulators
// (the epilogue of one tile runs under the main loop of the next). MH = 2: a CTA owns 256 rows - two MMAs
// per k step share every B tile, which cuts the bytes staged per FLOP by a quarter and doubles the work
// buffered per ring stage - and the 128 x 512 TMEM holds that one 256 x 256 accumulator, so the epilogue
// (two warp sets, one per half) is not overlapped and has to be short.
template <int CTAS, int STAGES_, int KSUB_ = 1, int MH_ = 1>
struct Shape {
  static constexpr int kStages = STAGES_;
  static constexpr int kSub = KSUB_;                          // 64-wide k-blocks per ring stage
  static constexpr int kARows = BM * MH_;                     // A rows staged by one CTA
  static constexpr uint32_t kATileBytes = kARows * BK * 2;    // 16 KB or 32 KB
  static constexpr int kBRows = BN / CTAS;                    // B columns staged by one CTA
  static constexpr uint32_t kBTileBytes = kBRows * BK * 2;    // 32 KB or 16 KB
  static constexpr uint32_t kSubBytes = kATileBytes + kBTileBytes;
  static constexpr uint32_t kStageBytes = kSub * kSubBytes;
  static constexpr int kAccumulators = MH_ == 1 ? 2 : 1;
  static constexpr int kEpilogueWarps = 4 * MH_;
  static constexpr int kThreads = 64 + 32 * kEpilogueWarps;
  static constexpr size_t kSmemBytes =
      kStages * kStageBytes + STORE_STAGING_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
};
constexpr int GROUP_M = 16;                     // tile rasterisation: 16 row tiles share a sweep over columns
                                                // (CT_B200_GEMM_GROUP_M overrides it for experiments; 16 is
                                                // 0.4 % ahead of 8 and 12 inside a training step, 4, 32 and 64
                                                // are slower)
constexpr uint64_t kWaitLimitNs = 2000000000ull;

struct TcSegment {
  CUtensorMap a, b;
  int k_blocks;
  int a_mn, b_mn;
  // Read by the gated kernel only (zero elsewhere).
  int n_half;       // 1: the segment's B has N / 2 columns and its MMAs (N = 128) add to accumulator columns
  int d_col;        //    [d_col, d_col + 128) only: the low-rank term of ONE of the two interleaved projections
  int b_k_block;    // > 0: B is MN-major and its k rows live in a buffer of interleaved 128-row blocks: row k of
  int b_k_offset;   //    this operand is row k + (k / 128) * 128 + b_k_offset of the buffer
};

struct TcParams {
  TcSegment seg[kMaxSegments];
  int nseg;
  int k_blocks_total;
  int splits;
  int m_tiles, n_tiles;
  int group_m;          // tile rasterisation: this many row tiles share a sweep over the columns
  int64_t M, N;
  void* out;
  int64_t ldo;
  int64_t split_stride;  // elements between partial planes
  int out_f32;
  int beta;
  int vec_store;
  int tma_store;        // epilogue goes through shared memory and cp.async.bulk.tensor stores of `out_map`
  CUtensorMap out_map;  // bf16 output, boxes of 32 rows x 64 columns (128-byte swizzle) or x 32 columns (64-byte swizzle, MH == 2)
  const __nv_bfloat16* bias;
  const __nv_bfloat16* residual;
  int64_t ld_res;
  int* error_flag;
  // Gated epilogue (gemm_tcgen05_gated_kernel only). The accumulator tile holds 128 columns of the gate
  // projection and the same 128 columns of the up projection side by side (B is the two weights interleaved in
  // 128-row blocks). gated = 1: h = silu(gate) * up is written (and gate, up when their pointers are given);
  // gated = 2: with the upstream gradient dh of h, (d_gate, d_up, h) are written - gate and up never reach
  // memory. All five matrices are [M, N / 2] with leading dimension gated_ld; gated_h may alias gated_dh.
  // gated = 3: the accumulator itself is the gradient of h (the input gradient of the down projection, N columns)
  // and gate / up are read from memory (gated_src_g / gated_src_u, leading dimension gated_src_ld, kept by the
  // forward pass): (d_gate, d_up, h) go to (gated_g, gated_u, gated_h) and the gradient of h is never stored.
  int gated;
  __nv_bfloat16* gated_h;
  __nv_bfloat16* gated_g;
  __nv_bfloat16* gated_u;
  const __nv_bfloat16* gated_dh;
  int64_t gated_ld;
  const __nv_bfloat16* gated_src_g;
  const __nv_bfloat16* gated_src_u;
  int64_t gated_src_ld;
  // In-kernel NF4 decode of the B operand (gemm_tcgen05_nf4_kernel only): W[N, nf4_k] as packed codes, row-major,
  // two per byte, with one fp32 absmax per 64 elements and the 16-entry code table.
  const uint8_t* nf4_packed;
  const float* nf4_absmax;
  const float* nf4_code;
  int64_t nf4_k;

  // One problem per launch: every tile belongs to it.
  __device__ __forceinline__ int total_tiles() const { return m_tiles * n_tiles * splits; }
  __device__ __forceinline__ const TcParams& locate(int tile, int& local) const {
    local = tile;
    return *this;
  }
  __device__ __forceinline__ int* flag() const { return error_flag; }
  __device__ __forceinline__ const TcParams& problem_for_decode() const { return *this; }
};

// Several independent products in one launch: the persistent CTAs walk the concatenated tile lists, so that
// products with too few tiles to fill the machine on their own (the token-contracted adapter gradients of one
// operator) share its waves instead of each ending in a partial one.
constexpr int kMaxGroup = 6;
struct TcGroup {
  int count;
  int first[kMaxGroup + 1];     // first[i] = tiles of the problems before i; first[count] = all tiles
  TcParams problem[kMaxGroup];

  __device__ __forceinline__ int total_tiles() const { return first[count]; }
  __device__ __forceinline__ const TcParams& locate(int tile, int& local) const {
    int i = 0;
    while (i + 1 < count && tile >= first[i + 1]) ++i;
    local = tile - first[i];
    return problem[i];
  }
  __device__ __forceinline__ int* flag() const { return problem[0].error_flag; }
  __device__ __forceinline__ const TcParams& problem_for_decode() const { return problem[0]; }
};

// ---- PTX wrappers ---------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}
// The same test with acquire semantics at cluster scope: for a barrier whose arrivals publish shared-memory
// writes made by threads of the peer CTA.
__device__ __forceinline__ uint32_t mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}
__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Bounded wait. The common case (barrier already complete) is one try_wait; the polling loop with
// its wall-clock limit lives out of line so that the issue loops stay short. Returns false after
// kWaitLimitNs, having raised the error flag with `code` (which names the waiting role).
__device__ __forceinline__ bool mbar_wait_until(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                                int* error_flag, int code, uint64_t limit_ns) {
  const uint64_t start = global_timer_ns();
  uint32_t spins = 0;
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((++spins & 255u) == 0) {
      if (*abort_flag) return false;
      if (global_timer_ns() - start > limit_ns) {
        *abort_flag = 1;
        atomicCAS(error_flag, 0, code);
        return false;
      }
    }
  }
}
__device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* error_flag,
                                            int code) {
  return mbar_wait_until(bar, parity, abort_flag, error_flag, code, kWaitLimitNs);
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* error_flag,
                                          int code) {
  if (mbar_try_wait(bar, parity)) return true;
  return mbar_wait_slow(bar, parity, abort_flag, error_flag, code);
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, uint64_t map, uint32_t bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y)
      : "memory");
}

__device__ __forceinline__ void tcgen05_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// The 64-bit shared-memory descriptors are passed as (low, high) words: the high word is constant
// per operand orientation, only the start-address field in the low word moves.
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi,
                                          uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
      "mov.b64 da, {%1, %2};\n\t"
      "mov.b64 db, {%3, %4};\n\t"
      "setp.ne.b32 p, %6, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t}"
      ::"r"(tmem_d), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// ---- CTA-pair (cluster of two) helpers -----------------------------------------------
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// Address of this CTA's shared-memory location `addr` as seen in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}
// TMA load issued by either CTA of a pair; the completion bytes go to `cluster_bar`, which may
// live in the peer CTA. No multicast: the data lands in the issuing CTA only.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, uint64_t map, uint32_t cluster_bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(cluster_bar), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo,
                                               uint32_t b_hi, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
      "mov.b64 da, {%1, %2};\n\t"
      "mov.b64 db, {%3, %4};\n\t"
      "setp.ne.b32 p, %6, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %5, p;\n\t}"
      ::"r"(tmem_d), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive (once the MMAs issued so far are complete) on the barrier at this offset in BOTH CTAs.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
  const uint16_t both = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(bar), "h"(both)
               : "memory");
}

__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(map)), "r"(src), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int PENDING>
__device__ __forceinline__ void bulk_wait_read() {   // at most PENDING groups still READING their shared-memory source
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(PENDING) : "memory");
}
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_async_shared() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void tmem_load_32_issue(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}
// Wait for the TMEM loads issued so far. The registers travel through the statement as operands so that the
// compiler cannot move a use of them above the wait.
__device__ __forceinline__ void tmem_load_wait(uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.wait::ld.sync.aligned;"
      : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
        "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]),
        "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]),
        "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
      :
      : "memory");
}

__device__ __forceinline__ void tmem_load_16_issue(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_load_wait(uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.wait::ld.sync.aligned;"
      : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
        "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15])
      :
      : "memory");
}

__device__ __forceinline__ void tmem_load_32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor, 128-byte swizzle, descriptor version 1, as two 32-bit words.
// Low word: start address >> 4 (bits 0-13) and leading-dimension byte offset >> 4 (bits 16-29).
// High word: stride byte offset >> 4 (bits 0-13), version 1 (bits 14-15), swizzle mode 2 (bits 29-31).
__device__ __forceinline__ uint32_t desc_low(uint32_t addr, uint32_t leading_bytes) {
  return ((addr & 0x3FFFFu) >> 4) | (((leading_bytes >> 4) & 0x3FFFu) << 16);
}
__device__ __forceinline__ uint32_t desc_high(uint32_t stride_bytes) {
  return ((stride_bytes >> 4) & 0x3FFFu) | (1u << 14) | (2u << 29);
}

// Instruction descriptor: fp32 accumulate, bf16 x bf16, M = 128 (one CTA) or 256 (CTA pair), N = 256.
__device__ __forceinline__ uint32_t instr_desc(int a_mn, int b_mn, int m, int n = BN) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(a_mn) << 15) |
         (static_cast<uint32_t>(b_mn) << 16) | (static_cast<uint32_t>(n >> 3) << 17) |
         (static_cast<uint32_t>(m >> 4) << 24);
}

struct TileCoord {
  int m, n, split;
};

__device__ __forceinline__ TileCoord tile_coord(int tile, const TcParams& p) {
  const int per_split = p.m_tiles * p.n_tiles;
  TileCoord c;
  c.split = tile / per_split;
  const int rem = tile - c.split * per_split;
  const int per_group = p.group_m * p.n_tiles;
  const int group = rem / per_group;
  const int first_m = group * p.group_m;
  const int group_rows = min(p.group_m, p.m_tiles - first_m);
  const int in_group = rem - group * per_group;
  c.m = first_m + in_group % group_rows;
  c.n = in_group / group_rows;
  return c;
}

// k-block range [begin, end) of one split over the concatenated contraction.
__device__ __forceinline__ void split_range(const TcParams& p, int split, int& begin, int& end) {
  const int base = p.k_blocks_total / p.splits, extra = p.k_blocks_total % p.splits;
  begin = split * base + min(split, extra);
  end = begin + base + (split < extra ? 1 : 0);
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Epilogue of one 32-column chunk of one accumulator row: bias, previous value, rounding, residual, store.
__device__ __forceinline__ void store_chunk(const TcParams& p, float (&v)[32], char* out_plane, int64_t row,
                                            int64_t col0) {
  const bool full = col0 + 32 <= p.N;
  if (p.bias) {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (full || col0 + j < p.N) v[j] += __bfloat162float(p.bias[col0 + j]);
  }
  if (p.out_f32) {
    float* dst = reinterpret_cast<float*>(out_plane) + row * p.ldo + col0;
    if (full && p.vec_store) {
      float4* d4 = reinterpret_cast<float4*>(dst);
      if (p.beta) {
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          const float4 o = d4[q];
          v[4 * q] += o.x; v[4 * q + 1] += o.y; v[4 * q + 2] += o.z; v[4 * q + 3] += o.w;
        }
      }
#pragma unroll
      for (int q = 0; q < 8; ++q) d4[q] = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
    } else {
      for (int j = 0; j < 32 && col0 + j < p.N; ++j) dst[j] = p.beta ? dst[j] + v[j] : v[j];
    }
  } else {
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(out_plane) + row * p.ldo + col0;
    const __nv_bfloat16* res = p.residual ? p.residual + row * p.ld_res + col0 : nullptr;
    if (full && p.vec_store) {
      uint4* d4 = reinterpret_cast<uint4*>(dst);
      if (p.beta) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const uint4 o = d4[q];
          const uint32_t w[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[j]));
            v[8 * q + 2 * j] += f.x;
            v[8 * q + 2 * j + 1] += f.y;
          }
        }
      }
      if (res) {
        const uint4* r4 = reinterpret_cast<const uint4*>(res);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const uint4 o = __ldg(r4 + q);
          const uint32_t w[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[j]));
            v[8 * q + 2 * j] = __fadd_rn(__bfloat162float(__float2bfloat16_rn(v[8 * q + 2 * j])), f.x);
            v[8 * q + 2 * j + 1] = __fadd_rn(__bfloat162float(__float2bfloat16_rn(v[8 * q + 2 * j + 1])), f.y);
          }
        }
      }
#pragma unroll
      for (int q = 0; q < 4; ++q)
        d4[q] = make_uint4(pack_bf16(v[8 * q], v[8 * q + 1]), pack_bf16(v[8 * q + 2], v[8 * q + 3]),
                           pack_bf16(v[8 * q + 4], v[8 * q + 5]), pack_bf16(v[8 * q + 6], v[8 * q + 7]));
    } else {
      for (int j = 0; j < 32 && col0 + j < p.N; ++j) {
        float x = v[j];
        if (p.beta) x += __bfloat162float(dst[j]);
        if (res) x = __fadd_rn(__bfloat162float(__float2bfloat16_rn(x)), __bfloat162float(res[j]));
        dst[j] = __float2bfloat16_rn(x);
      }
    }
  }
}

// Epilogue of one COLS-column chunk (64 or 32) of one accumulator row through shared memory: bias, rounding,
// residual, then 16-byte pieces into this warp's staging tile of 32 rows x (2 * COLS) bytes, in the swizzle a
// tensor-map store of that width expects - 128-byte rows: piece j of row r sits at piece j ^ (r & 7); 64-byte
// rows: at piece j ^ ((r >> 1) & 3) - which also keeps the eight lanes of a store phase on different banks.
template <int COLS>
__device__ __forceinline__ void stage_chunk(const TcParams& p, float (&v)[COLS], uint32_t tile, int lane, int64_t row,
                                            int64_t col0) {
  const bool full = col0 + COLS <= p.N;
  if (p.bias) {
    if (full && p.vec_store) {
      const uint4* b4 = reinterpret_cast<const uint4*>(p.bias + col0);
#pragma unroll
      for (int q = 0; q < COLS / 8; ++q) {
        const uint4 o = __ldg(b4 + q);
        const uint32_t w[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[j]));
          v[8 * q + 2 * j] += f.x;
          v[8 * q + 2 * j + 1] += f.y;
        }
      }
    } else {
#pragma unroll
      for (int j = 0; j < COLS; ++j)
        if (col0 + j < p.N) v[j] += __bfloat162float(p.bias[col0 + j]);
    }
  }
  if (p.residual && row < p.M) {
    const __nv_bfloat16* res = p.residual + row * p.ld_res + col0;
    if (full && p.vec_store) {
      const uint4* r4 = reinterpret_cast<const uint4*>(res);
#pragma unroll
      for (int q = 0; q < COLS / 8; ++q) {
        const uint4 o = __ldg(r4 + q);
        const uint32_t w[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[j]));
          v[8 * q + 2 * j] = __fadd_rn(__bfloat162float(__float2bfloat16_rn(v[8 * q + 2 * j])), f.x);
          v[8 * q + 2 * j + 1] = __fadd_rn(__bfloat162float(__float2bfloat16_rn(v[8 * q + 2 * j + 1])), f.y);
        }
      }
    } else {
#pragma unroll
      for (int j = 0; j < COLS; ++j)
        if (col0 + j < p.N)
          v[j] = __fadd_rn(__bfloat162float(__float2bfloat16_rn(v[j])), __bfloat162float(res[j]));
    }
  }
  const uint32_t row_base = tile + static_cast<uint32_t>(lane) * (2u * COLS);
  const uint32_t twist = COLS == 64 ? (static_cast<uint32_t>(lane) & 7u) : ((static_cast<uint32_t>(lane) >> 1) & 3u);
#pragma unroll
  for (int q = 0; q < COLS / 8; ++q) {
    const uint32_t dst = row_base + ((static_cast<uint32_t>(q) ^ twist) << 4);
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(pack_bf16(v[8 * q], v[8 * q + 1])),
                 "r"(pack_bf16(v[8 * q + 2], v[8 * q + 3])), "r"(pack_bf16(v[8 * q + 4], v[8 * q + 5])),
                 "r"(pack_bf16(v[8 * q + 6], v[8 * q + 7]))
                 : "memory");
  }
}

// The same for 32 columns that were rounded to bf16 when the accumulator was drained (16 packed pairs): only the
// residual is left to add (round(value) + residual, rounded again - the arithmetic of stage_chunk).
__device__ __forceinline__ void stage_packed(const TcParams& p, const uint32_t* words, uint32_t tile, int lane,
                                             int64_t row, int64_t col0) {
  uint32_t w[16];
#pragma unroll
  for (int j = 0; j < 16; ++j) w[j] = words[j];
  if (p.residual && row < p.M) {
    const bool full = col0 + 32 <= p.N;
    const __nv_bfloat16* res = p.residual + row * p.ld_res + col0;
    if (full && p.vec_store) {
      const uint4* r4 = reinterpret_cast<const uint4*>(res);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const uint4 o = __ldg(r4 + q);
        const uint32_t r[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r[j]));
          const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[4 * q + j]));
          w[4 * q + j] = pack_bf16(__fadd_rn(v.x, f.x), __fadd_rn(v.y, f.y));
        }
      }
    } else {
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[j]));
        const float lo = col0 + 2 * j < p.N ? __fadd_rn(v.x, __bfloat162float(res[2 * j])) : v.x;
        const float hi = col0 + 2 * j + 1 < p.N ? __fadd_rn(v.y, __bfloat162float(res[2 * j + 1])) : v.y;
        w[j] = pack_bf16(lo, hi);
      }
    }
  }
  const uint32_t row_base = tile + static_cast<uint32_t>(lane) * 64u;
  const uint32_t twist = (static_cast<uint32_t>(lane) >> 1) & 3u;
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const uint32_t dst = row_base + ((static_cast<uint32_t>(q) ^ twist) << 4);
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(w[4 * q]), "r"(w[4 * q + 1]),
                 "r"(w[4 * q + 2]), "r"(w[4 * q + 3])
                 : "memory");
  }
}

// One body for all variants. CTAS == 1: every CTA owns a 128 x 256 tile. CTAS == 2: the two CTAs of a cluster
// own a (256 * MH) x 256 tile; each stages its 128 * MH rows of A and its 128 columns of B, the even ("leader")
// CTA issues the cta_group::2 MMAs (one per row half and k step) for both, and both run their own epilogue on
// their accumulator rows.
template <int CTAS, int STAGES_, int KSUB_, int MH, typename Params, bool DECODE = false, bool GATED = false>
__device__ __forceinline__ void gemm_body(const Params& params) {
  using S = Shape<CTAS, STAGES_, KSUB_, MH>;
  constexpr bool GATED_EPI = GATED && MH == 1;   // the SwiGLU epilogues exist in the 256 x 256-tile form only
  constexpr int KSUB = KSUB_;
  constexpr uint32_t A_BYTES = S::kATileBytes;
  constexpr int STAGES = S::kStages;
  constexpr uint32_t STAGE_BYTES = S::kStageBytes;
  constexpr int ACCS = S::kAccumulators;
  extern __shared__ uint8_t smem_raw[];
  // 128-byte-swizzled tiles need 1024-byte alignment.
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* staging = smem + STAGES * STAGE_BYTES;                 // 32 KB, 1024-byte aligned
  uint64_t* bars = reinterpret_cast<uint64_t*>(staging + STORE_STAGING_BYTES);
  // bars: [0, STAGES) full, [STAGES, 2*STAGES) empty, then tmem_full[2], tmem_empty[2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = CTAS == 2 ? cluster_rank() : 0u;  // position in the CTA pair; 0 leads
  const bool leader = rank == 0;
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_base = smem_u32(bars);
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto tmem_full_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
  auto tmem_empty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      // DECODE: besides the producer's expect-tx arrival, one arrival per decode warp of every CTA of the tile
      mbar_init(full_bar(s), DECODE ? 1 + 4 * CTAS : 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tmem_full_bar(a), 1);
      mbar_init(tmem_empty_bar(a), S::kEpilogueWarps * CTAS);  // one arrival per epilogue warp of every CTA of the tile
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    if constexpr (CTAS == 1) {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                   "r"(TMEM_COLS)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    } else {
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                   "r"(TMEM_COLS)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
  }
  tcgen05_fence_before();
  __syncthreads();
  if constexpr (CTAS == 2) cluster_sync_all();  // the peer's barriers exist before anything signals them
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // Everything above ran while the previous kernel of the stream may still have been finishing;
  // global memory is touched only below.
  grid_dependency_wait();

  const int total_tiles = params.total_tiles();
  int* const error_flag = params.flag();
  const int first_tile = blockIdx.x / CTAS, tile_step = gridDim.x / CTAS;
  constexpr int CTA_ROWS = BM * MH;             // accumulator rows of one CTA
  constexpr int TILE_M = CTA_ROWS * CTAS;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    // The whole warp walks the loop (uniform control flow keeps addresses and counters in
    // uniform registers); lane 0 alone issues the copies.
    {
      int stage = 0;
      uint32_t phase = 0;
      bool alive = true;
      const uint32_t lead_full0 = CTAS == 2 ? map_to_cta(full_bar(0), 0) : full_bar(0);
      for (int tile = first_tile; tile < total_tiles && alive; tile += tile_step) {
        int local;
        const TcParams& p = params.locate(tile, local);
        const TileCoord tc = tile_coord(local, p);
        int kb_begin, kb_end;
        split_range(p, tc.split, kb_begin, kb_end);
        const int a_row0 = tc.m * TILE_M + static_cast<int>(rank) * CTA_ROWS;
        const int b_row0 = tc.n * BN + static_cast<int>(rank) * S::kBRows;
        int seg_first = 0;
        for (int seg = 0; seg < p.nseg && alive; ++seg) {
          const TcSegment& sg = p.seg[seg];
          const int lo = max(kb_begin, seg_first) - seg_first;
          const int hi = min(kb_end, seg_first + sg.k_blocks) - seg_first;
          seg_first += sg.k_blocks;
          if (lo >= hi) continue;
          // Everything of the segment the copies need sits in registers before the k loop starts (the empty
          // statement pins it): a parameter read between a stage's release and its copies would delay them.
          uint64_t map_a = reinterpret_cast<uint64_t>(&sg.a), map_b = reinterpret_cast<uint64_t>(&sg.b);
          int a_mn = sg.a_mn, b_mn = sg.b_mn;
          int b_row = b_row0;
          uint32_t b_tx = DECODE ? 0u : S::kBTileBytes;     // bytes of B one CTA receives per k-block
          int k_block = 0, k_offset = 0;
          if constexpr (GATED) {
            if (sg.n_half) {     // half as many B columns: 64 rows of a K-major [N / 2, k] matrix per CTA
              b_row = tc.n * (BN / 2) + static_cast<int>(rank) * (S::kBRows / 2);
              b_tx = S::kBTileBytes / 2;
            }
            k_block = sg.b_k_block;
            k_offset = sg.b_k_offset;
          }
          asm volatile("" : "+l"(map_a), "+l"(map_b), "+r"(a_mn), "+r"(b_mn), "+r"(b_row), "+r"(b_tx), "+r"(k_block),
                       "+r"(k_offset));
          for (int kb = lo; kb < hi; kb += KSUB) {
            // A freed stage has to be on its way again within the time the MMAs of the other stages take, so
            // everything the copies need is worked out BEFORE the wait (the empty statement pins it there) and
            // only the expect-tx and the copy instructions themselves follow it.
            const int subs = min(KSUB, hi - kb);   // a stage holds up to KSUB 64-wide k-blocks
            // Completion bytes of both CTAs of a pair are counted on the leader's barrier.
            uint32_t bar = lead_full0 + 8u * stage;
            // an MN-major operand arrives as boxes of 64 columns x ALL the stage's k rows, whatever `subs` is
            uint32_t expected = CTAS * ((a_mn ? KSUB : subs) * A_BYTES + (b_mn ? KSUB : subs) * b_tx);
            uint32_t a_dst = smem_base + stage * STAGE_BYTES;
            int k_first = kb * BK;
            asm volatile("" : "+r"(bar), "+r"(expected), "+r"(a_dst), "+r"(k_first));
            if (!__all_sync(0xffffffffu, mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, error_flag, 1))) {
              alive = false;
              break;
            }
            if (lane == 0) {
              if (leader) mbar_expect_tx(full_bar(stage), expected);
              auto load = [&](uint32_t dst, uint64_t map, int x, int y) {
                if constexpr (CTAS == 1) tma_load_2d(dst, map, bar, x, y);
                else tma_load_2d_pair(dst, map, bar, x, y);
              };
              // A stage is [A: KSUB k-blocks][B: KSUB k-blocks]. A K-major operand takes one copy per k-block
              // (rows x 64 k, at k-block * tile bytes); an MN-major operand one copy per 64 columns for ALL the
              // stage's k rows (box j at j * KSUB * 8 KB, k-block s at s * 8 KB inside it): half the copy
              // instructions of a copy per k-block, and these are what a stage's turn-around waits for.
              const uint32_t b_dst = a_dst + KSUB * A_BYTES;
              if (!a_mn) {
#pragma unroll
                for (int sub = 0; sub < KSUB; ++sub)
                  if (sub < subs) load(a_dst + sub * A_BYTES, map_a, k_first + sub * BK, a_row0);   // CTA_ROWS rows
              } else {
#pragma unroll
                for (int j = 0; j < CTA_ROWS / 64; ++j)
                  load(a_dst + j * (KSUB * MN_BOX_BYTES), map_a, a_row0 + j * 64, k_first);
              }
              if constexpr (DECODE) {
                // the B tiles of this stage are written by the decode warps
              } else if (!b_mn) {
#pragma unroll
                for (int sub = 0; sub < KSUB; ++sub)
                  if (sub < subs) load(b_dst + sub * S::kBTileBytes, map_b, k_first + sub * BK, b_row);
              } else {
                int k_row = k_first;
                if constexpr (GATED) {      // B's k rows live in a buffer of interleaved 128-row blocks (a stage's
                  if (k_block) k_row = k_first + ((k_first >> 7) << 7) + k_offset;   // rows never straddle two)
                }
#pragma unroll
                for (int j = 0; j < S::kBRows / 64; ++j)
                  load(b_dst + j * (KSUB * MN_BOX_BYTES), map_b, b_row0 + j * 64, k_row);
              }
            }
            __syncwarp();
            if (++stage == STAGES) {
              stage = 0;
              phase ^= 1u;
            }
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (leader CTA only) ---------------
    // One thread feeds the tensor core, so the loop is kept to a handful of instructions per MMA:
    // everything that depends only on the segment (instruction descriptor, descriptor high words,
    // per-k-step increments) is hoisted, and a k-block costs one barrier test, 4 * MH MMAs, one commit.
    // The whole warp walks the loop so that control flow stays uniform; lane 0 issues.
    if (leader) {
      int stage = 0;
      uint32_t phase = 0;
      int local_tile = 0;
      bool alive = true;
      const uint32_t desc_hi = desc_high(1024);
      for (int tile = first_tile; tile < total_tiles && alive; tile += tile_step, ++local_tile) {
        int local;
        const TcParams& p = params.locate(tile, local);
        const TileCoord tc = tile_coord(local, p);
        int kb_begin, kb_end;
        split_range(p, tc.split, kb_begin, kb_end);
        const int acc = ACCS == 2 ? (local_tile & 1) : 0;
        const uint32_t acc_phase = (local_tile / ACCS) & 1;
        if (!__all_sync(0xffffffffu, mbar_wait(tmem_empty_bar(acc), acc_phase ^ 1u, abort_flag, error_flag, 2)))
          break;
        tcgen05_fence_after();
        const uint32_t tmem_d = tmem_base + acc * BN;      // MH == 2: row half h accumulates at column h * BN
        uint32_t accumulate = 0;
        int seg_first = 0;
        for (int seg = 0; seg < p.nseg && alive; ++seg) {
          const TcSegment& sg = p.seg[seg];
          const int lo = max(kb_begin, seg_first) - seg_first;
          const int hi = min(kb_end, seg_first + sg.k_blocks) - seg_first;
          seg_first += sg.k_blocks;
          if (lo >= hi) continue;
          uint32_t idesc = instr_desc(sg.a_mn, sg.b_mn, BM * CTAS);
          uint32_t tmem_seg = tmem_d;
          if constexpr (GATED) {
            if (sg.n_half) {
              idesc = instr_desc(sg.a_mn, sg.b_mn, BM * CTAS, BN / 2);
              tmem_seg = tmem_d + static_cast<uint32_t>(sg.d_col);
            }
          }
          // K-major: 8-row groups 1024 B apart, 32 B per 16-element k step inside the swizzle atom.
          // MN-major: 64-wide column groups one box (8 KB) apart, 8-k groups 1024 B apart,
          //           16 k rows (2 KB) per k step.
          const uint32_t a_lo0 = desc_low(smem_base, sg.a_mn ? KSUB * MN_BOX_BYTES : 16u);
          const uint32_t b_lo0 = desc_low(smem_base + KSUB * A_BYTES, sg.b_mn ? KSUB * MN_BOX_BYTES : 16u);
          // k-block s of a stage: K-major tiles follow one another; inside an MN-major box it is 8 KB further
          const uint32_t a_sub = (sg.a_mn ? MN_BOX_BYTES : A_BYTES) >> 4;
          const uint32_t b_sub = (sg.b_mn ? MN_BOX_BYTES : S::kBTileBytes) >> 4;
          const uint32_t a_step = sg.a_mn ? (2048u >> 4) : (32u >> 4);
          const uint32_t b_step = sg.b_mn ? (2048u >> 4) : (32u >> 4);
          for (int kb = lo; kb < hi; kb += KSUB) {
            if (!__all_sync(0xffffffffu, mbar_wait(full_bar(stage), phase, abort_flag, error_flag, 3))) {
              alive = false;
              break;
            }
            if constexpr (DECODE) {
              // the B tiles were written by ordinary stores of both CTAs' decode warps (released at cluster scope)
              while (!mbar_try_wait_cluster(full_bar(stage), phase)) {
              }
            }
            tcgen05_fence_after();
            const int subs = min(KSUB, hi - kb);
            if (lane == 0) {
#pragma unroll
              for (int sub = 0; sub < KSUB; ++sub) {
                if (sub >= subs) break;
                const uint32_t a_lo = a_lo0 + stage * (STAGE_BYTES >> 4) + sub * a_sub;
                const uint32_t b_lo = b_lo0 + stage * (STAGE_BYTES >> 4) + sub * b_sub;
#pragma unroll
                for (int j = 0; j < BK / UMMA_K; ++j) {
#pragma unroll
                  for (int h = 0; h < MH; ++h) {
                    // the 128 rows of half h are 16 KB further into the A tile in either orientation
                    const uint32_t a_h = a_lo + h * (A_HALF_BYTES >> 4) + a_step * j;
                    if constexpr (CTAS == 1)
                      umma_bf16(tmem_seg + h * BN, a_h, desc_hi, b_lo + b_step * j, desc_hi, idesc,
                                (accumulate | sub | j) ? 1u : 0u);
                    else
                      umma_bf16_pair(tmem_seg + h * BN, a_h, desc_hi, b_lo + b_step * j, desc_hi, idesc,
                                     (accumulate | sub | j) ? 1u : 0u);
                  }
                }
              }
              if constexpr (CTAS == 1) umma_commit(empty_bar(stage));
              else umma_commit_pair(empty_bar(stage));
            }
            __syncwarp();
            accumulate = 1;
            if (++stage == STAGES) {
              stage = 0;
              phase ^= 1u;
            }
          }
        }
        if (alive && lane == 0) {
          if constexpr (CTAS == 1) umma_commit(tmem_full_bar(acc));
          else umma_commit_pair(tmem_full_bar(acc));
        }
        __syncwarp();
      }
    }
    __syncwarp();
  } else if (DECODE && warp >= 6) {
    // ------------------------------ NF4 decode warps --------------------------
    // Thread d of the 128 owns row d of this CTA's 128 B rows: per 64-wide k-block it turns 32 packed bytes and
    // one absmax into 64 bf16 values (code[nibble] * absmax in fp32, rounded once: the arithmetic of the
    // stand-alone decode) and writes them as the K-major 128-byte-swizzled row the tensor core expects. The
    // packed bytes of the NEXT stage are requested before this stage is decoded, so the loads' latency hides
    // behind the arithmetic. One problem, one contraction segment, no slices: stage g of this CTA pair is
    // k-blocks (g % per_tile) * KSUB .. of its (g / per_tile)-th tile.
    const TcParams& p = params.problem_for_decode();
    const int d = static_cast<int>(threadIdx.x) - 192;
    float* lut = reinterpret_cast<float*>(staging);          // entry i of lane l at word 32 * i + l: no bank conflicts
    for (int i = d; i < 16 * 32; i += 128) lut[i] = __ldg(p.nf4_code + (i >> 5));
    asm volatile("bar.sync 1, 128;" ::: "memory");            // the four decode warps only
    const float* mine = lut + lane;
    const int per_tile = (p.k_blocks_total + KSUB - 1) / KSUB;
    const int my_tiles = first_tile < total_tiles ? (total_tiles - first_tile + tile_step - 1) / tile_step : 0;
    const int total_stages = my_tiles * per_tile;
    uint4 word[2][KSUB][2];
    float scale[2][KSUB];
    auto fetch = [&](int g, int slot) {
      const int tile = first_tile + (g / per_tile) * tile_step;
      const int kb = (g % per_tile) * KSUB;
      const TileCoord tc = tile_coord(tile, p);
      const int64_t n = static_cast<int64_t>(tc.n) * BN + static_cast<int64_t>(rank) * S::kBRows + d;
#pragma unroll
      for (int sub = 0; sub < KSUB; ++sub) {
        const bool live = n < p.N && kb + sub < p.k_blocks_total;
        const int64_t element = n * p.nf4_k + static_cast<int64_t>(kb + sub) * BK;
        const uint4* source = reinterpret_cast<const uint4*>(p.nf4_packed + element / 2);
        word[slot][sub][0] = live ? __ldg(source) : make_uint4(0, 0, 0, 0);
        word[slot][sub][1] = live ? __ldg(source + 1) : make_uint4(0, 0, 0, 0);
        scale[slot][sub] = live ? __ldg(p.nf4_absmax + element / 64) : 0.f;
      }
    };
    int stage = 0;
    uint32_t phase = 0;
    const uint32_t lead_full0 = CTAS == 2 ? map_to_cta(full_bar(0), 0) : full_bar(0);
    if (total_stages > 0) fetch(0, 0);
#pragma unroll 1
    for (int g = 0; g < total_stages; g += 2) {
#pragma unroll
      for (int slot = 0; slot < 2; ++slot) {       // two stages per trip so that the register slots are static
        const int current = g + slot;
        if (current >= total_stages) break;
        if (current + 1 < total_stages) fetch(current + 1, slot ^ 1);
        if (!__all_sync(0xffffffffu, mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, error_flag, 1))) {
          g = total_stages;
          break;
        }
        const int kb = (current % per_tile) * KSUB;
#pragma unroll
        for (int sub = 0; sub < KSUB; ++sub) {
          if (kb + sub >= p.k_blocks_total) break;
          const uint32_t row_base = smem_base + stage * STAGE_BYTES + KSUB * A_BYTES + sub * S::kBTileBytes +
                                    static_cast<uint32_t>(d) * 128u;
          const uint32_t words[8] = {word[slot][sub][0].x, word[slot][sub][0].y, word[slot][sub][0].z, word[slot][sub][0].w,
                                     word[slot][sub][1].x, word[slot][sub][1].y, word[slot][sub][1].z, word[slot][sub][1].w};
          const float s8 = scale[slot][sub];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            uint32_t packed[4];
#pragma unroll
            for (int b = 0; b < 4; ++b) {
              const uint32_t byte = (words[j] >> (8 * b)) & 255u;
              packed[b] = pack_bf16(__fmul_rn(mine[(byte >> 4) * 32], s8), __fmul_rn(mine[(byte & 15u) * 32], s8));
            }
            const uint32_t dst = row_base + ((static_cast<uint32_t>(j) ^ (static_cast<uint32_t>(d) & 7u)) << 4);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(packed[0]), "r"(packed[1]),
                         "r"(packed[2]), "r"(packed[3])
                         : "memory");
          }
        }
        fence_async_shared();
        __syncwarp();
        if (lane == 0) {
          if constexpr (CTAS == 1) mbar_arrive(full_bar(stage));
          else mbar_arrive_cluster(lead_full0 + 8u * stage);
        }
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
    __syncwarp();
  } else {
    // ------------------------------ epilogue ----------------------------------
    const int quarter = warp & 3;            // TMEM lanes [32*quarter, 32*quarter + 32) belong to this warp
    const int half = (warp - 2) >> 2;        // MH == 2: warps 2-5 drain row half 0, warps 6-9 row half 1
    // This warp's two staging tiles for the tensor-map store: 4 KB each (64 columns, MH == 1) or 2 KB each
    // (32 columns, MH == 2); 32 KB for all warps in both cases.
    const uint32_t stage_tile0 =
        smem_u32(staging) + static_cast<uint32_t>(warp - 2) * (STORE_STAGING_BYTES / S::kEpilogueWarps);
    int stored = 0;                           // chunks this warp has handed to the store engine
    int local_tile = 0;
    for (int tile = first_tile; tile < total_tiles; tile += tile_step, ++local_tile) {
      int local;
      const TcParams& p = params.locate(tile, local);
      const TileCoord tc = tile_coord(local, p);
      const int acc = ACCS == 2 ? (local_tile & 1) : 0;
      const uint32_t acc_phase = (local_tile / ACCS) & 1;
      const int row0 = tc.m * TILE_M + static_cast<int>(rank) * CTA_ROWS + half * BM + quarter * 32;
      const int64_t row = row0 + lane;
      const bool row_ok = row < p.M;
      // Gated backward: the upstream gradient of a 32-column chunk is requested one chunk ahead - the first
      // chunk's before the wait for the accumulator, while the tile's main loop is still running.
      uint4 upstream_next[GATED_EPI ? 4 : 1];
      uint4 second_next[GATED_EPI ? 4 : 1];     // gated = 3: gate in upstream_next, up here
      if constexpr (GATED_EPI) {
#pragma unroll
        for (int q = 0; q < 4; ++q) upstream_next[q] = second_next[q] = make_uint4(0, 0, 0, 0);
        if (p.gated == 2 && row_ok) {
          const uint4* source = reinterpret_cast<const uint4*>(p.gated_dh + row * p.gated_ld + static_cast<int64_t>(tc.n) * (BN / 2));
#pragma unroll
          for (int q = 0; q < 4; ++q) upstream_next[q] = source[q];
        }
        if (p.gated == 3 && row_ok) {
          const int64_t first = row * p.gated_src_ld + static_cast<int64_t>(tc.n) * BN;
          const uint4* gate_source = reinterpret_cast<const uint4*>(p.gated_src_g + first);
          const uint4* up_source = reinterpret_cast<const uint4*>(p.gated_src_u + first);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            upstream_next[q] = gate_source[q];
            second_next[q] = up_source[q];
          }
        }
      }
      int ok = 1;
      if (lane == 0) ok = mbar_wait(tmem_full_bar(acc), acc_phase, abort_flag, error_flag, 4) ? 1 : 0;
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      tcgen05_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + (MH == 2 ? half : acc) * BN;
      bool released = false;   // the accumulator has already been handed back to the MMA warp
      if (GATED_EPI && p.gated == 3) {
        if constexpr (GATED_EPI) {
          // The accumulator is the gradient of hidden = silu(gate) * up; it is rounded to bf16 as the stored
          // gradient would be and meets gate and up (requested from memory one 32-column chunk ahead) in the
          // in-place backward of the stand-alone kernel. N is a multiple of 32 here.
          const int64_t tile_col = static_cast<int64_t>(tc.n) * BN;
#pragma unroll 1
          for (int c = 0; c < BN / 32; ++c) {
            const int64_t col0 = tile_col + c * 32;
            if (col0 >= p.N) break;  // uniform across the warp
            uint32_t raw[32];
            __syncwarp();
            tmem_load_32_issue(taddr + c * 32, raw);
            uint4 gate_now[4], up_now[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              gate_now[q] = upstream_next[GATED_EPI ? q : 0];
              up_now[q] = second_next[GATED_EPI ? q : 0];
            }
            if (row_ok && c + 1 < BN / 32 && col0 + 32 < p.N) {
              const int64_t next = row * p.gated_src_ld + col0 + 32;
              const uint4* gate_source = reinterpret_cast<const uint4*>(p.gated_src_g + next);
              const uint4* up_source = reinterpret_cast<const uint4*>(p.gated_src_u + next);
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                upstream_next[GATED_EPI ? q : 0] = gate_source[q];
                second_next[GATED_EPI ? q : 0] = up_source[q];
              }
            }
            tmem_load_wait(raw);
            if (row_ok) {
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const uint32_t gate_words[4] = {gate_now[q].x, gate_now[q].y, gate_now[q].z, gate_now[q].w};
                const uint32_t up_words[4] = {up_now[q].x, up_now[q].y, up_now[q].z, up_now[q].w};
                uint32_t h_words[4], g_words[4], u_words[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const float2 g = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&gate_words[j]));
                  const float2 u = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&up_words[j]));
                  const float grad0 = round_to<__nv_bfloat16>(__uint_as_float(raw[8 * q + 2 * j]));
                  const float grad1 = round_to<__nv_bfloat16>(__uint_as_float(raw[8 * q + 2 * j + 1]));
                  float h0 = 0.f, h1 = 0.f, a0 = 0.f, a1 = 0.f, b0 = 0.f, b1 = 0.f;
                  swiglu_element<__nv_bfloat16>(g.x, u.x, grad0, true, true, h0, a0, b0);
                  swiglu_element<__nv_bfloat16>(g.y, u.y, grad1, true, true, h1, a1, b1);
                  h_words[j] = pack_bf16(h0, h1);
                  g_words[j] = pack_bf16(a0, a1);
                  u_words[j] = pack_bf16(b0, b1);
                }
                const int64_t at = row * p.gated_ld + col0 + q * 8;
                *reinterpret_cast<uint4*>(p.gated_h + at) = make_uint4(h_words[0], h_words[1], h_words[2], h_words[3]);
                *reinterpret_cast<uint4*>(p.gated_g + at) = make_uint4(g_words[0], g_words[1], g_words[2], g_words[3]);
                *reinterpret_cast<uint4*>(p.gated_u + at) = make_uint4(u_words[0], u_words[1], u_words[2], u_words[3]);
              }
            }
          }
        }
      } else if (GATED_EPI && p.gated) {
        if constexpr (GATED_EPI) {
          // Accumulator columns [0, 128) are the gate projection, [128, 256) the up projection of the same 128
          // output columns. Each is rounded to bf16 as a stored projection output would be; the SwiGLU element
          // arithmetic is the stand-alone kernel's.
          const bool backward = p.gated == 2;
          const int64_t offset = row * p.gated_ld + static_cast<int64_t>(tc.n) * (BN / 2);
          // The chunk loop stays a loop: unrolled, the epilogue is tens of KB of code that four warps stream
          // through the instruction cache the producer and MMA warps' short loops live in.
#pragma unroll 1
          for (int c = 0; c < BN / 64; ++c) {
            uint32_t gate_raw[32], up_raw[32];
            __syncwarp();
            tmem_load_32_issue(taddr + c * 32, gate_raw);
            tmem_load_32_issue(taddr + BN / 2 + c * 32, up_raw);
            uint4 upstream[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) upstream[q] = upstream_next[GATED_EPI ? q : 0];
            if (backward && row_ok && c + 1 < BN / 64) {
              const uint4* source = reinterpret_cast<const uint4*>(p.gated_dh + offset + (c + 1) * 32);
#pragma unroll
              for (int q = 0; q < 4; ++q) upstream_next[GATED_EPI ? q : 0] = source[q];
            }
            tmem_load_wait(gate_raw);
            tmem_load_wait(up_raw);
            if (row_ok) {
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const uint4 grad_vector = upstream[q];
                const uint32_t grad_words[4] = {grad_vector.x, grad_vector.y, grad_vector.z, grad_vector.w};
                uint32_t h_words[4], g_words[4], u_words[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const float g0 = round_to<__nv_bfloat16>(__uint_as_float(gate_raw[8 * q + 2 * j]));
                  const float g1 = round_to<__nv_bfloat16>(__uint_as_float(gate_raw[8 * q + 2 * j + 1]));
                  const float u0 = round_to<__nv_bfloat16>(__uint_as_float(up_raw[8 * q + 2 * j]));
                  const float u1 = round_to<__nv_bfloat16>(__uint_as_float(up_raw[8 * q + 2 * j + 1]));
                  const float2 grad = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&grad_words[j]));
                  float h0 = 0.f, h1 = 0.f, a0 = 0.f, a1 = 0.f, b0 = 0.f, b1 = 0.f;
                  swiglu_element<__nv_bfloat16>(g0, u0, grad.x, backward, true, h0, a0, b0);
                  swiglu_element<__nv_bfloat16>(g1, u1, grad.y, backward, true, h1, a1, b1);
                  h_words[j] = pack_bf16(h0, h1);
                  g_words[j] = backward ? pack_bf16(a0, a1) : pack_bf16(g0, g1);
                  u_words[j] = backward ? pack_bf16(b0, b1) : pack_bf16(u0, u1);
                }
                const int64_t at = offset + c * 32 + q * 8;
                *reinterpret_cast<uint4*>(p.gated_h + at) = make_uint4(h_words[0], h_words[1], h_words[2], h_words[3]);
                if (p.gated_g) *reinterpret_cast<uint4*>(p.gated_g + at) = make_uint4(g_words[0], g_words[1], g_words[2], g_words[3]);
                if (p.gated_u) *reinterpret_cast<uint4*>(p.gated_u + at) = make_uint4(u_words[0], u_words[1], u_words[2], u_words[3]);
              }
            }
          }
        }
      } else if (p.tma_store) {
        if constexpr (MH == 1) {
          // 64-column chunks, two 4 KB staging tiles per warp (this epilogue runs under the next tile's main loop)
#pragma unroll 1
          for (int c = 0; c < BN / 64; ++c) {
            const int64_t col0 = static_cast<int64_t>(tc.n) * BN + c * 64;
            if (col0 >= p.N) break;  // uniform across the warp
            uint32_t lo[32], hi[32];
            tmem_load_32_issue(taddr + c * 64, lo);
            tmem_load_32_issue(taddr + c * 64 + 32, hi);
            // the staging tile about to be overwritten must have been read by its previous store
            if (lane == 0) bulk_wait_read<1>();
            tmem_load_wait(lo);
            tmem_load_wait(hi);
            __syncwarp();
            float v[64];
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              v[j] = __uint_as_float(lo[j]);
              v[32 + j] = __uint_as_float(hi[j]);
            }
            const uint32_t tile_smem = stage_tile0 + static_cast<uint32_t>(stored & 1) * STORE_TILE_BYTES;
            stage_chunk<64>(p, v, tile_smem, lane, row, col0);
            fence_async_shared();
            __syncwarp();
            if (lane == 0 && row0 < p.M) {      // rows and columns past the matrix are clipped by the store
              tma_store_2d(&p.out_map, tile_smem, static_cast<int>(col0), row0);
              bulk_commit();
            }
            ++stored;
          }
        } else {
          // Not overlapped with a main loop, so the accumulator is handed back as early as possible: the row's 256
          // columns are read (16 at a time, the next load in flight), given their bias, rounded to bf16 and kept
          // in 128 registers; the accumulator is released to the MMA warp; only then do residual, staging and
          // tensor-map stores run - under the next tile's main loop.
          constexpr int PIECES = BN / 16;
          uint32_t kept[BN / 2];
          uint32_t raw[2][16];
          tmem_load_16_issue(taddr, raw[0]);
#pragma unroll
          for (int c = 0; c < PIECES; ++c) {
            tmem_load_wait(raw[c & 1]);
            if (c + 1 < PIECES) tmem_load_16_issue(taddr + (c + 1) * 16, raw[(c + 1) & 1]);
            float v[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = __uint_as_float(raw[c & 1][j]);
            if (p.bias) {
              const int64_t col0 = static_cast<int64_t>(tc.n) * BN + c * 16;
#pragma unroll
              for (int j = 0; j < 16; ++j)
                if (col0 + j < p.N) v[j] += __bfloat162float(__ldg(p.bias + col0 + j));
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) kept[c * 8 + j] = pack_bf16(v[2 * j], v[2 * j + 1]);
          }
          tcgen05_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(map_to_cta(tmem_empty_bar(acc), 0));
          released = true;
#pragma unroll
          for (int c = 0; c < BN / 32; ++c) {
            const int64_t col0 = static_cast<int64_t>(tc.n) * BN + c * 32;
            if (col0 < p.N) {  // uniform across the warp
              if (lane == 0) bulk_wait_read<1>();
              __syncwarp();
              const uint32_t tile_smem = stage_tile0 + static_cast<uint32_t>(stored & 1) * (STORE_TILE_BYTES / 2);
              stage_packed(p, kept + c * 16, tile_smem, lane, row, col0);
              fence_async_shared();
              __syncwarp();
              if (lane == 0 && row0 < p.M) {
                tma_store_2d(&p.out_map, tile_smem, static_cast<int>(col0), row0);
                bulk_commit();
              }
              ++stored;
            }
          }
        }
      } else {
        char* out_plane = static_cast<char*>(p.out) +
                          static_cast<int64_t>(tc.split) * p.split_stride * (p.out_f32 ? 4 : 2);
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          const int64_t col0 = static_cast<int64_t>(tc.n) * BN + c * 32;
          if (col0 >= p.N) break;  // uniform across the warp
          uint32_t raw[32];
          __syncwarp();  // tcgen05.ld is warp-collective: rejoin lanes that skipped the previous stores
          tmem_load_32(taddr + c * 32, raw);
          if (!row_ok) continue;
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(raw[j]);
          store_chunk(p, v, out_plane, row, col0);
        }
      }
      if (!released) {
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) {
          if constexpr (CTAS == 1) mbar_arrive(tmem_empty_bar(acc));
          else mbar_arrive_cluster(map_to_cta(tmem_empty_bar(acc), 0));
        }
      }
    }
    // Shared memory must stay valid until the stores have read it, and the stores must be complete before the
    // kernel's writes count as done.
    if (lane == 0) bulk_wait_all();
    __syncwarp();
  }

  tcgen05_fence_before();
  __syncthreads();
  if constexpr (CTAS == 2) cluster_sync_all();  // neither CTA leaves while the other may still touch it
  if (warp == 1) {
    __syncwarp();
    tcgen05_fence_after();
    if constexpr (CTAS == 1)
      asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    else
      asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

__global__ void __launch_bounds__(Shape<1, 4, 1, 1>::kThreads, 1) gemm_tcgen05_kernel(const __grid_constant__ TcParams p) {
  gemm_body<1, 4, 1, 1>(p);
}

template <int STAGES_, int KSUB_>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(Shape<2, STAGES_, KSUB_, 1>::kThreads, 1)
    gemm_tcgen05_pair_kernel(const __grid_constant__ TcParams p) {
  gemm_body<2, STAGES_, KSUB_, 1>(p);
}

// Several products per launch (256 x 256 pair tiles, register-store epilogue: fp32 slice planes).
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(Shape<2, 3, 2, 1>::kThreads, 1)
    gemm_tcgen05_group_kernel(const __grid_constant__ TcGroup group) {
  gemm_body<2, 3, 2, 1>(group);
}

// y = x . dequant(W)^T with the NF4 decode inside the kernel: four more warps per CTA write the B tiles.
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(Shape<2, 3, 2, 1>::kThreads + 128, 1)
    gemm_tcgen05_nf4_kernel(const __grid_constant__ TcParams p) {
  gemm_body<2, 3, 2, 1, TcParams, true>(p);
}

// The pair kernel with the extras of a SwiGLU MLP: B operands made of two projections' weights interleaved in
// 128-row blocks, per-projection low-rank segments that add to half of the accumulator columns, and the SwiGLU
// forward or backward applied to the accumulator in the epilogue (TcParams::gated).
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(Shape<2, 3, 2, 1>::kThreads, 1)
    gemm_tcgen05_gated_kernel(const __grid_constant__ TcParams p) {
  gemm_body<2, 3, 2, 1, TcParams, false, true>(p);
}

// The wide kernel with the gated kernel's operand handling (interleaved weight buffers); plain epilogue.
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(Shape<2, 4, 1, 2>::kThreads, 1)
    gemm_tcgen05_gated_wide_kernel(const __grid_constant__ TcParams p) {
  gemm_body<2, 4, 1, 2, TcParams, false, true>(p);
}

// The 512 x 256 tile: two row halves per CTA, four ring stages of one 48 KB k-block, two epilogue warp sets.
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(Shape<2, 4, 1, 2>::kThreads, 1)
    gemm_tcgen05_wide_kernel(const __grid_constant__ TcParams p) {
  gemm_body<2, 4, 1, 2>(p);
}

// ---- host side ------------------------------------------------------------------
PFN_cuTensorMapEncodeTiled_v12000 encode_fn() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult status;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &status) != cudaSuccess ||
        status != cudaDriverEntryPointSuccess)
      ptr = nullptr;
    return reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(ptr);
  }();
  return fn;
}

// Tensor map over a bf16 matrix whose contiguous dimension has `inner` elements and
// whose rows are `ld` elements apart; tiles are `box_rows` rows of 64 elements.
// Encoding a map is a driver call of a microsecond or two and a training step asks for the same few
// hundred (pointer, shape) combinations over and over (the caching allocator hands the same blocks back),
// so encoded maps are kept in a small direct-mapped table. A map depends on nothing but its key.
struct MapKey {
  const void* base;
  int64_t inner, outer, ld;
  int box_rows, box_inner;
  bool operator==(const MapKey& o) const {
    return base == o.base && inner == o.inner && outer == o.outer && ld == o.ld && box_rows == o.box_rows &&
           box_inner == o.box_inner;
  }
};
struct MapSlot {
  MapKey key;
  CUtensorMap map;
  bool used;
};
constexpr int kMapSlots = 4096;
MapSlot g_map_table[kMapSlots];
std::mutex g_map_mutex;

// `box_inner` = 64 elements (128-byte rows, 128-byte swizzle: every operand tile and the 64-column store tile) or
// 32 elements (64-byte rows, 64-byte swizzle: the 32-column store tile).
int make_map(CUtensorMap* map, const void* base, int64_t inner, int64_t outer, int64_t ld, int box_rows,
             int box_inner = 64) {
  const MapKey key{base, inner, outer, ld, box_rows, box_inner};
  uint64_t h = reinterpret_cast<uintptr_t>(base) >> 4;
  h = (h ^ static_cast<uint64_t>(inner) * 0x9E3779B97F4A7C15ull) * 0xBF58476D1CE4E5B9ull;
  h = (h ^ static_cast<uint64_t>(outer) * 0x94D049BB133111EBull ^ static_cast<uint64_t>(ld) << 7 ^ static_cast<uint64_t>(box_rows) ^ static_cast<uint64_t>(box_inner) << 20) * 0x9E3779B97F4A7C15ull;
  MapSlot& slot = g_map_table[(h >> 32) % kMapSlots];
  {
    std::lock_guard<std::mutex> lock(g_map_mutex);
    if (slot.used && slot.key == key) {
      std::memcpy(map, &slot.map, sizeof(CUtensorMap));
      return CT_OK;
    }
  }
  auto fn = encode_fn();
  if (!fn) return fail(CT_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(inner), static_cast<cuuint64_t>(outer)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 2};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(box_inner), static_cast<cuuint32_t>(box_rows)};
  cuuint32_t elem[2] = {1, 1};
  const CUresult rc = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                         CU_TENSOR_MAP_INTERLEAVE_NONE,
                         box_inner == 64 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS) return fail(CT_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)rc);
  {
    std::lock_guard<std::mutex> lock(g_map_mutex);
    slot.key = key;
    std::memcpy(&slot.map, map, sizeof(CUtensorMap));
    slot.used = true;
  }
  return CT_OK;
}

bool operand_ok(const void* ptr, int64_t rs, int64_t cs) {
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) != 0) return false;
  const int64_t ld = (cs == 1) ? rs : cs;
  if (rs != 1 && cs != 1) return false;
  return ld % 8 == 0 && ld > 0;
}

int sm_count() {
  static int count = [] {
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    return n;
  }();
  return count;
}

// Self-test of the bounded wait: one thread waits on an mbarrier that nothing ever completes, with the
// GEMM's own wait routine and a short limit, gives up, raises the error flag (code 5) and returns.
__global__ void bounded_wait_selftest_kernel(int* error_flag, uint64_t limit_ns) {
  __shared__ uint64_t barrier;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(smem_u32(&barrier), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    mbar_wait_until(smem_u32(&barrier), 0, &abort_flag, error_flag, 5, limit_ns);
    asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(smem_u32(&barrier)) : "memory");
  }
}

}  // namespace

int bounded_wait_selftest(int64_t limit_us, cudaStream_t stream) {
  if (limit_us < 1 || limit_us > 100000)
    return fail(CT_ERR_ARG, "ct_selftest_bounded_wait: limit %lld us (1 .. 100000)", (long long)limit_us);
  int* flag = device_error_flag();
  if (!flag) return fail(CT_ERR_CUDA, "ct_selftest_bounded_wait: no device error flag");
  bounded_wait_selftest_kernel<<<1, 32, 0, stream>>>(flag, static_cast<uint64_t>(limit_us) * 1000ull);
  count_launch(false);
  return check_launch("ct_selftest_bounded_wait");
}

bool gemm_tcgen05_supported(const GemmArgs& g) {
  if (g.in_dtype != CT_BF16) return false;
  if (g.out_dtype != CT_BF16 && g.out_dtype != CT_F32) return false;
  if (g.M <= 0 || g.N <= 0 || g.nseg < 1 || g.nseg > kMaxSegments) return false;
  if (g.M > (1LL << 31) - BM || g.N > (1LL << 31) - BN) return false;
  int64_t k_blocks = 0;
  for (int s = 0; s < g.nseg; ++s) {
    const Segment& sg = g.seg[s];
    if (sg.k <= 0 || sg.k > (1LL << 31) - BK) return false;
    if (!operand_ok(sg.a, sg.a_rs, sg.a_cs) || !operand_ok(sg.b, sg.b_cs, sg.b_rs)) return false;
    // A dimension of extent 1 makes "which stride is 1" ambiguous; leave those to the SIMT kernel.
    if (sg.a_rs == 1 && sg.a_cs == 1) return false;
    if (sg.b_rs == 1 && sg.b_cs == 1) return false;
    k_blocks += (sg.k + BK - 1) / BK;
  }
  if (g.residual && (g.out_dtype != CT_BF16 || g.beta)) return false;
  const int splits = g.split_k > 1 ? g.split_k : 1;
  if (splits > 1 && (g.out_dtype != CT_F32 || g.beta || g.bias || g.residual)) return false;
  if (k_blocks < splits) return false;
  const int64_t tiles = ((g.M + BM - 1) / BM) * ((g.N + BN - 1) / BN) * splits;
  return tiles < (1LL << 30);
}

// CTA pairs pay off once a tile's 256 rows are real rows; products with fewer than 256 rows stay
// on the single-CTA kernel.
// The environment variable CT_B200_GEMM_CTAS (1 or 2) pins the choice for experiments and tests.
int env_int(const char* name, int fallback) {
  const char* text = getenv(name);
  return text ? atoi(text) : fallback;
}

int ctas_for(const GemmArgs& g) {
  const int pinned = env_int("CT_B200_GEMM_CTAS", 0);   // read per call: tests and comparison runs switch it in-process
  if (pinned == 1 || pinned == 2) return pinned;
  return g.M >= 2 * BM ? 2 : 1;
}

template <typename Kernel>
int configure(Kernel kernel, size_t smem, bool* configured) {
  if (!*configured) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) !=
        cudaSuccess)
      return fail(CT_ERR_CUDA, "gemm_tcgen05: cannot opt in to %zu bytes of shared memory: %s", smem,
                  cudaGetErrorString(cudaGetLastError()));
    *configured = true;
  }
  return CT_OK;
}

template <int STAGES_, int KSUB_>
int launch_pair(const TcParams& p, unsigned grid, int device, cudaStream_t stream) {
  static bool configured[64] = {};
  const size_t smem = Shape<2, STAGES_, KSUB_>::kSmemBytes;
  const int rc = configure(gemm_tcgen05_pair_kernel<STAGES_, KSUB_>, smem, &configured[device]);
  if (rc != CT_OK) return rc;
  launch_dependent(gemm_tcgen05_pair_kernel<STAGES_, KSUB_>, dim3(grid), dim3(Shape<2, STAGES_, KSUB_>::kThreads), smem,
                   stream, p);
  return CT_OK;
}

int launch_wide(const TcParams& p, unsigned grid, int device, cudaStream_t stream) {
  static bool configured[64] = {};
  using S = Shape<2, 4, 1, 2>;
  const int rc = configure(gemm_tcgen05_wide_kernel, S::kSmemBytes, &configured[device]);
  if (rc != CT_OK) return rc;
  launch_dependent(gemm_tcgen05_wide_kernel, dim3(grid), dim3(S::kThreads), S::kSmemBytes, stream, p);
  return CT_OK;
}

int launch_single(const TcParams& p, unsigned grid, int device, cudaStream_t stream) {
  static bool configured[64] = {};
  const size_t smem = Shape<1, 4, 1>::kSmemBytes;
  const int rc = configure(gemm_tcgen05_kernel, smem, &configured[device]);
  if (rc != CT_OK) return rc;
  launch_dependent(gemm_tcgen05_kernel, dim3(grid), dim3(Shape<1, 4, 1>::kThreads), smem, stream, p);
  return CT_OK;
}

// Row halves per CTA and the kind of epilogue, chosen from same-device comparisons of the four combinations on
// the shapes of a training step (CT_B200_GEMM_MH = 1 / 2 and CT_B200_GEMM_TMA_STORE = 0 / 1 pin them):
//  * the 512 x 256 tile stages a quarter fewer bytes per FLOP (47 instead of 64 bytes per SM and cycle, the latter
//    being about what an SM can take from L2) and doubles the work buffered per ring stage. Its accumulator
//    fills the whole TMEM, so its epilogue cannot run under the next main loop; since that epilogue drains the
//    accumulator into registers first and hands it back before it stores anything, the exposed part is about a
//    microsecond per tile and the wide tile is ahead on every large product (2 to 4 % on K-major B, 6 to 9 % on
//    MN-major B; 14 ms of a 600 ms training step against the 256 x 256 tile everywhere). It needs the
//    tensor-map store (a bf16 result written once), at least 1024 columns (enough tiles to fill the machine)
//    and rows that fill 512-row tiles (a multiple of 512, or so many that the padding is below 7 %);
//  * a product whose tiles fit in one wave (the skinny low-rank products) has no next tile to hide its
//    epilogue behind either: the tensor-map store is 4 to 9 % ahead there;
//  * where the epilogue runs under the next tile's main loop the register store is kept (the staged store
//    costs a few per cent there).
struct Variant {
  int halves;
  bool tma_store;
};

bool wide_tile_fits(int64_t M, int64_t N) {
  const bool rows_fill = M % (4 * BM) == 0 || M >= 15 * 4 * BM;
  return M >= 4 * BM && N >= 4 * BN && rows_fill;
}

Variant variant_for(const GemmArgs& g, int ctas, bool store_ok) {
  const int pinned_halves = env_int("CT_B200_GEMM_MH", 0);
  const int pinned_store = env_int("CT_B200_GEMM_TMA_STORE", -1);
  const int64_t pair_tiles = ((g.M + 2 * BM - 1) / (2 * BM)) * ((g.N + BN - 1) / BN);
  Variant v;
  v.halves = 1;
  if (ctas == 2 && store_ok && wide_tile_fits(g.M, g.N)) v.halves = 2;
  if (ctas == 2 && (pinned_halves == 1 || pinned_halves == 2)) v.halves = pinned_halves;
  v.tma_store = store_ok && (v.halves == 2 || pair_tiles <= 74);
  if (pinned_store == 0) v.tma_store = false;
  if (pinned_store == 1) v.tma_store = store_ok;
  return v;
}

// Everything of a launch's TcParams that depends on the problem alone.
int fill_params(const GemmArgs& g, int ctas, const Variant& variant, TcParams* out) {
  TcParams& p = *out;
  int rc = CT_OK;
  p.splits = g.split_k > 1 ? g.split_k : 1;
  p.out_f32 = g.out_dtype == CT_F32;
  p.beta = g.beta;
  const int vec = p.out_f32 ? 4 : 8;
  p.vec_store = (reinterpret_cast<uintptr_t>(g.out) & 15) == 0 && g.ldo % vec == 0 &&
                (!g.residual || ((reinterpret_cast<uintptr_t>(g.residual) & 15) == 0 && g.ld_res % 8 == 0)) &&
                (!g.bias || (reinterpret_cast<uintptr_t>(g.bias) & 15) == 0);
  p.tma_store = variant.tma_store ? 1 : 0;
  const int halves = variant.halves;
  const int tile_m = BM * ctas * halves, b_rows = BN / ctas;
  const int stage_blocks = (ctas == 2 && halves == 1) ? 2 : 1;
  p.nseg = g.nseg;
  p.k_blocks_total = 0;
  for (int s = 0; s < g.nseg; ++s) {
    const Segment& sg = g.seg[s];
    TcSegment& t = p.seg[s];
    t.k_blocks = static_cast<int>((sg.k + BK - 1) / BK);
    p.k_blocks_total += t.k_blocks;
    t.a_mn = sg.a_cs == 1 ? 0 : 1;
    t.b_mn = sg.b_rs == 1 ? 0 : 1;
    t.n_half = t.d_col = t.b_k_block = t.b_k_offset = 0;
    // K-major: contiguous index is k, rows are m (or n). MN-major: contiguous index is m (or n), rows are k.
    // An MN-major operand is fetched in boxes of 64 columns x all the k rows of a ring stage (two k-blocks in the
    // 256 x 256 CTA-pair kernels, one elsewhere).
    rc = t.a_mn ? make_map(&t.a, sg.a, g.M, sg.k, sg.a_cs, BK * stage_blocks)
                : make_map(&t.a, sg.a, sg.k, g.M, sg.a_rs, BM * halves);
    if (rc != CT_OK) return rc;
    rc = t.b_mn ? make_map(&t.b, sg.b, g.N, sg.k, sg.b_rs, BK * stage_blocks)
                : make_map(&t.b, sg.b, sg.k, g.N, sg.b_cs, b_rows);
    if (rc != CT_OK) return rc;
  }
  if (p.tma_store) {
    rc = make_map(&p.out_map, g.out, g.N, g.M, g.ldo, 32, halves == 2 ? 32 : 64);
    if (rc != CT_OK) return rc;
  }
  p.m_tiles = static_cast<int>((g.M + tile_m - 1) / tile_m);
  p.n_tiles = static_cast<int>((g.N + BN - 1) / BN);
  {
    const int value = env_int("CT_B200_GEMM_GROUP_M", 0);
    p.group_m = value > 0 ? value : (halves == 2 ? GROUP_M / 2 : GROUP_M);   // the same 4096 rows per sweep
  }
  p.M = g.M;
  p.N = g.N;
  p.out = g.out;
  p.ldo = g.ldo;
  p.split_stride = g.M * g.ldo;
  p.bias = static_cast<const __nv_bfloat16*>(g.bias);
  p.residual = static_cast<const __nv_bfloat16*>(g.residual);
  p.ld_res = g.ld_res;
  p.error_flag = device_error_flag();
  if (!p.error_flag) return fail(CT_ERR_CUDA, "gemm_tcgen05: no device error flag");
  p.nf4_packed = nullptr;
  p.nf4_absmax = nullptr;
  p.nf4_code = nullptr;
  p.nf4_k = 0;
  p.gated = 0;
  p.gated_h = p.gated_g = p.gated_u = nullptr;
  p.gated_dh = nullptr;
  p.gated_ld = 0;
  p.gated_src_g = p.gated_src_u = nullptr;
  p.gated_src_ld = 0;
  return CT_OK;
}

int gemm_tcgen05(const GemmArgs& g, cudaStream_t stream) {
  if (!gemm_tcgen05_supported(g)) return fail(CT_ERR_UNSUPPORTED, "gemm_tcgen05: operands break a TMA rule");
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64)
    return fail(CT_ERR_CUDA, "gemm_tcgen05: no current device");
  const int ctas = ctas_for(g);
  // Tensor-map store: possible for a bf16 result that is written exactly once, rows 16-byte aligned.
  const bool store_ok = g.out_dtype != CT_F32 && !g.beta && g.split_k <= 1 &&
                        (reinterpret_cast<uintptr_t>(g.out) & 15) == 0 && g.ldo % 8 == 0;
  const Variant variant = variant_for(g, ctas, store_ok);
  TcParams p;
  int rc = fill_params(g, ctas, variant, &p);
  if (rc != CT_OK) return rc;
  const int64_t tiles = static_cast<int64_t>(p.m_tiles) * p.n_tiles * p.splits;
  int sms = sm_count();
  if (sms <= 0) return fail(CT_ERR_CUDA, "gemm_tcgen05: cannot read the SM count");
  const int64_t slots = sms / ctas;  // resident tiles: one CTA (or one CTA pair) per SM (pair)
  const unsigned grid = static_cast<unsigned>((tiles < slots ? tiles : slots) * ctas);
  const bool timed = timing_enabled();
  if (timed) timing_begin(stream);
  if (ctas == 2 && variant.halves == 2) {
    rc = launch_wide(p, grid, device, stream);
  } else if (ctas == 2) {
    rc = launch_pair<3, 2>(p, grid, device, stream);   // 3 stages of two 64-wide k-blocks: one barrier round per 8 MMAs
  } else {
    rc = launch_single(p, grid, device, stream);
  }
  if (rc != CT_OK) return rc;
  if (timed) {
    double k_total = 0;
    for (int s = 0; s < g.nseg; ++s) k_total += static_cast<double>(g.seg[s].k);
    timing_end(stream, 2.0 * static_cast<double>(g.M) * static_cast<double>(g.N) * k_total, g.M, g.N,
               static_cast<long long>(k_total));
  }
  count_launch(true);
  return check_launch("gemm_tcgen05");
}

// `count` independent products (2 .. kMaxGroup) in one launch of the CTA-pair kernel. Every problem must pass
// gemm_tcgen05_supported; outputs go through the register-store epilogue (fp32 slice planes, beta).
int gemm_tcgen05_group(const GemmArgs* problems, int count, cudaStream_t stream) {
  if (count < 1 || count > kMaxGroup) return fail(CT_ERR_ARG, "gemm_tcgen05_group: %d problems (1 .. %d)", count, kMaxGroup);
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64)
    return fail(CT_ERR_CUDA, "gemm_tcgen05_group: no current device");
  static TcGroup staging_area[64];          // 13 KB each: too large for the stack of a host thread to take lightly
  static std::mutex mutex;
  std::lock_guard<std::mutex> lock(mutex);
  TcGroup& group = staging_area[device];
  group.count = count;
  group.first[0] = 0;
  double flops = 0;
  const Variant plain{1, false};
  for (int i = 0; i < count; ++i) {
    if (!gemm_tcgen05_supported(problems[i]))
      return fail(CT_ERR_UNSUPPORTED, "gemm_tcgen05_group: problem %d breaks a TMA rule", i);
    const int rc = fill_params(problems[i], 2, plain, &group.problem[i]);
    if (rc != CT_OK) return rc;
    const TcParams& p = group.problem[i];
    group.first[i + 1] = group.first[i] + p.m_tiles * p.n_tiles * p.splits;
    double k_total = 0;
    for (int s = 0; s < problems[i].nseg; ++s) k_total += static_cast<double>(problems[i].seg[s].k);
    flops += 2.0 * static_cast<double>(problems[i].M) * static_cast<double>(problems[i].N) * k_total;
  }
  const int sms = sm_count();
  if (sms <= 0) return fail(CT_ERR_CUDA, "gemm_tcgen05_group: cannot read the SM count");
  const int64_t tiles = group.first[count], slots = sms / 2;
  const unsigned grid = static_cast<unsigned>((tiles < slots ? tiles : slots) * 2);
  static bool configured[64] = {};
  using S = Shape<2, 3, 2, 1>;
  const int rc = configure(gemm_tcgen05_group_kernel, S::kSmemBytes, &configured[device]);
  if (rc != CT_OK) return rc;
  const bool timed = timing_enabled();
  if (timed) timing_begin(stream);
  launch_dependent(gemm_tcgen05_group_kernel, dim3(grid), dim3(S::kThreads), S::kSmemBytes, stream, group);
  if (timed) timing_end(stream, flops, problems[0].M, problems[0].N, -count);   // k = -count marks a grouped launch
  count_launch(true);
  return check_launch("gemm_tcgen05_group");
}

// out[T, N] (bf16) = x[T, K] . dequant(W)^T with W[N, K] given as packed NF4 codes (two per byte, row-major), one
// fp32 absmax per 64 elements and the 16-entry code table: the decode runs inside the GEMM (four extra warps per
// CTA write the B tiles), so the dense weight never exists in memory. K must be a multiple of 64.
bool gemm_tcgen05_nf4_supported(const void* x, int64_t ldx, const void* packed, const void* absmax, const void* code,
                                const void* out, int64_t ldo, int64_t T, int64_t K, int64_t N) {
  if (T <= 0 || N <= 0 || K <= 0 || K % BK != 0) return false;
  if (T > (1LL << 31) - 2 * BM || N > (1LL << 31) - BN || K > (1LL << 31) - BK) return false;
  if (!x || !packed || !absmax || !code || !out) return false;
  if (!operand_ok(x, ldx, 1) || ldx < K) return false;
  if ((reinterpret_cast<uintptr_t>(packed) & 15) != 0 || (reinterpret_cast<uintptr_t>(absmax) & 3) != 0) return false;
  return ldo >= N;
}

int gemm_tcgen05_nf4(const void* x, int64_t ldx, const uint8_t* packed, const float* absmax, const float* code,
                     void* out, int64_t ldo, int64_t T, int64_t K, int64_t N, cudaStream_t stream) {
  if (!gemm_tcgen05_nf4_supported(x, ldx, packed, absmax, code, out, ldo, T, K, N))
    return fail(CT_ERR_UNSUPPORTED, "gemm_tcgen05_nf4: needs bf16 x with 16-byte aligned rows, K a multiple of 64, 16-byte aligned codes");
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64)
    return fail(CT_ERR_CUDA, "gemm_tcgen05_nf4: no current device");
  GemmArgs g;
  g.M = T; g.N = N; g.nseg = 1; g.in_dtype = CT_BF16;
  g.seg[0].a = x; g.seg[0].a_rs = ldx; g.seg[0].a_cs = 1;
  g.seg[0].b = x; g.seg[0].b_rs = 1; g.seg[0].b_cs = ldx; g.seg[0].k = K;     // B is never loaded: any valid map will do
  g.out = out; g.ldo = ldo; g.out_dtype = CT_BF16; g.beta = 0; g.bias = nullptr; g.residual = nullptr; g.ld_res = 0;
  g.split_k = 1;
  TcParams p;
  const Variant plain{1, false};
  int rc = fill_params(g, 2, plain, &p);
  if (rc != CT_OK) return rc;
  p.nf4_packed = packed;
  p.nf4_absmax = absmax;
  p.nf4_code = code;
  p.nf4_k = K;
  const int sms = sm_count();
  if (sms <= 0) return fail(CT_ERR_CUDA, "gemm_tcgen05_nf4: cannot read the SM count");
  const int64_t tiles = static_cast<int64_t>(p.m_tiles) * p.n_tiles, slots = sms / 2;
  const unsigned grid = static_cast<unsigned>((tiles < slots ? tiles : slots) * 2);
  static bool configured[64] = {};
  using S = Shape<2, 3, 2, 1>;
  rc = configure(gemm_tcgen05_nf4_kernel, S::kSmemBytes, &configured[device]);
  if (rc != CT_OK) return rc;
  const bool timed = timing_enabled();
  if (timed) timing_begin(stream);
  launch_dependent(gemm_tcgen05_nf4_kernel, dim3(grid), dim3(S::kThreads + 128), S::kSmemBytes, stream, p);
  if (timed) timing_end(stream, 2.0 * static_cast<double>(T) * static_cast<double>(N) * static_cast<double>(K), T, N, K);
  count_launch(true);
  return check_launch("gemm_tcgen05_nf4");
}

namespace {

int launch_gated(const TcParams& p, bool wide, double flops, int64_t M, int64_t N, int64_t K, const char* what,
                 cudaStream_t stream) {
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64)
    return fail(CT_ERR_CUDA, "%s: no current device", what);
  const int sms = sm_count();
  if (sms <= 0) return fail(CT_ERR_CUDA, "%s: cannot read the SM count", what);
  const int64_t tiles = static_cast<int64_t>(p.m_tiles) * p.n_tiles, slots = sms / 2;
  const unsigned grid = static_cast<unsigned>((tiles < slots ? tiles : slots) * 2);
  static bool configured[2][64] = {};
  using S = Shape<2, 3, 2, 1>;
  using W = Shape<2, 4, 1, 2>;
  const int rc = wide ? configure(gemm_tcgen05_gated_wide_kernel, W::kSmemBytes, &configured[1][device])
                      : configure(gemm_tcgen05_gated_kernel, S::kSmemBytes, &configured[0][device]);
  if (rc != CT_OK) return rc;
  const bool timed = timing_enabled();
  if (timed) timing_begin(stream);
  if (wide) launch_dependent(gemm_tcgen05_gated_wide_kernel, dim3(grid), dim3(W::kThreads), W::kSmemBytes, stream, p);
  else launch_dependent(gemm_tcgen05_gated_kernel, dim3(grid), dim3(S::kThreads), S::kSmemBytes, stream, p);
  if (timed) timing_end(stream, flops, M, N, K);
  count_launch(true);
  return check_launch(what);
}

bool aligned16(const void* pointer) { return (reinterpret_cast<uintptr_t>(pointer) & 15) == 0; }

}  // namespace

bool gemm_tcgen05_gated_supported(const GatedArgs& a) {
  if (a.T <= 0 || a.K <= 0 || a.N <= 0 || a.N % (BN / 2) != 0 || a.r_gate <= 0 || a.r_up <= 0) return false;
  if (a.T > (1LL << 31) - 2 * BM || 2 * a.N > (1LL << 31) - BN || a.K > (1LL << 31) - BK) return false;
  if (!a.x || !a.w_pair || !a.xa_gate || !a.xa_up || !a.b_gate || !a.b_up || !a.h) return false;
  if (!operand_ok(a.x, a.ldx, 1) || !operand_ok(a.w_pair, a.ldw, 1) || a.ldx < a.K || a.ldw < a.K) return false;
  if (!operand_ok(a.xa_gate, a.ld_xa, 1) || !operand_ok(a.xa_up, a.ld_xa, 1)) return false;
  if (!operand_ok(a.b_gate, a.r_gate, 1) || !operand_ok(a.b_up, a.r_up, 1)) return false;
  if (a.ld_out < a.N || a.ld_out % 8 != 0) return false;
  if (!aligned16(a.h) || !aligned16(a.gate) || !aligned16(a.up) || !aligned16(a.dh)) return false;
  if (a.dh && (!a.gate || !a.up)) return false;
  return true;
}

// One launch for gate(x), up(x) and the SwiGLU between them and the down projection. `w_pair` is
// [2 N, K]: rows [256 t, 256 t + 128) are rows [128 t, 128 t + 128) of the gate weight, the next 128 rows the
// same rows of the up weight. Forward (dh == null): h = silu(gate) * up, and gate / up themselves where
// their pointers are given (the cached mode). Backward (dh given): gate and up are recomputed in the
// accumulator and (d_gate, d_up, h) are written to (gate, up, h); h may be dh.
int gemm_tcgen05_gated(const GatedArgs& a, cudaStream_t stream) {
  if (!gemm_tcgen05_gated_supported(a))
    return fail(CT_ERR_UNSUPPORTED, "gemm_tcgen05_gated: needs bf16 operands with 16-byte aligned rows and a width that is a multiple of 128");
  GemmArgs g;
  g.M = a.T; g.N = 2 * a.N; g.nseg = 3; g.in_dtype = CT_BF16;
  g.seg[0].a = a.x; g.seg[0].a_rs = a.ldx; g.seg[0].a_cs = 1;
  g.seg[0].b = a.w_pair; g.seg[0].b_rs = 1; g.seg[0].b_cs = a.ldw; g.seg[0].k = a.K;
  g.seg[1].a = a.xa_gate; g.seg[1].a_rs = a.ld_xa; g.seg[1].a_cs = 1;
  g.seg[1].b = a.b_gate; g.seg[1].b_rs = 1; g.seg[1].b_cs = a.r_gate; g.seg[1].k = a.r_gate;
  g.seg[2].a = a.xa_up; g.seg[2].a_rs = a.ld_xa; g.seg[2].a_cs = 1;
  g.seg[2].b = a.b_up; g.seg[2].b_rs = 1; g.seg[2].b_cs = a.r_up; g.seg[2].k = a.r_up;
  g.out = a.h; g.ldo = a.ld_out; g.out_dtype = CT_BF16; g.beta = 0; g.bias = nullptr; g.residual = nullptr;
  g.ld_res = 0; g.split_k = 1;
  TcParams p;
  const Variant plain{1, false};
  int rc = fill_params(g, 2, plain, &p);
  if (rc != CT_OK) return rc;
  // The low-rank segments: B is [N, r], 64 rows of it per CTA, their MMAs cover half of the accumulator.
  for (int s = 1; s <= 2; ++s) {
    TcSegment& t = p.seg[s];
    rc = make_map(&t.b, g.seg[s].b, g.seg[s].k, a.N, g.seg[s].b_cs, BN / 4);
    if (rc != CT_OK) return rc;
    t.n_half = 1;
    t.d_col = s == 1 ? 0 : BN / 2;
  }
  p.gated = a.dh ? 2 : 1;
  p.gated_h = static_cast<__nv_bfloat16*>(a.h);
  p.gated_g = static_cast<__nv_bfloat16*>(a.gate);
  p.gated_u = static_cast<__nv_bfloat16*>(a.up);
  p.gated_dh = static_cast<const __nv_bfloat16*>(a.dh);
  p.gated_ld = a.ld_out;
  const double flops = 2.0 * static_cast<double>(a.T) * static_cast<double>(a.N) *
                       (2.0 * static_cast<double>(a.K) + static_cast<double>(a.r_gate + a.r_up));
  return launch_gated(p, false, flops, a.T, 2 * a.N, a.K, "gemm_tcgen05_gated", stream);
}

// dx[T, K] = (add ? dx : 0) + dg . W_gate + low_g . A_gate + du . W_up + low_u . A_up with the two weights read from
// the interleaved [2 N, K] buffer of gemm_tcgen05_gated (MN-major B: a k-block of 64 weight rows is 64 consecutive
// rows of the buffer).
int gemm_tcgen05_gated_input_gradient(const GatedGradientArgs& a, cudaStream_t stream) {
  GemmArgs g;
  g.M = a.T; g.N = a.K; g.nseg = 4; g.in_dtype = CT_BF16;
  const void* signal[2] = {a.dg, a.du};
  const void* low[2] = {a.low_gate, a.low_up};
  const void* adapter[2] = {a.a_gate, a.a_up};
  const int64_t rank[2] = {a.r_gate, a.r_up};
  for (int i = 0; i < 2; ++i) {
    Segment& base = g.seg[2 * i];
    base.a = signal[i]; base.a_rs = a.ld_signal; base.a_cs = 1;
    base.b = a.w_pair; base.b_rs = a.ldw; base.b_cs = 1; base.k = a.N;
    Segment& lora = g.seg[2 * i + 1];
    lora.a = low[i]; lora.a_rs = a.ld_low; lora.a_cs = 1;
    lora.b = adapter[i]; lora.b_rs = a.K; lora.b_cs = 1; lora.k = rank[i];
  }
  g.out = a.dx; g.ldo = a.ld_dx; g.out_dtype = CT_BF16; g.beta = a.add; g.bias = nullptr; g.residual = nullptr;
  g.ld_res = 0; g.split_k = 1;
  if (a.N % (BN / 2) != 0 || !gemm_tcgen05_supported(g))
    return fail(CT_ERR_UNSUPPORTED, "gemm_tcgen05_gated_input_gradient: operands break a TMA rule");
  TcParams p;
  // The 512 x 256 tile (tensor-map store) where the result is written once and its rows fill such tiles.
  const bool wide = !a.add && aligned16(a.dx) && a.ld_dx % 8 == 0 && wide_tile_fits(a.T, a.K) &&
                    env_int("CT_B200_GEMM_MH", 0) != 1;
  const Variant variant{wide ? 2 : 1, wide};
  int rc = fill_params(g, 2, variant, &p);
  if (rc != CT_OK) return rc;
  for (int i = 0; i < 2; ++i) {
    TcSegment& t = p.seg[2 * i];
    rc = make_map(&t.b, a.w_pair, a.K, 2 * a.N, a.ldw, wide ? BK : 2 * BK);     // all 2 N rows of the interleaved buffer
    if (rc != CT_OK) return rc;
    t.b_k_block = BN / 2;
    t.b_k_offset = i * (BN / 2);
  }
  const double flops = 2.0 * static_cast<double>(a.T) * static_cast<double>(a.K) *
                       (2.0 * static_cast<double>(a.N) + static_cast<double>(a.r_gate + a.r_up));
  return launch_gated(p, wide, flops, a.T, a.K, 2 * a.N + a.r_gate + a.r_up, "gemm_tcgen05_gated_input_gradient", stream);
}

// (d_gate, d_up, hidden) of a SwiGLU from the input gradient of the projection that follows it, in that
// projection's input-gradient GEMM: the accumulator dh = dy . W + low . A ([T, K], K the MLP width) is not stored;
// the epilogue reads the kept gate and up and applies the in-place backward to each element.
int gemm_tcgen05_gated_down_gradient(const GatedDownArgs& a, cudaStream_t stream) {
  GemmArgs g;
  g.M = a.T; g.N = a.K; g.nseg = a.r > 0 ? 2 : 1; g.in_dtype = CT_BF16;
  g.seg[0].a = a.dy; g.seg[0].a_rs = a.ld_dy; g.seg[0].a_cs = 1;
  g.seg[0].b = a.w; g.seg[0].b_rs = a.ldw; g.seg[0].b_cs = 1; g.seg[0].k = a.N;
  if (a.r > 0) {
    g.seg[1].a = a.low; g.seg[1].a_rs = a.ld_low; g.seg[1].a_cs = 1;
    g.seg[1].b = a.a; g.seg[1].b_rs = a.K; g.seg[1].b_cs = 1; g.seg[1].k = a.r;
  }
  g.out = a.hidden; g.ldo = a.ld_out; g.out_dtype = CT_BF16; g.beta = 0; g.bias = nullptr; g.residual = nullptr;
  g.ld_res = 0; g.split_k = 1;
  const bool pointers = aligned16(a.gate) && aligned16(a.up) && aligned16(a.d_gate) && aligned16(a.d_up) &&
                        aligned16(a.hidden) && a.gate && a.up && a.d_gate && a.d_up && a.hidden;
  if (!pointers || a.K % 32 != 0 || a.ld_out % 8 != 0 || a.ld_saved % 8 != 0 || a.ld_out < a.K || a.ld_saved < a.K ||
      !gemm_tcgen05_supported(g))
    return fail(CT_ERR_UNSUPPORTED, "gemm_tcgen05_gated_down_gradient: needs bf16 operands with 16-byte aligned rows and a width that is a multiple of 32");
  TcParams p;
  const Variant plain{1, false};
  const int rc = fill_params(g, 2, plain, &p);
  if (rc != CT_OK) return rc;
  p.gated = 3;
  p.gated_h = static_cast<__nv_bfloat16*>(a.hidden);
  p.gated_g = static_cast<__nv_bfloat16*>(a.d_gate);
  p.gated_u = static_cast<__nv_bfloat16*>(a.d_up);
  p.gated_ld = a.ld_out;
  p.gated_src_g = static_cast<const __nv_bfloat16*>(a.gate);
  p.gated_src_u = static_cast<const __nv_bfloat16*>(a.up);
  p.gated_src_ld = a.ld_saved;
  const double flops = 2.0 * static_cast<double>(a.T) * static_cast<double>(a.K) * static_cast<double>(a.N + a.r);
  return launch_gated(p, false, flops, a.T, a.K, a.N + a.r, "gemm_tcgen05_gated_down_gradient", stream);
}

int gemm_dispatch(const GemmArgs& g, int path, cudaStream_t stream) {
  if (g.M == 0 || g.N == 0) return CT_OK;
  if (path == CT_PATH_SIMT) return gemm_simt(g, stream);
  if (path == CT_PATH_TCGEN05) return gemm_tcgen05(g, stream);
  if (path != CT_PATH_AUTO) return fail(CT_ERR_ARG, "unknown path %d", path);
  return gemm_tcgen05_supported(g) ? gemm_tcgen05(g, stream) : gemm_simt(g, stream);
}

}  // namespace ct

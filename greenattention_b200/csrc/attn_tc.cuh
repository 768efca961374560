// FP8 paged attention for large query blocks (extend / chunked prefill) on the 5th-generation tensor
// cores: tcgen05.mma (kind::f8f6f4, e4m3 x e4m3 -> f32) with accumulators in tensor memory.
//
// Replaces the reference's SM90 WGMMA extend kernel (csrc/sm90/attn_decode_fp8/extend_kernel.cuh:162-457;
// work decomposition extend_kernel.cuh:140-160) for head_dim 128 and 256, any GQA, causal with an optional
// left window. Same math as the reference kernels: bf16 Q rounded to e4m3, S = scale * k_descale * Q K^T,
// bottom-right causal mask and left window, online softmax in the log2 domain, P rounded to e4m3, O = v_descale
// * P V / l, natural-log LSE (kernel.cuh:468-474,489-496,621-653).
//
// A CTA works on 128 query rows at a time (128 / GQA tokens x the GQA heads of one kv head) against the keys they
// can see, 128 keys per iteration, and is persistent: it walks a list of such segments (see TcWork) with tensor
// memory, barriers and pipelines set up once. 23 warps:
//   * one scheduler warp derives the CTA's segments a ring's depth ahead and publishes them in shared memory;
//   * four producer warps (K / V x even / odd tiles) gather pages with TMA (128-byte swizzle, one box per page
//     and 128-byte head slice, never multicast) into a K ring and a V ring;
//   * two issuing lanes in two warps of their own: one issues S = Q K^T with both operands K-major straight from
//     the swizzled tiles, the other O += P V with P as a K-major A operand from shared memory and V as an MN-major
//     B operand, i.e. the [token, dim] page layout as it is: no transpose of V anywhere. S (2 or 3 buffers of 128
//     columns) and O (head_dim columns) live in tensor memory;
//   * 16 softmax warps in two groups that alternate over the key tiles, two threads per query row (= tensor-memory
//     lane), one per half of the 128 keys. Each reads its S half-row with tcgen05.ld, exchanges the row maximum
//     with its partner through shared memory, runs the exp2 pass and writes P as e4m3 (plus a residual term while
//     a row rests on few keys, so that a probability carries ~2^-8 relative error) into swizzled shared memory,
//     and rescales O in tensor memory only when the running max moved by more than 1.5 in log2 (the stale max
//     keeps P below the e4m3 limit: 2^(7 + 1.5) < 448).
// The verify instance (REP: at most 32 query rows, replicated into the four lane quarters) has a softmax role of
// its own: four groups of 128 threads, four tiles in flight, one 32-row P tile per group and a deeper V ring.
// Every wait is bounded; a wait that runs out records a status word and the CTA drains to its common exit,
// where tensor memory is released.
#pragma once

#include "attn_rows.cuh"

namespace ga {
namespace attn {
namespace tc {

constexpr int TM = 128;             // query rows per CTA
constexpr int TNK = 128;            // keys per iteration
constexpr int SLAB = TNK * 128;     // one 128-byte-wide swizzled slab of a 128-row tile
constexpr float TC_SHIFT = 7.f;     // P = 2^(s - m + 7)
constexpr float TC_LAZY = 1.5f;     // rescale O only when the row max grew by more than this (log2 units)
// The residual term of P is kept while some thread's running share of a row sum is below this many "keys at the
// row maximum" (P = 2^7 there). A thread's share is a lower bound of the row's sum, so past it the row rests on at
// least that many effective keys and the e4m3 rounding of the single-term P (2^-4 relative per probability, the
// reference's P everywhere) averages out to about 2^-4 / sqrt(3 n) of the output scale. Measured against the oracle:
// flat rows (N(0, 0.5) keys) sit at 0.10 of the atol / rtol 2e-2 bound with 8 and at 0.05 with 32, peaked rows at 0.19
// with either (they keep the term); 8 takes 7 % off the windowed extend, where a thread's share of a 1 024-key
// window never reached 32.
#ifndef GA_TC_LO_KEYS
#define GA_TC_LO_KEYS 8
#endif
constexpr float TC_LO_BELOW = GA_TC_LO_KEYS * 128.f;

__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= static_cast<uint64_t>(1) << 46;  // descriptor version of sm_100
  d |= static_cast<uint64_t>(2) << 61;  // 128-byte swizzle
  return d;
}
// Instruction descriptor of kind::f8f6f4: f32 accumulate, e4m3 A and B, A K-major, B K-major or MN-major.
__device__ __forceinline__ uint32_t instr_desc(int m, int n, int b_mn_major) {
  return (1u << 4) | (static_cast<uint32_t>(b_mn_major) << 16) | (static_cast<uint32_t>(n >> 3) << 17) |
         (static_cast<uint32_t>(m >> 4) << 24);
}
__device__ __forceinline__ void mma_f8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, int accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// The same MMA with both descriptors given as (low, high) words. The issuing thread is a single lane whose
// instruction stream is the limit (about 90 cycles per MMA when each 64-bit descriptor is rebuilt, against
// 64 cycles of tensor time for M 128, N 128, K 32), so the high words are loop constants and a K step is one
// 32-bit add on the low word: the 14-bit address field (bytes / 16) never carries into the stride fields for
// addresses inside the 228 KiB window.
__device__ __forceinline__ void mma_f8_w(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi,
                                         uint32_t idesc, int accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tsetp.ne.b32 p, %6, 0;\n\t"
      "mov.b64 da, {%1, %2};\n\tmov.b64 db, {%3, %4};\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], da, db, %5, p;\n\t}"
      ::"r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,"
      "%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,"
      "%30,%31,%32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
        "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
        "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Verify instance: only the first 32 rows of the A operand of the PV MMAs are query rows, and whatever rows 32..127
// hold only reaches rows of O that nobody reads. So a P tile is 32 rows (4 KB), the MMA reads on into the tiles
// behind it, and the P region has room for one tile (both terms) per softmax group.
constexpr int TC_P4_BYTES = 32 * 128;

template <int HD, bool REP = false>
struct TcCfg {
  static constexpr int ATOMS = HD / 128;
  static constexpr int Q_BYTES = ATOMS * SLAB;
  static constexpr int P_BYTES = SLAB;                // one e4m3 term of P: 128 rows x 128 keys
  static constexpr int KV_BYTES = ATOMS * SLAB;       // one K (or V) tile
  static constexpr int NK = HD == 128 ? 4 : 2;        // depth of the K ring
  // Depth of the V ring. A V tile waits in its stage for the whole softmax of its keys (several thousand cycles
  // after the K tile that came with it is done), so where shared memory allows (the verify instance, whose P tiles
  // are small) the V ring is the deeper one: with four stages the stream of the verify call was bound by the turn-
  // around of a V stage, not by HBM.
  static constexpr int NV = REP ? (HD == 128 ? 7 : 3) : NK;
  // Header (barriers, row-max / row-sum exchange) first, then the 1024-byte aligned operand tiles. At head_dim
  // 256 this fills the 227 KiB of an SM exactly, so the kernel relies on the 1024-byte alignment it declares for
  // its dynamic shared memory and checks it at run time.
  static constexpr int BAR_OFF = 0;
  static constexpr int X_OFF = 512;                   // part maxima [2][2][128] bf16, running max [2][128] f32; row sums overlay both
  static constexpr int SEG_OFF = X_OFF + 2048;        // ring of segment descriptors written by the scheduler warp
  static constexpr int Q_OFF = 3072;
  static constexpr int P_OFF = Q_OFF + Q_BYTES;       // [buffer 0|1][hi|lo]; verify instance: [group][hi|lo] of 32 rows
  static constexpr int K_OFF = P_OFF + (REP ? 8 * TC_P4_BYTES : 4 * P_BYTES);
  static constexpr int V_OFF = K_OFF + NK * KV_BYTES;
  static constexpr int SMEM_BYTES = V_OFF + NV * KV_BYTES;
  static constexpr int TMEM_COLS = 512;
  // Tensor memory: NS score buffers of 128 columns, then O (head_dim columns). Head dim 128 leaves room for a
  // third score buffer, so the QK MMAs of tile t + 2 need not wait for the softmax of tile t.
  static constexpr int NS = HD == 128 ? 3 : 2;
  static constexpr int S_COL = 0;
  static constexpr int O_COL = NS * 128;
  static_assert(SMEM_BYTES <= SMEM_OPTIN, "shared memory");
};

// Position in a ring of N stages for the issuing lanes: the stage and the parity of its use count, kept by
// increments (a lane's instruction stream is what bounds a tile there, and % and / by 3 or 7 are not cheap).
template <int N>
struct RingPos {
  int i = 0;
  uint32_t par = 0;
  __device__ __forceinline__ void advance() {
    if (++i == N) {
      i = 0;
      par ^= 1u;
    }
  }
};

// Bounded wait that never returns early from the kernel: a wait that runs out is recorded and every later
// wait of this thread is skipped, so all warps still reach the common exit.
__device__ __forceinline__ void wait_or_flag(uint32_t bar, uint32_t parity, bool& failed, int* status, int code) {
  if (failed) return;
  if (!mbar_wait(bar, parity)) {
    failed = true;
    atomicExch(status, code);
  }
}

// exp2 pass over N = 32 (or 16) scores of one row held in registers: P = 2^(v * sl2 + sh) as e4m3 (plus the residual term when
// LO) into two 16-byte chunks of the swizzled P row(s); returns the sum of the unrounded P. MASK and LO are template
// parameters so that the common tile (below the diagonal, long row) runs the bare FFMA / EX2 / FADD / CVT sequence.
template <bool MASK, bool LO, int N = 32>
__device__ __forceinline__ float exp_chunk32(const uint32_t (&v)[N], float sl2, float sh, int col0, int pos, int lo_key,
                                             uint32_t p_hi, uint32_t p_lo, uint32_t chunk0, uint32_t rx) {
  float l4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int c16 = 0; c16 < N / 16; ++c16) {  // 16 keys = one 16-byte chunk of the P row
    uint32_t hi[4], lo[4];
#pragma unroll
    for (int q4 = 0; q4 < 4; ++q4) {
      float e[4], h[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int jj = c16 * 16 + q4 * 4 + j;
        float x = fmaf(__uint_as_float(v[jj]), sl2, sh);
        if (MASK) {
          const int col = col0 + jj;
          x = (col <= pos && col >= lo_key) ? x : -INFINITY;
        }
        e[j] = ex2(x);
        l4[j] += e[j];
        if (LO) h[j] = __uint_as_float((__float_as_uint(e[j]) + 0x00080000u) & 0xfff00000u);
      }
      if (LO) {
        hi[q4] = pack_e4m3x4(h[0], h[1], h[2], h[3]);
        lo[q4] = pack_e4m3x4(e[0] - h[0], e[1] - h[1], e[2] - h[2], e[3] - h[3]);
      } else {
        hi[q4] = pack_e4m3x4(e[0], e[1], e[2], e[3]);
      }
    }
    const uint32_t chunk = ((chunk0 + c16) ^ rx) << 4;
    asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(p_hi + chunk), "r"(hi[0]), "r"(hi[1]), "r"(hi[2]),
                 "r"(hi[3])
                 : "memory");
    if (LO)
      asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(p_lo + chunk), "r"(lo[0]), "r"(lo[1]), "r"(lo[2]),
                   "r"(lo[3])
                   : "memory");
  }
  return (l4[0] + l4[1]) + (l4[2] + l4[3]);
}

// The same pass with the result kept in registers (32 already masked scores of one row): the e4m3 words of the
// row's two 16-byte chunks, and of the residual term when LO. Lets a thread finish its exp2 work before the P
// buffer it will store to is free.
template <bool LO>
__device__ __forceinline__ float exp_regs32(const uint32_t (&v)[32], float sl2, float sh, uint32_t (&hi)[8], uint32_t (&lo)[8]) {
  float l4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int q4 = 0; q4 < 8; ++q4) {
    float e[4], h[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      e[j] = ex2(fmaf(__uint_as_float(v[q4 * 4 + j]), sl2, sh));
      l4[j] += e[j];
      if (LO) h[j] = __uint_as_float((__float_as_uint(e[j]) + 0x00080000u) & 0xfff00000u);
    }
    if (LO) {
      hi[q4] = pack_e4m3x4(h[0], h[1], h[2], h[3]);
      lo[q4] = pack_e4m3x4(e[0] - h[0], e[1] - h[1], e[2] - h[2], e[3] - h[3]);
    } else {
      hi[q4] = pack_e4m3x4(e[0], e[1], e[2], e[3]);
    }
  }
  return (l4[0] + l4[1]) + (l4[2] + l4[3]);
}

// Class of the 32 key columns starting at `col0` for the 32 rows of a warp (row of this lane: visible keys are
// [lo_key, pos], pos = -1 for a padding row): 4 = no row sees any of them, 0 = every row sees all of them, else a
// mixed chunk with bit 0 set when some row is cut by its upper bound (the causal diagonal) and bit 1 when some row
// is cut by its lower bound (the window edge). Warp-uniform; all lanes call it together.
__device__ __forceinline__ int chunk_class(int col0, int pos, int lo_key) {
  if (__all_sync(0xffffffffu, col0 > pos || col0 + 31 < lo_key)) return 4;
  const int hi = __all_sync(0xffffffffu, col0 + 31 <= pos) ? 0 : 1;
  const int lo = __all_sync(0xffffffffu, col0 >= lo_key) ? 0 : 2;
  return hi | lo;
}
// Masks a mixed chunk of raw scores in registers (hidden keys become -inf) and folds the visible ones into the
// four partial maxima. HI / LO: which of the two bounds can cut a row of this warp here.
template <bool HI, bool LO>
__device__ __forceinline__ void mask_chunk32(uint32_t (&v)[32], int col0, int pos, int lo_key, float (&m4)[4]) {
#pragma unroll
  for (int j = 0; j < 32; ++j) {
    const int col = col0 + j;
    const bool vis = (!HI || col <= pos) && (!LO || col >= lo_key);
    const float x = vis ? __uint_as_float(v[j]) : -INFINITY;
    v[j] = __float_as_uint(x);
    m4[j & 3] = fmaxf(m4[j & 3], x);
  }
}

// Optional timeline of one CTA (build with -DGA_TC_TRACE): a handful of threads, one per role, append
// (event, tile, SM clock) words to a device array that a profiling script reads back. Compiles to nothing
// in the product build.
#ifdef GA_TC_TRACE
constexpr int TC_TRACE_ROLES = 8, TC_TRACE_CAP = 8192;
__device__ long long g_tc_trace[TC_TRACE_ROLES][TC_TRACE_CAP];
#ifdef GA_TC_ACC
// Cheaper variant: per role and event kind, the summed cycles since the role's event before (words [kind]) and the
// number of times (words [256 + kind]), by fire-and-forget reductions.
#define TC_TRACE(kind, tile)                                                                                    \
  do {                                                                                                          \
    if (trc != nullptr) {                                                                                       \
      const unsigned now_ = static_cast<unsigned>(clock());                                                    \
      atomicAdd(reinterpret_cast<unsigned long long*>(trc) + ((kind) & 255), static_cast<unsigned long long>(now_ - static_cast<unsigned>(trc_n))); \
      atomicAdd(reinterpret_cast<unsigned long long*>(trc) + 256 + ((kind) & 255), 1ull);                       \
      trc_n = static_cast<int>(now_);                                                                           \
    }                                                                                                           \
  } while (0)
#else
#define TC_TRACE(kind, tile)                                                                                    \
  do {                                                                                                          \
    if (trc != nullptr && trc_n < TC_TRACE_CAP)                                                                 \
      trc[trc_n++] = (static_cast<long long>(((kind) << 16) | ((tile) & 0xffff)) << 40) | (clock64() & 0xffffffffffll); \
  } while (0)
#endif
#else
#define TC_TRACE(kind, tile)
#endif
// Second optional instrument (-DGA_TC_TRACE -DGA_TC_LANEACC): the two MMA-issuing lanes sum the cycles of their
// loop stages in registers and write the sums once, at the end, so the loop itself is not disturbed.
#if defined(GA_TC_TRACE) && defined(GA_TC_LANEACC)
#define LANE_ACC_DECL unsigned la_[8] = {0, 0, 0, 0, 0, 0, 0, 0}, la_t_ = static_cast<unsigned>(clock()), la_n_ = 0
#define LANE_ACC(i)                                   \
  do {                                                \
    const unsigned now_ = static_cast<unsigned>(clock()); \
    la_[i] += now_ - la_t_;                           \
    la_t_ = now_;                                     \
  } while (0)
#define LANE_ACC_TILE ++la_n_
#define LANE_ACC_DUMP(role)                                                         \
  do {                                                                              \
    if (blockIdx.x == 3 && lane == 0) {                                             \
      for (int i_ = 0; i_ < 8; ++i_) g_tc_trace[role][i_] = la_[i_];                \
      g_tc_trace[role][8] = la_n_;                                                  \
    }                                                                               \
  } while (0)
#else
#define LANE_ACC_DECL
#define LANE_ACC(i)
#define LANE_ACC_TILE
#define LANE_ACC_DUMP(role)
#endif

// Threads: 16 softmax warps, 4 producer warps, 2 MMA-issuing warps, 1 scheduler warp.
constexpr int TC_SOFTMAX = 512;
constexpr int TC_GROUP = 256;
constexpr int TC_GROUP4 = 128;   // verify instance: four softmax groups of four warps
constexpr int TC_THREADS = TC_SOFTMAX + 224;
constexpr int SEGQ = 8;          // depth of the segment ring
constexpr int SEG_WORDS = 10;    // b, h, q0, nq, pos0, L, t_lo, t_hi, slot, valid
constexpr int SEG_READERS = 22;  // warps that consume every segment: 16 softmax, 4 producers, 2 issuing

// Work source of a persistent CTA, run by its scheduler warp (all 32 lanes call next()).
//   mode 0 (decode / verify route): the call is one stream of 128-key tiles and contiguous slices of it go to the
//     CTAs, exactly as in the warp-level decode kernel, so any batch and any mix of lengths balances to one tile; a
//     unit that a slice cuts is finished by the combine kernel from the partial (O, LSE) the CTAs leave in the
//     workspace slots. With `p.gang` the CTAs work in gangs of kv_heads: a unit is a whole request, a slice belongs
//     to a gang, and CTA (gang, h) runs kv head h of it. The kv heads of a page (128-byte pieces of each token's
//     kv_heads * 128 bytes) are then fetched by neighbouring SMs at the same time, and DRAM sees the contiguous run
//     of the page instead of one piece in eight: measured 6.8 - 7.1 TB/s against 5.3 - 5.8 TB/s for the same gather
//     with every CTA on its own (request, kv head) units.
//   mode 1 (extend): items are (query block, kv head) pairs, latest (heaviest) blocks first; item i is block
//     i % nblk of kv head i / nblk, where nblk is the host's upper bound on the number of blocks (items past the
//     real count are skipped). CTAs claim items one at a time from a counter in the workspace header, so SMs that
//     drew lighter items take more of them; the last CTA to finish puts the counters back to zero for the next call.
struct TcWork {
  SliceWalker walk;
  int mode, item_end, nblk;
  int* counters;  // [0] next item, [1] CTAs that have finished claiming
  __device__ void init(const AttnDev& p, int lane) {
    mode = p.tc_mode;
    nblk = p.nblk;
    item_end = p.nblk * p.kvh;
    counters = p.status + 1;
    if (mode == 0 && p.gang) walk.init(p, blockIdx.x / p.kvh, gridDim.x / p.kvh, lane, TNK, 1);
    else if (mode == 0) walk.init(p, blockIdx.x, gridDim.x, lane, TNK);
  }
  __device__ bool next(const AttnDev& p, int lane, Seg& s) {
    if (mode == 0) {
      if (!walk.next(p, s)) return false;
      if (p.gang) {  // the walker speaks of gangs and whole requests: this CTA's kv head and its own slots
        s.h = blockIdx.x % p.kvh;
        if (s.slot >= 0) s.slot = 2 * static_cast<int>(blockIdx.x) + (s.slot & 1);
      }
      return true;
    }
    while (true) {
      int i = 0;
      if (lane == 0) i = atomicAdd(counters, 1);
      i = __shfl_sync(0xffffffffu, i, 0);
      if (i >= item_end) return false;
      const int h = i / nblk;
      if (extend_block(p, i - h * nblk, h, TNK, lane, s)) return true;
    }
  }
  // Called once by every CTA after its last claim.
  __device__ void finish(int lane) {
    if (mode == 1 && lane == 0) {
      __threadfence();
      if (atomicAdd(counters + 1, 1) == static_cast<int>(gridDim.x) - 1) {
        atomicExch(counters, 0);
        atomicExch(counters + 1, 0);
      }
    }
  }
};

// REP: instance for calls with at most 32 rows per kv head (see the softmax section); extend uses REP = false so
// that its inner loops carry none of that mode's branches.
//
// The CTA is persistent: tensor memory, barriers and the zeroed parts of shared memory are set up once and the
// CTA then walks its segments (TcWork). Ring stages, score buffers, P buffers and the running-max chain are
// indexed by the CTA's running tile count `it`, so the producers, the two issuing lanes and the softmax groups
// run on across segment boundaries: the K/V tiles of the next segment are in flight while the current one is
// in its last tiles and its epilogue. Two more barriers order what a segment boundary shares: `qfree` (the last
// QK MMA of a segment has read the Q tile, committed by the QK lane) before the softmax warps overwrite Q, and
// `ofree` (every softmax thread has read O out of tensor memory) before the PV lane starts a new accumulation.
// Q of segment `s`: each of the 512 softmax threads takes 16-element chunks of the 128 x HD tile, rounds them to
// e4m3 and stores them into the swizzled A tile at `sQ`.
template <int HD, bool REP>
__device__ __forceinline__ void load_q_body(const AttnDev& p, const Seg& s, uint32_t sQ, int tid) {
      // 16-element chunks of the 128 x HD tile are dealt to the 512 threads so that the lanes of a warp read whole
      // rows (32 contiguous bytes per lane, 2 or 4 rows per warp) instead of one 32-byte piece from each of 32 rows.
      constexpr int NC = HD / 64;   // chunks per thread
      constexpr int CPR = HD / 16;  // chunks per row
      uint4 x[NC], y[NC];           // all global loads are issued before the first conversion
  #pragma unroll
      for (int i = 0; i < NC; ++i) {
        const int id = i * TC_SOFTMAX + tid, row = id / CPR, c = id - row * CPR;
        const int qrow = REP ? (row & 31) : row;
        const int tq = qrow / p.gqa, hq = qrow - tq * p.gqa;
        x[i] = y[i] = make_uint4(0, 0, 0, 0);
        if (tq < s.nq) {
          const long long off = static_cast<long long>(s.q0 + tq) * p.q_s0 + static_cast<long long>(s.h * p.gqa + hq) * p.q_s1 + c * 16;
          if (p.q_bf16) {
            const uint4* src = reinterpret_cast<const uint4*>(p.q + off * 2);
            x[i] = src[0];
            y[i] = src[1];
          } else {
            x[i] = *reinterpret_cast<const uint4*>(p.q + off);
          }
        }
      }
  #pragma unroll
      for (int i = 0; i < NC; ++i) {
        const int id = i * TC_SOFTMAX + tid, row = id / CPR, c = id - row * CPR;
        uint4 pk = x[i];
        if (p.q_bf16) {
          auto cv = [](uint32_t a, uint32_t b) {
            return pack_e4m3x4(bf16_bits_to_f32(a & 0xffffu), bf16_bits_to_f32(a >> 16), bf16_bits_to_f32(b & 0xffffu),
                               bf16_bits_to_f32(b >> 16));
          };
          pk = make_uint4(cv(x[i].x, x[i].y), cv(x[i].z, x[i].w), cv(y[i].x, y[i].y), cv(y[i].z, y[i].w));
        }
        const uint32_t dst = sQ + (c >> 3) * SLAB + row * 128 + (((c & 7) ^ (row & 7)) << 4);
        asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(dst), "r"(pk.x), "r"(pk.y), "r"(pk.z), "r"(pk.w)
                     : "memory");
      }
}
template <int HD, bool REP>
__global__ void __launch_bounds__(TC_THREADS, 1)
attn_tc_kernel(const __grid_constant__ AttnDev p, const __grid_constant__ CUtensorMap kmap,
               const __grid_constant__ CUtensorMap vmap) {
  using C = TcCfg<HD, REP>;
  constexpr int CW = TNK / 2;          // key columns per softmax thread (two threads per row and tile)
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t base = smem_u32(smem_raw);
  if (base & 1023u) {  // the swizzled tiles need 1024-byte alignment; never seen, but never silently wrong
    if (threadIdx.x == 0) atomicExch(p.status, GA_ST_BAD_PAGE);
    return;
  }
  uint8_t* gen = smem_raw;
  const uint32_t sQ = base + C::Q_OFF, sP = base + C::P_OFF, sK = base + C::K_OFF, sV = base + C::V_OFF;
  const uint32_t bars = base + C::BAR_OFF;
  // barrier slots; the [2] ones are indexed by tile parity = softmax group
  const uint32_t b_q = bars, b_sfull = bars + 8, b_sfree = bars + 32, b_pready = bars + 56, b_pfree = bars + 72,
                 b_mpub = bars + 88;
  const uint32_t b_kfull = bars + 104, b_kempty = b_kfull + 8 * C::NK, b_vfull = b_kempty + 8 * C::NK,
                 b_vempty = b_vfull + 8 * C::NV;
  const uint32_t b_qfree = b_vempty + 8 * C::NV, b_ofree = b_qfree + 8;
  const uint32_t b_segfull = b_ofree + 8, b_segfree = b_segfull + 8 * SEGQ;
  const uint32_t b_mpub4 = b_segfree + 8 * SEGQ;  // verify instance: one running-max barrier per softmax group
  const uint32_t b_pready4 = base + C::SEG_OFF + SEGQ * SEG_WORDS * 4;  // verify instance: one P tile per group
  static_assert(C::SEG_OFF + SEGQ * SEG_WORDS * 4 + 32 + 8 + 16 + 48 + 16 <= C::Q_OFF, "words behind the segment ring overrun the Q tile");
  const int* segq = reinterpret_cast<const int*>(gen + C::SEG_OFF);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(gen + C::SEG_OFF + SEGQ * SEG_WORDS * 4 + 32);  // behind b_pready4
  uint32_t* lo_flag = tmem_slot + 2;  // [group][2]: the residual term of P is wanted for the group's tile 2u + g
  uint32_t* lo4 = lo_flag + 4;        // verify instance, [group][3]: the same vote, from a group's tile to its next one
  uint32_t* lo_term = lo4 + 12;       // verify instance, [group]: the group's P tile has its residual term
  __nv_bfloat16* mxbuf = reinterpret_cast<__nv_bfloat16*>(gen + C::X_OFF);  // [group][part][128], rounded up
  float* mrun = reinterpret_cast<float*>(gen + C::X_OFF + 1024);            // [group][128] running max after a tile
  float* lbuf = reinterpret_cast<float*>(gen + C::X_OFF);  // [4][128] row sums, after the last tile (overlay)
  static_assert(104 + 16 * C::NK + 16 * C::NV + 16 + 16 * SEGQ + 32 <= C::X_OFF, "barrier block overruns the exchange buffers");
  static_assert(C::SEG_OFF + SEGQ * SEG_WORDS * 4 <= C::Q_OFF, "segment ring overruns the Q tile");

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    mbar_init(b_q, TC_SOFTMAX);
    mbar_init(b_qfree, 1);
    mbar_init(b_ofree, TC_SOFTMAX);
    for (int i = 0; i < SEGQ; ++i) {
      mbar_init(b_segfull + 8 * i, 1);
      mbar_init(b_segfree + 8 * i, SEG_READERS);
    }
    constexpr int GROUP = REP ? TC_GROUP4 : TC_GROUP;  // softmax threads per tile
    for (int i = 0; i < 2; ++i) {
      mbar_init(b_pready + 8 * i, GROUP);
      mbar_init(b_pfree + 8 * i, 1);
      // verify instance: the two slots after b_pfree are P-buffer barriers too (four in turn, one per group: a
      // group's wait then never looks at a barrier that can be two phases behind)
      mbar_init(b_mpub + 8 * i, REP ? 1 : TC_GROUP);
    }
    for (int i = 0; i < 4; ++i) {
      mbar_init(b_mpub4 + 8 * i, TC_GROUP4);
      mbar_init(b_pready4 + 8 * i, TC_GROUP4);
    }
    for (int i = 0; i < C::NS; ++i) {
      mbar_init(b_sfull + 8 * i, 1);
      mbar_init(b_sfree + 8 * i, GROUP);
    }
    for (int i = 0; i < C::NK; ++i) {
      mbar_init(b_kfull + 8 * i, 1);
      mbar_init(b_kempty + 8 * i, 1);
    }
    for (int i = 0; i < C::NV; ++i) {
      mbar_init(b_vfull + 8 * i, 1);
      mbar_init(b_vempty + 8 * i, 1);
    }
    lo_flag[0] = lo_flag[1] = lo_flag[2] = lo_flag[3] = 0u;
    for (int i = 0; i < 16; ++i) lo4[i] = 0u;
    mbar_fence_init();
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(C::TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  bool failed = false;
  int it = 0;  // tiles of this CTA so far: position in every ring, shared by all roles
  int sq = 0;  // segments with at least one tile so far: phase of the Q / O hand-over barriers
  int sk = 0;  // segments read from the scheduler's ring so far
#ifdef GA_TC_TRACE
  long long* trc = nullptr;
  int trc_n = 0;
  if (blockIdx.x == 3) {
    int role = tid == 0 ? 0 : tid == 256 ? 1 : tid == 640 ? 2 : tid == 672 ? 3 : tid == 512 ? 4 : tid == 544 ? 5 : (REP && tid == 128) ? 6 : (REP && tid == 384) ? 7 : -1;
#ifdef GA_TC_TRACE_MASK
    if (role >= 0 && !((GA_TC_TRACE_MASK >> role) & 1)) role = -1;
#endif
    if (role >= 0) trc = g_tc_trace[role];
  }
#endif
  // Segment `k` of this CTA from the scheduler's ring (all lanes of a consumer warp call this together). With
  // `release` the warp hands the ring slot back; a peek at the next segment leaves it in place. False at the end
  // of the list or after a wait ran out anywhere in the warp.
  auto read_seg = [&](int k, Seg& s, bool release) -> bool {
    const int slot = k % SEGQ;
    wait_or_flag(b_segfull + 8 * slot, (k / SEGQ) & 1, failed, p.status, GA_ST_WAIT_FULL);
    TC_TRACE(17, k);
    failed = __any_sync(0xffffffffu, failed);
    if (failed) return false;
    const int* q = segq + slot * SEG_WORDS;
    s.b = q[0], s.h = q[1], s.q0 = q[2], s.nq = q[3], s.pos0 = q[4], s.L = q[5], s.t_lo = q[6], s.t_hi = q[7], s.slot = q[8];
    const bool valid = q[9] != 0;
    if (release) {
      __syncwarp();
      if (lane == 0) mbar_arrive(b_segfree + 8 * slot);
    }
    return valid;
  };
  Seg cur;

  // Q of segment `s`: a quarter of this thread's row, rounded to e4m3, into the swizzled A tile; then the
  // arrival that lets the QK lane start the segment.
  auto load_q = [&](const Seg& s) {
    load_q_body<HD, REP>(p, s, sQ, tid);
    TC_TRACE(18, 0);
    fence_proxy_async();
    mbar_arrive(b_q);
  };

  if (warp >= 16 && warp < 20) {
    // ---------------------------------------------------------------- producers: four warps
    // One warp's issue loop (barrier wait, expect_tx, page lookup, TMA issue) takes more than a thousand cycles
    // per tile, so K and V have their own warps, and even and odd tiles too. With an odd ring depth the two warps
    // of a ring take turns on a stage; a warp's wait for a stage still never meets a barrier two phases behind,
    // because its own tile before (two tiles back) already waited for a later MMA than the one two turns ago.
    const int pw = warp - 16, kv = pw & 1, par = pw >> 1;
    PtWindow win;
    win.b = -1;
    win.base = win.cur = win.nxt = 0;
    if (lane == 0) tma_prefetch_desc(kv ? &vmap : &kmap);
    const int nbox = TNK / p.box_tok;
    while (read_seg(sk++, cur, true)) {
      const Seg& s = cur;
      const int n_tiles = s.t_hi - s.t_lo;
      for (int t = 0; t < n_tiles && !failed; ++t, ++it) {
        if ((it & 1) != par) continue;
        const int depth = kv ? C::NV : C::NK;
        const int st = it % depth, use = it / depth;
        const int n0 = (s.t_lo + t) * TNK;
        int boxes = 0;
        for (int i = 0; i < nbox; ++i) boxes += (n0 + i * p.box_tok) < s.L;
        const uint32_t bytes = static_cast<uint32_t>(boxes) * p.box_tok * 128 * C::ATOMS;
        const uint32_t full = (kv ? b_vfull : b_kfull) + 8 * st, empty = (kv ? b_vempty : b_kempty) + 8 * st;
        if (use > 0) wait_or_flag(empty, (use - 1) & 1, failed, p.status, GA_ST_WAIT_EMPTY);
        if (failed) break;
        TC_TRACE(40, it);
        if (lane == 0) mbar_expect_tx(full, bytes);
        __syncwarp();
        for (int i = 0; i < boxes; ++i) {
          const int n = n0 + i * p.box_tok;
          int page = pt_lookup(p, win, s.b, n >> p.page_shift, lane);
          if ((page < 0 || page >= p.num_pages) && lane == 0) atomicExch(p.status, GA_ST_BAD_PAGE);
          if (lane < C::ATOMS) {
            const uint32_t dst = (kv ? sV : sK) + st * C::KV_BYTES + lane * SLAB + i * p.box_tok * 128;
            tma_load_4d(dst, kv ? &vmap : &kmap, full, lane * 128, s.h, n & p.page_mask, page);
          }
        }
        TC_TRACE(41, it);
      }
    }
  } else if (warp == 20) {
    // ---------------------------------------------------------------- QK issue: one lane
    // The two issuing lanes (this one and the PV one) run on their own: the next scores are what a softmax group
    // waits for once it hands back its S buffer, so they must not queue behind the PV wait. A lane's own
    // instruction stream bounds a tile here (barrier tests, four to eight MMAs at 64 - 90 cycles of issue each, two
    // commits), so descriptors are whole 64-bit registers prepared before the waits, ring positions are kept by
    // increments and both barriers of a tile are tested in one round trip. (A second lane per stream, taking turns
    // at the issue, was measured: no gain, and a 25th warp costs every thread 8 registers.)
    const uint32_t id_qk = instr_desc(TM, TNK, 0);
    const uint64_t dq = smem_desc(sQ, 16, 1024), dk = smem_desc(sK, 16, 1024);
    RingPos<C::NK> kp;  // K stage of tile `it` and (it / NK) & 1
    RingPos<C::NS> sp;  // score buffer of tile `it` and (it / NS) & 1
    LANE_ACC_DECL;
    while (read_seg(sk++, cur, true)) {
      const int n_tiles = cur.t_hi - cur.t_lo;
      LANE_ACC(0);
      if (lane == 0 && n_tiles > 0 && !failed) {
        wait_or_flag(b_q, sq & 1, failed, p.status, GA_ST_WAIT_FULL);  // this segment's Q tile is in place
        LANE_ACC(1);
        TC_TRACE(20, it);
        for (int t = 0; t < n_tiles; ++t, ++it, kp.advance(), sp.advance()) {
          const uint64_t kb = dk + static_cast<uint64_t>(kp.i * (C::KV_BYTES >> 4));
          const uint32_t sd = tmem + C::S_COL + sp.i * 128;
          const uint32_t bk = b_kfull + 8 * kp.i, bs = b_sfree + 8 * sp.i;
          LANE_ACC(2);
          // both barriers at once when they are through already (the common case: one shared-memory round trip)
          if (!(mbar_test_wait(bk, kp.par) & (it < C::NS || mbar_test_wait(bs, sp.par ^ 1u)))) {
            wait_or_flag(bk, kp.par, failed, p.status, GA_ST_WAIT_FULL);
            LANE_ACC(3);
            TC_TRACE(21, it);
            if (it >= C::NS) wait_or_flag(bs, sp.par ^ 1u, failed, p.status, GA_ST_WAIT_EMPTY);
            if (failed) break;
          }
          LANE_ACC(4);
          TC_TRACE(22, it);
          tc_fence_after();
#pragma unroll
          for (int ks = 0; ks < HD / 32; ++ks) {
            const uint64_t off = static_cast<uint64_t>(((ks >> 2) * SLAB + (ks & 3) * 32) >> 4);
            mma_f8(sd, dq + off, kb + off, id_qk, ks > 0 ? 1 : 0);
          }
          LANE_ACC(5);
          mma_commit(b_kempty + 8 * kp.i);
          mma_commit(b_sfull + 8 * sp.i);
          LANE_ACC(6);
          LANE_ACC_TILE;
          TC_TRACE(23, it);
        }
        if (!failed) mma_commit(b_qfree);  // every QK MMA of the segment has read Q
      }
      if (n_tiles > 0) ++sq;
      __syncwarp();
    }
    LANE_ACC_DUMP(2);
  } else if (warp == 21) {
    // ---------------------------------------------------------------- PV issue: one lane
    // O += P V with V as an MN-major B operand covering all head dims in one instruction (N = head_dim: at 256
    // the second 128-dim slab is found through the leading-dimension stride of the descriptor).
    const uint32_t id_pv = instr_desc(TM, HD, 1);
    const uint64_t dp = smem_desc(sP, 16, 1024), dv = smem_desc(sV, SLAB, 1024);
    constexpr int PT = REP ? TC_P4_BYTES : C::P_BYTES;  // bytes of one term of a P tile
    constexpr int NG = REP ? 4 : 2;                     // softmax groups = P tiles
    const uint32_t b_pr = REP ? b_pready4 : b_pready;
    RingPos<C::NV> vp;  // V stage of tile `it` and (it / NV) & 1
    RingPos<NG> gp;     // softmax group of tile `it` and the parity of the group's tile count
    LANE_ACC_DECL;
    while (read_seg(sk++, cur, true)) {
      const int n_tiles = cur.t_hi - cur.t_lo;
      LANE_ACC(0);
      if (lane == 0 && n_tiles > 0 && !failed) {
        // the first PV MMA of a segment overwrites O: the epilogue of the segment before must have read it
        if (sq > 0) wait_or_flag(b_ofree, (sq - 1) & 1, failed, p.status, GA_ST_WAIT_EMPTY);
        LANE_ACC(1);
        TC_TRACE(30, it);
        for (int t = 0; t < n_tiles; ++t, ++it, vp.advance(), gp.advance()) {
          TC_TRACE(37, it);
          const int g = gp.i;
          const uint64_t vb = dv + static_cast<uint64_t>(vp.i * (C::KV_BYTES >> 4));
          const uint64_t pb = dp + static_cast<uint64_t>(g * 2 * (PT >> 4));
          const uint32_t bp = b_pr + 8 * g, bv = b_vfull + 8 * vp.i;
          LANE_ACC(2);
          if (!(mbar_test_wait(bp, gp.par) & mbar_test_wait(bv, vp.par))) {  // see the QK lane
            wait_or_flag(bp, gp.par, failed, p.status, GA_ST_WAIT_FULL);
            LANE_ACC(3);
            TC_TRACE(31, it);
            wait_or_flag(bv, vp.par, failed, p.status, GA_ST_WAIT_FULL);
            if (failed) break;
          }
          LANE_ACC(4);
          TC_TRACE(32, it);
          tc_fence_after();
          // residual term: always on the first tile of each group in a segment, later by the softmax threads' vote
          int terms;
          if (REP) {
            terms = *reinterpret_cast<volatile uint32_t*>(lo_term + g) != 0u ? 2 : 1;  // written before the group's arrivals
          } else {
            const bool voted = atomicExch(lo_flag + g * 2 + gp.par, 0u) != 0u;
            terms = (voted || t < 2) ? 2 : 1;
          }
          TC_TRACE(35, it);
#pragma unroll 1
          for (int term = 0; term < terms; ++term) {  // hi term, then the residual term while some row needs it
            const uint64_t pa = pb + static_cast<uint64_t>(term * (PT >> 4));
#pragma unroll
            for (int ks = 0; ks < TNK / 32; ++ks)
              mma_f8(tmem + C::O_COL, pa + static_cast<uint64_t>(ks * 2), vb + static_cast<uint64_t>(ks * (32 * 128 >> 4)), id_pv,
                     (t > 0 || term > 0 || ks > 0) ? 1 : 0);
          }
          TC_TRACE(36, it);
          LANE_ACC(5);
          mma_commit(b_vempty + 8 * vp.i);
          mma_commit(b_pfree + 8 * g);
          LANE_ACC(6);
          LANE_ACC_TILE;
          TC_TRACE(33 + (terms - 1), it);
        }
      }
      if (n_tiles > 0) ++sq;
      __syncwarp();
    }
    LANE_ACC_DUMP(3);
  } else if (warp == 22) {
    // ---------------------------------------------------------------- scheduler: one warp
    // Derives this CTA's segments (device split plan / item list, with the global reads that takes) a ring's depth
    // ahead of the warps that consume them, so neither those reads nor the walker's state sit in the other roles.
    TcWork work;
    work.init(p, lane);
    if (p.tc_mode == 0 && blockIdx.x == 0) publish_prefix(p, lane, TNK);  // for the combine kernel
    int* wq = reinterpret_cast<int*>(gen + C::SEG_OFF);
    for (int k = 0;; ++k) {
      const int slot = k % SEGQ;
      if (k >= SEGQ) wait_or_flag(b_segfree + 8 * slot, ((k / SEGQ) - 1) & 1, failed, p.status, GA_ST_WAIT_EMPTY);
      // extend items are claimed from a counter all CTAs share: take the next one only when every warp has picked
      // up the one before, so a CTA never sits on more than one item it has not started
      if (p.tc_mode == 1 && k >= 1)
        wait_or_flag(b_segfree + 8 * ((k - 1) % SEGQ), ((k - 1) / SEGQ) & 1, failed, p.status, GA_ST_WAIT_EMPTY);
      failed = __any_sync(0xffffffffu, failed);
      if (failed) break;
      Seg s;
      const bool more = work.next(p, lane, s);
      if (more && s.t_hi > s.t_lo) {
        // the segment's query rows, pulled into the L2 now: the softmax warps load them one segment from here
        const int esz = p.q_bf16 ? 2 : 1, lines = (HD * esz + 127) / 128, rows = s.nq * p.gqa;
        for (int i = lane; i < rows * lines; i += 32) {
          const int row = i / lines, ln = i - row * lines;
          const int tq = row / p.gqa, hq = row - tq * p.gqa;
          const uint8_t* a = p.q + (static_cast<long long>(s.q0 + tq) * p.q_s0 + static_cast<long long>(s.h * p.gqa + hq) * p.q_s1) * esz + ln * 128;
          asm volatile("prefetch.global.L2 [%0];" ::"l"(a));
        }
      }
      if (lane == 0) {
        int* q = wq + slot * SEG_WORDS;
        q[0] = s.b, q[1] = s.h, q[2] = s.q0, q[3] = s.nq, q[4] = s.pos0, q[5] = s.L, q[6] = s.t_lo, q[7] = s.t_hi, q[8] = s.slot;
        q[9] = more ? 1 : 0;
        mbar_arrive(b_segfull + 8 * slot);  // release: the words above are visible to whoever sees the phase
      }
      __syncwarp();
      if (!more) break;
    }
    work.finish(lane);
  } else if (REP && warp < 16) {
    // ---------------------------------------------------------------- softmax, verify instance: four groups of 128
    // At most 32 query rows (query tokens x GQA): the rows are replicated into all four 32-lane quarters of the Q
    // tile, so S comes out four times and the warp of quarter qt takes key columns [32 qt, 32 qt + 32) of all 32
    // rows, one row per lane (a warp can only read its own quarter of tensor memory, and a quarter maps to one
    // scheduler: without the replication the whole softmax would sit on one scheduler's exp2 unit). A group is the
    // four warps of one tile; group gq takes the tiles with running index = gq mod 4, so four tiles are in
    // flight: a tile's chain of dependent steps (scores, row max, exchange, exp2, P) is several times longer than
    // the time the HBM stream allows per tile, and only tiles in flight hide it. The 32 scores of a thread stay in
    // registers from the max pass to the exp2 pass, so the score buffer goes back to the QK lane right after it is
    // read. Each group has its own 32-row P tile (TC_P4_BYTES per term); O rows 0..31 are the result.
    const int gq = warp >> 2, qt = warp & 3, rr = lane;
    const bool owns_o = qt == 0;         // quarter 0 of O holds the result rows; warp (gq, 0) writes dims quarter gq
    const int col_first = 32 * qt;
    const uint32_t lane_base = tmem + (static_cast<uint32_t>(qt * 32) << 16);
    const uint32_t grp_bar = 2 + gq;     // named barrier of this group (128 threads)
    const int krow = tid & 127;          // key row of a V tile this thread keeps finite past the end of a sequence
    __nv_bfloat16* mx4 = mxbuf;          // [group][quarter][32], rounded up
    float* mrun4 = mrun;                 // [group][32] running max after a tile
    bool q_ready = false;
    int gn = 0;  // tiles of this group so far
    while (read_seg(sk++, cur, true)) {
      const Seg& s = cur;
      const int n_tiles = s.t_hi - s.t_lo;
      const bool valid = rr / p.gqa < s.nq;
      TC_TRACE(1, n_tiles);
      if (n_tiles <= 0) {
        if (valid && owns_o) {
          const int tq = rr / p.gqa, hq = rr - tq * p.gqa;
          __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(p.out) + static_cast<long long>(s.q0 + tq) * p.o_s0 +
                               static_cast<long long>(s.h * p.gqa + hq) * p.o_s1 + gq * (HD / 4);
          for (int c0 = 0; c0 < HD / 4; c0 += 8) *reinterpret_cast<uint4*>(dst + c0) = make_uint4(0, 0, 0, 0);
          if (gq == 0 && p.lse != nullptr)
            p.lse[static_cast<long long>(s.h * p.gqa + hq) * p.total_q + s.q0 + tq] = -INFINITY;
        }
        continue;
      }
      if (!q_ready) {
        if (sq > 0) wait_or_flag(b_qfree, (sq - 1) & 1, failed, p.status, GA_ST_WAIT_EMPTY);
        load_q(s);
      }
      q_ready = false;
      TC_TRACE(2, it);
      const int pos = valid ? s.pos0 + rr / p.gqa : -1;
      const int lo_key = p.window_left >= 0 ? pos - p.window_left : -(1 << 30);
      const float sl2 = p.scale_log2 * (p.kd ? p.kd[s.b * p.kd_s0 + s.h * p.kd_s1] : 1.f);
      float m_seen = -INFINITY, l = 0.f;  // l is relative to m_seen
      const int it0 = it;
      for (int t = (gq - it0) & 3; t < n_tiles; t += 4) {
        const int gi = it0 + t;           // running tile index: buffers and barrier phases
        const int n0 = (s.t_lo + t) * TNK;
        const int c_base = n0 + col_first;
        const bool need_mask = (n0 + TNK > s.pos0 + 1) || (p.window_left >= 0 && n0 < s.pos0 + s.nq - 1 - p.window_left);
        const int sb = gi % C::NS;
        TC_TRACE(3, gi);
        // A parity wait tells "phase j done" from "phase j - 1 still pending" only while the barrier is at most one
        // phase behind. The tile that had this score buffer before (gi - NS) is another group's, and nothing this
        // group has waited for so far proves that its scores exist; that group's published max does (its barrier
        // cannot be two phases behind: the chain of max hand-overs this group joined at tile gi - 4 covers tile
        // gi - 7). 
        if (gi >= C::NS) wait_or_flag(b_mpub4 + 8 * ((gi - C::NS) & 3), ((gi - C::NS) >> 2) & 1, failed, p.status, GA_ST_WAIT_FULL);
        wait_or_flag(b_sfull + 8 * sb, (gi / C::NS) & 1, failed, p.status, GA_ST_WAIT_FULL);
        TC_TRACE(4, gi);
        tc_fence_after();
        uint32_t v[32];
        tmem_ld32(lane_base + C::S_COL + sb * 128 + col_first, v);
        tmem_wait_ld();
        tc_fence_before();
        mbar_arrive(b_sfree + 8 * sb);  // the scores are in registers: the buffer may take a later tile
        float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
        if (need_mask) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int col = c_base + j;
            const float x = (col <= pos && col >= lo_key) ? __uint_as_float(v[j]) : -INFINITY;
            v[j] = __float_as_uint(x);
            m4[j & 3] = fmaxf(m4[j & 3], x);
          }
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) m4[j & 3] = fmaxf(m4[j & 3], __uint_as_float(v[j]));
        }
        float mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3])) * sl2;  // sl2 > 0; -inf stays -inf
        mx4[(gq * 4 + qt) * 32 + rr] = __float2bfloat16_ru(mx);
        TC_TRACE(5, gi);
        // the running max after the tile before (another group's), and this tile's P buffer (free once the PV MMAs
        // of the tile two before are done; the residual flag of this tile is complete by then)
        float m_prev = -INFINITY;
        if (gi >= 1) {
          wait_or_flag(b_mpub4 + 8 * ((gi - 1) & 3), ((gi - 1) >> 2) & 1, failed, p.status, GA_ST_WAIT_FULL);
          if (t >= 1) m_prev = mrun4[((gi - 1) & 3) * 32 + rr];
        }
        TC_TRACE(6, gi);
        named_bar_sync(grp_bar, TC_GROUP4);
        TC_TRACE(7, gi);
        mx = fmaxf(fmaxf(__bfloat162float(mx4[(gq * 4) * 32 + rr]), __bfloat162float(mx4[(gq * 4 + 1) * 32 + rr])),
                   fmaxf(__bfloat162float(mx4[(gq * 4 + 2) * 32 + rr]), __bfloat162float(mx4[(gq * 4 + 3) * 32 + rr])));
        float m_new = m_prev, alpha = 1.f;  // alpha: what O (relative to m_prev) is multiplied by
        if (mx > m_prev + TC_LAZY || (m_prev == -INFINITY && mx > -INFINITY)) {
          alpha = m_prev == -INFINITY ? 0.f : ex2(m_prev - mx);
          m_new = mx;
        }
        if (qt == 0) mrun4[gq * 32 + rr] = m_new;
        mbar_arrive(b_mpub4 + 8 * gq);
        if (m_new != m_seen) {  // this thread's row sum is relative to the max it saw four tiles ago
          l = m_seen == -INFINITY ? 0.f : l * ex2(m_seen - m_new);
          m_seen = m_new;
        }
        const float sh = TC_SHIFT - (m_new == -INFINITY ? 0.f : m_new);
        // The residual term: always on a group's first tile of a segment, later by the vote of the group's threads
        // at its tile before (three flags per group in turn: read here, voted on below, cleared for the turn after).
        const bool with_lo = t < 4 || lo4[gq * 3 + gn % 3] != 0u;
        if ((tid & 127) == 0) lo4[gq * 3 + (gn + 2) % 3] = 0u;
        uint32_t e_hi[8], e_lo[8];
        l += with_lo ? exp_regs32<true>(v, sl2, sh, e_hi, e_lo) : exp_regs32<false>(v, sl2, sh, e_hi, e_lo);
        if (valid && l < TC_LO_BELOW) atomicOr(lo4 + gq * 3 + (gn + 1) % 3, 1u);
        ++gn;
        // The group's P tile is free once the PV MMAs of its own tile before are done: long ago, as a rule.
        if (gi >= 4) wait_or_flag(b_pfree + 8 * gq, ((gi - 4) >> 2) & 1, failed, p.status, GA_ST_WAIT_EMPTY);
        {
          const uint32_t p_hi = sP + (gq * 2) * TC_P4_BYTES + rr * 128, p_lo = p_hi + TC_P4_BYTES;
          const uint32_t chunk0 = static_cast<uint32_t>(col_first >> 4), rx = static_cast<uint32_t>(rr & 7);
#pragma unroll
          for (int c16 = 0; c16 < 2; ++c16) {
            const uint32_t chunk = ((chunk0 + c16) ^ rx) << 4;
            asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(p_hi + chunk), "r"(e_hi[c16 * 4]), "r"(e_hi[c16 * 4 + 1]),
                         "r"(e_hi[c16 * 4 + 2]), "r"(e_hi[c16 * 4 + 3])
                         : "memory");
            if (with_lo)
              asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(p_lo + chunk), "r"(e_lo[c16 * 4]), "r"(e_lo[c16 * 4 + 1]),
                           "r"(e_lo[c16 * 4 + 2]), "r"(e_lo[c16 * 4 + 3])
                           : "memory");
          }
          if ((tid & 127) == 0) *reinterpret_cast<volatile uint32_t*>(lo_term + gq) = with_lo ? 1u : 0u;
        }
        TC_TRACE(8 + (with_lo ? 100 : 0) + (need_mask ? 50 : 0), gi);
        // O in tensor memory is rescaled only when some row moved its max; needs the PV MMAs of the tile before
        if (t >= 1 && owns_o && __any_sync(0xffffffffu, alpha != 1.f)) {
          wait_or_flag(b_pfree + 8 * ((gi - 1) & 3), ((gi - 1) >> 2) & 1, failed, p.status, GA_ST_WAIT_EMPTY);
          tc_fence_after();
#pragma unroll 1
          for (int c0 = 0; c0 < HD; c0 += 32) {
            uint32_t w[32];
            tmem_ld32(lane_base + C::O_COL + c0, w);
            tmem_wait_ld();
#pragma unroll
            for (int j = 0; j < 32; ++j) w[j] = __float_as_uint(__uint_as_float(w[j]) * alpha);
            tmem_st32(lane_base + C::O_COL + c0, w);
          }
          tmem_wait_st();
        }
        // rows past the end of the sequence in the last tile: V must be finite where P is exactly 0
        if (n0 + TNK > s.L) {
          const int st = gi % C::NV;
          wait_or_flag(b_vfull + 8 * st, (gi / C::NV) & 1, failed, p.status, GA_ST_WAIT_FULL);
          if (n0 + krow >= s.L) {
#pragma unroll 1
            for (int c = 0; c < C::ATOMS * 8; ++c) {
              const uint32_t a = sV + st * C::KV_BYTES + (c >> 3) * SLAB + krow * 128 + ((c & 7) << 4);
              asm volatile("st.shared.v4.b32 [%0], {%1,%1,%1,%1};" ::"r"(a), "r"(0) : "memory");
            }
          }
        }
        fence_proxy_async();
        tc_fence_before();
        mbar_arrive(b_pready4 + 8 * gq);
        TC_TRACE(9, gi);
      }
      it = it0 + n_tiles;
      TC_TRACE(10, it);
      {  // the next segment's Q tile, as soon as this thread is through its tiles
        Seg nxt;
        if (read_seg(sk, nxt, false) && nxt.t_hi > nxt.t_lo) {
          wait_or_flag(b_qfree, sq & 1, failed, p.status, GA_ST_WAIT_EMPTY);
          load_q(nxt);
          q_ready = true;
        }
      }
      // ---- end of the segment: row sums over the 16 shares of a row (4 groups x 4 quarters), then O / l
      named_bar_sync(1, TC_SOFTMAX);  // all tiles of all groups are through their max exchange
      TC_TRACE(12, it);
      const int gi_last = it - 1;
      const float m_fin = mrun4[(gi_last & 3) * 32 + rr];
      if (m_seen != m_fin) l = m_seen == -INFINITY ? 0.f : l * ex2(m_seen - m_fin);
      named_bar_sync(1, TC_SOFTMAX);  // the row sums overlay the max buffers
      lbuf[(gq * 4 + qt) * 32 + rr] = l;
      named_bar_sync(1, TC_SOFTMAX);
      l = 0.f;
#pragma unroll
      for (int k4 = 0; k4 < 4; ++k4)
        l += (lbuf[(k4 * 4) * 32 + rr] + lbuf[(k4 * 4 + 1) * 32 + rr]) + (lbuf[(k4 * 4 + 2) * 32 + rr] + lbuf[(k4 * 4 + 3) * 32 + rr]);
      named_bar_sync(1, TC_SOFTMAX);  // the sums are read: the next segment may write the max buffers again
      TC_TRACE(11, it);
      wait_or_flag(b_pfree + 8 * (gi_last & 3), (gi_last >> 2) & 1, failed, p.status, GA_ST_WAIT_EMPTY);
      TC_TRACE(13, it);
      tc_fence_after();
      const bool bad = __any_sync(0xffffffffu, failed);
      const bool partial = s.slot >= 0;
      const int tq = rr / p.gqa, hq = rr - tq * p.gqa;
      const float vds = p.vd ? p.vd[s.b * p.vd_s0 + s.h * p.vd_s1] : 1.f;
      const float inv = l > 0.f ? (partial ? 1.f : vds) / l : 0.f;
      if (owns_o) {
#pragma unroll 1
        for (int c0 = 0; c0 < HD / 4; c0 += 32) {
          uint32_t w[32];
          if (!bad) {
            tmem_ld32(lane_base + C::O_COL + gq * (HD / 4) + c0, w);
            tmem_wait_ld();
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) w[j] = 0u;
          }
          if (valid && partial) {
            float* wdst = p.ws_o + (static_cast<long long>(s.slot) * p.rows_cap + rr) * HD + gq * (HD / 4) + c0;
#pragma unroll
            for (int q4 = 0; q4 < 8; ++q4)
              *reinterpret_cast<float4*>(wdst + q4 * 4) =
                  make_float4(__uint_as_float(w[q4 * 4]) * inv, __uint_as_float(w[q4 * 4 + 1]) * inv,
                              __uint_as_float(w[q4 * 4 + 2]) * inv, __uint_as_float(w[q4 * 4 + 3]) * inv);
          } else if (valid) {
            __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(p.out) + static_cast<long long>(s.q0 + tq) * p.o_s0 +
                                 static_cast<long long>(s.h * p.gqa + hq) * p.o_s1 + gq * (HD / 4) + c0;
#pragma unroll
            for (int q8 = 0; q8 < 4; ++q8) {
              uint32_t o4[4];
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                __nv_bfloat162 b2 = __floats2bfloat162_rn(__uint_as_float(w[q8 * 8 + 2 * j]) * inv,
                                                          __uint_as_float(w[q8 * 8 + 2 * j + 1]) * inv);
                o4[j] = *reinterpret_cast<uint32_t*>(&b2);
              }
              *reinterpret_cast<uint4*>(dst + q8 * 8) = make_uint4(o4[0], o4[1], o4[2], o4[3]);
            }
          }
        }
      }
      // O has been read: the PV lane may start the next segment's accumulation
      tc_fence_before();
      mbar_arrive(b_ofree);
      TC_TRACE(14, it);
      if (valid && owns_o && gq == 0) {
        const float lse2 = l > 0.f ? m_fin + lg2(l) - TC_SHIFT : -INFINITY;
        if (partial) p.ws_lse[static_cast<long long>(s.slot) * p.rows_cap + rr] = lse2;
        else if (p.lse != nullptr)
          p.lse[static_cast<long long>(s.h * p.gqa + hq) * p.total_q + s.q0 + tq] = lse2 * 0.6931471805599453f;
      }
      ++sq;
    }
  } else if (warp < 16) {
    // ---------------------------------------------------------------- softmax: two groups of 256 threads
    // Group g takes the tiles of parity g of the CTA's running tile count (its own S and P buffers), two threads per
    // query row: thread (r, hf) owns row r = tensor-memory lane, key columns [64 hf, 64 hf + 64) of the tile and the
    // matching part of the output dims. While one group is in its exp2 pass (the SM's 16 exp2 per clock are the
    // floor of a tile), the other waits for scores, reads them and finds its row maxima. The running max is one
    // chain over the tiles of a segment: a group takes the value the other group published for the tile before,
    // decides, and publishes its own.
    //
    // Few rows (speculative verify: query tokens x GQA <= 32): the rows are replicated into all four 32-lane
    // quarters of the Q tile, so S comes out four times and each quarter's warps take a quarter of the key
    // columns of the same rows (16 per thread instead of 64). A warp can only read its own quarter of tensor
    // memory, and a quarter maps to one scheduler: without this the whole softmax of such a call would sit on
    // one scheduler's exp2 unit. P rows 32..127 are zeroed once; O rows 0..31 are the result.
    const int g = tid >> 8, hf = (tid >> 7) & 1, r = tid & 127;
    const int part = g * 2 + hf;  // quarter of the head dims this thread loads of Q and stores of O
    constexpr bool rep = false;          // the verify instance has its own role above
    const int qt = warp & 3;             // lane quarter of this warp
    const int rr = rep ? (r & 31) : r;   // the query row this thread works for
    const bool owns_o = !rep || qt == 0; // this warp's lanes of O are result rows
    const int col_first = rep ? 32 * qt + 16 * hf : hf * CW;  // first key column of this thread's share of a tile
    const uint32_t lane_base = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16);
    const uint32_t grp_bar = 2 + g;      // named barrier of this group
    if (rep) {  // P rows 32..127 are never written in this mode and must read as zero
      for (int i = tid; i < 4 * C::P_BYTES / 16; i += TC_SOFTMAX)
        asm volatile("st.shared.v4.b32 [%0], {%1,%1,%1,%1};" ::"r"(sP + i * 16), "r"(0) : "memory");
      fence_proxy_async();
      named_bar_sync(1, TC_SOFTMAX);  // every zero is in place before any thread writes a P row
    }
    bool q_ready = false;  // the Q tile of `cur` was already loaded during the segment before
    while (read_seg(sk++, cur, true)) {
      const Seg& s = cur;
      const int n_tiles = s.t_hi - s.t_lo;
      TC_TRACE(1, n_tiles);
      // What only the end of the segment needs (output offsets, the value scale) is worked out there, so that it
      // does not sit in registers through the tile loop.
      const bool valid = rr / p.gqa < s.nq;
      const bool warp_live = rep || qt * 32 < s.nq * p.gqa;  // some row of this warp is a real query row
      if (n_tiles <= 0) {
        // nothing visible (an empty cache or a window past the end): zero rows, -inf LSE; no barrier is touched
        if (valid && owns_o) {
          const int tq = rr / p.gqa, hq = rr - tq * p.gqa;
          __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(p.out) + static_cast<long long>(s.q0 + tq) * p.o_s0 +
                               static_cast<long long>(s.h * p.gqa + hq) * p.o_s1 + part * (HD / 4);
          for (int c0 = 0; c0 < HD / 4; c0 += 8) *reinterpret_cast<uint4*>(dst + c0) = make_uint4(0, 0, 0, 0);
          if (part == 0 && p.lse != nullptr)
            p.lse[static_cast<long long>(s.h * p.gqa + hq) * p.total_q + s.q0 + tq] = -INFINITY;
        }
        continue;
      }
      if (!q_ready) {
        if (sq > 0) wait_or_flag(b_qfree, (sq - 1) & 1, failed, p.status, GA_ST_WAIT_EMPTY);
        load_q(s);
      }
      TC_TRACE(2, it);
      q_ready = false;
      const int pos = valid ? s.pos0 + rr / p.gqa : -1;
      const int lo_key = p.window_left >= 0 ? pos - p.window_left : -(1 << 30);
      const float sl2 = p.scale_log2 * (p.kd ? p.kd[s.b * p.kd_s0 + s.h * p.kd_s1] : 1.f);
      float m_seen = -INFINITY, l = 0.f;     // l is relative to m_seen
      const int it0 = it;
      for (int t = (g - it0) & 1; t < n_tiles; t += 2) {
        const int gi = it0 + t;              // running tile index: buffers and barrier phases
        const int u = gi >> 1;               // this group's iteration
        const int n0 = (s.t_lo + t) * TNK;
        const int c_base = n0 + col_first;
        const bool need_mask = (n0 + TNK > s.pos0 + 1) || (p.window_left >= 0 && n0 < s.pos0 + s.nq - 1 - p.window_left);
        const int sb = gi % C::NS;           // score buffer of this tile
        TC_TRACE(3, gi);
        wait_or_flag(b_sfull + 8 * sb, (gi / C::NS) & 1, failed, p.status, GA_ST_WAIT_FULL);
        TC_TRACE(4, gi);
        tc_fence_after();
        const uint32_t s_addr = lane_base + C::S_COL + sb * 128 + col_first;
        // pass 1: row max of the masked, scaled scores, 32 columns at a time (the scores stay in tensor memory)
        float mx = -INFINITY;
        if (warp_live) {
          float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
          if (rep) {
            uint32_t v[16];
            tmem_ld16(s_addr, v);
            tmem_wait_ld();
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int col = c_base + j;
              const float x = (!need_mask || (col <= pos && col >= lo_key)) ? __uint_as_float(v[j]) : -INFINITY;
              m4[j & 3] = fmaxf(m4[j & 3], x);
            }
          }
#pragma unroll 1
          for (int c0 = 0; c0 < (rep ? 0 : CW); c0 += 32) {
            // A 32-column chunk is classed for the whole warp: nothing visible (skipped), everything visible (the
            // bare loop) or mixed (compares per element). On a diagonal or window-edge tile most chunks of a warp's
            // 32 rows fall in the first two classes.
            const int cls = need_mask ? chunk_class(c_base + c0, pos, lo_key) : 0;
            if (cls == 4) continue;
            uint32_t v[32];
            tmem_ld32(s_addr + c0, v);
            tmem_wait_ld();
            if (cls != 0) {
              // The masked scores go back into tensor memory, so the exp2 pass below reads every chunk the same
              // way and needs no masked variant of its own.
              if (cls == 1) mask_chunk32<true, false>(v, c_base + c0, pos, lo_key, m4);
              else if (cls == 2) mask_chunk32<false, true>(v, c_base + c0, pos, lo_key, m4);
              else mask_chunk32<true, true>(v, c_base + c0, pos, lo_key, m4);
              tmem_st32(s_addr + c0, v);
              tmem_wait_st();
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) m4[j & 3] = fmaxf(m4[j & 3], __uint_as_float(v[j]));
            }
          }
          mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3])) * sl2;  // sl2 > 0; -inf stays -inf
        }
        // both parts publish their maximum rounded UP to bf16 and take the larger (a slightly high running max
        // only makes P a little smaller)
        TC_TRACE(5, gi);
        mxbuf[(g * 2 + hf) * 128 + r] = __float2bfloat16_ru(mx);
        // What does not depend on the partner's maximum is fetched before the exchange barrier, so that these
        // round trips overlap the wait for the slowest warp of the group: the running max after the tile before
        // from the other group, and the P buffer of this group (free once the PV MMAs of this group's previous
        // tile are done; the residual flag of this tile is complete by then, every vote having preceded its
        // thread's arrival for that tile). The waits follow the running tile count, also across a segment
        // boundary, so every barrier is waited on once per phase.
        float m_prev = -INFINITY;
        if (gi >= 1) {
          wait_or_flag(b_mpub + 8 * (g ^ 1), ((gi - 1) >> 1) & 1, failed, p.status, GA_ST_WAIT_FULL);
          if (t >= 1) m_prev = mrun[(g ^ 1) * 128 + r];
        }
        if (gi >= 2) wait_or_flag(b_pfree + 8 * g, (u - 1) & 1, failed, p.status, GA_ST_WAIT_EMPTY);
        const bool with_lo = t < 2 || lo_flag[g * 2 + (u & 1)] != 0u;
        TC_TRACE(6, gi);
        named_bar_sync(grp_bar, TC_GROUP);
        TC_TRACE(7, gi);
        if (rep) {  // eight shares of a row: two parts in each of the four quarters
          mx = -INFINITY;
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4)
            mx = fmaxf(mx, fmaxf(__bfloat162float(mxbuf[(g * 2) * 128 + rr + 32 * q4]),
                                 __bfloat162float(mxbuf[(g * 2 + 1) * 128 + rr + 32 * q4])));
        } else {
          mx = fmaxf(__bfloat162float(mxbuf[(g * 2) * 128 + r]), __bfloat162float(mxbuf[(g * 2 + 1) * 128 + r]));
        }
        float m_new = m_prev, alpha = 1.f;  // alpha: what O (relative to m_prev) is multiplied by
        if (mx > m_prev + TC_LAZY || (m_prev == -INFINITY && mx > -INFINITY)) {
          alpha = m_prev == -INFINITY ? 0.f : ex2(m_prev - mx);
          m_new = mx;
        }
        if (hf == 0) mrun[g * 128 + r] = m_new;
        mbar_arrive(b_mpub + 8 * g);
        if (m_new != m_seen) {  // this group's row sum is relative to the max it saw two tiles ago
          l = m_seen == -INFINITY ? 0.f : l * ex2(m_seen - m_new);
          m_seen = m_new;
        }
        const float sh = TC_SHIFT - (m_new == -INFINITY ? 0.f : m_new);
        // pass 2: P = 2^(s - m + 7), e4m3 (plus the residual term while needed), into the swizzled A tiles
        if (warp_live) {
          const uint32_t p_hi = sP + (g * 2) * C::P_BYTES + rr * 128, p_lo = p_hi + C::P_BYTES;
          float lsum = 0.f;
          if (rep) {
            uint32_t v[16];
            tmem_ld16(s_addr, v);
            tmem_wait_ld();
            const uint32_t chunk0 = static_cast<uint32_t>(col_first >> 4), rx = static_cast<uint32_t>(rr & 7);
            if (with_lo) {
              lsum += need_mask ? exp_chunk32<true, true, 16>(v, sl2, sh, c_base, pos, lo_key, p_hi, p_lo, chunk0, rx)
                                : exp_chunk32<false, true, 16>(v, sl2, sh, c_base, pos, lo_key, p_hi, p_lo, chunk0, rx);
            } else {
              lsum += need_mask ? exp_chunk32<true, false, 16>(v, sl2, sh, c_base, pos, lo_key, p_hi, p_lo, chunk0, rx)
                                : exp_chunk32<false, false, 16>(v, sl2, sh, c_base, pos, lo_key, p_hi, p_lo, chunk0, rx);
            }
          }
#pragma unroll 1
          for (int c0 = 0; c0 < (rep ? 0 : CW); c0 += 32) {
            const uint32_t chunk0 = static_cast<uint32_t>(hf * (CW / 16) + (c0 >> 4)), rx = static_cast<uint32_t>(r & 7);
            if (need_mask && chunk_class(c_base + c0, pos, lo_key) == 4) {  // nothing visible: P is exactly zero here
#pragma unroll
              for (int c16 = 0; c16 < 2; ++c16) {
                const uint32_t chunk = ((chunk0 + c16) ^ rx) << 4;
                asm volatile("st.shared.v4.b32 [%0], {%1,%1,%1,%1};" ::"r"(p_hi + chunk), "r"(0) : "memory");
                if (with_lo) asm volatile("st.shared.v4.b32 [%0], {%1,%1,%1,%1};" ::"r"(p_lo + chunk), "r"(0) : "memory");
              }
              continue;
            }
            uint32_t v[32];
            tmem_ld32(s_addr + c0, v);  // hidden keys of a mixed chunk were set to -inf by the max pass
            tmem_wait_ld();
            lsum += with_lo ? exp_chunk32<false, true>(v, sl2, sh, c_base + c0, pos, lo_key, p_hi, p_lo, chunk0, rx)
                            : exp_chunk32<false, false>(v, sl2, sh, c_base + c0, pos, lo_key, p_hi, p_lo, chunk0, rx);
          }
          l += lsum;
        }
        // S has been read for the last time: the buffer may take the scores of a later tile
        TC_TRACE(8 + (with_lo ? 100 : 0) + (need_mask ? 50 : 0), gi);
        tc_fence_before();
        mbar_arrive(b_sfree + 8 * sb);
        // The residual term of P is only needed while a row rests on few keys: once this thread's share of the row
        // sum stands for at least 32 keys at the running max, the e4m3 rounding of P averages out far below the
        // tolerance. The vote is for this group's next tile (read there after the wait for this tile's PV MMAs,
        // which follow every thread's arrival below).
        if (valid && l < TC_LO_BELOW) atomicOr(lo_flag + g * 2 + ((u + 1) & 1), 1u);
        // O in tensor memory is rescaled only when some row of this warp moved its max; needs PV of tile t-1 done.
        if (t >= 1 && owns_o && __any_sync(0xffffffffu, alpha != 1.f)) {
          wait_or_flag(b_pfree + 8 * (g ^ 1), ((gi - 1) >> 1) & 1, failed, p.status, GA_ST_WAIT_EMPTY);
          tc_fence_after();
#pragma unroll 1
          for (int c0 = 0; c0 < HD / 2; c0 += 32) {
            uint32_t v[32];
            tmem_ld32(lane_base + C::O_COL + hf * (HD / 2) + c0, v);
            tmem_wait_ld();
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) * alpha);
            tmem_st32(lane_base + C::O_COL + hf * (HD / 2) + c0, v);
          }
          tmem_wait_st();
        }
        // rows past the end of the sequence in the last tile: V must be finite where P is exactly 0
        if (n0 + TNK > s.L) {
          const int st = gi % C::NV;
          wait_or_flag(b_vfull + 8 * st, (gi / C::NV) & 1, failed, p.status, GA_ST_WAIT_FULL);
          if (n0 + r >= s.L) {
#pragma unroll 1
            for (int c = hf * (C::ATOMS * 4); c < (hf + 1) * (C::ATOMS * 4); ++c) {
              const uint32_t a = sV + st * C::KV_BYTES + (c >> 3) * SLAB + r * 128 + ((c & 7) << 4);
              asm volatile("st.shared.v4.b32 [%0], {%1,%1,%1,%1};" ::"r"(a), "r"(0) : "memory");
            }
          }
        }
        fence_proxy_async();
        tc_fence_before();
        mbar_arrive(b_pready + 8 * g);
        TC_TRACE(9, gi);
      }
      it = it0 + n_tiles;
      TC_TRACE(10, it);
      // ---- the next segment's Q goes in as soon as this thread is through its tiles: the group that finishes
      // first does its share under the other group's last tile, and the QK lane starts the next segment's scores
      // under this segment's output pass. The QK MMAs of this segment were issued tiles ago, so the wait for them is
      // normally over.
      {
        Seg nxt;
        if (read_seg(sk, nxt, false) && nxt.t_hi > nxt.t_lo) {
          wait_or_flag(b_qfree, sq & 1, failed, p.status, GA_ST_WAIT_EMPTY);
          load_q(nxt);
          q_ready = true;
        }
      }
      TC_TRACE(12, it);
      // ---- end of the segment, part 1: the row sums
      named_bar_sync(1, TC_SOFTMAX);  // all tiles of both groups are through their max exchange
      const int gi_last = it - 1, g_last = gi_last & 1;
      const float m_fin = mrun[g_last * 128 + r];
      if (m_seen != m_fin) l = m_seen == -INFINITY ? 0.f : l * ex2(m_seen - m_fin);
      named_bar_sync(1, TC_SOFTMAX);  // the row sums overlay the max buffers
      lbuf[part * 128 + r] = l;
      named_bar_sync(1, TC_SOFTMAX);
      if (rep) {  // a row's sum is spread over the four parts in each of the four quarters
        l = 0.f;
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4)
          l += (lbuf[rr + 32 * q4] + lbuf[128 + rr + 32 * q4]) + (lbuf[256 + rr + 32 * q4] + lbuf[384 + rr + 32 * q4]);
      } else {
        l = (lbuf[r] + lbuf[128 + r]) + (lbuf[256 + r] + lbuf[384 + r]);
      }
      named_bar_sync(1, TC_SOFTMAX);  // the sums are read: the next segment may write the max buffers again
      TC_TRACE(11, it);
      // ---- part 2: O / l, each thread one quarter of the output dims of its row
      wait_or_flag(b_pfree + 8 * g_last, (gi_last >> 1) & 1, failed, p.status, GA_ST_WAIT_EMPTY);
      TC_TRACE(13, it);
      tc_fence_after();
      const bool bad = __any_sync(0xffffffffu, failed);  // tensor-memory loads are warp-collective
      const bool partial = s.slot >= 0;  // a piece of a unit that other CTAs share: fp32 into the workspace slot
      const int tq = rr / p.gqa, hq = rr - tq * p.gqa;
      const long long ooff = static_cast<long long>(s.q0 + tq) * p.o_s0 + static_cast<long long>(s.h * p.gqa + hq) * p.o_s1 +
                             part * (HD / 4);
      const float vds = p.vd ? p.vd[s.b * p.vd_s0 + s.h * p.vd_s1] : 1.f;
      const float inv = l > 0.f ? (partial ? 1.f : vds) / l : 0.f;
      if (!rep && !partial) {
        // bf16 rows go through a warp-private patch of shared memory (this group's P buffers: every MMA that read
        // them has completed, and no warp of the group writes P again before all of them are past this point) so
        // that the global stores are whole 64- or 128-byte runs of a row instead of 16 bytes from each of 32 rows.
        constexpr int CH = HD / 32;   // 16-byte chunks of this thread's quarter row
        constexpr int ROWB = CH * 16;
        const uint32_t stage = sP + (g * 2) * C::P_BYTES + (warp & 7) * (32 * ROWB);
#pragma unroll 1
        for (int c0 = 0; c0 < HD / 4; c0 += 32) {
          uint32_t v[32];
          if (!bad) {
            tmem_ld32(lane_base + C::O_COL + part * (HD / 4) + c0, v);
            tmem_wait_ld();
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = 0u;
          }
#pragma unroll
          for (int q8 = 0; q8 < 4; ++q8) {
            uint32_t w[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              __nv_bfloat162 b2 = __floats2bfloat162_rn(__uint_as_float(v[q8 * 8 + 2 * j]) * inv,
                                                        __uint_as_float(v[q8 * 8 + 2 * j + 1]) * inv);
              w[j] = *reinterpret_cast<uint32_t*>(&b2);
            }
            const uint32_t dst = stage + lane * ROWB + ((((c0 >> 3) + q8) ^ (lane & (CH - 1))) << 4);
            asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(dst), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3])
                         : "memory");
          }
        }
        // O has been read: the PV lane may start the next segment's accumulation
        tc_fence_before();
        mbar_arrive(b_ofree);
        TC_TRACE(14, it);
        __syncwarp();
        const long long row_off = valid ? ooff : -1;
#pragma unroll
        for (int i = 0; i < CH; ++i) {
          const int row = i * (32 / CH) + lane / CH, j = lane % CH;
          uint4 w;
          asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];"
                       : "=r"(w.x), "=r"(w.y), "=r"(w.z), "=r"(w.w)
                       : "r"(stage + row * ROWB + ((j ^ (row & (CH - 1))) << 4)));
          const long long o = __shfl_sync(0xffffffffu, row_off, row);
          if (o >= 0) *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(p.out) + o + j * 8) = w;
        }
        __syncwarp();
        TC_TRACE(15, it);
      } else {
        float* wdst = partial ? p.ws_o + (static_cast<long long>(s.slot) * p.rows_cap + rr) * HD + part * (HD / 4) : nullptr;
#pragma unroll 1
        for (int c0 = 0; c0 < (owns_o ? HD / 4 : 0); c0 += 32) {
          uint32_t v[32];
          if (!bad) {
            tmem_ld32(lane_base + C::O_COL + part * (HD / 4) + c0, v);
            tmem_wait_ld();
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = 0u;
          }
          if (valid && partial) {
#pragma unroll
            for (int q4 = 0; q4 < 8; ++q4)
              *reinterpret_cast<float4*>(wdst + c0 + q4 * 4) =
                  make_float4(__uint_as_float(v[q4 * 4]) * inv, __uint_as_float(v[q4 * 4 + 1]) * inv,
                              __uint_as_float(v[q4 * 4 + 2]) * inv, __uint_as_float(v[q4 * 4 + 3]) * inv);
          } else if (valid) {
            __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(p.out) + ooff + c0;
#pragma unroll
            for (int q8 = 0; q8 < 4; ++q8) {
              uint32_t w[4];
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                __nv_bfloat162 b2 = __floats2bfloat162_rn(__uint_as_float(v[q8 * 8 + 2 * j]) * inv,
                                                          __uint_as_float(v[q8 * 8 + 2 * j + 1]) * inv);
                w[j] = *reinterpret_cast<uint32_t*>(&b2);
              }
              *reinterpret_cast<uint4*>(dst + q8 * 8) = make_uint4(w[0], w[1], w[2], w[3]);
            }
          }
        }
        // O has been read: the PV lane may start the next segment's accumulation
        tc_fence_before();
        mbar_arrive(b_ofree);
        TC_TRACE(14, it);
      }
      if (valid && owns_o && part == 0) {
        const float lse2 = l > 0.f ? m_fin + lg2(l) - TC_SHIFT : -INFINITY;
        if (partial) p.ws_lse[static_cast<long long>(s.slot) * p.rows_cap + rr] = lse2;
        else if (p.lse != nullptr)
          p.lse[static_cast<long long>(s.h * p.gqa + hq) * p.total_q + s.q0 + tq] = lse2 * 0.6931471805599453f;
      }
      ++sq;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(C::TMEM_COLS) : "memory");
  }
}

// Issue-rate probe: every SM issues `iters` e4m3 MMAs (M 128, N 256, K 32) on zeroed operands and waits for
// them once. Gives the dense FP8 tensor peak of the device the extend kernel is measured against.
__global__ void __launch_bounds__(128) fp8_peak_kernel(int iters, int* status) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  __shared__ uint64_t bar;
  __shared__ uint32_t slot;
  const uint32_t base = smem_u32(smem_raw);
  const int tid = threadIdx.x, warp = tid >> 5;
  for (int i = tid; i < 49152 / 4; i += 128) reinterpret_cast<uint32_t*>(smem_raw)[i] = 0u;
  if (tid == 0) {
    mbar_init(smem_u32(&bar), 1);
    mbar_fence_init();
  }
  fence_proxy_async();
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&slot)), "r"(512)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = slot;
  if (tid == 0 && (base & 1023u) == 0) {
    const uint32_t idesc = instr_desc(128, 256, 0);
    for (int it = 0; it < iters; ++it) {
      const int ks = it & 3;
      mma_f8(tmem + (it & 1) * 256, smem_desc(base + ks * 32, 16, 1024), smem_desc(base + 16384 + ks * 32, 16, 1024),
             idesc, 1);
    }
    mma_commit(smem_u32(&bar));
  } else if (tid == 0) {
    mbar_arrive(smem_u32(&bar));
    atomicExch(status, GA_ST_BAD_PAGE);
  }
  if (!mbar_wait(smem_u32(&bar), 0) && tid == 0) atomicExch(status, GA_ST_WAIT_TMEM);
  tc_fence_before();
  __syncthreads();
  if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
}

}  // namespace tc
}  // namespace attn
}  // namespace ga

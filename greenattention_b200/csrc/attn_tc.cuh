// FP8 paged attention for large query blocks (extend / chunked prefill) on the 5th-generation tensor
// cores: tcgen05.mma (kind::f8f6f4, e4m3 x e4m3 -> f32) with accumulators in tensor memory.
//
// Replaces the reference's SM90 WGMMA extend kernel (csrc/sm90/attn_decode_fp8/extend_kernel.cuh:162-457;
// work decomposition extend_kernel.cuh:140-160) for head_dim 128 and 256, any GQA, causal with an optional
// left window. Same math as the reference kernels: bf16 Q rounded to e4m3, S = scale * k_descale * Q K^T,
// bottom-right causal mask and left window, online softmax in the log2 domain, P rounded to e4m3, O = v_descale
// * P V / l, natural-log LSE (kernel.cuh:468-474,489-496,621-653).
//
// One CTA = 128 query rows (128 / GQA tokens x the GQA heads of one kv head) against the keys they can see,
// 128 keys per iteration:
//   * four producer warps (K / V x even / odd tiles) gather pages with TMA (128-byte swizzle, one box per page
//     and 128-byte head slice, never multicast) into a K ring and a V ring;
//   * one lane of the last warp issues the MMAs: S = Q K^T with both operands K-major straight from the swizzled
//     tiles, and O += P V with P as a K-major A operand from shared memory and V as an MN-major B operand, i.e.
//     the [token, dim] page layout as it is: no transpose of V anywhere. S (2 x 128 columns, double
//     buffered) and O (head_dim columns) live in tensor memory;
//   * warps 0-7 (softmax): two threads per query row (= tensor-memory lane), one per half of the 128 keys. Each reads its S half-row with
//     tcgen05.ld, does mask / max / exp2 without any cross-thread traffic, writes P as two e4m3 terms
//     (4 significant bits + residual, so a probability carries ~2^-8 relative error) into swizzled shared
//     memory, and rescales O in tensor memory only when its running max moved by more than 1.5 in log2 (the
//     stale max keeps P below the e4m3 limit: 2^(7 + 1.5) < 448).
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

template <int HD>
struct TcCfg {
  static constexpr int ATOMS = HD / 128;
  static constexpr int Q_BYTES = ATOMS * SLAB;
  static constexpr int P_BYTES = SLAB;                // one e4m3 term of P: 128 rows x 128 keys
  static constexpr int KV_BYTES = ATOMS * SLAB;       // one K (or V) tile
  static constexpr int NKV = HD == 128 ? 4 : 2;       // ring depth of each of the K and V rings (even: see producers)
  // Header (barriers, row-max / row-sum exchange) first, then the 1024-byte aligned operand tiles. At head_dim
  // 256 this fills the 227 KiB of an SM exactly, so the kernel relies on the 1024-byte alignment it declares for
  // its dynamic shared memory and checks it at run time.
  static constexpr int BAR_OFF = 0;
  static constexpr int X_OFF = 256;                   // part maxima [2][2][128] bf16, running max [2][128] f32; row sums overlay both
  static constexpr int Q_OFF = 3072;
  static constexpr int P_OFF = Q_OFF + Q_BYTES;       // [buffer 0|1][hi|lo]
  static constexpr int K_OFF = P_OFF + 4 * P_BYTES;
  static constexpr int V_OFF = K_OFF + NKV * KV_BYTES;
  static constexpr int SMEM_BYTES = V_OFF + NKV * KV_BYTES;
  static constexpr int TMEM_COLS = 512;
  // Tensor memory: NS score buffers of 128 columns, then O (head_dim columns). Head dim 128 leaves room for a
  // third score buffer, so the QK MMAs of tile t + 2 need not wait for the softmax of tile t.
  static constexpr int NS = HD == 128 ? 3 : 2;
  static constexpr int S_COL = 0;
  static constexpr int O_COL = NS * 128;
  static_assert(SMEM_BYTES <= SMEM_OPTIN, "shared memory");
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

// Threads: 16 softmax warps (two groups of 8), 4 producer warps, 2 MMA-issuing warps.
constexpr int TC_SOFTMAX = 512;
constexpr int TC_GROUP = 256;
constexpr int TC_THREADS = TC_SOFTMAX + 192;

// REP: instance for calls with at most 32 rows per kv head (see the softmax section); extend uses REP = false so
// that its inner loops carry none of that mode's branches.
template <int HD, bool REP>
__global__ void __launch_bounds__(TC_THREADS, 1)
attn_tc_kernel(const __grid_constant__ AttnDev p, const __grid_constant__ CUtensorMap kmap,
               const __grid_constant__ CUtensorMap vmap) {
  using C = TcCfg<HD>;
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
  const uint32_t b_kfull = bars + 104, b_kempty = b_kfull + 8 * C::NKV, b_vfull = b_kempty + 8 * C::NKV,
                 b_vempty = b_vfull + 8 * C::NKV;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(gen + C::BAR_OFF + 104 + 32 * C::NKV);
  uint32_t* lo_flag = tmem_slot + 2;  // [group][2]: the residual term of P is wanted for the group's tile 2u + g
  __nv_bfloat16* mxbuf = reinterpret_cast<__nv_bfloat16*>(gen + C::X_OFF);  // [group][part][128], rounded up
  float* mrun = reinterpret_cast<float*>(gen + C::X_OFF + 1024);            // [group][128] running max after a tile
  float* lbuf = reinterpret_cast<float*>(gen + C::X_OFF);  // [4][128] row sums, after the last tile (overlay)

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    mbar_init(b_q, TC_SOFTMAX);
    for (int i = 0; i < 2; ++i) {
      mbar_init(b_pready + 8 * i, TC_GROUP);
      mbar_init(b_pfree + 8 * i, 1);
      mbar_init(b_mpub + 8 * i, TC_GROUP);
    }
    for (int i = 0; i < C::NS; ++i) {
      mbar_init(b_sfull + 8 * i, 1);
      mbar_init(b_sfree + 8 * i, TC_GROUP);
    }
    for (int i = 0; i < C::NKV; ++i) {
      mbar_init(b_kfull + 8 * i, 1);
      mbar_init(b_kempty + 8 * i, 1);
      mbar_init(b_vfull + 8 * i, 1);
      mbar_init(b_vempty + 8 * i, 1);
    }
    // the first tile of each group always carries the residual term; later tiles by vote
    lo_flag[0] = lo_flag[2] = 1u;
    lo_flag[1] = lo_flag[3] = 0u;
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

  Seg s;
  const bool have = extend_block(p, static_cast<int>(blockIdx.x), static_cast<int>(blockIdx.y), TNK, lane, s);
  const int n_tiles = have ? s.t_hi - s.t_lo : 0;
  bool failed = false;

  if (have && warp >= 16 && warp < 20) {
    // ---------------------------------------------------------------- producers: four warps
    // One warp's issue loop (barrier wait, expect_tx, page lookup, TMA issue) takes more than a thousand cycles
    // per tile, so K and V have their own warps, and even and odd tiles too. The ring depth is even, so a stage
    // is always refilled by the same warp (its parity waits stay within one phase).
    const int pw = warp - 16, kv = pw & 1, par = pw >> 1;
    PtWindow win;
    win.b = -1;
    win.base = win.cur = win.nxt = 0;
    if (lane == 0) tma_prefetch_desc(kv ? &vmap : &kmap);
    const int nbox = TNK / p.box_tok;
    for (int t = par; t < n_tiles; t += 2) {
      const int st = t % C::NKV, use = t / C::NKV;
      const int n0 = (s.t_lo + t) * TNK;
      int boxes = 0;
      for (int i = 0; i < nbox; ++i) boxes += (n0 + i * p.box_tok) < s.L;
      const uint32_t bytes = static_cast<uint32_t>(boxes) * p.box_tok * 128 * C::ATOMS;
      const uint32_t full = (kv ? b_vfull : b_kfull) + 8 * st, empty = (kv ? b_vempty : b_kempty) + 8 * st;
      if (use > 0) wait_or_flag(empty, (use - 1) & 1, failed, p.status, GA_ST_WAIT_EMPTY);
      if (failed) break;
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
    }
  } else if (have && warp == 20) {
    // ---------------------------------------------------------------- QK issue: one lane
    // The two issuing lanes (this one and the PV one) run on their own: the next scores are what a softmax group
    // waits for once it hands back its S buffer, so they must not queue behind the PV wait. Each lane's
    // instruction stream is the limit of the tensor pipe here, so descriptors are whole 64-bit registers
    // prepared before the waits, and a K step is one add.
    if (lane == 0) {
      const uint32_t id_qk = instr_desc(TM, TNK, 0);
      const uint64_t dq = smem_desc(sQ, 16, 1024), dk = smem_desc(sK, 16, 1024);
      wait_or_flag(b_q, 0, failed, p.status, GA_ST_WAIT_FULL);
      for (int t = 0; t < n_tiles && !failed; ++t) {
        const int st = t % C::NKV;
        const uint64_t kb = dk + static_cast<uint64_t>(st * (C::KV_BYTES >> 4));
        const int sb = t % C::NS;
        const uint32_t sd = tmem + C::S_COL + sb * 128;
        wait_or_flag(b_kfull + 8 * st, (t / C::NKV) & 1, failed, p.status, GA_ST_WAIT_FULL);
        if (t >= C::NS) wait_or_flag(b_sfree + 8 * sb, ((t / C::NS) - 1) & 1, failed, p.status, GA_ST_WAIT_EMPTY);
        if (failed) break;
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < HD / 32; ++ks) {
          const uint64_t off = static_cast<uint64_t>(((ks >> 2) * SLAB + (ks & 3) * 32) >> 4);
          mma_f8(sd, dq + off, kb + off, id_qk, ks > 0 ? 1 : 0);
        }
        mma_commit(b_kempty + 8 * st);
        mma_commit(b_sfull + 8 * sb);
      }
    }
  } else if (have && warp == 21) {
    // ---------------------------------------------------------------- PV issue: one lane
    // O += P V with V as an MN-major B operand covering all head dims in one instruction (N = head_dim: at 256
    // the second 128-dim slab is found through the leading-dimension stride of the descriptor).
    if (lane == 0) {
      const uint32_t id_pv = instr_desc(TM, HD, 1);
      const uint64_t dp = smem_desc(sP, 16, 1024), dv = smem_desc(sV, SLAB, 1024);
      for (int t = 0; t < n_tiles && !failed; ++t) {
        const int st = t % C::NKV;
        const uint64_t vb = dv + static_cast<uint64_t>(st * (C::KV_BYTES >> 4));
        const uint64_t pb = dp + static_cast<uint64_t>((t & 1) * 2 * (C::P_BYTES >> 4));
        wait_or_flag(b_pready + 8 * (t & 1), (t >> 1) & 1, failed, p.status, GA_ST_WAIT_FULL);
        wait_or_flag(b_vfull + 8 * st, (t / C::NKV) & 1, failed, p.status, GA_ST_WAIT_FULL);
        if (failed) break;
        tc_fence_after();
        const int terms = atomicExch(lo_flag + (t & 1) * 2 + ((t >> 1) & 1), 0u) ? 2 : 1;
#pragma unroll 1
        for (int term = 0; term < terms; ++term) {  // hi term, then the residual term while some row needs it
          const uint64_t pa = pb + static_cast<uint64_t>(term * (C::P_BYTES >> 4));
#pragma unroll
          for (int ks = 0; ks < TNK / 32; ++ks)
            mma_f8(tmem + C::O_COL, pa + static_cast<uint64_t>(ks * 2), vb + static_cast<uint64_t>(ks * (32 * 128 >> 4)), id_pv,
                   (t > 0 || term > 0 || ks > 0) ? 1 : 0);
        }
        mma_commit(b_vempty + 8 * st);
        mma_commit(b_pfree + 8 * (t & 1));
      }
    }
  } else if (have && warp < 16) {
    // ---------------------------------------------------------------- softmax: two groups of 256 threads
    // Group g takes the tiles of parity g (its own S and P buffers), two threads per query row: thread (r, hf) owns
    // row r = tensor-memory lane, key columns [64 hf, 64 hf + 64) of the tile and the matching part of the output
    // dims. While one group is in its exp2 pass (the SM's 16 exp2 per clock are the floor of a tile), the other
    // waits for scores, reads them and finds its row maxima. The running max is one chain over all tiles: a group
    // takes the value the other group published for the tile before, decides, and publishes its own.
    //
    // Few rows (speculative verify: query tokens x GQA <= 32): the rows are replicated into all four 32-lane
    // quarters of the Q tile, so S comes out four times and each quarter's warps take a quarter of the key
    // columns of the same rows (16 per thread instead of 64). A warp can only read its own quarter of tensor
    // memory, and a quarter maps to one scheduler: without this the whole softmax of such a call would sit on
    // one scheduler's exp2 unit. P rows 32..127 are zeroed once; O rows 0..31 are the result.
    const int g = tid >> 8, hf = (tid >> 7) & 1, r = tid & 127;
    const int part = g * 2 + hf;  // quarter of the head dims this thread loads of Q and stores of O
    const bool rep = REP && s.nq * p.gqa <= 32;
    const int qt = warp & 3;             // lane quarter of this warp
    const int rr = rep ? (r & 31) : r;   // the query row this thread works for
    const int tq = rr / p.gqa, hq = rr - tq * p.gqa;
    const bool valid = tq < s.nq;
    const bool warp_live = rep || qt * 32 < s.nq * p.gqa;  // some row of this warp is a real query row
    const bool owns_o = !rep || qt == 0;                   // this warp's lanes of O are result rows
    const int col_first = rep ? 32 * qt + 16 * hf : hf * CW;  // first key column of this thread's share of a tile
    const int pos = valid ? s.pos0 + tq : -1;
    const int lo_key = p.window_left >= 0 ? pos - p.window_left : -(1 << 30);
    {  // Q: a quarter of this row, rounded to e4m3, into the swizzled A tile
      const long long off = static_cast<long long>(s.q0 + tq) * p.q_s0 + static_cast<long long>(s.h * p.gqa + hq) * p.q_s1;
#pragma unroll 1
      for (int c = part * (HD / 64); c < (part + 1) * (HD / 64); ++c) {
        uint4 pk = make_uint4(0, 0, 0, 0);
        if (valid) {
          if (p.q_bf16) {
            const uint4* src = reinterpret_cast<const uint4*>(p.q + (off + c * 16) * 2);
            uint4 x = src[0], y = src[1];
            auto cv = [](uint32_t a, uint32_t b) {
              return pack_e4m3x4(bf16_bits_to_f32(a & 0xffffu), bf16_bits_to_f32(a >> 16), bf16_bits_to_f32(b & 0xffffu),
                                 bf16_bits_to_f32(b >> 16));
            };
            pk = make_uint4(cv(x.x, x.y), cv(x.z, x.w), cv(y.x, y.y), cv(y.z, y.w));
          } else {
            pk = *reinterpret_cast<const uint4*>(p.q + off + c * 16);
          }
        }
        const uint32_t dst = sQ + (c >> 3) * SLAB + r * 128 + (((c & 7) ^ (r & 7)) << 4);
        asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(dst), "r"(pk.x), "r"(pk.y), "r"(pk.z), "r"(pk.w)
                     : "memory");
      }
      if (rep) {  // P rows 32..127 are never written in this mode and must read as zero
        for (int i = tid; i < 4 * C::P_BYTES / 16; i += TC_SOFTMAX)
          asm volatile("st.shared.v4.b32 [%0], {%1,%1,%1,%1};" ::"r"(sP + i * 16), "r"(0) : "memory");
      }
      fence_proxy_async();
      mbar_arrive(b_q);
      if (rep) named_bar_sync(1, TC_SOFTMAX);  // every zero is in place before any thread writes a P row
    }
    const float kds = p.kd ? p.kd[s.b * p.kd_s0 + s.h * p.kd_s1] : 1.f;
    const float vds = p.vd ? p.vd[s.b * p.vd_s0 + s.h * p.vd_s1] : 1.f;
    const float sl2 = p.scale_log2 * kds;
    const uint32_t lane_base = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16);
    const uint32_t grp_bar = 2 + g;        // named barrier of this group
    float m_seen = -INFINITY, l = 0.f;     // l is relative to m_seen
    for (int t = g; t < n_tiles; t += 2) {
      const int u = t >> 1;                // this group's iteration: phases of its own barriers
      const int n0 = (s.t_lo + t) * TNK;
      const int c_base = n0 + col_first;
      const bool need_mask = (n0 + TNK > s.pos0 + 1) || (p.window_left >= 0 && n0 < s.pos0 + s.nq - 1 - p.window_left);
      const int sb = t % C::NS;            // score buffer of this tile
      wait_or_flag(b_sfull + 8 * sb, (t / C::NS) & 1, failed, p.status, GA_ST_WAIT_FULL);
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
          uint32_t v[32];
          tmem_ld32(s_addr + c0, v);
          tmem_wait_ld();
          if (need_mask) {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const int col = c_base + c0 + j;
              const float x = (col <= pos && col >= lo_key) ? __uint_as_float(v[j]) : -INFINITY;
              m4[j & 3] = fmaxf(m4[j & 3], x);
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) m4[j & 3] = fmaxf(m4[j & 3], __uint_as_float(v[j]));
          }
        }
        mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3])) * sl2;  // sl2 > 0; -inf stays -inf
      }
      // both parts publish their maximum rounded UP to bf16 and take the larger (a slightly high running max
      // only makes P a little smaller)
      mxbuf[(g * 2 + hf) * 128 + r] = __float2bfloat16_ru(mx);
      // What does not depend on the partner's maximum is fetched before the exchange barrier, so that these
      // round trips overlap the wait for the slowest warp of the group: the running max after tile t - 1 from the
      // other group, and the P buffer of this group (free once the PV MMAs of tile t - 2 are done; the residual
      // flag of this tile is complete by then, every vote having preceded its thread's arrival for that tile).
      float m_prev = -INFINITY;
      if (t >= 1) {
        wait_or_flag(b_mpub + 8 * (g ^ 1), ((t - 1) >> 1) & 1, failed, p.status, GA_ST_WAIT_FULL);
        m_prev = mrun[(g ^ 1) * 128 + r];
      }
      if (t >= 2) wait_or_flag(b_pfree + 8 * g, (u - 1) & 1, failed, p.status, GA_ST_WAIT_EMPTY);
      const bool with_lo = lo_flag[g * 2 + (u & 1)] != 0u;
      named_bar_sync(grp_bar, TC_GROUP);
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
          uint32_t v[32];
          tmem_ld32(s_addr + c0, v);
          tmem_wait_ld();
          const uint32_t chunk0 = static_cast<uint32_t>(hf * (CW / 16) + (c0 >> 4)), rx = static_cast<uint32_t>(r & 7);
          if (with_lo) {
            lsum += need_mask ? exp_chunk32<true, true>(v, sl2, sh, c_base + c0, pos, lo_key, p_hi, p_lo, chunk0, rx)
                              : exp_chunk32<false, true>(v, sl2, sh, c_base + c0, pos, lo_key, p_hi, p_lo, chunk0, rx);
          } else {
            lsum += need_mask ? exp_chunk32<true, false>(v, sl2, sh, c_base + c0, pos, lo_key, p_hi, p_lo, chunk0, rx)
                              : exp_chunk32<false, false>(v, sl2, sh, c_base + c0, pos, lo_key, p_hi, p_lo, chunk0, rx);
          }
        }
        l += lsum;
      }
      // S has been read for the last time: the buffer may take the scores of tile t + 2
      tc_fence_before();
      mbar_arrive(b_sfree + 8 * sb);
      // The residual term of P is only needed while a row rests on few keys: once this thread's share of the row
      // sum stands for at least 32 keys at the running max, the e4m3 rounding of P averages out far below the
      // tolerance. The vote is for this group's next tile (read there after the wait for this tile's PV MMAs,
      // which follow every thread's arrival below).
      if (valid && l < 32.f * 128.f) atomicOr(lo_flag + g * 2 + ((u + 1) & 1), 1u);
      // O in tensor memory is rescaled only when some row of this warp moved its max; needs PV of tile t-1 done.
      if (t >= 1 && owns_o && __any_sync(0xffffffffu, alpha != 1.f)) {
        wait_or_flag(b_pfree + 8 * (g ^ 1), ((t - 1) >> 1) & 1, failed, p.status, GA_ST_WAIT_EMPTY);
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
        const int st = t % C::NKV;
        wait_or_flag(b_vfull + 8 * st, (t / C::NKV) & 1, failed, p.status, GA_ST_WAIT_FULL);
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
    }
    // ---- epilogue: O / l, each thread one quarter of the output dims of its row
    named_bar_sync(1, TC_SOFTMAX);  // all tiles of both groups are through their max exchange
    const int g_last = (n_tiles - 1) & 1;
    const float m_fin = n_tiles > 0 ? mrun[g_last * 128 + r] : -INFINITY;
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
    if (n_tiles > 0) {
      wait_or_flag(b_pfree + 8 * g_last, ((n_tiles - 1) >> 1) & 1, failed, p.status, GA_ST_WAIT_EMPTY);
      tc_fence_after();
    }
    const bool bad = __any_sync(0xffffffffu, failed);  // tensor-memory loads are warp-collective
    const float inv = l > 0.f ? vds / l : 0.f;
    const long long ooff = static_cast<long long>(s.q0 + tq) * p.o_s0 + static_cast<long long>(s.h * p.gqa + hq) * p.o_s1 +
                           part * (HD / 4);
#pragma unroll 1
    for (int c0 = 0; c0 < (owns_o ? HD / 4 : 0); c0 += 32) {
      uint32_t v[32];
      if (n_tiles > 0 && !bad) {
        tmem_ld32(lane_base + C::O_COL + part * (HD / 4) + c0, v);
        tmem_wait_ld();
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = 0u;
      }
      if (valid) {
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
    if (valid && owns_o && part == 0 && p.lse != nullptr) {
      p.lse[static_cast<long long>(s.h * p.gqa + hq) * p.total_q + s.q0 + tq] =
          l > 0.f ? (m_fin + lg2(l) - TC_SHIFT) * 0.6931471805599453f : -INFINITY;
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

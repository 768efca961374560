// FP8 paged-KV decode for the production shape (one query token, head_dim 128, 4..8 kv heads, GQA <= 8): the
// split-KV kernel of attn_rows.cuh with a different gather. Same math and the same device split plan as there
// (reference: csrc/sm90/attn_decode_fp8/kernel.cuh:339-657, 142-153, 207-253); what changes is what one TMA box
// holds.
//
// A page is [tokens, kv_heads, 128 B], so one kv head's keys are 128-byte pieces at a kv_heads * 128 byte stride.
// Gathering one head at a time (attn_rows.cuh) asks DRAM for 128-byte pieces, and the other heads of the same page
// are fetched at other times by other CTAs: measured on B200 that stream tops out at 5.3 - 5.8 TB/s. A box that takes
// ALL kv heads of a run of tokens is one contiguous run of the page (32 tokens x 8 heads x 128 B = 32 KB) and
// streams at 6.8 - 7.1 TB/s (same probe, same pool, same random page order). So here:
//   * a tile is 32 tokens of ALL kv heads (K box + V box); the tensor map lists the dimensions as (dim, token, head,
//     page), so the box lands in shared memory head-major: each head's [32 tokens x 128 B] sub-tile is swizzled by
//     token exactly like the tiles of attn_rows.cuh and feeds the same ldmatrix / mma.sync code;
//   * a unit of the tile stream is a whole request (all its kv heads advance together), CTA c takes the contiguous
//     slice [c T / G, (c + 1) T / G) of the stream and only the first and last request of a slice can be partial:
//     two workspace slots per CTA, 8 rows per kv head each, merged by attn_combine_kernel (wide = 1);
//   * consumer warp w serves kv head w: its own 8 query rows, its own running (max, sum, O), no merge between
//     warps. Two producer warps alternate over the tiles.
#pragma once

#include "attn_rows.cuh"

namespace ga {
namespace attn {

constexpr int WIDE_T = 32;        // tokens per tile
constexpr int WIDE_HEADS = 8;     // consumer warps = kv heads one CTA can serve
constexpr int WIDE_NP = 2;        // producer warps
constexpr int WIDE_THREADS = (WIDE_HEADS + WIDE_NP) * 32;
constexpr int WIDE_ROWS = 8 * WIDE_HEADS;  // rows of a workspace slot
constexpr int WIDE_MAX_STAGES = 8;

// Shared memory: the ring (1024-byte aligned stages of 2 * kv_heads * WIDE_T * 128 bytes), then the barriers.
__host__ __device__ constexpr int wide_stage_bytes(int kvh) { return 2 * kvh * WIDE_T * 128; }
__host__ __device__ constexpr int wide_stages(int kvh) {
  int n = (SMEM_OPTIN - 2048) / wide_stage_bytes(kvh);
  return n > WIDE_MAX_STAGES ? WIDE_MAX_STAGES : n;
}
__host__ __device__ constexpr int wide_smem_bytes(int kvh) { return 1024 + wide_stages(kvh) * wide_stage_bytes(kvh) + 1024; }

// BOX: tokens per TMA box, 32 (one box per tile) or 16 (pools with 16-token pages: two boxes per tile). A template
// parameter so that the 32-token form carries none of the second box's arithmetic.
template <int BOX>
__global__ void __launch_bounds__(WIDE_THREADS, 1)
attn_wide_kernel(const __grid_constant__ AttnDev p, const __grid_constant__ CUtensorMap kmap,
                 const __grid_constant__ CUtensorMap vmap) {
  static_assert(BOX == WIDE_T || BOX * 2 == WIDE_T, "box size");
  using C = Cfg<128, 1, 1, 1, 2, 1>;  // head_dim 128: fragment shapes of the 8-row path
  extern __shared__ uint8_t smem_raw[];
  const uint32_t ring = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const int kvh = p.kvh;
  const int stage_bytes = wide_stage_bytes(kvh), nst = wide_stages(kvh);
  const uint32_t bars = ring + nst * stage_bytes;  // full[nst], empty[nst]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int i = 0; i < nst; ++i) {
      mbar_init(bars + i * 8, 1);
      mbar_init(bars + (nst + i) * 8, kvh);
    }
    mbar_fence_init();
  }
  __syncthreads();
  // Programmatic dependent launch, as in attn_rows_kernel: the set-up above overlapped the kernel before this one.
  grid_dep_wait();
  grid_dep_launch();

  SliceWalker walk;
  walk.init(p, blockIdx.x, gridDim.x, lane, WIDE_T, 1);
  if (blockIdx.x == 0 && warp == 0) publish_prefix(p, lane, WIDE_T);
  Seg s;
  int it = 0;  // tiles of this CTA so far: ring position shared by producers and consumers

  if (warp >= WIDE_HEADS) {
    // ------------------------------------------------------------------ producer warps
    const int pw = warp - WIDE_HEADS;
    PtWindow win;
    win.b = -1;
    win.base = win.cur = win.nxt = 0;
    if (lane == 0) {
      tma_prefetch_desc(&kmap);
      tma_prefetch_desc(&vmap);
    }
    while (walk.next(p, s)) {
      for (int tt = s.t_lo; tt < s.t_hi; ++tt, ++it) {
        if ((it % WIDE_NP) != pw) continue;
        const int stage = it % nst, use = it / nst;
        if (use > 0 && !mbar_wait(bars + (nst + stage) * 8, (use - 1) & 1)) {
          if (lane == 0) atomicExch(p.status, GA_ST_WAIT_EMPTY);
          return;
        }
        // A box never straddles a page (pages hold a multiple of its tokens) and lies in the page as a whole. A
        // tile is one box of 32 tokens or, on 16-token pages, two boxes of 16 from two pages; a second box that
        // starts past the end of the sequence is not asked for (its page-table entry may be padding). Tokens past
        // the end of the sequence inside a box are masked later.
        const int n0 = tt * WIDE_T;
        const int nbx = (BOX < WIDE_T && n0 + BOX < s.L) ? 2 : 1;
        const int box_bytes = kvh * BOX * 128;
        if (lane == 0) mbar_expect_tx(bars + stage * 8, static_cast<uint32_t>(2 * nbx * box_bytes));
        __syncwarp();
        for (int i = 0; i < nbx; ++i) {
          const int n = n0 + i * BOX;
          int page = pt_lookup(p, win, s.b, n >> p.page_shift, lane);
          if (page < 0 || page >= p.num_pages) {
            if (lane == 0) atomicExch(p.status, GA_ST_BAD_PAGE);  // recorded; an out-of-range box reads as zeros
          }
          if (lane < 2) {
            const uint32_t dst = ring + stage * stage_bytes + lane * (stage_bytes / 2) + i * box_bytes;
            tma_load_4d(dst, lane ? &vmap : &kmap, bars + stage * 8, 0, n & p.page_mask, 0, page);
          }
        }
      }
    }
    return;
  }
  if (warp >= kvh) return;  // fewer kv heads than consumer warps

  // -------------------------------------------------------------------- consumer warp = kv head
  const int g = lane >> 2, t = lane & 3;
  const uint32_t hop = BOX == WIDE_T ? 0u : static_cast<uint32_t>((kvh - 1) * BOX * 128);
  RowAcc8<C> acc;
  uint32_t qf[4][2];
  int pos;
  bool failed = false;
  while (walk.next(p, s)) {
    Seg sw = s;
    sw.h = warp;
    load_q_frags8<C>(p, sw, lane, qf, pos, 0);
    acc.reset();
    const float kds = p.kd ? p.kd[s.b * p.kd_s0 + warp * p.kd_s1] : 1.f;
    const float vds = p.vd ? p.vd[s.b * p.vd_s0 + warp * p.vd_s1] : 1.f;
    const float sl2 = p.scale_log2 * kds;
    for (int tt = s.t_lo; tt < s.t_hi; ++tt, ++it) {
      const int stage = it % nst, use = it / nst;
      if (!failed && !mbar_wait(bars + stage * 8, use & 1)) {
        if (lane == 0) atomicExch(p.status, GA_ST_WAIT_FULL);
        failed = true;
      }
      if (failed) continue;
      // head `warp` of a box is BOX tokens x 128 bytes; with two boxes its second 16 tokens sit a box further
      const uint32_t k_addr = ring + stage * stage_bytes + warp * (BOX * 128);
      consume_tile8<C, WIDE_T>(p, sw, tt * WIDE_T, k_addr, k_addr + stage_bytes / 2, qf, pos, sl2, acc, lane, 0, hop);
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(bars + (nst + stage) * 8);
    }
    acc.l += __shfl_xor_sync(0xffffffffu, acc.l, 1);
    acc.l += __shfl_xor_sync(0xffffffffu, acc.l, 2);
    const int valid_rows = s.nq * p.gqa;
    // this lane's two output columns are rows 2t and 2t+1; their statistics live in quads 2t, 2t+1
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const float m_r = __shfl_sync(0xffffffffu, acc.m, (2 * t + e) * 4);
      const float l_r = __shfl_sync(0xffffffffu, acc.l, (2 * t + e) * 4);
      const int r = 2 * t + e;
      if (r >= valid_rows) continue;
      const float inv = l_r > 0.f ? 1.f / l_r : 0.f;
      const float lse2 = l_r > 0.f ? m_r + lg2(l_r) - P_SHIFT : -INFINITY;
      if (s.slot >= 0) {
        // a piece of a request that other CTAs share: normalised fp32 rows and the log2-domain LSE into the slot
        const long long row = static_cast<long long>(s.slot) * WIDE_ROWS + warp * 8 + r;
#pragma unroll
        for (int db = 0; db < 8; ++db)
          *reinterpret_cast<float2*>(p.ws_o + row * 128 + db * 16 + 2 * g) = make_float2(acc.ot[db][e] * inv, acc.ot[db][2 + e] * inv);
        if (g == 0) p.ws_lse[row] = lse2;
      } else {
#pragma unroll
        for (int db = 0; db < 8; ++db) store_pair(p, sw, 128, WIDE_ROWS, r, db * 16 + 2 * g, acc.ot[db][e], acc.ot[db][2 + e], inv, vds);
        if (g == 0) store_lse(p, sw, WIDE_ROWS, r, m_r, l_r);
      }
    }
  }
}

}  // namespace attn
}  // namespace ga

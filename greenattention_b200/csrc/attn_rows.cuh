// FP8 (e4m3) paged-KV attention for a block of query rows against a range of KV tiles: the kernel
// behind decode and speculative verify (split-KV, persistent, load-balanced over the SMs) and the
// warp-level extend path.
//
// Replaces the reference's SM90 decode/verify kernel (csrc/sm90/attn_decode_fp8/kernel.cuh:339-657), its
// device split planner (kernel.cuh:142-153,207-253) and its page gather (kernel.cuh:160-195). Same math:
// rows = (query token, q head of one kv head) packed token-major (row = token * GQA + head, kernel.cuh:6-8),
// S = scale * k_descale * Q K^T with a bf16 Q rounded to e4m3 (kernel.cuh:489-496), bottom-right causal mask
// and optional left window (kernel.cuh:468-474,540-556), online softmax in the log2 domain with P rounded to
// e4m3 after a x256 scale (kernel.cuh:296-336), O = v_descale * P V / l, natural-log LSE (kernel.cuh:621-653).
//
// B200 design (not the SM90 structure):
//  * One persistent CTA per SM. The whole call is one stream of 64-token KV tiles ordered by (request, kv
//    head); CTA c owns the contiguous slice [c*T/G, (c+1)*T/G) of it, so ragged contexts balance to within
//    one tile and only the first and last unit of a slice can be partial (two workspace slots per CTA).
//    The slice is derived on the device from the live cache_seqlens, so the grid is static under CUDA
//    graphs (the property green_attention/attn_decode.py:28-31 asks of the split plan).
//  * A producer warp gathers pages into a deep shared-memory ring with TMA tensor copies (128B swizzle,
//    one box per page and 128-byte head slice; never multicast), or with 16-byte cp.async for pages too
//    small for a swizzle-aligned box. Consumer warps read operands with ldmatrix straight from the swizzled
//    tiles: K as the col-major B operand of e4m3 mma.sync, V through ldmatrix.trans + byte permutes.
//  * Consumer warps are arranged MT (16-row tiles) x WN (tile groups); each group keeps its own running
//    (max, sum, O) and the groups are merged in a fixed order at the end of a unit, so results are
//    bit-reproducible run to run.
#pragma once

#include "ga_common.cuh"

namespace ga {
namespace attn {

constexpr int TN = 64;                 // tokens per ring stage
constexpr int ATOM_BYTES = TN * 128;   // one 128-byte-wide swizzled slab of a tile
constexpr int SMEM_OPTIN = 232448;     // 227 KiB
constexpr int MAX_ROWS = 128;
constexpr float P_SHIFT = 8.f;         // P is scaled by 2^8 before the e4m3 rounding

struct AttnDev {
  const uint8_t* q;
  int q_bf16;
  long long q_s0, q_s1;  // elements
  const uint8_t* k;
  const uint8_t* v;
  long long k_s0, k_s1, k_s2;  // page, token, head strides (bytes)
  long long v_s0, v_s1, v_s2;
  int page_shift, page_mask, num_pages;
  int kvh, gqa;
  const int* pt;
  long long pt_s0, pt_s1;
  int pt_cols;       // entries per page-table row
  const int* seqlens;
  const int* cu;
  const float* kd;
  long long kd_s0, kd_s1;
  const float* vd;
  long long vd_s0, vd_s1;
  void* out;
  int out_f32;
  long long o_s0, o_s1;
  float* lse;
  long long total_q;
  int batch;
  int window_left;
  float scale_log2;  // softmax_scale * log2(e)
  int use_tma;
  int box_tok;       // tokens per TMA box = min(page_size, TN)
  int max_q;         // decode/verify: query tokens per request are capped here (rows <= 16*MT)
  int bq;            // extend: query tokens per row block
  int tc_mode;       // tcgen05 kernel: 0 = slices of the tile stream (decode / verify route), 1 = extend items
  int nblk;          // tcgen05 extend: the host's upper bound on the number of query blocks
  int rows_cap;      // rows per workspace slot (row stride of ws_o / ws_lse)
  int gang;          // split-KV kernels: CTAs work in gangs of kv_heads on slices of whole requests
  // split-KV workspace
  int* status;
  int* prefix;       // [batch + 1] exclusive prefix of per-request tile counts (written by CTA 0)
  float* ws_o;       // [2*grid][16*MT][HD] normalised partial outputs
  float* ws_lse;     // [2*grid][16*MT] log2-domain LSE of each partial
};

// Per-request tile bookkeeping shared by the main kernel and the combine kernel.
struct SeqInfo {
  int L, ql, tlo, cnt;
};
// Keys of request b. A length beyond what the page-table row can address (a caller error that live lengths
// under graph replay can produce) is cut to the addressable range and recorded in the status word, so neither
// gather path ever indexes past the row.
__device__ __forceinline__ int seq_len_checked(const AttnDev& p, int b) {
  int L = p.seqlens[b];
  const long long cap = static_cast<long long>(p.pt_cols) << p.page_shift;
  if (L > cap) {
    L = static_cast<int>(cap);
    atomicExch(p.status, GA_ST_LEN_RANGE);
  }
  return L;
}
// `tile`: KV tokens per tile of the caller's stream (TN for the warp-level kernel, 128 for the tcgen05 one).
__device__ __forceinline__ SeqInfo seq_info(const AttnDev& p, int b, int tile = TN) {
  SeqInfo s;
  s.L = seq_len_checked(p, b);
  int ql = p.cu[b + 1] - p.cu[b];
  s.ql = ql < p.max_q ? ql : p.max_q;
  if (s.L <= 0 || s.ql <= 0) {
    s.tlo = 0;
    s.cnt = 0;
    return s;
  }
  int thi = (s.L + tile - 1) / tile;
  int lower = 0;
  if (p.window_left >= 0) {
    lower = s.L - s.ql - p.window_left;
    if (lower < 0) lower = 0;
  }
  s.tlo = lower / tile;
  s.cnt = thi - s.tlo;
  return s;
}

__device__ __forceinline__ int warp_incl_scan(int v, int lane) {
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    int o = __shfl_up_sync(0xffffffffu, v, d);
    if (lane >= d) v += o;
  }
  return v;
}

// First tile of CTA c's slice of T tiles over G CTAs.
__device__ __forceinline__ long long slice_start(long long T, int G, int c) { return (T * c) / G; }

struct Seg {
  int b, h;
  int q0, nq;      // first query token (row of q) and token count of the row block
  int pos0;        // absolute position of query token 0 of the block
  int L;
  int t_lo, t_hi;  // KV tiles [t_lo, t_hi) to process
  int slot;        // < 0: the block's final result; >= 0: partial into workspace slot
};

// Walks the units (request, kv head) of one CTA's slice. Every warp of the CTA runs an identical copy.
struct SliceWalker {
  long long g0, g1, u0;
  int b, h, cnt, tlo, L, ql;
  int cta, tile, kvh;
  bool live;

  // `heads`: units per request. The kv heads of the call when a unit is one (request, kv head); 1 when a unit is a
  // whole request and every tile carries all kv heads (the all-heads decode kernel), in which case s.h stays 0.
  __device__ void init(const AttnDev& p, int cta_, int G, int lane, int tile_ = TN, int heads = 0) {
    cta = cta_;
    tile = tile_;
    kvh = heads > 0 ? heads : p.kvh;
    long long sum = 0;
    for (int b0 = 0; b0 < p.batch; b0 += 32) {
      int bb = b0 + lane;
      sum += bb < p.batch ? seq_info(p, bb, tile).cnt : 0;
    }
#pragma unroll
    for (int d = 16; d; d >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, d);
    long long T = sum * kvh;
    g0 = slice_start(T, G, cta);
    g1 = slice_start(T, G, cta + 1);
    live = g1 > g0;
    if (!live) return;
    long long pre = 0;
    b = -1;
    for (int b0 = 0; b0 < p.batch && b < 0; b0 += 32) {
      int bb = b0 + lane;
      int c = bb < p.batch ? seq_info(p, bb, tile).cnt : 0;
      int incl = warp_incl_scan(c, lane);
      unsigned hit = __ballot_sync(0xffffffffu, (pre + incl) * kvh > g0);
      if (hit) {
        int src = __ffs(hit) - 1;
        int incl_s = __shfl_sync(0xffffffffu, incl, src);
        int c_s = __shfl_sync(0xffffffffu, c, src);
        b = b0 + src;
        pre += incl_s - c_s;
      } else {
        pre += __shfl_sync(0xffffffffu, incl, 31);
      }
    }
    if (b < 0) {
      live = false;
      return;
    }
    load(p);
    h = static_cast<int>((g0 - pre * kvh) / cnt);
    u0 = pre * kvh + static_cast<long long>(h) * cnt;
  }
  __device__ void load(const AttnDev& p) {
    SeqInfo s = seq_info(p, b, tile);
    cnt = s.cnt;
    tlo = s.tlo;
    L = s.L;
    ql = s.ql;
  }
  __device__ bool next(const AttnDev& p, Seg& s) {
    if (!live) return false;
    long long lo = u0 > g0 ? u0 : g0;
    long long u1 = u0 + cnt;
    long long hi = u1 < g1 ? u1 : g1;
    s.b = b;
    s.h = h;
    s.q0 = p.cu[b];
    s.nq = ql;
    s.pos0 = L - ql;
    s.L = L;
    s.t_lo = tlo + static_cast<int>(lo - u0);
    s.t_hi = tlo + static_cast<int>(hi - u0);
    s.slot = (lo == u0 && hi == u1) ? -1 : 2 * cta + (u0 <= g0 ? 0 : 1);
    // advance
    u0 = u1;
    if (u0 >= g1) {
      live = false;
    } else if (++h == kvh) {
      h = 0;
      do {
        ++b;
        if (b >= p.batch) {
          live = false;
          break;
        }
        load(p);
      } while (cnt == 0);
    }
    return true;
  }
};

// Next segment of a CTA of the split-KV kernels. In a ganged launch the walker speaks of gangs and whole requests:
// the segment becomes this CTA's kv head and its own workspace slots.
__device__ __forceinline__ bool walk_next(const AttnDev& p, SliceWalker& walk, Seg& s) {
  if (!walk.next(p, s)) return false;
  if (p.gang) {
    s.h = blockIdx.x % p.kvh;
    if (s.slot >= 0) s.slot = 2 * static_cast<int>(blockIdx.x) + (s.slot & 1);
  }
  return true;
}

// One warp writes the exclusive prefix of the per-request tile counts the combine kernel works from.
__device__ __forceinline__ void publish_prefix(const AttnDev& p, int lane, int tile) {
  int pre = 0;
  for (int b0 = 0; b0 < p.batch; b0 += 32) {
    int bb = b0 + lane;
    int c = bb < p.batch ? seq_info(p, bb, tile).cnt : 0;
    int incl = warp_incl_scan(c, lane);
    if (bb < p.batch) p.prefix[bb] = pre + incl - c;
    pre += __shfl_sync(0xffffffffu, incl, 31);
  }
  if (lane == 0) p.prefix[p.batch] = pre;
}

// Extend: row block `x` of the call (heaviest, i.e. latest, blocks first) for kv head `h`. Every warp runs an
// identical copy. `tile` is the KV tile size the caller iterates in. Returns false when x is past the last block.
__device__ __forceinline__ bool extend_block(const AttnDev& p, int x_in, int h, int tile, int lane, Seg& one) {
  int total = 0, found_b = -1, found_pre = 0, pre = 0;
  for (int b0 = 0; b0 < p.batch; b0 += 32) {
    int bb = b0 + lane;
    int ql = bb < p.batch ? p.cu[bb + 1] - p.cu[bb] : 0;
    total += (ql + p.bq - 1) / p.bq;
  }
#pragma unroll
  for (int d = 16; d; d >>= 1) total += __shfl_xor_sync(0xffffffffu, total, d);
  const int x = total - 1 - x_in;
  if (x < 0) return false;
  for (int b0 = 0; b0 < p.batch && found_b < 0; b0 += 32) {
    int bb = b0 + lane;
    int ql = bb < p.batch ? p.cu[bb + 1] - p.cu[bb] : 0;
    int nb = (ql + p.bq - 1) / p.bq;
    int incl = warp_incl_scan(nb, lane);
    unsigned hit = __ballot_sync(0xffffffffu, pre + incl > x);
    if (hit) {
      int src = __ffs(hit) - 1;
      found_b = b0 + src;
      found_pre = pre + __shfl_sync(0xffffffffu, incl, src) - __shfl_sync(0xffffffffu, nb, src);
    } else {
      pre += __shfl_sync(0xffffffffu, incl, 31);
    }
  }
  if (found_b < 0) return false;
  const int b = found_b, j = x - found_pre;
  const int ql = p.cu[b + 1] - p.cu[b];
  one.b = b;
  one.h = h;
  one.q0 = p.cu[b] + j * p.bq;
  one.nq = min(p.bq, ql - j * p.bq);
  one.L = seq_len_checked(p, b);
  one.pos0 = one.L - ql + j * p.bq;
  int last = one.pos0 + one.nq - 1;
  if (last > one.L - 1) last = one.L - 1;
  one.t_hi = last >= 0 ? last / tile + 1 : 0;
  int lower = p.window_left >= 0 ? one.pos0 - p.window_left : 0;
  one.t_lo = lower > 0 ? lower / tile : 0;
  if (one.t_lo > one.t_hi) one.t_lo = one.t_hi;
  one.slot = -1;
  return true;
}

constexpr int gcd_(int a, int b) { return b == 0 ? a : gcd_(b, a % b); }

template <int HD, int MT, int WN, int NP_ = 4, int CAP_ = 24, int SUB_ = 1, int DS_ = 1>
struct Cfg {
  static constexpr int ATOMS = HD / 128;
  // 8-row path only: the DS warps that share a tile work on the SAME rows and take a 1/DS share of the output dims
  // each (both do the whole QK product). At head_dim 512 this halves the O accumulators to 64 registers per thread.
  static constexpr int DS = DS_;
  static constexpr int NCW = MT * WN;               // consumer warps
  // Producer warps: each issues every NP-th tile. One warp's issue loop (barrier wait, expect_tx, TMA
  // issue) takes on the order of a thousand cycles per tile, far too slow to keep HBM busy on its own.
  static constexpr int NP = NP_;
  static constexpr int THREADS = (NCW + NP) * 32;
  static constexpr int ROWS = MT * 16 / DS_;
  static constexpr int SUB = SUB_;                               // 64-token tiles per ring stage
  static constexpr int TILE_BYTES = 2 * ATOMS * ATOM_BYTES;      // one tile: K slabs then V slabs
  static constexpr int STAGE_BYTES = SUB * TILE_BYTES;
  static constexpr int V_OFF = ATOMS * ATOM_BYTES;
  static constexpr int PITCH = HD + 4;              // floats per row of the merge buffer
  static constexpr int MERGE_BYTES = WN > 1 ? ROWS * PITCH * 4 + ROWS * 8 : 0;
  static constexpr int TAIL_BYTES = 1024;           // barriers
  static constexpr int NST_RAW = (SMEM_OPTIN - 1024 - MERGE_BYTES - TAIL_BYTES) / STAGE_BYTES;
  // The ring depth is a multiple of both WN and NP, so a stage is always filled by the same producer warp
  // and always drained by the same consumer group. That is what makes the parity waits sound: a warp that
  // waits for use u of a stage has itself gone through use u-1, so the barrier can never be a whole phase
  // behind the waiter (a parity wait cannot tell phase u-2 from phase u).
  static constexpr int LCM = WN * NP / gcd_(WN, NP);
  static constexpr int NST_CAP = NST_RAW > CAP_ ? CAP_ : NST_RAW;
  static constexpr int NST = NST_CAP / LCM * LCM;
  static constexpr int SMEM_BYTES = 1024 + NST * STAGE_BYTES + MERGE_BYTES + TAIL_BYTES;
  static_assert(HD == 128 || HD == 256 || HD == 512, "head_dim");
  static_assert(NST >= 2 && NST >= LCM, "ring too shallow for this warp arrangement");
};

// ---------------------------------------------------------------------------------------------------
// Producer: one warp, gathers the KV tiles of every segment into the ring.
//
// Page ids come from a register-resident window of the page table: each lane holds one entry of the
// current 32-entry window and one of the next, so a tile costs a shuffle instead of a dependent global
// load and the next window is already in flight when the current one runs out.
struct PtWindow {
  int b, base, cur, nxt;
};
__device__ __forceinline__ int pt_entry(const AttnDev& p, int b, int e) {
  return e < p.pt_cols ? __ldg(p.pt + b * p.pt_s0 + e * p.pt_s1) : 0;
}
__device__ __forceinline__ int pt_lookup(const AttnDev& p, PtWindow& w, int b, int e, int lane) {
  if (w.b != b || e < w.base || e >= w.base + 64) {
    w.b = b;
    w.base = e & ~31;
    w.cur = pt_entry(p, b, w.base + lane);
    w.nxt = pt_entry(p, b, w.base + 32 + lane);
  } else if (e >= w.base + 32) {
    w.base += 32;
    w.cur = w.nxt;
    w.nxt = pt_entry(p, b, w.base + 32 + lane);
  }
  return __shfl_sync(0xffffffffu, w.cur, e - w.base);
}

// Fills one ring stage with the `nsub` consecutive 64-token tiles that start at tile `tt` of segment `s`.
template <class C>
__device__ __forceinline__ void produce_stage(const AttnDev& p, const CUtensorMap* kmap, const CUtensorMap* vmap,
                                              const Seg& s, int tt, int nsub, uint32_t stage_addr, uint32_t full_bar,
                                              int lane, PtWindow& win) {
  if (p.use_tma) {
    const int nbox = TN / p.box_tok;
    int boxes = 0;  // boxes that hold at least one live token
    for (int u = 0; u < nsub; ++u)
      for (int i = 0; i < nbox; ++i) boxes += ((tt + u) * TN + i * p.box_tok) < s.L;
    if (lane == 0) mbar_expect_tx(full_bar, static_cast<uint32_t>(boxes) * p.box_tok * 128 * C::ATOMS * 2);
    __syncwarp();
    for (int u = 0; u < nsub; ++u) {
      const int n0 = (tt + u) * TN;
      for (int i = 0; i < nbox; ++i) {
        const int n = n0 + i * p.box_tok;
        if (n >= s.L) break;
        int page = pt_lookup(p, win, s.b, n >> p.page_shift, lane);
        if (page < 0 || page >= p.num_pages) {
          if (lane == 0) atomicExch(p.status, GA_ST_BAD_PAGE);  // recorded; an out-of-range box reads as zeros
        }
        if (lane < C::ATOMS * 2) {
          const int is_v = lane / C::ATOMS, atom = lane - is_v * C::ATOMS;
          uint32_t dst = stage_addr + u * C::TILE_BYTES + (is_v ? C::V_OFF : 0) + atom * ATOM_BYTES + i * p.box_tok * 128;
          tma_load_4d(dst, is_v ? vmap : kmap, full_bar, atom * 128, s.h, n & p.page_mask, page);
        }
      }
    }
  } else {
    for (int u = 0; u < nsub; ++u) {
      for (int r = lane; r < TN; r += 32) {
        int n = (tt + u) * TN + r;
        if (n < s.L) {
          int page = p.pt[s.b * p.pt_s0 + (n >> p.page_shift) * p.pt_s1];
          if (page < 0 || page >= p.num_pages) {
            atomicExch(p.status, GA_ST_BAD_PAGE);
            page = 0;
          }
          const uint8_t* ksrc = p.k + page * p.k_s0 + (n & p.page_mask) * p.k_s1 + s.h * p.k_s2;
          const uint8_t* vsrc = p.v + page * p.v_s0 + (n & p.page_mask) * p.v_s1 + s.h * p.v_s2;
#pragma unroll
          for (int c = 0; c < C::ATOMS * 8; ++c) {
            uint32_t off = u * C::TILE_BYTES + (c >> 3) * ATOM_BYTES + r * 128 + (((c & 7) ^ (r & 7)) << 4);
            cp_async_16(stage_addr + off, ksrc + c * 16);
            cp_async_16(stage_addr + C::V_OFF + off, vsrc + c * 16);
          }
        }
      }
    }
    cp_async_mbar_arrive_noinc(full_bar);
  }
}

// ---------------------------------------------------------------------------------------------------
// Consumer state of one warp: 16 query rows (g and g+8 per lane) x HD output dims.
template <class C>
struct RowAcc {
  float o[C::ATOMS * 16][4];  // [16-dim block * 2 + (even|odd dims)][c0..c3]
  float m[2], l[2];
  __device__ __forceinline__ void reset() {
#pragma unroll
    for (int i = 0; i < C::ATOMS * 16; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    m[0] = m[1] = -INFINITY;
    l[0] = l[1] = 0.f;
  }
};

template <class C>
__device__ __forceinline__ void load_q_frags(const AttnDev& p, const Seg& s, int mt, int lane,
                                             uint32_t (&qf)[C::ATOMS * 4][4], int (&pos)[2]) {
  const int g = lane >> 2, t = lane & 3;
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    int r = mt * 16 + g + half * 8;
    int tq = r / p.gqa;
    int hq = r - tq * p.gqa;
    bool valid = tq < s.nq;
    pos[half] = valid ? s.pos0 + tq : -1;
    const uint8_t* base = p.q;
    long long off = (static_cast<long long>(s.q0 + tq) * p.q_s0 + static_cast<long long>(s.h * p.gqa + hq) * p.q_s1);
#pragma unroll
    for (int ks = 0; ks < C::ATOMS * 4; ++ks) {
#pragma unroll
      for (int sub = 0; sub < 2; ++sub) {
        int d = ks * 32 + sub * 16 + t * 4;
        uint32_t packed = 0;
        if (valid) {
          if (p.q_bf16) {
            uint2 raw = *reinterpret_cast<const uint2*>(base + (off + d) * 2);
            packed = pack_e4m3x4(bf16_bits_to_f32(raw.x & 0xffffu), bf16_bits_to_f32(raw.x >> 16),
                                 bf16_bits_to_f32(raw.y & 0xffffu), bf16_bits_to_f32(raw.y >> 16));
          } else {
            packed = *reinterpret_cast<const uint32_t*>(base + off + d);
          }
        }
        qf[ks][sub * 2 + half] = packed;  // a0: row g k-lo, a1: row g+8 k-lo, a2: row g k-hi, a3: row g+8 k-hi
      }
    }
  }
}

// One 64-token tile: S = Q K^T, mask, online softmax, O += P V.
template <class C, bool HALF>
__device__ __forceinline__ void consume_tile(const AttnDev& p, const Seg& s, int tt, uint32_t stage_addr,
                                             const uint32_t (&qf)[C::ATOMS * 4][4], const int (&pos)[2],
                                             bool hi_rows_in, float sl2, RowAcc<C>& acc, int lane) {
  const int g = lane >> 2, t = lane & 3;
  const bool hi_rows = HALF ? false : hi_rows_in;
  const int n0 = tt * TN;
  const int lrow = lane & 7, lmat = lane >> 3;

  float sc[8][4];
#pragma unroll
  for (int j = 0; j < 8; ++j) sc[j][0] = sc[j][1] = sc[j][2] = sc[j][3] = 0.f;
  // B fragments of four 8-token groups are fetched first, then the MMAs run k-step-major so that
  // consecutive MMAs accumulate into different registers (no back-to-back dependency).
  const uint32_t xr = static_cast<uint32_t>(lrow) << 4;
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    uint32_t kb[4][C::ATOMS * 2][4];
#pragma unroll
    for (int jj = 0; jj < 4; ++jj) {
      const uint32_t rowaddr = stage_addr + ((half * 4 + jj) * 8 + lrow) * 128;
#pragma unroll
      for (int q4 = 0; q4 < C::ATOMS * 2; ++q4) {  // 64 dims (two k-steps) per ldmatrix.x4
        const int c = q4 * 4 + lmat;               // 16-byte chunk of the head vector
        ldsm_x4(rowaddr + (c >> 3) * ATOM_BYTES + ((static_cast<uint32_t>(c & 7) << 4) ^ xr), kb[jj][q4][0],
                kb[jj][q4][1], kb[jj][q4][2], kb[jj][q4][3]);
      }
    }
#pragma unroll
    for (int q4 = 0; q4 < C::ATOMS * 2; ++q4) {
#pragma unroll
      for (int sub = 0; sub < 2; ++sub) {
#pragma unroll
        for (int jj = 0; jj < 4; ++jj)
          mma_e4m3_16x8x32(sc[half * 4 + jj], qf[q4 * 2 + sub], kb[jj][q4][sub * 2], kb[jj][q4][sub * 2 + 1]);
      }
    }
  }

  // Mask only where the tile touches the causal diagonal, the window edge or the end of the sequence.
  const int first_pos = s.pos0, last_pos = s.pos0 + s.nq - 1;
  const bool need_mask = (n0 + TN > first_pos + 1) || (p.window_left >= 0 && n0 < last_pos - p.window_left);
  float mx0 = -INFINITY, mx1 = -INFINITY;
  if (need_mask) {
    const int lo0 = p.window_left >= 0 ? pos[0] - p.window_left : -(1 << 30);
    const int lo1 = p.window_left >= 0 ? pos[1] - p.window_left : -(1 << 30);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        int col = n0 + j * 8 + t * 2 + e;
        float a = sc[j][e] * sl2, b = sc[j][2 + e] * sl2;
        a = (col <= pos[0] && col >= lo0) ? a : -INFINITY;
        b = (col <= pos[1] && col >= lo1) ? b : -INFINITY;
        sc[j][e] = a;
        sc[j][2 + e] = b;
        mx0 = fmaxf(mx0, a);
        mx1 = fmaxf(mx1, b);
      }
    }
    // Rows past the end of the sequence may hold stale bytes (NaN patterns): their P is exactly 0, so
    // V must be finite there. Zero those V rows in place before they are read.
    if (n0 + TN > s.L) {
      int first = s.L - n0;
      if (first < 0) first = 0;
      for (int idx = first * (C::ATOMS * 8) + lane; idx < TN * C::ATOMS * 8; idx += 32) {
        int row = idx / (C::ATOMS * 8), c = idx - row * (C::ATOMS * 8);
        uint32_t a = stage_addr + C::V_OFF + (c >> 3) * ATOM_BYTES + row * 128 + ((c & 7) << 4);
        asm volatile("st.shared.v4.b32 [%0], {%1,%1,%1,%1};" ::"r"(a), "r"(0) : "memory");
      }
      __syncwarp();
    }
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        sc[j][e] *= sl2;
        sc[j][2 + e] *= sl2;
        mx0 = fmaxf(mx0, sc[j][e]);
        mx1 = fmaxf(mx1, sc[j][2 + e]);
      }
    }
  }
  mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
  mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
  mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
  mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
  const float mn0 = fmaxf(acc.m[0], mx0), mn1 = fmaxf(acc.m[1], mx1);
  const float mu0 = mn0 == -INFINITY ? 0.f : mn0, mu1 = mn1 == -INFINITY ? 0.f : mn1;
  const float al0 = ex2(acc.m[0] - mu0), al1 = ex2(acc.m[1] - mu1);
  acc.m[0] = mn0;
  acc.m[1] = mn1;
  if (__any_sync(0xffffffffu, al0 != 1.f || al1 != 1.f)) {
    acc.l[0] *= al0;
    acc.l[1] *= al1;
#pragma unroll
    for (int i = 0; i < C::ATOMS * 16; ++i) {
      acc.o[i][0] *= al0;
      acc.o[i][1] *= al0;
      acc.o[i][2] *= al1;
      acc.o[i][3] *= al1;
    }
  }
  const float sh0 = P_SHIFT - mu0, sh1 = P_SHIFT - mu1;
  // P is split into two e4m3 terms, hi = P rounded to 4 significant bits and lo = P - hi, and both are
  // multiplied with V into the same accumulators: the product then carries ~2^-8 relative error per
  // probability instead of the 2^-4 of a single e4m3 rounding, which is what keeps short and sharply
  // peaked rows inside the parity tolerance. The decode path is HBM-bound, the extra MMAs are free.
  uint32_t pa[2][4], pl[2][4];
#pragma unroll
  for (int c2 = 0; c2 < 2; ++c2) {
    float e[4][4], r[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      e[i][0] = ex2(sc[c2 * 4 + i][0] + sh0);
      e[i][1] = ex2(sc[c2 * 4 + i][1] + sh0);
      acc.l[0] += e[i][0] + e[i][1];
      if (hi_rows) {
        e[i][2] = ex2(sc[c2 * 4 + i][2] + sh1);
        e[i][3] = ex2(sc[c2 * 4 + i][3] + sh1);
        acc.l[1] += e[i][2] + e[i][3];
      } else {
        e[i][2] = e[i][3] = 0.f;
      }
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        float hi = __uint_as_float((__float_as_uint(e[i][c]) + 0x00080000u) & 0xfff00000u);
        r[i][c] = e[i][c] - hi;
        e[i][c] = hi;
      }
    }
    pa[c2][0] = pack_e4m3x4(e[0][0], e[0][1], e[1][0], e[1][1]);
    pa[c2][1] = hi_rows ? pack_e4m3x4(e[0][2], e[0][3], e[1][2], e[1][3]) : 0u;
    pa[c2][2] = pack_e4m3x4(e[2][0], e[2][1], e[3][0], e[3][1]);
    pa[c2][3] = hi_rows ? pack_e4m3x4(e[2][2], e[2][3], e[3][2], e[3][3]) : 0u;
    pl[c2][0] = pack_e4m3x4(r[0][0], r[0][1], r[1][0], r[1][1]);
    pl[c2][1] = hi_rows ? pack_e4m3x4(r[0][2], r[0][3], r[1][2], r[1][3]) : 0u;
    pl[c2][2] = pack_e4m3x4(r[2][0], r[2][1], r[3][0], r[3][1]);
    pl[c2][3] = hi_rows ? pack_e4m3x4(r[2][2], r[2][3], r[3][2], r[3][3]) : 0u;
  }
  // O += P V. ldmatrix.trans hands each lane V bytes of two tokens x two dims; one byte permute per
  // register pair turns them into the (4 tokens, 1 dim) words of the B fragment. The token order this
  // induces inside a 32-token chunk is the order the P fragments above already have.
  const uint32_t vbase = stage_addr + C::V_OFF;
#pragma unroll
  for (int c2 = 0; c2 < 2; ++c2) {
    const uint32_t rowaddr = vbase + ((c2 * 4 + lmat) * 8 + lrow) * 128;
#pragma unroll
    for (int grp = 0; grp < C::ATOMS * 2; ++grp) {  // four 16-dim blocks at a time
      uint32_t ve[4][2], vo[4][2];
#pragma unroll
      for (int d4 = 0; d4 < 4; ++d4) {
        const int db = grp * 4 + d4;
        uint32_t r0, r1, r2, r3;
        ldsm_x4_trans(rowaddr + (db >> 3) * ATOM_BYTES + ((static_cast<uint32_t>(db & 7) << 4) ^ xr), r0, r1, r2, r3);
        ve[d4][0] = prmt(r0, r1, 0x6420);
        ve[d4][1] = prmt(r2, r3, 0x6420);
        vo[d4][0] = prmt(r0, r1, 0x7531);
        vo[d4][1] = prmt(r2, r3, 0x7531);
      }
#pragma unroll
      for (int d4 = 0; d4 < 4; ++d4) {
        mma_e4m3_16x8x32(acc.o[(grp * 4 + d4) * 2], pa[c2], ve[d4][0], ve[d4][1]);
        mma_e4m3_16x8x32(acc.o[(grp * 4 + d4) * 2 + 1], pa[c2], vo[d4][0], vo[d4][1]);
      }
#pragma unroll
      for (int d4 = 0; d4 < 4; ++d4) {
        mma_e4m3_16x8x32(acc.o[(grp * 4 + d4) * 2], pl[c2], ve[d4][0], ve[d4][1]);
        mma_e4m3_16x8x32(acc.o[(grp * 4 + d4) * 2 + 1], pl[c2], vo[d4][0], vo[d4][1]);
      }
    }
  }
}

// Final value of one (row, 4 consecutive dims) cell, to the output tensor or to a workspace slot.
__device__ __forceinline__ void store_cell(const AttnDev& p, const Seg& s, int hd, int rows, int r, int d,
                                           float4 o, float inv, float vds) {
  if (s.slot >= 0) {
    float4 w = make_float4(o.x * inv, o.y * inv, o.z * inv, o.w * inv);
    *reinterpret_cast<float4*>(p.ws_o + (static_cast<long long>(s.slot) * rows + r) * hd + d) = w;
    return;
  }
  int tq = r / p.gqa, hq = r - tq * p.gqa;
  long long off = static_cast<long long>(s.q0 + tq) * p.o_s0 + static_cast<long long>(s.h * p.gqa + hq) * p.o_s1 + d;
  float f = inv * vds;
  if (p.out_f32) {
    *reinterpret_cast<float4*>(static_cast<float*>(p.out) + off) = make_float4(o.x * f, o.y * f, o.z * f, o.w * f);
  } else {
    __nv_bfloat162 lo = __floats2bfloat162_rn(o.x * f, o.y * f);
    __nv_bfloat162 hi = __floats2bfloat162_rn(o.z * f, o.w * f);
    uint2 pk;
    pk.x = *reinterpret_cast<uint32_t*>(&lo);
    pk.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(p.out) + off) = pk;
  }
}
__device__ __forceinline__ void store_lse(const AttnDev& p, const Seg& s, int rows, int r, float m, float l) {
  float lse2 = l > 0.f ? m + lg2(l) - P_SHIFT : -INFINITY;
  if (s.slot >= 0) {
    p.ws_lse[static_cast<long long>(s.slot) * rows + r] = lse2;
  } else if (p.lse != nullptr) {
    int tq = r / p.gqa, hq = r - tq * p.gqa;
    p.lse[static_cast<long long>(s.h * p.gqa + hq) * p.total_q + s.q0 + tq] = lse2 * 0.6931471805599453f;
  }
}

// ---------------------------------------------------------------------------------------------------
// Decode with at most 8 live rows per (request, kv head) (one query token, GQA <= 8): the shape the
// production decode runs. S = Q K^T keeps the query rows in the M dimension (rows 8..15 are padding), but
// O is accumulated TRANSPOSED, O^T[dims, rows] += V^T[dims, tokens] P^T[tokens, rows], so the 8 rows sit
// exactly in the N = 8 dimension of the MMA: half the PV MMAs and half the accumulator registers of the
// general path. The A operand V^T comes from ldmatrix.trans plus byte permutes (rows 0..7 of a 16-dim block
// take the even dims, rows 8..15 the odd ones); the B operand P^T is, lane for lane, the S accumulator
// fragment packed to e4m3. Loads and MMAs are written k-step-major / block-major so that consecutive MMAs
// never depend on each other.
template <class C>
struct RowAcc8 {
  float ot[C::ATOMS * 8 / C::DS][4];  // [16-dim block]: {even dim, row 2t}, {even, row 2t+1}, {odd, 2t}, {odd, 2t+1}
  float m, l;                 // running max / sum of row g (identical in the four lanes of a quad)
  __device__ __forceinline__ void reset() {
#pragma unroll
    for (int i = 0; i < C::ATOMS * 8 / C::DS; ++i) ot[i][0] = ot[i][1] = ot[i][2] = ot[i][3] = 0.f;
    m = -INFINITY;
    l = 0.f;
  }
};

template <class C>
__device__ __forceinline__ void load_q_frags8(const AttnDev& p, const Seg& s, int lane,
                                              uint32_t (&qf)[C::ATOMS * 4][2], int& pos, int row0) {
  const int g = lane >> 2, t = lane & 3;
  const int row = row0 + g;  // row0: first row of this warp's group of 8
  const int tq = row / p.gqa, hq = row - tq * p.gqa;
  const bool valid = tq < s.nq;
  pos = valid ? s.pos0 + tq : -1;
  const long long off = static_cast<long long>(s.q0 + tq) * p.q_s0 + static_cast<long long>(s.h * p.gqa + hq) * p.q_s1;
#pragma unroll
  for (int ks = 0; ks < C::ATOMS * 4; ++ks) {
#pragma unroll
    for (int sub = 0; sub < 2; ++sub) {
      const int d = ks * 32 + sub * 16 + t * 4;
      uint32_t packed = 0;
      if (valid) {
        if (p.q_bf16) {
          uint2 raw = *reinterpret_cast<const uint2*>(p.q + (off + d) * 2);
          packed = pack_e4m3x4(bf16_bits_to_f32(raw.x & 0xffffu), bf16_bits_to_f32(raw.x >> 16),
                               bf16_bits_to_f32(raw.y & 0xffffu), bf16_bits_to_f32(raw.y >> 16));
        } else {
          packed = *reinterpret_cast<const uint32_t*>(p.q + off + d);
        }
      }
      qf[ks][sub] = packed;
    }
  }
}

// NT: tokens of the tile (a multiple of 32); K rows at `k_addr`, V rows at `v_addr`, each NT x 128 bytes per
// 128-dim slab, swizzled by token. `hop`: extra bytes between token 15 and token 16 (a tile that arrived as two
// 16-token boxes whose halves of one head do not follow each other); 0 for every other caller.
template <class C, int NT = TN>
__device__ __forceinline__ void consume_tile8(const AttnDev& p, const Seg& s, int n0, uint32_t k_addr, uint32_t v_addr,
                                              const uint32_t (&qf)[C::ATOMS * 4][2], int pos, float sl2,
                                              RowAcc8<C>& acc, int lane, int dsel = 0, uint32_t hop = 0) {
  static_assert(NT % 32 == 0, "tile length");
  constexpr int SLABB = NT * 128;  // bytes between the 128-dim slabs of a wider head
  constexpr int NG = NT / 8;       // 8-token groups
  const int t = lane & 3;
  const int lrow = lane & 7, lmat = lane >> 3;
  const uint32_t xr = static_cast<uint32_t>(lrow) << 4;

  float sc[NG][4];
#pragma unroll
  for (int j = 0; j < NG; ++j) sc[j][0] = sc[j][1] = sc[j][2] = sc[j][3] = 0.f;
  // K fragments are fetched one 128-dim slab at a time (four 8-token groups x 64 dims per ldmatrix.x4), then the MMAs
  // of that slab run k-step-major so that consecutive MMAs accumulate into different registers. Going slab by slab
  // keeps the fragment registers at 32 whatever the head dim (holding both slabs of a 256-dim head spilled).
#pragma unroll
  for (int half = 0; half < NT / 32; ++half) {
#pragma unroll
    for (int slab = 0; slab < C::ATOMS; ++slab) {
      uint32_t kb[4][2][4];
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        const uint32_t rowaddr = k_addr + slab * SLABB + ((half * 4 + jj) * 8 + lrow) * 128 + ((half * 4 + jj) >= 2 ? hop : 0u);
#pragma unroll
        for (int q2 = 0; q2 < 2; ++q2) {
          const int c = q2 * 4 + lmat;  // 16-byte chunk of the slab
          ldsm_x4(rowaddr + ((static_cast<uint32_t>(c) << 4) ^ xr), kb[jj][q2][0], kb[jj][q2][1], kb[jj][q2][2], kb[jj][q2][3]);
        }
      }
#pragma unroll
      for (int q2 = 0; q2 < 2; ++q2) {
#pragma unroll
        for (int sub = 0; sub < 2; ++sub) {
#pragma unroll
          for (int jj = 0; jj < 4; ++jj) {
            const int ks = (slab * 2 + q2) * 2 + sub;
            mma_e4m3_16x8x32_a(sc[half * 4 + jj], qf[ks][0], 0u, qf[ks][1], 0u, kb[jj][q2][sub * 2], kb[jj][q2][sub * 2 + 1]);
          }
        }
      }
    }
  }

  const bool need_mask = (n0 + NT > s.pos0 + 1) || (p.window_left >= 0 && n0 < s.pos0 + s.nq - 1 - p.window_left);
  float mx = -INFINITY;
  if (need_mask) {
    const int lo = p.window_left >= 0 ? pos - p.window_left : -(1 << 30);
#pragma unroll
    for (int j = 0; j < NG; ++j) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int col = n0 + j * 8 + t * 2 + e;
        float a = sc[j][e] * sl2;
        a = (col <= pos && col >= lo) ? a : -INFINITY;
        sc[j][e] = a;
        mx = fmaxf(mx, a);
      }
    }
    if (n0 + NT > s.L) {  // stale rows past the end of the sequence: make V finite where P is exactly 0
      int first = s.L - n0;
      if (first < 0) first = 0;
      for (int idx = first * (C::ATOMS * 8) + lane; idx < NT * C::ATOMS * 8; idx += 32) {
        int row = idx / (C::ATOMS * 8), c = idx - row * (C::ATOMS * 8);
        uint32_t a = v_addr + (c >> 3) * SLABB + row * 128 + ((c & 7) << 4) + (row >= 16 ? hop : 0u);
        asm volatile("st.shared.v4.b32 [%0], {%1,%1,%1,%1};" ::"r"(a), "r"(0) : "memory");
      }
      __syncwarp();
    }
  } else {
#pragma unroll
    for (int j = 0; j < NG; ++j) {
      sc[j][0] *= sl2;
      sc[j][1] *= sl2;
      mx = fmaxf(mx, fmaxf(sc[j][0], sc[j][1]));
    }
  }
  mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
  mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
  const float mn = fmaxf(acc.m, mx);
  const float mu = mn == -INFINITY ? 0.f : mn;
  const float al = ex2(acc.m - mu);
  acc.m = mn;
  if (__any_sync(0xffffffffu, al != 1.f)) {
    acc.l *= al;
    const float a0 = __shfl_sync(0xffffffffu, al, (2 * t) * 4), a1 = __shfl_sync(0xffffffffu, al, (2 * t + 1) * 4);
#pragma unroll
    for (int i = 0; i < C::ATOMS * 8 / C::DS; ++i) {
      acc.ot[i][0] *= a0;
      acc.ot[i][1] *= a1;
      acc.ot[i][2] *= a0;
      acc.ot[i][3] *= a1;
    }
  }
  // P = 2^(s - m + 8), split into two e4m3 terms (4 significant bits + residual), see the general path.
  const float sh = P_SHIFT - mu;
  uint32_t ph[NG], pl[NG];
#pragma unroll
  for (int j = 0; j < NG; ++j) {
    float e0 = ex2(sc[j][0] + sh), e1 = ex2(sc[j][1] + sh);
    acc.l += e0 + e1;
    float h0 = __uint_as_float((__float_as_uint(e0) + 0x00080000u) & 0xfff00000u);
    float h1 = __uint_as_float((__float_as_uint(e1) + 0x00080000u) & 0xfff00000u);
    ph[j] = pack_e4m3x2(h0, h1);
    pl[j] = pack_e4m3x2(e0 - h0, e1 - h1);
  }
  const uint32_t vbase = v_addr;
#pragma unroll
  for (int c2 = 0; c2 < NT / 32; ++c2) {
    const uint32_t bh0 = ph[c2 * 4] | (ph[c2 * 4 + 1] << 16), bh1 = ph[c2 * 4 + 2] | (ph[c2 * 4 + 3] << 16);
    const uint32_t bl0 = pl[c2 * 4] | (pl[c2 * 4 + 1] << 16), bl1 = pl[c2 * 4 + 2] | (pl[c2 * 4 + 3] << 16);
    const uint32_t rowaddr = vbase + ((c2 * 4 + lmat) * 8 + lrow) * 128 + ((c2 * 4 + lmat) >= 2 ? hop : 0u);
#pragma unroll
    for (int grp = 0; grp < C::ATOMS / C::DS; ++grp) {  // eight 16-dim blocks at a time; slabs of this warp's share
      uint32_t va[8][4];
#pragma unroll
      for (int d8 = 0; d8 < 8; ++d8) {
        uint32_t r0, r1, r2, r3;
        ldsm_x4_trans(rowaddr + (dsel * (C::ATOMS / C::DS) + grp) * SLABB + ((static_cast<uint32_t>(d8) << 4) ^ xr), r0, r1, r2, r3);
        va[d8][0] = prmt(r0, r1, 0x6420);
        va[d8][1] = prmt(r0, r1, 0x7531);
        va[d8][2] = prmt(r2, r3, 0x6420);
        va[d8][3] = prmt(r2, r3, 0x7531);
      }
#pragma unroll
      for (int d8 = 0; d8 < 8; ++d8)
        mma_e4m3_16x8x32_a(acc.ot[grp * 8 + d8], va[d8][0], va[d8][1], va[d8][2], va[d8][3], bh0, bh1);
#pragma unroll
      for (int d8 = 0; d8 < 8; ++d8)
        mma_e4m3_16x8x32_a(acc.ot[grp * 8 + d8], va[d8][0], va[d8][1], va[d8][2], va[d8][3], bl0, bl1);
    }
  }
}

// Final value of one (row, 2 consecutive dims) cell of the 8-row path.
__device__ __forceinline__ void store_pair(const AttnDev& p, const Seg& s, int hd, int rows, int r, int d, float v0,
                                           float v1, float inv, float vds) {
  if (s.slot >= 0) {
    *reinterpret_cast<float2*>(p.ws_o + (static_cast<long long>(s.slot) * rows + r) * hd + d) =
        make_float2(v0 * inv, v1 * inv);
    return;
  }
  int tq = r / p.gqa, hq = r - tq * p.gqa;
  long long off = static_cast<long long>(s.q0 + tq) * p.o_s0 + static_cast<long long>(s.h * p.gqa + hq) * p.o_s1 + d;
  float f = inv * vds;
  if (p.out_f32) {
    *reinterpret_cast<float2*>(static_cast<float*>(p.out) + off) = make_float2(v0 * f, v1 * f);
  } else {
    *reinterpret_cast<__nv_bfloat162*>(static_cast<__nv_bfloat16*>(p.out) + off) = __floats2bfloat162_rn(v0 * f, v1 * f);
  }
}

// MODE 0: persistent split-KV over the tile stream (decode / verify). MODE 1: one row block of
// p.bq query tokens per CTA over everything it can see (extend). HALF: at most 8 live rows per CTA
// (decode with GQA <= 8): rows 8..15 of the MMA tile carry no accumulators.
template <int HD, int MT, int WN, int NP, int MODE, bool HALF, int CAP = 24, int SUB = 1, int OCC = 1, int DS = 1>
__global__ void __launch_bounds__(Cfg<HD, MT, WN, NP, CAP, SUB, DS>::THREADS, OCC)
attn_rows_kernel(const __grid_constant__ AttnDev p, const __grid_constant__ CUtensorMap kmap,
                 const __grid_constant__ CUtensorMap vmap) {
  using C = Cfg<HD, MT, WN, NP, CAP, SUB, DS>;
  static_assert(DS == 1 || (HALF && MT == DS && C::ATOMS % DS == 0), "the dims are split between the warps that share a tile");
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t ring = base;
  const uint32_t merge = ring + C::NST * C::STAGE_BYTES;
  const uint32_t bars = merge + C::MERGE_BYTES;  // full[NST], empty[NST]
  uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
  float* mergeO = reinterpret_cast<float*>(gen_base + C::NST * C::STAGE_BYTES);
  float* mergeM = mergeO + C::ROWS * C::PITCH;
  float* mergeL = mergeM + C::ROWS;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int i = 0; i < C::NST; ++i) {
      mbar_init(bars + i * 8, p.use_tma ? 1 : 32);
      mbar_init(bars + (C::NST + i) * 8, MT);
    }
    mbar_fence_init();
  }
  __syncthreads();
  // Programmatic dependent launch: everything above overlapped the tail of the kernel before this one in the
  // stream; nothing it wrote is read, and nothing it reads is written, before this wait. The combine kernel
  // that follows may be scheduled from now on (it waits for this whole grid before it reads a partial).
  grid_dep_wait();
  grid_dep_launch();

  // ---- segment source
  SliceWalker walk;
  Seg one;
  bool one_pending = false;
  if (MODE == 0) {
    // p.gang: the CTAs work in gangs of kv_heads on slices of whole requests, CTA (gang, h) taking kv head h, so
    // that the kv heads of a page (128-byte pieces of each token's kv_heads * 128 bytes) are fetched by
    // neighbouring CTAs at the same time and DRAM sees the contiguous run of the page (see attn_wide.cuh)
    if (p.gang) walk.init(p, blockIdx.x / p.kvh, gridDim.x / p.kvh, lane, TN, 1);
    else walk.init(p, blockIdx.x, gridDim.x, lane);
    if (blockIdx.x == 0 && warp == 0) publish_prefix(p, lane, TN);
  } else {
    one_pending = extend_block(p, static_cast<int>(blockIdx.x), static_cast<int>(blockIdx.y), TN, lane, one);
  }

  Seg s;
  int it = 0;  // tiles of this CTA so far: ring position shared by producer and consumers
  if (warp >= C::NCW) {
    // ------------------------------------------------------------------ producer warps
    const int pw = warp - C::NCW;
    PtWindow win;
    win.b = -1;
    win.base = win.cur = win.nxt = 0;
    if (p.use_tma && lane == 0) {
      tma_prefetch_desc(&kmap);
      tma_prefetch_desc(&vmap);
    }
    while (true) {
      if (MODE == 0) {
        if (!walk_next(p, walk, s)) break;
      } else {
        if (!one_pending) break;
        s = one;
        one_pending = false;
      }
      for (int tt = s.t_lo; tt < s.t_hi; tt += C::SUB, ++it) {
        if ((it % C::NP) != pw) continue;
        const int stage = it % C::NST, use = it / C::NST;
        if (use > 0 && !mbar_wait(bars + (C::NST + stage) * 8, (use - 1) & 1)) {
          if (lane == 0) atomicExch(p.status, GA_ST_WAIT_EMPTY);
          return;
        }
        const int nsub = s.t_hi - tt < C::SUB ? s.t_hi - tt : C::SUB;
        produce_stage<C>(p, &kmap, &vmap, s, tt, nsub, ring + stage * C::STAGE_BYTES, bars + stage * 8, lane, win);
      }
    }
    return;
  }

  // -------------------------------------------------------------------- consumer warps
  const int mt = warp % MT, wn = warp / MT;
  const int g = lane >> 2, t = lane & 3;
  bool failed = false;
  if constexpr (HALF) {
    RowAcc8<C> acc;
    uint32_t qf[C::ATOMS * 4][2];
    int pos;
    const int dsel = DS > 1 ? mt : 0;   // share of the output dims (all warps of a tile on the same rows)
    const int row0 = DS > 1 ? 0 : 8 * mt;  // first of this warp's 8 rows
    constexpr int NDB = C::ATOMS * 8 / DS;  // 16-dim blocks of this warp's share
    const int db0 = dsel * NDB;
    while (true) {
      if (MODE == 0) {
        if (!walk_next(p, walk, s)) break;
      } else {
        if (!one_pending) break;
        s = one;
        one_pending = false;
      }
      load_q_frags8<C>(p, s, lane, qf, pos, row0);
      acc.reset();
      const float kds = p.kd ? p.kd[s.b * p.kd_s0 + s.h * p.kd_s1] : 1.f;
      const float vds = p.vd ? p.vd[s.b * p.vd_s0 + s.h * p.vd_s1] : 1.f;
      const float sl2 = p.scale_log2 * kds;
      for (int tt = s.t_lo; tt < s.t_hi; tt += C::SUB, ++it) {
        if (WN > 1 && (it % WN) != wn) continue;
        const int stage = it % C::NST, use = it / C::NST;
        if (!failed && !mbar_wait(bars + stage * 8, use & 1)) {
          if (lane == 0) atomicExch(p.status, GA_ST_WAIT_FULL);
          failed = true;
        }
        if (failed) continue;
#pragma unroll 1
        for (int u = 0; u < C::SUB && tt + u < s.t_hi; ++u)
          consume_tile8<C>(p, s, (tt + u) * TN, ring + stage * C::STAGE_BYTES + u * C::TILE_BYTES,
                           ring + stage * C::STAGE_BYTES + u * C::TILE_BYTES + C::V_OFF, qf, pos, sl2, acc, lane, dsel);
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) mbar_arrive(bars + (C::NST + stage) * 8);
      }
      acc.l += __shfl_xor_sync(0xffffffffu, acc.l, 1);
      acc.l += __shfl_xor_sync(0xffffffffu, acc.l, 2);
      const int valid_rows = s.nq * p.gqa;
      // this lane's two output columns are rows 2t and 2t+1 of the warp's group of 8 (group mt when several warps
      // share the tiles, each with its own 8 rows); their statistics live in quads 2t, 2t+1
      float m_r[2], l_r[2];
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        m_r[e] = __shfl_sync(0xffffffffu, acc.m, (2 * t + e) * 4);
        l_r[e] = __shfl_sync(0xffffffffu, acc.l, (2 * t + e) * 4);
      }
      if (WN == 1) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int r = row0 + 2 * t + e;
          if (r < valid_rows) {
            const float inv = l_r[e] > 0.f ? 1.f / l_r[e] : 0.f;
#pragma unroll
            for (int db = 0; db < NDB; ++db)
              store_pair(p, s, HD, C::ROWS, r, (db0 + db) * 16 + 2 * g, acc.ot[db][e], acc.ot[db][2 + e], inv, vds);
            if (g == 0 && dsel == 0) store_lse(p, s, C::ROWS, r, m_r[e], l_r[e]);
          }
        }
      } else {
        for (int round = 0; round < WN; ++round) {
          if (wn == round) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const int r = row0 + 2 * t + e;
              float f_old = 0.f, f_own = 1.f, m_new = m_r[e], l_new = l_r[e];
              // with the dims split, each share keeps its own copy of the row statistics (slots 8.. of the 16)
              const int rs = r + 8 * dsel;
              if (round > 0) {
                const float m_old = mergeM[rs], l_old = mergeL[rs];
                m_new = fmaxf(m_old, m_r[e]);
                const float mu = m_new == -INFINITY ? 0.f : m_new;
                f_old = ex2(m_old - mu);
                f_own = ex2(m_r[e] - mu);
                l_new = l_old * f_old + l_r[e] * f_own;
              }
#pragma unroll
              for (int db = 0; db < NDB; ++db) {
                float2* cell = reinterpret_cast<float2*>(mergeO + r * C::PITCH + (db0 + db) * 16 + 2 * g);
                float2 o = make_float2(acc.ot[db][e], acc.ot[db][2 + e]);
                if (round > 0) {
                  const float2 old = *cell;
                  o = make_float2(old.x * f_old + o.x * f_own, old.y * f_old + o.y * f_own);
                }
                *cell = o;
              }
              __syncwarp();
              if (g == 0) {
                mergeM[rs] = m_new;
                mergeL[rs] = l_new;
              }
            }
          }
          named_bar_sync(1, C::NCW * 32);
        }
        const int tid = threadIdx.x;
        for (int idx = tid; idx < valid_rows * (HD / 4); idx += C::NCW * 32) {
          int r = idx / (HD / 4), d = (idx - r * (HD / 4)) * 4;
          float l = mergeL[r];
          float inv = l > 0.f ? 1.f / l : 0.f;
          float4 o = *reinterpret_cast<const float4*>(mergeO + r * C::PITCH + d);
          store_cell(p, s, HD, C::ROWS, r, d, o, inv, vds);
          if (d == 0) store_lse(p, s, C::ROWS, r, mergeM[r], l);
        }
        named_bar_sync(1, C::NCW * 32);
      }
    }
    return;
  }
  RowAcc<C> acc;
  uint32_t qf[C::ATOMS * 4][4];
  int pos[2];
  while (true) {
    if (MODE == 0) {
      if (!walk_next(p, walk, s)) break;
    } else {
      if (!one_pending) break;
      s = one;
      one_pending = false;
    }
    load_q_frags<C>(p, s, mt, lane, qf, pos);
    acc.reset();
    const bool hi_rows = s.nq * p.gqa > mt * 16 + 8;
    const bool any_rows = s.nq * p.gqa > mt * 16;
    const float kds = p.kd ? p.kd[s.b * p.kd_s0 + s.h * p.kd_s1] : 1.f;
    const float vds = p.vd ? p.vd[s.b * p.vd_s0 + s.h * p.vd_s1] : 1.f;
    const float sl2 = p.scale_log2 * kds;
    for (int tt = s.t_lo; tt < s.t_hi; tt += C::SUB, ++it) {
      if (WN > 1 && (it % WN) != wn) continue;
      const int stage = it % C::NST, use = it / C::NST;
      // A wait that runs out is recorded once; the warp then drains its loops without touching the
      // ring so that it still reaches the named barriers the other consumer warps wait on.
      if (!failed && !mbar_wait(bars + stage * 8, use & 1)) {
        if (lane == 0) atomicExch(p.status, GA_ST_WAIT_FULL);
        failed = true;
      }
      if (failed) continue;
      if (any_rows) {
#pragma unroll 1
        for (int u = 0; u < C::SUB && tt + u < s.t_hi; ++u)
          consume_tile<C, HALF>(p, s, tt + u, ring + stage * C::STAGE_BYTES + u * C::TILE_BYTES, qf, pos, hi_rows, sl2,
                                acc, lane);
      }
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(bars + (C::NST + stage) * 8);
    }
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
      acc.l[hf] += __shfl_xor_sync(0xffffffffu, acc.l[hf], 1);
      acc.l[hf] += __shfl_xor_sync(0xffffffffu, acc.l[hf], 2);
    }
    const int valid_rows = s.nq * p.gqa;
    if (WN == 1) {
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        int r = mt * 16 + g + hf * 8;
        if (r < valid_rows) {
          float inv = acc.l[hf] > 0.f ? 1.f / acc.l[hf] : 0.f;
#pragma unroll
          for (int db = 0; db < C::ATOMS * 8; ++db) {
            float4 o = make_float4(acc.o[db * 2][hf * 2], acc.o[db * 2 + 1][hf * 2], acc.o[db * 2][hf * 2 + 1],
                                   acc.o[db * 2 + 1][hf * 2 + 1]);
            store_cell(p, s, HD, C::ROWS, r, db * 16 + t * 4, o, inv, vds);
          }
          if (t == 0) store_lse(p, s, C::ROWS, r, acc.m[hf], acc.l[hf]);
        }
      }
    } else {
      // Fold the WN tile groups in a fixed order through one shared buffer.
      for (int round = 0; round < WN; ++round) {
        if (wn == round) {
#pragma unroll
          for (int hf = 0; hf < 2; ++hf) {
            int r = mt * 16 + g + hf * 8;
            float f_old = 0.f, f_own = 1.f, m_new = acc.m[hf], l_new = acc.l[hf];
            if (round > 0) {
              float m_old = mergeM[r], l_old = mergeL[r];
              m_new = fmaxf(m_old, acc.m[hf]);
              float mu = m_new == -INFINITY ? 0.f : m_new;
              f_old = ex2(m_old - mu);
              f_own = ex2(acc.m[hf] - mu);
              l_new = l_old * f_old + acc.l[hf] * f_own;
            }
            float* orow = mergeO + r * C::PITCH + t * 4;
#pragma unroll
            for (int db = 0; db < C::ATOMS * 8; ++db) {
              float4 o = make_float4(acc.o[db * 2][hf * 2], acc.o[db * 2 + 1][hf * 2], acc.o[db * 2][hf * 2 + 1],
                                     acc.o[db * 2 + 1][hf * 2 + 1]);
              float4* cell = reinterpret_cast<float4*>(orow + db * 16);
              if (round > 0) {
                float4 old = *cell;
                o = make_float4(old.x * f_old + o.x * f_own, old.y * f_old + o.y * f_own,
                                old.z * f_old + o.z * f_own, old.w * f_old + o.w * f_own);
              }
              *cell = o;
            }
            __syncwarp();
            if (t == 0) {
              mergeM[r] = m_new;
              mergeL[r] = l_new;
            }
          }
        }
        named_bar_sync(1, C::NCW * 32);
      }
      const int tid = threadIdx.x;  // consumer threads are 0 .. NCW*32-1
      for (int idx = tid; idx < valid_rows * (HD / 4); idx += C::NCW * 32) {
        int r = idx / (HD / 4), d = (idx - r * (HD / 4)) * 4;
        float l = mergeL[r];
        float inv = l > 0.f ? 1.f / l : 0.f;
        float4 o = *reinterpret_cast<const float4*>(mergeO + r * C::PITCH + d);
        store_cell(p, s, HD, C::ROWS, r, d, o, inv, vds);
        if (d == 0) store_lse(p, s, C::ROWS, r, mergeM[r], l);
      }
      named_bar_sync(1, C::NCW * 32);
    }
  }
}

// ---------------------------------------------------------------------------------------------------
// Combine: one CTA per (request, kv head). Writes zeros / -inf for requests without keys, leaves units
// that a single CTA finished alone, and merges the partials of split units in slice order
// (math of the reference's combine kernel, kernel.cuh:665-749; no atomics, so bit-reproducible).
// `wide` = 1: the partials come from the all-heads decode kernel: a unit is a whole request (so every kv head of a
// request was cut at the same tiles) and a slot holds 8 rows per kv head, head-major. `wide` = 2: they come from
// ganged CTAs of the tcgen05 kernel: a unit is a whole request, slices belong to the G / kv_heads gangs, and the
// slots of kv head h in gang c are those of CTA c * kv_heads + h.
template <int HD>
__global__ void __launch_bounds__(128) attn_combine_kernel(const __grid_constant__ AttnDev p, int G, int rows_cap,
                                                          int tile, int wide = 0) {
  const int b = blockIdx.x, h = blockIdx.y;
  // What only depends on the call's inputs (lengths, query offsets, scales) is read while the decode grid is still
  // running; everything the decode grid writes (split plan, partials) comes after the wait.
  SeqInfo si = seq_info(p, b, tile);
  int ql_all = p.cu[b + 1] - p.cu[b];
  const int q0 = p.cu[b];
  const int nq = si.ql > 0 ? si.ql : (ql_all < p.max_q ? ql_all : p.max_q);
  const int rows = nq * p.gqa;
  const float vds = p.vd ? p.vd[b * p.vd_s0 + h * p.vd_s1] : 1.f;
  grid_dep_wait();    // the whole decode grid has finished and its partials are visible
  grid_dep_launch();  // the next kernel in the stream may start its own prologue
  if (ql_all <= 0) return;
  Seg s;
  s.h = h;
  s.q0 = q0;
  s.slot = -1;
  if (si.cnt == 0) {
    for (int idx = threadIdx.x; blockIdx.z == 0 && idx < rows * (HD / 4); idx += blockDim.x) {
      int r = idx / (HD / 4), d = (idx - r * (HD / 4)) * 4;
      store_cell(p, s, HD, rows_cap, r, d, make_float4(0.f, 0.f, 0.f, 0.f), 0.f, vds);
      if (d == 0) store_lse(p, s, rows_cap, r, -INFINITY, 0.f);
    }
    return;
  }
  const int upr = wide ? 1 : p.kvh;         // units per request
  const int rbase = wide == 1 ? 8 * h : 0;  // first row of this kv head inside a slot
  const int cta_mul = wide == 2 ? p.kvh : 1, cta_add = wide == 2 ? h : 0;  // CTA that ran slice c for this kv head
  if (wide == 2) G /= p.kvh;                // slices = gangs
  const long long T = static_cast<long long>(p.prefix[p.batch]) * upr;
  const long long u0 = static_cast<long long>(p.prefix[b]) * upr + (wide ? 0 : static_cast<long long>(h) * si.cnt);
  const long long u1 = u0 + si.cnt;
  auto cta_of = [&](long long x) {
    long long c = ((x + 1) * G - 1) / T;
    if (c > G - 1) c = G - 1;
    if (c < 0) c = 0;
    while (c > 0 && slice_start(T, G, static_cast<int>(c)) > x) --c;
    while (c < G - 1 && slice_start(T, G, static_cast<int>(c) + 1) <= x) ++c;
    return static_cast<int>(c);
  };
  const int c0 = cta_of(u0), c1 = cta_of(u1 - 1);
  if (c0 == c1) return;
  const int slot0 = 2 * (c0 * cta_mul + cta_add) + (u0 <= slice_start(T, G, c0) ? 0 : 1);
  // The workspace slot of every CTA that holds a piece of this unit, worked out once (a long sequence at a small
  // batch is cut into dozens of slices; the slice bounds cost a 64-bit division each).
  constexpr int MAX_LIST = 1024;
  __shared__ int slot_list[MAX_LIST];
  const int n_list = c1 - c0 + 1 <= MAX_LIST ? c1 - c0 + 1 : MAX_LIST;  // grids here stay far below the bound
  for (int i = threadIdx.x; i < n_list; i += blockDim.x) {
    const int c = c0 + i;
    const bool empty = slice_start(T, G, c + 1) == slice_start(T, G, c);  // a CTA with an empty slice wrote nothing
    slot_list[i] = empty ? -1 : (c == c0 ? slot0 : 2 * (c * cta_mul + cta_add));
  }
  __syncthreads();
  // Rows r = blockIdx.z, blockIdx.z + gridDim.z, ... belong to this CTA (a call with few (request, kv head) pairs
  // spreads its rows over grid.z). A unit in many pieces (a long sequence at a small batch) goes one row at a time:
  // the 128 threads are 4 groups of 32: group pg folds the partials pg, pg + 4, ...
  // of the row, lane `ln` the dims 4 ln .. 4 ln + 3 (+128 at head_dim 256), and the four groups are then added in a
  // fixed order, so a unit cut into 148 slices costs 37 dependent steps instead of 148 and the result does not
  // depend on scheduling.
  __shared__ float red_mx[4];
  __shared__ float red_den[4];
  __shared__ float4 red_o[4][HD / 4];
  const int pg = threadIdx.x >> 5, ln = threadIdx.x & 31;
  if (n_list <= 8) {
    // A unit in a few pieces (the usual case in a large batch): all (row, 4 dims) cells of this CTA's rows at once,
    // each thread folding the pieces of its cells in slice order. The pieces' LSE go through shared memory first
    // (one round trip for the whole CTA) and a cell's O rows are all requested before the first is used, so the
    // kernel is two dependent round trips to the L2 however many cells a thread has (it was two per cell).
    __shared__ float lse_few[8][MAX_ROWS];
    const int my_rows = (rows - static_cast<int>(blockIdx.z) + static_cast<int>(gridDim.z) - 1) / static_cast<int>(gridDim.z);
    for (int idx = threadIdx.x; idx < n_list * my_rows; idx += blockDim.x) {
      const int i = idx / my_rows, k = idx - i * my_rows;
      const int slot = slot_list[i];
      const int r = blockIdx.z + k * gridDim.z;
      lse_few[i][k] = slot >= 0 ? __ldcg(p.ws_lse + static_cast<long long>(slot) * rows_cap + rbase + r) : -INFINITY;
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < my_rows * (HD / 4); idx += blockDim.x) {
      const int k = idx / (HD / 4), d = (idx % (HD / 4)) * 4;
      const int r = blockIdx.z + k * gridDim.z;
      float mx = -INFINITY;
#pragma unroll
      for (int i = 0; i < 8; ++i)
        if (i < n_list) mx = fmaxf(mx, lse_few[i][k]);
      float den = 0.f;
      float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
      if (mx != -INFINITY) {
        float4 v[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int slot = i < n_list ? slot_list[i] : -1;
          if (slot >= 0)
            v[i] = __ldcg(reinterpret_cast<const float4*>(p.ws_o + (static_cast<long long>(slot) * rows_cap + rbase + r) * HD + d));
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int slot = i < n_list ? slot_list[i] : -1;
          if (slot < 0) continue;
          const float w = ex2(lse_few[i][k] - mx);
          den += w;
          o.x += w * v[i].x;
          o.y += w * v[i].y;
          o.z += w * v[i].z;
          o.w += w * v[i].w;
        }
      }
      const float inv = den > 0.f ? 1.f / den : 0.f;
      store_cell(p, s, HD, rows_cap, r, d, o, inv, vds);
      if (d == 0) store_lse(p, s, rows_cap, r, mx, den * exp2f(P_SHIFT));  // l carries the main kernel's 2^P_SHIFT
    }
    return;
  }
  // The pieces' LSE of the row are read once (max pass) and kept in shared memory for the fold; the fold then has
  // eight pieces' O rows in flight per thread: one long sequence over 148 CTAs was 37 dependent round trips to the
  // L2 per row (19 us per call), now it is five.
  __shared__ float lse_list[MAX_LIST];
  constexpr int UNR = 8;
  for (int r = blockIdx.z; r < rows; r += gridDim.z) {
    float mx = -INFINITY;
    for (int i = threadIdx.x; i < n_list; i += 128) {
      const int slot = slot_list[i];
      const float v = slot >= 0 ? __ldcg(p.ws_lse + static_cast<long long>(slot) * rows_cap + rbase + r) : -INFINITY;
      lse_list[i] = v;
      mx = fmaxf(mx, v);
    }
#pragma unroll
    for (int d = 16; d; d >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, d));
    if (ln == 0) red_mx[pg] = mx;
    __syncthreads();
    mx = fmaxf(fmaxf(red_mx[0], red_mx[1]), fmaxf(red_mx[2], red_mx[3]));
    float den = 0.f;
    float4 o[HD / 128];
#pragma unroll
    for (int k = 0; k < HD / 128; ++k) o[k] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (mx != -INFINITY) {
#pragma unroll 1
      for (int i0 = pg; i0 < n_list; i0 += 4 * UNR) {
        float4 v[UNR][HD / 128];
        float w[UNR];
        bool live[UNR];
#pragma unroll
        for (int u = 0; u < UNR; ++u) {
          const int i = i0 + 4 * u;
          const int slot = i < n_list ? slot_list[i] : -1;
          live[u] = slot >= 0;
          if (live[u]) {
            const long long row = static_cast<long long>(slot) * rows_cap + rbase + r;
            w[u] = ex2(lse_list[i] - mx);
#pragma unroll
            for (int k = 0; k < HD / 128; ++k)
              v[u][k] = __ldcg(reinterpret_cast<const float4*>(p.ws_o + row * HD + k * 128 + ln * 4));
          }
        }
#pragma unroll
        for (int u = 0; u < UNR; ++u) {  // folded in slice order, as before
          if (!live[u]) continue;
          den += w[u];
#pragma unroll
          for (int k = 0; k < HD / 128; ++k) {
            o[k].x += w[u] * v[u][k].x;
            o[k].y += w[u] * v[u][k].y;
            o[k].z += w[u] * v[u][k].z;
            o[k].w += w[u] * v[u][k].w;
          }
        }
      }
    }
#pragma unroll
    for (int k = 0; k < HD / 128; ++k) red_o[pg][k * 32 + ln] = o[k];
    if (ln == 0) red_den[pg] = den;
    __syncthreads();
    if (pg == 0) {
      den = (red_den[0] + red_den[1]) + (red_den[2] + red_den[3]);
      const float inv = den > 0.f ? 1.f / den : 0.f;
#pragma unroll
      for (int k = 0; k < HD / 128; ++k) {
        const float4 a0 = red_o[0][k * 32 + ln], a1 = red_o[1][k * 32 + ln], a2 = red_o[2][k * 32 + ln], a3 = red_o[3][k * 32 + ln];
        const float4 sum = make_float4((a0.x + a1.x) + (a2.x + a3.x), (a0.y + a1.y) + (a2.y + a3.y),
                                       (a0.z + a1.z) + (a2.z + a3.z), (a0.w + a1.w) + (a2.w + a3.w));
        store_cell(p, s, HD, rows_cap, r, k * 128 + ln * 4, sum, inv, vds);
      }
      // store_lse expects (m, l) with l carrying the 2^P_SHIFT factor of the main kernel
      if (ln == 0) store_lse(p, s, rows_cap, r, mx, den * exp2f(P_SHIFT));
    }
    __syncthreads();  // the reduction buffers are reused by the next row
  }
}

}  // namespace attn
}  // namespace ga

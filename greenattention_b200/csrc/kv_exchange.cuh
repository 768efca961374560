// Cross-GPU step of a decode call whose KV range is split over GPUs (one process per GPU): exchange of the
// per-rank partial results and their LSE-weighted merge in ONE kernel over peer memory.
//
// The reference has no multi-GPU path; the merge is the math of its split-KV combine kernel one level up
// (csrc/sm90/attn_decode_fp8/kernel.cuh:665-749). Each rank holds a packed partial [rows * head_dim] O (normalised,
// fp32) followed by [rows] natural-log LSE. CTA r of every rank
//   1. stores row r of its own partial into slot [parity][rank] of every peer's gather buffer with plain peer
//      stores (the buffers are ordinary device memory mapped into every process, no multicast object is used).
//      Every float travels as an 8-byte (value, call number) pair written by one store, so the value is there when
//      its call number is: no fence and no separate flag, the exchange costs one one-way trip over NVLink;
//   2. polls, with an iteration limit, the pairs of row r in its own buffer until they carry the call number, and
//   3. merges the `world` partials of row r (its own straight from local memory).
// Rows are independent, so no grid-wide step exists. The call number lives in device memory and is advanced by the
// last CTA to finish, so a CUDA graph can replay the kernel. Buffers are double-buffered by the parity of the call
// number: a rank can be at most one call ahead of a peer (it needs the peer's rows of the call it is in), so slot
// parity p of call n + 2 is never written while a peer still reads call n, and a slot's stale pairs carry n - 2.
// A wait that runs out sets the status word and the row is merged from whatever is there: the kernel always ends.
#pragma once

#include "ga_common.cuh"

namespace ga {
namespace kvx {

constexpr int GA_ST_PEER_WAIT = 6;  // a peer's partial did not arrive within the limit
constexpr int MAX_WORLD = 16;

struct ExchDev {
  const float* mine;          // this rank's packed partial (local)
  uint2* const* bufs;         // [world] gather buffers as mapped here: [2][world][rows * (hd + 1)] (value, call) pairs
  unsigned* epoch;            // local: [0] calls finished so far, [1] CTAs of the running call that are through
  int rank, world, rows, hd;
  __nv_bfloat16* out;         // [rows, hd]
  float* lse;                 // [rows] or null
  int* status;                // local status word (sticky)
  unsigned max_polls;
};

__device__ __forceinline__ void st_pair(uint2* p, float v, unsigned e) {
  asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(__float_as_uint(v)), "r"(e) : "memory");
}
__device__ __forceinline__ uint2 ld_pair(const uint2* p) {
  uint2 v;
  asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
  return v;
}
// The value of a pair once it carries call number `e`; `ok` goes false when the limit runs out.
__device__ __forceinline__ float wait_pair(const uint2* p, unsigned e, unsigned max_polls, bool& ok) {
  uint2 v = ld_pair(p);
  for (unsigned i = 0; v.y != e && i < max_polls; ++i) {
    __nanosleep(32);
    v = ld_pair(p);
  }
  if (v.y != e) ok = false;
  return __uint_as_float(v.x);
}

__global__ void __launch_bounds__(128) exchange_merge_kernel(const ExchDev p) {
  const int r = blockIdx.x, tid = threadIdx.x;
  // Launched with programmatic stream serialization: the launch overlaps the tail of the kernel before it in the
  // stream (the combine kernel that writes `mine`); nothing is read or written before this wait.
  grid_dep_wait();
  grid_dep_launch();
  const unsigned e = *reinterpret_cast<volatile unsigned*>(p.epoch) + 1u;  // number of this call, from 1
  const int par = static_cast<int>(e & 1u);
  const long long n = static_cast<long long>(p.rows) * (p.hd + 1);  // pairs of one partial
  const long long slot_mine = static_cast<long long>(par * p.world + p.rank) * n;
  const long long lse_at = static_cast<long long>(p.rows) * p.hd + r;
  __shared__ float s_lse[MAX_WORLD];
  __shared__ int s_bad;
  if (tid == 0) s_bad = 0;

  // 1. row r of my partial to every peer
  const float my_lse = p.mine[lse_at];
  for (int j = 0; j < p.world; ++j) {
    if (j == p.rank) continue;
    uint2* dst = p.bufs[j] + slot_mine;
    for (int d = tid; d < p.hd; d += blockDim.x) st_pair(dst + static_cast<long long>(r) * p.hd + d, p.mine[static_cast<long long>(r) * p.hd + d], e);
    if (tid == 0) st_pair(dst + lse_at, my_lse, e);
  }
  // 2. the peers' LSE of the row (thread j waits for rank j), then every thread its own dims of the peers' rows
  const uint2* local = p.bufs[p.rank] + static_cast<long long>(par * p.world) * n;
  bool ok = true;
  __syncthreads();
  if (tid < p.world) s_lse[tid] = tid == p.rank ? my_lse : wait_pair(local + tid * n + lse_at, e, p.max_polls, ok);
  __syncthreads();
  float mx = -INFINITY;
  for (int s = 0; s < p.world; ++s) mx = fmaxf(mx, s_lse[s]);
  float den = 0.f;
  if (mx != -INFINITY)
    for (int s = 0; s < p.world; ++s) den += expf(s_lse[s] - mx);
  // 3. merge: every thread folds the parts in rank order, so the result does not depend on timing
  const unsigned peers = ((p.world >= 32 ? 0u : (1u << p.world)) - 1u) & ~(1u << p.rank);
  for (int d = tid; d < p.hd; d += blockDim.x) {
    // all peers' values of this dim are asked for at once; only the ones whose call number is not there yet again
    float v[MAX_WORLD];
    unsigned pending = peers;
    for (unsigned i = 0; pending != 0u && i <= p.max_polls; ++i) {
      uint2 t[MAX_WORLD];
#pragma unroll
      for (int s = 0; s < MAX_WORLD; ++s)
        if ((pending >> s) & 1u) t[s] = ld_pair(local + s * n + static_cast<long long>(r) * p.hd + d);
#pragma unroll
      for (int s = 0; s < MAX_WORLD; ++s)
        if (((pending >> s) & 1u) && t[s].y == e) {
          v[s] = __uint_as_float(t[s].x);
          pending &= ~(1u << s);
        }
      if (pending != 0u) __nanosleep(32);
    }
    if (pending != 0u) ok = false;
    float acc = 0.f;
#pragma unroll
    for (int s = 0; s < MAX_WORLD; ++s) {
      if (s >= p.world) break;
      const float x = s == p.rank ? p.mine[static_cast<long long>(r) * p.hd + d] : (((pending >> s) & 1u) ? 0.f : v[s]);
      if (mx != -INFINITY) acc += expf(s_lse[s] - mx) * x;
    }
    p.out[static_cast<long long>(r) * p.hd + d] = __float2bfloat16(den > 0.f ? acc / den : 0.f);
  }
  if (p.lse && tid == 0) p.lse[r] = den > 0.f ? mx + logf(den) : -INFINITY;
  if (!ok) s_bad = 1;
  // the last CTA through advances the call number for the next launch
  __syncthreads();
  if (tid == 0) {
    if (s_bad) atomicExch(p.status, GA_ST_PEER_WAIT);
    __threadfence();
    if (atomicAdd(p.epoch + 1, 1u) == gridDim.x - 1) {
      p.epoch[1] = 0u;
      __threadfence();
      atomicExch(p.epoch, e);
    }
  }
}

}  // namespace kvx
}  // namespace ga

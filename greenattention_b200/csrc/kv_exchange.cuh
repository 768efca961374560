// Cross-GPU step of a decode call whose KV range is split over GPUs (one process per GPU): exchange of the
// per-rank partial results and their LSE-weighted merge in ONE kernel over peer memory.
//
// The reference has no multi-GPU path; the merge is the math of its split-KV combine kernel one level up
// (csrc/sm90/attn_decode_fp8/kernel.cuh:665-749). Each rank holds a packed partial [rows * head_dim] O (normalised,
// fp32) followed by [rows] natural-log LSE. CTA r of every rank
//   1. stores row r of its own partial into slot [parity][rank] of every peer's gather buffer with plain peer
//      stores (about 0.5 KB per peer; the buffers are ordinary device memory mapped into every process, no multicast
//      object is used),
//   2. publishes the row with a release store of the call number into the peer's flag word [parity][rank][r],
//   3. waits, with an iteration limit, until its own flag words [parity][*][r] carry the call number, and
//   4. merges the `world` partials of row r (its own straight from local memory).
// Rows are independent, so no grid-wide step exists. The call number lives in device memory and is advanced by the
// last CTA to finish, so a CUDA graph can replay the kernel. Buffers are double-buffered by the parity of the call
// number: a rank can be at most one call ahead of a peer (it needs the peer's flags of the call it is in), so slot
// parity p of call n + 2 is never written while a peer still reads call n.
// A wait that runs out sets the status word and the row is merged from whatever is there: the kernel always ends.
#pragma once

#include "ga_common.cuh"

namespace ga {
namespace kvx {

constexpr int GA_ST_PEER_WAIT = 6;  // a peer's partial did not arrive within the limit
constexpr int MAX_WORLD = 16;

struct ExchDev {
  const float* mine;          // this rank's packed partial (local)
  float* const* bufs;         // [world] gather buffers as mapped here: [2][world][rows * (hd + 1)] floats each
  unsigned* const* flags;     // [world] flag arrays as mapped here: [2][world][rows] words each
  unsigned* epoch;            // local: [0] calls finished so far, [1] CTAs of the running call that are through
  int rank, world, rows, hd;
  __nv_bfloat16* out;         // [rows, hd]
  float* lse;                 // [rows] or null
  int* status;                // local status word (sticky)
  unsigned max_polls;
};

__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__global__ void __launch_bounds__(128) exchange_merge_kernel(const ExchDev p) {
  const int r = blockIdx.x, tid = threadIdx.x;
  const unsigned e = *reinterpret_cast<volatile unsigned*>(p.epoch) + 1u;  // number of this call, from 1
  const int par = static_cast<int>(e & 1u);
  const long long n = static_cast<long long>(p.rows) * (p.hd + 1);  // floats of one partial
  const long long slot_mine = static_cast<long long>(par * p.world + p.rank) * n;
  __shared__ float s_lse[MAX_WORLD];

  // 1. row r of my partial to every peer
  for (int j = 0; j < p.world; ++j) {
    if (j == p.rank) continue;
    float* dst = p.bufs[j] + slot_mine;
    for (int d = tid; d < p.hd; d += blockDim.x) dst[static_cast<long long>(r) * p.hd + d] = p.mine[static_cast<long long>(r) * p.hd + d];
    if (tid == 0) dst[static_cast<long long>(p.rows) * p.hd + r] = p.mine[static_cast<long long>(p.rows) * p.hd + r];
  }
  __threadfence_system();
  __syncthreads();
  // 2. publish, 3. wait: thread j talks to rank j
  if (tid < p.world && tid != p.rank) {
    st_release_sys(p.flags[tid] + static_cast<long long>(par * p.world + p.rank) * p.rows + r, e);
    const unsigned* f = p.flags[p.rank] + static_cast<long long>(par * p.world + tid) * p.rows + r;
    bool ok = false;
    for (unsigned i = 0; i < p.max_polls; ++i) {
      if (ld_acquire_sys(f) == e) {
        ok = true;
        break;
      }
      __nanosleep(64);
    }
    if (!ok) atomicExch(p.status, GA_ST_PEER_WAIT);
  }
  __syncthreads();
  // 4. merge: every thread folds the parts in rank order, so the result does not depend on timing
  const float* local = p.bufs[p.rank] + static_cast<long long>(par * p.world) * n;
  if (tid < p.world)
    s_lse[tid] = tid == p.rank ? p.mine[static_cast<long long>(p.rows) * p.hd + r]
                               : __ldcg(local + tid * n + static_cast<long long>(p.rows) * p.hd + r);
  __syncthreads();
  float mx = -INFINITY;
  for (int s = 0; s < p.world; ++s) mx = fmaxf(mx, s_lse[s]);
  float den = 0.f;
  if (mx != -INFINITY)
    for (int s = 0; s < p.world; ++s) den += expf(s_lse[s] - mx);
  for (int d = tid; d < p.hd; d += blockDim.x) {
    float acc = 0.f;
    if (mx != -INFINITY)
      for (int s = 0; s < p.world; ++s) {
        // peers' rows were written from other GPUs: read them past the L1
        const float v = s == p.rank ? p.mine[static_cast<long long>(r) * p.hd + d]
                                    : __ldcg(local + s * n + static_cast<long long>(r) * p.hd + d);
        acc += expf(s_lse[s] - mx) * v;
      }
    p.out[static_cast<long long>(r) * p.hd + d] = __float2bfloat16(den > 0.f ? acc / den : 0.f);
  }
  if (p.lse && tid == 0) p.lse[r] = den > 0.f ? mx + logf(den) : -INFINITY;
  // the last CTA through advances the call number for the next launch
  __syncthreads();
  if (tid == 0) {
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

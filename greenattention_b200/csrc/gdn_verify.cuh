// Replay-SSM speculative verify of Gated-DeltaNet: up to 4 chained tokens per request against a READ-ONLY
// checkpoint state plus the ring of deltas committed since that checkpoint; the new deltas go to the ring,
// the state is never written.
//
// Replaces the reference's verify pair (csrc/sm90/gdn_recurrent/verify.cuh:212-778: verify_prep_kernel +
// verify_kernel, launched by launcher.cu:117-177) for the call documented in docs/gdn-contract.md:75-132.
// Math (docs/gdn-contract.md:111-124), with W = clamp(write_pos, 0, L) history entries c at ring positions
// (cache_base + c) & (L-1), G = inclusive cumsum of the new tokens' g:
//     hw_x[v,j] = e^{sum g_hist} (S0[v] . x'_j) + sum_c e^{sum_{i>c} g_hist_i} d_c[v] (khist_c . x'_j)     x in {q, k}
//     u_j = beta_j (v_j - e^{G_j} hw_k[.,j] - sum_{i<j} e^{G_j-G_i} (k'_i.k'_j) u_i)      (= D = R T^T, T = (I+A)^-1)
//     o_j = e^{G_j} hw_q[.,j] + sum_{i<=j} e^{G_j-G_i} (k'_i.q'_j) u_i
// History d and k are the bf16 high parts only, as in the reference. Written (verify.cuh:317-323,765-775):
// out[bos+j]; for write_pos + j < L the pair (bf16(u_j), bf16(u_j - hi)) into d_cache / rawv_cache, g_j into
// g_cache, and by the first value head of each key head the pair of k'_j into k_cache / rawk_cache, all at
// (cache_base + write_pos + j) & (L-1). PAD state slot: zero output rows only. Ring slot under flush: nothing.
//
// B200 mapping: same as the recurrent kernel next door (gdn_recurrent.cuh): one CTA of four warps per
// (request, value head), the 64 KB state tile streamed once from HBM straight into registers, every dot taken
// from those registers. One kernel instead of the reference's two: the per-request scalars, the history
// scores and the d history tile (<= 32 x 128) are prepared in shared memory while the first state rows are
// in flight. The state is read once and nothing of its size is written, so the call moves half the bytes of
// the committing form.
#pragma once

#include "gdn_recurrent.cuh"

namespace ga {
namespace gdn {

constexpr int VT = 4;         // chained tokens per request
constexpr int MAX_RING = 32;  // ring length L is 16 or 32

struct GdnVerifyDev {
  const __nv_bfloat16* q;
  const __nv_bfloat16* k;
  const __nv_bfloat16* v;
  const __nv_bfloat16* a;
  const __nv_bfloat16* b;
  long long q_ts, k_ts, v_ts, a_ts, b_ts;  // token strides, elements
  const float* A_log;
  const void* dt_bias;
  int dt_bias_bf16;
  const void* state;
  int state_bf16;
  long long state_slot;
  __nv_bfloat16* d_cache;
  __nv_bfloat16* rawv_cache;
  __nv_bfloat16* k_cache;
  __nv_bfloat16* rawk_cache;
  float* g_cache;
  long long d_ss, rawv_ss, k_ss, rawk_ss, g_ss;  // ring-slot strides, elements
  const void* sidx;
  int sidx_i64;
  const void* ridx;
  int ridx_i64;
  const int* qsl;
  const int* write_pos;
  const int* cache_base;
  const signed char* is_flush;
  __nv_bfloat16* out;
  long long o_ts;
  int batch, h, hv, L;
  float scale;
};

struct VerifyShared {
  float qn[VT][KD];
  float kn[VT][KD];
  float vv[VT][VD];
  float du[VT][VD];            // the new deltas u_j, for the ring write
  __align__(16) __nv_bfloat16 dh[MAX_RING][VD];  // history deltas (bf16 high part), filled by cp.async
  float w[MAX_RING][2 * VT];   // decay_c * (khist_c . x'_m), m = k'_0..3, q'_0..3
  float red[4][32];
  float tot[32];
  float g[VT], beta[VT], eG[VT];
  float wkk[VT][VT];
  float wkq[VT][VT];
  float gh[MAX_RING];
  float total;                 // e^{sum g_hist}
};

template <typename ST>
__global__ void __launch_bounds__(THREADS, 4) gdn_verify_kernel(const GdnVerifyDev p) {
  constexpr int T = VT;
  __shared__ VerifyShared sh;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n = blockIdx.x / p.hv, hv = blockIdx.x - n * p.hv;
  const int gsz = p.hv / p.h, h = hv / gsz;
  const int grp = lane >> 3, l8 = lane & 7;

  const long long slot = p.sidx_i64 ? static_cast<const long long*>(p.sidx)[n] : static_cast<const int*>(p.sidx)[n];
  const int bos = p.qsl[n];
  int nt = p.qsl[n + 1] - bos;
  nt = nt < T ? nt : T;
  if (nt <= 0) return;
  if (slot < 0) {  // PAD: zero output rows, nothing else
    for (int j = 0; j < nt; ++j) p.out[(bos + j) * p.o_ts + hv * VD + tid] = __float2bfloat16(0.f);
    return;
  }
  const long long r = p.ridx_i64 ? static_cast<const long long*>(p.ridx)[n] : static_cast<const int*>(p.ridx)[n];
  if (p.is_flush[r] != 0) return;  // the flush path owns this row
  const int L = p.L, Lm = L - 1;
  const int base = p.cache_base[r], wp = p.write_pos[r];
  const int W = wp < 0 ? 0 : (wp > L ? L : wp);

  const ST* tile = static_cast<const ST*>(p.state) + slot * p.state_slot + static_cast<long long>(hv) * VD * KD;
  float4 s[4][4];
  auto load_pass = [&](int pass) {
#pragma unroll
    for (int ri = 0; ri < 4; ++ri) {
      const int row = warp * 32 + pass * 16 + grp * 4 + ri;
#pragma unroll
      for (int i = 0; i < 4; ++i) s[ri][i] = load_state4<ST>(tile + static_cast<long long>(row) * KD + i * 32 + l8 * 4);
    }
  };
  load_pass(0);

  // ---------------------------------------------------------------- prologue (whole CTA)
  {
    float qd[T], kd[T];
    uint4 kraw[4] = {};
#pragma unroll
    for (int t = 0; t < T; ++t) {
      const bool on = t < nt;
      qd[t] = on ? __bfloat162float(p.q[(bos + t) * p.q_ts + h * KD + tid]) : 0.f;
      kd[t] = on ? __bfloat162float(p.k[(bos + t) * p.k_ts + h * KD + tid]) : 0.f;
      sh.vv[t][tid] = on ? __bfloat162float(p.v[(bos + t) * p.v_ts + hv * VD + tid]) : 0.f;
    }
    // History, all requested now so that the latency hides under the reductions below: the deltas of this value
    // head straight into shared memory (16 threads x 16 bytes per 256-byte ring row), the gates, and this
    // thread's share of the history keys (four threads per ring entry, 32 of the 128 dims each) into registers.
    for (int i = tid; i < W * 16; i += THREADS) {
      const int c = i >> 4, ch = i & 15;
      cp_async_16(smem_u32(&sh.dh[c][ch * 8]),
                  p.d_cache + r * p.d_ss + (static_cast<long long>(hv) * L + ((base + c) & Lm)) * VD + ch * 8);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    if (tid < MAX_RING) sh.gh[tid] = tid < W ? p.g_cache[r * p.g_ss + static_cast<long long>(hv) * L + ((base + tid) & Lm)] : 0.f;
    if ((tid >> 2) < W) {
      const __nv_bfloat16* ksrc = p.k_cache + r * p.k_ss + (static_cast<long long>(h) * L + ((base + (tid >> 2)) & Lm)) * KD;
#pragma unroll
      for (int i = 0; i < 4; ++i) kraw[i] = *reinterpret_cast<const uint4*>(ksrc + ((tid & 3) + 4 * i) * 8);
    }
    // one fused block reduction: |q|^2, |k|^2, k_i.k_j (i < j), k_i.q_j (i <= j)
    float pv[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) pv[i] = 0.f;
    {
      int c = 0;
#pragma unroll
      for (int t = 0; t < T; ++t) pv[c++] = qd[t] * qd[t];
#pragma unroll
      for (int t = 0; t < T; ++t) pv[c++] = kd[t] * kd[t];
#pragma unroll
      for (int j = 0; j < T; ++j)
#pragma unroll
        for (int i = 0; i < j; ++i) pv[c++] = kd[i] * kd[j];
#pragma unroll
      for (int j = 0; j < T; ++j)
#pragma unroll
        for (int i = 0; i <= j; ++i) pv[c++] = kd[i] * qd[j];
    }
    reduce_scatter<32, 32>(pv, lane);
    sh.red[warp][lane] = pv[0];
    if (tid < T) {
      const bool on = tid < nt;
      const float x = on ? __bfloat162float(p.a[(bos + tid) * p.a_ts + hv]) : 0.f;
      const float dtb = p.dt_bias_bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(p.dt_bias)[hv])
                                       : static_cast<const float*>(p.dt_bias)[hv];
      const float bb = on ? __bfloat162float(p.b[(bos + tid) * p.b_ts + hv]) : 0.f;
      sh.g[tid] = on ? -expf(p.A_log[hv]) * softplus20(x + dtb) : 0.f;
      sh.beta[tid] = on ? 1.f / (1.f + expf(-bb)) : 0.f;
    }
    __syncthreads();
    if (tid < 32) sh.tot[tid] = sh.red[0][tid] + sh.red[1][tid] + sh.red[2][tid] + sh.red[3][tid];
    if (warp == 1) {  // decay of every history entry: e^{sum_{i>c} g_i}; lane = ring offset
      float pre = sh.gh[lane];
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const float up = __shfl_up_sync(0xffffffffu, pre, o);
        if (lane >= o) pre += up;
      }
      const float total = __shfl_sync(0xffffffffu, pre, 31);
      sh.gh[lane] = lane < W ? expf(total - pre) : 0.f;  // from here on: the decay
      if (lane == 0) sh.total = expf(total);
    }
    __syncthreads();
    float rq[T], rk[T];
#pragma unroll
    for (int t = 0; t < T; ++t) {
      rq[t] = rsqrtf(sh.tot[t] + 1e-6f) * p.scale;
      rk[t] = rsqrtf(sh.tot[T + t] + 1e-6f);
      const float kv = kd[t] * rk[t];
      sh.qn[t][tid] = qd[t] * rq[t];
      sh.kn[t][tid] = kv;
      // the first value head of a key head stores k' as a (high, residual) bf16 pair in the ring
      if (hv == h * gsz && t < nt && wp + t < L) {
        const long long at = (static_cast<long long>(h) * L + ((base + wp + t) & Lm)) * KD + tid;
        const __nv_bfloat16 hi = __float2bfloat16(kv);
        p.k_cache[r * p.k_ss + at] = hi;
        p.rawk_cache[r * p.rawk_ss + at] = __float2bfloat16(kv - __bfloat162float(hi));
      }
    }
    if (tid < T * T) {
      const int i = tid / T, j = tid - i * T;
      float Gi = 0.f, Gj = 0.f;
      for (int t = 0; t < T; ++t) {
        Gi += t <= i ? sh.g[t] : 0.f;
        Gj += t <= j ? sh.g[t] : 0.f;
      }
      const float dec = expf(Gj - Gi);
      if (i < j) sh.wkk[i][j] = dec * sh.tot[2 * T + j * (j - 1) / 2 + i] * rk[i] * rk[j];
      if (i <= j) sh.wkq[i][j] = dec * sh.tot[2 * T + T * (T - 1) / 2 + j * (j + 1) / 2 + i] * rk[i] * rq[j];
      if (i == j) sh.eG[i] = expf(Gi);
    }
    __syncthreads();
    // history scores: four threads per ring entry, each 32 of the 128 dims of the bf16 key against the 8 vectors
    if (W > 0) {
      const int c = tid >> 2, sub = tid & 3;
      float sc[2 * T];
#pragma unroll
      for (int m = 0; m < 2 * T; ++m) sc[m] = 0.f;
      if (c < W) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int d0 = (sub + 4 * i) * 8;
          const uint32_t wds[4] = {kraw[i].x, kraw[i].y, kraw[i].z, kraw[i].w};
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const float kx = bf16_bits_to_f32((wds[e >> 1] >> ((e & 1) * 16)) & 0xffffu);
#pragma unroll
            for (int m = 0; m < T; ++m) {
              sc[m] += kx * sh.kn[m][d0 + e];
              sc[T + m] += kx * sh.qn[m][d0 + e];
            }
          }
        }
      }
#pragma unroll
      for (int m = 0; m < 2 * T; ++m) {
        sc[m] += __shfl_xor_sync(0xffffffffu, sc[m], 1);
        sc[m] += __shfl_xor_sync(0xffffffffu, sc[m], 2);
      }
      if (sub == 0 && c < W) {
        const float dec = sh.gh[c];
#pragma unroll
        for (int m = 0; m < 2 * T; ++m) sh.w[c][m] = dec * sc[m];
      }
      asm volatile("cp.async.wait_group 0;" ::: "memory");
      __syncthreads();
    }
  }

  // ---------------------------------------------------------------- two passes of 16 rows per warp
  const float total = W > 0 ? sh.total : 1.f;
#pragma unroll 1
  for (int pass = 0; pass < 2; ++pass) {
    if (pass > 0) load_pass(pass);
    // all 2T dots of 4 rows against this lane's 16 columns; value order: row-major, [hk_0..hk_T-1, hq_0..hq_T-1]
    float dots[4 * 2 * T];
#pragma unroll
    for (int i = 0; i < 4 * 2 * T; ++i) dots[i] = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
#pragma unroll
      for (int t = 0; t < T; ++t) {
        const float4 kv = *reinterpret_cast<const float4*>(&sh.kn[t][i * 32 + l8 * 4]);
        const float4 qv = *reinterpret_cast<const float4*>(&sh.qn[t][i * 32 + l8 * 4]);
#pragma unroll
        for (int ri = 0; ri < 4; ++ri) {
          const float4 sv = s[ri][i];
          dots[ri * 2 * T + t] += sv.x * kv.x + sv.y * kv.y + sv.z * kv.z + sv.w * kv.w;
          dots[ri * 2 * T + T + t] += sv.x * qv.x + sv.y * qv.y + sv.z * qv.z + sv.w * qv.w;
        }
      }
    }
    reduce_scatter<4 * 2 * T, 8>(dots, lane);
    // lane pair (l8 even: hw_k, l8 odd: hw_q) of row ri = l8 / 2; the history folds in here
    const int my_ri = l8 >> 1;
    const int my_row = warp * 32 + pass * 16 + grp * 4 + my_ri;
    const int mofs = (l8 & 1) * T;
#pragma unroll
    for (int j = 0; j < T; ++j) dots[j] *= total;
    for (int c = 0; c < W; ++c) {
      const float dv = __bfloat162float(sh.dh[c][my_row]);
#pragma unroll
      for (int j = 0; j < T; ++j) dots[j] += dv * sh.w[c][mofs + j];
    }
    float u[T];
    if ((l8 & 1) == 0) {
#pragma unroll
      for (int j = 0; j < T; ++j) {
        float rr = sh.vv[j][my_row] - sh.eG[j] * dots[j];
#pragma unroll
        for (int i = 0; i < j; ++i) rr -= sh.wkk[i][j] * u[i];
        u[j] = sh.beta[j] * rr;
      }
    }
#pragma unroll
    for (int j = 0; j < T; ++j) u[j] = __shfl_sync(0xffffffffu, u[j], lane & ~1);
    if ((l8 & 1) == 0) {
#pragma unroll
      for (int j = 0; j < T; ++j) sh.du[j][my_row] = u[j];
    } else {
#pragma unroll
      for (int j = 0; j < T; ++j) {
        if (j < nt) {
          float o = sh.eG[j] * dots[j];
#pragma unroll
          for (int i = 0; i <= j; ++i) o += sh.wkq[i][j] * u[i];
          p.out[(bos + j) * p.o_ts + hv * VD + my_row] = __float2bfloat16(o);
        }
      }
    }
  }
  __syncthreads();
  // ---------------------------------------------------------------- ring write of the new deltas and gates
  for (int j = 0; j < nt; ++j) {
    if (wp + j >= L) break;
    const long long at = static_cast<long long>(hv) * L + ((base + wp + j) & Lm);
    const float d = sh.du[j][tid];
    const __nv_bfloat16 hi = __float2bfloat16(d);
    p.d_cache[r * p.d_ss + at * VD + tid] = hi;
    p.rawv_cache[r * p.rawv_ss + at * VD + tid] = __float2bfloat16(d - __bfloat162float(hi));
    if (tid == 0) p.g_cache[r * p.g_ss + at] = sh.g[j];
  }
}


// ---------------------------------------------------------------------------------------------------
// The same call with one CTA per (request, KEY head): the G value heads that share a key head run through one
// prologue (q' / k' norms, Gram terms, ring write of k', history scores are per key head) and their 2 G passes
// of state rows form one software pipeline: the rows of the next pass are requested as soon as the dots of the
// current one are out of the registers (verify never writes the state, so nothing else needs them).
template <int G>
struct VerifyGroupShared {
  float qn[VT][KD];
  float kn[VT][KD];
  float vv[G][VT][VD];
  float du[G][VT][VD];
  __align__(16) __nv_bfloat16 dh[G][MAX_RING][VD];
  float w[G][MAX_RING][2 * VT];
  float sc[MAX_RING][2 * VT];  // khist_c . x'_m, before the decay
  float red[4][32];
  float tot[32];
  float g[G][VT], beta[G][VT], eG[G][VT];
  float wkk[G][VT][VT];
  float wkq[G][VT][VT];
  float gh[G][MAX_RING];
  float total[G];
  float rq[VT], rk[VT];
};

template <typename ST, int G>
__global__ void __launch_bounds__(THREADS, 4) gdn_verify_group_kernel(const GdnVerifyDev p) {
  constexpr int T = VT;
  __shared__ VerifyGroupShared<G> sh;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n = blockIdx.x / p.h, h = blockIdx.x - n * p.h;
  const int hv0 = h * G;
  const int grp = lane >> 3, l8 = lane & 7;

  const long long slot = p.sidx_i64 ? static_cast<const long long*>(p.sidx)[n] : static_cast<const int*>(p.sidx)[n];
  const int bos = p.qsl[n];
  int nt = p.qsl[n + 1] - bos;
  nt = nt < T ? nt : T;
  if (nt <= 0) return;
  if (slot < 0) {  // PAD: zero output rows, nothing else
    for (int j = 0; j < nt; ++j)
      for (int gi = 0; gi < G; ++gi) p.out[(bos + j) * p.o_ts + (hv0 + gi) * VD + tid] = __float2bfloat16(0.f);
    return;
  }
  const long long r = p.ridx_i64 ? static_cast<const long long*>(p.ridx)[n] : static_cast<const int*>(p.ridx)[n];
  if (p.is_flush[r] != 0) return;  // the flush path owns this row
  const int L = p.L, Lm = L - 1;
  const int base = p.cache_base[r], wp = p.write_pos[r];
  const int W = wp < 0 ? 0 : (wp > L ? L : wp);

  const ST* tiles = static_cast<const ST*>(p.state) + slot * p.state_slot + static_cast<long long>(hv0) * VD * KD;
  float4 s[4][4];
  auto load_pass = [&](int ps) {  // ps = value head * 2 + half
    const ST* tile = tiles + static_cast<long long>(ps >> 1) * VD * KD;
#pragma unroll
    for (int ri = 0; ri < 4; ++ri) {
      const int row = warp * 32 + (ps & 1) * 16 + grp * 4 + ri;
#pragma unroll
      for (int i = 0; i < 4; ++i) s[ri][i] = load_state4<ST>(tile + static_cast<long long>(row) * KD + i * 32 + l8 * 4);
    }
  };
  load_pass(0);

  // ---------------------------------------------------------------- prologue (whole CTA)
  {
    float qd[T], kd[T];
    uint4 kraw[4] = {};
#pragma unroll
    for (int t = 0; t < T; ++t) {
      const bool on = t < nt;
      qd[t] = on ? __bfloat162float(p.q[(bos + t) * p.q_ts + h * KD + tid]) : 0.f;
      kd[t] = on ? __bfloat162float(p.k[(bos + t) * p.k_ts + h * KD + tid]) : 0.f;
#pragma unroll
      for (int gi = 0; gi < G; ++gi)
        sh.vv[gi][t][tid] = on ? __bfloat162float(p.v[(bos + t) * p.v_ts + (hv0 + gi) * VD + tid]) : 0.f;
    }
    // history of every value head of the group, requested now (see the one-head kernel above)
    for (int i = tid; i < G * W * 16; i += THREADS) {
      const int gi = i / (W * 16), rem = i - gi * (W * 16);
      const int c = rem >> 4, ch = rem & 15;
      cp_async_16(smem_u32(&sh.dh[gi][c][ch * 8]),
                  p.d_cache + r * p.d_ss + (static_cast<long long>(hv0 + gi) * L + ((base + c) & Lm)) * VD + ch * 8);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    if (warp < G)
      sh.gh[warp][lane] = lane < W ? p.g_cache[r * p.g_ss + static_cast<long long>(hv0 + warp) * L + ((base + lane) & Lm)] : 0.f;
    if ((tid >> 2) < W) {
      const __nv_bfloat16* ksrc = p.k_cache + r * p.k_ss + (static_cast<long long>(h) * L + ((base + (tid >> 2)) & Lm)) * KD;
#pragma unroll
      for (int i = 0; i < 4; ++i) kraw[i] = *reinterpret_cast<const uint4*>(ksrc + ((tid & 3) + 4 * i) * 8);
    }
    float pv[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) pv[i] = 0.f;
    {
      int c = 0;
#pragma unroll
      for (int t = 0; t < T; ++t) pv[c++] = qd[t] * qd[t];
#pragma unroll
      for (int t = 0; t < T; ++t) pv[c++] = kd[t] * kd[t];
#pragma unroll
      for (int j = 0; j < T; ++j)
#pragma unroll
        for (int i = 0; i < j; ++i) pv[c++] = kd[i] * kd[j];
#pragma unroll
      for (int j = 0; j < T; ++j)
#pragma unroll
        for (int i = 0; i <= j; ++i) pv[c++] = kd[i] * qd[j];
    }
    reduce_scatter<32, 32>(pv, lane);
    sh.red[warp][lane] = pv[0];
    if (tid < G * T) {
      const int gi = tid / T, t = tid - gi * T, hv = hv0 + gi;
      const bool on = t < nt;
      const float x = on ? __bfloat162float(p.a[(bos + t) * p.a_ts + hv]) : 0.f;
      const float dtb = p.dt_bias_bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(p.dt_bias)[hv])
                                       : static_cast<const float*>(p.dt_bias)[hv];
      const float bb = on ? __bfloat162float(p.b[(bos + t) * p.b_ts + hv]) : 0.f;
      sh.g[gi][t] = on ? -expf(p.A_log[hv]) * softplus20(x + dtb) : 0.f;
      sh.beta[gi][t] = on ? 1.f / (1.f + expf(-bb)) : 0.f;
    }
    __syncthreads();
    if (tid < 32) sh.tot[tid] = sh.red[0][tid] + sh.red[1][tid] + sh.red[2][tid] + sh.red[3][tid];
    if (warp < G) {  // decay of every history entry of value head `warp`: e^{sum_{i>c} g_i}; lane = ring offset
      float pre = sh.gh[warp][lane];
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const float up = __shfl_up_sync(0xffffffffu, pre, o);
        if (lane >= o) pre += up;
      }
      const float total = __shfl_sync(0xffffffffu, pre, 31);
      sh.gh[warp][lane] = lane < W ? expf(total - pre) : 0.f;
      if (lane == 0) sh.total[warp] = W > 0 ? expf(total) : 1.f;
    }
    __syncthreads();
#pragma unroll
    for (int t = 0; t < T; ++t) {
      const float rq = rsqrtf(sh.tot[t] + 1e-6f) * p.scale, rk = rsqrtf(sh.tot[T + t] + 1e-6f);
      if (tid == 0) sh.rq[t] = rq, sh.rk[t] = rk;
      const float kv = kd[t] * rk;
      sh.qn[t][tid] = qd[t] * rq;
      sh.kn[t][tid] = kv;
      if (t < nt && wp + t < L) {  // k' as a (high, residual) bf16 pair in the ring
        const long long at = (static_cast<long long>(h) * L + ((base + wp + t) & Lm)) * KD + tid;
        const __nv_bfloat16 hi = __float2bfloat16(kv);
        p.k_cache[r * p.k_ss + at] = hi;
        p.rawk_cache[r * p.rawk_ss + at] = __float2bfloat16(kv - __bfloat162float(hi));
      }
    }
    if (tid < G * T * T) {
      const int gi = tid / (T * T), ij = tid - gi * T * T, i = ij / T, j = ij - i * T;
      float Gi = 0.f, Gj = 0.f;
      for (int t = 0; t < T; ++t) {
        Gi += t <= i ? sh.g[gi][t] : 0.f;
        Gj += t <= j ? sh.g[gi][t] : 0.f;
      }
      const float dec = expf(Gj - Gi);
      const float rki = rsqrtf(sh.tot[T + i] + 1e-6f), rkj = rsqrtf(sh.tot[T + j] + 1e-6f);
      const float rqj = rsqrtf(sh.tot[j] + 1e-6f) * p.scale;
      if (i < j) sh.wkk[gi][i][j] = dec * sh.tot[2 * T + j * (j - 1) / 2 + i] * rki * rkj;
      if (i <= j) sh.wkq[gi][i][j] = dec * sh.tot[2 * T + T * (T - 1) / 2 + j * (j + 1) / 2 + i] * rki * rqj;
      if (i == j) sh.eG[gi][i] = expf(Gi);
    }
    __syncthreads();
    if (W > 0) {
      const int c = tid >> 2, sub = tid & 3;
      float sc[2 * T];
#pragma unroll
      for (int m = 0; m < 2 * T; ++m) sc[m] = 0.f;
      if (c < W) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int d0 = (sub + 4 * i) * 8;
          const uint32_t wds[4] = {kraw[i].x, kraw[i].y, kraw[i].z, kraw[i].w};
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const float kx = bf16_bits_to_f32((wds[e >> 1] >> ((e & 1) * 16)) & 0xffffu);
#pragma unroll
            for (int m = 0; m < T; ++m) {
              sc[m] += kx * sh.kn[m][d0 + e];
              sc[T + m] += kx * sh.qn[m][d0 + e];
            }
          }
        }
      }
#pragma unroll
      for (int m = 0; m < 2 * T; ++m) {
        sc[m] += __shfl_xor_sync(0xffffffffu, sc[m], 1);
        sc[m] += __shfl_xor_sync(0xffffffffu, sc[m], 2);
      }
      if (sub == 0 && c < W) {
#pragma unroll
        for (int gi = 0; gi < G; ++gi) {
          const float dec = sh.gh[gi][c];
#pragma unroll
          for (int m = 0; m < 2 * T; ++m) sh.w[gi][c][m] = dec * sc[m];
        }
      }
      asm volatile("cp.async.wait_group 0;" ::: "memory");
      __syncthreads();
    }
  }

  // ---------------------------------------------------------------- 2 G passes of 16 rows per warp, pipelined
#pragma unroll 1
  for (int ps = 0; ps < 2 * G; ++ps) {
    const int gi = ps >> 1;
    float dots[4 * 2 * T];
#pragma unroll
    for (int i = 0; i < 4 * 2 * T; ++i) dots[i] = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
#pragma unroll
      for (int t = 0; t < T; ++t) {
        const float4 kv = *reinterpret_cast<const float4*>(&sh.kn[t][i * 32 + l8 * 4]);
        const float4 qv = *reinterpret_cast<const float4*>(&sh.qn[t][i * 32 + l8 * 4]);
#pragma unroll
        for (int ri = 0; ri < 4; ++ri) {
          const float4 sv = s[ri][i];
          dots[ri * 2 * T + t] += sv.x * kv.x + sv.y * kv.y + sv.z * kv.z + sv.w * kv.w;
          dots[ri * 2 * T + T + t] += sv.x * qv.x + sv.y * qv.y + sv.z * qv.z + sv.w * qv.w;
        }
      }
    }
    if (ps + 1 < 2 * G) load_pass(ps + 1);  // the registers are free: the next rows fly under the rest of this pass
    reduce_scatter<4 * 2 * T, 8>(dots, lane);
    const int my_ri = l8 >> 1;
    const int my_row = warp * 32 + (ps & 1) * 16 + grp * 4 + my_ri;
    const int mofs = (l8 & 1) * T;
    const float total = sh.total[gi];
#pragma unroll
    for (int j = 0; j < T; ++j) dots[j] *= total;
    for (int c = 0; c < W; ++c) {
      const float dv = __bfloat162float(sh.dh[gi][c][my_row]);
#pragma unroll
      for (int j = 0; j < T; ++j) dots[j] += dv * sh.w[gi][c][mofs + j];
    }
    float u[T];
    if ((l8 & 1) == 0) {
#pragma unroll
      for (int j = 0; j < T; ++j) {
        float rr = sh.vv[gi][j][my_row] - sh.eG[gi][j] * dots[j];
#pragma unroll
        for (int i = 0; i < j; ++i) rr -= sh.wkk[gi][i][j] * u[i];
        u[j] = sh.beta[gi][j] * rr;
      }
    }
#pragma unroll
    for (int j = 0; j < T; ++j) u[j] = __shfl_sync(0xffffffffu, u[j], lane & ~1);
    if ((l8 & 1) == 0) {
#pragma unroll
      for (int j = 0; j < T; ++j) sh.du[gi][j][my_row] = u[j];
    } else {
#pragma unroll
      for (int j = 0; j < T; ++j) {
        if (j < nt) {
          float o = sh.eG[gi][j] * dots[j];
#pragma unroll
          for (int i = 0; i <= j; ++i) o += sh.wkq[gi][i][j] * u[i];
          p.out[(bos + j) * p.o_ts + (hv0 + gi) * VD + my_row] = __float2bfloat16(o);
        }
      }
    }
  }
  __syncthreads();
  // ---------------------------------------------------------------- ring write of the new deltas and gates
  for (int j = 0; j < nt; ++j) {
    if (wp + j >= L) break;
#pragma unroll
    for (int gi = 0; gi < G; ++gi) {
      const long long at = static_cast<long long>(hv0 + gi) * L + ((base + wp + j) & Lm);
      const float d = sh.du[gi][j][tid];
      const __nv_bfloat16 hi = __float2bfloat16(d);
      p.d_cache[r * p.d_ss + at * VD + tid] = hi;
      p.rawv_cache[r * p.rawv_ss + at * VD + tid] = __float2bfloat16(d - __bfloat162float(hi));
      if (tid == 0) p.g_cache[r * p.g_ss + at] = sh.g[gi][j];
    }
  }
}

}  // namespace gdn
}  // namespace ga

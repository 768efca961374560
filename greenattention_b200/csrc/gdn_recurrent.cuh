// Gated-DeltaNet recurrent update for 1..8 chained tokens per request with accepted-prefix commit.
//
// Replaces the reference's one-token decode kernel (csrc/sm90/gdn_recurrent/kernel.cuh:177-296) and the
// chained-token arithmetic of its verify pair (csrc/sm90/gdn_recurrent/verify.cuh:212-778) for the
// speculative-decode contract in which the state after the accepted prefix is committed in place.
// Per-token math (docs/gdn-contract.md:25-37):
//     g = -exp(A_log) * softplus(a + dt_bias),  beta = sigmoid(b),  q' = l2norm(q) * scale,  k' = l2norm(k)
//     S <- e^g S ;  u = beta (v - S k') ;  S <- S + u k'^T ;  o = S q'
// evaluated in the re-associated form the reference's verify kernel uses (docs/gdn-contract.md:111-124):
// every dot product is taken against the ORIGINAL state S0, so the state tile is read once, stays
// read-only while all T outputs are produced, and is written once, only for requests that accept tokens:
//     hk_j = S0 k'_j,  hq_j = S0 q'_j,  G_j = g_0 + .. + g_j
//     u_j = beta_j (v_j - e^{G_j} hk_j - sum_{i<j} e^{G_j-G_i} (k'_i.k'_j) u_i)
//     o_j = e^{G_j} hq_j + sum_{i<=j} e^{G_j-G_i} (k'_i.q'_j) u_i
//     S_a = e^{G_{a-1}} S0 + sum_{i<a} e^{G_{a-1}-G_i} u_i k'_i^T          (a = accepted tokens)
//
// B200 mapping: the op is a pure HBM stream (64 KB fp32 state tile per (request, value head), read once
// and written at most once), so there is no shared-memory or tensor-core staging of the state: one CTA of
// four warps per tile, each warp streams rows straight from global memory into registers with fully
// coalesced 16-byte loads (8 lanes span a 128-byte row segment, 4 rows per load instruction), all 2T dot
// products of a row are accumulated from the same registers, reduced inside the 8-lane group with a
// reduce-scatter (28 shuffles per 16 rows at T = 4), and the committed state is produced from the same
// registers. The T normalised q/k vectors, gates and the small Gram terms are computed once per CTA while
// the first state loads are in flight.
#pragma once

#include "ga_common.cuh"

namespace ga {
namespace gdn {

constexpr int KD = 128;  // d_k
constexpr int VD = 128;  // d_v
constexpr int THREADS = 128;

struct GdnDev {
  const __nv_bfloat16* q;
  const __nv_bfloat16* k;
  const __nv_bfloat16* v;
  long long q_sn, q_st, k_sn, k_st, v_sn, v_st;
  const __nv_bfloat16* a;
  const __nv_bfloat16* b;
  long long a_sn, a_st, b_sn, b_st;
  const float* A_log;
  const void* dt_bias;
  int dt_bias_bf16;
  void* state;
  long long state_slot;  // elements
  const void* idx;
  int idx_i64;
  const int* accept;
  const int* qsl;
  void* out;
  int out_f32;
  long long o_sn, o_st;
  int batch, tokens, h, hv;
  int l2norm, round_beta, pad_reads_zero;
  float scale;
};

__device__ __forceinline__ float softplus20(float x) { return x <= 20.f ? log1pf(expf(x)) : x; }

template <typename ST>
__device__ __forceinline__ float4 load_state4(const ST* p);
template <>
__device__ __forceinline__ float4 load_state4<float>(const float* p) {
  return __ldcs(reinterpret_cast<const float4*>(p));
}
template <>
__device__ __forceinline__ float4 load_state4<__nv_bfloat16>(const __nv_bfloat16* p) {
  uint2 raw = __ldcs(reinterpret_cast<const uint2*>(p));
  return make_float4(bf16_bits_to_f32(raw.x & 0xffffu), bf16_bits_to_f32(raw.x >> 16),
                     bf16_bits_to_f32(raw.y & 0xffffu), bf16_bits_to_f32(raw.y >> 16));
}
__device__ __forceinline__ void store_state4(float* p, float4 v) { __stcs(reinterpret_cast<float4*>(p), v); }
__device__ __forceinline__ void store_state4(__nv_bfloat16* p, float4 v) {
  __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
  uint2 pk;
  pk.x = *reinterpret_cast<uint32_t*>(&lo);
  pk.y = *reinterpret_cast<uint32_t*>(&hi);
  __stcs(reinterpret_cast<uint2*>(p), pk);
}

// Reduce N values per lane over a group of W lanes (W = 8 or 32); afterwards lane l holds, in
// vals[0 .. N/W), the group totals of vals[(l % W) * N/W + j].
template <int N, int W>
__device__ __forceinline__ void reduce_scatter(float (&vals)[N], int lane) {
  static_assert(N % W == 0 || N < W, "reduce_scatter shape");
  int n = N;
#pragma unroll
  for (int d = W / 2; d >= 1; d >>= 1) {
    if (n > 1) {
      const int half = n / 2;
      const bool upper = (lane & d) != 0;
#pragma unroll
      for (int i = 0; i < N / 2; ++i) {
        if (i < half) {
          float send = upper ? vals[i] : vals[i + half];
          float keep = upper ? vals[i + half] : vals[i];
          vals[i] = keep + __shfl_xor_sync(0xffffffffu, send, d);
        }
      }
      n = half;
    } else {
      vals[0] += __shfl_xor_sync(0xffffffffu, vals[0], d);
    }
  }
}

template <int T>
struct Shared {
  float qn[T][KD];
  float kn[T][KD];
  float vv[T][VD];
  float red[4][96];
  float tot[96];
  float g[T], beta[T], eG[T];
  float wkk[T][T];  // [i][j], i < j: e^{G_j-G_i} k'_i.k'_j
  float wkq[T][T];  // [i][j], i <= j: e^{G_j-G_i} k'_i.q'_j
  float cA;         // e^{G_{a-1}}
  float cC[T];      // e^{G_{a-1}-G_i} for i < a, else 0
  float ubuf[4][16][T];  // per warp: u_j of the 16 rows of a pass
};

template <int T, typename ST>
__global__ void __launch_bounds__(THREADS, 4) gdn_recurrent_kernel(const GdnDev p) {
  __shared__ Shared<T> sh;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n = blockIdx.x / p.hv, hv = blockIdx.x - n * p.hv;
  const int h = hv / (p.hv / p.h);
  const int grp = lane >> 3, l8 = lane & 7;

  long long slot = p.idx_i64 ? static_cast<const long long*>(p.idx)[n] : static_cast<const int*>(p.idx)[n];
  const bool pad = slot < 0;
  bool dead = pad && !p.pad_reads_zero;
  if (p.qsl != nullptr && (p.qsl[n + 1] - p.qsl[n]) != p.tokens) dead = true;
  const long long out_base = n * p.o_sn + static_cast<long long>(hv) * VD;
  if (dead) {  // zero output rows, state untouched
    for (int t = 0; t < p.tokens; ++t) {
      long long o = out_base + t * p.o_st + tid;
      if (p.out_f32) static_cast<float*>(p.out)[o] = 0.f;
      else static_cast<__nv_bfloat16*>(p.out)[o] = __float2bfloat16(0.f);
    }
    return;
  }
  int acc_n = p.accept ? p.accept[n] : p.tokens;
  if (acc_n > p.tokens) acc_n = p.tokens;
  if (acc_n < 0 || pad) acc_n = 0;

  ST* tile = static_cast<ST*>(p.state) + (pad ? 0 : slot * p.state_slot) + static_cast<long long>(hv) * VD * KD;

  // First pass of state rows is requested before the prologue so the loads overlap it.
  float4 s[4][4];
  auto load_pass = [&](int pass) {
#pragma unroll
    for (int ri = 0; ri < 4; ++ri) {
      int row = warp * 32 + pass * 16 + grp * 4 + ri;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        s[ri][i] = pad ? make_float4(0.f, 0.f, 0.f, 0.f)
                       : load_state4<ST>(tile + static_cast<long long>(row) * KD + i * 32 + l8 * 4);
      }
    }
  };
  load_pass(0);

  // ---------------------------------------------------------------- prologue (whole CTA)
  constexpr int NV = 2 * T + T * (T - 1) / 2 + T * (T + 1) / 2;
  constexpr int NCH = (NV + 31) / 32;
  {
    float qd[T], kd[T];
#pragma unroll
    for (int t = 0; t < T; ++t) {
      bool on = t < p.tokens;
      qd[t] = on ? __bfloat162float(p.q[n * p.q_sn + t * p.q_st + h * KD + tid]) : 0.f;
      kd[t] = on ? __bfloat162float(p.k[n * p.k_sn + t * p.k_st + h * KD + tid]) : 0.f;
      sh.vv[t][tid] = on ? __bfloat162float(p.v[n * p.v_sn + t * p.v_st + hv * VD + tid]) : 0.f;
    }
    float pv[NCH * 32];
#pragma unroll
    for (int i = 0; i < NCH * 32; ++i) pv[i] = 0.f;
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
#pragma unroll
    for (int ch = 0; ch < NCH; ++ch) {
      float part[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) part[i] = pv[ch * 32 + i];
      reduce_scatter<32, 32>(part, lane);
      sh.red[warp][ch * 32 + lane] = part[0];
    }
    if (tid < T) {
      float x = __bfloat162float(p.a[n * p.a_sn + tid * p.a_st + hv]);
      float dtb = p.dt_bias_bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(p.dt_bias)[hv])
                                 : static_cast<const float*>(p.dt_bias)[hv];
      float bb = __bfloat162float(p.b[n * p.b_sn + tid * p.b_st + hv]);
      bool on = tid < p.tokens;
      float gg = on ? -expf(p.A_log[hv]) * softplus20(x + dtb) : 0.f;
      float be = on ? 1.f / (1.f + expf(-bb)) : 0.f;
      if (p.round_beta) be = __bfloat162float(__float2bfloat16(be));
      sh.g[tid] = gg;
      sh.beta[tid] = be;
    }
    __syncthreads();
    if (tid < NCH * 32) sh.tot[tid] = sh.red[0][tid] + sh.red[1][tid] + sh.red[2][tid] + sh.red[3][tid];
    __syncthreads();
    float rq[T], rk[T];
#pragma unroll
    for (int t = 0; t < T; ++t) {
      rq[t] = p.l2norm ? rsqrtf(sh.tot[t] + 1e-6f) * p.scale : p.scale;
      rk[t] = p.l2norm ? rsqrtf(sh.tot[T + t] + 1e-6f) : 1.f;
      sh.qn[t][tid] = qd[t] * rq[t];
      sh.kn[t][tid] = kd[t] * rk[t];
    }
    if (tid < T * T) {
      int i = tid / T, j = tid - i * T;
      float Gi = 0.f, Gj = 0.f;
      for (int t = 0; t < T; ++t) {
        Gi += t <= i ? sh.g[t] : 0.f;
        Gj += t <= j ? sh.g[t] : 0.f;
      }
      float dec = expf(Gj - Gi);
      if (i < j) sh.wkk[i][j] = dec * sh.tot[2 * T + j * (j - 1) / 2 + i] * rk[i] * rk[j];
      if (i <= j) sh.wkq[i][j] = dec * sh.tot[2 * T + T * (T - 1) / 2 + j * (j + 1) / 2 + i] * rk[i] * rq[j];
      if (i == j) sh.eG[i] = expf(Gi);
      if (j == 0) {  // commit coefficients for token i
        float Ga = 0.f;
        for (int t = 0; t < T; ++t) Ga += t < acc_n ? sh.g[t] : 0.f;
        sh.cC[i] = i < acc_n ? expf(Ga - Gi) : 0.f;
        if (i == 0) sh.cA = expf(Ga);
      }
    }
    __syncthreads();
  }

  // ---------------------------------------------------------------- two passes of 16 rows per warp
  const bool commit = acc_n > 0;
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
        float4 kv = *reinterpret_cast<const float4*>(&sh.kn[t][i * 32 + l8 * 4]);
        float4 qv = *reinterpret_cast<const float4*>(&sh.qn[t][i * 32 + l8 * 4]);
#pragma unroll
        for (int ri = 0; ri < 4; ++ri) {
          float4 sv = s[ri][i];
          dots[ri * 2 * T + t] += sv.x * kv.x + sv.y * kv.y + sv.z * kv.z + sv.w * kv.w;
          dots[ri * 2 * T + T + t] += sv.x * qv.x + sv.y * qv.y + sv.z * qv.z + sv.w * qv.w;
        }
      }
    }
    reduce_scatter<4 * 2 * T, 8>(dots, lane);
    // lane pair (l8 even: hk, l8 odd: hq) of row ri = l8 / 2
    const int my_ri = l8 >> 1;
    const int my_row = warp * 32 + pass * 16 + grp * 4 + my_ri;
    float u[T];
    if ((l8 & 1) == 0) {
#pragma unroll
      for (int j = 0; j < T; ++j) {
        float r = sh.vv[j][my_row] - sh.eG[j] * dots[j];
#pragma unroll
        for (int i = 0; i < j; ++i) r -= sh.wkk[i][j] * u[i];
        u[j] = sh.beta[j] * r;
      }
    }
#pragma unroll
    for (int j = 0; j < T; ++j) u[j] = __shfl_sync(0xffffffffu, u[j], lane & ~1);
    if ((l8 & 1) == 0) {
#pragma unroll
      for (int j = 0; j < T; ++j) sh.ubuf[warp][grp * 4 + my_ri][j] = u[j];
    } else {
#pragma unroll
      for (int j = 0; j < T; ++j) {
        if (j < p.tokens) {
          float o = sh.eG[j] * dots[j];
#pragma unroll
          for (int i = 0; i <= j; ++i) o += sh.wkq[i][j] * u[i];
          long long oo = out_base + j * p.o_st + my_row;
          if (p.out_f32) static_cast<float*>(p.out)[oo] = o;
          else static_cast<__nv_bfloat16*>(p.out)[oo] = __float2bfloat16(o);
        }
      }
    }
    if (commit) {
      __syncwarp();
      const float cA = sh.cA;
      float cu[4][T];
#pragma unroll
      for (int ri = 0; ri < 4; ++ri)
#pragma unroll
        for (int j = 0; j < T; ++j) cu[ri][j] = sh.cC[j] * sh.ubuf[warp][grp * 4 + ri][j];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float4 kv[T];
#pragma unroll
        for (int t = 0; t < T; ++t) kv[t] = *reinterpret_cast<const float4*>(&sh.kn[t][i * 32 + l8 * 4]);
#pragma unroll
        for (int ri = 0; ri < 4; ++ri) {
          float4 sv = s[ri][i];
          sv.x *= cA;
          sv.y *= cA;
          sv.z *= cA;
          sv.w *= cA;
#pragma unroll
          for (int t = 0; t < T; ++t) {
            sv.x += cu[ri][t] * kv[t].x;
            sv.y += cu[ri][t] * kv[t].y;
            sv.z += cu[ri][t] * kv[t].z;
            sv.w += cu[ri][t] * kv[t].w;
          }
          int row = warp * 32 + pass * 16 + grp * 4 + ri;
          store_state4(tile + static_cast<long long>(row) * KD + i * 32 + l8 * 4, sv);
        }
      }
      __syncwarp();
    }
  }
}

}  // namespace gdn
}  // namespace ga

// C ABI of the library (declared in include/green_attention.h): argument validation, TMA descriptor
// encoding, kernel-instance selection and launches. Replaces the reference's tvm_ffi launchers
// (csrc/sm90/attn_decode_fp8/launcher.cu:34-214, csrc/sm90/gdn_recurrent/launcher.cu:18-177).
#include <cuda.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <cstdlib>
#include <mutex>
#include <vector>

#include "../../include/green_attention.h"
#include "attn_rows.cuh"
#include "kv_exchange.cuh"
#include "attn_tc.cuh"
#include "attn_wide.cuh"
#include "gdn_recurrent.cuh"
#include "gdn_verify.cuh"

namespace {

thread_local char g_err[512] = "";
thread_local int g_launches = 0;

int fail(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return 1;
}

#define GA_CUDA(expr)                                                                         \
  do {                                                                                        \
    cudaError_t e_ = (expr);                                                                  \
    if (e_ != cudaSuccess) return fail("%s failed: %s", #expr, cudaGetErrorString(e_));       \
  } while (0)

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

struct DeviceState {
  bool ready = false;
  int sm_count = 0;
};
std::mutex g_mu;
DeviceState g_dev[64];
EncodeTiledFn g_encode = nullptr;

struct MapKey {
  const void* base;
  long long s_page, s_tok, s_head;
  int pages, page, kvh, hd, box_tok;
  int all_heads;  // 1: dimensions listed as (dim, token, head, page) with a box of box_tok tokens x all heads
  bool operator==(const MapKey& o) const { return std::memcmp(this, &o, sizeof(MapKey)) == 0; }
};
struct MapEntry {
  MapKey key;
  CUtensorMap map;
};
std::vector<MapEntry> g_maps;  // small most-recently-used list; guarded by g_mu

// Descriptor of a paged pool [pages, page, kv_heads, head_dim] (bytes) for boxes of
// [1 page, box_tok tokens, 1 head, 128 bytes] with the 128-byte swizzle the kernels' ldmatrix addressing expects.
int get_map(const MapKey& key, CUtensorMap* out) {
  std::lock_guard<std::mutex> lock(g_mu);
  for (size_t i = 0; i < g_maps.size(); ++i) {
    if (g_maps[i].key == key) {
      *out = g_maps[i].map;
      return 0;
    }
  }
  if (!g_encode) return fail("ga_init() has not run");
  cuuint64_t dims[4] = {(cuuint64_t)key.hd, (cuuint64_t)key.kvh, (cuuint64_t)key.page, (cuuint64_t)key.pages};
  cuuint64_t strides[3] = {(cuuint64_t)key.s_head, (cuuint64_t)key.s_tok, (cuuint64_t)key.s_page};
  cuuint32_t box[4] = {128, 1, (cuuint32_t)key.box_tok, 1};
  if (key.all_heads) {
    // Token before head: the box then lands in shared memory head-major, each head's rows swizzled by token.
    dims[1] = (cuuint64_t)key.page, dims[2] = (cuuint64_t)key.kvh;
    strides[0] = (cuuint64_t)key.s_tok, strides[1] = (cuuint64_t)key.s_head;
    box[1] = (cuuint32_t)key.box_tok, box[2] = (cuuint32_t)key.kvh;
  }
  cuuint32_t estr[4] = {1, 1, 1, 1};
  MapEntry e;
  std::memset(&e, 0, sizeof(e));
  e.key = key;
  CUresult r = g_encode(&e.map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<void*>(key.base), dims, strides, box,
                        estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail("cuTensorMapEncodeTiled failed with code %d", (int)r);
  if (g_maps.size() >= 32) g_maps.erase(g_maps.begin());
  g_maps.push_back(e);
  *out = e.map;
  return 0;
}

using AttnKernel = void (*)(const ga::attn::AttnDev, const CUtensorMap, const CUtensorMap);

struct AttnInstance {
  AttnKernel fn;
  int threads, smem, rows, occ;
};

template <int HD, int MT, int WN, int NP, int MODE, bool HALF = false, int CAP = 24, int SUB = 1, int OCC = 1, int DS = 1>
AttnInstance make_instance() {
  using C = ga::attn::Cfg<HD, MT, WN, NP, CAP, SUB, DS>;
  return {ga::attn::attn_rows_kernel<HD, MT, WN, NP, MODE, HALF, CAP, SUB, OCC, DS>, C::THREADS, C::SMEM_BYTES, C::ROWS,
          OCC};
}

// Row capacity 8/16/32/64/128 per (request, kv head) for decode / verify; extend always uses 128 rows.
// Warps per SM are chosen against the register file (16K registers per SM sub-partition): up to 8 warps may
// use 255 registers each, up to 12 warps 168. The 8-row decode instance runs two CTAs per SM (3 consumer
// warps + 1 producer warp and a 6-stage ring each): two independent TMA streams per SM measured 9 % faster
// than one CTA with the same warps.
const AttnInstance* decode_instance(int hd, int rows) {
  static const AttnInstance t128[5] = {make_instance<128, 1, 3, 1, 0, true, 6, 1, 2>(), make_instance<128, 1, 4, 4, 0>(),
                                       make_instance<128, 2, 3, 2, 0>(), make_instance<128, 4, 1, 4, 0>(),
                                       make_instance<128, 8, 1, 4, 0>()};
  static const AttnInstance t256[5] = {make_instance<256, 1, 6, 2, 0, true>(), make_instance<256, 1, 4, 2, 0>(),
                                       make_instance<256, 2, 2, 2, 0>(), make_instance<256, 4, 1, 2, 0>(),
                                       make_instance<256, 8, 1, 2, 0>()};
  // 17..24 rows at head_dim 128 (e.g. 5 draft tokens x 4 heads per kv head) when the batch is too small for the
  // tcgen05 route: three warps with 8 rows each share every tile (transposed-PV path), two such sets alternate
  // over the tiles. Measured 529 us on the B=64 verify configuration against 590 us for the 32-row instance
  // (and 340 us for the tcgen05 kernel, which is why large batches go there).
  // head_dim 512 (four 128-byte slabs per head), at most 8 rows: three 64 KB stages fit, a pair of warps takes each
  // (both do the QK product of the same 8 rows, each accumulates 256 of the output dims: 64 accumulator registers
  // per thread instead of 128, which spilled). Anything with more rows at this head dim is rejected before it gets here.
  static const AttnInstance t512 = make_instance<512, 2, 3, 1, 0, true, 24, 1, 1, 2>();
  if (hd == 512) return &t512;
  static const AttnInstance r24 = make_instance<128, 3, 2, 2, 0, true>();
  if (hd == 128 && rows > 16 && rows <= 24) return &r24;
  int i = rows <= 8 ? 0 : rows <= 16 ? 1 : rows <= 32 ? 2 : rows <= 64 ? 3 : 4;
  return hd == 128 ? &t128[i] : &t256[i];
}
// The combine kernel of a head dim, after the main kernel with programmatic stream serialization or as a plain launch.
template <typename... Args>
cudaError_t launch_combine(int hd, bool pdl, dim3 grid, cudaStream_t st, Args... args);

const AttnInstance* extend_instance(int hd) {
  static const AttnInstance e128 = make_instance<128, 8, 1, 4, 1>();
  static const AttnInstance e256 = make_instance<256, 8, 1, 2, 1>();
  return hd == 128 ? &e128 : &e256;
}

// Launch with programmatic stream serialization: the kernel may be scheduled while its predecessor in the
// stream drains, and orders itself with griddepcontrol.wait (replaces the reference's PDL launch of its
// combine kernel, csrc/sm90/attn_decode_fp8/launcher.cu:115-128).
template <typename... KArgs, typename... Args>
cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
  cudaLaunchConfig_t cfg;
  std::memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

template <typename... Args>
cudaError_t launch_combine(int hd, bool pdl, dim3 grid, cudaStream_t st, Args... args) {
  auto go = [&](auto kernel) -> cudaError_t {
    if (pdl) return launch_pdl(kernel, grid, dim3(128), 0, st, args...);
    kernel<<<grid, 128, 0, st>>>(args...);
    return cudaGetLastError();
  };
  if (hd == 128) return go(ga::attn::attn_combine_kernel<128>);
  if (hd == 256) return go(ga::attn::attn_combine_kernel<256>);
  return go(ga::attn::attn_combine_kernel<512>);
}

template <int HD, bool REP>
AttnInstance make_tc_instance() {
  return {ga::attn::tc::attn_tc_kernel<HD, REP>, ga::attn::tc::TC_THREADS, ga::attn::tc::TcCfg<HD, REP>::SMEM_BYTES, 128, 1};
}
// tcgen05 extend kernel: 128 query rows per CTA, two softmax groups alternating over the key tiles.
const AttnInstance* extend_tc_instance(int hd) {
  static const AttnInstance e128 = make_tc_instance<128, false>();
  static const AttnInstance e256 = make_tc_instance<256, false>();
  return hd == 128 ? &e128 : &e256;
}
// The same kernel for speculative verify with at most 32 rows per kv head: the rows are replicated over the four
// lane quarters of the query tile so that all four schedulers share the softmax.
const AttnInstance* verify_tc_instance(int hd) {
  static const AttnInstance v128 = make_tc_instance<128, true>();
  static const AttnInstance v256 = make_tc_instance<256, true>();
  return hd == 128 ? &v128 : &v256;
}

// The tcgen05 kernel wants TMA-sized pages and 16-byte aligned q / out rows.
bool tc_aligned(const GaAttnParams* a, const ga::attn::AttnDev& d) {
  const uintptr_t qa = reinterpret_cast<uintptr_t>(a->q), oa = reinterpret_cast<uintptr_t>(a->out);
  const int qel = a->q_is_bf16 ? 8 : 16;
  return d.use_tma && qa % 16 == 0 && oa % 16 == 0 && a->q_stride_tok % qel == 0 && a->q_stride_head % qel == 0 &&
         a->o_stride_tok % 8 == 0 && a->o_stride_head % 8 == 0;
}

int set_smem(const AttnInstance& k) {
  GA_CUDA(cudaFuncSetAttribute(reinterpret_cast<const void*>(k.fn), cudaFuncAttributeMaxDynamicSharedMemorySize,
                               k.smem));
  return 0;
}

// Raises the dynamic shared memory limit of every kernel instance on the current device.
int set_all_smem_limits() {
  GA_CUDA(cudaFuncSetAttribute(reinterpret_cast<const void*>(ga::attn::attn_wide_kernel<ga::attn::WIDE_T>),
                               cudaFuncAttributeMaxDynamicSharedMemorySize, ga::attn::SMEM_OPTIN));
  GA_CUDA(cudaFuncSetAttribute(reinterpret_cast<const void*>(ga::attn::attn_wide_kernel<ga::attn::WIDE_T / 2>),
                               cudaFuncAttributeMaxDynamicSharedMemorySize, ga::attn::SMEM_OPTIN));
  if (set_smem(*decode_instance(512, 8))) return 1;
  for (int hd : {128, 256}) {
    for (int rows : {8, 16, 24, 32, 64, 128})
      if (set_smem(*decode_instance(hd, rows))) return 1;
    if (set_smem(*extend_instance(hd)) || set_smem(*extend_tc_instance(hd)) || set_smem(*verify_tc_instance(hd))) return 1;
  }
  return 0;
}

// Per-head gather of the split-KV kernel: gangs of kv_heads CTAs walk the same pages at the same time, one kv head
// each, which gives DRAM the contiguous run of a page that the all-heads boxes of attn_wide.cuh give it
// (GREEN_ATTN_NO_GANG=1: every CTA on its own (request, kv head) units). A few CTAs are dropped when kv_heads does
// not divide the grid. Both decode entry points apply the same rule, so they cut the work identically.
void gang_by_kv_head(const GaAttnParams* a, ga::attn::AttnDev* d, int* grid) {
  static const bool no_gang = [] { const char* e = std::getenv("GREEN_ATTN_NO_GANG"); return e && e[0] == '1'; }();
  // Only the 8-row head_dim 128 instance is bound by its gather; the others are bound by their consumer warps and
  // measured 1 - 2 % slower ganged (fewer CTAs), so they keep one CTA per (request, kv head) slice.
  const bool stream_bound = a->head_dim == 128 && a->max_seqlen_q * (a->q_heads / a->kv_heads) <= 8;
  d->gang = (!no_gang && stream_bound && a->kv_heads >= 2 && *grid / a->kv_heads >= 1 && a->k_stride_head < a->k_stride_tok) ? 1 : 0;
  if (d->gang) *grid = *grid / a->kv_heads * a->kv_heads;
}

// Rows of a (request, kv head) pair are spread over grid.z of the combine kernel when the call has too few pairs
// to fill the SMs (one long sequence: batch 1 x 8 kv heads would otherwise merge ~150 partials on 8 CTAs).
unsigned combine_z(long long pairs, int rows, int sm) {
  if (pairs >= 2LL * sm || rows <= 1) return 1;
  const long long want = (2LL * sm + pairs - 1) / pairs;
  return static_cast<unsigned>(want < rows ? want : rows);
}

constexpr size_t kWsHeader = 256;
size_t ws_prefix_bytes(int batch) { return ((static_cast<size_t>(batch) + 1) * 4 + 255) / 256 * 256; }
size_t ws_lse_bytes(int sm) { return static_cast<size_t>(2 * sm) * ga::attn::MAX_ROWS * 4; }
size_t ws_o_bytes(int sm) { return static_cast<size_t>(2 * sm) * ga::attn::MAX_ROWS * 256 * 4; }

int current_device(int* dev) {
  GA_CUDA(cudaGetDevice(dev));
  if (*dev < 0 || *dev >= 64) return fail("device index %d out of range", *dev);
  if (!g_dev[*dev].ready) return fail("ga_init(%d) has not run", *dev);
  return 0;
}

bool pow2(int x) { return x > 0 && (x & (x - 1)) == 0; }

// Shared validation + device-struct fill for decode and extend.
int fill_attn(const GaAttnParams* a, ga::attn::AttnDev* d, CUtensorMap* kmap, CUtensorMap* vmap) {
  if (!a) return fail("null params");
  if (a->head_dim != 128 && a->head_dim != 256 && a->head_dim != 512)
    return fail("head_dim %d: only 128, 256 and 512 are built", a->head_dim);
  if (a->kv_heads <= 0 || a->q_heads <= 0 || a->q_heads % a->kv_heads) return fail("q_heads %d / kv_heads %d", a->q_heads, a->kv_heads);
  if (a->head_dim == 512 && static_cast<long long>(a->max_seqlen_q) * (a->q_heads / a->kv_heads) > 8)
    return fail("head_dim 512: only decode with at most 8 rows per kv head is built (max_seqlen_q %d x GQA %d)",
                a->max_seqlen_q, a->q_heads / a->kv_heads);
  if (!pow2(a->page_size)) return fail("page_size %d is not a power of two", a->page_size);
  if (a->batch <= 0) return fail("batch %d", a->batch);
  if (!a->q || !a->k_cache || !a->v_cache || !a->page_table || !a->cache_seqlens || !a->cu_seqlens_q || !a->out)
    return fail("null tensor pointer");
  const long long kstr[6] = {a->k_stride_page, a->k_stride_tok, a->k_stride_head,
                             a->v_stride_page, a->v_stride_tok, a->v_stride_head};
  for (long long s : kstr)
    if (s % 16) return fail("k/v cache strides must be multiples of 16 bytes");
  if ((reinterpret_cast<uintptr_t>(a->k_cache) | reinterpret_cast<uintptr_t>(a->v_cache)) & 15)
    return fail("k/v cache base must be 16-byte aligned");
  const int qalign = a->q_is_bf16 ? 4 : 4;  // elements: 8-byte bf16 loads, 4-byte e4m3 loads
  if (a->q_stride_tok % qalign || a->q_stride_head % qalign ||
      reinterpret_cast<uintptr_t>(a->q) % (a->q_is_bf16 ? 8 : 4))
    return fail("q strides/base must allow %d-byte vector loads", a->q_is_bf16 ? 8 : 4);
  if (a->o_stride_tok % 4 || a->o_stride_head % 4 || reinterpret_cast<uintptr_t>(a->out) % (a->out_is_f32 ? 16 : 8))
    return fail("out strides/base must allow 4-element vector stores");

  std::memset(d, 0, sizeof(*d));
  d->q = static_cast<const uint8_t*>(a->q);
  d->q_bf16 = a->q_is_bf16;
  d->q_s0 = a->q_stride_tok;
  d->q_s1 = a->q_stride_head;
  d->k = static_cast<const uint8_t*>(a->k_cache);
  d->v = static_cast<const uint8_t*>(a->v_cache);
  d->k_s0 = a->k_stride_page, d->k_s1 = a->k_stride_tok, d->k_s2 = a->k_stride_head;
  d->v_s0 = a->v_stride_page, d->v_s1 = a->v_stride_tok, d->v_s2 = a->v_stride_head;
  d->page_shift = __builtin_ctz(a->page_size);
  d->page_mask = a->page_size - 1;
  d->num_pages = a->num_pages;
  d->kvh = a->kv_heads;
  d->gqa = a->q_heads / a->kv_heads;
  d->pt = a->page_table;
  d->pt_s0 = a->pt_stride_row;
  d->pt_s1 = a->pt_stride_col;
  d->pt_cols = a->pt_cols;
  d->seqlens = a->cache_seqlens;
  d->cu = a->cu_seqlens_q;
  d->kd = a->k_descale, d->kd_s0 = a->kd_stride_b, d->kd_s1 = a->kd_stride_h;
  d->vd = a->v_descale, d->vd_s0 = a->vd_stride_b, d->vd_s1 = a->vd_stride_h;
  d->out = a->out;
  d->out_f32 = a->out_is_f32;
  d->o_s0 = a->o_stride_tok, d->o_s1 = a->o_stride_head;
  d->lse = a->lse;
  d->total_q = a->total_q;
  d->batch = a->batch;
  d->window_left = a->window_left < 0 ? -1 : a->window_left;
  d->scale_log2 = a->softmax_scale * 1.4426950408889634f;
  // TMA boxes need a swizzle-aligned (1024-byte) destination: pages of >= 8 tokens. Smaller pages are
  // gathered row by row with 16-byte cp.async.
  d->use_tma = a->page_size >= 8;
  d->box_tok = a->page_size < ga::attn::TN ? a->page_size : ga::attn::TN;
  std::memset(kmap, 0, sizeof(*kmap));
  std::memset(vmap, 0, sizeof(*vmap));
  if (d->use_tma) {
    MapKey kk = {a->k_cache, a->k_stride_page, a->k_stride_tok, a->k_stride_head, a->num_pages, a->page_size,
                 a->kv_heads, a->head_dim, d->box_tok, 0};
    MapKey vk = {a->v_cache, a->v_stride_page, a->v_stride_tok, a->v_stride_head, a->num_pages, a->page_size,
                 a->kv_heads, a->head_dim, d->box_tok, 0};
    if (get_map(kk, kmap) || get_map(vk, vmap)) return 1;
  }
  return 0;
}

template <int T>
int launch_gdn(const ga::gdn::GdnDev& d, bool bf16_state, int blocks, cudaStream_t st) {
  if (bf16_state) ga::gdn::gdn_recurrent_kernel<T, __nv_bfloat16><<<blocks, ga::gdn::THREADS, 0, st>>>(d);
  else ga::gdn::gdn_recurrent_kernel<T, float><<<blocks, ga::gdn::THREADS, 0, st>>>(d);
  GA_CUDA(cudaGetLastError());
  return 0;
}

// One CTA per row; thread d owns output dims d, d + blockDim, ...; the parts are folded in index order by every
// thread, so the result does not depend on scheduling.
__global__ void merge_parts_kernel(const float* o_parts, const float* lse_parts, long long o_ps, long long l_ps,
                                   int parts, int rows, int hd, __nv_bfloat16* out, float* lse) {
  const int r = blockIdx.x;
  float mx = -INFINITY;
  for (int s = 0; s < parts; ++s) mx = fmaxf(mx, lse_parts[s * l_ps + r]);
  float den = 0.f;
  if (mx != -INFINITY)
    for (int s = 0; s < parts; ++s) den += expf(lse_parts[s * l_ps + r] - mx);
  for (int d = threadIdx.x; d < hd; d += blockDim.x) {
    float acc = 0.f;
    if (mx != -INFINITY)
      for (int s = 0; s < parts; ++s)
        acc += expf(lse_parts[s * l_ps + r] - mx) * o_parts[s * o_ps + static_cast<long long>(r) * hd + d];
    out[static_cast<long long>(r) * hd + d] = __float2bfloat16(den > 0.f ? acc / den : 0.f);
  }
  if (lse && threadIdx.x == 0) lse[r] = den > 0.f ? mx + logf(den) : -INFINITY;
}

// Body of ga_init with `device` current; the caller restores the previous device whatever this returns.
int init_current_device(int device) {
  cudaDeviceProp prop;
  GA_CUDA(cudaGetDeviceProperties(&prop, device));
  if (prop.major != 10)
    return fail("device %d is sm_%d%d; this library holds sm_100a code only", device, prop.major, prop.minor);
  if (!g_encode) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    GA_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
    if (qres != cudaDriverEntryPointSuccess || !fn) return fail("cuTensorMapEncodeTiled is not available");
    g_encode = reinterpret_cast<EncodeTiledFn>(fn);
  }
  if (set_all_smem_limits()) return 1;
  std::lock_guard<std::mutex> lock(g_mu);
  g_dev[device].sm_count = prop.multiProcessorCount;
  g_dev[device].ready = true;
  return 0;
}

}  // namespace

extern "C" {

int ga_abi_version(void) { return GA_ABI_VERSION; }
const char* ga_last_error(void) { return g_err; }
int ga_last_launch_count(void) { return g_launches; }

int ga_init(int device) {
  if (device < 0 || device >= 64) return fail("device index %d out of range", device);
  {
    std::lock_guard<std::mutex> lock(g_mu);
    if (g_dev[device].ready) return 0;
  }
  int prev = 0;
  GA_CUDA(cudaGetDevice(&prev));
  GA_CUDA(cudaSetDevice(device));
  const int rc = init_current_device(device);
  const cudaError_t back = cudaSetDevice(prev);  // also on the error paths: the caller's device stays current
  if (rc) return rc;
  if (back != cudaSuccess) return fail("cudaSetDevice(%d) failed: %s", prev, cudaGetErrorString(back));
  return 0;
}

int ga_sm_count(int device) {
  if (device < 0 || device >= 64 || !g_dev[device].ready) return -1;
  return g_dev[device].sm_count;
}

size_t ga_attn_workspace_bytes(int device, int max_batch) {
  int sm = (device >= 0 && device < 64 && g_dev[device].ready) ? g_dev[device].sm_count : 160;
  return kWsHeader + ws_prefix_bytes(max_batch) + ws_lse_bytes(sm) + ws_o_bytes(sm);
}

int ga_attn_decode(const GaAttnParams* a, void* stream) {
  int dev;
  if (current_device(&dev)) return 1;
  ga::attn::AttnDev d;
  CUtensorMap kmap, vmap;
  if (fill_attn(a, &d, &kmap, &vmap)) return 1;
  const int rows = a->max_seqlen_q * d.gqa;
  if (a->max_seqlen_q < 1 || rows > ga::attn::MAX_ROWS)
    return fail("max_seqlen_q %d x GQA %d exceeds %d rows", a->max_seqlen_q, d.gqa, ga::attn::MAX_ROWS);
  const int sm = g_dev[dev].sm_count;
  const size_t need = kWsHeader + ws_prefix_bytes(a->batch) + ws_lse_bytes(sm) + ws_o_bytes(sm);
  if (!a->workspace || a->workspace_bytes < need) return fail("workspace too small: %zu < %zu bytes", a->workspace_bytes, need);
  if (reinterpret_cast<uintptr_t>(a->workspace) % 256) return fail("workspace must be 256-byte aligned");
  uint8_t* ws = static_cast<uint8_t*>(a->workspace);
  d.status = reinterpret_cast<int*>(ws);
  d.prefix = reinterpret_cast<int*>(ws + kWsHeader);
  d.ws_lse = reinterpret_cast<float*>(ws + kWsHeader + ws_prefix_bytes(a->batch));
  d.ws_o = reinterpret_cast<float*>(ws + kWsHeader + ws_prefix_bytes(a->batch) + ws_lse_bytes(sm));
  d.max_q = a->max_seqlen_q;
  d.bq = 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // The persistent tcgen05 kernel in split mode: the same tile-stream split as the warp-level kernel (128-key tiles,
  // one CTA per SM, partials merged by the combine kernel), so it balances at any batch.
  // Rows per kv head from which a call takes the tcgen05 kernel. The warp-level MMA of e4m3 runs at the f16 rate
  // with conversions on top on this part, so wherever the tcgen05 kernel applies it wins although at most 32 of its
  // 128 rows are query rows (measured, B=64 x 8 192 tokens: head_dim 256 one token GQA 2 585 -> 357 us and GQA 6
  // 325 -> 200 us; head_dim 128 with 12 or 16 rows 338 -> 226 us). At head_dim 128 up to 8 rows stay on the stream-
  // bound kernels above / below (all-heads boxes, ganged per-head gather), which are at the copy bandwidth.
  static const int tc_min_rows_256 = [] { const char* e = std::getenv("GREEN_ATTN_TC_MIN_ROWS_256"); return e ? std::atoi(e) : 1; }();
  static const int tc_min_rows_128 = [] { const char* e = std::getenv("GREEN_ATTN_TC_MIN_ROWS_128"); return e ? std::atoi(e) : 9; }();
  if (rows >= (a->head_dim == 256 ? tc_min_rows_256 : tc_min_rows_128) && a->head_dim != 512 && !a->out_is_f32 && tc_aligned(a, d)) {
    const bool rep = rows <= 32;
    const AttnInstance* tk = rep ? verify_tc_instance(a->head_dim) : extend_tc_instance(a->head_dim);
    d.tc_mode = 0;
    d.rows_cap = rep ? 32 : ga::attn::MAX_ROWS;
    // GREEN_ATTN_GANG=1: gangs of kv_heads CTAs walk the same pages at the same time, one kv head each (see
    // TcWork). The gather streams a fifth faster that way, but this kernel is bound by its per-tile softmax chain,
    // not by the gather (measured: 257 us ganged on 144 SMs against 253 us on 148 for the B=64 verify shape), so
    // it is off unless asked for.
    static const bool gang_on = [] { const char* e = std::getenv("GREEN_ATTN_GANG"); return e && e[0] == '1'; }();
    d.gang = (gang_on && a->kv_heads >= 2 && a->kv_heads <= 16 && sm / a->kv_heads >= 1) ? 1 : 0;
    const int tgrid_x = d.gang ? sm / a->kv_heads * a->kv_heads : sm;
    tk->fn<<<tgrid_x, tk->threads, tk->smem, st>>>(d, kmap, vmap);
    GA_CUDA(cudaGetLastError());
    dim3 tgrid(a->batch, a->kv_heads, combine_z(a->batch * a->kv_heads, rows, sm));
    const int wide_mode = d.gang ? 2 : 0;
    GA_CUDA(launch_combine(a->head_dim, true, tgrid, st, d, tgrid_x, d.rows_cap, ga::attn::tc::TNK, wide_mode));
    g_launches = 2;
    return 0;
  }
  dim3 cgrid(a->batch, a->kv_heads, combine_z(a->batch * a->kv_heads, rows, sm));
  // The production decode shape (at most 8 rows per kv head, head_dim 128, 4..8 kv heads, pages of at least 16
  // tokens) gathers all kv heads of a token run per TMA box: contiguous 16 - 32 KB runs of a page stream about a
  // fifth faster than one head's 128-byte pieces. GREEN_ATTN_NO_WIDE=1 keeps such calls on the per-head kernel.
  static const bool no_wide = [] { const char* e = std::getenv("GREEN_ATTN_NO_WIDE"); return e && e[0] == '1'; }();
  if (!no_wide && rows <= 8 && a->head_dim == 128 && d.use_tma && a->page_size >= ga::attn::WIDE_T / 2 && a->kv_heads >= 4 &&
      a->kv_heads <= ga::attn::WIDE_HEADS) {
    const int wide_box = a->page_size >= ga::attn::WIDE_T ? ga::attn::WIDE_T : ga::attn::WIDE_T / 2;
    MapKey kk = {a->k_cache, a->k_stride_page, a->k_stride_tok, a->k_stride_head, a->num_pages, a->page_size,
                 a->kv_heads, a->head_dim, wide_box, 1};
    MapKey vk = {a->v_cache, a->v_stride_page, a->v_stride_tok, a->v_stride_head, a->num_pages, a->page_size,
                 a->kv_heads, a->head_dim, wide_box, 1};
    if (get_map(kk, &kmap) || get_map(vk, &vmap)) return 1;
    if (wide_box == ga::attn::WIDE_T)
      GA_CUDA(launch_pdl(ga::attn::attn_wide_kernel<ga::attn::WIDE_T>, dim3(sm), dim3(ga::attn::WIDE_THREADS),
                         static_cast<size_t>(ga::attn::wide_smem_bytes(a->kv_heads)), st, d, kmap, vmap));
    else
      GA_CUDA(launch_pdl(ga::attn::attn_wide_kernel<ga::attn::WIDE_T / 2>, dim3(sm), dim3(ga::attn::WIDE_THREADS),
                         static_cast<size_t>(ga::attn::wide_smem_bytes(a->kv_heads)), st, d, kmap, vmap));
    GA_CUDA(launch_pdl(ga::attn::attn_combine_kernel<128>, cgrid, dim3(128), 0, st, d, sm, ga::attn::WIDE_ROWS, ga::attn::WIDE_T, 1));
    g_launches = 2;
    return 0;
  }
  const AttnInstance* k = decode_instance(a->head_dim, rows);
  int grid = sm * k->occ;
  gang_by_kv_head(a, &d, &grid);
  const int wide_mode = d.gang ? 2 : 0;
  GA_CUDA(launch_pdl(k->fn, dim3(grid), dim3(k->threads), k->smem, st, d, kmap, vmap));
  GA_CUDA(launch_combine(a->head_dim, true, cgrid, st, d, grid, k->rows, ga::attn::TN, wide_mode));
  g_launches = 2;
  return 0;
}

// ---- decode without a caller-provided workspace -------------------------------------------------
// Scratch for ga_attn_decode_noalloc: lives in the library image, one copy per GPU that loads the
// library, held until the process exits. Sized for the limits below and nothing larger.
constexpr int kNoAllocMaxBatch = 1024;   // requests per call
constexpr int kNoAllocMaxSm = 160;       // CTAs of the persistent grid (one per SM)
constexpr int kNoAllocRows = 16;         // max_seqlen_q * (q_heads / kv_heads) per (request, kv head)
constexpr size_t kNoAllocPrefixBytes = ((kNoAllocMaxBatch + 1) * 4 + 255) / 256 * 256;
constexpr size_t kNoAllocLseBytes = static_cast<size_t>(2 * 2 * kNoAllocMaxSm) * kNoAllocRows * 4;  // up to 2 CTAs per SM
constexpr size_t kNoAllocOBytes = static_cast<size_t>(2 * kNoAllocMaxSm) * kNoAllocRows * 256 * 4;
constexpr size_t kNoAllocBytes = kWsHeader + kNoAllocPrefixBytes + kNoAllocLseBytes + kNoAllocOBytes;  // ~5.03 MiB
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocBytes];
// In host code `g_noalloc_scratch` is only a handle for the symbol; the address a kernel can use is
// looked up per device and cached here.
static unsigned char* g_noalloc_ptr[64] = {nullptr};

int ga_attn_decode_noalloc(const GaAttnParams* a, void* stream) {
  int dev;
  if (current_device(&dev)) return 1;
  ga::attn::AttnDev d;
  CUtensorMap kmap, vmap;
  if (fill_attn(a, &d, &kmap, &vmap)) return 1;
  const int rows = a->max_seqlen_q * d.gqa;
  const int sm = g_dev[dev].sm_count;
  if (a->max_seqlen_q < 1 || rows > kNoAllocRows)
    return fail("ga_attn_decode_noalloc: max_seqlen_q %d x GQA %d = %d rows exceeds the built-in scratch (%d rows); "
                "use ga_attn_decode with a workspace", a->max_seqlen_q, d.gqa, rows, kNoAllocRows);
  if (a->batch > kNoAllocMaxBatch)
    return fail("ga_attn_decode_noalloc: batch %d exceeds the built-in scratch (%d requests); use ga_attn_decode "
                "with a workspace", a->batch, kNoAllocMaxBatch);
  const AttnInstance* k = decode_instance(a->head_dim, rows);  // rows <= 16: a 16-row instance
  const int full_grid = sm * k->occ;  // the scratch is checked against the full grid; ganging can only drop CTAs
  int grid = full_grid;  // same grid and the same ganging as ga_attn_decode, so both entry points cut the work identically
  gang_by_kv_head(a, &d, &grid);
  if (sm > kNoAllocMaxSm || static_cast<size_t>(2 * full_grid) * kNoAllocRows * a->head_dim * 4 > kNoAllocOBytes ||
      static_cast<size_t>(2 * full_grid) * kNoAllocRows * 4 > kNoAllocLseBytes)
    return fail("ga_attn_decode_noalloc: a grid of %d CTAs on %d SMs exceeds the built-in scratch (%d SMs)", grid, sm,
                kNoAllocMaxSm);
  if (g_noalloc_ptr[dev] == nullptr) {
    // First call on this device (it is the current one): resolve the device address of the array.
    void* ptr = nullptr;
    GA_CUDA(cudaGetSymbolAddress(&ptr, g_noalloc_scratch));
    if (ptr == nullptr) return fail("ga_attn_decode_noalloc: no device address for the built-in scratch");
    g_noalloc_ptr[dev] = static_cast<unsigned char*>(ptr);
  }
  unsigned char* ws = g_noalloc_ptr[dev];
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // The array keeps whatever the previous call left. Only the status word has to start at zero; the
  // prefix table and the partial slots are rewritten by every call before they are read.
  GA_CUDA(cudaMemsetAsync(ws, 0, sizeof(int), st));
  d.status = reinterpret_cast<int*>(ws);
  d.prefix = reinterpret_cast<int*>(ws + kWsHeader);
  d.ws_lse = reinterpret_cast<float*>(ws + kWsHeader + kNoAllocPrefixBytes);
  d.ws_o = reinterpret_cast<float*>(ws + kWsHeader + kNoAllocPrefixBytes + kNoAllocLseBytes);
  d.max_q = a->max_seqlen_q;
  d.bq = 0;
  k->fn<<<grid, k->threads, k->smem, st>>>(d, kmap, vmap);
  GA_CUDA(cudaGetLastError());
  dim3 cgrid(a->batch, a->kv_heads);
  GA_CUDA(launch_combine(a->head_dim, false, cgrid, st, d, grid, k->rows, ga::attn::TN, d.gang ? 2 : 0));
  g_launches = 2;
  return 0;
}

int ga_attn_extend(const GaAttnParams* a, void* stream) {
  int dev;
  if (current_device(&dev)) return 1;
  ga::attn::AttnDev d;
  CUtensorMap kmap, vmap;
  if (fill_attn(a, &d, &kmap, &vmap)) return 1;
  if (d.gqa > ga::attn::MAX_ROWS) return fail("GQA %d exceeds %d rows", d.gqa, ga::attn::MAX_ROWS);
  if (a->out_is_f32) return fail("extend writes bf16 only");
  d.bq = ga::attn::MAX_ROWS / d.gqa;
  d.max_q = 1 << 30;
  if (!a->workspace || a->workspace_bytes < kWsHeader) return fail("workspace (status word) missing");
  d.status = static_cast<int*>(a->workspace);
  const long long blocks = a->total_q / d.bq + a->batch;
  if (blocks > 0x7fffffffLL) return fail("too many query blocks");
  if (a->total_q <= 0) {
    g_launches = 0;
    return 0;
  }
  // The tcgen05 kernel wants TMA-sized pages and 16-byte aligned q / out rows; anything else runs on the
  // warp-level MMA kernel. The tcgen05 kernel is persistent: one CTA per SM deals itself (block, kv head) items.
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (tc_aligned(a, d)) {
    const AttnInstance* k = extend_tc_instance(a->head_dim);
    d.tc_mode = 1;
    d.nblk = static_cast<int>(blocks);
    d.rows_cap = ga::attn::MAX_ROWS;
    const long long items = blocks * a->kv_heads;
    if (items > 0x7fffffffLL) return fail("too many (block, kv head) items");
    const int sm = g_dev[dev].sm_count;
    const unsigned grid = static_cast<unsigned>(items < sm ? items : sm);
    k->fn<<<grid, k->threads, k->smem, st>>>(d, kmap, vmap);
  } else {
    const AttnInstance* k = extend_instance(a->head_dim);
    dim3 grid(static_cast<unsigned>(blocks), a->kv_heads);
    k->fn<<<grid, k->threads, k->smem, st>>>(d, kmap, vmap);
  }
  GA_CUDA(cudaGetLastError());
  g_launches = 1;
  return 0;
}

int ga_attn_merge(const GaMergeParams* m, void* stream) {
  if (!m || !m->o_parts || !m->lse_parts || !m->out) return fail("null params");
  if (m->parts <= 0 || m->rows <= 0 || m->head_dim <= 0) return fail("bad merge shape");
  if (m->o_part_stride < 0 || m->lse_part_stride < 0) return fail("negative part stride");
  const long long o_ps = m->o_part_stride ? m->o_part_stride : static_cast<long long>(m->rows) * m->head_dim;
  const long long l_ps = m->lse_part_stride ? m->lse_part_stride : m->rows;
  merge_parts_kernel<<<m->rows, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      m->o_parts, m->lse_parts, o_ps, l_ps, m->parts, m->rows, m->head_dim, static_cast<__nv_bfloat16*>(m->out), m->lse);
  GA_CUDA(cudaGetLastError());
  g_launches = 1;
  return 0;
}

int ga_attn_exchange_merge(const GaExchangeParams* x, void* stream) {
  if (!x || !x->mine || !x->peer_bufs || !x->epoch || !x->out || !x->status) return fail("null params");
  if (x->world < 1 || x->world > ga::kvx::MAX_WORLD) return fail("world %d outside 1..%d", x->world, ga::kvx::MAX_WORLD);
  if (x->rank < 0 || x->rank >= x->world) return fail("rank %d outside the world of %d", x->rank, x->world);
  if (x->rows <= 0 || x->head_dim <= 0) return fail("bad merge shape");
  ga::kvx::ExchDev d;
  d.mine = x->mine;
  d.bufs = static_cast<uint2* const*>(x->peer_bufs);
  d.epoch = static_cast<unsigned*>(x->epoch);
  d.rank = x->rank, d.world = x->world, d.rows = x->rows, d.hd = x->head_dim;
  d.out = static_cast<__nv_bfloat16*>(x->out);
  d.lse = x->lse;
  d.status = x->status;
  d.max_polls = x->wait_polls ? x->wait_polls : (1u << 23);
  GA_CUDA(launch_pdl(ga::kvx::exchange_merge_kernel, dim3(x->rows), dim3(128), 0, static_cast<cudaStream_t>(stream), d));
  g_launches = 1;
  return 0;
}

int ga_gdn_recurrent(const GaGdnParams* g, void* stream) {
  int dev;
  if (current_device(&dev)) return 1;
  if (!g) return fail("null params");
  if (g->k_dim != ga::gdn::KD || g->v_dim != ga::gdn::VD) return fail("k_dim/v_dim must be 128");
  if (g->h <= 0 || g->hv <= 0 || g->hv % g->h) return fail("hv %d must be a multiple of h %d", g->hv, g->h);
  if (g->tokens < 1 || g->tokens > 8) return fail("tokens %d outside 1..8", g->tokens);
  if (g->batch <= 0) return fail("batch %d", g->batch);
  if (!g->q || !g->k || !g->v || !g->a || !g->b || !g->A_log || !g->dt_bias || !g->state || !g->cache_indices || !g->out)
    return fail("null tensor pointer");
  if (reinterpret_cast<uintptr_t>(g->state) % 16 || g->state_stride_slot % 4) return fail("state must be 16-byte aligned");
  ga::gdn::GdnDev d;
  std::memset(&d, 0, sizeof(d));
  d.q = static_cast<const __nv_bfloat16*>(g->q);
  d.k = static_cast<const __nv_bfloat16*>(g->k);
  d.v = static_cast<const __nv_bfloat16*>(g->v);
  d.q_sn = g->q_stride_seq, d.q_st = g->q_stride_tok;
  d.k_sn = g->k_stride_seq, d.k_st = g->k_stride_tok;
  d.v_sn = g->v_stride_seq, d.v_st = g->v_stride_tok;
  d.a = static_cast<const __nv_bfloat16*>(g->a);
  d.b = static_cast<const __nv_bfloat16*>(g->b);
  d.a_sn = g->a_stride_seq, d.a_st = g->a_stride_tok, d.b_sn = g->b_stride_seq, d.b_st = g->b_stride_tok;
  d.A_log = g->A_log;
  d.dt_bias = g->dt_bias;
  d.dt_bias_bf16 = g->dt_bias_is_bf16;
  d.state = g->state;
  d.state_slot = g->state_stride_slot;
  d.idx = g->cache_indices;
  d.idx_i64 = g->cache_indices_is_i64;
  d.accept = g->accept_lens;
  d.qsl = g->query_start_loc;
  d.out = g->out;
  d.out_f32 = g->out_is_f32;
  d.o_sn = g->o_stride_seq, d.o_st = g->o_stride_tok;
  d.batch = g->batch, d.tokens = g->tokens, d.h = g->h, d.hv = g->hv;
  d.l2norm = g->l2norm_qk, d.round_beta = g->round_beta_bf16, d.pad_reads_zero = g->pad_reads_zero;
  d.scale = g->scale;
  const long long blocks = static_cast<long long>(g->batch) * g->hv;
  if (blocks > 0x7fffffffLL) return fail("batch * hv too large");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool bf = g->state_is_bf16 != 0;
  int rc;
  if (g->tokens == 1) rc = launch_gdn<1>(d, bf, (int)blocks, st);
  else if (g->tokens == 2) rc = launch_gdn<2>(d, bf, (int)blocks, st);
  else if (g->tokens <= 4) rc = launch_gdn<4>(d, bf, (int)blocks, st);
  else rc = launch_gdn<8>(d, bf, (int)blocks, st);
  if (rc) return rc;
  g_launches = 1;
  return 0;
}

int ga_gdn_verify(const GaGdnVerifyParams* g, void* stream) {
  int dev;
  if (current_device(&dev)) return 1;
  if (!g) return fail("null params");
  if (g->k_dim != ga::gdn::KD || g->v_dim != ga::gdn::VD) return fail("k_dim/v_dim must be 128");
  if (g->h <= 0 || g->hv <= 0 || g->hv % g->h) return fail("hv %d must be a multiple of h %d", g->hv, g->h);
  if (g->ring_len != 16 && g->ring_len != 32) return fail("ring_len %d must be 16 or 32", g->ring_len);
  if (g->batch <= 0) return fail("batch %d", g->batch);
  if (!g->q || !g->k || !g->v || !g->a || !g->b || !g->A_log || !g->dt_bias || !g->checkpoint_state || !g->d_cache ||
      !g->rawv_cache || !g->k_cache || !g->rawk_cache || !g->g_cache || !g->ssm_state_indices || !g->replay_indices ||
      !g->query_start_loc || !g->write_pos || !g->cache_base || !g->is_flush || !g->out)
    return fail("null tensor pointer");
  if (reinterpret_cast<uintptr_t>(g->checkpoint_state) % 16 || g->state_stride_slot % 4)
    return fail("state must be 16-byte aligned");
  if (reinterpret_cast<uintptr_t>(g->k_cache) % 16 || g->k_stride_slot % 8)
    return fail("k_cache rows must be 16-byte aligned");
  ga::gdn::GdnVerifyDev d;
  std::memset(&d, 0, sizeof(d));
  d.q = static_cast<const __nv_bfloat16*>(g->q);
  d.k = static_cast<const __nv_bfloat16*>(g->k);
  d.v = static_cast<const __nv_bfloat16*>(g->v);
  d.a = static_cast<const __nv_bfloat16*>(g->a);
  d.b = static_cast<const __nv_bfloat16*>(g->b);
  d.q_ts = g->q_stride_tok, d.k_ts = g->k_stride_tok, d.v_ts = g->v_stride_tok;
  d.a_ts = g->a_stride_tok, d.b_ts = g->b_stride_tok;
  d.A_log = g->A_log;
  d.dt_bias = g->dt_bias;
  d.dt_bias_bf16 = g->dt_bias_is_bf16;
  d.state = g->checkpoint_state;
  d.state_bf16 = g->state_is_bf16;
  d.state_slot = g->state_stride_slot;
  d.d_cache = static_cast<__nv_bfloat16*>(g->d_cache);
  d.rawv_cache = static_cast<__nv_bfloat16*>(g->rawv_cache);
  d.k_cache = static_cast<__nv_bfloat16*>(g->k_cache);
  d.rawk_cache = static_cast<__nv_bfloat16*>(g->rawk_cache);
  d.g_cache = g->g_cache;
  d.d_ss = g->d_stride_slot, d.rawv_ss = g->rawv_stride_slot, d.k_ss = g->k_stride_slot;
  d.rawk_ss = g->rawk_stride_slot, d.g_ss = g->g_stride_slot;
  d.sidx = g->ssm_state_indices;
  d.sidx_i64 = g->state_indices_is_i64;
  d.ridx = g->replay_indices;
  d.ridx_i64 = g->replay_indices_is_i64;
  d.qsl = g->query_start_loc;
  d.write_pos = g->write_pos;
  d.cache_base = g->cache_base;
  d.is_flush = reinterpret_cast<const signed char*>(g->is_flush);
  d.out = static_cast<__nv_bfloat16*>(g->out);
  d.o_ts = g->o_stride_tok;
  d.batch = g->batch, d.h = g->h, d.hv = g->hv, d.L = g->ring_len;
  d.scale = g->scale;
  const long long blocks = static_cast<long long>(g->batch) * g->hv;
  if (blocks > 0x7fffffffLL) return fail("batch * hv too large");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // One CTA per (request, key head) when the value heads of a key head fit its shared memory (2 or 3 per key
  // head in the served models), else one per (request, value head).
  const int gsz = g->hv / g->h;
  const unsigned gblocks = static_cast<unsigned>(static_cast<long long>(g->batch) * g->h);
  const bool bf = g->state_is_bf16 != 0;
  if (gsz == 2) {
    if (bf) ga::gdn::gdn_verify_group_kernel<__nv_bfloat16, 2><<<gblocks, ga::gdn::THREADS, 0, st>>>(d);
    else ga::gdn::gdn_verify_group_kernel<float, 2><<<gblocks, ga::gdn::THREADS, 0, st>>>(d);
  } else if (gsz == 3) {
    if (bf) ga::gdn::gdn_verify_group_kernel<__nv_bfloat16, 3><<<gblocks, ga::gdn::THREADS, 0, st>>>(d);
    else ga::gdn::gdn_verify_group_kernel<float, 3><<<gblocks, ga::gdn::THREADS, 0, st>>>(d);
  } else {
    if (bf) ga::gdn::gdn_verify_kernel<__nv_bfloat16><<<static_cast<unsigned>(blocks), ga::gdn::THREADS, 0, st>>>(d);
    else ga::gdn::gdn_verify_kernel<float><<<static_cast<unsigned>(blocks), ga::gdn::THREADS, 0, st>>>(d);
  }
  GA_CUDA(cudaGetLastError());
  g_launches = 1;
  return 0;
}

int ga_fp8_tensor_peak(void* status_word, void* stream, float* tflops) {
  int dev;
  if (current_device(&dev)) return 1;
  if (!status_word || !tflops) return fail("null pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  static bool attr_set[64] = {false};
  if (!attr_set[dev]) {
    GA_CUDA(cudaFuncSetAttribute(reinterpret_cast<const void*>(ga::attn::tc::fp8_peak_kernel),
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, 49152));
    attr_set[dev] = true;
  }
  const int sm = g_dev[dev].sm_count, iters = 100000;
  cudaEvent_t e0, e1;
  GA_CUDA(cudaEventCreate(&e0));
  GA_CUDA(cudaEventCreate(&e1));
  ga::attn::tc::fp8_peak_kernel<<<sm, 128, 49152, st>>>(1000, static_cast<int*>(status_word));
  GA_CUDA(cudaEventRecord(e0, st));
  ga::attn::tc::fp8_peak_kernel<<<sm, 128, 49152, st>>>(iters, static_cast<int*>(status_word));
  GA_CUDA(cudaEventRecord(e1, st));
  GA_CUDA(cudaEventSynchronize(e1));
  float ms = 0.f;
  GA_CUDA(cudaEventElapsedTime(&ms, e0, e1));
  GA_CUDA(cudaEventDestroy(e0));
  GA_CUDA(cudaEventDestroy(e1));
  *tflops = static_cast<float>(2.0 * 128 * 256 * 32 * static_cast<double>(iters) * sm / (ms * 1e-3) / 1e12);
  g_launches = 2;
  return 0;
}

// The status word of `workspace`, or of the array ga_attn_decode_noalloc works on when `workspace` is NULL
// (NULL before that entry point's first call on the current device reads as an error).
static int status_word_address(const void* workspace, const int** word) {
  if (workspace) {
    *word = static_cast<const int*>(workspace);
    return 0;
  }
  int dev;
  if (current_device(&dev)) return 1;
  if (g_noalloc_ptr[dev] == nullptr) return fail("ga_attn_decode_noalloc has not run on device %d", dev);
  *word = reinterpret_cast<const int*>(g_noalloc_ptr[dev]);
  return 0;
}

int ga_attn_workspace_status(const void* workspace, void* stream, int* status) {
  if (!status) return fail("null pointer");
  const int* word;
  if (status_word_address(workspace, &word)) return 1;
  GA_CUDA(cudaMemcpyAsync(status, word, sizeof(int), cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream)));
  GA_CUDA(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
  return 0;
}

int ga_attn_workspace_clear_status(void* workspace, void* stream) {
  const int* word;
  if (status_word_address(workspace, &word)) return 1;
  GA_CUDA(cudaMemsetAsync(const_cast<int*>(word), 0, sizeof(int), static_cast<cudaStream_t>(stream)));
  return 0;
}

#ifdef GA_TC_TRACE
// Profiling builds only: copies the timeline the traced CTA of the tcgen05 kernel left behind to `host_dst`
// (TC_TRACE_ROLES x TC_TRACE_CAP int64 words) and clears it.
int ga_tc_trace_read(void* host_dst) {
  constexpr size_t n = sizeof(long long) * ga::attn::tc::TC_TRACE_ROLES * ga::attn::tc::TC_TRACE_CAP;
  GA_CUDA(cudaDeviceSynchronize());
  GA_CUDA(cudaMemcpyFromSymbol(host_dst, ga::attn::tc::g_tc_trace, n));
  void* dev = nullptr;
  GA_CUDA(cudaGetSymbolAddress(&dev, ga::attn::tc::g_tc_trace));
  GA_CUDA(cudaMemset(dev, 0, n));
  return 0;
}
#endif

}  // extern "C"

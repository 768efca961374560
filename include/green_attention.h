/* C ABI of the B200 (sm_100a) kernels behind the green_attention plugin interface.
 *
 * One shared library, plain pointers and sizes, no framework types. Every pointer is a DEVICE pointer
 * unless stated otherwise; the caller owns all memory (outputs, LSE, workspaces): the library allocates
 * and frees nothing on the device. Strides are in ELEMENTS of the tensor they describe. Functions return
 * 0 on success; on failure they return a non-zero code and ga_last_error() describes it (thread-local).
 * A call is asynchronous on `stream` (a cudaStream_t passed as void*) and performs no host
 * synchronisation, so it may be captured into a CUDA graph once ga_init() has run on the device.
 * Calls on one device that share a workspace must be ordered on one stream (the reference has the same
 * rule: green_attention/gdn_recurrent.py:65-69).
 *
 * Reference interfaces replaced (paths inside the reference project):
 *   ga_init            <- `init` export,             csrc/sm90/attn_decode_fp8/launcher.cu:34-49,212
 *   ga_attn_decode     <- `attn_decode` export,      csrc/sm90/attn_decode_fp8/launcher.cu:164-186,213
 *   ga_attn_extend     <- `attn_extend` export,      csrc/sm90/attn_decode_fp8/launcher.cu:190-208,214
 *   GaAttnParams       <- `Params`,                  csrc/sm90/attn_decode_fp8/kernel.cuh:88-116
 *   ga_gdn_recurrent   <- `gdn_decode` export,       csrc/sm90/gdn_recurrent/launcher.cu:69-112
 *                         (and the chained-token part of `gdn_verify`, launcher.cu:117-177)
 *   GaGdnParams        <- `DecodeParams`,            csrc/sm90/gdn_recurrent/kernel.cuh:155-173
 *   ga_gdn_verify      <- `gdn_verify` export,       csrc/sm90/gdn_recurrent/launcher.cu:117-177
 *   GaGdnVerifyParams  <- `VerifyParams`,            csrc/sm90/gdn_recurrent/verify.cuh:67-100
 *   the loader itself  <- green_attention/jit.py:139-183 (runtime nvcc build + tvm_ffi module)
 */
#ifndef GREEN_ATTENTION_H_
#define GREEN_ATTENTION_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define GA_ABI_VERSION 3

/* Paged FP8 attention call (decode, speculative verify, extend). Mirrors the keyword arguments the
 * reference's selectors accept (green_attention/attn_decode.py:152-258). */
typedef struct GaAttnParams {
  const void* q;            /* [total_q, q_heads, head_dim] e4m3 (1 B) or bf16 (2 B); last stride 1 */
  int32_t q_is_bf16;        /* bf16 queries are rounded to e4m3 in the kernel, like the reference */
  int64_t q_stride_tok, q_stride_head;
  const void* k_cache;      /* [num_pages, page_size, kv_heads, head_dim] e4m3; last stride 1 */
  const void* v_cache;
  int64_t k_stride_page, k_stride_tok, k_stride_head; /* multiples of 16, base 16-byte aligned */
  int64_t v_stride_page, v_stride_tok, v_stride_head;
  int32_t num_pages, page_size; /* page_size a power of two */
  int32_t q_heads, kv_heads, head_dim; /* head_dim 128 or 256; q_heads % kv_heads == 0 */
  const int32_t* page_table;    /* [batch, max_pages]; entries past ceil(len / page_size) are never read */
  int64_t pt_stride_row, pt_stride_col;
  int32_t pt_cols;              /* max_pages: entries per page-table row */
  const int32_t* cache_seqlens; /* [batch] keys per request, new tokens included */
  const int32_t* cu_seqlens_q;  /* [batch + 1] */
  const float* k_descale;       /* [batch | 1, kv_heads] or NULL (= 1); multiplies the logits */
  int64_t kd_stride_b, kd_stride_h; /* any strides, (0, 0) for an expanded scalar */
  const float* v_descale;       /* or NULL; multiplies the output */
  int64_t vd_stride_b, vd_stride_h;
  void* out;                /* [total_q, q_heads, head_dim] bf16, or fp32 when out_is_f32; last stride 1 */
  int32_t out_is_f32;       /* 1: fp32 output for the KV-range-sharded path (partials merged by ga_attn_merge) */
  int64_t o_stride_tok, o_stride_head;
  float* lse;               /* [q_heads, total_q] natural log, or NULL */
  int64_t total_q;
  int32_t batch;
  int32_t max_seqlen_q;     /* decode/verify: max_seqlen_q * (q_heads / kv_heads) <= 128 */
  int32_t window_left;      /* -1 none; W: query at position p sees keys [p - W, p] */
  float softmax_scale;
  void* workspace;          /* ga_attn_workspace_bytes() bytes, 256-byte aligned; unused by extend */
  size_t workspace_bytes;
} GaAttnParams;

/* LSE-weighted merge of per-shard partial results of one decode call (the cross-GPU step of a single
 * KV-range-sharded sequence). Math of the reference's combine kernel, kernel.cuh:665-749. */
typedef struct GaMergeParams {
  const float* o_parts;   /* [parts, rows, head_dim] normalised partial outputs (all parts in LOCAL memory) */
  const float* lse_parts; /* [parts, rows] natural-log LSE, -inf where a part saw no key */
  int64_t o_part_stride;  /* elements between consecutive parts of o_parts; 0 = dense (rows * head_dim) */
  int64_t lse_part_stride;/* elements between consecutive parts of lse_parts; 0 = dense (rows). With both set to
                             rows * (head_dim + 1) and lse_parts = o_parts + rows * head_dim the kernel reads an
                             all-gathered buffer of packed (O, LSE) partials where it landed */
  int32_t parts, rows, head_dim;
  void* out;              /* [rows, head_dim] bf16 */
  float* lse;             /* [rows] or NULL */
} GaMergeParams;

/* The same merge with the exchange of the partials inside the kernel, for one process per GPU: every rank stores
 * its packed partial ([rows * head_dim] O then [rows] natural-log LSE, fp32) into a slot of every peer's gather
 * buffer with peer stores, each float as an 8-byte (value, call number) pair, polls (bounded) its own buffer for the
 * peers' rows and merges. `peer_bufs` is a DEVICE array of `world` pointers: entry j is rank j's gather buffer as
 * mapped into this process (entry `rank` is the local one). A gather buffer holds 2 * world * rows * (head_dim + 1)
 * pairs (8 bytes each), `epoch` two 32-bit words; all zeroed once, on every rank, before the first call, and used by
 * no one else. Every rank must make the same sequence of calls. A wait that runs out (about `wait_polls` x 0.05 us
 * per value; 0 = 2^23) sets *status to 6 and the call still returns. `peer_flags` is not used (kept for layout).
 * No counterpart in the reference (single GPU only). */
typedef struct GaExchangeParams {
  const float* mine;
  const void* peer_bufs;
  const void* peer_flags;
  void* epoch;
  int32_t rank, world, rows, head_dim;
  void* out;              /* [rows, head_dim] bf16 */
  float* lse;             /* [rows] or NULL */
  int32_t* status;        /* device word, sticky */
  uint32_t wait_polls;
} GaExchangeParams;

/* Gated-DeltaNet recurrent update over `tokens` chained tokens per request with accepted-prefix commit.
 * tokens == 1 with accept_lens == NULL is the plain decode step. */
typedef struct GaGdnParams {
  const void* q;  /* bf16; element (n, t, h, :) at q + n*q_stride_seq + t*q_stride_tok + h*k_dim */
  const void* k;
  const void* v;  /* bf16; element (n, t, hv, :) at v + n*v_stride_seq + t*v_stride_tok + hv*v_dim */
  int64_t q_stride_seq, q_stride_tok, k_stride_seq, k_stride_tok, v_stride_seq, v_stride_tok;
  const void* a;  /* bf16 [.., HV]: element (n, t, hv) at a + n*ab_stride_seq + t*ab_stride_tok + hv */
  const void* b;
  int64_t a_stride_seq, a_stride_tok, b_stride_seq, b_stride_tok;
  const float* A_log;     /* [HV] fp32 */
  const void* dt_bias;    /* [HV] fp32 or bf16 */
  int32_t dt_bias_is_bf16;
  void* state;            /* [slots, HV, V, K], K contiguous, fp32 or bf16; updated in place */
  int32_t state_is_bf16;
  int64_t state_stride_slot;
  const void* cache_indices; /* [batch] int32 or int64; < 0 = PAD */
  int32_t cache_indices_is_i64;
  const int32_t* accept_lens; /* [batch] in 0..tokens, or NULL = commit all tokens */
  const int32_t* query_start_loc; /* [batch + 1] or NULL; when given (split decode form) a request whose
                                     length != tokens gets zero output and an untouched state */
  void* out;              /* bf16 or fp32; element (n, t, hv, :) at out + n*o_stride_seq + t*o_stride_tok + hv*v_dim */
  int32_t out_is_f32;
  int64_t o_stride_seq, o_stride_tok;
  int32_t batch, tokens;  /* tokens 1..8 */
  int32_t h, hv, k_dim, v_dim; /* k_dim == v_dim == 128; hv % h == 0 */
  int32_t l2norm_qk;      /* 1: q' = q/sqrt(sum q^2 + 1e-6)*scale, k' likewise (without scale) */
  int32_t round_beta_bf16;/* 1: beta rounded to bf16 (the packed decode form) */
  int32_t pad_reads_zero; /* 0: PAD row gives zero output (packed form); 1: computes from a zero state (split form) */
  float scale;
} GaGdnParams;

/* Replay-SSM speculative verify (docs/gdn-contract.md:75-132 of the reference): up to 4 chained tokens per
 * request against a read-only checkpoint state plus the ring of deltas committed since that checkpoint. Writes
 * `out` and, while the ring has room (write_pos + j < ring_len), the new delta / key / gate rows of the ring;
 * never the state, write_pos, cache_base or is_flush. A request whose state slot is < 0 gets zero output rows
 * and nothing else; one whose ring slot has is_flush != 0 is skipped entirely. */
typedef struct GaGdnVerifyParams {
  const void* q;  /* bf16 [T, H, K]: token t, head h at q + t*q_stride_tok + h*k_dim (T = sum of spec lens) */
  const void* k;
  const void* v;  /* bf16 [T, HV, V] */
  const void* a;  /* bf16 [T, HV] */
  const void* b;
  int64_t q_stride_tok, k_stride_tok, v_stride_tok, a_stride_tok, b_stride_tok; /* elements */
  const float* A_log;    /* [HV] fp32 */
  const void* dt_bias;   /* [HV] fp32 or bf16 */
  int32_t dt_bias_is_bf16;
  const void* checkpoint_state; /* [slots, HV, V, K], K contiguous, fp32 or bf16; read only */
  int32_t state_is_bf16;
  int64_t state_stride_slot;
  void* d_cache;         /* bf16 [ring, HV, L, V]: high part of the committed deltas (read: history; written: new) */
  void* rawv_cache;      /* bf16 [ring, HV, L, V]: residual of the new deltas (written only) */
  void* k_cache;         /* bf16 [ring, H, L, K]: high part of the normalised keys */
  void* rawk_cache;      /* bf16 [ring, H, L, K]: residual of the new keys (written only) */
  float* g_cache;        /* fp32 [ring, HV, L] */
  int64_t d_stride_slot, rawv_stride_slot, k_stride_slot, rawk_stride_slot, g_stride_slot; /* elements; dense within a slot */
  const void* ssm_state_indices; /* [batch] int32 or int64 checkpoint slot; < 0 = PAD */
  int32_t state_indices_is_i64;
  const void* replay_indices;    /* [batch] int32 or int64 ring slot */
  int32_t replay_indices_is_i64;
  const int32_t* query_start_loc; /* [batch + 1]; spec len of request n = qsl[n+1] - qsl[n] in 0..4 */
  const int32_t* write_pos;       /* [ring + 1] entries already in the ring of a slot */
  const int32_t* cache_base;      /* [ring + 1] physical position of entry 0 */
  const int8_t* is_flush;         /* [ring + 1] */
  void* out;             /* bf16 [T, HV, V]: token t at out + t*o_stride_tok */
  int64_t o_stride_tok;
  int32_t batch;
  int32_t h, hv, k_dim, v_dim;   /* k_dim == v_dim == 128; hv % h == 0 */
  int32_t ring_len;              /* L: 16 or 32 */
  float scale;
} GaGdnVerifyParams;

/* Once per process and device, before the first launch and before any graph capture: resolves the
 * driver entry point used to encode TMA descriptors and raises the dynamic shared memory limit of every
 * kernel instance. Idempotent. */
int ga_init(int device);

/* Bytes of scratch the split-KV decode path needs on `device` for calls of at most `max_batch` requests. */
size_t ga_attn_workspace_bytes(int device, int max_batch);

int ga_attn_decode(const GaAttnParams* p, void* stream);
int ga_attn_extend(const GaAttnParams* p, void* stream);

/* Decode / verify for hosts that cannot give the library a workspace. No counterpart in the reference
 * (there Python always allocates the split workspace: green_attention/attn_decode.py:109-115).
 *
 * Same call and same result as ga_attn_decode, but `workspace` / `workspace_bytes` are ignored: the split-KV
 * scratch is a fixed array inside the library image (about 5 MiB, resident on every GPU that loads the library
 * until the process exits). It is meant for callers that own no device allocator or may not use one where
 * they call from: an engine that handed all free HBM to its KV pool at start-up, a latency-critical loop that
 * bans allocation after warm-up, or a thin C / Go / Rust host that links this library and nothing else. The
 * function itself calls no cudaMalloc / cudaFree and no allocating library routine; inputs and outputs are
 * still the caller's.
 * Limits (larger calls are rejected with an error, use ga_attn_decode for them): batch <= 1024,
 * max_seqlen_q * (q_heads / kv_heads) <= 16 rows, at most 160 SMs.
 * The first call on each device looks up the device address of the array (that device must be current, as
 * for every call); make that first call before any stream capture. All calls on a device share the one
 * array and it keeps the previous call's contents (the status word is cleared on the stream at every call,
 * everything else is rewritten before it is read), so two calls that may overlap on the GPU (different
 * streams, or different host threads without ordering) race: serialise them. The status word of the last
 * call is read with ga_attn_workspace_status(NULL, stream, &status). */
int ga_attn_decode_noalloc(const GaAttnParams* p, void* stream);
int ga_attn_merge(const GaMergeParams* p, void* stream);
int ga_attn_exchange_merge(const GaExchangeParams* p, void* stream);
int ga_gdn_recurrent(const GaGdnParams* p, void* stream);
int ga_gdn_verify(const GaGdnVerifyParams* p, void* stream);

/* Number of kernels the last successful call on this thread launched (bench bookkeeping). */
int ga_last_launch_count(void);
/* Reads the status word a kernel leaves in a decode workspace (0 = fine; non-zero = a bounded wait ran
 * out, a page id was out of range, or a cache_seqlens entry exceeded what its page-table row can address).
 * The word is sticky: kernels only ever set it, so one read covers every call since the last clear.
 * `workspace` NULL reads the word of the array ga_attn_decode_noalloc works on (current device; that entry
 * point clears its word at the start of every call, so read it after the call you care about and before the
 * next one). Synchronises `stream`. No allocation. */
int ga_attn_workspace_status(const void* workspace, void* stream, int* status);
/* Sets the status word back to 0, ordered on `stream` (NULL workspace as above). No synchronisation. */
int ga_attn_workspace_clear_status(void* workspace, void* stream);

/* Measures the dense FP8 (e4m3) tensor-core issue rate of the current device with a loop of tcgen05 MMAs on
 * zeroed shared-memory operands (M 128, N 256, K 32 per instruction, every SM busy): the denominator the extend
 * kernel's tensor roofline is quoted against. `status_word` is any 4-byte device location that receives a
 * non-zero value if a bounded wait runs out (a decode workspace header will do). Synchronises `stream`.
 * No counterpart in the reference (its benches quote a data-sheet peak, bench/bench_attn_extend.py:104). */
int ga_fp8_tensor_peak(void* status_word, void* stream, float* tflops);

const char* ga_last_error(void);
int ga_abi_version(void);
int ga_sm_count(int device);

#ifdef __cplusplus
}
#endif
#endif /* GREEN_ATTENTION_H_ */

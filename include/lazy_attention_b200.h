/*
 * lazy_attention_b200 -- C ABI of the deferred-RoPE paged attention path for
 * NVIDIA B200 (sm_100a).
 *
 * Everything here is plain C: raw device pointers, sizes, strides in ELEMENTS
 * and enums as ints.  Every function returns 0 on success or a negative
 * LA_ERR_* code; the text of the last failure on the calling thread is
 * available from la_last_error().  No function throws, exits, traps the
 * device or keeps a pointer after it returns.  All work is enqueued on the
 * CUDA stream the caller passes (a cudaStream_t given as void*; NULL = the
 * legacy default stream); no call synchronises the device.
 *
 * The entry points stand in for the following pieces of the reference
 * (paths relative to the reference repository):
 *   la_prefill_fwd          lazy_attn/lazy/attention/ops/prefix_prefill.py:599-744
 *                           (context_attention_fwd -> _fwd_kernel :34-592) and
 *                           lazy_attn/lazy/attention/old_ops/prefix_prefill.py:410-555
 *   la_decode_fwd           lazy_attn/lazy/attention/ops/chunked_prefill_paged_decode.py:108-221
 *                           (kernel_paged_attention_2d_llama,
 *                           lazy_attn/lazy/attention/ops/models/llama_v1.py:18-434) and
 *                           lazy_attn/lazy/attention/old_ops/chunked_prefill_paged_decode.py:23-280
 *   la_pack_block_table     lazy_attn/lazy/worker/gpu_model_runner.py:296-343
 *   la_build_cos_sin_table  lazy_attn/lazy/model_executor/rope/cos_sin.py:24-66,127-148
 *                           (the table vLLM's rotary layer hands the kernels)
 */
#ifndef LAZY_ATTENTION_B200_H_
#define LAZY_ATTENTION_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LA_VERSION 101

/* error codes */
#define LA_OK 0
#define LA_ERR_INVALID_ARGUMENT (-1) /* ValueError / assert in the reference   */
#define LA_ERR_UNSUPPORTED (-2)      /* NotImplementedError in the reference   */
#define LA_ERR_CUDA (-3)             /* a CUDA runtime/driver call failed      */
#define LA_ERR_WORKSPACE (-4)        /* workspace missing or too small         */
#define LA_ERR_DEVICE_STATUS (-5)    /* a kernel reported a bounded-wait expiry */

/* element types */
#define LA_DTYPE_F32 0
#define LA_DTYPE_F16 1
#define LA_DTYPE_BF16 2
#define LA_DTYPE_FP8_E4M3 3
#define LA_DTYPE_FP8_E5M2 4

/* rotation modes */
#define LA_ROT_LAZY 0  /* one rotation offset per cached page (reference variant "lazy")  */
#define LA_ROT_MEPIC 1 /* one rotation per cached token (reference variant "mepic")       */

/* kernel selection (diagnostics and tests; 0 is what production uses) */
#define LA_KERNEL_AUTO 0
#define LA_KERNEL_GENERAL 1 /* SIMT kernel: every dtype, layout and option            */
#define LA_KERNEL_TENSOR 2  /* TMA + tcgen05 prefill / bulk-copy + mma decode kernels */

/*
 * Output gather fused into the kernel's epilogue (multi-GPU only; no counterpart
 * in the reference, whose tensor-parallel ranks call the op on their own heads and
 * gather with a collective afterwards).  When num_peers > 0 the tensor-core prefill
 * kernel and the split-KV decode kernel write every result row straight into the
 * full-size output buffers of all ranks (plain stores over NVLink to peer-mapped
 * memory, this rank's own buffer included) instead of args->out; the caller then
 * only needs a barrier across the ranks.  The general kernel does not support it.
 */
#define LA_MAX_PEERS 8
typedef struct LaPeerOut {
  void* out[LA_MAX_PEERS]; /* the ranks' output buffers [rows, heads, head_dim], same dtype as out */
  int32_t num_peers;       /* 0: disabled */
  int32_t head_offset;     /* index of this rank's first head in the peers' buffers */
  int64_t stride_t, stride_h; /* element strides of the peers' buffers */
  const int32_t* rows;     /* device: row in the peers' buffers of each local output row; NULL = same row */
} LaPeerOut;

/*
 * Prefix-prefill attention over a batch of requests.
 *
 * Replaces context_attention_fwd(q, k, v, o, kv_cache_dtype, k_cache, v_cache,
 * b_loc, b_start_loc, b_seq_len, max_seq_len, max_input_len, k_scale, v_scale,
 * alibi_slopes, sliding_window, sm_scale, skip_decode, cos_sin_cache,
 * rotary_dim, is_neox_style, is_lazy, q_offset, q_mask)
 * (lazy_attn/lazy/attention/ops/prefix_prefill.py:600-625) and its per-token
 * twin (lazy_attn/lazy/attention/old_ops/prefix_prefill.py:411-435).
 */
typedef struct LaPrefillArgs {
  /* activations, [num_tokens, heads, head_dim], last dim contiguous */
  const void* q;
  const void* k;
  const void* v;
  void* out;
  int64_t q_stride_t, q_stride_h;
  int64_t k_stride_t, k_stride_h;
  int64_t v_stride_t, v_stride_h;
  int64_t o_stride_t, o_stride_h;
  /* paged caches: K [nb, Hkv, D/x, BS, x], V [nb, Hkv, D, BS]; the three
   * (two) innermost dims must be contiguous */
  const void* k_cache;
  const void* v_cache;
  int64_t kc_stride_block, kc_stride_head;
  int64_t vc_stride_block, vc_stride_head;
  int64_t num_blocks; /* pages in the caches (dim 0); bounds the page ids */
  /* per-request tables, all int32 [batch, >= pages] sharing one row stride */
  const int32_t* block_table;
  const int32_t* q_offset; /* may be NULL when no request is lazy */
  const int32_t* q_mask;   /* may be NULL when no request is lazy */
  int64_t table_stride;
  const int32_t* query_start_loc; /* [batch + 1] */
  const int32_t* seq_lens;        /* [batch]     */
  const uint8_t* is_lazy;         /* [batch] bool; NULL = none lazy (LA_ROT_LAZY only) */
  const float* k_scale;           /* 1 element, device */
  const float* v_scale;           /* 1 element, device */
  const void* cos_sin_cache;      /* [max_position, rotary_dim]: cos half | sin half */
  int64_t cos_sin_rows;           /* rows of cos_sin_cache (bounds for index checks) */
  int32_t cos_sin_dtype;          /* LA_DTYPE_F32 / F16 / BF16 */
  int32_t batch;
  int32_t num_q_heads, num_kv_heads, head_dim;
  int32_t block_size, x;
  int32_t max_query_len; /* the reference's max_input_len */
  int32_t max_seq_len;   /* upper bound of seq_lens (host-side planning only) */
  int32_t q_dtype;       /* dtype of q, k, v, out */
  int32_t kv_dtype;      /* dtype of the caches */
  int32_t rotary_dim;    /* must equal head_dim */
  int32_t sliding_window; /* <= 0: disabled */
  int32_t skip_decode;    /* leave requests with one query token untouched */
  int32_t rot_mode;       /* LA_ROT_* */
  int32_t is_mepic;       /* LA_ROT_MEPIC only: 1 = rotate at the absolute slot */
  float sm_scale;
  int32_t kernel;         /* LA_KERNEL_* */
  void* workspace;        /* split-KV scratch, see la_prefill_workspace_bytes */
  size_t workspace_bytes;
  LaPeerOut peer;         /* optional fused output gather */
  /* Optional packed table, int64 [batch, >= pages]: block << 32 | q_offset << 16 | q_mask
   * (what la_pack_block_table writes and the decode kernel reads,
   * lazy_attn/lazy/worker/gpu_model_runner.py:322-330).  When non-NULL the kernels take a
   * page's block id, rotation offset and pad count from this one 8-byte entry instead of
   * three gathers from block_table / q_offset / q_mask (which may then be NULL); the
   * reference's prefill kernel always does the three gathers
   * (lazy_attn/lazy/attention/ops/prefix_prefill.py:171,180-185,267-268). */
  const int64_t* packed_block_table;
  int64_t packed_stride;
  /* Optional fused cache write, int64 [num_tokens]: when non-NULL the call also stores the
   * new K/V rows of its requests into the paged caches at these slots (negative = skip),
   * exactly as la_write_paged_cache does -- the step that precedes the attention op in
   * lazy_attn/lazy/attention/backends/triton_attn.py:100-109 -- so that the separate launch
   * can be dropped.  The caches are written through k_cache / v_cache although the struct
   * declares them const.  Requests the call skips (skip_decode) are not written. */
  const int64_t* slot_mapping;
  /* Optional fused rotary op, int64 [num_tokens]: when non-NULL, q arrives WITHOUT rotary
   * embedding and the kernel applies it (NeoX halves, row q_positions[t] of cos_sin_cache,
   * result rounded to q's dtype) while it stages the query -- what the query-only rotary op
   * does in place just before the attention op
   * (lazy_attn/lazy/model_executor/layers/rotary_embedding.py:66-94).  q itself is not
   * modified.  Tensor-core kernel only (LA_ERR_UNSUPPORTED otherwise). */
  const int64_t* q_positions;
} LaPrefillArgs;

/*
 * Paged decode attention: one query token per sequence; sequences whose query
 * length is not 1 are skipped.
 *
 * Replaces the decode launch of chunked_prefill_paged_decode
 * (lazy_attn/lazy/attention/ops/chunked_prefill_paged_decode.py:108-221) and
 * of its per-token twin
 * (lazy_attn/lazy/attention/old_ops/chunked_prefill_paged_decode.py:353-442).
 */
typedef struct LaDecodeArgs {
  const void* q;  /* [num_tokens(+1), Hq, D] */
  void* out;      /* [num_tokens, Hq, D]     */
  int64_t q_stride_t, q_stride_h;
  int64_t o_stride_t, o_stride_h;
  const void* k_cache;
  const void* v_cache;
  int64_t kc_stride_block, kc_stride_head;
  int64_t vc_stride_block, vc_stride_head;
  int64_t num_blocks;
  /* LA_ROT_LAZY: packed int64 [num_seqs, >= pages] =
   *   block << 32 | q_offset << 16 | q_mask.
   * LA_ROT_MEPIC: NULL */
  const int64_t* packed_block_table;
  int64_t packed_stride;
  /* LA_ROT_MEPIC: plain int32 tables; LA_ROT_LAZY: NULL */
  const int32_t* block_table;
  const int32_t* q_mask;
  int64_t table_stride;
  const int32_t* query_start_loc; /* [num_seqs + 1] */
  const int32_t* seq_lens;        /* [num_seqs]     */
  const uint8_t* is_lazy;         /* [num_seqs] bool, LA_ROT_LAZY only; NULL = none */
  const float* alibi_slopes;      /* [Hq] or NULL */
  const float* k_scale;
  const float* v_scale;
  const void* cos_sin_cache;
  int64_t cos_sin_rows;
  int32_t cos_sin_dtype;
  int32_t num_seqs;
  int32_t num_q_heads, num_kv_heads, head_dim;
  int32_t block_size, x;
  int32_t max_seq_len;
  int32_t q_dtype;
  int32_t kv_dtype;
  int32_t rotary_dim;
  int32_t sliding_window;
  int32_t rot_mode;
  int32_t ignore_q_mask; /* the reference's IGNORE_Q_MASK switch */
  float sm_scale;
  int32_t kernel;
  void* workspace; /* split-KV scratch, see la_decode_workspace_bytes */
  size_t workspace_bytes;
  LaPeerOut peer;  /* optional fused output gather */
  /* Optional fused cache write for the decode rows: key / value [num_tokens, Hkv, D] of the
   * step and slot_mapping int64 [num_tokens].  When slot_mapping is non-NULL the kernel
   * stores each sequence's new K/V row into the caches (as la_write_paged_cache would have
   * before the call: a negative slot is skipped) and attends to what the page then holds;
   * seq_lens counts the new token, as in the reference. */
  const void* key;
  const void* value;
  int64_t k_stride_t, k_stride_h, v_stride_t, v_stride_h;
  const int64_t* slot_mapping;
  /* Optional fused rotary op for the decode rows (see LaPrefillArgs.q_positions).
   * Split-KV kernel only. */
  const int64_t* q_positions;
  /* Optional in-kernel cos/sin: with compute_cos_sin != 0 the rotation of the query by a
   * page's offset takes cos/sin(position * inv_freq) computed in the kernel from these
   * parameters instead of a row of cos_sin_cache (which may then be NULL unless q_positions
   * is given) -- the reference's COMPUTE_COS_SIN path with the frequencies of
   * lazy_attn/lazy/model_executor/rope/cos_sin.py:24-66; parameters as rope_meta_from_layer
   * (:94-124) returns them.  rope_type: 0 = plain, 1 = llama3 smoothing.  Split-KV kernel,
   * LA_ROT_LAZY only. */
  int32_t compute_cos_sin;
  int32_t rope_type;
  float rope_base, rope_scaling_factor, rope_low_freq_factor, rope_high_freq_factor;
  int32_t rope_orig_max_position;
  int32_t reserved0;
} LaDecodeArgs;

/* Replaces context_attention_fwd / _fwd_kernel (see LaPrefillArgs). */
int la_prefill_fwd(const LaPrefillArgs* args, void* stream);

/* Replaces the decode kernel launch (see LaDecodeArgs). */
int la_decode_fwd(const LaDecodeArgs* args, void* stream);

/*
 * la_prefill_fwd for callers that must not allocate device memory.  It has no
 * counterpart in the reference (the reference's kernels never split the KV range,
 * so they need no scratch at all).
 *
 * Who needs it: an integration that has handed every free byte of HBM to the
 * paged KV cache, or that runs the layer where cudaMalloc / cudaFree (and the
 * device-wide synchronisation they imply) are forbidden, cannot give the
 * split-KV kernel a workspace.  This entry point takes the same arguments
 * (args->workspace and args->workspace_bytes are ignored) and keeps the partial
 * results in a 32 MiB array that is part of the library image, so it calls no
 * cudaMalloc, cudaFree or other allocating routine.
 *
 * Limits and rules:
 *  - only calls the tensor-core prefill kernel accepts (LA_ERR_UNSUPPORTED
 *    otherwise) and whose la_prefill_workspace_bytes() is at most 32 MiB
 *    (LA_ERR_WORKSPACE otherwise, with both sizes in la_last_error());
 *  - the array costs 32 MiB on every GPU that loads the library, for the life of
 *    the process;
 *  - the first call on each device looks up the array's device address
 *    (cudaGetSymbolAddress) and sets kernel attributes; make that first call
 *    before any stream capture;
 *  - all calls share the one array per device: two calls that overlap on the GPU
 *    (different streams) race on it.  Calls on one stream are safe.  The array
 *    keeps the previous call's contents; nothing in it needs clearing because
 *    every entry a call reads is written earlier in that same call.
 */
int la_prefill_fwd_noalloc(const LaPrefillArgs* args, void* stream);

/* Bytes of split-KV scratch la_prefill_fwd / la_decode_fwd need for these
 * arguments (0 when the selected kernel needs none).  Only the shape fields
 * are read.  The reference allocates nothing of the kind: its kernels do not
 * split the KV range (lazy_attn/lazy/attention/ops/chunked_prefill_paged_decode.py:171-174). */
size_t la_prefill_workspace_bytes(const LaPrefillArgs* args);
size_t la_decode_workspace_bytes(const LaDecodeArgs* args);

/*
 * packed[r, c] = (int64)block_table[r, c] << 32 | (int64)q_offset[r, c] << 16
 *              | (int64)q_mask[r, c]
 * for the rows listed in `rows` (n_rows of them) or, when rows == NULL, for
 * rows 0 .. n_rows-1.  Replaces the full and the row-wise rebuild of
 * LazyGPUModelRunner._rebuild_packed_block_table
 * (lazy_attn/lazy/worker/gpu_model_runner.py:322-339).  No range check is
 * applied here: like the reference, the caller refuses q_offset > 0xFFFF
 * before packing (:217-225).
 */
int la_pack_block_table(const int32_t* block_table, const int32_t* q_offset,
                        const int32_t* q_mask, int64_t* packed,
                        const int32_t* rows, int32_t n_rows, int32_t n_cols,
                        int64_t in_stride, int64_t packed_stride, void* stream);

/*
 * out[pos, 0:rd/2] = cos(pos * inv_freq), out[pos, rd/2:rd] = sin(pos * inv_freq)
 * with inv_freq[i] = base^(-2i/rd), optionally with llama3 frequency smoothing
 * (rope_type 1).  Replaces the table vLLM's rotary layer builds and the
 * reference mirrors in lazy_attn/lazy/model_executor/rope/cos_sin.py:24-66,127-148.
 */
int la_build_cos_sin_table(void* out, int32_t out_dtype, int64_t max_position,
                           int32_t rotary_dim, double base, int32_t rope_type,
                           double scaling_factor, double low_freq_factor,
                           double high_freq_factor, int64_t orig_max_position,
                           void* stream);

/*
 * Scatter of the step's new K/V rows into the paged caches by slot:
 *   k_cache[slot / BS, h, d / x, slot % BS, d % x] = key[t, h, d]
 *   v_cache[slot / BS, h, d, slot % BS]            = value[t, h, d]
 * with slot = slot_mapping[t] (negative = skip); an fp8 cache stores
 * fp8(value / scale), saturating.  Stands in for the call
 * PagedAttention.write_to_paged_cache(key, value, key_cache, value_cache,
 * slot_mapping, kv_cache_dtype, k_scale, v_scale) that precedes the attention op
 * in lazy_attn/lazy/attention/backends/triton_attn.py:100-109 (the callee is vLLM
 * 0.9.2's reshape_and_cache, not part of the reference's own sources).
 */
typedef struct LaWriteCacheArgs {
  const void* key;   /* [num_tokens, Hkv, D] */
  const void* value; /* [num_tokens, Hkv, D] */
  void* k_cache;     /* [nb, Hkv, D/x, BS, x] */
  void* v_cache;     /* [nb, Hkv, D, BS]      */
  const int64_t* slot_mapping; /* [num_tokens] */
  const float* k_scale;        /* 1 element, device (fp8 caches only) */
  const float* v_scale;
  int64_t k_stride_t, k_stride_h, v_stride_t, v_stride_h;
  int64_t kc_stride_block, kc_stride_head, vc_stride_block, vc_stride_head;
  int64_t num_tokens;
  int32_t num_kv_heads, head_dim, block_size, x;
  int32_t dtype;    /* of key / value */
  int32_t kv_dtype; /* of the caches  */
} LaWriteCacheArgs;

int la_write_paged_cache(const LaWriteCacheArgs* args, void* stream);

/*
 * Buffers for the fused output gather (LaPeerOut), shared between the processes of one node
 * with CUDA IPC.  No counterpart in the reference (its ranks gather with a collective).
 *   la_peer_alloc   cudaMalloc of `bytes` on the current device, zero-filled
 *   la_peer_export  the 64-byte CUDA IPC handle of a buffer from la_peer_alloc
 *   la_peer_open    maps another process's buffer into this process for the CURRENT device
 *                   (the device whose kernels will store through the mapping)
 *   la_peer_close   unmaps a pointer from la_peer_open
 *   la_peer_free    frees a buffer from la_peer_alloc (after every peer has closed it)
 *   la_peer_barrier one small kernel on `stream` that ends the step of a fused gather: it tells
 *                   every rank "my kernels before this point have finished, their stores into your
 *                   buffer have landed" and returns once every rank has said so.  `signals[r]` is
 *                   rank r's signal buffer (LA_PEER_SIGNAL_BYTES from la_peer_alloc, own or
 *                   mapped with la_peer_open; never written by anything else).  Every rank must
 *                   call it the same number of times (the round counter lives in the buffer, so a
 *                   captured launch can be replayed).  One process per GPU: ranks that share a GPU
 *                   must not use it (their kernels would wait on one another on one device).  The
 *                   wait is bounded (about 10 s of GPU clock; LAZY_ATTN_B200_BARRIER_LIMIT_MS in the
 *                   environment overrides it); a rank that never arrives leaves the code 300 + its
 *                   number for la_device_status() / la_check_device() and the kernel returns.
 */
#define LA_IPC_HANDLE_BYTES 64
#define LA_PEER_SIGNAL_BYTES 256
int la_peer_alloc(size_t bytes, void** out);
int la_peer_export(const void* buffer, unsigned char handle[LA_IPC_HANDLE_BYTES]);
int la_peer_open(const unsigned char handle[LA_IPC_HANDLE_BYTES], void** out);
int la_peer_close(void* mapped);
int la_peer_free(void* buffer);
int la_peer_barrier(void* const* signals, int32_t world, int32_t rank, void* stream);

/* Text of the last error on this thread ("" if none). */
const char* la_last_error(void);

/* LA_VERSION of the loaded library. */
int la_version(void);

/* Number of kernels this library has launched in this process so far. */
int64_t la_launch_count(void);

/* Kernels with bounded waits record a non-zero code in a device status word
 * when a wait expires.  This call synchronises the device, returns that code
 * (0 = none) and clears it.  A negative value is an LA_ERR_* of the call itself. */
int la_device_status(void);

/* The same check as a status: synchronises the device and returns LA_OK, or
 * LA_ERR_DEVICE_STATUS with the code in la_last_error() (the word is cleared).  The kernels
 * never report through the calls that launched them (those do not synchronise): an
 * integration polls one of these two, e.g. once per engine step. */
int la_check_device(void);

/* sizeof(LaPrefillArgs) / sizeof(LaDecodeArgs) as compiled into the library, so
 * that a foreign-function binding can verify its mirror of the structs. */
size_t la_sizeof_prefill_args(void);
size_t la_sizeof_decode_args(void);

#ifdef __cplusplus
}
#endif
#endif /* LAZY_ATTENTION_B200_H_ */

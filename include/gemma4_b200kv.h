/*
 * C ABI of libgemma4_b200kv.so: the B200 (sm_100a) implementation of gemma.c's
 * KV-cache hot path -- per-layer K/V append with QK-norm + RoPE fused into the
 * write, the paged ring / linear cache, and the GQA split-KV flash-decode.
 *
 * Conventions shared by every entry point (they are the reference's,
 * src/gemma4_kv_cache.cu:149-180 and src/gemma4_flash_attention_decode.cu:1122-1157):
 *   - plain pointers and sizes only; every buffer is owned by the caller;
 *     nothing here allocates or frees device memory unless its name says
 *     "runtime_state";
 *   - device pointers unless the parameter name starts with h_;
 *   - the return value is a cudaError_t carried as int: 0 = cudaSuccess,
 *     1 = cudaErrorInvalidValue for rejected host arguments; launch errors
 *     come from cudaGetLastError();
 *   - rows whose page, batch or position is invalid on the device are
 *     silently skipped (tests/test_kv_cache.cu:94-133 pins this);
 *   - work is enqueued on `stream` and is asynchronous; no call synchronises.
 *
 * bf16 tensors are passed as uint16_t* (bit patterns of __nv_bfloat16), fp8
 * e4m3 as uint8_t*; `stream` is a cudaStream_t passed as void*.
 */
#ifndef GEMMA4_B200KV_H_
#define GEMMA4_B200KV_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef uint16_t b200kv_bf16;
typedef void *b200kv_stream;

/* Same layout as src/gemma4_kv_cache.cuh:9-18 (8 x int32, passed by value).
 * Cache tensors are [num_layers, num_pages, page_size, num_heads, head_dim];
 * window_size == 0 means a linear (global) cache, > 0 a sliding ring. */
#ifndef GEMMA4_KV_CACHE_CONFIG_DEFINED
#define GEMMA4_KV_CACHE_CONFIG_DEFINED
typedef struct Gemma4KvCacheConfig {
  int32_t num_layers;
  int32_t num_pages;
  int32_t page_size;
  int32_t max_pages_per_seq;
  int32_t batch_size;
  int32_t num_heads;
  int32_t head_dim;
  int32_t window_size;
} Gemma4KvCacheConfig;
#endif

/* How the RMSNorm scale 1/sqrt(mean(x^2)+eps) is evaluated in the prep. */
enum {
  /* rsqrt.approx.f32 as the reference's GPU code does
   * (src/gemma4_rmsnorm.cu:100): bit-identical to the reference kernels on
   * the same GPU. */
  B200KV_NORM_RSQRT_APPROX = 0,
  /* IEEE sqrt and divide, round-to-nearest: bit-identical to a host
   * restatement. */
  B200KV_NORM_IEEE = 1
};

/* ------------------------------------------------------------------ *
 * Cache write of already prepared rows.
 * Replaces gemma4_kv_cache_write_bf16, src/gemma4_kv_cache.cuh:55-66
 * (same name, argument order and error behaviour).
 * ------------------------------------------------------------------ */
#ifndef GEMMA4_B200KV_TYPED_CACHE_WRITE /* the .hpp declares it with CUDA types */
int gemma4_kv_cache_write_bf16(b200kv_bf16 *d_cache_k, b200kv_bf16 *d_cache_v,
                               Gemma4KvCacheConfig config,
                               const int32_t *d_page_table,
                               const int32_t *d_token_batch,
                               const int32_t *d_token_position,
                               int32_t token_count, int32_t layer,
                               const b200kv_bf16 *d_k, const b200kv_bf16 *d_v,
                               b200kv_stream stream);
#endif

/* ------------------------------------------------------------------ *
 * Host-side geometry and page bookkeeping.
 * ------------------------------------------------------------------ */
/* gemma4_kv_cache_offset, src/gemma4_kv_cache.cuh:28-38. */
int64_t b200kv_cache_offset(const Gemma4KvCacheConfig *config, int32_t layer,
                            int32_t page, int32_t page_offset, int32_t head,
                            int32_t dim);
/* gemma4_kv_cache_make_config, src/gemma4_kv_cache.cu:76-91. */
void b200kv_make_config(Gemma4KvCacheConfig *out, int32_t global,
                        int32_t num_pages, int32_t page_size,
                        int32_t max_pages_per_seq);
/* gemma4_is_global_layer, src/gemma4.h:105-108. */
int32_t b200kv_is_global_layer(int32_t model_layer);
/* gemma4_kv_cache_layer_index, src/gemma4_kv_cache.cu:94-105. */
int32_t b200kv_layer_index(int32_t model_layer, int32_t global_cache);
/* gemma4_kv_cache_ensure_page, src/gemma4_kv_cache.cu:108-123. Arrays are
 * host int32 [batch_size * max_pages_per_seq]. Returns the physical page or -1. */
int32_t b200kv_ensure_page(int32_t *h_page_table, int32_t *h_slot_logical_pages,
                           const Gemma4KvCacheConfig *config, int32_t batch,
                           int32_t position);
/* gemma4_kv_cache_ensure_range, src/gemma4_kv_cache.cu:126-146. 0 or -1. */
int32_t b200kv_ensure_range(int32_t *h_page_table,
                            int32_t *h_slot_logical_pages,
                            const Gemma4KvCacheConfig *config, int32_t batch,
                            int32_t first_position, int32_t token_count);
/* sliding_pages_per_sequence, src/gemma4_runtime.cu:18-24. */
int32_t b200kv_sliding_pages_per_sequence(int32_t max_seq_len,
                                          int32_t page_size);
/* fill_rope_tables, src/gemma4_runtime.cu:27-45: host fp32 tables
 * [max_seq_len, rotary_half]. */
void b200kv_fill_rope_tables(float *h_cos, float *h_sin, int32_t max_seq_len,
                             int32_t rotary_half, float theta,
                             int32_t exponent_dim);

/* ------------------------------------------------------------------ *
 * Runtime state (owner of caches, page tables and per-step metadata).
 * Replaces Gemma4RuntimeState and its four functions,
 * src/gemma4_runtime.cuh:12-64. The C++ struct of the same name and field
 * order is in gemma4_b200kv.hpp; these wrappers give C callers a handle.
 * ------------------------------------------------------------------ */
typedef struct B200KvRuntimeState B200KvRuntimeState;

/* Geometry of the two caches the state owns. The reference fixes these as
 * compile-time constants (src/gemma4.h:17-23); here they are arguments so the
 * same owner serves 8 KV x 256 global layers as well as the 1 KV x 512 ones. */
typedef struct B200KvRuntimeGeometry {
  int32_t sliding_layers, sliding_kv_heads, sliding_head_dim, sliding_window;
  int32_t sliding_rotary_dim;
  float sliding_rope_theta;
  int32_t global_layers, global_kv_heads, global_head_dim;
  int32_t global_rotary_dim;
  float global_rope_theta;
  int32_t global_rope_exponent_dim;
} B200KvRuntimeGeometry;

/* Reference geometry (src/gemma4.h:8-29). */
void b200kv_runtime_geometry_default(B200KvRuntimeGeometry *out);
/* gemma4_runtime_state_init, src/gemma4_runtime.cu:95-234. geometry may be
 * NULL for the reference geometry. *out is NULL on failure. */
int b200kv_runtime_state_create(B200KvRuntimeState **out, int32_t batch_size,
                                int32_t max_seq_len, int32_t page_size,
                                const B200KvRuntimeGeometry *geometry,
                                b200kv_stream stream);
/* gemma4_runtime_state_free, src/gemma4_runtime.cu:77-92. */
void b200kv_runtime_state_destroy(B200KvRuntimeState *state);
/* gemma4_runtime_prepare_prefill, src/gemma4_runtime.cu:237-273. */
int b200kv_runtime_prepare_prefill(B200KvRuntimeState *state, int32_t seq_len,
                                   b200kv_stream stream);
/* gemma4_runtime_prepare_decode_step, src/gemma4_runtime.cu:276-341: all
 * sequences are validated before anything is changed. */
int b200kv_runtime_prepare_decode_step(B200KvRuntimeState *state,
                                       b200kv_stream stream);

typedef struct B200KvRuntimeView {
  int32_t batch_size, max_seq_len, page_size, token_count;
  Gemma4KvCacheConfig sliding_cache_config, global_cache_config;
  b200kv_bf16 *sliding_cache_k, *sliding_cache_v;
  b200kv_bf16 *global_cache_k, *global_cache_v;
  int32_t *sliding_page_table, *global_page_table;
  int32_t *seq_lengths, *token_batch, *token_position;
  float *sliding_cos, *sliding_sin, *global_cos, *global_sin;
  /* host mirrors (read/write: the reference's tests edit h_seq_lengths) */
  int32_t *h_sliding_page_table, *h_global_page_table;
  int32_t *h_sliding_slot_logical_pages, *h_global_slot_logical_pages;
  int32_t *h_seq_lengths, *h_token_batch, *h_token_position;
  int64_t h_sliding_page_table_size, h_global_page_table_size;
  int64_t h_token_rows;
} B200KvRuntimeView;
void b200kv_runtime_state_view(B200KvRuntimeState *state,
                               B200KvRuntimeView *out);

/* ------------------------------------------------------------------ *
 * Prep (per-head RMSNorm + RoPE) for a whole prompt into contiguous tensors:
 * the first stage of gemma4_flash_attention_{sliding,global}_fwd_bf16_norm_rope,
 * src/gemma4_flash_attention.cuh:9-45 (kernel src/gemma4_flash_attention_prefill.cu:1022-1103).
 * q/q_prepared are [rows, q_heads, head_dim]; k, v and their outputs
 * [rows, kv_heads, head_dim]; d_v == NULL derives V from raw K (global
 * layers). Rows with a negative position are left untouched.
 * ------------------------------------------------------------------ */
int b200kv_prefill_prep_bf16(b200kv_bf16 *d_q_prepared,
                             b200kv_bf16 *d_k_prepared,
                             b200kv_bf16 *d_v_prepared, const b200kv_bf16 *d_q,
                             const b200kv_bf16 *d_k, const b200kv_bf16 *d_v,
                             const b200kv_bf16 *d_q_norm_weight,
                             const b200kv_bf16 *d_k_norm_weight,
                             const float *d_cos, const float *d_sin,
                             const int32_t *d_token_position, int64_t rows,
                             int32_t q_heads, int32_t kv_heads,
                             int32_t head_dim, int32_t rotary_dim,
                             int32_t norm_mode, b200kv_stream stream);

/* ------------------------------------------------------------------ *
 * Prompt attention, C bindings of gemma4_flash_attention_sliding_fwd_bf16_norm_rope
 * and gemma4_flash_attention_global_fwd_bf16_norm_rope
 * (src/gemma4_flash_attention.cuh:9-45): prep of every row (as
 * b200kv_prefill_prep_bf16, norm mode rsqrt.approx like the reference's GPU
 * code) into d_*_prepared, then causal attention of each sequence over its own
 * prepared rows -- query row r sees keys c <= r and, for the sliding variant,
 * c >= max(0, r - window_size + 1) -- into d_out [row, 16, D]. seqlen_q must
 * equal seqlen_k (cudaErrorInvalidValue otherwise, as the reference).
 * b200kv_prefill_attention_bf16 is the attention stage alone on rows that are
 * already prepared (window_size 0: causal only; head_dim 256 or 512).
 * b200kv_prefill_attention_fault synchronises the device and returns 0, or
 * which bounded wait of the head_dim-256 tensor-core kernel ran out in the
 * last launch (1..3; its output is then undefined), or -1 if the word could
 * not be read. The reference has no counterpart: its kernels do not wait.
 * ------------------------------------------------------------------ */
int b200kv_flash_attention_sliding_fwd_bf16_norm_rope(
    b200kv_bf16 *d_out, b200kv_bf16 *d_q_prepared, b200kv_bf16 *d_k_prepared,
    b200kv_bf16 *d_v_prepared, const b200kv_bf16 *d_q, const b200kv_bf16 *d_k,
    const b200kv_bf16 *d_v, const b200kv_bf16 *d_q_norm_weight,
    const b200kv_bf16 *d_k_norm_weight, const float *d_cos, const float *d_sin,
    const int32_t *d_token_position, int32_t batch_size, int32_t seqlen_q,
    int32_t seqlen_k, int32_t window_size, float softmax_scale,
    b200kv_stream stream);
int b200kv_flash_attention_global_fwd_bf16_norm_rope(
    b200kv_bf16 *d_out, b200kv_bf16 *d_q_prepared, b200kv_bf16 *d_k_prepared,
    b200kv_bf16 *d_v_prepared, const b200kv_bf16 *d_q, const b200kv_bf16 *d_k,
    const b200kv_bf16 *d_q_norm_weight, const b200kv_bf16 *d_k_norm_weight,
    const float *d_cos, const float *d_sin, const int32_t *d_token_position,
    int32_t batch_size, int32_t seqlen_q, int32_t seqlen_k, float softmax_scale,
    b200kv_stream stream);
int b200kv_prefill_attention_bf16(b200kv_bf16 *d_out,
                                  const b200kv_bf16 *d_q_prepared,
                                  const b200kv_bf16 *d_k_prepared,
                                  const b200kv_bf16 *d_v_prepared,
                                  int32_t batch_size, int32_t seq_len,
                                  int32_t q_heads, int32_t kv_heads,
                                  int32_t head_dim, int32_t window_size,
                                  float softmax_scale, b200kv_stream stream);
int b200kv_prefill_attention_fault(void);

/* ------------------------------------------------------------------ *
 * Cache fill after a prompt: the prepared K/V rows of batch_size sequences of
 * seq_len tokens each (row b * seq_len + t, with d_token_batch / d_token_position
 * as gemma4_runtime_prepare_prefill leaves them) go into the cache in one
 * launch. A linear cache, or a prompt no longer than the window, takes every
 * row; a sliding cache with a longer prompt takes only the last window_size
 * rows of each sequence. Replaces the write step of gemma4_prefill_megakernel,
 * src/gemma4_prefill_megakernel.cu:189-207 (which loops over sequences with
 * one gemma4_kv_cache_write_bf16 call each for the second case).
 * ------------------------------------------------------------------ */
int b200kv_prefill_cache_fill_bf16(b200kv_bf16 *d_cache_k,
                                   b200kv_bf16 *d_cache_v,
                                   Gemma4KvCacheConfig config,
                                   const int32_t *d_page_table,
                                   const int32_t *d_token_batch,
                                   const int32_t *d_token_position,
                                   int32_t batch_size, int32_t seq_len,
                                   int32_t layer, const b200kv_bf16 *d_k_prepared,
                                   const b200kv_bf16 *d_v_prepared,
                                   b200kv_stream stream);

/* ------------------------------------------------------------------ *
 * Fused decode append: for every sequence b < batch_count, prep the new
 * token's q heads into d_q_prepared and prep + store its K and V rows in the
 * paged cache at position d_token_position[b].
 * Replaces phase_decode_q_paged_kv_norm_rope,
 * src/gemma4_flash_attention_decode.cu:305-375 (argument names follow it).
 * q is [batch, q_heads, head_dim]; k, v are [batch, kv_heads, head_dim];
 * d_v == NULL derives V from raw K.
 * ------------------------------------------------------------------ */
int b200kv_decode_append_bf16(b200kv_bf16 *d_q_prepared,
                              b200kv_bf16 *d_cache_k, b200kv_bf16 *d_cache_v,
                              Gemma4KvCacheConfig cache_config,
                              const int32_t *d_page_table,
                              const int32_t *d_token_position,
                              int32_t cache_layer, const b200kv_bf16 *d_q,
                              const b200kv_bf16 *d_k, const b200kv_bf16 *d_v,
                              const b200kv_bf16 *d_q_norm_weight,
                              const b200kv_bf16 *d_k_norm_weight,
                              const float *d_cos, const float *d_sin,
                              int32_t batch_count, int32_t q_heads,
                              int32_t rotary_dim, int32_t norm_mode,
                              b200kv_stream stream);

/* ------------------------------------------------------------------ *
 * Split-KV flash-decode over the paged cache, then the combine.
 * Replaces phase_decode_paged_grouped_split + phase_decode_paged_reduce
 * (+ the single-split direct path), src/gemma4_flash_attention_decode.cu:613-977,
 * with the meaning of split_size / num_splits kept: split s of sequence b
 * covers keys [first_key + s*split_size, min(seq_len, ... + split_size)),
 * first_key = max(0, seq_len - window); splits beyond the live count do
 * nothing; num_splits == 1 writes the output directly and needs no scratch.
 *
 * d_out [batch, q_heads, head_dim] bf16; d_lse [batch, q_heads] fp32 natural
 * log-sum-exp of the scaled scores (may be NULL; -inf when no key is live);
 * scratch as in src/gemma4_prompt.cu:231-248:
 *   d_partial_m, d_partial_l  [batch * q_heads * num_splits] fp32
 *   d_partial_acc             [batch * q_heads * num_splits * head_dim] fp32
 * d_status: optional int32[4] device word block; a kernel that gives up a
 * bounded wait writes a non-zero code to d_status[0] (see B200KV_STATUS_*).
 *
 * split_size == 0 (not a value the reference accepts) asks for the balanced
 * partition instead: the live keys of the whole batch are divided evenly over
 * a fixed grid of two CTAs per SM, whatever the individual lengths, so ragged
 * batches leave no SM idle. num_splits then only states how large the scratch
 * is (still batch * q_heads * num_splits rows; use b200kv_plan_balanced).
 * Available for 8 KV heads x 256 with 16 query heads and batch <= 1024, and
 * for the reference's native global-layer geometry, 1 KV head x 512 with 16
 * query heads and batch <= 256 (src/gemma4_flash_attention_decode.cu:150-157;
 * this geometry has no fixed-split form here); cudaErrorInvalidValue otherwise.
 *
 * Ordering: the call may follow b200kv_decode_append_* on the same stream
 * with nothing in between (as b200kv_decode_layer_step_bf16 does). The
 * kernels are launched programmatically dependent: the attention starts
 * streaming keys while that append is still running and only waits for it
 * before it touches the prepared q or the page that holds each sequence's
 * newest key. The append must therefore be the one of this decode step, i.e.
 * write position seq_length - 1; rows of older pages must have been written
 * by earlier work on the stream. Any other predecessor is waited for in full.
 * ------------------------------------------------------------------ */
int b200kv_decode_attention_bf16(b200kv_bf16 *d_out, float *d_lse,
                                 const b200kv_bf16 *d_q_prepared,
                                 const b200kv_bf16 *d_cache_k,
                                 const b200kv_bf16 *d_cache_v,
                                 Gemma4KvCacheConfig cache_config,
                                 const int32_t *d_page_table,
                                 const int32_t *d_seq_lengths,
                                 int32_t cache_layer, float softmax_scale,
                                 int32_t split_size, int32_t num_splits,
                                 int32_t batch_count, int32_t q_heads,
                                 float *d_partial_m, float *d_partial_l,
                                 float *d_partial_acc, int32_t *d_status,
                                 b200kv_stream stream);

/* ------------------------------------------------------------------ *
 * FP8 e4m3 KV cache with one fp32 scale per (16-token page, KV head) and
 * tensor. No counterpart in the reference, whose caches are bf16 only. Cache
 * tensors keep the [layer, page, offset, head, dim] layout with one byte per
 * element; d_scale_k / d_scale_v are fp32 [layer, page, head] and must be
 * zero before a cache is first used. Quantisation rule, per tensor, page and
 * head, per call: with R the rows of the call landing in the page and o0 the
 * offset of the first, s_old = (o0 == 0 ? 0 : scale), s_new = max(s_old,
 * max(amax(R)/448, FLT_MIN)); if s_new > s_old the rows already stored below
 * o0 are re-encoded as enc(dec(byte)*s_old/s_new); R is stored as enc(x/s_new)
 * (round to nearest even, saturating at +-448) and the scale becomes s_new.
 * Built for 8 KV heads x 256 (16 query heads, rotary 256).
 * ------------------------------------------------------------------ */
/* Fused decode append (prep as b200kv_decode_append_bf16, then the rule above
 * for the one new row of every sequence). */
int b200kv_decode_append_fp8(b200kv_bf16 *d_q_prepared, uint8_t *d_cache_k,
                             uint8_t *d_cache_v, float *d_scale_k,
                             float *d_scale_v, Gemma4KvCacheConfig cache_config,
                             const int32_t *d_page_table,
                             const int32_t *d_token_position,
                             int32_t cache_layer, const b200kv_bf16 *d_q,
                             const b200kv_bf16 *d_k, const b200kv_bf16 *d_v,
                             const b200kv_bf16 *d_q_norm_weight,
                             const b200kv_bf16 *d_k_norm_weight,
                             const float *d_cos, const float *d_sin,
                             int32_t batch_count, int32_t q_heads,
                             int32_t rotary_dim, int32_t norm_mode,
                             b200kv_stream stream);
/* Bulk append of already prepared rows (a prompt): run i covers positions
 * [d_first_position[i], + d_row_count[i]) of sequence d_seq_batch[i]; its rows
 * start at row d_row_start[i] of d_k_prepared / d_v_prepared
 * ([rows, kv_heads, head_dim] bf16). max_row_count >= every d_row_count[i]
 * (sizes the grid). All rows of a run that share a page are quantised as one
 * group. The rows of one call must map to distinct cache rows. */
int b200kv_fp8_append_rows(uint8_t *d_cache_k, uint8_t *d_cache_v,
                           float *d_scale_k, float *d_scale_v,
                           Gemma4KvCacheConfig cache_config,
                           const int32_t *d_page_table,
                           const int32_t *d_seq_batch,
                           const int32_t *d_first_position,
                           const int32_t *d_row_count,
                           const int32_t *d_row_start, int32_t run_count,
                           int32_t max_row_count, int32_t cache_layer,
                           const b200kv_bf16 *d_k_prepared,
                           const b200kv_bf16 *d_v_prepared,
                           b200kv_stream stream);
/* Decode attention over the fp8 cache, dequantisation fused (K scale on the
 * score, V scale on the softmax weight). Always the balanced partition; the
 * scratch holds batch * q_heads * num_splits rows (b200kv_plan_balanced). */
int b200kv_decode_attention_fp8(b200kv_bf16 *d_out, float *d_lse,
                                const b200kv_bf16 *d_q_prepared,
                                const uint8_t *d_cache_k,
                                const uint8_t *d_cache_v,
                                const float *d_scale_k, const float *d_scale_v,
                                Gemma4KvCacheConfig cache_config,
                                const int32_t *d_page_table,
                                const int32_t *d_seq_lengths,
                                int32_t cache_layer, float softmax_scale,
                                int32_t num_splits, int32_t batch_count,
                                int32_t q_heads, float *d_partial_m,
                                float *d_partial_l, float *d_partial_acc,
                                int32_t *d_status, b200kv_stream stream);

enum {
  B200KV_STATUS_OK = 0,
  B200KV_STATUS_WAIT_TIMEOUT = 1 /* a bounded mbarrier wait ran out */
};

/* The same attention for callers that cannot hand over scratch buffers: a
 * serving engine that gave all device memory to its page pool at start-up, a
 * plug-in that owns no allocator, or a latency path that must not pay the
 * device-wide synchronisation of cudaMalloc / cudaFree. This entry point has
 * no counterpart in the reference (whose callers always pass the partial
 * buffers, src/gemma4_prompt.cu:231-248). The split partials live in an array
 * of B200KV_STATIC_SCRATCH_BYTES that is part of the library image, held on
 * every GPU the library is loaded on until the process exits; the call makes
 * no cudaMalloc, cudaFree or other allocating call.
 *   - Refused with cudaErrorInvalidValue (and a line on stderr) when
 *     2 * round_up(batch*q_heads*num_splits, 64) * 4
 *       + batch*q_heads*num_splits*head_dim*4 bytes exceed that size.
 *     With fixed splits (split_size > 0) num_splits == 1 needs no scratch and
 *     is never refused for size; the balanced partition (split_size == 0)
 *     always works through scratch, so it needs num_splits >= 2 (take it from
 *     b200kv_plan_balanced) and returns cudaErrorInvalidValue for 1.
 *   - The first call on each device looks the array's device address up
 *     (cudaGetSymbolAddress, with that device current) and keeps it for the
 *     life of the process; make that first call before any stream capture
 *     begins. The kept address belongs to the device's primary context: after
 *     cudaDeviceReset (or anything else that destroys that context) it is
 *     stale, so a process that resets a device must not call this entry point
 *     on it afterwards.
 *   - All calls on a device share the array and it keeps the last call's
 *     contents. Nothing needs clearing between calls, but calls whose kernels
 *     may overlap on the GPU race on it: keep them on one stream.
 * Arguments and results are those of b200kv_decode_attention_bf16 minus the
 * three partial pointers. */
#define B200KV_STATIC_SCRATCH_BYTES (16u << 20)
int b200kv_decode_attention_static_scratch_bf16(
    b200kv_bf16 *d_out, float *d_lse, const b200kv_bf16 *d_q_prepared,
    const b200kv_bf16 *d_cache_k, const b200kv_bf16 *d_cache_v,
    Gemma4KvCacheConfig cache_config, const int32_t *d_page_table,
    const int32_t *d_seq_lengths, int32_t cache_layer, float softmax_scale,
    int32_t split_size, int32_t num_splits, int32_t batch_count,
    int32_t q_heads, int32_t *d_status, b200kv_stream stream);

/* Bytes of scratch for the three partial buffers, in the order m, l, acc. */
void b200kv_decode_workspace_bytes(int32_t batch_count, int32_t q_heads,
                                   int32_t head_dim, int32_t num_splits,
                                   size_t *partial_m_bytes,
                                   size_t *partial_l_bytes,
                                   size_t *partial_acc_bytes);

/* Picks a split size (a multiple of the kernel's key tile) and the matching
 * split count so that batch_count * num_splits fills the GPU's SMs a few
 * times over; max_live_keys is the largest min(seq_len, window) in the batch.
 * The reference hard-codes 20 keys per split (src/gemma4.h:24), tuned for an
 * 84-SM GPU. */
void b200kv_plan_splits(int32_t batch_count, int32_t max_live_keys,
                        int32_t kv_heads, int32_t sm_count,
                        int32_t *split_size, int32_t *num_splits);
/* num_splits to pass with split_size == 0 so that the scratch can hold one
 * partial per CTA and sequence boundary: ceil(2 * sm_count / batch) + 1. */
void b200kv_plan_balanced(int32_t batch_count, int32_t sm_count,
                          int32_t *num_splits);
/* Same, when the host also knows the sum of live keys over the batch (it does:
 * the runtime state mirrors seq_lengths on the host, src/gemma4_runtime.cuh:38):
 * picks the split size that minimises waves x per-CTA time plus the traffic of
 * the partials for that many CTAs. */
void b200kv_plan_splits_total(int32_t batch_count, int32_t max_live_keys,
                              int64_t total_live_keys, int32_t kv_heads,
                              int32_t sm_count, int32_t *split_size,
                              int32_t *num_splits);

/* ------------------------------------------------------------------ *
 * One layer-step = fused append + split-KV decode + combine, enqueued back to
 * back on one stream. The fields carry the attention_* members of
 * Gemma4DecodeMegakernelLayerArgs, src/gemma4_megakernel.cuh:42-66, with the
 * same names minus the prefix; it stands where the three bracketed phases of
 * decode_megakernel_fused_layer_kernel run
 * (src/gemma4_flash_attention_decode.cu:514-523,1004-1031).
 *
 * With split_size == 0, 8 KV heads x 256, 16 query heads, rotary_dim 256 and
 * batch <= 1024 the append runs inside the attention kernel (one launch plus
 * the combine): the CTA that streams a sequence's newest key prepares that
 * row, uses it from shared memory and writes it to the cache; q is prepared
 * by the warps that use it and written to `q` as the separate append would.
 * Cache bytes, `q`, `out` and `lse` are the same bits as those of
 * b200kv_decode_append_bf16 followed by b200kv_decode_attention_bf16.
 * The environment variable B200KV_FUSED_LAYER_STEP=0 (read once) keeps the two
 * launches apart, for comparison.
 * ------------------------------------------------------------------ */
/* Words of the layer-step's `ticket` buffer per sequence and KV head: one for
 * the (sequence, head) pair and one per group of 32 key ranges. */
#define B200KV_TICKETS_PER_HEAD 11

typedef struct B200KvLayerStepArgs {
  b200kv_bf16 *q;                 /* out: prepared q [batch, q_heads, head_dim] */
  b200kv_bf16 *out;               /* out: attention [batch, q_heads, head_dim] */
  float *lse;                     /* out, optional */
  float *partial_m, *partial_l, *partial_acc;
  b200kv_bf16 *cache_k, *cache_v;
  Gemma4KvCacheConfig cache_config;
  const int32_t *page_table;
  const int32_t *token_position;
  const int32_t *seq_lengths;
  int32_t cache_layer;
  int32_t split_size;
  int32_t num_splits;
  float softmax_scale;
  const b200kv_bf16 *raw_q, *raw_k, *raw_v; /* this step's projections */
  const b200kv_bf16 *q_norm_weight, *k_norm_weight;
  const float *cos, *sin;
  int32_t batch_count;
  int32_t q_heads;
  int32_t rotary_dim;
  int32_t norm_mode;
  int32_t *status;                /* optional int32[4] */
  /* Optional profiling hooks: cudaEvent_t handles recorded on `stream` right
   * before and right after the attention (split + combine) launches; when the
   * layer-step runs as one fused launch (append inside the attention kernel),
   * right before and after that launch and its combine. */
  void *event_before_attention;
  void *event_after_attention;
  /* Optional: uint32 [batch_count * cache_config.num_heads *
   * B200KV_TICKETS_PER_HEAD], zero before the first call; every call leaves
   * it zero again (unless a bounded wait ran
   * out, which `status` reports). With it, and split_size == 0, small jobs --
   * a sliding-window layer of up to 32 sequences, or one sequence on a linear
   * cache (with 8 KV heads: one with room for at most 32768 keys; with fewer,
   * the cache of a KV-head-sharded rank, any) (head_dim 256, two query heads
   * per KV head, rotary_dim 256) -- run as ONE launch: a CTA per (sequence, KV head, key
   * range) fetches that head's rows as TMA tiles, and the last CTA of each
   * (sequence, head) to finish merges the ranges' partials, the job of the
   * reference's grid-wide barrier + reduce phase
   * (src/gemma4_flash_attention_decode.cu:1017-1031). Results as without it,
   * within the summation order of the partials. Calls that may overlap on the
   * GPU need tickets (and scratch) of their own. */
  uint32_t *ticket;
  /* Optional, KV-head-sharded mode: a connected handle of
   * b200kv_peer_buffer_create. The step then ends with the all-gather of `out`
   * ([batch, q_heads, head_dim] of this rank, <= the handle's slot_bytes) over
   * peer memory, as if b200kv_peer_allgather(handle, out, ...) followed it; read
   * the result with b200kv_peer_buffer_gathered. Where the step runs as the
   * one-launch kernel the exchange is part of that kernel: the CTA that
   * finishes a (sequence, head) stores its rows into this rank's slot on every
   * GPU, the last of them publishes the flag and waits (bounded, see `status`)
   * for the peers' -- compute and collective in one launch. Every rank makes
   * the call with the same batch and head counts. */
  void *peer_gather;
} B200KvLayerStepArgs;

int b200kv_decode_layer_step_bf16(const B200KvLayerStepArgs *args,
                                  b200kv_stream stream);

/* How many kernels b200kv_decode_layer_step_bf16 would launch for these
 * arguments (1: the one-launch form; 2: fused attention + combine, or append +
 * a single-split attention; 3: append, split attention, combine). */
int32_t b200kv_layer_step_launches(const B200KvLayerStepArgs *args);

/* The one-launch form chosen explicitly (see `ticket` above): the same
 * layer-step through the per-(sequence, KV head, key range) kernel whatever
 * the batch size; cudaErrorInvalidValue without a ticket, with split_size != 0,
 * or for a geometry it is not built for (head_dim 256, q_heads == 2 * KV heads,
 * rotary_dim 256, a page size of 2, 4, 8 or a multiple of 16). Key ranges are
 * cut per sequence, so very uneven lengths leave CTAs idle; the default entry
 * point picks the balanced partition there. num_splits still sizes the scratch
 * (two rows per key range and head). */
int b200kv_decode_layer_step_tiled_bf16(const B200KvLayerStepArgs *args,
                                        b200kv_stream stream);
/* The attention alone in that form, on rows already appended and a q already
 * prepared: arguments of b200kv_decode_attention_bf16 with the balanced
 * partition's num_splits, plus the tickets. */
int b200kv_decode_attention_tiled_bf16(
    b200kv_bf16 *d_out, float *d_lse, const b200kv_bf16 *d_q_prepared,
    const b200kv_bf16 *d_cache_k, const b200kv_bf16 *d_cache_v,
    Gemma4KvCacheConfig cache_config, const int32_t *d_page_table,
    const int32_t *d_seq_lengths, int32_t cache_layer, float softmax_scale,
    int32_t num_splits, int32_t batch_count, int32_t q_heads, float *d_partial_m,
    float *d_partial_l, float *d_partial_acc, uint32_t *d_ticket,
    int32_t *d_status, b200kv_stream stream);

/* One decode step over `layer_count` layers, enqueued in order on `stream`:
 * the layer loop of gemma4_decode_megakernel, src/gemma4_decode_megakernel.cu:172-183,
 * restricted to the KV path (the caller supplies each layer's projections).
 * Entries are either different cache layers (caches that do not overlap in
 * memory), as in the model -- a layer's kernel then streams all of its keys
 * under the tails of the layers before it -- or, where two entries name the same
 * cache_k / cache_v and cache_layer, consecutive decode steps of that layer in
 * order (each appends the position after the one its predecessor appended, for
 * every sequence): the later step then does not read the rows its unfinished
 * predecessors append from the cache -- it prepares them itself from those
 * entries' raw rows (the same arithmetic, the same bits), or, where a
 * predecessor is not an entry of this call, leaves their pages until it is
 * complete. Several steps of one layer in one call are the way to keep a
 * one-layer decode loop's launches overlapped. */
int b200kv_decode_step_bf16(const B200KvLayerStepArgs *layers,
                            int32_t layer_count, b200kv_stream stream);
/* What b200kv_decode_step_bf16 would tell each entry's launch, without
 * launching anything (host only; every output may be NULL):
 * steps_in_flight[i] -- how many of the launches that can still be running
 * when entry i's kernel starts are taken to be earlier decode steps of entry
 * i's own cache layer (0: none of them writes that cache), release_early[i]
 * -- whether entry i's kernel lets entry i + 1's start at once, forwarded[i]
 * -- for how many of those earlier steps entry i's kernel prepares the
 * appended rows itself from their raw rows instead of waiting for them to reach
 * the cache (all of them when they are entries of this call, else none).
 * Entries that do not run as the one-launch layer-step neither release early
 * nor are released early. */
int b200kv_decode_step_plan(const B200KvLayerStepArgs *layers, int32_t layer_count,
                            int32_t *steps_in_flight, int32_t *release_early,
                            int32_t *forwarded);

/* ------------------------------------------------------------------ *
 * The steps either side of the KV path inside the reference's fused decode
 * layer, for `batch_count` rows of one token each and hidden size 3840
 * (GEMMA4_HIDDEN_SIZE, src/gemma4.h:6). Matrices are column-major as the
 * reference packs them (`*_proj_col_major`): output column c is `width`
 * contiguous bf16. The sums are added in the order of the reference's
 * 512-thread block, so the bf16 results are the bits its kernels write
 * (norm_mode B200KV_NORM_RSQRT_APPROX) or the host oracle's (B200KV_NORM_IEEE).
 *
 * b200kv_decode_ingress_bf16 replaces phase_decode_rmsnorm_project_bf16,
 * src/gemma4_flash_attention_decode.cu:447-496: RMSNorm of the layer input with
 * `input_norm_weight`, then the [Q|K|V] projection. `raw_qkv` receives raw q
 * [batch, q_width], then raw k [batch, k_width], then raw v [batch, cols -
 * q_width - k_width] (for one row the reference's raw scratch; v is absent for
 * the global geometry, whose V comes from raw K).
 *
 * b200kv_decode_egress_bf16 replaces project_attention_out_post_attention,
 * src/gemma4_flash_attention_decode.cu:35-129, and the pre-FFN norm that
 * follows it (:1049-1058): residual_out = attention_out x O; normed_out =
 * RMSNorm(residual_out, post_norm_weight); ffn_residual = x + normed_out;
 * ffn_x = RMSNorm(ffn_residual, pre_ffn_norm_weight) when ffn_x is given.
 * attention_width is 4096 or 8192. `ticket` is uint32[batch_count], zero before
 * the first call (the kernel leaves it zero): the CTA that finishes a row last
 * runs the norms, where the reference uses two grid-wide barriers.
 *
 * Both return cudaErrorInvalidValue for null or misaligned (16 B) pointers and
 * sizes other than the above; batch_count 0 is a no-op.
 * ------------------------------------------------------------------ */
typedef struct B200KvIngressArgs {
  b200kv_bf16 *raw_qkv;
  const b200kv_bf16 *x;                    /* [batch, 3840] */
  const b200kv_bf16 *input_norm_weight;    /* [3840] */
  const b200kv_bf16 *qkv_proj_col_major;   /* [cols, 3840] */
  int32_t batch_count;
  int32_t hidden_size;                     /* 3840 */
  int32_t cols, q_width, k_width;
  int32_t norm_mode;
  int32_t *status;                         /* optional, as for the decode kernels */
} B200KvIngressArgs;

int b200kv_decode_ingress_bf16(const B200KvIngressArgs *args,
                               b200kv_stream stream);

typedef struct B200KvEgressArgs {
  b200kv_bf16 *residual_out, *normed_out, *ffn_residual;  /* [batch, 3840] */
  b200kv_bf16 *ffn_x;                      /* optional [batch, 3840] */
  const b200kv_bf16 *attention_out;        /* [batch, attention_width] */
  const b200kv_bf16 *o_proj_col_major;     /* [3840, attention_width] */
  const b200kv_bf16 *post_norm_weight, *pre_ffn_norm_weight;
  const b200kv_bf16 *x;                    /* [batch, 3840]: the layer input */
  uint32_t *ticket;
  int32_t batch_count;
  int32_t hidden_size;
  int32_t attention_width;
  int32_t norm_mode;
  int32_t *status;
} B200KvEgressArgs;

int b200kv_decode_egress_bf16(const B200KvEgressArgs *args,
                              b200kv_stream stream);

/* One decode layer from the layer input to the FFN input: ingress, the
 * layer-step above (append + attention + combine) and egress, enqueued in order
 * on `stream` -- the work of gemma4_decode_megakernel_flash_attention_layer_bf16,
 * src/gemma4_flash_attention_decode.cu:1033-1058,1122-1157, up to the call of the
 * FFN (which is not part of this library). Field names follow
 * Gemma4DecodeMegakernelLayerArgs, src/gemma4_megakernel.cuh:32-66. `kv.raw_q /
 * raw_k / raw_v` are ignored and set from `raw_qkv`; the geometry (q_heads,
 * head_dim, KV heads) is `kv`'s; has_v_projection 0 = the global geometry
 * (no V columns; V from raw K). */
typedef struct B200KvAttentionLayerArgs {
  B200KvLayerStepArgs kv;
  const b200kv_bf16 *attention_x;
  const b200kv_bf16 *attention_input_norm_weight;
  const b200kv_bf16 *attention_qkv_proj_col_major;
  const b200kv_bf16 *attention_o_proj_col_major;
  const b200kv_bf16 *attention_post_norm_weight;
  const b200kv_bf16 *attention_pre_ffn_norm_weight;
  b200kv_bf16 *raw_qkv;                    /* scratch, see the ingress */
  b200kv_bf16 *residual_out, *normed_out, *ffn_residual, *ffn_x;
  uint32_t *ticket;
  int32_t hidden_size;
  int32_t has_v_projection;
} B200KvAttentionLayerArgs;

int b200kv_decode_attention_layer_bf16(const B200KvAttentionLayerArgs *args,
                                       b200kv_stream stream);

/* ------------------------------------------------------------------ *
 * KV-head-sharded mode, one process per GPU: all-gather of the per-rank
 * attention rows over NVLink peer memory in one small kernel per rank (peer
 * stores + flags; no multicast, no library collective). No counterpart in the
 * reference, which is single-GPU; it takes the place of an ncclAllGather of a
 * few KiB, whose cost is launch and protocol latency.
 *
 * b200kv_peer_buffer_create allocates this rank's buffer (cudaMalloc:
 * 2 x world x slot_bytes + flags, zeroed) and writes a 64-byte export
 * (a cudaIpcMemHandle_t) that the caller passes to the other ranks by any
 * means (e.g. an all-gather of 64 bytes over its process group).
 * b200kv_peer_buffer_connect maps the other ranks' buffers from
 * `exports` = world x 64 bytes in rank order. All ranks must have connected
 * (a host barrier) before the first gather.
 * b200kv_peer_allgather enqueues the kernel on `stream`: `bytes` (multiple of
 * 16, <= slot_bytes) from `src` land in slot `rank` of every rank's buffer;
 * when the kernel has run, `*gathered` (device pointer, [world][slot_bytes],
 * valid until the call after next) holds every rank's rows. Every rank calls it
 * the same number of times. Waits are bounded (about a second): a rank whose
 * peers do not arrive writes B200KV_STATUS_WAIT_TIMEOUT to status[0]
 * (optional) and returns. Not for CUDA-graph replay: the host counts the calls
 * to pick the buffer half. world <= 8.
 * ------------------------------------------------------------------ */
int b200kv_peer_buffer_create(int64_t slot_bytes, int32_t world, int32_t rank,
                              void **handle, void *export_64_bytes);
int b200kv_peer_buffer_connect(void *handle, const void *exports);
int b200kv_peer_allgather(void *handle, const void *src, int64_t bytes,
                          int32_t *status, b200kv_stream stream,
                          void **gathered);
/* Key-range sharding (every rank holds all KV heads of a range of the keys and
 * attends the full query over it): the same kernel exchanges each rank's
 * normalised rows `out` [rows, head_dim] bf16 with their log-sum-exp `lse`
 * [rows] fp32 and, after the wait, merges them on every rank,
 *   merged = sum_r exp(lse_r - LSE) out_r,  LSE = log sum_r exp(lse_r)
 * (the combine of src/gemma4_flash_attention_decode.cu:881-977 across ranks;
 * a rank without live keys has lse = -inf and weight 0). `merged_out` may be
 * `out`; `merged_lse` is optional. rows <= 64,
 * slot_bytes >= rows * (head_dim * 2 + 4). */
int b200kv_peer_merge_attention(void *handle, b200kv_bf16 *merged_out,
                                float *merged_lse, const b200kv_bf16 *out,
                                const float *lse, int32_t rows, int32_t head_dim,
                                int32_t *status, b200kv_stream stream);
int b200kv_peer_buffer_destroy(void *handle);

/* Failure handling of the exchange. No counterpart in the reference.
 * b200kv_peer_buffer_set_wait_clocks: how many SM clocks later calls wait for a
 * peer's flag before they give up with B200KV_STATUS_WAIT_TIMEOUT (default
 * 2^31, about a second).
 * After a call timed out (a peer died, hung, or skipped a call) the ranks'
 * call counters no longer agree and later gathers would pair the wrong buffer
 * halves. b200kv_peer_buffer_reset brings a rank back to "no call made yet"
 * (synchronises the device, clears its flags and counter): every surviving
 * rank calls it, with a host-side barrier before and after, and the next
 * matched call gathers correctly again.
 * b200kv_peer_buffer_create_loopback / b200kv_peer_buffer_post are a one-GPU
 * stand-in for bring-up and tests: the other ranks' buffers are local
 * allocations that nobody writes, and _post stores `epoch` into this rank's
 * flags (both halves) in the name of rank `from_rank`, as that rank's kernel
 * would -- so a wait can be seen to run out (nothing posted) and to succeed
 * (posted) without a second GPU. */
int b200kv_peer_buffer_set_wait_clocks(void *handle, int64_t clocks);
/* Device pointer to what the most recent gather through `handle` delivered
 * ([world][slot_bytes]; valid until the call after next). */
int b200kv_peer_buffer_gathered(void *handle, void **gathered);
int b200kv_peer_buffer_reset(void *handle);
int b200kv_peer_buffer_create_loopback(int64_t slot_bytes, int32_t world,
                                       int32_t rank, void **handle);
int b200kv_peer_buffer_post(void *handle, int32_t from_rank, uint32_t epoch,
                            b200kv_stream stream);

/* Self-test of the bounded wait all kernels of the library share: one warp
 * waits, with that helper, on an mbarrier nothing arrives at, for clock_limit
 * SM clocks (1 .. 2^28), then writes B200KV_STATUS_WAIT_TIMEOUT to d_status[0]
 * (if it is 0) and the clocks it waited to *d_waited_clocks (optional) and
 * returns normally: the give-up path exercised without a fault. No counterpart
 * in the reference, whose kernels do not wait on one another. */
int b200kv_bounded_wait_selftest(int64_t clock_limit, int32_t *d_status,
                                 int64_t *d_waited_clocks, b200kv_stream stream);

/* ------------------------------------------------------------------ *
 * Host bookkeeping of the three ways the path shards over the GPUs of a node
 * (one process per GPU). No counterpart in the reference, which is single-GPU
 * and batch 1 (src/gemma4_decode_megakernel.cu:143). All return 0, or -1 for
 * arguments that make no sense; none touches a device.
 *
 * b200kv_shard_sequences: sequences are independent units (own pages, own
 * length, own output rows), so whole sequences are dealt to ranks and no
 * collective is on the data path. Greedy, longest first by h_live_keys[i]
 * (min(length, window) for sliding caches); h_owner[i] receives sequence i's
 * rank. The largest and smallest rank load differ by at most one sequence.
 *
 * b200kv_kv_head_range: KV heads are independent until the output row is
 * assembled; rank r holds caches with num_heads = kv_heads / world for heads
 * [*first_head, *first_head + *head_count) and their query heads, and the
 * step ends with b200kv_peer_allgather of the head outputs. kv_heads must be a
 * multiple of world.
 *
 * b200kv_key_range_page_table: one long sequence split by key range; rank r
 * holds all KV heads of a contiguous run of the sequence's pages. Writes the
 * rank's view of the one-row page table (its pages moved to the front, so that
 * its keys sit at local positions 0 .. *local_length - 1; the rest -1) and the
 * absolute position of its first key (the offset by which the RoPE tables are
 * entered for the new token's row). Pages are dealt whole, the last rank takes
 * the remainder; the ranks' rows are merged with b200kv_peer_merge_attention.
 * ------------------------------------------------------------------ */
int32_t b200kv_shard_sequences(const int64_t *h_live_keys, int32_t sequences,
                               int32_t world, int32_t *h_owner);
int32_t b200kv_kv_head_range(int32_t kv_heads, int32_t world, int32_t rank,
                             int32_t *first_head, int32_t *head_count);
int32_t b200kv_key_range_page_table(const int32_t *h_page_table,
                                    int32_t max_pages_per_seq, int32_t seq_len,
                                    int32_t page_size, int32_t world, int32_t rank,
                                    int32_t *h_rank_table, int32_t *local_length,
                                    int32_t *first_position);

/* Timing events for the hooks above (cudaEventCreate / Destroy / ElapsedTime).
 * No counterpart in the reference library; its benches time with the same
 * CUDA events, src/benches/gemma4_bench_utils.cuh:336-370. */
int b200kv_timer_create(void **event);
int b200kv_timer_destroy(void *event);
int b200kv_timer_record(void *event, b200kv_stream stream);
int b200kv_timer_elapsed_ms(void *begin, void *end, float *ms);

/* Library/version probe: returns the compiled SM architecture (1000 for
 * sm_100a) so a loader can check it got the CUDA build. */
int32_t b200kv_compiled_arch(void);

#ifdef __cplusplus
}
#endif

#endif /* GEMMA4_B200KV_H_ */

// Internal C++ interface between the kernel translation units and the C ABI.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/gemma4_b200kv.hpp"

namespace b200kv {

struct DecodeArgs {
  __nv_bfloat16 *out = nullptr;
  float *lse = nullptr;
  const __nv_bfloat16 *q = nullptr;
  const __nv_bfloat16 *cache_k = nullptr;
  const __nv_bfloat16 *cache_v = nullptr;
  Gemma4KvCacheConfig cfg = {};
  const int32_t *page_table = nullptr;
  const int32_t *seq_lengths = nullptr;
  int32_t layer = 0;
  float softmax_scale = 0.0f;
  int32_t split_size = 0;
  int32_t num_splits = 0;
  int32_t batch_count = 0;
  int32_t q_heads = 0;
  float *partial_m = nullptr;
  float *partial_l = nullptr;
  float *partial_acc = nullptr;
  int32_t *status = nullptr;
};

cudaError_t decode_attention_bf16(const DecodeArgs &args, cudaStream_t stream);

// split_size == 0 in DecodeArgs selects this path (see decode_balanced.cu):
// the batch's live keys are divided evenly over a fixed grid; num_splits then
// only sizes the scratch (batch * num_splits slots per head).
cudaError_t decode_attention_balanced_bf16(const DecodeArgs &args,
                                           cudaStream_t stream);
// FP8 e4m3 cache (one fp32 scale per page and KV head): balanced partition
// only; args.cache_k / cache_v are ignored in favour of the byte pointers.
cudaError_t decode_attention_fp8(const DecodeArgs &args, const void *cache_k,
                                 const void *cache_v, const float *scale_k,
                                 const float *scale_v, cudaStream_t stream);
bool decode_balanced_supported(const Gemma4KvCacheConfig &cfg, int q_heads,
                               int batch_count);
// The reference's native global-layer geometry, 16 query heads on one KV head
// of 512 dims (decode_gqa16.cu): balanced partition only (split_size == 0).
bool decode_gqa16_supported(const Gemma4KvCacheConfig &cfg, int q_heads,
                            int batch_count);
cudaError_t decode_attention_gqa16_bf16(const DecodeArgs &args,
                                        cudaStream_t stream);
int decode_balanced_num_splits(int batch_count, int sm_count);

// Key tile of the split kernel for a given KV-head count: split sizes that
// are multiples of it keep every shared-memory stage full.
int decode_stage_tokens(int kv_heads);

struct AppendArgs {
  __nv_bfloat16 *q_prepared = nullptr;
  __nv_bfloat16 *cache_k = nullptr;
  __nv_bfloat16 *cache_v = nullptr;
  Gemma4KvCacheConfig cfg = {};
  const int32_t *page_table = nullptr;
  const int32_t *token_position = nullptr;
  int32_t cache_layer = 0;
  const __nv_bfloat16 *q = nullptr;
  const __nv_bfloat16 *k = nullptr;
  const __nv_bfloat16 *v = nullptr;  // nullptr: V is derived from raw K
  const __nv_bfloat16 *q_norm_weight = nullptr;
  const __nv_bfloat16 *k_norm_weight = nullptr;
  const float *cos = nullptr;
  const float *sin = nullptr;
  int32_t batch_count = 0;
  int32_t q_heads = 0;
  int32_t rotary_dim = 0;
  int32_t norm_mode = B200KV_NORM_RSQRT_APPROX;
  // The raw rows are written by the kernel enqueued just before this call (the
  // QKV projection). Only the fused layer-step needs to be told: it reads raw
  // rows before it waits for its predecessor unless this is set. The append
  // kernels wait before anything else.
  bool raw_from_predecessor = false;
  // How many of the launches that can still be running when this layer-step's
  // kernel starts (with programmatic dependent launch: the ones just before it
  // on the stream) are decode steps of THIS cache layer. Each of them appends
  // the position before the next one's, so the kernel holds back the pages of
  // the newest `steps_in_flight` positions before its own until its predecessor
  // is complete, and streams everything older at once. 0: none of them writes a
  // row of this layer's cache (they are layer-steps of other cache layers).
  // Only the one-launch layer-step (decode_pagetile.cu) makes use of it; the
  // other kernels allow for one such step.
  int32_t steps_in_flight = 1;
  // Let the launch behind this one start as soon as this one runs, instead of
  // when this one's own predecessor is complete. The caller vouches for the
  // launch behind: it is a one-launch layer-step whose steps_in_flight covers
  // every launch that can then still be in flight when it starts (see
  // b200kv_decode_step_bf16). Only the one-launch layer-step makes use of it.
  bool release_early = false;
  // This launch is one of a run whose launches overlap one another that way:
  // the grid is then sized for one CTA per SM instead of two, so that two
  // launches of the run fit on the GPU side by side.
  bool chained = false;
  // The raw K / V rows (nullptr V: derived from raw K) and positions of the
  // `forward_count` decode steps of this cache layer just before this one,
  // nearest first. With forward_count == steps_in_flight the kernel does not
  // wait for those steps' rows to reach the cache: it prepares them itself from
  // the same inputs (the same arithmetic, so the same bits) and puts them where
  // the tiles of the cache would have brought them.
  static constexpr int kMaxForward = 7;
  int32_t forward_count = 0;
  const __nv_bfloat16 *forward_k[kMaxForward] = {};
  const __nv_bfloat16 *forward_v[kMaxForward] = {};
  const int32_t *forward_position[kMaxForward] = {};
};

cudaError_t decode_append_bf16(const AppendArgs &args, cudaStream_t stream);

// Argument checks of the two launches above without the launch
// (cudaSuccess or cudaErrorInvalidValue).
cudaError_t validate_append_args(const AppendArgs &args);
cudaError_t validate_decode_args(const DecodeArgs &args);

// One layer-step in one attention launch (plus the combine): the balanced
// kernel prepares and appends the step's rows itself. Only for the geometry
// decode_fused_supported() accepts; the results are those of
// decode_append_bf16 followed by decode_attention_bf16 with split_size == 0.
bool decode_fused_supported(const AppendArgs &append, const DecodeArgs &decode);
cudaError_t decode_layer_step_fused_bf16(const AppendArgs &append,
                                         const DecodeArgs &decode,
                                         cudaStream_t stream);

// One layer-step (or, with append == nullptr, the attention alone) in a single
// launch: a CTA per (sequence, KV head, key range), TMA tiles of one head's rows,
// the ranges' partials merged by the last CTA of each (sequence, head) through
// `ticket` (uint32 [batch * kv_heads], zero between launches). decode_pagetile.cu.
// _supported: the geometry the kernel is built for (head_dim 256, two query
// heads per KV head, page sizes that tile into 32); _preferred: where the layer-
// step picks it over the balanced partition.
bool decode_pagetile_supported(const Gemma4KvCacheConfig &cfg, int q_heads,
                               int batch_count);
bool decode_pagetile_preferred(const Gemma4KvCacheConfig &cfg, int q_heads,
                               int batch_count, bool has_ticket);
// What the one-launch layer-step needs to finish with the all-gather of its
// output rows over peer memory (peer_gather.cu holds the buffers; world == 0:
// no exchange): every final CTA stores its rows into slot `rank` of every rank's
// buffer, the last of them on this GPU publishes the epoch flag to the peers and
// waits (bounded) for theirs.
struct PeerEpilogue {
  uint4 *data[8];      // rank r's gathered buffer [2][world][slot_packs]
  uint32_t *flags[8];  // rank r's flags [2][world]
  uint32_t *epoch;     // this rank's call counter
  uint32_t *done;      // this rank's count of finished (sequence, head) pairs, zero between calls
  int64_t slot_packs;
  long long wait_clocks;
  int32_t rank;
  int32_t world;
};
// Fills `out` from a peer buffer handle for a call that gathers `bytes` per
// rank and counts the call; cudaErrorInvalidValue if it does not fit.
cudaError_t peer_epilogue_begin(void *handle, int64_t bytes, PeerEpilogue *out);
cudaError_t decode_layer_step_pagetile_bf16(const AppendArgs *append,
                                            const DecodeArgs &decode,
                                            uint32_t *ticket, cudaStream_t stream,
                                            const PeerEpilogue *peer = nullptr);

// Decode projections either side of the KV path (decode_projection.cu), rows of
// one token each; hidden size 3840. Weights are column-major: output column c
// is `width` contiguous bf16 (the reference's *_proj_col_major layout).
struct IngressArgs {
  // out: raw q [rows][q_width], then raw k [rows][k_width], then raw v
  // [rows][cols - q_width - k_width] (one row: the reference's [q|k|v] scratch)
  __nv_bfloat16 *raw_qkv = nullptr;
  const __nv_bfloat16 *x = nullptr;  // [rows][hidden]
  const __nv_bfloat16 *input_norm_weight = nullptr;
  const __nv_bfloat16 *qkv_proj_col_major = nullptr;  // [cols][hidden]
  int32_t rows = 0;
  int32_t hidden = 0;
  int32_t cols = 0;
  int32_t q_width = 0;
  int32_t k_width = 0;
  int32_t norm_mode = B200KV_NORM_RSQRT_APPROX;
  int32_t *status = nullptr;
};
cudaError_t decode_ingress_bf16(const IngressArgs &args, cudaStream_t stream);

struct EgressArgs {
  __nv_bfloat16 *residual_out = nullptr;  // out [rows][hidden]: O projection
  __nv_bfloat16 *normed_out = nullptr;    // out [rows][hidden]
  __nv_bfloat16 *ffn_residual = nullptr;  // out [rows][hidden]
  __nv_bfloat16 *ffn_x = nullptr;         // out, optional
  const __nv_bfloat16 *attention_out = nullptr;  // [rows][attention_width]
  const __nv_bfloat16 *o_proj_col_major = nullptr;  // [hidden][attention_width]
  const __nv_bfloat16 *post_norm_weight = nullptr;
  const __nv_bfloat16 *pre_ffn_norm_weight = nullptr;
  const __nv_bfloat16 *x = nullptr;       // [rows][hidden]: the layer's input
  unsigned int *ticket = nullptr;         // [rows], zero before the first call
  int32_t rows = 0;
  int32_t hidden = 0;
  int32_t attention_width = 0;
  int32_t norm_mode = B200KV_NORM_RSQRT_APPROX;
  int32_t *status = nullptr;
};
cudaError_t decode_egress_bf16(const EgressArgs &args, cudaStream_t stream);

// All-gather of per-rank rows over peer memory (peer_gather.cu), one process
// per GPU. create: allocates this rank's buffer ([2][world][slot_bytes] + flags)
// and fills a 64-byte export for the other ranks; connect: maps the other
// ranks' buffers from their exports ([world][64] bytes, own entry ignored);
// allgather: one kernel on `stream`, *gathered = this rank's [world][slot_bytes]
// view that holds the result once the kernel has run.
cudaError_t peer_buffer_create(int64_t slot_bytes, int world, int rank,
                               void **handle, void *export_64_bytes);
cudaError_t peer_buffer_connect(void *handle, const void *exports);
cudaError_t peer_allgather(void *handle, const void *src, int64_t bytes,
                           int32_t *status, cudaStream_t stream,
                           void **gathered);
// Key-range sharding: every rank passes its normalised rows `out`
// [rows][head_dim] bf16 with their log-sum-exp `lse` [rows]; every rank gets
// the merged rows (merged_out may be `out`) and, optionally, the merged lse.
// slot_bytes >= rows * (head_dim * 2 + 4); rows <= 64.
cudaError_t peer_merge_attention(void *handle, __nv_bfloat16 *merged_out,
                                 float *merged_lse, const __nv_bfloat16 *out,
                                 const float *lse, int32_t rows, int32_t head_dim,
                                 int32_t *status, cudaStream_t stream);
cudaError_t peer_buffer_destroy(void *handle);
// One-GPU stand-in (every peer's buffer is a local allocation nobody writes),
// the wait limit of later calls, a flag posted from the host in a peer's name,
// and the re-synchronisation after a rank missed a call (peer_gather.cu).
cudaError_t peer_buffer_create_loopback(int64_t slot_bytes, int world, int rank,
                                        void **handle);
cudaError_t peer_buffer_set_wait_clocks(void *handle, long long clocks);
cudaError_t peer_buffer_post(void *handle, int from_rank, uint32_t epoch,
                             cudaStream_t stream);
cudaError_t peer_buffer_reset(void *handle);
// The half of the gathered buffer the most recent call filled ([world][slot_bytes]).
cudaError_t peer_buffer_gathered(void *handle, void **gathered);
// One warp waits on an mbarrier that nothing arrives at, with the bounded wait
// every kernel of the library uses, for `clock_limit` SM clocks (bounded_wait.cu).
cudaError_t bounded_wait_selftest(long long clock_limit, int32_t *status,
                                  long long *waited_clocks, cudaStream_t stream);

struct PrefillPrepArgs {
  __nv_bfloat16 *q_prepared = nullptr;
  __nv_bfloat16 *k_prepared = nullptr;
  __nv_bfloat16 *v_prepared = nullptr;
  const __nv_bfloat16 *q = nullptr;
  const __nv_bfloat16 *k = nullptr;
  const __nv_bfloat16 *v = nullptr;  // nullptr: V is derived from raw K
  const __nv_bfloat16 *q_norm_weight = nullptr;
  const __nv_bfloat16 *k_norm_weight = nullptr;
  const float *cos = nullptr;
  const float *sin = nullptr;
  const int32_t *token_position = nullptr;
  int64_t rows = 0;
  int32_t q_heads = 0;
  int32_t kv_heads = 0;
  int32_t head_dim = 0;
  int32_t rotary_dim = 0;
  int32_t norm_mode = B200KV_NORM_RSQRT_APPROX;
};

cudaError_t prefill_prep_bf16(const PrefillPrepArgs &args,
                              cudaStream_t stream);

// Causal (+ sliding window) attention of every sequence over its own prepared
// rows (prefill_attention.cu); window 0 = causal only; head_dim 256 or 512.
cudaError_t prefill_attention_bf16(__nv_bfloat16 *out, const __nv_bfloat16 *q,
                                   const __nv_bfloat16 *k, const __nv_bfloat16 *v,
                                   int batch, int seq_len, int q_heads,
                                   int kv_heads, int head_dim, int window,
                                   float softmax_scale, cudaStream_t stream);
// The same on tcgen05 tensor cores with accumulators in tensor memory
// (prefill_attention_sm100.cu), head_dim 256 or 512; arguments already validated
// by the caller.
cudaError_t prefill_attention_sm100_bf16(__nv_bfloat16 *out,
                                         const __nv_bfloat16 *q,
                                         const __nv_bfloat16 *k,
                                         const __nv_bfloat16 *v, int batch,
                                         int seq_len, int q_heads, int kv_heads,
                                         int head_dim, int window,
                                         float softmax_scale, cudaStream_t stream);
// Synchronises; 0, or which wait of the last launch of that kernel ran out.
int prefill_attention_sm100_fault();

// FP8 e4m3 cache (fp8_cache.cu). args.cache_k / cache_v are unused.
cudaError_t decode_append_fp8(const AppendArgs &args, uint8_t *cache_k,
                              uint8_t *cache_v, float *scale_k, float *scale_v,
                              cudaStream_t stream);
cudaError_t fp8_append_rows(uint8_t *cache_k, uint8_t *cache_v, float *scale_k,
                            float *scale_v, Gemma4KvCacheConfig config,
                            const int32_t *page_table, const int32_t *seq_batch,
                            const int32_t *first_position,
                            const int32_t *row_count, const int32_t *row_start,
                            int32_t seq_count, int32_t max_row_count,
                            int32_t layer, const __nv_bfloat16 *k,
                            const __nv_bfloat16 *v, cudaStream_t stream);

cudaError_t kv_cache_write_bf16(__nv_bfloat16 *cache_k, __nv_bfloat16 *cache_v,
                                Gemma4KvCacheConfig config,
                                const int32_t *page_table,
                                const int32_t *token_batch,
                                const int32_t *token_position,
                                int32_t token_count, int32_t layer,
                                const __nv_bfloat16 *k, const __nv_bfloat16 *v,
                                cudaStream_t stream);

// Cache fill after a prompt of batch_size x seq_len prepared rows (row
// b * seq_len + t is token t of sequence b): one launch that writes every row,
// or for a sliding cache and a prompt longer than its window only the last
// window_size rows of each sequence.
cudaError_t prefill_cache_fill_bf16(__nv_bfloat16 *cache_k,
                                    __nv_bfloat16 *cache_v,
                                    Gemma4KvCacheConfig config,
                                    const int32_t *page_table,
                                    const int32_t *token_batch,
                                    const int32_t *token_position,
                                    int32_t batch_size, int32_t seq_len,
                                    int32_t layer, const __nv_bfloat16 *k,
                                    const __nv_bfloat16 *v, cudaStream_t stream);

}  // namespace b200kv

// CPU oracle for the gemma.c KV-cache hot path (append + paged/ring cache +
// split-KV decode attention).
//
// TEST INFRASTRUCTURE ONLY. This is a plain host restatement of the reference
// algorithm used as the checker in tests, in the smoke run and as the timed
// CPU baseline of the benchmark. No product code may call into it.
//
// Every function cites the reference file:line it follows (paths are relative
// to the gemma.c project root).
//
// Parity pinning: the reference ships no numerical test of the decode split /
// reduce phases nor of the fused decode append; the restatement is pinned
//   (1) against the reference's own tests that do touch this path
//       (tests/test_kv_cache.cu, tests/test_runtime_state.cu,
//        tests/test_flash_attention.cu prep semantics), restated in
//       tests/test_oracle_pins.py, and
//   (2) against outputs of the reference's own CUDA kernels compiled from the
//       reference sources (oracle/_ref) and run on a B200; those outputs are
//       committed as fixtures under tests/golden/.
#pragma once

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// Mirror of Gemma4KvCacheConfig (src/gemma4_kv_cache.cuh:9-18): 8 x int32.
typedef struct OrcKvConfig {
  int32_t num_layers;
  int32_t num_pages;
  int32_t page_size;
  int32_t max_pages_per_seq;
  int32_t batch_size;
  int32_t num_heads;
  int32_t head_dim;
  int32_t window_size;
} OrcKvConfig;

// ---- scalar helpers -------------------------------------------------------
uint16_t orc_f32_to_bf16(float x);
float orc_bf16_to_f32(uint16_t x);
void orc_f32_to_bf16_n(uint16_t *out, const float *in, int64_t n);
void orc_bf16_to_f32_n(float *out, const uint16_t *in, int64_t n);
uint8_t orc_f32_to_e4m3(float x);
float orc_e4m3_to_f32(uint8_t x);

// ---- geometry / host paging (kv_cache.cuh:28-38, kv_cache.cu:76-146) -----
int64_t orc_cache_offset(const OrcKvConfig *cfg, int32_t layer, int32_t page,
                         int32_t page_offset, int32_t head, int32_t dim);
void orc_make_config(OrcKvConfig *out, int32_t global, int32_t num_pages,
                     int32_t page_size, int32_t max_pages_per_seq);
int32_t orc_is_global_layer(int32_t model_layer);
int32_t orc_layer_index(int32_t model_layer, int32_t global_cache);
int32_t orc_ensure_page(int32_t *page_table, int32_t *slot_logical_pages,
                        const OrcKvConfig *cfg, int32_t batch,
                        int32_t position);
int32_t orc_ensure_range(int32_t *page_table, int32_t *slot_logical_pages,
                         const OrcKvConfig *cfg, int32_t batch,
                         int32_t first_position, int32_t token_count);
int32_t orc_sliding_pages_per_sequence(int32_t max_seq_len, int32_t page_size);

// ---- runtime state bookkeeping (runtime.cu:95-341), host arrays only -----
typedef struct OrcRuntime OrcRuntime;
OrcRuntime *orc_runtime_create(int32_t batch_size, int32_t max_seq_len,
                               int32_t page_size);
void orc_runtime_destroy(OrcRuntime *rt);
int32_t orc_runtime_prepare_prefill(OrcRuntime *rt, int32_t seq_len);
int32_t orc_runtime_prepare_decode_step(OrcRuntime *rt);
// which: 0 sliding page table, 1 global page table, 2 sliding slot pages,
// 3 global slot pages, 4 seq_lengths, 5 token_batch, 6 token_position.
int64_t orc_runtime_array(OrcRuntime *rt, int32_t which, int32_t **data);
void orc_runtime_configs(OrcRuntime *rt, OrcKvConfig *sliding,
                         OrcKvConfig *global, int32_t *token_count);

// ---- RoPE tables (runtime.cu:27-45) ---------------------------------------
void orc_fill_rope_tables(float *cos_table, float *sin_table,
                          int32_t max_seq_len, int32_t rotary_half,
                          float theta, int32_t exponent_dim);

// ---- prep (decode.cu:216-280, rmsnorm.cu:90-101, rope.cu:8-20) ------------
float orc_rms_scale(const uint16_t *head, int32_t head_dim, float eps);
void orc_prep_weighted_rope_head(uint16_t *out, const uint16_t *in,
                                 const uint16_t *weight, const float *cos_row,
                                 const float *sin_row, int32_t head_dim,
                                 int32_t rotary_dim);
void orc_prep_scale_free_head(uint16_t *out, const uint16_t *in,
                              int32_t head_dim);
// Whole-prompt prep into contiguous tensors (prefill.cu:1022-1081).
void orc_prefill_prep(uint16_t *q_prepared, uint16_t *k_prepared,
                      uint16_t *v_prepared, const uint16_t *q,
                      const uint16_t *k, const uint16_t *v,
                      const uint16_t *q_w, const uint16_t *k_w,
                      const float *cos_table, const float *sin_table,
                      const int32_t *token_position, int64_t rows,
                      int32_t q_heads, int32_t kv_heads, int32_t head_dim,
                      int32_t rotary_dim, int32_t has_v_proj);

// ---- cache write (kv_cache.cu:11-71,149-180) ------------------------------
int32_t orc_kv_cache_write(uint16_t *cache_k, uint16_t *cache_v,
                           const OrcKvConfig *cfg, const int32_t *page_table,
                           const int32_t *token_batch,
                           const int32_t *token_position, int32_t token_count,
                           int32_t layer, const uint16_t *k,
                           const uint16_t *v);

// ---- fused decode append (decode.cu:285-375) ------------------------------
void orc_decode_append(uint16_t *q_prepared, uint16_t *cache_k,
                       uint16_t *cache_v, const OrcKvConfig *cfg,
                       const int32_t *page_table,
                       const int32_t *token_position, int32_t cache_layer,
                       const uint16_t *q, const uint16_t *k,
                       const uint16_t *v, const uint16_t *q_w,
                       const uint16_t *k_w, const float *cos_table,
                       const float *sin_table, int32_t batch_count,
                       int32_t q_heads, int32_t rotary_dim,
                       int32_t has_v_proj);

// ---- decode attention -----------------------------------------------------
// Reference-order restatement (decode.cu:530-542,692-977): per split a
// sequential fp32 online softmax, partials in scratch, LSE-style reduce.
// partial_* may be NULL when num_splits == 1.
void orc_decode_attention_ref(uint16_t *out, float *partial_m,
                              float *partial_l, float *partial_acc,
                              const uint16_t *q, const uint16_t *cache_k,
                              const uint16_t *cache_v,
                              const int32_t *page_table,
                              const int32_t *seq_lengths,
                              const OrcKvConfig *cfg, int32_t layer,
                              float softmax_scale, int32_t split_size,
                              int32_t num_splits, int32_t batch_count,
                              int32_t q_heads);
// Double-precision direct softmax over the same live keys; writes fp32 output
// (not rounded) and the natural-log LSE of the scaled scores (-inf when no
// key is live). Used for tolerance bands.
void orc_decode_attention_f64(float *out_f32, float *lse,
                              const uint16_t *q, const uint16_t *cache_k,
                              const uint16_t *cache_v,
                              const int32_t *page_table,
                              const int32_t *seq_lengths,
                              const OrcKvConfig *cfg, int32_t layer,
                              float softmax_scale, int32_t batch_count,
                              int32_t q_heads);

// ---- FP8 e4m3 cache with one fp32 scale per (page, kv head) ---------------
// No counterpart in the reference; this file defines the rule.
// scale_* are [num_layers, num_pages, num_heads] fp32, zero before first use.
// Byte index of a K element in the fp8 cache (half-page blocks, head-major,
// swizzled rows); V uses orc_cache_offset.
int64_t orc_fp8_k_index(const OrcKvConfig *cfg, int32_t layer, int32_t page,
                        int32_t token, int32_t head, int32_t dim);
void orc_fp8_append(uint8_t *cache_k, uint8_t *cache_v, float *scale_k,
                    float *scale_v, const OrcKvConfig *cfg,
                    const int32_t *page_table, const int32_t *seq_batch,
                    const int32_t *first_position, const int32_t *row_count,
                    int32_t seq_count, int32_t layer,
                    const uint16_t *k_prepared, const uint16_t *v_prepared);
void orc_fp8_decode_attention_f64(float *out_f32, float *lse,
                                  const uint16_t *q, const uint8_t *cache_k,
                                  const uint8_t *cache_v,
                                  const float *scale_k, const float *scale_v,
                                  const int32_t *page_table,
                                  const int32_t *seq_lengths,
                                  const OrcKvConfig *cfg, int32_t layer,
                                  float softmax_scale, int32_t batch_count,
                                  int32_t q_heads);

// ---- prompt attention (prefill.cu:502-540,1110-1257): causal (+ window) over
// contiguous prepared rows q [batch*seq, q_heads, D], k/v [batch*seq, kv_heads, D];
// double precision; fp32 output, natural-log LSE (may be NULL).
void orc_prefill_attention_f64(float *out_f32, float *lse, const uint16_t *q,
                               const uint16_t *k, const uint16_t *v,
                               int32_t batch, int32_t seq_len, int32_t q_heads,
                               int32_t kv_heads, int32_t head_dim,
                               int32_t window, float softmax_scale,
                               int32_t threads);

// ---- decode projections either side of the KV path -------------------------
// (decode.cu:35-129 O projection + post-attention norm + residual;
//  decode.cu:395-496 input RMSNorm + [Q|K|V] projection; rmsnorm.cu:27-87).
// Weights are column-major: column c is `width` contiguous bf16. Sums follow
// the 512-thread block's order; `threads` are host threads over columns.
void orc_hidden_rmsnorm(uint16_t *out, const uint16_t *in,
                        const uint16_t *weight, int32_t width);
void orc_project_cols(uint16_t *out, const uint16_t *x,
                      const uint16_t *w_col_major, int32_t width, int32_t cols,
                      int32_t active_threads, int32_t threads);
// normed (the bf16 normed row, [hidden]) may be NULL.
void orc_decode_ingress(uint16_t *raw_qkv, uint16_t *normed, const uint16_t *x,
                        const uint16_t *input_norm_weight,
                        const uint16_t *qkv_proj_col_major, int32_t hidden,
                        int32_t cols, int32_t threads);
// ffn_x may be NULL (then pre_ffn_norm_weight is unused).
void orc_decode_egress(uint16_t *residual_out, uint16_t *normed_out,
                       uint16_t *ffn_residual, uint16_t *ffn_x,
                       const uint16_t *attention_out,
                       const uint16_t *o_proj_col_major,
                       const uint16_t *post_norm_weight,
                       const uint16_t *pre_ffn_norm_weight, const uint16_t *x,
                       int32_t attention_width, int32_t hidden,
                       int32_t threads);

// ---- timed CPU baseline: one layer-step (append + attention + reduce) -----
// Runs orc_decode_append then the reference-order attention with `threads`
// host threads over (sequence, kv head) units. Returns seconds of wall time.
double orc_layer_step_timed(int32_t threads, uint16_t *out,
                            uint16_t *q_prepared, uint16_t *cache_k,
                            uint16_t *cache_v, const OrcKvConfig *cfg,
                            const int32_t *page_table,
                            const int32_t *token_position,
                            const int32_t *seq_lengths, int32_t cache_layer,
                            const uint16_t *q, const uint16_t *k,
                            const uint16_t *v, const uint16_t *q_w,
                            const uint16_t *k_w, const float *cos_table,
                            const float *sin_table, int32_t batch_count,
                            int32_t q_heads, float softmax_scale,
                            int32_t split_size);
int32_t orc_hardware_threads(void);

#ifdef __cplusplus
}
#endif

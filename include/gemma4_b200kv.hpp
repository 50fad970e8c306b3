// C++ host interface of libgemma4_b200kv.so, source-compatible with the
// declarations a gemma.c translation unit gets from
//   src/gemma4_kv_cache.cuh:9-66        (config, offset, page helpers, cache write)
//   src/gemma4_runtime.cuh:12-64        (Gemma4RuntimeState and its four functions)
//   src/gemma4_flash_attention.cuh:9-45 (prompt attention entry points)
// so that code written against those headers builds against this one and
// links to the B200 library instead of gemma4_kv_cache.cu / gemma4_runtime.cu /
// gemma4_flash_attention_prefill.cu. Two ways to use it:
//   * instead of the reference's headers: include it directly, or put
//     include/compat (files named like the reference's, forwarding here) ahead
//     of gemma.c's src/ on the include path;
//   * on top of them, in a translation unit that already sees gemma.c's own
//     headers (anything inside gemma.c's src/, e.g. the decode layer loop):
//     define GEMMA4_B200KV_USE_REFERENCE_HEADERS before including it; the types
//     and functions then come from the reference's headers and this file only
//     adds the layout checks and the library's extra entry points.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <stddef.h>
#include <stdint.h>
#include <vector>

#define GEMMA4_KV_CACHE_CONFIG_DEFINED
#define GEMMA4_B200KV_TYPED_CACHE_WRITE
#if defined(GEMMA4_B200KV_USE_REFERENCE_HEADERS)
#include "gemma4_flash_attention.cuh"
#include "gemma4_kv_cache.cuh"
#include "gemma4_runtime.cuh"
#include "gemma4_b200kv.h"
#else
struct Gemma4KvCacheConfig {
  int32_t num_layers;
  int32_t num_pages;
  int32_t page_size;
  int32_t max_pages_per_seq;
  int32_t batch_size;
  int32_t num_heads;
  int32_t head_dim;
  int32_t window_size;
};

#include "gemma4_b200kv.h"

// src/gemma4_kv_cache.cuh:55-66, same symbol as the C declaration.
extern "C" cudaError_t gemma4_kv_cache_write_bf16(
    __nv_bfloat16 *__restrict__ d_cache_k,
    __nv_bfloat16 *__restrict__ d_cache_v, Gemma4KvCacheConfig config,
    const int32_t *__restrict__ d_page_table,
    const int32_t *__restrict__ d_token_batch,
    const int32_t *__restrict__ d_token_position, int32_t token_count,
    int32_t layer, const __nv_bfloat16 *__restrict__ d_k,
    const __nv_bfloat16 *__restrict__ d_v, cudaStream_t stream);

// src/gemma4_flash_attention.cuh:9-45: prompt attention with the norm + RoPE
// prep fused in front. Same names, argument order and error behaviour; rows are
// batch * seq_len + t, q / out [row, 16, D], k / v [row, kv_heads, D] with
// 8 KV heads x 256 (sliding) or 1 KV head x 512, rotary 128, V from K (global).
cudaError_t gemma4_flash_attention_sliding_fwd_bf16_norm_rope(
    __nv_bfloat16 *__restrict__ d_out, __nv_bfloat16 *__restrict__ d_q_prepared,
    __nv_bfloat16 *__restrict__ d_k_prepared,
    __nv_bfloat16 *__restrict__ d_v_prepared, const __nv_bfloat16 *__restrict__ d_q,
    const __nv_bfloat16 *__restrict__ d_k, const __nv_bfloat16 *__restrict__ d_v,
    const __nv_bfloat16 *__restrict__ d_q_norm_weight,
    const __nv_bfloat16 *__restrict__ d_k_norm_weight,
    const float *__restrict__ d_cos, const float *__restrict__ d_sin,
    const int32_t *__restrict__ d_token_position, int batch_size, int seqlen_q,
    int seqlen_k, int window_size, float softmax_scale, cudaStream_t stream);

cudaError_t gemma4_flash_attention_global_fwd_bf16_norm_rope(
    __nv_bfloat16 *__restrict__ d_out, __nv_bfloat16 *__restrict__ d_q_prepared,
    __nv_bfloat16 *__restrict__ d_k_prepared,
    __nv_bfloat16 *__restrict__ d_v_prepared, const __nv_bfloat16 *__restrict__ d_q,
    const __nv_bfloat16 *__restrict__ d_k,
    const __nv_bfloat16 *__restrict__ d_q_norm_weight,
    const __nv_bfloat16 *__restrict__ d_k_norm_weight,
    const float *__restrict__ d_cos, const float *__restrict__ d_sin,
    const int32_t *__restrict__ d_token_position, int batch_size, int seqlen_q,
    int seqlen_k, float softmax_scale, cudaStream_t stream);

// src/gemma4_kv_cache.cu:76-91
Gemma4KvCacheConfig gemma4_kv_cache_make_config(bool global, int32_t num_pages,
                                                int32_t page_size,
                                                int32_t max_pages_per_seq);

// src/gemma4_kv_cache.cu:94-105
int32_t gemma4_kv_cache_layer_index(int32_t model_layer, bool global_cache);

// src/gemma4_kv_cache.cuh:28-38: flat offset into
// [layer, page, page_offset, head, dim].
__host__ __device__ constexpr inline int64_t gemma4_kv_cache_offset(
    const Gemma4KvCacheConfig &config, int32_t layer, int32_t page,
    int32_t page_offset, int32_t head, int32_t dim) {
  return (((int64_t(layer) * config.num_pages + page) * config.page_size +
           page_offset) *
              config.num_heads +
          head) *
             config.head_dim +
         dim;
}

// src/gemma4_kv_cache.cu:108-123
int32_t gemma4_kv_cache_ensure_page(std::vector<int32_t> &page_table,
                                    std::vector<int32_t> &slot_logical_pages,
                                    const Gemma4KvCacheConfig &config,
                                    int32_t batch, int32_t position);

// src/gemma4_kv_cache.cu:126-146
int32_t gemma4_kv_cache_ensure_range(std::vector<int32_t> &page_table,
                                     std::vector<int32_t> &slot_logical_pages,
                                     const Gemma4KvCacheConfig &config,
                                     int32_t batch, int32_t first_position,
                                     int32_t token_count);

// src/gemma4_runtime.cuh:12-42: the same members, types, order and default
// initialisers, nothing added, so that an object a gemma.c translation unit
// built against the reference's header has exactly the size and layout the
// library writes (static_asserts below).
struct Gemma4RuntimeState {
  int32_t batch_size = 0;
  int32_t max_seq_len = 0;
  int32_t page_size = 0;
  int32_t token_count = 0;

  Gemma4KvCacheConfig sliding_cache_config = {};
  Gemma4KvCacheConfig global_cache_config = {};
  __nv_bfloat16 *sliding_cache_k = nullptr;
  __nv_bfloat16 *sliding_cache_v = nullptr;
  __nv_bfloat16 *global_cache_k = nullptr;
  __nv_bfloat16 *global_cache_v = nullptr;

  int32_t *sliding_page_table = nullptr;
  int32_t *global_page_table = nullptr;
  int32_t *seq_lengths = nullptr;
  int32_t *token_batch = nullptr;
  int32_t *token_position = nullptr;
  float *sliding_cos = nullptr;
  float *sliding_sin = nullptr;
  float *global_cos = nullptr;
  float *global_sin = nullptr;

  std::vector<int32_t> h_sliding_page_table;
  std::vector<int32_t> h_global_page_table;
  std::vector<int32_t> h_sliding_slot_logical_pages;
  std::vector<int32_t> h_global_slot_logical_pages;
  std::vector<int32_t> h_seq_lengths;
  std::vector<int32_t> h_token_batch;
  std::vector<int32_t> h_token_position;
};

#endif  // GEMMA4_B200KV_USE_REFERENCE_HEADERS

// The reference's layout on an LP64 host: four int32, two 32-byte configs,
// thirteen pointers, seven std::vector (three pointers each).
static_assert(sizeof(Gemma4KvCacheConfig) == 32, "src/gemma4_kv_cache.cuh:9-18");
static_assert(offsetof(Gemma4RuntimeState, sliding_cache_config) == 16 &&
                  offsetof(Gemma4RuntimeState, global_cache_config) == 48 &&
                  offsetof(Gemma4RuntimeState, sliding_cache_k) == 80 &&
                  offsetof(Gemma4RuntimeState, sliding_page_table) == 112 &&
                  offsetof(Gemma4RuntimeState, global_sin) == 176 &&
                  offsetof(Gemma4RuntimeState, h_sliding_page_table) == 184 &&
                  offsetof(Gemma4RuntimeState, h_token_position) ==
                      184 + 6 * sizeof(std::vector<int32_t>) &&
                  sizeof(Gemma4RuntimeState) ==
                      184 + 7 * sizeof(std::vector<int32_t>),
              "Gemma4RuntimeState must keep the layout of src/gemma4_runtime.cuh:12-42");

// src/gemma4_runtime.cu:95-234. `state` must be zero-initialised or freed.
cudaError_t gemma4_runtime_state_init(Gemma4RuntimeState *state,
                                      int32_t batch_size, int32_t max_seq_len,
                                      int32_t page_size, cudaStream_t stream);
// Same, for caches of another geometry (the state does not record it: the two
// cache configs carry everything the other functions need).
cudaError_t gemma4_runtime_state_init_geometry(
    Gemma4RuntimeState *state, int32_t batch_size, int32_t max_seq_len,
    int32_t page_size, const B200KvRuntimeGeometry &geometry,
    cudaStream_t stream);
// src/gemma4_runtime.cu:77-92
void gemma4_runtime_state_free(Gemma4RuntimeState *state);
// src/gemma4_runtime.cu:237-273
cudaError_t gemma4_runtime_prepare_prefill(Gemma4RuntimeState *state,
                                           int32_t seq_len,
                                           cudaStream_t stream);
// src/gemma4_runtime.cu:276-341
cudaError_t gemma4_runtime_prepare_decode_step(Gemma4RuntimeState *state,
                                               cudaStream_t stream);

// The attention half of gemma4_decode_megakernel_flash_attention_layer_bf16
// (src/gemma4_flash_attention_decode.cu:1122-1157), called from the layer loop
// of gemma4_decode_megakernel (src/gemma4_decode_megakernel.cu:172-183) with
// the reference's own per-layer argument struct: `LayerArgs` is any type with
// the attention_* / residual_out / normed_out / ffn_residual / ffn_x members of
// Gemma4DecodeMegakernelLayerArgs (src/gemma4_megakernel.cuh:32-66), which this
// header therefore does not need to see. Enqueues input norm + QKV projection,
// append + decode attention + combine, O projection + post-attention norm +
// residual + pre-FFN norm on `stream`; the caller's FFN launch follows.
// `raw_qkv_scratch`: 8704 bf16 per row (the reference reuses attention_out /
// attention_q for it; here it is a buffer of its own); `ticket`: uint32
// [batch_count * (1 + KV heads * B200KV_TICKETS_PER_HEAD)], zero before the
// first call and left zero by every call (one word per row for the O
// projection's last-CTA epilogue, then the one-launch attention's tickets). Geometry as the reference derives it from
// the cache config: 8 KV heads x 256 (sliding, own V projection, rotary 256) or
// 1 KV head x 512 (global, V from raw K, rotary 128), 16 query heads.
template <class LayerArgs>
inline cudaError_t gemma4_b200kv_decode_attention_layer(
    const LayerArgs &args, __nv_bfloat16 *raw_qkv_scratch, uint32_t *ticket,
    int32_t batch_count, cudaStream_t stream, int32_t *status = nullptr) {
  const Gemma4KvCacheConfig &cfg = args.attention_cache_config;
  const bool global_geometry = cfg.head_dim == 512 && cfg.num_heads == 1;
  if (!global_geometry && !(cfg.head_dim == 256 && cfg.num_heads == 8)) {
    return cudaErrorInvalidValue;  // as the reference's dispatch, decode.cu:1126-1156
  }
  auto bits = [](auto *p) {
    return reinterpret_cast<b200kv_bf16 *>(const_cast<__nv_bfloat16 *>(p));
  };
  B200KvAttentionLayerArgs a = {};
  a.kv.q = bits(args.attention_q);
  a.kv.out = bits(args.attention_out);
  a.kv.partial_m = args.attention_partial_m;
  a.kv.partial_l = args.attention_partial_l;
  a.kv.partial_acc = args.attention_partial_acc;
  a.kv.cache_k = bits(args.attention_cache_k);
  a.kv.cache_v = bits(args.attention_cache_v);
  a.kv.cache_config = cfg;
  a.kv.page_table = args.attention_page_table;
  a.kv.token_position = args.attention_token_position;
  a.kv.seq_lengths = args.attention_seq_lengths;
  a.kv.cache_layer = args.attention_cache_layer;
  a.kv.split_size = args.attention_split_size;
  a.kv.num_splits = args.attention_num_splits;
  a.kv.softmax_scale = args.attention_softmax_scale;
  a.kv.q_norm_weight = bits(args.attention_q_norm_weight);
  a.kv.k_norm_weight = bits(args.attention_k_norm_weight);
  a.kv.cos = args.attention_cos;
  a.kv.sin = args.attention_sin;
  a.kv.batch_count = batch_count;
  a.kv.q_heads = 16;
  a.kv.rotary_dim = global_geometry ? 128 : 256;
  a.kv.norm_mode = B200KV_NORM_RSQRT_APPROX;
  a.kv.status = status;
  a.kv.ticket = ticket != nullptr ? ticket + batch_count : nullptr;
  a.attention_x = bits(args.attention_x);
  a.attention_input_norm_weight = bits(args.attention_input_norm_weight);
  a.attention_qkv_proj_col_major = bits(args.attention_qkv_proj_col_major);
  a.attention_o_proj_col_major = bits(args.attention_o_proj_col_major);
  a.attention_post_norm_weight = bits(args.attention_post_norm_weight);
  a.attention_pre_ffn_norm_weight = bits(args.attention_pre_ffn_norm_weight);
  a.raw_qkv = bits(raw_qkv_scratch);
  a.residual_out = bits(args.residual_out);
  a.normed_out = bits(args.normed_out);
  a.ffn_residual = bits(args.ffn_residual);
  a.ffn_x = bits(args.ffn_x);
  a.ticket = ticket;
  a.hidden_size = 3840;
  a.has_v_projection = global_geometry ? 0 : 1;
  return static_cast<cudaError_t>(b200kv_decode_attention_layer_bf16(&a, stream));
}

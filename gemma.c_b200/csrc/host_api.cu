// Host side of libgemma4_b200kv.so: geometry and page bookkeeping, the runtime
// state that owns caches and per-step metadata, launch planning, and the
// extern "C" boundary. The device work lives in append_prep.cu and
// decode_attention.cu; nothing here computes on the CPU what a kernel is
// meant to compute.
#include "common.cuh"
#include "kernels.cuh"

#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <new>
#include <vector>

namespace {

// Model constants of the reference (src/gemma4.h:8-29).
constexpr int kNumLayers = 48;
constexpr int kGlobalLayerPeriod = 6;
constexpr int kGlobalLayerCount =
    kNumLayers / kGlobalLayerPeriod + (kNumLayers % kGlobalLayerPeriod ? 1 : 0);
constexpr int kSlidingLayerCount = kNumLayers - kGlobalLayerCount;
constexpr int kMaxPositions = 262144;

constexpr bool is_global_layer(int32_t layer) {
  return layer == kNumLayers - 1 || (layer + 1) % kGlobalLayerPeriod == 0;
}

B200KvRuntimeGeometry default_geometry() {
  B200KvRuntimeGeometry g;
  g.sliding_layers = kSlidingLayerCount;
  g.sliding_kv_heads = 8;
  g.sliding_head_dim = 256;
  g.sliding_window = 1024;
  g.sliding_rotary_dim = 256;
  g.sliding_rope_theta = 10000.0f;
  g.global_layers = kGlobalLayerCount;
  g.global_kv_heads = 1;
  g.global_head_dim = 512;
  g.global_rotary_dim = 128;  // partial rotary factor 0.25
  g.global_rope_theta = 1000000.0f;
  g.global_rope_exponent_dim = 512;
  return g;
}

size_t cache_elements(const Gemma4KvCacheConfig &c) {
  return size_t(c.num_layers) * c.num_pages * c.page_size * c.num_heads *
         c.head_dim;
}

int32_t sliding_pages(int32_t max_seq_len, int32_t page_size, int32_t window) {
  // src/gemma4_runtime.cu:18-24: a live window may straddle one extra page.
  if (max_seq_len <= window) return b200kv::div_up(max_seq_len, page_size);
  return b200kv::div_up(window + page_size - 1, page_size);
}

void fill_rope(std::vector<float> &cos_t, std::vector<float> &sin_t,
               int32_t max_seq_len, int32_t rotary_half, float theta,
               int32_t exponent_dim) {
  cos_t.resize(size_t(max_seq_len) * rotary_half);
  sin_t.resize(cos_t.size());
  b200kv_fill_rope_tables(cos_t.data(), sin_t.data(), max_seq_len, rotary_half,
                          theta, exponent_dim);
}

template <typename T>
cudaError_t upload(T *dst, const std::vector<T> &src, size_t count,
                   cudaStream_t stream) {
  if (count == 0) return cudaSuccess;
  return cudaMemcpyAsync(dst, src.data(), count * sizeof(T),
                         cudaMemcpyHostToDevice, stream);
}

#define B200KV_TRY(expr)                        \
  do {                                          \
    const cudaError_t b200kv_st__ = (expr);     \
    if (b200kv_st__ != cudaSuccess) return b200kv_st__; \
  } while (0)

cudaError_t upload_all_metadata(Gemma4RuntimeState *s, size_t token_count,
                                cudaStream_t stream) {
  B200KV_TRY(upload(s->sliding_page_table, s->h_sliding_page_table,
                    s->h_sliding_page_table.size(), stream));
  B200KV_TRY(upload(s->global_page_table, s->h_global_page_table,
                    s->h_global_page_table.size(), stream));
  B200KV_TRY(upload(s->seq_lengths, s->h_seq_lengths, s->h_seq_lengths.size(),
                    stream));
  B200KV_TRY(upload(s->token_batch, s->h_token_batch, token_count, stream));
  return upload(s->token_position, s->h_token_position, token_count, stream);
}

}  // namespace

// ===========================================================================
// C++ interface (names and behaviour of the reference's host functions)
// ===========================================================================

Gemma4KvCacheConfig gemma4_kv_cache_make_config(bool global, int32_t num_pages,
                                                int32_t page_size,
                                                int32_t max_pages_per_seq) {
  const B200KvRuntimeGeometry g = default_geometry();
  Gemma4KvCacheConfig c;
  c.num_layers = global ? g.global_layers : g.sliding_layers;
  c.num_pages = num_pages;
  c.page_size = page_size;
  c.max_pages_per_seq = max_pages_per_seq;
  c.batch_size = num_pages / max_pages_per_seq;
  c.num_heads = global ? g.global_kv_heads : g.sliding_kv_heads;
  c.head_dim = global ? g.global_head_dim : g.sliding_head_dim;
  c.window_size = global ? 0 : g.sliding_window;
  return c;
}

int32_t gemma4_kv_cache_layer_index(int32_t model_layer, bool global_cache) {
  if (model_layer < 0 || model_layer >= kNumLayers) return -1;
  if (is_global_layer(model_layer) != global_cache) return -1;
  int32_t index = 0;
  for (int32_t layer = 0; layer < model_layer; ++layer) {
    index += is_global_layer(layer) == global_cache ? 1 : 0;
  }
  return index;
}

int32_t gemma4_kv_cache_ensure_page(std::vector<int32_t> &page_table,
                                    std::vector<int32_t> &slot_logical_pages,
                                    const Gemma4KvCacheConfig &config,
                                    int32_t batch, int32_t position) {
  return b200kv_ensure_page(page_table.data(), slot_logical_pages.data(),
                            &config, batch, position);
}

int32_t gemma4_kv_cache_ensure_range(std::vector<int32_t> &page_table,
                                     std::vector<int32_t> &slot_logical_pages,
                                     const Gemma4KvCacheConfig &config,
                                     int32_t batch, int32_t first_position,
                                     int32_t token_count) {
  return b200kv_ensure_range(page_table.data(), slot_logical_pages.data(),
                             &config, batch, first_position, token_count);
}

void gemma4_runtime_state_free(Gemma4RuntimeState *state) {
  cudaFree(state->sliding_cache_k);
  cudaFree(state->sliding_cache_v);
  cudaFree(state->global_cache_k);
  cudaFree(state->global_cache_v);
  cudaFree(state->sliding_page_table);
  cudaFree(state->global_page_table);
  cudaFree(state->seq_lengths);
  cudaFree(state->token_batch);
  cudaFree(state->token_position);
  cudaFree(state->sliding_cos);
  cudaFree(state->sliding_sin);
  cudaFree(state->global_cos);
  cudaFree(state->global_sin);
  *state = Gemma4RuntimeState();
}

cudaError_t gemma4_runtime_state_init_geometry(
    Gemma4RuntimeState *state, int32_t batch_size, int32_t max_seq_len,
    int32_t page_size, const B200KvRuntimeGeometry &g, cudaStream_t stream) {
  if (state == nullptr || batch_size <= 0 || max_seq_len <= 0 ||
      page_size <= 0 || max_seq_len > kMaxPositions ||
      g.sliding_layers <= 0 || g.global_layers <= 0 ||
      g.sliding_kv_heads <= 0 || g.global_kv_heads <= 0 ||
      g.sliding_head_dim <= 0 || g.global_head_dim <= 0 ||
      g.sliding_window <= 0 || g.sliding_rotary_dim <= 0 ||
      g.global_rotary_dim <= 0 || g.global_rope_exponent_dim <= 0) {
    return cudaErrorInvalidValue;
  }
  const int32_t global_pps = b200kv::div_up(max_seq_len, page_size);
  const int32_t sliding_pps =
      sliding_pages(max_seq_len, page_size, g.sliding_window);
  const size_t token_rows = size_t(batch_size) * max_seq_len;

  *state = Gemma4RuntimeState();
  Gemma4RuntimeState &s = *state;
  s.batch_size = batch_size;
  s.max_seq_len = max_seq_len;
  s.page_size = page_size;
  s.sliding_cache_config = {g.sliding_layers,
                            batch_size * sliding_pps,
                            page_size,
                            sliding_pps,
                            batch_size,
                            g.sliding_kv_heads,
                            g.sliding_head_dim,
                            std::min(max_seq_len, g.sliding_window)};
  s.global_cache_config = {g.global_layers, batch_size * global_pps,
                           page_size,       global_pps,
                           batch_size,      g.global_kv_heads,
                           g.global_head_dim, 0};
  s.h_sliding_page_table.assign(size_t(batch_size) * sliding_pps, -1);
  s.h_global_page_table.assign(size_t(batch_size) * global_pps, -1);
  s.h_sliding_slot_logical_pages.assign(s.h_sliding_page_table.size(), -1);
  s.h_global_slot_logical_pages.assign(s.h_global_page_table.size(), -1);
  s.h_seq_lengths.assign(batch_size, 0);
  s.h_token_batch.resize(token_rows);
  s.h_token_position.resize(token_rows);

  auto body = [&]() -> cudaError_t {
    const size_t sliding_bytes =
        cache_elements(s.sliding_cache_config) * sizeof(__nv_bfloat16);
    const size_t global_bytes =
        cache_elements(s.global_cache_config) * sizeof(__nv_bfloat16);
    B200KV_TRY(cudaMalloc(&s.sliding_cache_k, sliding_bytes));
    B200KV_TRY(cudaMalloc(&s.sliding_cache_v, sliding_bytes));
    B200KV_TRY(cudaMalloc(&s.global_cache_k, global_bytes));
    B200KV_TRY(cudaMalloc(&s.global_cache_v, global_bytes));
    B200KV_TRY(cudaMalloc(&s.sliding_page_table,
                          s.h_sliding_page_table.size() * sizeof(int32_t)));
    B200KV_TRY(cudaMalloc(&s.global_page_table,
                          s.h_global_page_table.size() * sizeof(int32_t)));
    B200KV_TRY(cudaMalloc(&s.seq_lengths, size_t(batch_size) * sizeof(int32_t)));
    B200KV_TRY(cudaMalloc(&s.token_batch, token_rows * sizeof(int32_t)));
    B200KV_TRY(cudaMalloc(&s.token_position, token_rows * sizeof(int32_t)));

    std::vector<float> cos_t, sin_t;
    fill_rope(cos_t, sin_t, max_seq_len, g.sliding_rotary_dim / 2,
              g.sliding_rope_theta, g.sliding_head_dim);
    B200KV_TRY(cudaMalloc(&s.sliding_cos, cos_t.size() * sizeof(float)));
    B200KV_TRY(cudaMalloc(&s.sliding_sin, sin_t.size() * sizeof(float)));
    B200KV_TRY(upload(s.sliding_cos, cos_t, cos_t.size(), stream));
    B200KV_TRY(upload(s.sliding_sin, sin_t, sin_t.size(), stream));
    // The tables are pageable host vectors about to go out of scope.
    B200KV_TRY(cudaStreamSynchronize(stream));
    fill_rope(cos_t, sin_t, max_seq_len, g.global_rotary_dim / 2,
              g.global_rope_theta, g.global_rope_exponent_dim);
    B200KV_TRY(cudaMalloc(&s.global_cos, cos_t.size() * sizeof(float)));
    B200KV_TRY(cudaMalloc(&s.global_sin, sin_t.size() * sizeof(float)));
    B200KV_TRY(upload(s.global_cos, cos_t, cos_t.size(), stream));
    B200KV_TRY(upload(s.global_sin, sin_t, sin_t.size(), stream));
    B200KV_TRY(cudaStreamSynchronize(stream));
    return upload_all_metadata(&s, 0, stream);
  };
  const cudaError_t st = body();
  if (st != cudaSuccess) gemma4_runtime_state_free(state);
  return st;
}

cudaError_t gemma4_runtime_state_init(Gemma4RuntimeState *state,
                                      int32_t batch_size, int32_t max_seq_len,
                                      int32_t page_size, cudaStream_t stream) {
  return gemma4_runtime_state_init_geometry(state, batch_size, max_seq_len,
                                            page_size, default_geometry(),
                                            stream);
}

cudaError_t gemma4_runtime_prepare_prefill(Gemma4RuntimeState *state,
                                           int32_t seq_len,
                                           cudaStream_t stream) {
  Gemma4RuntimeState &s = *state;
  if (seq_len < 0 || seq_len > s.max_seq_len) return cudaErrorInvalidValue;
  std::fill(s.h_sliding_page_table.begin(), s.h_sliding_page_table.end(), -1);
  std::fill(s.h_global_page_table.begin(), s.h_global_page_table.end(), -1);
  std::fill(s.h_sliding_slot_logical_pages.begin(),
            s.h_sliding_slot_logical_pages.end(), -1);
  std::fill(s.h_global_slot_logical_pages.begin(),
            s.h_global_slot_logical_pages.end(), -1);
  for (int32_t b = 0; b < s.batch_size; ++b) {
    if (gemma4_kv_cache_ensure_range(s.h_sliding_page_table,
                                     s.h_sliding_slot_logical_pages,
                                     s.sliding_cache_config, b, 0,
                                     seq_len) < 0 ||
        gemma4_kv_cache_ensure_range(s.h_global_page_table,
                                     s.h_global_slot_logical_pages,
                                     s.global_cache_config, b, 0,
                                     seq_len) < 0) {
      return cudaErrorInvalidValue;
    }
    s.h_seq_lengths[b] = seq_len;
    for (int32_t pos = 0; pos < seq_len; ++pos) {
      const size_t row = size_t(b) * seq_len + pos;  // batch-major rows
      s.h_token_batch[row] = b;
      s.h_token_position[row] = pos;
    }
  }
  s.token_count = s.batch_size * seq_len;
  return upload_all_metadata(&s, size_t(s.token_count), stream);
}

cudaError_t gemma4_runtime_prepare_decode_step(Gemma4RuntimeState *state,
                                               cudaStream_t stream) {
  Gemma4RuntimeState &s = *state;
  // All-or-nothing: reject the step before touching any table
  // (tests/test_runtime_state.cu:83-105).
  for (int32_t b = 0; b < s.batch_size; ++b) {
    const int32_t pos = s.h_seq_lengths[b];
    if (pos < 0 || pos >= s.max_seq_len) return cudaErrorInvalidValue;
  }
  for (int32_t b = 0; b < s.batch_size; ++b) {
    const int32_t pos = s.h_seq_lengths[b];
    if (gemma4_kv_cache_ensure_page(s.h_sliding_page_table,
                                    s.h_sliding_slot_logical_pages,
                                    s.sliding_cache_config, b, pos) < 0 ||
        gemma4_kv_cache_ensure_page(s.h_global_page_table,
                                    s.h_global_slot_logical_pages,
                                    s.global_cache_config, b, pos) < 0) {
      return cudaErrorInvalidValue;
    }
    s.h_token_batch[b] = b;
    s.h_token_position[b] = pos;
    // Only the one entry per table that this position touches changes.
    const size_t si = size_t(b) * s.sliding_cache_config.max_pages_per_seq +
                      (pos / s.page_size) %
                          s.sliding_cache_config.max_pages_per_seq;
    const size_t gi = size_t(b) * s.global_cache_config.max_pages_per_seq +
                      (pos / s.page_size) %
                          s.global_cache_config.max_pages_per_seq;
    B200KV_TRY(cudaMemcpyAsync(s.sliding_page_table + si,
                               s.h_sliding_page_table.data() + si,
                               sizeof(int32_t), cudaMemcpyHostToDevice,
                               stream));
    B200KV_TRY(cudaMemcpyAsync(s.global_page_table + gi,
                               s.h_global_page_table.data() + gi,
                               sizeof(int32_t), cudaMemcpyHostToDevice,
                               stream));
  }
  for (int32_t b = 0; b < s.batch_size; ++b) ++s.h_seq_lengths[b];
  s.token_count = s.batch_size;
  B200KV_TRY(upload(s.seq_lengths, s.h_seq_lengths, s.h_seq_lengths.size(),
                    stream));
  B200KV_TRY(upload(s.token_batch, s.h_token_batch, size_t(s.token_count),
                    stream));
  return upload(s.token_position, s.h_token_position, size_t(s.token_count),
                stream);
}

// ===========================================================================
// extern "C" boundary
// ===========================================================================

// The C handle: the reference-layout state plus the geometry it was created
// with (kept here, outside the struct gemma.c code shares with the library).
struct B200KvRuntimeState {
  Gemma4RuntimeState state;
  B200KvRuntimeGeometry geometry;
};

// ===========================================================================
// Prompt attention entry points of src/gemma4_flash_attention.cuh
// ===========================================================================
namespace {
// Geometry constants of src/gemma4.h:13-28 for the two layer kinds.
constexpr int kQueryHeads = 16;
constexpr int kSlidingKvHeads = 8, kSlidingHeadDim = 256;
constexpr int kGlobalKvHeads = 1, kGlobalHeadDim = 512, kGlobalRotaryDim = 128;

cudaError_t prompt_forward(__nv_bfloat16 *out, __nv_bfloat16 *q_prepared,
                           __nv_bfloat16 *k_prepared, __nv_bfloat16 *v_prepared,
                           const __nv_bfloat16 *q, const __nv_bfloat16 *k,
                           const __nv_bfloat16 *v, const __nv_bfloat16 *q_w,
                           const __nv_bfloat16 *k_w, const float *cos,
                           const float *sin, const int32_t *token_position,
                           int batch_size, int seqlen_q, int seqlen_k,
                           int kv_heads, int head_dim, int rotary_dim, int window,
                           float softmax_scale, cudaStream_t stream) {
  // src/gemma4_flash_attention_prefill.cu:1131-1139
  if (batch_size <= 0 || seqlen_q <= 0 || seqlen_q != seqlen_k ||
      out == nullptr || q_prepared == nullptr || k_prepared == nullptr ||
      v_prepared == nullptr || token_position == nullptr) {
    return cudaErrorInvalidValue;
  }
  b200kv::PrefillPrepArgs prep;
  prep.q_prepared = q_prepared;
  prep.k_prepared = k_prepared;
  prep.v_prepared = v_prepared;
  prep.q = q;
  prep.k = k;
  prep.v = v;
  prep.q_norm_weight = q_w;
  prep.k_norm_weight = k_w;
  prep.cos = cos;
  prep.sin = sin;
  prep.token_position = token_position;
  prep.rows = int64_t(batch_size) * seqlen_q;
  prep.q_heads = kQueryHeads;
  prep.kv_heads = kv_heads;
  prep.head_dim = head_dim;
  prep.rotary_dim = rotary_dim;
  prep.norm_mode = B200KV_NORM_RSQRT_APPROX;
  const cudaError_t st = b200kv::prefill_prep_bf16(prep, stream);
  if (st != cudaSuccess) return st;
  return b200kv::prefill_attention_bf16(out, q_prepared, k_prepared, v_prepared,
                                        batch_size, seqlen_q, kQueryHeads, kv_heads,
                                        head_dim, window, softmax_scale, stream);
}
}  // namespace

cudaError_t gemma4_flash_attention_sliding_fwd_bf16_norm_rope(
    __nv_bfloat16 *__restrict__ d_out, __nv_bfloat16 *__restrict__ d_q_prepared,
    __nv_bfloat16 *__restrict__ d_k_prepared,
    __nv_bfloat16 *__restrict__ d_v_prepared, const __nv_bfloat16 *__restrict__ d_q,
    const __nv_bfloat16 *__restrict__ d_k, const __nv_bfloat16 *__restrict__ d_v,
    const __nv_bfloat16 *__restrict__ d_q_norm_weight,
    const __nv_bfloat16 *__restrict__ d_k_norm_weight,
    const float *__restrict__ d_cos, const float *__restrict__ d_sin,
    const int32_t *__restrict__ d_token_position, int batch_size, int seqlen_q,
    int seqlen_k, int window_size, float softmax_scale, cudaStream_t stream) {
  if (window_size <= 0 || d_v == nullptr) return cudaErrorInvalidValue;
  return prompt_forward(d_out, d_q_prepared, d_k_prepared, d_v_prepared, d_q, d_k,
                        d_v, d_q_norm_weight, d_k_norm_weight, d_cos, d_sin,
                        d_token_position, batch_size, seqlen_q, seqlen_k,
                        kSlidingKvHeads, kSlidingHeadDim, kSlidingHeadDim,
                        window_size, softmax_scale, stream);
}

cudaError_t gemma4_flash_attention_global_fwd_bf16_norm_rope(
    __nv_bfloat16 *__restrict__ d_out, __nv_bfloat16 *__restrict__ d_q_prepared,
    __nv_bfloat16 *__restrict__ d_k_prepared,
    __nv_bfloat16 *__restrict__ d_v_prepared, const __nv_bfloat16 *__restrict__ d_q,
    const __nv_bfloat16 *__restrict__ d_k,
    const __nv_bfloat16 *__restrict__ d_q_norm_weight,
    const __nv_bfloat16 *__restrict__ d_k_norm_weight,
    const float *__restrict__ d_cos, const float *__restrict__ d_sin,
    const int32_t *__restrict__ d_token_position, int batch_size, int seqlen_q,
    int seqlen_k, float softmax_scale, cudaStream_t stream) {
  return prompt_forward(d_out, d_q_prepared, d_k_prepared, d_v_prepared, d_q, d_k,
                        nullptr, d_q_norm_weight, d_k_norm_weight, d_cos, d_sin,
                        d_token_position, batch_size, seqlen_q, seqlen_k,
                        kGlobalKvHeads, kGlobalHeadDim, kGlobalRotaryDim, 0,
                        softmax_scale, stream);
}

namespace {
// B200KV_FUSED_LAYER_STEP=0 keeps the layer-step on separate append and
// attention launches (for A/B timing); read once.
bool fused_layer_step_enabled() {
  static const bool enabled = [] {
    const char *v = std::getenv("B200KV_FUSED_LAYER_STEP");
    return v == nullptr || std::strcmp(v, "0") != 0;
  }();
  return enabled;
}
}  // namespace

extern "C" {

cudaError_t gemma4_kv_cache_write_bf16(
    __nv_bfloat16 *__restrict__ d_cache_k,
    __nv_bfloat16 *__restrict__ d_cache_v, Gemma4KvCacheConfig config,
    const int32_t *__restrict__ d_page_table,
    const int32_t *__restrict__ d_token_batch,
    const int32_t *__restrict__ d_token_position, int32_t token_count,
    int32_t layer, const __nv_bfloat16 *__restrict__ d_k,
    const __nv_bfloat16 *__restrict__ d_v, cudaStream_t stream) {
  return b200kv::kv_cache_write_bf16(d_cache_k, d_cache_v, config,
                                     d_page_table, d_token_batch,
                                     d_token_position, token_count, layer, d_k,
                                     d_v, stream);
}

int b200kv_flash_attention_sliding_fwd_bf16_norm_rope(
    b200kv_bf16 *d_out, b200kv_bf16 *d_q_prepared, b200kv_bf16 *d_k_prepared,
    b200kv_bf16 *d_v_prepared, const b200kv_bf16 *d_q, const b200kv_bf16 *d_k,
    const b200kv_bf16 *d_v, const b200kv_bf16 *d_q_norm_weight,
    const b200kv_bf16 *d_k_norm_weight, const float *d_cos, const float *d_sin,
    const int32_t *d_token_position, int32_t batch_size, int32_t seqlen_q,
    int32_t seqlen_k, int32_t window_size, float softmax_scale,
    b200kv_stream stream) {
  using bf = __nv_bfloat16;
  return gemma4_flash_attention_sliding_fwd_bf16_norm_rope(
      reinterpret_cast<bf *>(d_out), reinterpret_cast<bf *>(d_q_prepared),
      reinterpret_cast<bf *>(d_k_prepared), reinterpret_cast<bf *>(d_v_prepared),
      reinterpret_cast<const bf *>(d_q), reinterpret_cast<const bf *>(d_k),
      reinterpret_cast<const bf *>(d_v),
      reinterpret_cast<const bf *>(d_q_norm_weight),
      reinterpret_cast<const bf *>(d_k_norm_weight), d_cos, d_sin,
      d_token_position, batch_size, seqlen_q, seqlen_k, window_size,
      softmax_scale, static_cast<cudaStream_t>(stream));
}

int b200kv_flash_attention_global_fwd_bf16_norm_rope(
    b200kv_bf16 *d_out, b200kv_bf16 *d_q_prepared, b200kv_bf16 *d_k_prepared,
    b200kv_bf16 *d_v_prepared, const b200kv_bf16 *d_q, const b200kv_bf16 *d_k,
    const b200kv_bf16 *d_q_norm_weight, const b200kv_bf16 *d_k_norm_weight,
    const float *d_cos, const float *d_sin, const int32_t *d_token_position,
    int32_t batch_size, int32_t seqlen_q, int32_t seqlen_k, float softmax_scale,
    b200kv_stream stream) {
  using bf = __nv_bfloat16;
  return gemma4_flash_attention_global_fwd_bf16_norm_rope(
      reinterpret_cast<bf *>(d_out), reinterpret_cast<bf *>(d_q_prepared),
      reinterpret_cast<bf *>(d_k_prepared), reinterpret_cast<bf *>(d_v_prepared),
      reinterpret_cast<const bf *>(d_q), reinterpret_cast<const bf *>(d_k),
      reinterpret_cast<const bf *>(d_q_norm_weight),
      reinterpret_cast<const bf *>(d_k_norm_weight), d_cos, d_sin,
      d_token_position, batch_size, seqlen_q, seqlen_k, softmax_scale,
      static_cast<cudaStream_t>(stream));
}

int b200kv_prefill_attention_fault(void) {
  return b200kv::prefill_attention_sm100_fault();
}

int b200kv_prefill_attention_bf16(b200kv_bf16 *d_out,
                                  const b200kv_bf16 *d_q_prepared,
                                  const b200kv_bf16 *d_k_prepared,
                                  const b200kv_bf16 *d_v_prepared,
                                  int32_t batch_size, int32_t seq_len,
                                  int32_t q_heads, int32_t kv_heads,
                                  int32_t head_dim, int32_t window_size,
                                  float softmax_scale, b200kv_stream stream) {
  using bf = __nv_bfloat16;
  return b200kv::prefill_attention_bf16(
      reinterpret_cast<bf *>(d_out), reinterpret_cast<const bf *>(d_q_prepared),
      reinterpret_cast<const bf *>(d_k_prepared),
      reinterpret_cast<const bf *>(d_v_prepared), batch_size, seq_len, q_heads,
      kv_heads, head_dim, window_size, softmax_scale,
      static_cast<cudaStream_t>(stream));
}

int b200kv_prefill_cache_fill_bf16(b200kv_bf16 *d_cache_k,
                                   b200kv_bf16 *d_cache_v,
                                   Gemma4KvCacheConfig config,
                                   const int32_t *d_page_table,
                                   const int32_t *d_token_batch,
                                   const int32_t *d_token_position,
                                   int32_t batch_size, int32_t seq_len,
                                   int32_t layer, const b200kv_bf16 *d_k_prepared,
                                   const b200kv_bf16 *d_v_prepared,
                                   b200kv_stream stream) {
  using bf = __nv_bfloat16;
  return b200kv::prefill_cache_fill_bf16(
      reinterpret_cast<bf *>(d_cache_k), reinterpret_cast<bf *>(d_cache_v),
      config, d_page_table, d_token_batch, d_token_position, batch_size, seq_len,
      layer, reinterpret_cast<const bf *>(d_k_prepared),
      reinterpret_cast<const bf *>(d_v_prepared),
      static_cast<cudaStream_t>(stream));
}

int64_t b200kv_cache_offset(const Gemma4KvCacheConfig *config, int32_t layer,
                            int32_t page, int32_t page_offset, int32_t head,
                            int32_t dim) {
  return gemma4_kv_cache_offset(*config, layer, page, page_offset, head, dim);
}

void b200kv_make_config(Gemma4KvCacheConfig *out, int32_t global,
                        int32_t num_pages, int32_t page_size,
                        int32_t max_pages_per_seq) {
  *out = gemma4_kv_cache_make_config(global != 0, num_pages, page_size,
                                     max_pages_per_seq);
}

int32_t b200kv_is_global_layer(int32_t model_layer) {
  return is_global_layer(model_layer) ? 1 : 0;
}

int32_t b200kv_layer_index(int32_t model_layer, int32_t global_cache) {
  return gemma4_kv_cache_layer_index(model_layer, global_cache != 0);
}

int32_t b200kv_ensure_page(int32_t *h_page_table, int32_t *h_slot_logical_pages,
                           const Gemma4KvCacheConfig *config, int32_t batch,
                           int32_t position) {
  // Direct map: sequence b owns physical pages [b*width, (b+1)*width). A slot
  // that already holds a later logical page is stale for this position.
  const int32_t logical_page = position / config->page_size;
  const int32_t slot = logical_page % config->max_pages_per_seq;
  const int64_t index = int64_t(batch) * config->max_pages_per_seq + slot;
  if (h_slot_logical_pages[index] > logical_page) return -1;
  const int32_t physical = batch * config->max_pages_per_seq + slot;
  h_page_table[index] = physical;
  h_slot_logical_pages[index] = logical_page;
  return physical;
}

int32_t b200kv_ensure_range(int32_t *h_page_table,
                            int32_t *h_slot_logical_pages,
                            const Gemma4KvCacheConfig *config, int32_t batch,
                            int32_t first_position, int32_t token_count) {
  if (token_count == 0) return 0;
  const int32_t first_page = first_position / config->page_size;
  const int32_t last_page =
      (first_position + token_count - 1) / config->page_size;
  for (int32_t page = first_page; page <= last_page; ++page) {
    if (b200kv_ensure_page(h_page_table, h_slot_logical_pages, config, batch,
                           page * config->page_size) < 0) {
      return -1;
    }
  }
  return 0;
}

int32_t b200kv_sliding_pages_per_sequence(int32_t max_seq_len,
                                          int32_t page_size) {
  return sliding_pages(max_seq_len, page_size, 1024);
}

void b200kv_fill_rope_tables(float *h_cos, float *h_sin, int32_t max_seq_len,
                             int32_t rotary_half, float theta,
                             int32_t exponent_dim) {
  // fp32 throughout, as the reference's table builder: the angle is the fp32
  // product of the position and powf(theta, -2i/exponent_dim).
  for (int32_t pos = 0; pos < max_seq_len; ++pos) {
    float *c = h_cos + size_t(pos) * rotary_half;
    float *s = h_sin + size_t(pos) * rotary_half;
    for (int32_t i = 0; i < rotary_half; ++i) {
      const float exponent = -2.0f * float(i) / float(exponent_dim);
      const float angle = float(pos) * std::pow(theta, exponent);
      c[i] = std::cos(angle);
      s[i] = std::sin(angle);
    }
  }
}

void b200kv_runtime_geometry_default(B200KvRuntimeGeometry *out) {
  *out = default_geometry();
}

int b200kv_runtime_state_create(B200KvRuntimeState **out, int32_t batch_size,
                                int32_t max_seq_len, int32_t page_size,
                                const B200KvRuntimeGeometry *geometry,
                                b200kv_stream stream) {
  if (out == nullptr) return cudaErrorInvalidValue;
  *out = nullptr;
  B200KvRuntimeState *handle = new (std::nothrow) B200KvRuntimeState();
  if (handle == nullptr) return cudaErrorMemoryAllocation;
  handle->geometry = geometry != nullptr ? *geometry : default_geometry();
  const cudaError_t st = gemma4_runtime_state_init_geometry(
      &handle->state, batch_size, max_seq_len, page_size, handle->geometry,
      static_cast<cudaStream_t>(stream));
  if (st != cudaSuccess) {
    delete handle;
    return st;
  }
  *out = handle;
  return cudaSuccess;
}

void b200kv_runtime_state_destroy(B200KvRuntimeState *state) {
  if (state == nullptr) return;
  gemma4_runtime_state_free(&state->state);
  delete state;
}

int b200kv_runtime_prepare_prefill(B200KvRuntimeState *state, int32_t seq_len,
                                   b200kv_stream stream) {
  if (state == nullptr) return cudaErrorInvalidValue;
  return gemma4_runtime_prepare_prefill(&state->state, seq_len,
                                        static_cast<cudaStream_t>(stream));
}

int b200kv_runtime_prepare_decode_step(B200KvRuntimeState *state,
                                       b200kv_stream stream) {
  if (state == nullptr) return cudaErrorInvalidValue;
  return gemma4_runtime_prepare_decode_step(&state->state,
                                            static_cast<cudaStream_t>(stream));
}

void b200kv_runtime_state_view(B200KvRuntimeState *state,
                               B200KvRuntimeView *out) {
  Gemma4RuntimeState &s = state->state;
  out->batch_size = s.batch_size;
  out->max_seq_len = s.max_seq_len;
  out->page_size = s.page_size;
  out->token_count = s.token_count;
  out->sliding_cache_config = s.sliding_cache_config;
  out->global_cache_config = s.global_cache_config;
  out->sliding_cache_k = reinterpret_cast<b200kv_bf16 *>(s.sliding_cache_k);
  out->sliding_cache_v = reinterpret_cast<b200kv_bf16 *>(s.sliding_cache_v);
  out->global_cache_k = reinterpret_cast<b200kv_bf16 *>(s.global_cache_k);
  out->global_cache_v = reinterpret_cast<b200kv_bf16 *>(s.global_cache_v);
  out->sliding_page_table = s.sliding_page_table;
  out->global_page_table = s.global_page_table;
  out->seq_lengths = s.seq_lengths;
  out->token_batch = s.token_batch;
  out->token_position = s.token_position;
  out->sliding_cos = s.sliding_cos;
  out->sliding_sin = s.sliding_sin;
  out->global_cos = s.global_cos;
  out->global_sin = s.global_sin;
  out->h_sliding_page_table = s.h_sliding_page_table.data();
  out->h_global_page_table = s.h_global_page_table.data();
  out->h_sliding_slot_logical_pages = s.h_sliding_slot_logical_pages.data();
  out->h_global_slot_logical_pages = s.h_global_slot_logical_pages.data();
  out->h_seq_lengths = s.h_seq_lengths.data();
  out->h_token_batch = s.h_token_batch.data();
  out->h_token_position = s.h_token_position.data();
  out->h_sliding_page_table_size = int64_t(s.h_sliding_page_table.size());
  out->h_global_page_table_size = int64_t(s.h_global_page_table.size());
  out->h_token_rows = int64_t(s.h_token_batch.size());
}

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
                             int32_t norm_mode, b200kv_stream stream) {
  using bf = __nv_bfloat16;
  b200kv::PrefillPrepArgs a;
  a.q_prepared = reinterpret_cast<bf *>(d_q_prepared);
  a.k_prepared = reinterpret_cast<bf *>(d_k_prepared);
  a.v_prepared = reinterpret_cast<bf *>(d_v_prepared);
  a.q = reinterpret_cast<const bf *>(d_q);
  a.k = reinterpret_cast<const bf *>(d_k);
  a.v = reinterpret_cast<const bf *>(d_v);
  a.q_norm_weight = reinterpret_cast<const bf *>(d_q_norm_weight);
  a.k_norm_weight = reinterpret_cast<const bf *>(d_k_norm_weight);
  a.cos = d_cos;
  a.sin = d_sin;
  a.token_position = d_token_position;
  a.rows = rows;
  a.q_heads = q_heads;
  a.kv_heads = kv_heads;
  a.head_dim = head_dim;
  a.rotary_dim = rotary_dim;
  a.norm_mode = norm_mode;
  return b200kv::prefill_prep_bf16(a, static_cast<cudaStream_t>(stream));
}

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
                              b200kv_stream stream) {
  using bf = __nv_bfloat16;
  b200kv::AppendArgs a;
  a.q_prepared = reinterpret_cast<bf *>(d_q_prepared);
  a.cache_k = reinterpret_cast<bf *>(d_cache_k);
  a.cache_v = reinterpret_cast<bf *>(d_cache_v);
  a.cfg = cache_config;
  a.page_table = d_page_table;
  a.token_position = d_token_position;
  a.cache_layer = cache_layer;
  a.q = reinterpret_cast<const bf *>(d_q);
  a.k = reinterpret_cast<const bf *>(d_k);
  a.v = reinterpret_cast<const bf *>(d_v);
  a.q_norm_weight = reinterpret_cast<const bf *>(d_q_norm_weight);
  a.k_norm_weight = reinterpret_cast<const bf *>(d_k_norm_weight);
  a.cos = d_cos;
  a.sin = d_sin;
  a.batch_count = batch_count;
  a.q_heads = q_heads;
  a.rotary_dim = rotary_dim;
  a.norm_mode = norm_mode;
  return b200kv::decode_append_bf16(a, static_cast<cudaStream_t>(stream));
}

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
                                 b200kv_stream stream) {
  using bf = __nv_bfloat16;
  b200kv::DecodeArgs a;
  a.out = reinterpret_cast<bf *>(d_out);
  a.lse = d_lse;
  a.q = reinterpret_cast<const bf *>(d_q_prepared);
  a.cache_k = reinterpret_cast<const bf *>(d_cache_k);
  a.cache_v = reinterpret_cast<const bf *>(d_cache_v);
  a.cfg = cache_config;
  a.page_table = d_page_table;
  a.seq_lengths = d_seq_lengths;
  a.layer = cache_layer;
  a.softmax_scale = softmax_scale;
  a.split_size = split_size;
  a.num_splits = num_splits;
  a.batch_count = batch_count;
  a.q_heads = q_heads;
  a.partial_m = d_partial_m;
  a.partial_l = d_partial_l;
  a.partial_acc = d_partial_acc;
  a.status = d_status;
  return b200kv::decode_attention_bf16(a, static_cast<cudaStream_t>(stream));
}

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
                             b200kv_stream stream) {
  using bf = __nv_bfloat16;
  b200kv::AppendArgs a;
  a.q_prepared = reinterpret_cast<bf *>(d_q_prepared);
  a.cfg = cache_config;
  a.page_table = d_page_table;
  a.token_position = d_token_position;
  a.cache_layer = cache_layer;
  a.q = reinterpret_cast<const bf *>(d_q);
  a.k = reinterpret_cast<const bf *>(d_k);
  a.v = reinterpret_cast<const bf *>(d_v);
  a.q_norm_weight = reinterpret_cast<const bf *>(d_q_norm_weight);
  a.k_norm_weight = reinterpret_cast<const bf *>(d_k_norm_weight);
  a.cos = d_cos;
  a.sin = d_sin;
  a.batch_count = batch_count;
  a.q_heads = q_heads;
  a.rotary_dim = rotary_dim;
  a.norm_mode = norm_mode;
  return b200kv::decode_append_fp8(a, d_cache_k, d_cache_v, d_scale_k,
                                   d_scale_v, static_cast<cudaStream_t>(stream));
}

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
                           b200kv_stream stream) {
  using bf = __nv_bfloat16;
  return b200kv::fp8_append_rows(
      d_cache_k, d_cache_v, d_scale_k, d_scale_v, cache_config, d_page_table,
      d_seq_batch, d_first_position, d_row_count, d_row_start, run_count,
      max_row_count, cache_layer, reinterpret_cast<const bf *>(d_k_prepared),
      reinterpret_cast<const bf *>(d_v_prepared),
      static_cast<cudaStream_t>(stream));
}

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
                                int32_t *d_status, b200kv_stream stream) {
  using bf = __nv_bfloat16;
  b200kv::DecodeArgs a;
  a.out = reinterpret_cast<bf *>(d_out);
  a.lse = d_lse;
  a.q = reinterpret_cast<const bf *>(d_q_prepared);
  a.cfg = cache_config;
  a.page_table = d_page_table;
  a.seq_lengths = d_seq_lengths;
  a.layer = cache_layer;
  a.softmax_scale = softmax_scale;
  a.split_size = 0;
  a.num_splits = num_splits;
  a.batch_count = batch_count;
  a.q_heads = q_heads;
  a.partial_m = d_partial_m;
  a.partial_l = d_partial_l;
  a.partial_acc = d_partial_acc;
  a.status = d_status;
  return b200kv::decode_attention_fp8(a, d_cache_k, d_cache_v, d_scale_k,
                                      d_scale_v,
                                      static_cast<cudaStream_t>(stream));
}

void b200kv_decode_workspace_bytes(int32_t batch_count, int32_t q_heads,
                                   int32_t head_dim, int32_t num_splits,
                                   size_t *partial_m_bytes,
                                   size_t *partial_l_bytes,
                                   size_t *partial_acc_bytes) {
  const size_t rows = num_splits > 1
                          ? size_t(batch_count) * q_heads * num_splits
                          : 0;
  if (partial_m_bytes) *partial_m_bytes = rows * sizeof(float);
  if (partial_l_bytes) *partial_l_bytes = rows * sizeof(float);
  if (partial_acc_bytes) *partial_acc_bytes = rows * head_dim * sizeof(float);
}

void b200kv_plan_balanced(int32_t batch_count, int32_t sm_count,
                          int32_t *num_splits) {
  *num_splits = b200kv::decode_balanced_num_splits(batch_count, sm_count);
}

void b200kv_plan_splits_total(int32_t batch_count, int32_t max_live_keys,
                              int64_t total_live_keys, int32_t kv_heads,
                              int32_t sm_count, int32_t *split_size,
                              int32_t *num_splits) {
  const int tile = b200kv::decode_stage_tokens(kv_heads);
  const int64_t batch = std::max(batch_count, 1);
  const int64_t longest = std::max(max_live_keys, 1);
  const int64_t total = std::max<int64_t>(total_live_keys, 1);
  // Resident CTAs: two per SM for the 8-KV-head kernel, one otherwise.
  const int64_t slots = int64_t(std::max(sm_count, 1)) * (kv_heads == 8 ? 2 : 1);
  // Cost in "keys of streaming time per slot": a CTA pays its keys plus a
  // fixed fill/drain of about 6 keys' worth, and its partials (written once,
  // read once) cost about 4 keys' worth of bandwidth shared by all slots.
  int64_t best_size = tile;
  double best_cost = 1e300;
  for (int64_t size = tile; size <= 64 * tile; size += tile) {
    // Upper bound of live CTAs: every sequence may end in a partial split.
    const int64_t ctas = std::min(total / size + batch,
                                  batch * b200kv::div_up(longest, size));
    const int64_t waves = (ctas + slots - 1) / slots;
    const bool single = size >= longest;  // one split per row: no partials
    const double cost = double(waves) * double(size + 6) +
                        (single ? 0.0 : 4.0 * double(ctas) / double(slots));
    if (cost < best_cost - 1e-9 || (cost < best_cost + 1e-9 && size > best_size)) {
      best_cost = cost;
      best_size = size;
    }
    if (size >= longest) break;
  }
  *split_size = int32_t(best_size);
  *num_splits = int32_t(std::max<int64_t>(1, b200kv::div_up(longest, best_size)));
}

void b200kv_plan_splits(int32_t batch_count, int32_t max_live_keys,
                        int32_t kv_heads, int32_t sm_count,
                        int32_t *split_size, int32_t *num_splits) {
  // Without the true sum, assume sequences average half the longest one.
  const int64_t total = int64_t(std::max(batch_count, 1)) *
                        ((int64_t(std::max(max_live_keys, 1)) + 1) / 2);
  b200kv_plan_splits_total(batch_count, max_live_keys,
                           batch_count <= 1 ? max_live_keys : total, kv_heads,
                           sm_count, split_size, num_splits);
}

}  // extern "C"

namespace {

// The exchange of a layer-step that did not run as the one-launch kernel: the
// stand-alone all-gather kernel behind the step's last launch.
int gather_after(const B200KvLayerStepArgs *s, cudaStream_t st) {
  if (s->peer_gather == nullptr) return cudaSuccess;
  return b200kv::peer_allgather(
      s->peer_gather, s->out,
      int64_t(s->batch_count) * s->q_heads * s->cache_config.head_dim * 2, s->status,
      st, nullptr);
}

// raw_from_predecessor: the raw rows come from the kernel enqueued just before
// (the attention-layer call's QKV projection), not from an earlier step.
// Whether layer_step() gives this layer-step to the one-launch kernel.
bool takes_one_launch_kernel(const B200KvLayerStepArgs *s) {
  return s->batch_count > 0 && s->split_size == 0 && s->rotary_dim == 256 &&
         fused_layer_step_enabled() &&
         b200kv::decode_pagetile_preferred(s->cache_config, s->q_heads, s->batch_count,
                                           s->ticket != nullptr);
}

// What b200kv_decode_step_bf16 tells an entry's launch about its place in a run
// of overlapping launches (see plan_entry below). Default: a launch on its own.
struct StepPlan {
  int32_t steps_in_flight = 1;  // unfinished launches entry i can meet that are steps of its cache layer
  bool release_early = false;   // its kernel releases the next entry's at once
  bool chained = false;         // part of a run: sized for one CTA per SM
  // the entries (nearest first) whose appended rows entry i prepares itself
  // instead of waiting for them; either all steps_in_flight of them or none
  int32_t forward_count = 0;
  int32_t forward_entry[b200kv::AppendArgs::kMaxForward] = {};
};

int layer_step(const B200KvLayerStepArgs *s, bool raw_from_predecessor,
               b200kv_stream stream, bool force_tiled = false,
               const StepPlan &plan = StepPlan(),
               const B200KvLayerStepArgs *entries = nullptr) {
  if (s == nullptr) return cudaErrorInvalidValue;
  using bf = __nv_bfloat16;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  b200kv::AppendArgs a;
  a.q_prepared = reinterpret_cast<bf *>(s->q);
  a.cache_k = reinterpret_cast<bf *>(s->cache_k);
  a.cache_v = reinterpret_cast<bf *>(s->cache_v);
  a.cfg = s->cache_config;
  a.page_table = s->page_table;
  a.token_position = s->token_position;
  a.cache_layer = s->cache_layer;
  a.q = reinterpret_cast<const bf *>(s->raw_q);
  a.k = reinterpret_cast<const bf *>(s->raw_k);
  a.v = reinterpret_cast<const bf *>(s->raw_v);
  a.q_norm_weight = reinterpret_cast<const bf *>(s->q_norm_weight);
  a.k_norm_weight = reinterpret_cast<const bf *>(s->k_norm_weight);
  a.cos = s->cos;
  a.sin = s->sin;
  a.batch_count = s->batch_count;
  a.q_heads = s->q_heads;
  a.rotary_dim = s->rotary_dim;
  a.norm_mode = s->norm_mode;
  a.raw_from_predecessor = raw_from_predecessor;
  a.steps_in_flight = plan.steps_in_flight;
  a.release_early = plan.release_early;
  a.chained = plan.chained;
  if (entries != nullptr) {
    a.forward_count = plan.forward_count;
    for (int32_t j = 0; j < plan.forward_count; ++j) {
      const B200KvLayerStepArgs &e = entries[plan.forward_entry[j]];
      a.forward_k[j] = reinterpret_cast<const bf *>(e.raw_k);
      a.forward_v[j] = reinterpret_cast<const bf *>(e.raw_v);
      a.forward_position[j] = e.token_position;
    }
  }

  b200kv::DecodeArgs d;
  d.out = reinterpret_cast<bf *>(s->out);
  d.lse = s->lse;
  d.q = reinterpret_cast<const bf *>(s->q);
  d.cache_k = reinterpret_cast<const bf *>(s->cache_k);
  d.cache_v = reinterpret_cast<const bf *>(s->cache_v);
  d.cfg = s->cache_config;
  d.page_table = s->page_table;
  d.seq_lengths = s->seq_lengths;
  d.layer = s->cache_layer;
  d.softmax_scale = s->softmax_scale;
  d.split_size = s->split_size;
  d.num_splits = s->num_splits;
  d.batch_count = s->batch_count;
  d.q_heads = s->q_heads;
  d.partial_m = s->partial_m;
  d.partial_l = s->partial_l;
  d.partial_acc = s->partial_acc;
  d.status = s->status;

  // Small jobs: one launch for append + attention + merge, a CTA per (sequence,
  // KV head, key range) (decode_pagetile.cu); needs the caller's tickets.
  if (force_tiled && (s->batch_count <= 0 || s->split_size != 0 ||
                      s->rotary_dim != 256 || s->ticket == nullptr)) {
    return cudaErrorInvalidValue;
  }
  if (force_tiled || takes_one_launch_kernel(s)) {
    if (s->event_before_attention != nullptr) {
      B200KV_TRY(cudaEventRecord(
          static_cast<cudaEvent_t>(s->event_before_attention), st));
    }
    b200kv::PeerEpilogue peer = {};
    if (s->peer_gather != nullptr) {
      B200KV_TRY(b200kv::peer_epilogue_begin(
          s->peer_gather, int64_t(s->batch_count) * s->q_heads * d.cfg.head_dim * 2,
          &peer));
    }
    const cudaError_t st_tile = b200kv::decode_layer_step_pagetile_bf16(
        &a, d, s->ticket, st, s->peer_gather != nullptr ? &peer : nullptr);
    if (st_tile != cudaSuccess) return st_tile;
    if (s->event_after_attention != nullptr) {
      B200KV_TRY(cudaEventRecord(
          static_cast<cudaEvent_t>(s->event_after_attention), st));
    }
    return cudaSuccess;
  }
  // One launch for append + attention where the balanced kernel can do both
  // (the reference's decode_megakernel_fused_layer_kernel is one launch too,
  // src/gemma4_flash_attention_decode.cu:1004-1031). The profiling hooks then
  // bracket that launch and its combine.
  if (s->batch_count > 0 && fused_layer_step_enabled() &&
      b200kv::decode_fused_supported(a, d)) {
    if (s->event_before_attention != nullptr) {
      B200KV_TRY(cudaEventRecord(
          static_cast<cudaEvent_t>(s->event_before_attention), st));
    }
    const cudaError_t st_fused = b200kv::decode_layer_step_fused_bf16(a, d, st);
    if (st_fused != cudaSuccess) return st_fused;
    if (s->event_after_attention != nullptr) {
      B200KV_TRY(cudaEventRecord(
          static_cast<cudaEvent_t>(s->event_after_attention), st));
    }
    return gather_after(s, st);
  }
  // Two launches: stream order makes the appended row visible to the attention
  // kernel, the job the grid-wide barrier does inside the reference's fused
  // layer kernel (src/gemma4_flash_attention_decode.cu:524).
  const cudaError_t st_append = b200kv::decode_append_bf16(a, st);
  if (st_append != cudaSuccess) return st_append;
  if (s->event_before_attention != nullptr) {
    B200KV_TRY(cudaEventRecord(
        static_cast<cudaEvent_t>(s->event_before_attention), st));
  }
  const cudaError_t st_attn = b200kv::decode_attention_bf16(d, st);
  if (st_attn != cudaSuccess) return st_attn;
  if (s->event_after_attention != nullptr) {
    B200KV_TRY(cudaEventRecord(
        static_cast<cudaEvent_t>(s->event_after_attention), st));
  }
  return gather_after(s, st);
}

}  // namespace

extern "C" {

int b200kv_decode_layer_step_bf16(const B200KvLayerStepArgs *s,
                                  b200kv_stream stream) {
  return layer_step(s, false, stream);
}

int32_t b200kv_layer_step_launches(const B200KvLayerStepArgs *s) {
  if (s == nullptr || s->batch_count <= 0) return 0;
  const Gemma4KvCacheConfig &c = s->cache_config;
  if (s->split_size == 0 && s->rotary_dim == 256 && fused_layer_step_enabled() &&
      b200kv::decode_pagetile_preferred(c, s->q_heads, s->batch_count,
                                        s->ticket != nullptr)) {
    return 1;  // the exchange, if any, is part of it
  }
  const int32_t gather = s->peer_gather != nullptr ? 1 : 0;  // the stand-alone gather kernel
  if (s->split_size == 0 && fused_layer_step_enabled() && s->rotary_dim == 256 &&
      b200kv::decode_balanced_supported(c, s->q_heads, s->batch_count)) {
    return 2 + gather;  // fused attention kernel + combine
  }
  return ((s->split_size > 0 && s->num_splits == 1) ? 2 : 3) + gather;  // append, attention[, combine]
}

int b200kv_decode_layer_step_tiled_bf16(const B200KvLayerStepArgs *s,
                                        b200kv_stream stream) {
  return layer_step(s, false, stream, true);
}

int b200kv_decode_attention_tiled_bf16(
    b200kv_bf16 *d_out, float *d_lse, const b200kv_bf16 *d_q_prepared,
    const b200kv_bf16 *d_cache_k, const b200kv_bf16 *d_cache_v,
    Gemma4KvCacheConfig cache_config, const int32_t *d_page_table,
    const int32_t *d_seq_lengths, int32_t cache_layer, float softmax_scale,
    int32_t num_splits, int32_t batch_count, int32_t q_heads, float *d_partial_m,
    float *d_partial_l, float *d_partial_acc, uint32_t *d_ticket,
    int32_t *d_status, b200kv_stream stream) {
  using bf = __nv_bfloat16;
  b200kv::DecodeArgs d;
  d.out = reinterpret_cast<bf *>(d_out);
  d.lse = d_lse;
  d.q = reinterpret_cast<const bf *>(d_q_prepared);
  d.cache_k = reinterpret_cast<const bf *>(d_cache_k);
  d.cache_v = reinterpret_cast<const bf *>(d_cache_v);
  d.cfg = cache_config;
  d.page_table = d_page_table;
  d.seq_lengths = d_seq_lengths;
  d.layer = cache_layer;
  d.softmax_scale = softmax_scale;
  d.split_size = 0;
  d.num_splits = num_splits;
  d.batch_count = batch_count;
  d.q_heads = q_heads;
  d.partial_m = d_partial_m;
  d.partial_l = d_partial_l;
  d.partial_acc = d_partial_acc;
  d.status = d_status;
  return b200kv::decode_layer_step_pagetile_bf16(
      nullptr, d, d_ticket, static_cast<cudaStream_t>(stream));
}

namespace {

// An entry's kernel normally lets the next entry's kernel start once its own
// predecessor is complete, so that a starting kernel meets one unfinished
// launch. A run of one-launch layer-steps does better: entry i releases entry
// i + 1 at once, and entry i + 1 is told how many of the launches it can then
// meet -- the entries of the run so far -- are earlier decode steps of its own
// cache layer, whose newest rows are not in the cache yet. (Entries that name
// the same cache layer are consecutive decode steps, in order: each appends the
// position after its predecessor's.) Where all of those steps are entries of
// this call, the kernel is given their raw K / V rows and positions and prepares
// the rows itself; otherwise it leaves their pages until its predecessor is
// complete. The first entry never releases early (what precedes it is not known
// here) and allows for one step of its own layer in flight; a run is cut after
// kMaxEarlyRun entries, which bounds the launches in flight whatever their size.
constexpr int32_t kMaxEarlyRun = 6;
static_assert(kMaxEarlyRun + 1 <= b200kv::AppendArgs::kMaxForward, "every step in flight can be forwarded");

// B200KV_MAX_EARLY_RUN=n (0..6): tuning aid, shorter runs.
int32_t max_early_run() {
  static const int32_t n = [] {
    const char *v = std::getenv("B200KV_MAX_EARLY_RUN");
    if (v == nullptr) return kMaxEarlyRun;
    return std::min(kMaxEarlyRun, std::max(0, std::atoi(v)));
  }();
  return n;
}

// Plan of entry i given the early releases in a row up to entry i - 1.
StepPlan plan_entry(const B200KvLayerStepArgs *layers, int32_t layer_count, int32_t i,
                    int32_t run) {
  auto same_cache = [&](int32_t a, int32_t b) {
    const B200KvLayerStepArgs &p = layers[a];
    const B200KvLayerStepArgs &c = layers[b];
    return (p.cache_k == c.cache_k || p.cache_v == c.cache_v) && p.cache_layer == c.cache_layer;
  };
  StepPlan plan;
  plan.steps_in_flight = 0;
  const int32_t in_flight = 1 + run;  // unfinished launches entry i can meet
  bool all_known = true;
  for (int32_t k = 1; k <= in_flight; ++k) {
    if (i - k < 0 || layers[i - k].batch_count <= 0) {
      ++plan.steps_in_flight;  // not known here: taken to be a step of this layer
      all_known = false;
    } else if (same_cache(i - k, i)) {
      const B200KvLayerStepArgs &e = layers[i - k];
      const B200KvLayerStepArgs &c = layers[i];
      if (plan.steps_in_flight < b200kv::AppendArgs::kMaxForward && e.raw_k != nullptr &&
          e.token_position != nullptr && e.batch_count == c.batch_count &&
          e.k_norm_weight == c.k_norm_weight && e.cos == c.cos && e.sin == c.sin &&
          e.norm_mode == c.norm_mode && e.page_table == c.page_table) {
        plan.forward_entry[plan.steps_in_flight] = i - k;
      } else {
        all_known = false;
      }
      ++plan.steps_in_flight;
    }
  }
  plan.forward_count = all_known && takes_one_launch_kernel(layers + i) ? plan.steps_in_flight : 0;
  plan.release_early = i >= 1 && i + 1 < layer_count && run < max_early_run() &&
                       takes_one_launch_kernel(layers + i) &&
                       takes_one_launch_kernel(layers + i + 1);
  // part of a run: released early, releasing early, or the run's first entry
  plan.chained = plan.release_early || run > 0 ||
                 (i + 2 < layer_count && takes_one_launch_kernel(layers + i) &&
                  takes_one_launch_kernel(layers + i + 1) &&
                  takes_one_launch_kernel(layers + i + 2));
  return plan;
}

}  // namespace

int b200kv_decode_step_bf16(const B200KvLayerStepArgs *layers,
                            int32_t layer_count, b200kv_stream stream) {
  if (layers == nullptr || layer_count < 0) return cudaErrorInvalidValue;
  int32_t run = 0;  // early releases in a row up to the entry before this one
  for (int32_t i = 0; i < layer_count; ++i) {
    const StepPlan plan = plan_entry(layers, layer_count, i, run);
    const int st = layer_step(layers + i, false, stream, false, plan, layers);
    if (st != cudaSuccess) return st;
    run = plan.release_early ? run + 1 : 0;
  }
  return cudaSuccess;
}

int b200kv_decode_step_plan(const B200KvLayerStepArgs *layers, int32_t layer_count,
                            int32_t *steps_in_flight, int32_t *release_early,
                            int32_t *forwarded) {
  if (layers == nullptr || layer_count < 0) return cudaErrorInvalidValue;
  int32_t run = 0;
  for (int32_t i = 0; i < layer_count; ++i) {
    const StepPlan plan = plan_entry(layers, layer_count, i, run);
    if (steps_in_flight != nullptr) steps_in_flight[i] = plan.steps_in_flight;
    if (release_early != nullptr) release_early[i] = plan.release_early ? 1 : 0;
    if (forwarded != nullptr) forwarded[i] = plan.forward_count;
    run = plan.release_early ? run + 1 : 0;
  }
  return cudaSuccess;
}

int b200kv_decode_ingress_bf16(const B200KvIngressArgs *s,
                               b200kv_stream stream) {
  if (s == nullptr) return cudaErrorInvalidValue;
  using bf = __nv_bfloat16;
  b200kv::IngressArgs a;
  a.raw_qkv = reinterpret_cast<bf *>(s->raw_qkv);
  a.x = reinterpret_cast<const bf *>(s->x);
  a.input_norm_weight = reinterpret_cast<const bf *>(s->input_norm_weight);
  a.qkv_proj_col_major = reinterpret_cast<const bf *>(s->qkv_proj_col_major);
  a.rows = s->batch_count;
  a.hidden = s->hidden_size;
  a.cols = s->cols;
  a.q_width = s->q_width;
  a.k_width = s->k_width;
  a.norm_mode = s->norm_mode;
  a.status = s->status;
  return b200kv::decode_ingress_bf16(a, static_cast<cudaStream_t>(stream));
}

int b200kv_decode_egress_bf16(const B200KvEgressArgs *s, b200kv_stream stream) {
  if (s == nullptr) return cudaErrorInvalidValue;
  using bf = __nv_bfloat16;
  b200kv::EgressArgs a;
  a.residual_out = reinterpret_cast<bf *>(s->residual_out);
  a.normed_out = reinterpret_cast<bf *>(s->normed_out);
  a.ffn_residual = reinterpret_cast<bf *>(s->ffn_residual);
  a.ffn_x = reinterpret_cast<bf *>(s->ffn_x);
  a.attention_out = reinterpret_cast<const bf *>(s->attention_out);
  a.o_proj_col_major = reinterpret_cast<const bf *>(s->o_proj_col_major);
  a.post_norm_weight = reinterpret_cast<const bf *>(s->post_norm_weight);
  a.pre_ffn_norm_weight = reinterpret_cast<const bf *>(s->pre_ffn_norm_weight);
  a.x = reinterpret_cast<const bf *>(s->x);
  a.ticket = s->ticket;
  a.rows = s->batch_count;
  a.hidden = s->hidden_size;
  a.attention_width = s->attention_width;
  a.norm_mode = s->norm_mode;
  a.status = s->status;
  return b200kv::decode_egress_bf16(a, static_cast<cudaStream_t>(stream));
}

int b200kv_decode_attention_layer_bf16(const B200KvAttentionLayerArgs *s,
                                       b200kv_stream stream) {
  if (s == nullptr) return cudaErrorInvalidValue;
  const B200KvLayerStepArgs &kv = s->kv;
  const Gemma4KvCacheConfig &cfg = kv.cache_config;
  if (kv.batch_count < 0 || kv.q_heads <= 0 || cfg.head_dim <= 0 ||
      cfg.num_heads <= 0 || s->raw_qkv == nullptr) {
    return cudaErrorInvalidValue;
  }
  if (kv.batch_count == 0) return cudaSuccess;
  const int32_t q_width = kv.q_heads * cfg.head_dim;
  const int32_t k_width = cfg.num_heads * cfg.head_dim;
  const int32_t cols = q_width + k_width * (s->has_v_projection ? 2 : 1);
  const int64_t rows = kv.batch_count;

  B200KvIngressArgs in = {};
  in.raw_qkv = s->raw_qkv;
  in.x = s->attention_x;
  in.input_norm_weight = s->attention_input_norm_weight;
  in.qkv_proj_col_major = s->attention_qkv_proj_col_major;
  in.batch_count = kv.batch_count;
  in.hidden_size = s->hidden_size;
  in.cols = cols;
  in.q_width = q_width;
  in.k_width = k_width;
  in.norm_mode = kv.norm_mode;
  in.status = kv.status;
  int st = b200kv_decode_ingress_bf16(&in, stream);
  if (st != cudaSuccess) return st;

  B200KvLayerStepArgs step = kv;
  step.raw_q = s->raw_qkv;
  step.raw_k = s->raw_qkv + rows * q_width;
  step.raw_v = s->has_v_projection ? s->raw_qkv + rows * (q_width + k_width)
                                   : nullptr;
  st = layer_step(&step, true, stream);
  if (st != cudaSuccess) return st;

  B200KvEgressArgs out = {};
  out.residual_out = s->residual_out;
  out.normed_out = s->normed_out;
  out.ffn_residual = s->ffn_residual;
  out.ffn_x = s->ffn_x;
  out.attention_out = kv.out;
  out.o_proj_col_major = s->attention_o_proj_col_major;
  out.post_norm_weight = s->attention_post_norm_weight;
  out.pre_ffn_norm_weight = s->attention_pre_ffn_norm_weight;
  out.x = s->attention_x;
  out.ticket = s->ticket;
  out.batch_count = kv.batch_count;
  out.hidden_size = s->hidden_size;
  out.attention_width = q_width;
  out.norm_mode = kv.norm_mode;
  out.status = kv.status;
  return b200kv_decode_egress_bf16(&out, stream);
}

int b200kv_peer_buffer_create(int64_t slot_bytes, int32_t world, int32_t rank,
                              void **handle, void *export_64_bytes) {
  return b200kv::peer_buffer_create(slot_bytes, world, rank, handle,
                                    export_64_bytes);
}

int b200kv_peer_buffer_connect(void *handle, const void *exports) {
  return b200kv::peer_buffer_connect(handle, exports);
}

int b200kv_peer_allgather(void *handle, const void *src, int64_t bytes,
                          int32_t *status, b200kv_stream stream,
                          void **gathered) {
  return b200kv::peer_allgather(handle, src, bytes, status,
                                static_cast<cudaStream_t>(stream), gathered);
}

int b200kv_peer_merge_attention(void *handle, b200kv_bf16 *merged_out,
                                float *merged_lse, const b200kv_bf16 *out,
                                const float *lse, int32_t rows, int32_t head_dim,
                                int32_t *status, b200kv_stream stream) {
  using bf = __nv_bfloat16;
  return b200kv::peer_merge_attention(
      handle, reinterpret_cast<bf *>(merged_out), merged_lse,
      reinterpret_cast<const bf *>(out), lse, rows, head_dim, status,
      static_cast<cudaStream_t>(stream));
}

int b200kv_peer_buffer_destroy(void *handle) {
  return b200kv::peer_buffer_destroy(handle);
}

int b200kv_peer_buffer_create_loopback(int64_t slot_bytes, int32_t world,
                                       int32_t rank, void **handle) {
  if (handle == nullptr) return cudaErrorInvalidValue;
  return b200kv::peer_buffer_create_loopback(slot_bytes, world, rank, handle);
}

int b200kv_peer_buffer_set_wait_clocks(void *handle, int64_t clocks) {
  return b200kv::peer_buffer_set_wait_clocks(handle, clocks);
}

int b200kv_peer_buffer_post(void *handle, int32_t from_rank, uint32_t epoch,
                            b200kv_stream stream) {
  return b200kv::peer_buffer_post(handle, from_rank, epoch,
                                  static_cast<cudaStream_t>(stream));
}

int b200kv_peer_buffer_reset(void *handle) {
  return b200kv::peer_buffer_reset(handle);
}

int b200kv_peer_buffer_gathered(void *handle, void **gathered) {
  return b200kv::peer_buffer_gathered(handle, gathered);
}

int b200kv_bounded_wait_selftest(int64_t clock_limit, int32_t *d_status,
                                 int64_t *d_waited_clocks, b200kv_stream stream) {
  return b200kv::bounded_wait_selftest(
      clock_limit, d_status, reinterpret_cast<long long *>(d_waited_clocks),
      static_cast<cudaStream_t>(stream));
}

// ---------------------------------------------------------------------------
// Partition of the path over the GPUs of a node (host bookkeeping only).
// ---------------------------------------------------------------------------
int32_t b200kv_shard_sequences(const int64_t *h_live_keys, int32_t sequences,
                               int32_t world, int32_t *h_owner) {
  if (h_live_keys == nullptr || h_owner == nullptr || sequences < 0 || world <= 0) {
    return -1;
  }
  // greedy, longest first: every sequence goes to the rank with the least keys
  std::vector<int32_t> order(static_cast<size_t>(sequences));
  for (int32_t i = 0; i < sequences; ++i) order[size_t(i)] = i;
  std::stable_sort(order.begin(), order.end(), [&](int32_t a, int32_t b) {
    return h_live_keys[a] > h_live_keys[b];
  });
  std::vector<int64_t> load(static_cast<size_t>(world), 0);
  for (const int32_t i : order) {
    const int32_t r =
        int32_t(std::min_element(load.begin(), load.end()) - load.begin());
    h_owner[i] = r;
    load[size_t(r)] += h_live_keys[i];
  }
  return 0;
}

int32_t b200kv_kv_head_range(int32_t kv_heads, int32_t world, int32_t rank,
                             int32_t *first_head, int32_t *head_count) {
  if (kv_heads <= 0 || world <= 0 || rank < 0 || rank >= world ||
      kv_heads % world != 0 || first_head == nullptr || head_count == nullptr) {
    return -1;
  }
  *head_count = kv_heads / world;
  *first_head = rank * *head_count;
  return 0;
}

int32_t b200kv_key_range_page_table(const int32_t *h_page_table,
                                    int32_t max_pages_per_seq, int32_t seq_len,
                                    int32_t page_size, int32_t world, int32_t rank,
                                    int32_t *h_rank_table, int32_t *local_length,
                                    int32_t *first_position) {
  if (h_page_table == nullptr || h_rank_table == nullptr || max_pages_per_seq <= 0 ||
      seq_len < 0 || page_size <= 0 || world <= 0 || rank < 0 || rank >= world) {
    return -1;
  }
  const int32_t pages = std::min(b200kv::div_up(seq_len, page_size), max_pages_per_seq);
  const int32_t per = b200kv::div_up(pages, world);
  const int32_t lo = std::min(rank * per, pages);
  const int32_t hi = std::min((rank + 1) * per, pages);
  for (int32_t i = 0; i < max_pages_per_seq; ++i) {
    h_rank_table[i] = i < hi - lo ? h_page_table[lo + i] : -1;
  }
  const int32_t first = lo * page_size;
  if (local_length != nullptr) {
    *local_length = std::max(0, std::min(seq_len, hi * page_size) - first);
  }
  if (first_position != nullptr) *first_position = first;
  return 0;
}

int b200kv_timer_create(void **event) {
  if (event == nullptr) return cudaErrorInvalidValue;
  cudaEvent_t ev = nullptr;
  const cudaError_t st = cudaEventCreate(&ev);
  *event = ev;
  return st;
}

int b200kv_timer_destroy(void *event) {
  return event == nullptr ? cudaSuccess
                          : cudaEventDestroy(static_cast<cudaEvent_t>(event));
}

int b200kv_timer_record(void *event, b200kv_stream stream) {
  if (event == nullptr) return cudaErrorInvalidValue;
  return cudaEventRecord(static_cast<cudaEvent_t>(event),
                         static_cast<cudaStream_t>(stream));
}

int b200kv_timer_elapsed_ms(void *begin, void *end, float *ms) {
  if (begin == nullptr || end == nullptr || ms == nullptr) {
    return cudaErrorInvalidValue;
  }
  return cudaEventElapsedTime(ms, static_cast<cudaEvent_t>(begin),
                              static_cast<cudaEvent_t>(end));
}

int32_t b200kv_compiled_arch(void) { return 1000; }

}  // extern "C"

// CPU oracle for the gemma.c KV-cache hot path. TEST INFRASTRUCTURE ONLY:
// used by tests, by the smoke check and as the timed CPU baseline. See
// kv_oracle.h for the pinning statement. Build with -ffp-contract=off so that
// every fp32 operation below rounds exactly where it is written.
#include "kv_oracle.h"

#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstring>
#include <limits>
#include <thread>
#include <vector>

namespace {

constexpr int kWarp = 32;
constexpr float kEps = 1.0e-6f;  // GEMMA4_RMS_NORM_EPS, src/gemma4.h:29
constexpr int kNumLayers = 48;   // src/gemma4.h:8
constexpr int kGlobalPeriod = 6; // src/gemma4.h:11
constexpr int kSlidingWindow = 1024;  // src/gemma4.h:23

inline float bf(uint16_t x) {
  uint32_t u = uint32_t(x) << 16;
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}

// Round-to-nearest-even fp32 -> bf16, NaN -> 0x7FFF (the behaviour of
// __float2bfloat16_rn used throughout the reference, e.g. rope.cu:18-19).
inline uint16_t to_bf(float f) {
  uint32_t u;
  std::memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return 0x7fff;
  const uint32_t lsb = (u >> 16) & 1u;
  u += 0x7fffu + lsb;
  return uint16_t(u >> 16);
}

inline int64_t cache_offset(const OrcKvConfig &c, int32_t layer, int32_t page,
                            int32_t off, int32_t head, int32_t dim) {
  // kv_cache.cuh:28-38
  const int64_t layer_page = int64_t(layer) * c.num_pages + page;
  const int64_t token = layer_page * c.page_size + off;
  return (token * c.num_heads + head) * c.head_dim + dim;
}

// Byte index of one K element in the FP8 cache (no counterpart in the
// reference). V keeps the [page, offset, head, dim] order; K pages are stored
// as half-page blocks of 8 tokens, head-major inside a block, and inside each
// 256-byte row the 16-byte granules are XOR-swizzled with the token's parity:
//   [layer][page][token / 8][head][token % 8][granule ^ 4*(token & 1)][16]
// (a block is the unit the decode kernel copies into shared memory, where the
// tensor-core fragment loads of 8 tokens then hit 32 distinct banks).
// Needs page_size % 8 == 0 and head_dim == 256.
inline int64_t fp8_k_index(const OrcKvConfig &c, int32_t layer, int32_t page,
                           int32_t token, int32_t head, int32_t dim) {
  const int64_t page_elems = int64_t(c.page_size) * c.num_heads * c.head_dim;
  const int64_t base = (int64_t(layer) * c.num_pages + page) * page_elems;
  const int block = token >> 3, tk = token & 7;
  const int granule = (dim >> 4) ^ ((tk & 1) << 2);
  return base + int64_t(block) * 8 * c.num_heads * c.head_dim +
         int64_t(head) * 8 * c.head_dim + int64_t(tk) * c.head_dim +
         granule * 16 + (dim & 15);
}

// rmsnorm.cu:90-101 with the lane ownership of decode.cu:216-227 and the xor
// butterfly of cuda_utils.cuh:165-170. The reference's rsqrtf is replaced by
// IEEE 1/sqrt: the one deliberate deviation (the GPU approximation cannot be
// restated on a host).
float warp_rms_scale(const float *x, int head_dim) {
  float ss[kWarp];
  const int per_lane = head_dim / kWarp;
  for (int lane = 0; lane < kWarp; ++lane) {
    float s = 0.0f;
    for (int i = 0; i < per_lane; ++i) {
      const float v = x[lane + i * kWarp];
      s = std::fmaf(v, v, s);
    }
    ss[lane] = s;
  }
  for (int offset = kWarp / 2; offset > 0; offset /= 2) {
    float next[kWarp];
    for (int lane = 0; lane < kWarp; ++lane) {
      next[lane] = ss[lane] + ss[lane ^ offset];
    }
    std::memcpy(ss, next, sizeof(ss));
  }
  const float mean = ss[0] / float(head_dim);
  return 1.0f / std::sqrt(mean + kEps);
}

void prep_weighted_rope(uint16_t *out, const uint16_t *in,
                        const uint16_t *weight, const float *cos_row,
                        const float *sin_row, int head_dim, int rotary_dim) {
  // decode.cu:231-264 + rope.cu:8-20
  std::vector<float> x(head_dim);
  for (int d = 0; d < head_dim; ++d) x[d] = bf(in[d]);
  const float scale = warp_rms_scale(x.data(), head_dim);
  const int half = rotary_dim / 2;
  for (int d = 0; d < half; ++d) {
    const float lo = (x[d] * scale) * bf(weight[d]);
    const float hi = (x[half + d] * scale) * bf(weight[half + d]);
    const float c = cos_row[d];
    const float s = sin_row[d];
    const float lo_c = lo * c;
    const float hi_c = hi * c;
    out[d] = to_bf(std::fmaf(-hi, s, lo_c));
    out[half + d] = to_bf(std::fmaf(lo, s, hi_c));
  }
  for (int d = rotary_dim; d < head_dim; ++d) {
    out[d] = to_bf((x[d] * scale) * bf(weight[d]));
  }
}

void prep_scale_free(uint16_t *out, const uint16_t *in, int head_dim) {
  // decode.cu:268-280
  std::vector<float> x(head_dim);
  for (int d = 0; d < head_dim; ++d) x[d] = bf(in[d]);
  const float scale = warp_rms_scale(x.data(), head_dim);
  for (int d = 0; d < head_dim; ++d) out[d] = to_bf(x[d] * scale);
}

// Address of one appended row; -1 when the write must be dropped
// (kv_cache.cu:25-43 and decode.cu:285-303).
int64_t append_row_offset(const OrcKvConfig &c, const int32_t *page_table,
                          int batch, int position, int layer, int head,
                          bool apply_linear_guard) {
  if (batch < 0 || position < 0) return -1;
  if (batch >= c.batch_size) return -1;
  const int logical_page = position / c.page_size;
  if (apply_linear_guard && c.window_size == 0 &&
      logical_page >= c.max_pages_per_seq) {
    return -1;
  }
  const int slot = logical_page % c.max_pages_per_seq;
  const int physical =
      page_table[int64_t(batch) * c.max_pages_per_seq + slot];
  if (physical < 0 || physical >= c.num_pages) return -1;
  const int off = position - logical_page * c.page_size;
  return cache_offset(c, layer, physical, off, head, 0);
}

// Block-wide sum in the shape of the reference's per-key reduction
// (decode.cu:588-596): a balanced tree inside each 32-dim group followed by a
// running sum over the groups.
float dot_tree(const float *q, const uint16_t *k, int head_dim) {
  float total = 0.0f;
  for (int w = 0; w < head_dim; w += kWarp) {
    float p[kWarp];
    for (int l = 0; l < kWarp; ++l) p[l] = q[w + l] * bf(k[w + l]);
    for (int off = 1; off < kWarp; off *= 2) {
      for (int l = 0; l + off < kWarp; l += 2 * off) p[l] += p[l + off];
    }
    total = (w == 0) ? p[0] : total + p[0];
  }
  return total;
}

// Same value up to fp32 summation order; written so the compiler vectorises
// it. Used only by the timed CPU baseline.
float dot_fast(const float *q, const uint16_t *k, int head_dim) {
  float lanes[16] = {0};
  for (int d = 0; d < head_dim; d += 16) {
    for (int j = 0; j < 16; ++j) lanes[j] += q[d + j] * bf(k[d + j]);
  }
  float total = 0.0f;
  for (int j = 0; j < 16; ++j) total += lanes[j];
  return total;
}

struct LiveRange {
  int first_key;
  int key_count;
  int actual_splits;
};

LiveRange live_range(const OrcKvConfig &c, int seq_len, int split_size) {
  // decode.cu:728-733
  LiveRange r;
  r.first_key = c.window_size > 0 ? std::max(0, seq_len - c.window_size) : 0;
  r.key_count = std::max(0, seq_len - r.first_key);
  r.actual_splits = (r.key_count + split_size - 1) / split_size;
  return r;
}

// One (batch, kv_head, split) task of decode.cu:692-878.
template <bool Fast>
void split_task(uint16_t *out, float *partial_m, float *partial_l,
                float *partial_acc, const uint16_t *q,
                const uint16_t *cache_k, const uint16_t *cache_v,
                const int32_t *page_table, const int32_t *seq_lengths,
                const OrcKvConfig &c, int layer, float scale, int split_size,
                int num_splits, int batch, int kv_head, int split,
                int q_heads) {
  const int D = c.head_dim;
  const int G = q_heads / c.num_heads;
  const int seq_len = seq_lengths[batch];
  const LiveRange r = live_range(c, seq_len, split_size);
  const bool write_direct = num_splits == 1;
  if (r.key_count == 0 && write_direct) {
    for (int g = 0; g < G; ++g) {
      const int64_t row = int64_t(batch) * q_heads + kv_head * G + g;
      for (int d = 0; d < D; ++d) out[row * D + d] = to_bf(0.0f);
    }
    return;
  }
  if (split >= r.actual_splits) return;  // decode.cu:746-748
  const int split_begin = r.first_key + split * split_size;
  const int split_end = std::min(seq_len, split_begin + split_size);

  std::vector<float> qv(size_t(G) * D), acc(size_t(G) * D, 0.0f);
  std::vector<float> m(G, -std::numeric_limits<float>::infinity()), l(G, 0.0f);
  for (int g = 0; g < G; ++g) {
    const int64_t row = int64_t(batch) * q_heads + kv_head * G + g;
    for (int d = 0; d < D; ++d) qv[size_t(g) * D + d] = bf(q[row * D + d]);
  }

  for (int pos = split_begin; pos < split_end;) {
    // decode.cu:791-812: one page-table load per page span.
    const int logical_page = pos / c.page_size;
    const int off0 = pos - logical_page * c.page_size;
    const int span_end = std::min(split_end, pos + c.page_size - off0);
    const int slot = logical_page % c.max_pages_per_seq;
    const int physical =
        page_table[int64_t(batch) * c.max_pages_per_seq + slot];
    if (physical < 0 || physical >= c.num_pages) {
      pos = span_end;
      continue;
    }
    int64_t base = cache_offset(c, layer, physical, off0, kv_head, 0);
    const int64_t stride = int64_t(c.num_heads) * D;
    for (; pos < span_end; ++pos, base += stride) {
      const uint16_t *krow = cache_k + base;
      const uint16_t *vrow = cache_v + base;
      for (int g = 0; g < G; ++g) {
        const float *qg = qv.data() + size_t(g) * D;
        const float score =
            (Fast ? dot_fast(qg, krow, D) : dot_tree(qg, krow, D)) * scale;
        // decode.cu:530-542
        const float new_m = std::max(m[g], score);
        const float old_scale = std::exp(m[g] - new_m);
        const float new_scale = std::exp(score - new_m);
        float *ag = acc.data() + size_t(g) * D;
        for (int d = 0; d < D; ++d) {
          ag[d] = ag[d] * old_scale + bf(vrow[d]) * new_scale;
        }
        l[g] = l[g] * old_scale + new_scale;
        m[g] = new_m;
      }
    }
  }

  for (int g = 0; g < G; ++g) {
    const int64_t row = int64_t(batch) * q_heads + kv_head * G + g;
    const float *ag = acc.data() + size_t(g) * D;
    if (write_direct) {  // decode.cu:849-863
      for (int d = 0; d < D; ++d) {
        out[row * D + d] = to_bf(l[g] > 0.0f ? ag[d] / l[g] : 0.0f);
      }
    } else {  // decode.cu:865-877
      const int64_t p = row * num_splits + split;
      partial_m[p] = m[g];
      partial_l[p] = l[g];
      std::memcpy(partial_acc + p * D, ag, sizeof(float) * D);
    }
  }
}

// One (batch, q_head) row of decode.cu:881-977.
void reduce_row(uint16_t *out, const float *partial_m, const float *partial_l,
                const float *partial_acc, const int32_t *seq_lengths,
                const OrcKvConfig &c, int split_size, int num_splits,
                int batch, int q_head, int q_heads) {
  const int D = c.head_dim;
  const int64_t row = int64_t(batch) * q_heads + q_head;
  const LiveRange r = live_range(c, seq_lengths[batch], split_size);
  const int reduce_splits = std::min(r.actual_splits, num_splits);
  if (reduce_splits == 0) {
    for (int d = 0; d < D; ++d) out[row * D + d] = to_bf(0.0f);
    return;
  }
  const float *pm = partial_m + row * num_splits;
  const float *pl = partial_l + row * num_splits;
  float M = -std::numeric_limits<float>::infinity();
  for (int s = 0; s < reduce_splits; ++s) M = std::max(M, pm[s]);
  float L = 0.0f;
  for (int s = 0; s < reduce_splits; ++s) {
    if (pl[s] > 0.0f) L += pl[s] * std::exp(pm[s] - M);
  }
  for (int d = 0; d < D; ++d) {
    float value = 0.0f;
    for (int s = 0; s < reduce_splits; ++s) {
      if (pl[s] > 0.0f) {
        value += partial_acc[(row * num_splits + s) * D + d] *
                 std::exp(pm[s] - M);
      }
    }
    out[row * D + d] = to_bf(L > 0.0f ? value / L : 0.0f);
  }
}

void append_unit(uint16_t *q_prepared, uint16_t *cache_k, uint16_t *cache_v,
                 const OrcKvConfig &c, const int32_t *page_table,
                 const int32_t *token_position, int cache_layer,
                 const uint16_t *q, const uint16_t *k, const uint16_t *v,
                 const uint16_t *q_w, const uint16_t *k_w,
                 const float *cos_table, const float *sin_table, int batch,
                 int kv_head, int q_heads, int rotary_dim, bool has_v_proj) {
  // decode.cu:305-375
  const int D = c.head_dim;
  const int G = q_heads / c.num_heads;
  const int half = rotary_dim / 2;
  const int position = token_position[batch];
  if (position < 0) return;
  const float *cos_row = cos_table + int64_t(position) * half;
  const float *sin_row = sin_table + int64_t(position) * half;
  for (int g = 0; g < G; ++g) {
    const int64_t off = (int64_t(batch) * q_heads + kv_head * G + g) * D;
    prep_weighted_rope(q_prepared + off, q + off, q_w, cos_row, sin_row, D,
                       rotary_dim);
  }
  // The fused append has no linear-capacity guard of its own
  // (decode.cu:285-303): the slot is the logical page modulo the table width.
  const int64_t dst = append_row_offset(c, page_table, batch, position,
                                        cache_layer, kv_head, false);
  if (dst < 0) return;
  const int64_t src = (int64_t(batch) * c.num_heads + kv_head) * D;
  prep_weighted_rope(cache_k + dst, k + src, k_w, cos_row, sin_row, D,
                     rotary_dim);
  prep_scale_free(cache_v + dst, has_v_proj ? v + src : k + src, D);
}

template <typename Fn>
void parallel_for(int threads, int count, Fn fn) {
  if (threads <= 1 || count <= 1) {
    for (int i = 0; i < count; ++i) fn(i);
    return;
  }
  std::vector<std::thread> pool;
  const int n = std::min(threads, count);
  for (int t = 0; t < n; ++t) {
    pool.emplace_back([=]() {
      for (int i = t; i < count; i += n) fn(i);
    });
  }
  for (auto &th : pool) th.join();
}

// e4m3 (fn flavour: bias 7, max 448, no inf) round-to-nearest-even with
// saturation to +-448; NaN -> 0x7F.
uint8_t enc_e4m3(float x) {
  uint32_t u;
  std::memcpy(&u, &x, 4);
  const uint8_t sign = uint8_t((u >> 24) & 0x80u);
  const float a = std::fabs(x);
  if (a != a) return uint8_t(sign | 0x7f);
  if (a >= 464.0f) return uint8_t(sign | 0x7e);  // rounds to or beyond 448
  if (a < 0.0009765625f) return sign;  // below half of the 2^-9 quantum
  int e;
  std::frexp(a, &e);  // a = f * 2^e, f in [0.5, 1)
  int exp = e - 1;    // a in [2^exp, 2^(exp+1))
  if (exp < -6) exp = -6;
  const float quantum = std::ldexp(1.0f, exp - 3);
  const float q = std::nearbyint(a / quantum);  // default mode: ties-to-even
  int mant = int(q);                             // in [0, 16]
  int biased;
  if (exp == -6 && mant < 8) {
    biased = 0;  // subnormal
  } else {
    if (mant == 16) {
      mant = 8;
      ++exp;
    }
    biased = exp + 7;
    mant -= 8;
  }
  int code = (biased << 3) | mant;
  if (code > 0x7e) code = 0x7e;
  return uint8_t(sign | code);
}

float dec_e4m3(uint8_t x) {
  const int sign = x & 0x80;
  const int biased = (x >> 3) & 0xf;
  const int mant = x & 7;
  float v;
  if (biased == 0xf && mant == 7) {
    v = std::numeric_limits<float>::quiet_NaN();
  } else if (biased == 0) {
    v = std::ldexp(float(mant), -9);
  } else {
    v = std::ldexp(float(8 + mant), biased - 7 - 3);
  }
  return sign ? -v : v;
}

struct RuntimeImpl {
  int32_t batch_size, max_seq_len, page_size, token_count;
  OrcKvConfig sliding, global;
  std::vector<int32_t> sliding_table, global_table, sliding_slots,
      global_slots, seq_lengths, token_batch, token_position;
};

}  // namespace

struct OrcRuntime {
  RuntimeImpl impl;
};

extern "C" {

uint16_t orc_f32_to_bf16(float x) { return to_bf(x); }
float orc_bf16_to_f32(uint16_t x) { return bf(x); }
void orc_f32_to_bf16_n(uint16_t *out, const float *in, int64_t n) {
  for (int64_t i = 0; i < n; ++i) out[i] = to_bf(in[i]);
}
void orc_bf16_to_f32_n(float *out, const uint16_t *in, int64_t n) {
  for (int64_t i = 0; i < n; ++i) out[i] = bf(in[i]);
}
uint8_t orc_f32_to_e4m3(float x) { return enc_e4m3(x); }
float orc_e4m3_to_f32(uint8_t x) { return dec_e4m3(x); }

int64_t orc_cache_offset(const OrcKvConfig *cfg, int32_t layer, int32_t page,
                         int32_t page_offset, int32_t head, int32_t dim) {
  return cache_offset(*cfg, layer, page, page_offset, head, dim);
}

int32_t orc_is_global_layer(int32_t layer) {
  // gemma4.h:105-108
  return layer == kNumLayers - 1 || (layer + 1) % kGlobalPeriod == 0;
}

void orc_make_config(OrcKvConfig *out, int32_t global, int32_t num_pages,
                     int32_t page_size, int32_t max_pages_per_seq) {
  // kv_cache.cu:76-91 with the constants of gemma4.h:8-23
  const int global_layers =
      kNumLayers / kGlobalPeriod + (kNumLayers % kGlobalPeriod != 0 ? 1 : 0);
  out->num_layers = global ? global_layers : kNumLayers - global_layers;
  out->num_pages = num_pages;
  out->page_size = page_size;
  out->max_pages_per_seq = max_pages_per_seq;
  out->batch_size = num_pages / max_pages_per_seq;
  out->num_heads = global ? 1 : 8;
  out->head_dim = global ? 512 : 256;
  out->window_size = global ? 0 : kSlidingWindow;
}

int32_t orc_layer_index(int32_t model_layer, int32_t global_cache) {
  // kv_cache.cu:94-105
  if (model_layer < 0 || model_layer >= kNumLayers) return -1;
  if ((orc_is_global_layer(model_layer) != 0) != (global_cache != 0)) {
    return -1;
  }
  int32_t index = 0;
  for (int32_t layer = 0; layer < model_layer; ++layer) {
    if ((orc_is_global_layer(layer) != 0) == (global_cache != 0)) ++index;
  }
  return index;
}

int32_t orc_ensure_page(int32_t *page_table, int32_t *slot_logical_pages,
                        const OrcKvConfig *cfg, int32_t batch,
                        int32_t position) {
  // kv_cache.cu:108-123
  const int32_t logical_page = position / cfg->page_size;
  const int32_t slot = logical_page % cfg->max_pages_per_seq;
  const int64_t index = int64_t(batch) * cfg->max_pages_per_seq + slot;
  if (slot_logical_pages[index] > logical_page) return -1;
  const int32_t physical = batch * cfg->max_pages_per_seq + slot;
  page_table[index] = physical;
  slot_logical_pages[index] = logical_page;
  return physical;
}

int32_t orc_ensure_range(int32_t *page_table, int32_t *slot_logical_pages,
                         const OrcKvConfig *cfg, int32_t batch,
                         int32_t first_position, int32_t token_count) {
  // kv_cache.cu:126-146
  if (token_count == 0) return 0;
  const int32_t first_page = first_position / cfg->page_size;
  const int32_t last_page =
      (first_position + token_count - 1) / cfg->page_size;
  for (int32_t page = first_page; page <= last_page; ++page) {
    if (orc_ensure_page(page_table, slot_logical_pages, cfg, batch,
                        page * cfg->page_size) < 0) {
      return -1;
    }
  }
  return 0;
}

int32_t orc_sliding_pages_per_sequence(int32_t max_seq_len,
                                       int32_t page_size) {
  // runtime.cu:18-24
  if (max_seq_len <= kSlidingWindow) {
    return (max_seq_len + page_size - 1) / page_size;
  }
  return (kSlidingWindow + page_size - 1 + page_size - 1) / page_size;
}

OrcRuntime *orc_runtime_create(int32_t batch_size, int32_t max_seq_len,
                               int32_t page_size) {
  // runtime.cu:95-136 (host bookkeeping part)
  if (batch_size <= 0 || max_seq_len <= 0 || page_size <= 0 ||
      max_seq_len > 262144) {
    return nullptr;
  }
  OrcRuntime *rt = new OrcRuntime();
  RuntimeImpl &s = rt->impl;
  s.batch_size = batch_size;
  s.max_seq_len = max_seq_len;
  s.page_size = page_size;
  s.token_count = 0;
  const int32_t global_pps = (max_seq_len + page_size - 1) / page_size;
  const int32_t sliding_pps =
      orc_sliding_pages_per_sequence(max_seq_len, page_size);
  orc_make_config(&s.sliding, 0, batch_size * sliding_pps, page_size,
                  sliding_pps);
  s.sliding.batch_size = batch_size;
  s.sliding.window_size = std::min(max_seq_len, kSlidingWindow);
  orc_make_config(&s.global, 1, batch_size * global_pps, page_size,
                  global_pps);
  s.global.batch_size = batch_size;
  s.sliding_table.assign(size_t(batch_size) * sliding_pps, -1);
  s.global_table.assign(size_t(batch_size) * global_pps, -1);
  s.sliding_slots.assign(s.sliding_table.size(), -1);
  s.global_slots.assign(s.global_table.size(), -1);
  s.seq_lengths.assign(batch_size, 0);
  s.token_batch.assign(size_t(batch_size) * max_seq_len, 0);
  s.token_position.assign(size_t(batch_size) * max_seq_len, 0);
  return rt;
}

void orc_runtime_destroy(OrcRuntime *rt) { delete rt; }

int32_t orc_runtime_prepare_prefill(OrcRuntime *rt, int32_t seq_len) {
  // runtime.cu:237-273
  RuntimeImpl &s = rt->impl;
  if (seq_len < 0 || seq_len > s.max_seq_len) return -1;
  std::fill(s.sliding_table.begin(), s.sliding_table.end(), -1);
  std::fill(s.global_table.begin(), s.global_table.end(), -1);
  std::fill(s.sliding_slots.begin(), s.sliding_slots.end(), -1);
  std::fill(s.global_slots.begin(), s.global_slots.end(), -1);
  for (int32_t b = 0; b < s.batch_size; ++b) {
    if (orc_ensure_range(s.sliding_table.data(), s.sliding_slots.data(),
                         &s.sliding, b, 0, seq_len) < 0) {
      return -1;
    }
    if (orc_ensure_range(s.global_table.data(), s.global_slots.data(),
                         &s.global, b, 0, seq_len) < 0) {
      return -1;
    }
    s.seq_lengths[b] = seq_len;
    for (int32_t pos = 0; pos < seq_len; ++pos) {
      const size_t row = size_t(b) * seq_len + pos;
      s.token_batch[row] = b;
      s.token_position[row] = pos;
    }
  }
  s.token_count = s.batch_size * seq_len;
  return 0;
}

int32_t orc_runtime_prepare_decode_step(OrcRuntime *rt) {
  // runtime.cu:276-341: validate every sequence before mutating anything.
  RuntimeImpl &s = rt->impl;
  for (int32_t b = 0; b < s.batch_size; ++b) {
    const int32_t pos = s.seq_lengths[b];
    if (pos < 0 || pos >= s.max_seq_len) return -1;
  }
  for (int32_t b = 0; b < s.batch_size; ++b) {
    const int32_t pos = s.seq_lengths[b];
    if (orc_ensure_page(s.sliding_table.data(), s.sliding_slots.data(),
                        &s.sliding, b, pos) < 0) {
      return -1;
    }
    if (orc_ensure_page(s.global_table.data(), s.global_slots.data(),
                        &s.global, b, pos) < 0) {
      return -1;
    }
    s.token_batch[b] = b;
    s.token_position[b] = pos;
  }
  for (int32_t b = 0; b < s.batch_size; ++b) ++s.seq_lengths[b];
  s.token_count = s.batch_size;
  return 0;
}

int64_t orc_runtime_array(OrcRuntime *rt, int32_t which, int32_t **data) {
  RuntimeImpl &s = rt->impl;
  std::vector<int32_t> *v = nullptr;
  switch (which) {
    case 0: v = &s.sliding_table; break;
    case 1: v = &s.global_table; break;
    case 2: v = &s.sliding_slots; break;
    case 3: v = &s.global_slots; break;
    case 4: v = &s.seq_lengths; break;
    case 5: v = &s.token_batch; break;
    case 6: v = &s.token_position; break;
    default: *data = nullptr; return -1;
  }
  *data = v->data();
  return int64_t(v->size());
}

void orc_runtime_configs(OrcRuntime *rt, OrcKvConfig *sliding,
                         OrcKvConfig *global, int32_t *token_count) {
  *sliding = rt->impl.sliding;
  *global = rt->impl.global;
  *token_count = rt->impl.token_count;
}

void orc_fill_rope_tables(float *cos_table, float *sin_table,
                          int32_t max_seq_len, int32_t rotary_half,
                          float theta, int32_t exponent_dim) {
  // runtime.cu:27-45: everything in fp32, std::pow/cos/sin float overloads.
  for (int32_t pos = 0; pos < max_seq_len; ++pos) {
    for (int32_t i = 0; i < rotary_half; ++i) {
      const float exponent = -2.0f * float(i) / float(exponent_dim);
      const float angle = float(pos) * std::pow(theta, exponent);
      const size_t off = size_t(pos) * rotary_half + i;
      cos_table[off] = std::cos(angle);
      sin_table[off] = std::sin(angle);
    }
  }
}

float orc_rms_scale(const uint16_t *head, int32_t head_dim, float eps) {
  (void)eps;
  std::vector<float> x(head_dim);
  for (int d = 0; d < head_dim; ++d) x[d] = bf(head[d]);
  return warp_rms_scale(x.data(), head_dim);
}

void orc_prep_weighted_rope_head(uint16_t *out, const uint16_t *in,
                                 const uint16_t *weight, const float *cos_row,
                                 const float *sin_row, int32_t head_dim,
                                 int32_t rotary_dim) {
  prep_weighted_rope(out, in, weight, cos_row, sin_row, head_dim, rotary_dim);
}

void orc_prep_scale_free_head(uint16_t *out, const uint16_t *in,
                              int32_t head_dim) {
  prep_scale_free(out, in, head_dim);
}

void orc_prefill_prep(uint16_t *q_prepared, uint16_t *k_prepared,
                      uint16_t *v_prepared, const uint16_t *q,
                      const uint16_t *k, const uint16_t *v,
                      const uint16_t *q_w, const uint16_t *k_w,
                      const float *cos_table, const float *sin_table,
                      const int32_t *token_position, int64_t rows,
                      int32_t q_heads, int32_t kv_heads, int32_t head_dim,
                      int32_t rotary_dim, int32_t has_v_proj) {
  // prefill.cu:1022-1081: rows with a negative position are left untouched.
  const int half = rotary_dim / 2;
  for (int64_t row = 0; row < rows; ++row) {
    const int position = token_position[row];
    if (position < 0) continue;
    const float *cos_row = cos_table + int64_t(position) * half;
    const float *sin_row = sin_table + int64_t(position) * half;
    for (int h = 0; h < q_heads; ++h) {
      const int64_t off = (row * q_heads + h) * head_dim;
      prep_weighted_rope(q_prepared + off, q + off, q_w, cos_row, sin_row,
                         head_dim, rotary_dim);
    }
    for (int h = 0; h < kv_heads; ++h) {
      const int64_t off = (row * kv_heads + h) * head_dim;
      prep_weighted_rope(k_prepared + off, k + off, k_w, cos_row, sin_row,
                         head_dim, rotary_dim);
      prep_scale_free(v_prepared + off, has_v_proj ? v + off : k + off,
                      head_dim);
    }
  }
}

int32_t orc_kv_cache_write(uint16_t *cache_k, uint16_t *cache_v,
                           const OrcKvConfig *cfg, const int32_t *page_table,
                           const int32_t *token_batch,
                           const int32_t *token_position, int32_t token_count,
                           int32_t layer, const uint16_t *k,
                           const uint16_t *v) {
  // kv_cache.cu:149-180 (argument checks) and :11-56 (row copy)
  const OrcKvConfig &c = *cfg;
  if (token_count == 0) return 0;
  if (token_count < 0 || layer < 0 || layer >= c.num_layers ||
      c.num_pages <= 0 || c.page_size <= 0 || c.max_pages_per_seq <= 0 ||
      c.batch_size <= 0 || c.window_size < 0 || c.num_heads <= 0 ||
      c.head_dim <= 0 || c.head_dim % 8 != 0 || !cache_k || !cache_v ||
      !page_table || !token_batch || !token_position || !k || !v) {
    return 1;  // cudaErrorInvalidValue
  }
  for (int32_t t = 0; t < token_count; ++t) {
    for (int32_t h = 0; h < c.num_heads; ++h) {
      const int64_t dst = append_row_offset(c, page_table, token_batch[t],
                                            token_position[t], layer, h, true);
      if (dst < 0) continue;
      const int64_t src = (int64_t(t) * c.num_heads + h) * c.head_dim;
      std::memcpy(cache_k + dst, k + src, sizeof(uint16_t) * c.head_dim);
      std::memcpy(cache_v + dst, v + src, sizeof(uint16_t) * c.head_dim);
    }
  }
  return 0;
}

void orc_decode_append(uint16_t *q_prepared, uint16_t *cache_k,
                       uint16_t *cache_v, const OrcKvConfig *cfg,
                       const int32_t *page_table,
                       const int32_t *token_position, int32_t cache_layer,
                       const uint16_t *q, const uint16_t *k,
                       const uint16_t *v, const uint16_t *q_w,
                       const uint16_t *k_w, const float *cos_table,
                       const float *sin_table, int32_t batch_count,
                       int32_t q_heads, int32_t rotary_dim,
                       int32_t has_v_proj) {
  for (int b = 0; b < batch_count; ++b) {
    for (int h = 0; h < cfg->num_heads; ++h) {
      append_unit(q_prepared, cache_k, cache_v, *cfg, page_table,
                  token_position, cache_layer, q, k, v, q_w, k_w, cos_table,
                  sin_table, b, h, q_heads, rotary_dim, has_v_proj != 0);
    }
  }
}

void orc_decode_attention_ref(uint16_t *out, float *partial_m,
                              float *partial_l, float *partial_acc,
                              const uint16_t *q, const uint16_t *cache_k,
                              const uint16_t *cache_v,
                              const int32_t *page_table,
                              const int32_t *seq_lengths,
                              const OrcKvConfig *cfg, int32_t layer,
                              float softmax_scale, int32_t split_size,
                              int32_t num_splits, int32_t batch_count,
                              int32_t q_heads) {
  // Task order of decode.cu:1004-1031 generalised over batch rows.
  for (int b = 0; b < batch_count; ++b) {
    for (int h = 0; h < cfg->num_heads; ++h) {
      for (int s = 0; s < num_splits; ++s) {
        split_task<false>(out, partial_m, partial_l, partial_acc, q, cache_k,
                          cache_v, page_table, seq_lengths, *cfg, layer,
                          softmax_scale, split_size, num_splits, b, h, s,
                          q_heads);
      }
    }
    if (num_splits > 1) {
      for (int qh = 0; qh < q_heads; ++qh) {
        reduce_row(out, partial_m, partial_l, partial_acc, seq_lengths, *cfg,
                   split_size, num_splits, b, qh, q_heads);
      }
    }
  }
}

void orc_decode_attention_f64(float *out_f32, float *lse, const uint16_t *q,
                              const uint16_t *cache_k,
                              const uint16_t *cache_v,
                              const int32_t *page_table,
                              const int32_t *seq_lengths,
                              const OrcKvConfig *cfg, int32_t layer,
                              float softmax_scale, int32_t batch_count,
                              int32_t q_heads) {
  const OrcKvConfig &c = *cfg;
  const int D = c.head_dim;
  const int G = q_heads / c.num_heads;
  // rows are independent: one (sequence, query head) per work item, on all host
  // threads; the arithmetic of a row does not depend on the thread count
  parallel_for(orc_hardware_threads(), batch_count * q_heads, [&](int unit) {
    const int b = unit / q_heads;
    const int seq_len = seq_lengths[b];
    const LiveRange r = live_range(c, seq_len, 1);
    {
      const int qh = unit - b * q_heads;
      const int kvh = qh / G;
      const int64_t row = int64_t(b) * q_heads + qh;
      std::vector<double> scores;
      std::vector<int64_t> bases;
      for (int pos = r.first_key; pos < seq_len; ++pos) {
        const int logical_page = pos / c.page_size;
        const int slot = logical_page % c.max_pages_per_seq;
        const int physical =
            page_table[int64_t(b) * c.max_pages_per_seq + slot];
        if (physical < 0 || physical >= c.num_pages) continue;
        const int64_t base = cache_offset(
            c, layer, physical, pos - logical_page * c.page_size, kvh, 0);
        double s = 0.0;
        for (int d = 0; d < D; ++d) {
          s += double(bf(q[row * D + d])) * double(bf(cache_k[base + d]));
        }
        scores.push_back(s * double(softmax_scale));
        bases.push_back(base);
      }
      if (scores.empty()) {
        for (int d = 0; d < D; ++d) out_f32[row * D + d] = 0.0f;
        lse[row] = -std::numeric_limits<float>::infinity();
        return;
      }
      const double M = *std::max_element(scores.begin(), scores.end());
      double L = 0.0;
      for (double &s : scores) {
        s = std::exp(s - M);
        L += s;
      }
      std::vector<double> acc(D, 0.0);
      for (size_t i = 0; i < scores.size(); ++i) {
        const uint16_t *vrow = cache_v + bases[i];
        for (int d = 0; d < D; ++d) acc[d] += scores[i] * double(bf(vrow[d]));
      }
      for (int d = 0; d < D; ++d) out_f32[row * D + d] = float(acc[d] / L);
      lse[row] = float(M + std::log(L));
    }
  });
}

int64_t orc_fp8_k_index(const OrcKvConfig *cfg, int32_t layer, int32_t page,
                        int32_t token, int32_t head, int32_t dim) {
  return fp8_k_index(*cfg, layer, page, token, head, dim);
}

void orc_fp8_append(uint8_t *cache_k, uint8_t *cache_v, float *scale_k,
                    float *scale_v, const OrcKvConfig *cfg,
                    const int32_t *page_table, const int32_t *seq_batch,
                    const int32_t *first_position, const int32_t *row_count,
                    int32_t seq_count, int32_t layer,
                    const uint16_t *k_prepared, const uint16_t *v_prepared) {
  // Rule (per tensor, per (page, kv head), per call): let R be the rows of
  // this call that land in the page, first offset o0.
  //   s_old = (o0 == 0) ? 0 : scale[page, head]
  //   s_new = max(s_old, max(amax(R) / 448, FLT_MIN))
  //   if s_new > s_old: every stored row r < o0 becomes
  //       enc((dec(byte) * s_old) / s_new)
  //   every row of R is stored as enc(x / s_new); scale[page, head] = s_new.
  // Rows arrive as [sum(row_count), num_heads, head_dim] bf16 in call order.
  const OrcKvConfig &c = *cfg;
  const int D = c.head_dim;
  int64_t src_row = 0;
  for (int s = 0; s < seq_count; ++s) {
    const int b = seq_batch[s];
    const int first = first_position[s];
    const int count = row_count[s];
    const int64_t seq_src_row = src_row;
    src_row += count;
    if (b < 0 || b >= c.batch_size || first < 0) continue;
    for (int pos = first; pos < first + count;) {
      const int logical_page = pos / c.page_size;
      const int o0 = pos - logical_page * c.page_size;
      const int span = std::min(first + count - pos, c.page_size - o0);
      const int page_pos = pos;
      pos += span;
      if (c.window_size == 0 && logical_page >= c.max_pages_per_seq) continue;
      const int slot = logical_page % c.max_pages_per_seq;
      const int physical =
          page_table[int64_t(b) * c.max_pages_per_seq + slot];
      if (physical < 0 || physical >= c.num_pages) continue;
      for (int h = 0; h < c.num_heads; ++h) {
        for (int tensor = 0; tensor < 2; ++tensor) {
          uint8_t *cache = tensor == 0 ? cache_k : cache_v;
          float *scales = tensor == 0 ? scale_k : scale_v;
          const uint16_t *src = tensor == 0 ? k_prepared : v_prepared;
          float *sp = scales +
                      (int64_t(layer) * c.num_pages + physical) * c.num_heads +
                      h;
          float amax = 0.0f;
          for (int r = 0; r < span; ++r) {
            const int64_t row = seq_src_row + (page_pos - first) + r;
            const uint16_t *x = src + (row * c.num_heads + h) * D;
            for (int d = 0; d < D; ++d) amax = std::max(amax, std::fabs(bf(x[d])));
          }
          const float s_old = o0 == 0 ? 0.0f : *sp;
          const float s_row =
              std::max(amax / 448.0f, std::numeric_limits<float>::min());
          const float s_new = std::max(s_old, s_row);
          auto at = [&](int token, int d) -> uint8_t & {
            return cache[tensor == 0
                             ? fp8_k_index(c, layer, physical, token, h, d)
                             : cache_offset(c, layer, physical, token, h, d)];
          };
          if (s_new > s_old) {
            for (int r = 0; r < o0; ++r) {
              for (int d = 0; d < D; ++d) {
                at(r, d) = enc_e4m3((dec_e4m3(at(r, d)) * s_old) / s_new);
              }
            }
          }
          for (int r = 0; r < span; ++r) {
            const int64_t row = seq_src_row + (page_pos - first) + r;
            const uint16_t *x = src + (row * c.num_heads + h) * D;
            for (int d = 0; d < D; ++d) at(o0 + r, d) = enc_e4m3(bf(x[d]) / s_new);
          }
          *sp = s_new;
        }
      }
    }
  }
}

void orc_fp8_decode_attention_f64(float *out_f32, float *lse,
                                  const uint16_t *q, const uint8_t *cache_k,
                                  const uint8_t *cache_v,
                                  const float *scale_k, const float *scale_v,
                                  const int32_t *page_table,
                                  const int32_t *seq_lengths,
                                  const OrcKvConfig *cfg, int32_t layer,
                                  float softmax_scale, int32_t batch_count,
                                  int32_t q_heads) {
  const OrcKvConfig &c = *cfg;
  const int D = c.head_dim;
  const int G = q_heads / c.num_heads;
  parallel_for(orc_hardware_threads(), batch_count * q_heads, [&](int unit) {
    const int b = unit / q_heads;
    const int seq_len = seq_lengths[b];
    const LiveRange r = live_range(c, seq_len, 1);
    {
      const int qh = unit - b * q_heads;
      const int kvh = qh / G;
      const int64_t row = int64_t(b) * q_heads + qh;
      std::vector<double> scores, vscale;
      std::vector<int64_t> bases;
      for (int pos = r.first_key; pos < seq_len; ++pos) {
        const int logical_page = pos / c.page_size;
        const int slot = logical_page % c.max_pages_per_seq;
        const int physical =
            page_table[int64_t(b) * c.max_pages_per_seq + slot];
        if (physical < 0 || physical >= c.num_pages) continue;
        const int64_t base = cache_offset(
            c, layer, physical, pos - logical_page * c.page_size, kvh, 0);
        const int64_t sidx =
            (int64_t(layer) * c.num_pages + physical) * c.num_heads + kvh;
        double s = 0.0;
        const int token = pos - logical_page * c.page_size;
        for (int d = 0; d < D; ++d) {
          s += double(bf(q[row * D + d])) *
               double(dec_e4m3(
                   cache_k[fp8_k_index(c, layer, physical, token, kvh, d)]));
        }
        scores.push_back(s * double(scale_k[sidx]) * double(softmax_scale));
        vscale.push_back(double(scale_v[sidx]));
        bases.push_back(base);
      }
      if (scores.empty()) {
        for (int d = 0; d < D; ++d) out_f32[row * D + d] = 0.0f;
        lse[row] = -std::numeric_limits<float>::infinity();
        return;
      }
      const double M = *std::max_element(scores.begin(), scores.end());
      double L = 0.0;
      for (double &s : scores) {
        s = std::exp(s - M);
        L += s;
      }
      std::vector<double> acc(D, 0.0);
      for (size_t i = 0; i < scores.size(); ++i) {
        const uint8_t *vrow = cache_v + bases[i];
        const double w = scores[i] * vscale[i];
        for (int d = 0; d < D; ++d) acc[d] += w * double(dec_e4m3(vrow[d]));
      }
      for (int d = 0; d < D; ++d) out_f32[row * D + d] = float(acc[d] / L);
      lse[row] = float(M + std::log(L));
    }
  });
}

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
                            int32_t split_size) {
  const OrcKvConfig c = *cfg;
  const int H = c.num_heads;
  int max_splits = 1;
  for (int b = 0; b < batch_count; ++b) {
    max_splits = std::max(
        max_splits, live_range(c, seq_lengths[b], split_size).actual_splits);
  }
  const int num_splits = max_splits;
  std::vector<float> pm, pl, pacc;
  if (num_splits > 1) {
    const size_t rows = size_t(batch_count) * q_heads * num_splits;
    pm.resize(rows);
    pl.resize(rows);
    pacc.resize(rows * c.head_dim);
  }
  const auto t0 = std::chrono::steady_clock::now();
  parallel_for(threads, batch_count * H, [&](int unit) {
    append_unit(q_prepared, cache_k, cache_v, c, page_table, token_position,
                cache_layer, q, k, v, q_w, k_w, cos_table, sin_table,
                unit / H, unit % H, q_heads, c.head_dim, true);
  });
  parallel_for(threads, batch_count * H * num_splits, [&](int task) {
    const int s = task % num_splits;
    const int unit = task / num_splits;
    split_task<true>(out, pm.data(), pl.data(), pacc.data(), q_prepared,
                     cache_k, cache_v, page_table, seq_lengths, c,
                     cache_layer, softmax_scale, split_size, num_splits,
                     unit / H, unit % H, s, q_heads);
  });
  if (num_splits > 1) {
    parallel_for(threads, batch_count * q_heads, [&](int row) {
      reduce_row(out, pm.data(), pl.data(), pacc.data(), seq_lengths, c,
                 split_size, num_splits, row / q_heads, row % q_heads,
                 q_heads);
    });
  }
  const auto t1 = std::chrono::steady_clock::now();
  return std::chrono::duration<double>(t1 - t0).count();
}

// Prompt attention over contiguous prepared rows, the second stage of
// gemma4_flash_attention_{sliding,global}_fwd_bf16_norm_rope
// (src/gemma4_flash_attention_prefill.cu:502-540 for the mask, :1110-1257 for
// the entry points): query row r of a sequence sees keys c <= r and, with a
// window, c >= max(0, r - window + 1). Double precision, direct softmax;
// fp32 output (not rounded) and natural-log LSE.
void orc_prefill_attention_f64(float *out_f32, float *lse, const uint16_t *q,
                               const uint16_t *k, const uint16_t *v,
                               int32_t batch, int32_t seq_len, int32_t q_heads,
                               int32_t kv_heads, int32_t head_dim,
                               int32_t window, float softmax_scale,
                               int32_t threads) {
  const int D = head_dim;
  const int G = q_heads / kv_heads;
  const int units = batch * q_heads;
  auto work = [&](int u0, int u1) {
    std::vector<double> scores, acc(D);
    for (int u = u0; u < u1; ++u) {
      const int b = u / q_heads, h = u % q_heads, kvh = h / G;
      for (int r = 0; r < seq_len; ++r) {
        const int64_t row = int64_t(b) * seq_len + r;
        const uint16_t *qr = q + (row * q_heads + h) * D;
        const int left = window > 0 ? std::max(0, r - window + 1) : 0;
        scores.assign(size_t(r - left + 1), 0.0);
        double M = -std::numeric_limits<double>::infinity();
        for (int c = left; c <= r; ++c) {
          const uint16_t *kr =
              k + ((int64_t(b) * seq_len + c) * kv_heads + kvh) * D;
          double s = 0.0;
          for (int d = 0; d < D; ++d) s += double(bf(qr[d])) * double(bf(kr[d]));
          s *= double(softmax_scale);
          scores[size_t(c - left)] = s;
          M = std::max(M, s);
        }
        double L = 0.0;
        std::fill(acc.begin(), acc.end(), 0.0);
        for (int c = left; c <= r; ++c) {
          const double p = std::exp(scores[size_t(c - left)] - M);
          L += p;
          const uint16_t *vr =
              v + ((int64_t(b) * seq_len + c) * kv_heads + kvh) * D;
          for (int d = 0; d < D; ++d) acc[size_t(d)] += p * double(bf(vr[d]));
        }
        float *o = out_f32 + (row * q_heads + h) * D;
        for (int d = 0; d < D; ++d) o[d] = float(acc[size_t(d)] / L);
        if (lse != nullptr) lse[row * q_heads + h] = float(M + std::log(L));
      }
    }
  };
  const int nt = std::max(1, std::min(threads, units));
  std::vector<std::thread> pool;
  for (int t = 0; t < nt; ++t) {
    pool.emplace_back(work, units * t / nt, units * (t + 1) / nt);
  }
  for (auto &th : pool) th.join();
}

}  // extern "C"

// ---------------------------------------------------------------------------
// Decode projections either side of the KV path: input RMSNorm + [Q|K|V]
// projection into the raw scratch (decode.cu:395-496) and the O projection
// with the post-attention norm and residual (decode.cu:35-129). The summation
// order is the 512-thread block's: thread t chains fmaf over packs t, t+512, ..
// (8 elements each, cuda_utils.cuh:88-103); every warp folds with
// __shfl_down 16..1 (cuda_utils.cuh:174-182); warp 0 folds the 16 warp sums
// the same way with zeros in lanes 16..31 (decode.cu:396-419).
// ---------------------------------------------------------------------------
namespace {

constexpr int kBlockThreads = 512;  // kDecodeMegaThreads, decode.cu:30

inline float shfl_down_tree(float (&v)[kWarp]) {
  for (int offset = kWarp / 2; offset > 0; offset >>= 1) {
    float next[kWarp];
    for (int i = 0; i < kWarp; ++i) {
      next[i] = v[i] + (i + offset < kWarp ? v[i + offset] : v[i]);
    }
    std::memcpy(v, next, sizeof(next));
  }
  return v[0];
}

inline float shfl_xor_tree(float (&v)[kWarp]) {
  // warp_reduce_sum, cuda_utils.cuh:165-170
  for (int offset = kWarp / 2; offset > 0; offset /= 2) {
    float next[kWarp];
    for (int i = 0; i < kWarp; ++i) next[i] = v[i] + v[i ^ offset];
    std::memcpy(v, next, sizeof(next));
  }
  return v[0];
}

// One output column: dot of x with one weight column, both bf16 [width].
// active_threads: threads that take part (480 for the 3840-wide input of the
// QKV projection, decode.cu:430-433; all 512 for the O projection).
inline float block_dot(const uint16_t *x, const uint16_t *w, int width,
                       int active_threads) {
  const int packs = width / 8;
  float warp_sums[kBlockThreads / kWarp];
  for (int warp = 0; warp < kBlockThreads / kWarp; ++warp) {
    float lanes[kWarp];
    for (int lane = 0; lane < kWarp; ++lane) {
      const int t = warp * kWarp + lane;
      float sum = 0.0f;
      if (t < active_threads) {
        for (int pack = t; pack < packs; pack += kBlockThreads) {
          for (int e = 0; e < 8; ++e) {
            sum = std::fmaf(bf(x[pack * 8 + e]), bf(w[pack * 8 + e]), sum);
          }
        }
      }
      lanes[lane] = sum;
    }
    warp_sums[warp] = shfl_down_tree(lanes);
  }
  float lanes[kWarp];
  for (int lane = 0; lane < kWarp; ++lane) {
    lanes[lane] = lane < kBlockThreads / kWarp ? warp_sums[lane] : 0.0f;
  }
  return shfl_down_tree(lanes);
}

// gemma4_rmsnorm_row_bf16 with 512 threads (rmsnorm.cu:27-87), IEEE 1/sqrt in
// place of rsqrtf (the oracle's one documented deviation).
void hidden_rmsnorm(uint16_t *out, const uint16_t *in, const uint16_t *weight,
                    int width) {
  const int packs = width / 8;
  float warp_sums[kBlockThreads / kWarp];
  for (int warp = 0; warp < kBlockThreads / kWarp; ++warp) {
    float lanes[kWarp];
    for (int lane = 0; lane < kWarp; ++lane) {
      const int t = warp * kWarp + lane;
      float ss = 0.0f;
      for (int pack = t; pack < packs; pack += kBlockThreads) {
        for (int e = 0; e < 8; ++e) {
          const float v = bf(in[pack * 8 + e]);
          ss = std::fmaf(v, v, ss);
        }
      }
      lanes[lane] = ss;
    }
    warp_sums[warp] = shfl_xor_tree(lanes);
  }
  float lanes[kWarp];
  for (int lane = 0; lane < kWarp; ++lane) {
    lanes[lane] = lane < kBlockThreads / kWarp ? warp_sums[lane] : 0.0f;
  }
  const float sum_sq = shfl_xor_tree(lanes);
  const float scale = 1.0f / std::sqrt(sum_sq / float(width) + kEps);
  for (int i = 0; i < width; ++i) {
    const float scaled = bf(in[i]) * scale;
    out[i] = to_bf(scaled * bf(weight[i]));
  }
}

}  // namespace

extern "C" {

void orc_hidden_rmsnorm(uint16_t *out, const uint16_t *in,
                        const uint16_t *weight, int32_t width) {
  hidden_rmsnorm(out, in, weight, width);
}

void orc_project_cols(uint16_t *out, const uint16_t *x,
                      const uint16_t *w_col_major, int32_t width, int32_t cols,
                      int32_t active_threads, int32_t threads) {
  parallel_for(threads, cols, [&](int col) {
    out[col] = to_bf(
        block_dot(x, w_col_major + int64_t(col) * width, width, active_threads));
  });
}

void orc_decode_ingress(uint16_t *raw_qkv, uint16_t *normed, const uint16_t *x,
                        const uint16_t *input_norm_weight,
                        const uint16_t *qkv_proj_col_major, int32_t hidden,
                        int32_t cols, int32_t threads) {
  // decode.cu:447-496: CTA 0 norms the row, every CTA projects column tiles.
  std::vector<uint16_t> local(size_t(hidden), uint16_t(0));
  uint16_t *n = normed != nullptr ? normed : local.data();
  hidden_rmsnorm(n, x, input_norm_weight, hidden);
  orc_project_cols(raw_qkv, n, qkv_proj_col_major, hidden, cols, hidden / 8,
                   threads);
}

void orc_decode_egress(uint16_t *residual_out, uint16_t *normed_out,
                       uint16_t *ffn_residual, uint16_t *ffn_x,
                       const uint16_t *attention_out,
                       const uint16_t *o_proj_col_major,
                       const uint16_t *post_norm_weight,
                       const uint16_t *pre_ffn_norm_weight, const uint16_t *x,
                       int32_t attention_width, int32_t hidden,
                       int32_t threads) {
  // decode.cu:35-129: O projection, post-attention norm, residual add;
  // decode.cu:1049-1058: the pre-FFN norm of that sum (ffn_x, optional here).
  orc_project_cols(residual_out, attention_out, o_proj_col_major,
                   attention_width, hidden, kBlockThreads, threads);
  hidden_rmsnorm(normed_out, residual_out, post_norm_weight, hidden);
  for (int i = 0; i < hidden; ++i) {
    ffn_residual[i] = to_bf(bf(x[i]) + bf(normed_out[i]));  // cuda_utils.cuh:105-122
  }
  if (ffn_x != nullptr) {
    hidden_rmsnorm(ffn_x, ffn_residual, pre_ffn_norm_weight, hidden);
  }
}

int32_t orc_hardware_threads(void) {
  const unsigned n = std::thread::hardware_concurrency();
  return n == 0 ? 1 : int32_t(n);
}

}  // extern "C"

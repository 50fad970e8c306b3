// One decode layer through the library from a translation unit that sees gemma.c's OWN headers: the per-layer
// argument struct is the reference's Gemma4DecodeMegakernelLayerArgs (src/gemma4_megakernel.cuh:32-66), filled the
// way gemma4_decode_megakernel's layer loop fills it (src/gemma4_decode_megakernel.cu:120-183), and handed to
// gemma4_b200kv_decode_attention_layer. The runtime state that supplies caches, page tables, positions and RoPE
// tables is the reference's Gemma4RuntimeState, created and advanced by the library's gemma4_runtime_* functions
// -- so the struct layout the library writes is the one this translation unit reads.
//
// Built by oracle/build_ref.sh (needs the gemma.c sources on the include path) into oracle/_ref/ and run by
// tests/test_gpu_reference_boundary.py:   megakernel_layer <dir> <prompt_len> <steps>
// reads   <dir>/{x,w_in,w_qkv,w_o,w_post,w_pre,q_w,k_w}.bin  (bf16 bit patterns)
// writes  <dir>/{raw,q,attn,residual_out,normed_out,ffn_residual,ffn_x,cache_k,cache_v}.bin and meta.txt
#include "gemma4_megakernel.cuh"

#define GEMMA4_B200KV_USE_REFERENCE_HEADERS
#include "gemma4_b200kv.hpp"

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <string>
#include <vector>

namespace {

#define CHECK(expr)                                                                              \
  do {                                                                                           \
    const cudaError_t st__ = (expr);                                                             \
    if (st__ != cudaSuccess) {                                                                   \
      std::fprintf(stderr, "%s:%d: %s -> %s\n", __FILE__, __LINE__, #expr, cudaGetErrorString(st__)); \
      std::exit(1);                                                                              \
    }                                                                                            \
  } while (0)

std::vector<uint16_t> read_bits(const std::string &path, size_t count) {
  std::vector<uint16_t> v(count);
  FILE *f = std::fopen(path.c_str(), "rb");
  if (f == nullptr || std::fread(v.data(), 2, count, f) != count) {
    std::fprintf(stderr, "cannot read %zu values from %s\n", count, path.c_str());
    std::exit(2);
  }
  std::fclose(f);
  return v;
}

__nv_bfloat16 *upload(const std::vector<uint16_t> &v) {
  __nv_bfloat16 *d = nullptr;
  CHECK(cudaMalloc(&d, v.size() * 2));
  CHECK(cudaMemcpy(d, v.data(), v.size() * 2, cudaMemcpyHostToDevice));
  return d;
}

template <class T>
void dump(const std::string &path, const T *device, size_t count) {
  std::vector<T> h(count);
  CHECK(cudaMemcpy(h.data(), device, count * sizeof(T), cudaMemcpyDeviceToHost));
  FILE *f = std::fopen(path.c_str(), "wb");
  if (f == nullptr || std::fwrite(h.data(), sizeof(T), count, f) != count) std::exit(3);
  std::fclose(f);
}

}  // namespace

int main(int argc, char **argv) {
  if (argc < 4) return 64;
  const std::string dir = argv[1];
  const int prompt_len = std::atoi(argv[2]);
  const int steps = std::atoi(argv[3]);
  constexpr int kHidden = GEMMA4_HIDDEN_SIZE;
  constexpr int kQHeads = GEMMA4_NUM_QUERY_HEADS;
  constexpr int kHeads = GEMMA4_SLIDING_KV_HEADS;
  constexpr int kDim = GEMMA4_SLIDING_HEAD_DIM;
  constexpr int kQWidth = kQHeads * kDim, kKWidth = kHeads * kDim;
  constexpr int kCols = kQWidth + 2 * kKWidth;

  // The reference's own owner of caches and per-step metadata (layout of src/gemma4_runtime.cuh:12-42),
  // initialised and advanced by the library.
  Gemma4RuntimeState state = {};
  CHECK(gemma4_runtime_state_init(&state, 1, prompt_len + steps + 1, 16, nullptr));
  CHECK(gemma4_runtime_prepare_prefill(&state, prompt_len, nullptr));
  const Gemma4KvCacheConfig &cfg = state.sliding_cache_config;
  // cache layer 0 is the one this program uses
  const size_t cache_elems = size_t(cfg.num_pages) * cfg.page_size * cfg.num_heads * cfg.head_dim;
  // "prompt" rows: a fixed pattern, so the Python side can rebuild the cache the attention sees
  {
    std::vector<uint16_t> fill(cache_elems);
    for (size_t i = 0; i < cache_elems; ++i) {
      const int centered = int((i * 37 + 17) % 257) - 128;   // the generator of tests/test_kv_cache.cu:43-46
      const __nv_bfloat16 b = __float2bfloat16_rn(float(centered) / 64.0f);
      fill[i] = *reinterpret_cast<const uint16_t *>(&b);
    }
    CHECK(cudaMemcpy(state.sliding_cache_k, fill.data(), cache_elems * 2, cudaMemcpyHostToDevice));
    for (size_t i = 0; i < cache_elems; ++i) {
      const int centered = int((i * 29 + 11) % 257) - 128;
      const __nv_bfloat16 b = __float2bfloat16_rn(float(centered) / 64.0f);
      fill[i] = *reinterpret_cast<const uint16_t *>(&b);
    }
    CHECK(cudaMemcpy(state.sliding_cache_v, fill.data(), cache_elems * 2, cudaMemcpyHostToDevice));
  }

  __nv_bfloat16 *x = upload(read_bits(dir + "/x.bin", kHidden));
  __nv_bfloat16 *w_in = upload(read_bits(dir + "/w_in.bin", kHidden));
  __nv_bfloat16 *w_qkv = upload(read_bits(dir + "/w_qkv.bin", size_t(kCols) * kHidden));
  __nv_bfloat16 *w_o = upload(read_bits(dir + "/w_o.bin", size_t(kHidden) * kQWidth));
  __nv_bfloat16 *w_post = upload(read_bits(dir + "/w_post.bin", kHidden));
  __nv_bfloat16 *w_pre = upload(read_bits(dir + "/w_pre.bin", kHidden));
  __nv_bfloat16 *q_w = upload(read_bits(dir + "/q_w.bin", kDim));
  __nv_bfloat16 *k_w = upload(read_bits(dir + "/k_w.bin", kDim));

  int device = 0, sms = 0;
  CHECK(cudaGetDevice(&device));
  CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
  int32_t num_splits = 0;
  b200kv_plan_balanced(1, sms, &num_splits);
  __nv_bfloat16 *q, *attn, *raw, *outs[4];
  float *pm, *pl, *pacc;
  uint32_t *ticket;
  int32_t *status;
  CHECK(cudaMalloc(&q, kQWidth * 2));
  CHECK(cudaMalloc(&attn, kQWidth * 2));
  CHECK(cudaMalloc(&raw, 8704 * 2));
  for (auto &o : outs) CHECK(cudaMalloc(&o, kHidden * 2));
  CHECK(cudaMalloc(&pm, size_t(kQHeads) * num_splits * 4));
  CHECK(cudaMalloc(&pl, size_t(kQHeads) * num_splits * 4));
  CHECK(cudaMalloc(&pacc, size_t(kQHeads) * num_splits * kDim * 4));
  CHECK(cudaMalloc(&ticket, (1 + kHeads * B200KV_TICKETS_PER_HEAD) * 4));  // one row: O projection + the attention's tickets
  CHECK(cudaMemset(ticket, 0, (1 + kHeads * B200KV_TICKETS_PER_HEAD) * 4));
  CHECK(cudaMalloc(&status, 16));
  CHECK(cudaMemset(status, 0, 16));

  const int32_t model_layer = 0;  // a sliding layer (src/gemma4.h:105-108)
  for (int s = 0; s < steps; ++s) {
    CHECK(gemma4_runtime_prepare_decode_step(&state, nullptr));
    Gemma4DecodeMegakernelLayerArgs args;  // the assignments of src/gemma4_decode_megakernel.cu:126-170
    args.residual_out = outs[0];
    args.normed_out = outs[1];
    args.ffn_residual = outs[2];
    args.ffn_x = outs[3];
    args.attention_q = q;
    args.attention_out = attn;
    args.attention_partial_m = pm;
    args.attention_partial_l = pl;
    args.attention_partial_acc = pacc;
    args.attention_cache_k = state.sliding_cache_k;
    args.attention_cache_v = state.sliding_cache_v;
    args.attention_cache_config = state.sliding_cache_config;
    args.attention_page_table = state.sliding_page_table;
    args.attention_token_position = state.token_position;
    args.attention_seq_lengths = state.seq_lengths;
    args.attention_cache_layer = gemma4_kv_cache_layer_index(model_layer, false);
    args.attention_split_size = 0;  // the library's balanced partition
    args.attention_num_splits = num_splits;
    args.attention_softmax_scale = 1.0f / std::sqrt(float(kDim));
    args.attention_x = x;
    args.attention_input_norm_weight = w_in;
    args.attention_qkv_proj_col_major = w_qkv;
    args.attention_o_proj_col_major = w_o;
    args.attention_post_norm_weight = w_post;
    args.attention_pre_ffn_norm_weight = w_pre;
    args.attention_q_norm_weight = q_w;
    args.attention_k_norm_weight = k_w;
    args.attention_cos = state.sliding_cos;
    args.attention_sin = state.sliding_sin;
    CHECK(gemma4_b200kv_decode_attention_layer(args, raw, ticket, 1, nullptr, status));
    CHECK(cudaDeviceSynchronize());
  }
  int32_t h_status = -1;
  CHECK(cudaMemcpy(&h_status, status, 4, cudaMemcpyDeviceToHost));

  dump(dir + "/raw.bin", reinterpret_cast<uint16_t *>(raw), kCols);
  dump(dir + "/q.bin", reinterpret_cast<uint16_t *>(q), kQWidth);
  dump(dir + "/attn.bin", reinterpret_cast<uint16_t *>(attn), kQWidth);
  const char *names[4] = {"residual_out", "normed_out", "ffn_residual", "ffn_x"};
  for (int i = 0; i < 4; ++i) dump(dir + "/" + names[i] + ".bin", reinterpret_cast<uint16_t *>(outs[i]), kHidden);
  dump(dir + "/cache_k.bin", reinterpret_cast<uint16_t *>(state.sliding_cache_k), cache_elems);
  dump(dir + "/cache_v.bin", reinterpret_cast<uint16_t *>(state.sliding_cache_v), cache_elems);
  dump(dir + "/page_table.bin", state.sliding_page_table, state.h_sliding_page_table.size());
  dump(dir + "/cos.bin", state.sliding_cos, size_t(state.max_seq_len) * (kDim / 2));
  dump(dir + "/sin.bin", state.sliding_sin, size_t(state.max_seq_len) * (kDim / 2));
  FILE *meta = std::fopen((dir + "/meta.txt").c_str(), "w");
  std::fprintf(meta, "%d %d %d %d %d %d %d %d\n%d %d %d %d %zu\n", cfg.num_layers, cfg.num_pages, cfg.page_size,
               cfg.max_pages_per_seq, cfg.batch_size, cfg.num_heads, cfg.head_dim, cfg.window_size,
               state.h_seq_lengths[0], state.h_token_position[0], num_splits, h_status, sizeof(Gemma4RuntimeState));
  std::fclose(meta);
  gemma4_runtime_state_free(&state);
  std::puts("megakernel layer ok");
  return h_status == 0 ? 0 : 4;
}

// Compile-and-link check of include/gemma4_b200kv.hpp from a translation unit shaped like the reference's
// src/gemma4_decode_megakernel.cu. With -DB200KV_TEST_WITH_GEMMA_C (and gemma.c's src/ on the include path) the
// per-layer argument struct is the reference's own Gemma4DecodeMegakernelLayerArgs from its gemma4_megakernel.cuh
// and the library's header sits on top of the reference's headers; without it, a struct with the same member
// names (src/gemma4_megakernel.cuh:32-66, the attention half) stands in. Either is handed to the header's binding
// template. Run by tests/test_host_api.py; needs no GPU: the arguments are rejected on the host (null pointers /
// unknown geometry) before anything is launched. (tests/cpp/megakernel_layer.cu runs a real layer on the GPU.)
#include <cstdio>

#ifdef B200KV_TEST_WITH_GEMMA_C
#include "gemma4_megakernel.cuh"
#define GEMMA4_B200KV_USE_REFERENCE_HEADERS
#include "gemma4_b200kv.hpp"
using LayerArgs = Gemma4DecodeMegakernelLayerArgs;
// an object laid out by the reference's header, initialised and freed by the library
static_assert(sizeof(Gemma4RuntimeState) == 184 + 7 * sizeof(std::vector<int32_t>), "layout");
#else
#include "gemma4_b200kv.hpp"

struct LayerArgs {
  __nv_bfloat16 *residual_out = nullptr;
  __nv_bfloat16 *normed_out = nullptr;
  __nv_bfloat16 *ffn_x = nullptr;
  __nv_bfloat16 *ffn_residual = nullptr;
  __nv_bfloat16 *attention_q = nullptr;
  __nv_bfloat16 *attention_out = nullptr;
  float *attention_partial_m = nullptr;
  float *attention_partial_l = nullptr;
  float *attention_partial_acc = nullptr;
  __nv_bfloat16 *attention_cache_k = nullptr;
  __nv_bfloat16 *attention_cache_v = nullptr;
  Gemma4KvCacheConfig attention_cache_config = {};
  const int32_t *attention_page_table = nullptr;
  const int32_t *attention_token_position = nullptr;
  const int32_t *attention_seq_lengths = nullptr;
  int32_t attention_cache_layer = 0;
  int32_t attention_split_size = 0;
  int32_t attention_num_splits = 0;
  float attention_softmax_scale = 0.0f;
  const __nv_bfloat16 *attention_x = nullptr;
  const __nv_bfloat16 *attention_input_norm_weight = nullptr;
  const __nv_bfloat16 *attention_qkv_proj_col_major = nullptr;
  const __nv_bfloat16 *attention_o_proj_col_major = nullptr;
  const __nv_bfloat16 *attention_post_norm_weight = nullptr;
  const __nv_bfloat16 *attention_pre_ffn_norm_weight = nullptr;
  const __nv_bfloat16 *attention_q_norm_weight = nullptr;
  const __nv_bfloat16 *attention_k_norm_weight = nullptr;
  const float *attention_cos = nullptr;
  const float *attention_sin = nullptr;
};
#endif

int main() {
  LayerArgs args;
  // geometry the library is not built for: refused like the reference's dispatch
  args.attention_cache_config = gemma4_kv_cache_make_config(false, 64, 16, 64);
  args.attention_cache_config.head_dim = 128;
  const cudaError_t odd = gemma4_b200kv_decode_attention_layer(args, nullptr, nullptr, 1, nullptr);
  // the sliding geometry with null buffers: refused by the entry point's own checks
  args.attention_cache_config.head_dim = 256;
  args.attention_cache_config.num_heads = 8;
  const cudaError_t null_buffers = gemma4_b200kv_decode_attention_layer(args, nullptr, nullptr, 1, nullptr);
  // zero rows: nothing to do (with a scratch pointer that is never touched)
  __nv_bfloat16 *fake = reinterpret_cast<__nv_bfloat16 *>(uintptr_t(4096));
  const cudaError_t empty = gemma4_b200kv_decode_attention_layer(args, fake, nullptr, 0, nullptr);
  std::printf("%d %d %d\n", int(odd), int(null_buffers), int(empty));
  return (odd == cudaErrorInvalidValue && null_buffers == cudaErrorInvalidValue && empty == cudaSuccess) ? 0 : 1;
}

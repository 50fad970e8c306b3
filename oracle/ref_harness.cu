// Harness around the reference's OWN CUDA code for the KV hot path. TEST INFRASTRUCTURE ONLY.
//
// This translation unit #includes the reference's decode source where it lies (the build recipe puts
// the reference's src/ directory on the include path; nothing of it is copied into this repository)
// and adds stand-alone __global__ wrappers around its three hot phases with the CTA mapping the phases
// were written for ("x = batch row, y = KV head, z = split", src/gemma4_flash_attention_decode.cu:715-716):
//   phase_decode_q_paged_kv_norm_rope   (:305-375)  fused append
//   phase_decode_paged_grouped_split    (:692-878)  split-KV attention
//   phase_decode_paged_reduce           (:881-977)  combine
// The fused layer kernel in that file also references the FFN device function, whose own source needs a
// CUTLASS example that is not available; it is never launched here, so a stub satisfies the linker.
// The result, oracle/_ref/libgemma4_ref.so, is a second checker beside the host oracle and the source
// of the golden fixtures in tests/golden (recorded on a B200).
#include "gemma4_flash_attention_decode.cu"
#include "gemma4_flash_attention.cuh"

extern "C" __device__ void gemma4_ffn_decode_fused_bf16_device(
    __nv_bfloat16 *__restrict__, __nv_bfloat16 *__restrict__, const __nv_bfloat16 *__restrict__,
    const __nv_bfloat16 *__restrict__, const __nv_bfloat16 *__restrict__, const __nv_bfloat16 *__restrict__,
    const __nv_bfloat16 *__restrict__, Gemma4FfnDecodeScratch *__restrict__, const __nv_bfloat16 *__restrict__,
    float) {}

namespace {

namespace ref = gemma4_flash_attention;
using Sliding = ref::Gemma4AttentionTraits<false>;   // 8 KV heads x 256, rotary 256, own V projection
using Global = ref::Gemma4AttentionTraits<true>;     // 1 KV head x 512, rotary 128, V derived from raw K
constexpr int kThreads = ref::kDecodeMegaThreads;    // 512, the block size the phases run with in the product

template <class Traits>
__global__ __launch_bounds__(kThreads) void ref_append_kernel(
    __nv_bfloat16 *q_prepared, __nv_bfloat16 *cache_k, __nv_bfloat16 *cache_v, Gemma4KvCacheConfig cfg,
    const int32_t *page_table, const int32_t *token_position, int cache_layer, const __nv_bfloat16 *q,
    const __nv_bfloat16 *k, const __nv_bfloat16 *v, const __nv_bfloat16 *q_w, const __nv_bfloat16 *k_w,
    const float *cos, const float *sin) {
  ref::phase_decode_q_paged_kv_norm_rope<Traits>(q_prepared, cache_k, cache_v, cfg, page_table, token_position,
                                                 cache_layer, q, k, v, q_w, k_w, cos, sin, int(blockIdx.x),
                                                 int(blockIdx.y), int(threadIdx.x));
}

template <class Traits>
__global__ __launch_bounds__(kThreads) void ref_split_kernel(
    __nv_bfloat16 *out, float *pm, float *pl, float *pacc, const __nv_bfloat16 *q, const __nv_bfloat16 *cache_k,
    const __nv_bfloat16 *cache_v, const int32_t *page_table, const int32_t *seq_lengths, Gemma4KvCacheConfig cfg,
    int32_t layer, float scale, int32_t split_size, int32_t num_splits, int32_t batch_count) {
  ref::phase_decode_paged_grouped_split<Traits, kThreads>(out, pm, pl, pacc, q, cache_k, cache_v, page_table,
                                                          seq_lengths, cfg, layer, scale, split_size, num_splits,
                                                          int(blockIdx.x), int(blockIdx.y), int(blockIdx.z),
                                                          int(threadIdx.x), batch_count);
}

template <class Traits>
__global__ __launch_bounds__(kThreads) void ref_reduce_kernel(
    __nv_bfloat16 *out, const float *pm, const float *pl, const float *pacc, const int32_t *seq_lengths,
    Gemma4KvCacheConfig cfg, int32_t split_size, int32_t num_splits) {
  ref::phase_decode_paged_reduce<Traits, kThreads>(out, pm, pl, pacc, seq_lengths, cfg, split_size, num_splits,
                                                   int(blockIdx.x), int(blockIdx.y), int(threadIdx.x),
                                                   int(blockDim.x));
}

template <class Traits>
bool geometry_is(const Gemma4KvCacheConfig &cfg) {
  return cfg.num_heads == Traits::kKvHeads && cfg.head_dim == Traits::kHeadDim;
}

template <class Traits>
int run_append(__nv_bfloat16 *q_prepared, __nv_bfloat16 *cache_k, __nv_bfloat16 *cache_v,
               Gemma4KvCacheConfig cfg, const int32_t *page_table, const int32_t *token_position,
               int cache_layer, const __nv_bfloat16 *q, const __nv_bfloat16 *k, const __nv_bfloat16 *v,
               const __nv_bfloat16 *q_w, const __nv_bfloat16 *k_w, const float *cos, const float *sin,
               int batch_count, cudaStream_t stream) {
  ref_append_kernel<Traits><<<dim3(batch_count, Traits::kKvHeads), kThreads, 0, stream>>>(
      q_prepared, cache_k, cache_v, cfg, page_table, token_position, cache_layer, q, k, v, q_w, k_w, cos, sin);
  return cudaGetLastError();
}

template <class Traits>
int run_attention(__nv_bfloat16 *out, float *pm, float *pl, float *pacc, const __nv_bfloat16 *q,
                  const __nv_bfloat16 *cache_k, const __nv_bfloat16 *cache_v, const int32_t *page_table,
                  const int32_t *seq_lengths, Gemma4KvCacheConfig cfg, int32_t layer, float scale,
                  int32_t split_size, int32_t num_splits, int32_t batch_count, cudaStream_t stream) {
  if (num_splits > 65535) return cudaErrorInvalidValue;
  ref_split_kernel<Traits><<<dim3(batch_count, Traits::kKvHeads, num_splits), kThreads, 0, stream>>>(
      out, pm, pl, pacc, q, cache_k, cache_v, page_table, seq_lengths, cfg, layer, scale, split_size, num_splits,
      batch_count);
  cudaError_t st = cudaGetLastError();
  if (st != cudaSuccess || num_splits == 1) return st;
  ref_reduce_kernel<Traits><<<dim3(batch_count, GEMMA4_NUM_QUERY_HEADS), kThreads, 0, stream>>>(
      out, pm, pl, pacc, seq_lengths, cfg, split_size, num_splits);
  return cudaGetLastError();
}

}  // namespace

// Both entry points pick the reference's traits from the cache geometry: 8 KV heads x 256 (sliding) or
// 1 KV head x 512 (global; `v` is ignored there, the phase derives V from raw K).
extern "C" int ref_decode_append(__nv_bfloat16 *q_prepared, __nv_bfloat16 *cache_k, __nv_bfloat16 *cache_v,
                                 Gemma4KvCacheConfig cfg, const int32_t *page_table, const int32_t *token_position,
                                 int cache_layer, const __nv_bfloat16 *q, const __nv_bfloat16 *k,
                                 const __nv_bfloat16 *v, const __nv_bfloat16 *q_w, const __nv_bfloat16 *k_w,
                                 const float *cos, const float *sin, int batch_count, cudaStream_t stream) {
  if (geometry_is<Sliding>(cfg)) {
    return run_append<Sliding>(q_prepared, cache_k, cache_v, cfg, page_table, token_position, cache_layer, q, k, v,
                               q_w, k_w, cos, sin, batch_count, stream);
  }
  if (geometry_is<Global>(cfg)) {
    return run_append<Global>(q_prepared, cache_k, cache_v, cfg, page_table, token_position, cache_layer, q, k, v,
                              q_w, k_w, cos, sin, batch_count, stream);
  }
  return cudaErrorInvalidValue;
}

extern "C" int ref_decode_attention(__nv_bfloat16 *out, float *pm, float *pl, float *pacc, const __nv_bfloat16 *q,
                                    const __nv_bfloat16 *cache_k, const __nv_bfloat16 *cache_v,
                                    const int32_t *page_table, const int32_t *seq_lengths, Gemma4KvCacheConfig cfg,
                                    int32_t layer, float scale, int32_t split_size, int32_t num_splits,
                                    int32_t batch_count, cudaStream_t stream) {
  if (geometry_is<Sliding>(cfg)) {
    return run_attention<Sliding>(out, pm, pl, pacc, q, cache_k, cache_v, page_table, seq_lengths, cfg, layer, scale,
                                  split_size, num_splits, batch_count, stream);
  }
  if (geometry_is<Global>(cfg)) {
    return run_attention<Global>(out, pm, pl, pacc, q, cache_k, cache_v, page_table, seq_lengths, cfg, layer, scale,
                                 split_size, num_splits, batch_count, stream);
  }
  return cudaErrorInvalidValue;
}

// C names for the reference's two prompt-attention entry points
// (src/gemma4_flash_attention.cuh:9-45; defined in gemma4_flash_attention_prefill.cu, linked in as it is).
extern "C" int ref_prefill_sliding(__nv_bfloat16 *out, __nv_bfloat16 *q_prepared, __nv_bfloat16 *k_prepared,
                                   __nv_bfloat16 *v_prepared, const __nv_bfloat16 *q, const __nv_bfloat16 *k,
                                   const __nv_bfloat16 *v, const __nv_bfloat16 *q_w, const __nv_bfloat16 *k_w,
                                   const float *cos, const float *sin, const int32_t *token_position,
                                   int batch_size, int seqlen_q, int seqlen_k, int window_size, float scale,
                                   cudaStream_t stream) {
  return gemma4_flash_attention_sliding_fwd_bf16_norm_rope(out, q_prepared, k_prepared, v_prepared, q, k, v, q_w,
                                                           k_w, cos, sin, token_position, batch_size, seqlen_q,
                                                           seqlen_k, window_size, scale, stream);
}

extern "C" int ref_prefill_global(__nv_bfloat16 *out, __nv_bfloat16 *q_prepared, __nv_bfloat16 *k_prepared,
                                  __nv_bfloat16 *v_prepared, const __nv_bfloat16 *q, const __nv_bfloat16 *k,
                                  const __nv_bfloat16 *q_w, const __nv_bfloat16 *k_w, const float *cos,
                                  const float *sin, const int32_t *token_position, int batch_size, int seqlen_q,
                                  int seqlen_k, float scale, cudaStream_t stream) {
  return gemma4_flash_attention_global_fwd_bf16_norm_rope(out, q_prepared, k_prepared, v_prepared, q, k, q_w, k_w,
                                                          cos, sin, token_position, batch_size, seqlen_q, seqlen_k,
                                                          scale, stream);
}

// ---- the steps either side of the KV path inside the reference's fused layer kernel ----------------
//   phase_decode_rmsnorm_project_bf16      (:447-496)  input RMSNorm + [Q|K|V] projection
//   project_attention_out_post_attention   (:35-129)   O projection + post-attention norm + residual
// and the pre-FFN norm the fused kernel runs next (:1049-1058, a call of the reference's own
// gemma4_rmsnorm_hidden_row_512_bf16_device). Both phases hold grid-wide barriers, so the wrappers are
// launched cooperatively with the grid the reference's launcher would use (:1076-1111).
namespace {

template <int Width>
__global__ __launch_bounds__(kThreads, 1) void ref_ingress_kernel(Gemma4DecodeMegakernelLayerArgs args,
                                                                  __nv_bfloat16 *raw) {
  ref::phase_decode_rmsnorm_project_bf16<Width>(args, raw, ref::cg::this_grid());
}

template <class Traits>
__global__ __launch_bounds__(kThreads, 1) void ref_egress_kernel(Gemma4DecodeMegakernelLayerArgs args) {
  ref::project_attention_out_post_attention<Traits>(args, ref::cg::this_grid());
  if (blockIdx.x == 0 && args.ffn_x != nullptr) {
    __shared__ Bf16Packed128 cached_input[ref::kFfnHiddenPacks];
    __shared__ float warp_sums[ref::kDecodeMegaWarps];
    __shared__ float scale;
    gemma4_rmsnorm_hidden_row_512_bf16_device(args.ffn_x, args.ffn_residual, args.attention_pre_ffn_norm_weight,
                                              GEMMA4_RMS_NORM_EPS, cached_input, warp_sums, &scale,
                                              int(threadIdx.x));
  }
}

template <class Kernel, class... Args>
int launch_cooperative(Kernel kernel, cudaStream_t stream, Args... args) {
  int device = 0, sms = 0, per_sm = 0;
  cudaError_t st = cudaGetDevice(&device);
  if (st != cudaSuccess) return st;
  st = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  if (st != cudaSuccess) return st;
  st = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kThreads, 0);
  if (st != cudaSuccess) return st;
  if (per_sm <= 0) return cudaErrorInvalidValue;
  void *params[] = {(void *)&args...};
  st = cudaLaunchCooperativeKernel((void *)kernel, dim3(per_sm * sms), dim3(kThreads), params, 0, stream);
  return st != cudaSuccess ? st : cudaGetLastError();
}

}  // namespace

// global_geometry 0: 16 Q + 8 K + 8 V heads of 256 (8192 columns); 1: 16 Q + 1 K head of 512 (8704 columns).
extern "C" int ref_decode_ingress(__nv_bfloat16 *raw_qkv, __nv_bfloat16 *normed_out, const __nv_bfloat16 *x,
                                  const __nv_bfloat16 *input_norm_weight, const __nv_bfloat16 *qkv_proj_col_major,
                                  int global_geometry, cudaStream_t stream) {
  Gemma4DecodeMegakernelLayerArgs args;
  args.normed_out = normed_out;
  args.attention_x = x;
  args.attention_input_norm_weight = input_norm_weight;
  args.attention_qkv_proj_col_major = qkv_proj_col_major;
  if (global_geometry) {
    return launch_cooperative(ref_ingress_kernel<GEMMA4_GLOBAL_QK_PROJ_SIZE>, stream, args, raw_qkv);
  }
  return launch_cooperative(ref_ingress_kernel<GEMMA4_SLIDING_QKV_SIZE>, stream, args, raw_qkv);
}

extern "C" int ref_decode_egress(__nv_bfloat16 *residual_out, __nv_bfloat16 *normed_out,
                                 __nv_bfloat16 *ffn_residual, __nv_bfloat16 *ffn_x,
                                 const __nv_bfloat16 *attention_out, const __nv_bfloat16 *o_proj_col_major,
                                 const __nv_bfloat16 *post_norm_weight, const __nv_bfloat16 *pre_ffn_norm_weight,
                                 const __nv_bfloat16 *x, int global_geometry, cudaStream_t stream) {
  Gemma4DecodeMegakernelLayerArgs args;
  args.residual_out = residual_out;
  args.normed_out = normed_out;
  args.ffn_residual = ffn_residual;
  args.ffn_x = ffn_x;
  args.attention_out = const_cast<__nv_bfloat16 *>(attention_out);
  args.attention_o_proj_col_major = o_proj_col_major;
  args.attention_post_norm_weight = post_norm_weight;
  args.attention_pre_ffn_norm_weight = pre_ffn_norm_weight;
  args.attention_x = x;
  if (global_geometry) return launch_cooperative(ref_egress_kernel<Global>, stream, args);
  return launch_cooperative(ref_egress_kernel<Sliding>, stream, args);
}

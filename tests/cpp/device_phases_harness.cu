// Test harness for include/gemma4_b200kv_device.cuh: one cooperative kernel that runs a decode layer-step the way
// the reference's decode megakernel does (src/gemma4_flash_attention_decode.cu:1004-1031) -- the fused append for
// every (sequence, KV head), a grid-wide barrier, the split attention over (sequence, KV head, split) tasks dealt
// grid-strided to the CTAs, a grid-wide barrier, the reduce over the output rows -- calling nothing but the
// header's __device__ phases. Built into a small shared library of its own; the library under test is not linked.
#include <cooperative_groups.h>

#include "../../include/gemma4_b200kv_device.cuh"

namespace cg = cooperative_groups;

namespace {

struct LayerArgs {
  __nv_bfloat16 *q_prepared, *cache_k, *cache_v, *out;
  float *lse, *partial_m, *partial_l, *partial_acc;
  Gemma4KvCacheConfig cfg;
  const int32_t *page_table, *token_position, *seq_lengths;
  const __nv_bfloat16 *raw_q, *raw_k, *raw_v, *q_w, *k_w;
  const float *cos, *sin;
  int32_t cache_layer, split_size, num_splits, batch_count, q_heads;
  float softmax_scale;
};

constexpr int kThreads = 256;

__global__ void __launch_bounds__(kThreads) layer_kernel(LayerArgs a) {
  extern __shared__ float smem[];
  cg::grid_group grid = cg::this_grid();
  const int H = a.cfg.num_heads;
  const int tid = int(threadIdx.x);
  for (int task = int(blockIdx.x); task < a.batch_count * H; task += int(gridDim.x)) {
    b200kv_device::append_phase(a.q_prepared, a.cache_k, a.cache_v, a.cfg, a.page_table, a.token_position,
                                a.cache_layer, a.raw_q, a.raw_k, a.raw_v, a.q_w, a.k_w, a.cos, a.sin, a.q_heads,
                                task / H, task % H, tid, kThreads);
  }
  grid.sync();
  const int tasks = a.batch_count * H * a.num_splits;
  for (int task = int(blockIdx.x); task < tasks; task += int(gridDim.x)) {
    const int split = task % a.num_splits;
    const int head = (task / a.num_splits) % H;
    const int batch = task / (a.num_splits * H);
    b200kv_device::split_phase(a.partial_m, a.partial_l, a.partial_acc, a.out, a.lse, a.q_prepared, a.cache_k,
                               a.cache_v, a.cfg, a.page_table, a.seq_lengths, a.cache_layer, a.softmax_scale,
                               a.split_size, a.num_splits, a.q_heads, batch, head, split, smem, tid, kThreads);
  }
  grid.sync();
  for (int row = int(blockIdx.x); row < a.batch_count * a.q_heads; row += int(gridDim.x)) {
    b200kv_device::reduce_phase(a.out, a.lse, a.partial_m, a.partial_l, a.partial_acc, a.cfg, a.seq_lengths,
                                a.split_size, a.num_splits, a.q_heads, row / a.q_heads, row % a.q_heads, tid,
                                kThreads);
  }
}

}  // namespace

// Returns a cudaError_t value. Every pointer is a device pointer; the layouts are those of
// b200kv_decode_layer_step_bf16 (include/gemma4_b200kv.h).
extern "C" int device_phases_layer_step(void *q_prepared, void *cache_k, void *cache_v, void *out, float *lse,
                                        float *partial_m, float *partial_l, float *partial_acc,
                                        Gemma4KvCacheConfig cfg, const int32_t *page_table,
                                        const int32_t *token_position, const int32_t *seq_lengths,
                                        const void *raw_q, const void *raw_k, const void *raw_v, const void *q_w,
                                        const void *k_w, const float *cos, const float *sin, int32_t cache_layer,
                                        int32_t split_size, int32_t num_splits, int32_t batch_count,
                                        int32_t q_heads, float softmax_scale) {
  using bf = __nv_bfloat16;
  if (cfg.head_dim != b200kv_device::kDim || q_heads != b200kv_device::kGroup * cfg.num_heads ||
      split_size <= 0 || num_splits <= 0 || batch_count <= 0) {
    return int(cudaErrorInvalidValue);
  }
  LayerArgs a = {};
  a.q_prepared = static_cast<bf *>(q_prepared);
  a.cache_k = static_cast<bf *>(cache_k);
  a.cache_v = static_cast<bf *>(cache_v);
  a.out = static_cast<bf *>(out);
  a.lse = lse;
  a.partial_m = partial_m;
  a.partial_l = partial_l;
  a.partial_acc = partial_acc;
  a.cfg = cfg;
  a.page_table = page_table;
  a.token_position = token_position;
  a.seq_lengths = seq_lengths;
  a.raw_q = static_cast<const bf *>(raw_q);
  a.raw_k = static_cast<const bf *>(raw_k);
  a.raw_v = static_cast<const bf *>(raw_v);
  a.q_w = static_cast<const bf *>(q_w);
  a.k_w = static_cast<const bf *>(k_w);
  a.cos = cos;
  a.sin = sin;
  a.cache_layer = cache_layer;
  a.split_size = split_size;
  a.num_splits = num_splits;
  a.batch_count = batch_count;
  a.q_heads = q_heads;
  a.softmax_scale = softmax_scale;
  const size_t smem = size_t(kThreads / 32) * b200kv_device::kSplitSmemFloatsPerWarp * sizeof(float);
  int device = 0, sms = 0, per_sm = 0, cooperative = 0;
  cudaError_t st = cudaGetDevice(&device);
  if (st != cudaSuccess) return int(st);
  cudaDeviceGetAttribute(&cooperative, cudaDevAttrCooperativeLaunch, device);
  if (!cooperative) return int(cudaErrorNotSupported);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  st = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, layer_kernel, kThreads, smem);
  if (st != cudaSuccess || per_sm < 1) return int(st != cudaSuccess ? st : cudaErrorLaunchOutOfResources);
  void *params[] = {&a};
  st = cudaLaunchCooperativeKernel(reinterpret_cast<void *>(layer_kernel), dim3(unsigned(per_sm * sms)),
                                   dim3(kThreads), params, smem, nullptr);
  if (st != cudaSuccess) return int(st);
  return int(cudaDeviceSynchronize());
}

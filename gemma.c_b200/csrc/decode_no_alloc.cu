// Split-KV decode attention for callers that have no way to provide scratch.
//
// The regular entry point (b200kv_decode_attention_bf16) follows the
// reference's ownership rule: the caller brings the three partial buffers.
// Some callers cannot. A serving engine that handed all free device memory to
// its KV page pool at start-up has nothing left for cudaMalloc to give; a
// plug-in that only ever receives tensors from its host framework owns no
// allocator of its own; and code on a latency path does not want the
// device-wide synchronisation that cudaMalloc/cudaFree imply. For them this
// file keeps the split partials in a fixed array that is part of the loaded
// library image, so the call itself allocates nothing, ever.
//
// Cost and limits, so nobody is surprised:
//   * every GPU on which the library is loaded holds the array
//     (B200KV_STATIC_SCRATCH_BYTES, 16 MiB) until the process exits;
//   * a call whose partials do not fit is refused (cudaErrorInvalidValue and
//     one line on stderr saying how much was asked for), never truncated;
//   * all calls on a device share the one array: two calls whose kernels can
//     overlap on the GPU (different streams, or different host threads on
//     different streams) race on it. Keep them on one stream or use the
//     regular entry point with separate buffers;
//   * the array keeps whatever the previous call left there. Nothing has to be
//     cleared: a split writes its slot before the combine reads it, and slots
//     of splits that are not live are never read.
#include "common.cuh"
#include "kernels.cuh"

#include <cstdio>
#include <mutex>

namespace {

constexpr size_t kScratchBytes = B200KV_STATIC_SCRATCH_BYTES;
constexpr size_t kScratchFloats = kScratchBytes / sizeof(float);
constexpr size_t kRowAlign = 64;  // floats; keeps the acc block 256-byte aligned
constexpr int kMaxDevices = 64;

// In host code this name is only a handle for the runtime, not an address a
// kernel can use; the device address is looked up per device below.
static __device__ __align__(256) float g_static_scratch[kScratchFloats];

std::mutex g_lookup_mutex;
float *g_device_address[kMaxDevices] = {};

// Device address of the array on the current device. The first call on a
// device asks the runtime for it (which may load the module); later calls
// read the cached pointer. The pointer belongs to the device's primary
// context and is not refreshed: it does not survive cudaDeviceReset.
cudaError_t static_scratch_address(float **out) {
  int device = -1;
  cudaError_t st = cudaGetDevice(&device);
  if (st != cudaSuccess) return st;
  if (device < 0 || device >= kMaxDevices) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lock(g_lookup_mutex);
  if (g_device_address[device] == nullptr) {
    void *address = nullptr;
    st = cudaGetSymbolAddress(&address, g_static_scratch);
    if (st != cudaSuccess) return st;
    if (address == nullptr) return cudaErrorInvalidSymbol;
    g_device_address[device] = static_cast<float *>(address);
  }
  *out = g_device_address[device];
  return cudaSuccess;
}

size_t round_up(size_t n, size_t to) { return (n + to - 1) / to * to; }

}  // namespace

extern "C" int b200kv_decode_attention_static_scratch_bf16(
    b200kv_bf16 *d_out, float *d_lse, const b200kv_bf16 *d_q_prepared,
    const b200kv_bf16 *d_cache_k, const b200kv_bf16 *d_cache_v,
    Gemma4KvCacheConfig cache_config, const int32_t *d_page_table,
    const int32_t *d_seq_lengths, int32_t cache_layer, float softmax_scale,
    int32_t split_size, int32_t num_splits, int32_t batch_count,
    int32_t q_heads, int32_t *d_status, b200kv_stream stream) {
  using bf = __nv_bfloat16;
  if (batch_count <= 0 || q_heads <= 0 || num_splits <= 0 ||
      cache_config.head_dim <= 0) {
    return cudaErrorInvalidValue;
  }
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
  a.status = d_status;

  if (num_splits > 1) {
    const size_t rows = size_t(batch_count) * size_t(q_heads) * size_t(num_splits);
    const size_t ml = round_up(rows, kRowAlign);
    const size_t need = 2 * ml + rows * size_t(cache_config.head_dim);
    if (need > kScratchFloats) {
      std::fprintf(stderr,
                   "b200kv_decode_attention_static_scratch_bf16: partials need "
                   "%zu bytes, the built-in scratch holds %zu; use fewer splits "
                   "or b200kv_decode_attention_bf16 with your own buffers\n",
                   need * sizeof(float), kScratchBytes);
      return cudaErrorInvalidValue;
    }
    float *base = nullptr;
    const cudaError_t st = static_scratch_address(&base);
    if (st != cudaSuccess) return st;
    a.partial_m = base;
    a.partial_l = base + ml;
    a.partial_acc = base + 2 * ml;
  }
  return b200kv::decode_attention_bf16(a, static_cast<cudaStream_t>(stream));
}

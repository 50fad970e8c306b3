// All-gather of the per-rank attention rows over NVLink peer memory, for the
// KV-head-sharded mode (one process per GPU, each rank attends its own KV
// heads, every rank needs all heads' rows for the O projection). The payload
// is a few KiB, so the cost of a library collective is its launch and protocol
// latency; here one small kernel per rank does the whole exchange:
//
//   1. stores this rank's rows into slot `rank` of every peer's gathered
//      buffer (plain peer stores through the NVLink mapping; no multicast),
//   2. fence.sys, then writes the call's epoch into flag `rank` on every peer,
//   3. waits (bounded) until its own flags show the epoch from every rank.
//
// When the kernel ends, the gathered buffer on this GPU holds every rank's
// rows and later work on the stream may read it. Buffers are double-buffered
// by epoch parity: a rank can be at most one call ahead of a peer (it needs the
// peer's flag of call e + 1 to get past call e + 1), so half (e & 1) is never
// overwritten while a peer still reads call e.
//
// The same kernel can finish a key-range-sharded attention (every rank holds
// all heads but only a range of the keys): each rank contributes its
// normalised rows and their log-sum-exp, and after the wait every rank merges
// them, out = sum_r exp(lse_r - LSE) out_r with LSE = log sum_r exp(lse_r) --
// the combine of src/gemma4_flash_attention_decode.cu:881-977 one level up.
//
// No counterpart in the reference (single GPU). Every wait is bounded; a rank
// whose peers do not show up within about a second records
// B200KV_STATUS_WAIT_TIMEOUT and returns.
#include <cstring>
#include <new>
#include <vector>

#include "common.cuh"
#include "kernels.cuh"

namespace b200kv {
namespace {

constexpr int kMaxPeers = 8;
constexpr int kGatherThreads = 256;
constexpr int kMaxMergeRows = 64;

struct PeerGatherParams {
  const uint4 *src;
  int64_t packs;               // 16-byte packs this rank contributes
  int64_t slot_packs;          // capacity of one slot, in packs
  uint4 *data[kMaxPeers];      // peer r's gathered buffer [2][world][slot_packs]
  uint32_t *flags[kMaxPeers];  // peer r's flags [2][world]
  uint32_t *epoch;             // this rank's call counter (device)
  int32_t rank;
  int32_t world;
  int32_t *status;
  long long wait_clocks;       // how long a thread waits for its peer's flag
  // optional second segment of 4-byte words, stored behind the packs
  const uint32_t *src_words;
  int32_t words;
  // optional merge (merge_rows > 0): the packs are [merge_rows][merge_dim] bf16
  // rows, the words their fp32 log-sum-exp
  int32_t merge_rows;
  int32_t merge_dim;
  __nv_bfloat16 *merged_out;
  float *merged_lse;
};

__device__ __forceinline__ void store_release_sys(uint32_t *addr, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}

__device__ __forceinline__ uint32_t load_acquire_sys(const uint32_t *addr) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}

__global__ void __launch_bounds__(kGatherThreads) peer_allgather_kernel(
    const PeerGatherParams p) {
  __shared__ uint32_t s_epoch;
  pdl_wait_for_predecessor();  // the rows come from the preceding kernel
  pdl_release_successor();
  if (threadIdx.x == 0) s_epoch = *p.epoch + 1u;
  __syncthreads();
  const uint32_t e = s_epoch;
  const int64_t half = int64_t(e & 1u) * p.world;
  // 1. this rank's rows into its slot on every rank (its own included)
  for (int r = 0; r < p.world; ++r) {
    uint4 *dst = p.data[r] + (half + p.rank) * p.slot_packs;
    for (int64_t i = threadIdx.x; i < p.packs; i += kGatherThreads) {
      dst[i] = p.src[i];
    }
    uint32_t *dst_words = reinterpret_cast<uint32_t *>(dst + p.packs);
    for (int i = threadIdx.x; i < p.words; i += kGatherThreads) {
      dst_words[i] = p.src_words[i];
    }
  }
  __threadfence_system();
  __syncthreads();
  // 2. + 3. one thread per peer: announce, then wait for that peer
  if (threadIdx.x < p.world) {
    const int r = int(threadIdx.x);
    store_release_sys(p.flags[r] + half + p.rank, e);
    const uint32_t *mine = p.flags[p.rank] + half + r;
    const long long start = clock64();
    while (int32_t(load_acquire_sys(mine) - e) < 0) {
      if (clock64() - start > p.wait_clocks) {
        set_status(p.status, B200KV_STATUS_WAIT_TIMEOUT);
        break;
      }
      __nanosleep(100);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) *p.epoch = e;
  if (p.merge_rows <= 0) return;

  // Merge of the ranks' partial attention rows. The slots were written by
  // other GPUs: read them past L1 (a line of the same half may be cached from
  // two calls ago).
  __shared__ float s_weight[kMaxMergeRows][kMaxPeers];
  const uint4 *mine = p.data[p.rank] + half * p.slot_packs;
  for (int row = threadIdx.x; row < p.merge_rows; row += kGatherThreads) {
    float lse[kMaxPeers];
    float top = -INFINITY;
    for (int r = 0; r < p.world; ++r) {
      const float *words =
          reinterpret_cast<const float *>(mine + r * p.slot_packs + p.packs);
      lse[r] = __ldcg(words + row);
      top = fmaxf(top, lse[r]);
    }
    float sum = 0.0f;
    for (int r = 0; r < p.world; ++r) {
      lse[r] = (top == -INFINITY) ? 0.0f : expf(lse[r] - top);
      sum += lse[r];
    }
    for (int r = 0; r < p.world; ++r) {
      s_weight[row][r] = sum > 0.0f ? lse[r] / sum : 0.0f;
    }
    if (p.merged_lse != nullptr) {
      p.merged_lse[row] = sum > 0.0f ? top + logf(sum) : -INFINITY;
    }
  }
  __syncthreads();
  const int pairs = p.merge_rows * p.merge_dim / 2;
  for (int i = threadIdx.x; i < pairs; i += kGatherThreads) {
    const int row = (2 * i) / p.merge_dim;
    float lo = 0.0f, hi = 0.0f;
    for (int r = 0; r < p.world; ++r) {
      const uint32_t *rows =
          reinterpret_cast<const uint32_t *>(mine + r * p.slot_packs);
      const uint32_t v = __ldcg(rows + i);
      const float w = s_weight[row][r];
      if (w != 0.0f) {  // a rank without keys may hold anything
        lo = fmaf(w, bf16_lo(v), lo);
        hi = fmaf(w, bf16_hi(v), hi);
      }
    }
    const __nv_bfloat162 packed = __floats2bfloat162_rn(lo, hi);
    reinterpret_cast<__nv_bfloat162 *>(p.merged_out)[i] = packed;
  }
}

struct PeerBuffer {
  int world = 0;
  int rank = 0;
  int64_t slot_bytes = 0;
  unsigned char *base = nullptr;          // own allocation
  unsigned char *peer[kMaxPeers] = {};    // mapped bases (peer[rank] == base)
  bool connected = false;
  bool loopback = false;                  // peers are local allocations (one-GPU stand-in)
  uint32_t calls = 0;                     // host mirror of the device epoch
  long long wait_clocks = kWaitClockLimit;
};

int64_t data_bytes(const PeerBuffer &b) { return 2 * int64_t(b.world) * b.slot_bytes; }
int64_t flag_offset(const PeerBuffer &b) { return (data_bytes(b) + 255) / 256 * 256; }
int64_t total_bytes(const PeerBuffer &b) { return flag_offset(b) + 256; }

}  // namespace

cudaError_t peer_buffer_create(int64_t slot_bytes, int world, int rank,
                               void **handle, void *export_64_bytes) {
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "export size");
  if (handle == nullptr || export_64_bytes == nullptr || world < 1 ||
      world > kMaxPeers || rank < 0 || rank >= world || slot_bytes <= 0 ||
      slot_bytes % 16 != 0) {
    return cudaErrorInvalidValue;
  }
  PeerBuffer *b = new (std::nothrow) PeerBuffer;
  if (b == nullptr) return cudaErrorMemoryAllocation;
  b->world = world;
  b->rank = rank;
  b->slot_bytes = slot_bytes;
  cudaError_t st = cudaMalloc(&b->base, size_t(total_bytes(*b)));
  if (st == cudaSuccess) st = cudaMemset(b->base, 0, size_t(total_bytes(*b)));
  if (st == cudaSuccess) st = cudaDeviceSynchronize();
  cudaIpcMemHandle_t h;
  if (st == cudaSuccess) st = cudaIpcGetMemHandle(&h, b->base);
  if (st != cudaSuccess) {
    if (b->base != nullptr) cudaFree(b->base);
    delete b;
    return st;
  }
  std::memcpy(export_64_bytes, &h, sizeof(h));
  b->peer[rank] = b->base;
  if (world == 1) b->connected = true;
  *handle = b;
  return cudaSuccess;
}

cudaError_t peer_buffer_connect(void *handle, const void *exports) {
  PeerBuffer *b = static_cast<PeerBuffer *>(handle);
  if (b == nullptr || exports == nullptr) return cudaErrorInvalidValue;
  for (int r = 0; r < b->world; ++r) {
    if (r == b->rank || b->peer[r] != nullptr) continue;
    cudaIpcMemHandle_t h;
    std::memcpy(&h, static_cast<const unsigned char *>(exports) + 64 * r, sizeof(h));
    void *mapped = nullptr;
    const cudaError_t st =
        cudaIpcOpenMemHandle(&mapped, h, cudaIpcMemLazyEnablePeerAccess);
    if (st != cudaSuccess) return st;
    b->peer[r] = static_cast<unsigned char *>(mapped);
  }
  b->connected = true;
  return cudaSuccess;
}

namespace {

cudaError_t launch_gather(PeerBuffer *b, PeerGatherParams p, const void *src,
                          int64_t bytes, int32_t *status, cudaStream_t stream,
                          void **gathered) {
  p.src = static_cast<const uint4 *>(src);
  p.packs = bytes / 16;
  p.slot_packs = b->slot_bytes / 16;
  for (int r = 0; r < b->world; ++r) {
    p.data[r] = reinterpret_cast<uint4 *>(b->peer[r]);
    p.flags[r] = reinterpret_cast<uint32_t *>(b->peer[r] + flag_offset(*b));
  }
  p.epoch = reinterpret_cast<uint32_t *>(b->base + flag_offset(*b)) + 2 * kMaxPeers;
  p.rank = b->rank;
  p.world = b->world;
  p.status = status;
  p.wait_clocks = b->wait_clocks;
  const cudaError_t st = launch_pdl(peer_allgather_kernel, dim3(1),
                                    dim3(kGatherThreads), 0, stream, p);
  if (st != cudaSuccess) return st;
  b->calls += 1;
  if (gathered != nullptr) {
    *gathered = b->base + int64_t(b->calls & 1u) * b->world * b->slot_bytes;
  }
  return cudaSuccess;
}

}  // namespace

cudaError_t peer_allgather(void *handle, const void *src, int64_t bytes,
                           int32_t *status, cudaStream_t stream,
                           void **gathered) {
  PeerBuffer *b = static_cast<PeerBuffer *>(handle);
  if (b == nullptr || !b->connected || src == nullptr || bytes <= 0 ||
      bytes % 16 != 0 || bytes > b->slot_bytes ||
      (reinterpret_cast<uintptr_t>(src) & 15u) != 0) {
    return cudaErrorInvalidValue;
  }
  return launch_gather(b, PeerGatherParams{}, src, bytes, status, stream, gathered);
}

cudaError_t peer_merge_attention(void *handle, __nv_bfloat16 *merged_out,
                                 float *merged_lse, const __nv_bfloat16 *out,
                                 const float *lse, int32_t rows, int32_t head_dim,
                                 int32_t *status, cudaStream_t stream) {
  PeerBuffer *b = static_cast<PeerBuffer *>(handle);
  const int64_t bytes = int64_t(rows) * head_dim * 2;
  if (b == nullptr || !b->connected || merged_out == nullptr || out == nullptr ||
      lse == nullptr || rows <= 0 || rows > kMaxMergeRows || head_dim <= 0 ||
      bytes % 16 != 0 || bytes + int64_t(rows) * 4 > b->slot_bytes ||
      (reinterpret_cast<uintptr_t>(out) & 15u) != 0 ||
      (reinterpret_cast<uintptr_t>(merged_out) & 3u) != 0) {
    return cudaErrorInvalidValue;
  }
  PeerGatherParams p = {};
  p.src_words = reinterpret_cast<const uint32_t *>(lse);
  p.words = rows;
  p.merge_rows = rows;
  p.merge_dim = head_dim;
  p.merged_out = merged_out;
  p.merged_lse = merged_lse;
  return launch_gather(b, p, out, bytes, status, stream, nullptr);
}

cudaError_t peer_buffer_create_loopback(int64_t slot_bytes, int world, int rank,
                                        void **handle) {
  unsigned char unused[64];
  const cudaError_t st = peer_buffer_create(slot_bytes, world, rank, handle, unused);
  if (st != cudaSuccess) return st;
  PeerBuffer *b = static_cast<PeerBuffer *>(*handle);
  b->loopback = true;
  for (int r = 0; r < world; ++r) {
    if (r == rank) continue;
    cudaError_t e = cudaMalloc(&b->peer[r], size_t(total_bytes(*b)));
    if (e == cudaSuccess) e = cudaMemset(b->peer[r], 0, size_t(total_bytes(*b)));
    if (e != cudaSuccess) {
      peer_buffer_destroy(b);
      *handle = nullptr;
      return e;
    }
  }
  b->connected = true;
  return cudaDeviceSynchronize();
}

cudaError_t peer_epilogue_begin(void *handle, int64_t bytes, PeerEpilogue *out) {
  PeerBuffer *b = static_cast<PeerBuffer *>(handle);
  if (b == nullptr || out == nullptr || !b->connected || bytes <= 0 || bytes % 16 != 0 ||
      bytes > b->slot_bytes) {
    return cudaErrorInvalidValue;
  }
  *out = PeerEpilogue{};
  for (int r = 0; r < b->world; ++r) {
    out->data[r] = reinterpret_cast<uint4 *>(b->peer[r]);
    out->flags[r] = reinterpret_cast<uint32_t *>(b->peer[r] + flag_offset(*b));
  }
  uint32_t *own = reinterpret_cast<uint32_t *>(b->base + flag_offset(*b));
  out->epoch = own + 2 * kMaxPeers;
  out->done = own + 2 * kMaxPeers + 1;
  out->slot_packs = b->slot_bytes / 16;
  out->wait_clocks = b->wait_clocks;
  out->rank = b->rank;
  out->world = b->world;
  b->calls += 1;
  return cudaSuccess;
}

cudaError_t peer_buffer_gathered(void *handle, void **gathered) {
  PeerBuffer *b = static_cast<PeerBuffer *>(handle);
  if (b == nullptr || gathered == nullptr) return cudaErrorInvalidValue;
  *gathered = b->base + int64_t(b->calls & 1u) * b->world * b->slot_bytes;
  return cudaSuccess;
}

cudaError_t peer_buffer_set_wait_clocks(void *handle, long long clocks) {
  PeerBuffer *b = static_cast<PeerBuffer *>(handle);
  if (b == nullptr || clocks <= 0) return cudaErrorInvalidValue;
  b->wait_clocks = clocks;
  return cudaSuccess;
}

cudaError_t peer_buffer_post(void *handle, int from_rank, uint32_t epoch,
                             cudaStream_t stream) {
  PeerBuffer *b = static_cast<PeerBuffer *>(handle);
  if (b == nullptr || from_rank < 0 || from_rank >= b->world) {
    return cudaErrorInvalidValue;
  }
  uint32_t *flags = reinterpret_cast<uint32_t *>(b->base + flag_offset(*b));
  for (int half = 0; half < 2; ++half) {
    const cudaError_t st =
        cudaMemcpyAsync(flags + half * b->world + from_rank, &epoch, sizeof(epoch),
                        cudaMemcpyHostToDevice, stream);
    if (st != cudaSuccess) return st;
  }
  return cudaStreamSynchronize(stream);  // `epoch` is a stack variable
}

cudaError_t peer_buffer_reset(void *handle) {
  PeerBuffer *b = static_cast<PeerBuffer *>(handle);
  if (b == nullptr) return cudaErrorInvalidValue;
  cudaError_t st = cudaDeviceSynchronize();
  if (st == cudaSuccess) {
    st = cudaMemset(b->base + flag_offset(*b), 0, 256);  // flags and the epoch
  }
  if (st == cudaSuccess) st = cudaDeviceSynchronize();
  if (st == cudaSuccess) b->calls = 0;
  return st;
}

cudaError_t peer_buffer_destroy(void *handle) {
  PeerBuffer *b = static_cast<PeerBuffer *>(handle);
  if (b == nullptr) return cudaSuccess;
  cudaError_t first = cudaSuccess;
  for (int r = 0; r < b->world; ++r) {
    if (r != b->rank && b->peer[r] != nullptr) {
      const cudaError_t st = b->loopback ? cudaFree(b->peer[r])
                                         : cudaIpcCloseMemHandle(b->peer[r]);
      if (first == cudaSuccess) first = st;
    }
  }
  const cudaError_t st = cudaFree(b->base);
  if (first == cudaSuccess) first = st;
  delete b;
  return first;
}

}  // namespace b200kv

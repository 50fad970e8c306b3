// Shared device/host helpers for the B200 KV-cache kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <utility>

#include "../../include/gemma4_b200kv.hpp"

namespace b200kv {

constexpr int kWarpSize = 32;

template <typename T, typename U>
__host__ __device__ constexpr auto div_up(T n, U d) {
  return (n + d - 1) / d;
}

// Flat Layout-A offset [layer, page, page_offset, head, dim]
// (gemma4_kv_cache_offset, src/gemma4_kv_cache.cuh:28-38).
__host__ __device__ inline int64_t cache_offset(const Gemma4KvCacheConfig &c,
                                                int32_t layer, int32_t page,
                                                int32_t page_offset,
                                                int32_t head, int32_t dim) {
  const int64_t layer_page = int64_t(layer) * c.num_pages + page;
  const int64_t token = layer_page * c.page_size + page_offset;
  return (token * c.num_heads + head) * c.head_dim + dim;
}

// ---------------------------------------------------------------------------
// mbarrier + bulk-async-copy wrappers (PTX, shared::cta addresses as u32).
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar),
               "r"(count));
}

__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar)
               : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar,
                                                      uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(
                   bar),
               "r"(bytes)
               : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(done)
      : "r"(bar), "r"(parity)
      : "memory");
  return done != 0;
}

// Bounded wait: gives up after about a second of SM clocks and returns false;
// the caller records a status code and unwinds. Nothing in this library spins
// without a limit.
constexpr long long kWaitClockLimit = 1ll << 31;

__device__ __forceinline__ bool mbar_wait_bounded(
    uint32_t bar, uint32_t parity, long long clock_limit = kWaitClockLimit) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long start = clock64();
  for (uint32_t poll = 0;; ++poll) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((poll & 63u) == 63u) {
      if (clock64() - start > clock_limit) return false;
      __nanosleep(64);
    }
  }
}

// One-dimensional bulk copy global -> this CTA's shared memory, completion
// counted in bytes on an mbarrier. Addresses and size are multiples of 16.
__device__ __forceinline__ void bulk_load(uint32_t dst_smem, const void *src,
                                          uint32_t bytes, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1], %2, [%3];" ::"r"(dst_smem),
      "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}

__device__ __forceinline__ void bulk_load_hint(uint32_t dst_smem,
                                               const void *src, uint32_t bytes,
                                               uint32_t bar, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes"
      ".L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(dst_smem),
      "l"(src), "r"(bytes), "r"(bar), "l"(policy)
      : "memory");
}

__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t policy;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;"
               : "=l"(policy));
  return policy;
}

__device__ __forceinline__ void named_barrier_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// Orders this thread's generic-proxy writes to shared memory before later
// async-proxy (bulk copy) accesses to the same locations.
__device__ __forceinline__ void fence_proxy_async_shared() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ float lg2_approx(float x) {
  float y;
  asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "r"(addr));
  return v;
}

// bf16 pair -> two fp32 (exact: bf16 is the upper half of an fp32).
__device__ __forceinline__ float bf16_lo(uint32_t w) {
  return __uint_as_float(w << 16);
}
__device__ __forceinline__ float bf16_hi(uint32_t w) {
  return __uint_as_float(w & 0xffff0000u);
}

// Programmatic dependent launch: a kernel launched with launch_pdl() may start
// while its predecessor in the stream is still draining; it must not touch
// anything the predecessor writes before pdl_wait_for_predecessor() returns
// (which is when the predecessor has completed and its writes are visible).
__device__ __forceinline__ void pdl_wait_for_predecessor() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}
__device__ __forceinline__ void pdl_release_successor() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

__device__ __forceinline__ void set_status(int32_t *status, int32_t code) {
  if (status != nullptr) atomicCAS(status, 0, code);
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block,
                              size_t smem_bytes, cudaStream_t stream,
                              Args &&...args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem_bytes;
  config.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attr;
  config.numAttrs = 1;
  return cudaLaunchKernelEx(&config, kernel, std::forward<Args>(args)...);
}

}  // namespace b200kv

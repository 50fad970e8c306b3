// Per-head prep (RMSNorm + RoPE) fused into the paged KV append, the
// whole-prompt prep, and the plain cache write of prepared rows.
//
// Replaces, with the same arithmetic order so that results are bit-identical:
//   prep_weighted_rope_head_values / prep_scale_free_head_values /
//   phase_decode_q_paged_kv_norm_rope   src/gemma4_flash_attention_decode.cu:216-375
//   gemma4_rmsnorm_warp_scale_f32_device src/gemma4_rmsnorm.cu:90-101
//   store_rotated_pair_bf16              src/gemma4_rope.cu:8-20
//   phase_qkv_norm_rope                  src/gemma4_flash_attention_prefill.cu:1022-1081
//   kv_cache_write_vec_kernel            src/gemma4_kv_cache.cu:11-71
//
// One warp owns one head; lane l holds elements l + 32*i (the reference's
// ownership), the sum of squares is an fma chain per lane followed by the xor
// butterfly 16,8,4,2,1 -- that order defines the bit pattern of the scale.
#include "kernels.cuh"
#include "prep_common.cuh"

#include <type_traits>

namespace b200kv {

namespace {

// grid (batch, kv_head); warps 0..G-1 prep the G query heads of the group,
// warp G preps and stores K, warp G+1 (only when V has its own projection)
// preps and stores V.
template <int D, int ROT, bool kIeee>
__global__ void decode_append_kernel(AppendArgs a) {
  const int batch = int(blockIdx.x);
  const int kv_head = int(blockIdx.y);
  const int warp = int(threadIdx.x) >> 5;
  const int lane = int(threadIdx.x) & 31;
  const Gemma4KvCacheConfig &c = a.cfg;
  const int G = a.q_heads / c.num_heads;
  const bool has_v = a.v != nullptr;

  // The launch before this one may still be reading the q buffer or the
  // cache this kernel is about to overwrite.
  pdl_wait_for_predecessor();
  pdl_release_successor();

  // The row this warp preps does not depend on the position: fetch it first
  // so its latency overlaps the position and page-table lookups.
  const int64_t src = (int64_t(batch) * c.num_heads + kv_head) * D;
  const __nv_bfloat16 *row_in =
      warp < G ? a.q + (int64_t(batch) * a.q_heads + kv_head * G + warp) * D
               : (warp == G || !has_v ? a.k + src : a.v + src);
  float x[D / 32];
  load_head<D>(row_in, lane, x);

  const int position = __ldg(a.token_position + batch);
  if (position < 0) return;
  const float *cos_row = a.cos + int64_t(position) * (ROT / 2);
  const float *sin_row = a.sin + int64_t(position) * (ROT / 2);

  if (warp < G) {
    const int64_t off = (int64_t(batch) * a.q_heads + kv_head * G + warp) * D;
    prep_weighted_rope<D, ROT, kIeee>(a.q_prepared + off, x, a.q_norm_weight,
                                      cos_row, sin_row, lane);
    return;
  }

  // Row address, src/gemma4_flash_attention_decode.cu:285-303: the slot is
  // the logical page modulo the table width; an unmapped page drops the row.
  const int logical_page = position / c.page_size;
  const int slot = logical_page % c.max_pages_per_seq;
  const int physical =
      __ldg(a.page_table + int64_t(batch) * c.max_pages_per_seq + slot);
  if (physical < 0 || physical >= c.num_pages) return;
  const int64_t dst = cache_offset(c, a.cache_layer, physical,
                                   position - logical_page * c.page_size,
                                   kv_head, 0);
  if (warp == G) {
    prep_weighted_rope<D, ROT, kIeee>(a.cache_k + dst, x, a.k_norm_weight,
                                      cos_row, sin_row, lane);
    if (!has_v) prep_scale_free<D, kIeee>(a.cache_v + dst, x, lane);
  } else if (has_v) {
    prep_scale_free<D, kIeee>(a.cache_v + dst, x, lane);
  }
}

// grid (rows). The q_heads + 2 * kv_heads rows of a token are dealt to the
// warps two at a time (for 16 + 8 + 8 rows and 16 warps: one query head and one
// K or V head each). Global memory is touched with 128-bit accesses only: a
// warp loads both of its rows up front, passes each through a shared-memory row
// to get the arithmetic's ownership (lane l holds elements l + 32 i, which
// fixes the order of the sum of squares) and back; the RoPE factors of the
// token and the norm weights sit in registers. With 2-byte accesses and the
// tables re-read per head the kernel was bound by L1 transactions (32 per KB
// moved) at 0.39 of the HBM peak.
template <int D, int ROT, bool kIeee>
__global__ void prefill_prep_kernel(PrefillPrepArgs a) {
  constexpr int kVecs = D / 8 / 32;  // 128-bit packs per lane and row
  __shared__ __align__(16) __nv_bfloat16 s_rows[16][D];
  const int64_t row = blockIdx.x;
  const int warp = int(threadIdx.x) >> 5;
  const int lane = int(threadIdx.x) & 31;
  const int position = __ldg(a.token_position + row);
  if (position < 0) return;
  const int warps = int(blockDim.x) >> 5;
  const int tasks = a.q_heads + 2 * a.kv_heads;  // q heads, then K heads, then V heads
  // Source / destination row of a task; V tasks read raw K when there is no V
  // projection.
  auto source = [&](int task) -> const __nv_bfloat16 * {
    if (task < a.q_heads) return a.q + (row * a.q_heads + task) * D;
    const int kv = task - a.q_heads;
    if (kv < a.kv_heads) return a.k + (row * a.kv_heads + kv) * D;
    const int64_t off = (row * a.kv_heads + (kv - a.kv_heads)) * D;
    return (a.v != nullptr ? a.v : a.k) + off;
  };
  auto destination = [&](int task) -> __nv_bfloat16 * {
    if (task < a.q_heads) return a.q_prepared + (row * a.q_heads + task) * D;
    const int kv = task - a.q_heads;
    if (kv < a.kv_heads) return a.k_prepared + (row * a.kv_heads + kv) * D;
    return a.v_prepared + (row * a.kv_heads + (kv - a.kv_heads)) * D;
  };
  PrepTables<D, ROT> tables;
  tables.load_rope(a.cos + int64_t(position) * (ROT / 2),
                   a.sin + int64_t(position) * (ROT / 2), lane);
  __nv_bfloat16 *mine = s_rows[warp];
  auto finish = [&](int task, const uint4 (&packs)[kVecs]) {
#pragma unroll
    for (int v = 0; v < kVecs; ++v) {
      reinterpret_cast<uint4 *>(mine)[lane + 32 * v] = packs[v];
    }
    __syncwarp();
    float x[D / 32];
    load_head<D>(mine, lane, x);
    __nv_bfloat16 y[D / 32];
    if (task < a.q_heads + a.kv_heads) {
      tables.load_weight(task < a.q_heads ? a.q_norm_weight : a.k_norm_weight, lane);
      prep_weighted_rope_tables<D, ROT, kIeee>(y, x, tables);
    } else {
      prep_scale_free_values<D, kIeee>(y, x);
    }
    __syncwarp();
    store_head<D>(mine, y, lane);
    __syncwarp();
    uint4 *dst = reinterpret_cast<uint4 *>(destination(task));
#pragma unroll
    for (int v = 0; v < kVecs; ++v) {
      dst[lane + 32 * v] = reinterpret_cast<const uint4 *>(mine)[lane + 32 * v];
    }
    __syncwarp();
  };
  for (int t0 = warp; t0 < tasks; t0 += 2 * warps) {
    const int t1 = t0 + warps;
    uint4 p0[kVecs], p1[kVecs];
    const uint4 *s0 = reinterpret_cast<const uint4 *>(source(t0));
#pragma unroll
    for (int v = 0; v < kVecs; ++v) p0[v] = __ldg(s0 + lane + 32 * v);
    if (t1 < tasks) {
      const uint4 *s1 = reinterpret_cast<const uint4 *>(source(t1));
#pragma unroll
      for (int v = 0; v < kVecs; ++v) p1[v] = __ldg(s1 + lane + 32 * v);
    }
    finish(t0, p0);
    if (t1 < tasks) finish(t1, p1);
  }
}

// One CTA per token: all heads of the token are one contiguous row in the
// source and in the cache page, moved as 128-bit packs. With live_rows > 0 the
// grid covers only the last live_rows rows of every run of seq_len source rows
// (a prompt longer than the sliding window: only its tail stays in the ring).
__global__ __launch_bounds__(256) void kv_cache_write_kernel(
    __nv_bfloat16 *cache_k, __nv_bfloat16 *cache_v, Gemma4KvCacheConfig c,
    const int32_t *token_batch, const int32_t *token_position,
    const int32_t *page_table, int32_t layer, const __nv_bfloat16 *k,
    const __nv_bfloat16 *v, int32_t seq_len, int32_t live_rows) {
  int token = int(blockIdx.x);
  if (live_rows > 0) {
    const int run = token / live_rows;
    token = run * seq_len + (seq_len - live_rows) + (token - run * live_rows);
  }
  const int batch = __ldg(token_batch + token);
  const int position = __ldg(token_position + token);
  // Guards of src/gemma4_kv_cache.cu:27-34.
  if (batch < 0 || position < 0) return;
  if (batch >= c.batch_size) return;
  const int logical_page = position / c.page_size;
  if (c.window_size == 0 && logical_page >= c.max_pages_per_seq) return;
  const int slot = logical_page % c.max_pages_per_seq;
  const int physical =
      __ldg(page_table + int64_t(batch) * c.max_pages_per_seq + slot);
  if (physical < 0 || physical >= c.num_pages) return;
  const int page_offset = position - logical_page * c.page_size;

  const int vecs = c.num_heads * c.head_dim / 8;
  const uint4 *src_k =
      reinterpret_cast<const uint4 *>(k) + int64_t(token) * vecs;
  const uint4 *src_v =
      reinterpret_cast<const uint4 *>(v) + int64_t(token) * vecs;
  const int64_t dst = cache_offset(c, layer, physical, page_offset, 0, 0) / 8;
  uint4 *dst_k = reinterpret_cast<uint4 *>(cache_k) + dst;
  uint4 *dst_v = reinterpret_cast<uint4 *>(cache_v) + dst;
  for (int i = int(threadIdx.x); i < vecs; i += int(blockDim.x)) {
    const uint4 kk = __ldg(src_k + i);
    const uint4 vv = __ldg(src_v + i);
    dst_k[i] = kk;
    dst_v[i] = vv;
  }
}

template <typename Launch>
cudaError_t dispatch_geometry(int head_dim, int rotary_dim, int norm_mode,
                              Launch launch) {
  const bool ieee = norm_mode == B200KV_NORM_IEEE;
  if (head_dim == 256 && rotary_dim == 256) {
    return ieee ? launch(std::integral_constant<int, 256>{},
                         std::integral_constant<int, 256>{},
                         std::true_type{})
                : launch(std::integral_constant<int, 256>{},
                         std::integral_constant<int, 256>{},
                         std::false_type{});
  }
  if (head_dim == 512 && rotary_dim == 128) {
    return ieee ? launch(std::integral_constant<int, 512>{},
                         std::integral_constant<int, 128>{},
                         std::true_type{})
                : launch(std::integral_constant<int, 512>{},
                         std::integral_constant<int, 128>{},
                         std::false_type{});
  }
  return cudaErrorInvalidValue;  // geometry the kernels are not built for
}

}  // namespace

cudaError_t validate_append_args(const AppendArgs &a) {
  const Gemma4KvCacheConfig &c = a.cfg;
  if (a.q_prepared == nullptr || a.cache_k == nullptr ||
      a.cache_v == nullptr || a.page_table == nullptr ||
      a.token_position == nullptr || a.q == nullptr || a.k == nullptr ||
      a.q_norm_weight == nullptr || a.k_norm_weight == nullptr ||
      a.cos == nullptr || a.sin == nullptr || a.batch_count < 0 ||
      a.cache_layer < 0 || a.cache_layer >= c.num_layers ||
      c.num_pages <= 0 || c.page_size <= 0 || c.max_pages_per_seq <= 0 ||
      c.batch_size <= 0 || c.window_size < 0 || c.num_heads <= 0 ||
      a.q_heads <= 0 || a.q_heads % c.num_heads != 0 ||
      (a.norm_mode != B200KV_NORM_IEEE &&
       a.norm_mode != B200KV_NORM_RSQRT_APPROX)) {
    return cudaErrorInvalidValue;
  }
  const int G = a.q_heads / c.num_heads;
  const int warps = G + (a.v != nullptr ? 2 : 1);
  if (warps > 32 || c.num_heads > 65535) return cudaErrorInvalidValue;
  return cudaSuccess;
}

cudaError_t decode_append_bf16(const AppendArgs &a, cudaStream_t stream) {
  const Gemma4KvCacheConfig &c = a.cfg;
  if (a.batch_count == 0) return cudaSuccess;
  const cudaError_t valid = validate_append_args(a);
  if (valid != cudaSuccess) return valid;
  const int G = a.q_heads / c.num_heads;
  const int warps = G + (a.v != nullptr ? 2 : 1);
  const dim3 grid(a.batch_count, c.num_heads);
  return dispatch_geometry(
      c.head_dim, a.rotary_dim, a.norm_mode, [&](auto d, auto rot, auto ieee) {
        return launch_pdl(
            decode_append_kernel<decltype(d)::value, decltype(rot)::value,
                                 decltype(ieee)::value>,
            grid, dim3(warps * 32), 0, stream, a);
      });
}

cudaError_t prefill_prep_bf16(const PrefillPrepArgs &a, cudaStream_t stream) {
  if (a.rows == 0) return cudaSuccess;
  if (a.q_prepared == nullptr || a.k_prepared == nullptr ||
      a.v_prepared == nullptr || a.q == nullptr || a.k == nullptr ||
      a.q_norm_weight == nullptr || a.k_norm_weight == nullptr ||
      a.cos == nullptr || a.sin == nullptr || a.token_position == nullptr ||
      a.rows < 0 || a.rows > 2147483647ll || a.q_heads <= 0 ||
      a.kv_heads <= 0 || a.kv_heads > a.q_heads ||
      (a.norm_mode != B200KV_NORM_IEEE &&
       a.norm_mode != B200KV_NORM_RSQRT_APPROX)) {
    return cudaErrorInvalidValue;
  }
  const uintptr_t align =
      reinterpret_cast<uintptr_t>(a.q) | reinterpret_cast<uintptr_t>(a.k) |
      reinterpret_cast<uintptr_t>(a.v) | reinterpret_cast<uintptr_t>(a.q_prepared) |
      reinterpret_cast<uintptr_t>(a.k_prepared) |
      reinterpret_cast<uintptr_t>(a.v_prepared);
  if ((align & 15u) != 0) return cudaErrorInvalidValue;  // rows move as 128-bit packs
  const int warps = a.q_heads < 16 ? a.q_heads : 16;
  return dispatch_geometry(
      a.head_dim, a.rotary_dim, a.norm_mode, [&](auto d, auto rot, auto ieee) {
        prefill_prep_kernel<decltype(d)::value, decltype(rot)::value,
                            decltype(ieee)::value>
            <<<unsigned(a.rows), warps * 32, 0, stream>>>(a);
        return cudaGetLastError();
      });
}

namespace {
// Argument contract of src/gemma4_kv_cache.cu:149-180.
bool valid_cache_write_args(const __nv_bfloat16 *cache_k,
                            const __nv_bfloat16 *cache_v,
                            const Gemma4KvCacheConfig &config,
                            const int32_t *page_table,
                            const int32_t *token_batch,
                            const int32_t *token_position, int32_t layer,
                            const __nv_bfloat16 *k, const __nv_bfloat16 *v) {
  return !(layer < 0 || layer >= config.num_layers || config.num_pages <= 0 ||
           config.page_size <= 0 || config.max_pages_per_seq <= 0 ||
           config.batch_size <= 0 || config.window_size < 0 ||
           config.num_heads <= 0 || config.head_dim <= 0 ||
           config.head_dim % 8 != 0 || cache_k == nullptr ||
           cache_v == nullptr || page_table == nullptr ||
           token_batch == nullptr || token_position == nullptr ||
           k == nullptr || v == nullptr);
}
}  // namespace

cudaError_t kv_cache_write_bf16(__nv_bfloat16 *cache_k, __nv_bfloat16 *cache_v,
                                Gemma4KvCacheConfig config,
                                const int32_t *page_table,
                                const int32_t *token_batch,
                                const int32_t *token_position,
                                int32_t token_count, int32_t layer,
                                const __nv_bfloat16 *k, const __nv_bfloat16 *v,
                                cudaStream_t stream) {
  if (token_count == 0) return cudaSuccess;
  if (token_count < 0 ||
      !valid_cache_write_args(cache_k, cache_v, config, page_table, token_batch,
                              token_position, layer, k, v)) {
    return cudaErrorInvalidValue;
  }
  const int vecs = config.num_heads * config.head_dim / 8;
  const int threads = vecs >= 256 ? 256 : ((vecs + 31) / 32) * 32;
  kv_cache_write_kernel<<<token_count, threads, 0, stream>>>(
      cache_k, cache_v, config, token_batch, token_position, page_table, layer,
      k, v, 0, 0);
  return cudaGetLastError();
}

cudaError_t prefill_cache_fill_bf16(__nv_bfloat16 *cache_k,
                                    __nv_bfloat16 *cache_v,
                                    Gemma4KvCacheConfig config,
                                    const int32_t *page_table,
                                    const int32_t *token_batch,
                                    const int32_t *token_position,
                                    int32_t batch_size, int32_t seq_len,
                                    int32_t layer, const __nv_bfloat16 *k,
                                    const __nv_bfloat16 *v,
                                    cudaStream_t stream) {
  if (batch_size < 0 || seq_len < 0) return cudaErrorInvalidValue;
  const int64_t rows = int64_t(batch_size) * seq_len;
  if (rows > 2147483647ll) return cudaErrorInvalidValue;
  // src/gemma4_prefill_megakernel.cu:189-207: everything for a linear cache or
  // a prompt that fits the window, else the last window_size rows of every
  // sequence (the reference issues one write per sequence for those).
  if (config.window_size == 0 || seq_len <= config.window_size) {
    return kv_cache_write_bf16(cache_k, cache_v, config, page_table, token_batch,
                               token_position, int32_t(rows), layer, k, v,
                               stream);
  }
  if (batch_size == 0) return cudaSuccess;
  if (!valid_cache_write_args(cache_k, cache_v, config, page_table, token_batch,
                              token_position, layer, k, v)) {
    return cudaErrorInvalidValue;
  }
  const int64_t live = int64_t(batch_size) * config.window_size;
  if (live > 2147483647ll) return cudaErrorInvalidValue;
  const int vecs = config.num_heads * config.head_dim / 8;
  const int threads = vecs >= 256 ? 256 : ((vecs + 31) / 32) * 32;
  kv_cache_write_kernel<<<unsigned(live), threads, 0, stream>>>(
      cache_k, cache_v, config, token_batch, token_position, page_table, layer,
      k, v, seq_len, config.window_size);
  return cudaGetLastError();
}

}  // namespace b200kv

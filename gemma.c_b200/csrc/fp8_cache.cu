// FP8 e4m3 KV cache: quantise-on-append with one fp32 scale per (page, KV
// head) and tensor. The reference has no FP8 cache; this file defines the rule
// and the host oracle (oracle/kv_oracle.cpp, orc_fp8_append) restates it, so
// stored bytes and scales are comparable bit for bit.
//
// Rule, per tensor, per (page, head), per call. Let R be the rows of the call
// that land in the page and o0 the page offset of the first of them:
//   s_old = (o0 == 0) ? 0 : scale[page, head]      (offset 0 restarts a page,
//                                                   which is what a ring slot
//                                                   needs when it is reused)
//   s_new = max(s_old, max(amax(R) / 448, FLT_MIN))
//   if s_new > s_old: every stored row r < o0 becomes enc((dec(byte)*s_old)/s_new)
//   rows of R are stored as enc(x / s_new);  scale[page, head] = s_new
// enc = round-to-nearest-even e4m3 with saturation to +-448; x are the
// prepared bf16 values (the same ones the bf16 cache would hold).
//
// V is [layer, page, offset, head, dim] with one byte per element (the bf16
// layout with the element size halved); scales are [layer, page, head].
// K has its own order inside a page, chosen for the tensor-core score step of
// the decode kernel (decode_fp8.cuh): blocks of 8 tokens, inside a block
// head-major, then token, then the 256-byte row with its 16-byte granules
// permuted: granule' = granule ^ 4 * (token & 1). A block of 8 tokens is still
// one contiguous 8 * heads * 256 bytes, so the decode producer copies it whole;
// one head's 8 rows are contiguous, so the MMA fragment loads are 128-bit and,
// with the permutation, free of bank conflicts. page_size must be a multiple
// of 8.
#include <cuda_fp8.h>

#include <cfloat>
#include <type_traits>

#include "kernels.cuh"
#include "prep_common.cuh"

namespace b200kv {

namespace {

__device__ __forceinline__ uint8_t enc_e4m3(float x) {
  return static_cast<uint8_t>(__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3));
}

// Two values to two codes in one conversion (low byte <- lo), the same rounding
// and saturation as enc_e4m3.
__device__ __forceinline__ uint32_t enc_e4m3x2(float lo, float hi) {
  return uint32_t(__nv_cvt_float2_to_fp8x2(make_float2(lo, hi), __NV_SATFINITE, __NV_E4M3));
}

__device__ __forceinline__ float dec_e4m3(uint8_t b) {
  const __half_raw h = __nv_cvt_fp8_to_halfraw(b, __NV_E4M3);
  return __half2float(*reinterpret_cast<const __half *>(&h));
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Byte index of element `dim` of row `r` (page offset) of `head`.
template <bool kIsK>
__device__ __forceinline__ int64_t fp8_byte_index(const Gemma4KvCacheConfig &c,
                                                  int layer, int physical, int r,
                                                  int head, int dim) {
  if constexpr (!kIsK) {
    return cache_offset(c, layer, physical, r, head, dim);
  } else {
    const int64_t page_bytes = int64_t(c.page_size) * c.num_heads * c.head_dim;
    const int64_t base = (int64_t(layer) * c.num_pages + physical) * page_bytes;
    const int tk = r & 7;
    const int granule = (dim >> 4) ^ ((tk & 1) << 2);
    return base + (int64_t(r >> 3) * c.num_heads + head) * 8 * c.head_dim +
           tk * c.head_dim + granule * 16 + (dim & 15);
  }
}

// First byte of the 256-byte row `r` of `head` (granule permutation aside).
template <bool kIsK>
__device__ __forceinline__ int64_t fp8_row_base(const Gemma4KvCacheConfig &c,
                                                int layer, int physical, int r,
                                                int head) {
  if constexpr (!kIsK) {
    return cache_offset(c, layer, physical, r, head, 0);
  } else {
    const int64_t page_bytes = int64_t(c.page_size) * c.num_heads * c.head_dim;
    return (int64_t(layer) * c.num_pages + physical) * page_bytes +
           (int64_t(r >> 3) * c.num_heads + head) * 8 * c.head_dim +
           (r & 7) * c.head_dim;
  }
}

// Re-encodes the rows < o0 already stored in a page for a grown scale.
template <int D, bool kIsK>
__device__ __forceinline__ void fp8_requantise_rows(uint8_t *cache,
                                                    const Gemma4KvCacheConfig &c,
                                                    int layer, int physical,
                                                    int head, int o0, float s_old,
                                                    float s_new, int lane) {
    // A stored row is 256 contiguous bytes in either layout (K only permutes
    // the granules inside it) and the re-encoding is elementwise, so a lane
    // takes 8 bytes of each row; 8 rows are in flight at a time.
    static_assert(D == 256, "a lane re-encodes 8 of a row's 256 bytes");
    constexpr int kBatch = 8;
    for (int r0 = 0; r0 < o0; r0 += kBatch) {
      uint2 w[kBatch];
#pragma unroll
      for (int i = 0; i < kBatch; ++i) {
        if (r0 + i < o0) {
          w[i] = *reinterpret_cast<const uint2 *>(
              cache + fp8_row_base<kIsK>(c, layer, physical, r0 + i, head) +
              lane * 8);
        }
      }
#pragma unroll
      for (int i = 0; i < kBatch; ++i) {
        if (r0 + i < o0) {
          uint32_t in[2] = {w[i].x, w[i].y}, out[2] = {0u, 0u};
#pragma unroll
          for (int b = 0; b < 8; ++b) {
            const float v =
                __fmul_rn(dec_e4m3(uint8_t(in[b >> 2] >> (8 * (b & 3)))), s_old);
            out[b >> 2] |= uint32_t(enc_e4m3(__fdiv_rn(v, s_new))) << (8 * (b & 3));
          }
          *reinterpret_cast<uint2 *>(
              cache + fp8_row_base<kIsK>(c, layer, physical, r0 + i, head) +
              lane * 8) = make_uint2(out[0], out[1]);
        }
      }
    }
}

// One warp stores `nrows` prepared rows of one (page, head, tensor) starting
// at page offset o0; value(r, j) is element lane + 32*j of row r as fp32.
// Applies the rule above, including the requantisation of the rows already in
// the page.
template <int D, bool kIsK, class RowValue>
__device__ __forceinline__ void fp8_store_rows(uint8_t *cache, float *scale_slot,
                                               const Gemma4KvCacheConfig &c,
                                               int layer, int physical, int head,
                                               int o0, int nrows, int lane,
                                               RowValue value) {
  float amax = 0.0f;
  for (int r = 0; r < nrows; ++r) {
#pragma unroll
    for (int j = 0; j < D / 32; ++j) amax = fmaxf(amax, fabsf(value(r, j)));
  }
  amax = warp_max(amax);
  float s_old = 0.0f;
  if (o0 != 0) {
    if (lane == 0) s_old = *scale_slot;
    s_old = __shfl_sync(0xffffffffu, s_old, 0);
  }
  const float s_new = fmaxf(s_old, fmaxf(__fdiv_rn(amax, 448.0f), FLT_MIN));
  if (s_new > s_old) {
    fp8_requantise_rows<D, kIsK>(cache, c, layer, physical, head, o0, s_old, s_new,
                                 lane);
  }
  for (int r = 0; r < nrows; ++r) {
#pragma unroll
    for (int j = 0; j < D / 32; ++j) {
      cache[fp8_byte_index<kIsK>(c, layer, physical, o0 + r, head,
                                 lane + 32 * j)] =
          enc_e4m3(__fdiv_rn(value(r, j), s_new));
    }
  }
  if (lane == 0) *scale_slot = s_new;
}

// The same rule for rows that come from memory (a prompt): row r of the call is
// 256 bf16 at src + r * row_stride. A lane takes 8 contiguous elements of every
// row (one 128-bit load, one 64-bit store); the rule is elementwise apart from
// the maximum, so the bytes are those of fp8_store_rows.
template <int D, bool kIsK>
__device__ __forceinline__ void fp8_store_rows_from_memory(
    uint8_t *cache, float *scale_slot, const Gemma4KvCacheConfig &c, int layer,
    int physical, int head, int o0, int nrows, int lane,
    const __nv_bfloat16 *src, int64_t row_stride) {
  static_assert(D == 256, "a lane owns 8 of a row's 256 elements");
  constexpr int kBatch = 8;
  const uint4 *rows = reinterpret_cast<const uint4 *>(src) + lane;
  const int64_t stride16 = row_stride / 8;
  float amax = 0.0f;
  for (int r0 = 0; r0 < nrows; r0 += kBatch) {
    uint4 w[kBatch];
#pragma unroll
    for (int i = 0; i < kBatch; ++i) {
      w[i] = r0 + i < nrows ? __ldg(rows + (r0 + i) * stride16)
                            : make_uint4(0u, 0u, 0u, 0u);
    }
#pragma unroll
    for (int i = 0; i < kBatch; ++i) {
      const uint32_t u[4] = {w[i].x, w[i].y, w[i].z, w[i].w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        amax = fmaxf(amax, fmaxf(fabsf(bf16_lo(u[k])), fabsf(bf16_hi(u[k]))));
      }
    }
  }
  amax = warp_max(amax);
  float s_old = 0.0f;
  if (o0 != 0) {
    if (lane == 0) s_old = *scale_slot;
    s_old = __shfl_sync(0xffffffffu, s_old, 0);
  }
  const float s_new = fmaxf(s_old, fmaxf(__fdiv_rn(amax, 448.0f), FLT_MIN));
  if (s_new > s_old) {
    fp8_requantise_rows<D, kIsK>(cache, c, layer, physical, head, o0, s_old, s_new,
                                 lane);
  }
  for (int r0 = 0; r0 < nrows; r0 += kBatch) {
    uint4 w[kBatch];
#pragma unroll
    for (int i = 0; i < kBatch; ++i) {
      w[i] = r0 + i < nrows ? __ldg(rows + (r0 + i) * stride16)
                            : make_uint4(0u, 0u, 0u, 0u);
    }
#pragma unroll
    for (int i = 0; i < kBatch; ++i) {
      if (r0 + i < nrows) {
        const int r = o0 + r0 + i;
        const uint32_t u[4] = {w[i].x, w[i].y, w[i].z, w[i].w};
        uint32_t out[2] = {0u, 0u};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          out[k >> 1] |= enc_e4m3x2(__fdiv_rn(bf16_lo(u[k]), s_new),
                                    __fdiv_rn(bf16_hi(u[k]), s_new))
                         << (16 * (k & 1));
        }
        // byte offset of elements 8 * lane .. + 7 inside the 256-byte row
        const int granule = kIsK ? ((lane >> 1) ^ ((r & 1) << 2)) : (lane >> 1);
        *reinterpret_cast<uint2 *>(cache +
                                   fp8_row_base<kIsK>(c, layer, physical, r, head) +
                                   granule * 16 + (lane & 1) * 8) =
            make_uint2(out[0], out[1]);
      }
    }
  }
  if (lane == 0) *scale_slot = s_new;
}

struct Fp8AppendArgs {
  AppendArgs base;     // cache_k / cache_v unused
  uint8_t *cache_k;
  uint8_t *cache_v;
  float *scale_k;
  float *scale_v;
};

// Fused decode append into the fp8 cache: same grid and warp roles as the bf16
// kernel (append_prep.cu); K and V warps quantise what they prepared.
template <int D, int ROT, bool kIeee>
__global__ void decode_append_fp8_kernel(Fp8AppendArgs args) {
  const AppendArgs &a = args.base;
  const int batch = int(blockIdx.x);
  const int kv_head = int(blockIdx.y);
  const int warp = int(threadIdx.x) >> 5;
  const int lane = int(threadIdx.x) & 31;
  const Gemma4KvCacheConfig &c = a.cfg;
  const int G = a.q_heads / c.num_heads;
  const bool has_v = a.v != nullptr;

  pdl_wait_for_predecessor();
  pdl_release_successor();

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
  const int logical_page = position / c.page_size;
  const int slot = logical_page % c.max_pages_per_seq;
  const int physical =
      __ldg(a.page_table + int64_t(batch) * c.max_pages_per_seq + slot);
  if (physical < 0 || physical >= c.num_pages) return;
  const int o0 = position - logical_page * c.page_size;
  const int64_t scale_index =
      (int64_t(a.cache_layer) * c.num_pages + physical) * c.num_heads + kv_head;

  __nv_bfloat16 y[D / 32] = {};
  auto from_registers = [&y](int, int j) { return __bfloat162float(y[j]); };
  if (warp == G) {
    prep_weighted_rope_values<D, ROT, kIeee>(y, x, a.k_norm_weight, cos_row,
                                             sin_row, lane);
    fp8_store_rows<D, true>(args.cache_k, args.scale_k + scale_index, c,
                            a.cache_layer, physical, kv_head, o0, 1, lane,
                            from_registers);
    if (!has_v) {
      prep_scale_free_values<D, kIeee>(y, x);
      fp8_store_rows<D, false>(args.cache_v, args.scale_v + scale_index, c,
                               a.cache_layer, physical, kv_head, o0, 1, lane,
                               from_registers);
    }
  } else if (has_v) {
    prep_scale_free_values<D, kIeee>(y, x);
    fp8_store_rows<D, false>(args.cache_v, args.scale_v + scale_index, c,
                             a.cache_layer, physical, kv_head, o0, 1, lane,
                             from_registers);
  }
}

struct Fp8RowsArgs {
  uint8_t *cache_k;
  uint8_t *cache_v;
  float *scale_k;
  float *scale_v;
  Gemma4KvCacheConfig cfg;
  const int32_t *page_table;
  const int32_t *seq_batch;
  const int32_t *first_position;
  const int32_t *row_count;
  const int32_t *row_start;
  int32_t layer;
  const __nv_bfloat16 *k;
  const __nv_bfloat16 *v;
};

// Bulk append of prepared rows (a prompt). grid (page of the call, sequence of
// the call, head); warp 0 handles K, warp 1 V; all rows of the call that land
// in the page form one group, so the page's scale is the group's amax. The
// rows of one call must map to distinct cache rows.
template <int D>
__global__ __launch_bounds__(64) void fp8_append_rows_kernel(Fp8RowsArgs a) {
  const int s = int(blockIdx.y);
  const int head = int(blockIdx.z);
  const int tensor = int(threadIdx.x) >> 5;
  const int lane = int(threadIdx.x) & 31;
  const Gemma4KvCacheConfig &c = a.cfg;
  const int batch = __ldg(a.seq_batch + s);
  const int first = __ldg(a.first_position + s);
  const int count = __ldg(a.row_count + s);
  if (batch < 0 || batch >= c.batch_size || first < 0 || count <= 0) return;
  const int ps = c.page_size;
  const int logical_page = first / ps + int(blockIdx.x);
  const int p0 = max(first, logical_page * ps);
  const int p1 = min(first + count, (logical_page + 1) * ps);
  if (p0 >= p1) return;
  if (c.window_size == 0 && logical_page >= c.max_pages_per_seq) return;
  const int slot = logical_page % c.max_pages_per_seq;
  const int physical =
      __ldg(a.page_table + int64_t(batch) * c.max_pages_per_seq + slot);
  if (physical < 0 || physical >= c.num_pages) return;
  const int64_t src_row0 = int64_t(__ldg(a.row_start + s)) + (p0 - first);
  const __nv_bfloat16 *src =
      (tensor == 0 ? a.k : a.v) + (src_row0 * c.num_heads + head) * D;
  const int64_t row_stride = int64_t(c.num_heads) * D;
  const int64_t scale_index =
      (int64_t(a.layer) * c.num_pages + physical) * c.num_heads + head;
  if (tensor == 0) {
    fp8_store_rows_from_memory<D, true>(a.cache_k, a.scale_k + scale_index, c,
                                        a.layer, physical, head,
                                        p0 - logical_page * ps, p1 - p0, lane, src,
                                        row_stride);
  } else {
    fp8_store_rows_from_memory<D, false>(a.cache_v, a.scale_v + scale_index, c,
                                         a.layer, physical, head,
                                         p0 - logical_page * ps, p1 - p0, lane, src,
                                         row_stride);
  }
}

}  // namespace

cudaError_t decode_append_fp8(const AppendArgs &a, uint8_t *cache_k,
                              uint8_t *cache_v, float *scale_k, float *scale_v,
                              cudaStream_t stream) {
  const Gemma4KvCacheConfig &c = a.cfg;
  if (a.batch_count == 0) return cudaSuccess;
  if (a.q_prepared == nullptr || cache_k == nullptr || cache_v == nullptr ||
      scale_k == nullptr || scale_v == nullptr || a.page_table == nullptr ||
      a.token_position == nullptr || a.q == nullptr || a.k == nullptr ||
      a.q_norm_weight == nullptr || a.k_norm_weight == nullptr ||
      a.cos == nullptr || a.sin == nullptr || a.batch_count < 0 ||
      a.cache_layer < 0 || a.cache_layer >= c.num_layers || c.num_pages <= 0 ||
      c.page_size <= 0 || c.max_pages_per_seq <= 0 || c.batch_size <= 0 ||
      c.window_size < 0 || c.num_heads <= 0 || a.q_heads <= 0 ||
      a.q_heads % c.num_heads != 0 ||
      (a.norm_mode != B200KV_NORM_IEEE &&
       a.norm_mode != B200KV_NORM_RSQRT_APPROX) ||
      ((reinterpret_cast<uintptr_t>(cache_k) |
        reinterpret_cast<uintptr_t>(cache_v)) & 15u) != 0) {
    return cudaErrorInvalidValue;
  }
  const int G = a.q_heads / c.num_heads;
  const int warps = G + (a.v != nullptr ? 2 : 1);
  if (warps > 32 || c.num_heads > 65535) return cudaErrorInvalidValue;
  if (c.head_dim != 256 || a.rotary_dim != 256 || c.page_size % 8 != 0) {
    return cudaErrorInvalidValue;
  }
  Fp8AppendArgs args = {a, cache_k, cache_v, scale_k, scale_v};
  const dim3 grid(a.batch_count, c.num_heads);
  if (a.norm_mode == B200KV_NORM_IEEE) {
    return launch_pdl(decode_append_fp8_kernel<256, 256, true>, grid,
                      dim3(warps * 32), 0, stream, args);
  }
  return launch_pdl(decode_append_fp8_kernel<256, 256, false>, grid,
                    dim3(warps * 32), 0, stream, args);
}

cudaError_t fp8_append_rows(uint8_t *cache_k, uint8_t *cache_v, float *scale_k,
                            float *scale_v, Gemma4KvCacheConfig c,
                            const int32_t *page_table, const int32_t *seq_batch,
                            const int32_t *first_position,
                            const int32_t *row_count, const int32_t *row_start,
                            int32_t seq_count, int32_t max_row_count,
                            int32_t layer, const __nv_bfloat16 *k,
                            const __nv_bfloat16 *v, cudaStream_t stream) {
  if (seq_count == 0 || max_row_count == 0) return cudaSuccess;
  if (cache_k == nullptr || cache_v == nullptr || scale_k == nullptr ||
      scale_v == nullptr || page_table == nullptr || seq_batch == nullptr ||
      first_position == nullptr || row_count == nullptr ||
      row_start == nullptr || k == nullptr || v == nullptr || seq_count < 0 ||
      seq_count > 65535 || max_row_count < 0 || layer < 0 ||
      layer >= c.num_layers || c.num_pages <= 0 || c.page_size <= 0 ||
      c.max_pages_per_seq <= 0 || c.batch_size <= 0 || c.window_size < 0 ||
      c.num_heads <= 0 || c.num_heads > 65535 || c.head_dim != 256 ||
      c.page_size % 8 != 0 ||
      ((reinterpret_cast<uintptr_t>(cache_k) |
        reinterpret_cast<uintptr_t>(cache_v) | reinterpret_cast<uintptr_t>(k) |
        reinterpret_cast<uintptr_t>(v)) & 15u) != 0) {
    return cudaErrorInvalidValue;
  }
  Fp8RowsArgs a = {cache_k, cache_v, scale_k, scale_v, c, page_table, seq_batch,
                   first_position, row_count, row_start, layer, k, v};
  // A run of max_row_count rows touches at most this many pages.
  const int pages = (max_row_count + c.page_size - 2) / c.page_size + 1;
  fp8_append_rows_kernel<256>
      <<<dim3(pages, seq_count, c.num_heads), 64, 0, stream>>>(a);
  return cudaGetLastError();
}

}  // namespace b200kv

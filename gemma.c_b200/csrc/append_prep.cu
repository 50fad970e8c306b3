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

#include <algorithm>
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

// ---------------------------------------------------------------------------
// Whole-prompt prep. grid (rows): a CTA per token; its q_heads + 2 * kv_heads
// head rows are dealt to the warps in PAIRS of the same kind (two query heads,
// two K heads, two V heads; a last odd head pairs with nothing).
//
// The arithmetic's ownership -- lane l holds elements l + 32 i, which fixes the
// order of the sum of squares and so the bits of the scale -- is not the order
// the rows lie in memory. Global memory is touched with 128-bit accesses only;
// the transposition goes through shared memory, and what made the first
// versions issue-bound (2-byte accesses: 32 L1 transactions per KB moved, 0.39 of
// the HBM peak; then sixteen 2-byte shared accesses and one scalar fp32 operation
// per element and step: 250 warp instructions per KB, 0.50) is halved twice:
//   * the two rows of a pair are interleaved element by element (byte permutes
//     on the 128-bit packs), so that every 32-bit shared-memory word holds one
//     element of each row: a lane reads its elements of BOTH rows with D / 32
//     word loads and writes both results with D / 32 word stores;
//   * the arithmetic runs on both rows at once in packed fp32 pairs
//     (fma.rn.f32x2 / mul.rn{.ftz}.f32x2: each half is the scalar operation with
//     the same rounding, so the bits are those of prep_common.cuh), and results
//     are rounded and packed two at a time (cvt.rn.bf16x2.f32).
// Shared-memory words are laid out so that neither side conflicts: a pack's
// eight words go to two regions (elements 0..3 and 4..7 of the pack, 16 bytes
// per lane and region), the second region 16 words off a multiple of 32.
// ---------------------------------------------------------------------------
using f32x2 = unsigned long long;  // two fp32: low half = first row of the pair

__device__ __forceinline__ f32x2 pack2(float lo, float hi) {
  f32x2 r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(f32x2 v, float &lo, float &hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ f32x2 fma2_rn(f32x2 a, f32x2 b, f32x2 c) {
  f32x2 r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ f32x2 mul2_rn(f32x2 a, f32x2 b) {
  f32x2 r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
// The prep multiplications (flush-to-zero in the approx mode, see mul_prep).
template <bool kIeee>
__device__ __forceinline__ f32x2 mul2_prep(f32x2 a, f32x2 b) {
  f32x2 r;
  if constexpr (kIeee) {
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  } else {
    asm("mul.rn.ftz.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  }
  return r;
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
  return r;
}
// bf16 pair from two floats: low half <- lo.
__device__ __forceinline__ uint32_t cvt_bf16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

template <int D>
struct PairLayout {
  static constexpr int kRegion = D / 2 + 16;  // words; the second region starts here
  static constexpr int kWords = D + 16;
  // word of element e of the interleaved pair
  __device__ static int word(int e) {
    return ((e & 7) >> 2) * kRegion + (e >> 3) * 4 + (e & 3);
  }
};

// rsqrt(mean of squares + eps) of one row from its warp-wide sum of squares.
template <int D, bool kIeee>
__device__ __forceinline__ float rms_scale_of(float ss) {
  const float t = __fadd_rn(__fdiv_rn(ss, float(D)), kRmsEps);
  if constexpr (kIeee) {
    return __fdiv_rn(1.0f, __fsqrt_rn(t));
  } else {
    return rsqrtf(t);
  }
}

// What a warp needs to know about pair `pr` of a token: kind 0 query heads, 1 K
// heads, 2 V heads; whether the pair has a second row; where its rows lie.
struct PrepPair {
  int kind;
  bool second;
  const __nv_bfloat16 *src;
  __nv_bfloat16 *dst;
};

template <int D>
__device__ __forceinline__ PrepPair prep_pair_of(const PrefillPrepArgs &a, int64_t row, int pr,
                                                 int pq, int pk) {
  PrepPair p;
  p.kind = pr < pq ? 0 : (pr < pq + pk ? 1 : 2);
  const int h0 = 2 * (p.kind == 0 ? pr : (p.kind == 1 ? pr - pq : pr - pq - pk));
  p.second = h0 + 1 < (p.kind == 0 ? a.q_heads : a.kv_heads);
  p.src = p.kind == 0
              ? a.q + (row * a.q_heads + h0) * D
              : ((p.kind == 1 || a.v == nullptr ? a.k : a.v) + (row * a.kv_heads + h0) * D);
  p.dst = p.kind == 0 ? a.q_prepared + (row * a.q_heads + h0) * D
                      : ((p.kind == 1 ? a.k_prepared : a.v_prepared) +
                         (row * a.kv_heads + h0) * D);
  return p;
}

// Up to 8 warps of two pairs each, four CTAs per SM: the kernel lives on loads in
// flight (a token's rows, then its position's RoPE factors), so the rows of a
// warp's first pair are asked for before anything else and the next pair's as
// soon as the current one is in shared memory.
constexpr int kPrepWarps = 8;

template <int D, int ROT, bool kIeee>
__global__ __launch_bounds__(kPrepWarps * 32, D == 256 ? 4 : 2) void prefill_prep_kernel(PrefillPrepArgs a) {
  constexpr int E = D / 32;          // elements per lane and row
  constexpr int kVecs = D / 8 / 32;  // 128-bit packs per lane and row
  constexpr int kPairs = ROT / 64;   // rotated (lo, hi) element pairs per lane
  using L = PairLayout<D>;
  __shared__ __align__(16) uint32_t s_pairs[kPrepWarps][L::kWords];
  const int64_t row = blockIdx.x;
  const int warp = int(threadIdx.x) >> 5;
  const int lane = int(threadIdx.x) & 31;
  const int warps = int(blockDim.x) >> 5;
  // pairs: of query heads, then of K heads, then of V heads
  const int pq = (a.q_heads + 1) / 2;
  const int pk = (a.kv_heads + 1) / 2;
  const int pairs = pq + 2 * pk;
  if (warp >= pairs) return;

  uint4 pa[kVecs], pb[kVecs];
  auto fetch = [&](const PrepPair &p) {
#pragma unroll
    for (int v = 0; v < kVecs; ++v) {
      pa[v] = __ldg(reinterpret_cast<const uint4 *>(p.src) + lane + 32 * v);
      pb[v] = p.second ? __ldg(reinterpret_cast<const uint4 *>(p.src + D) + lane + 32 * v)
                       : make_uint4(0u, 0u, 0u, 0u);
    }
  };
  PrepPair cur = prep_pair_of<D>(a, row, warp, pq, pk);
  fetch(cur);
  const int position = __ldg(a.token_position + row);
  if (position < 0) return;

  // RoPE factors of the token for this lane's rotated elements
  float rc[kPairs], rs[kPairs];
  {
    const float *cos_row = a.cos + int64_t(position) * (ROT / 2);
    const float *sin_row = a.sin + int64_t(position) * (ROT / 2);
#pragma unroll
    for (int i = 0; i < kPairs; ++i) {
      rc[i] = __ldg(cos_row + lane + i * 32);
      rs[i] = __ldg(sin_row + lane + i * 32);
    }
  }
  uint32_t *mine = s_pairs[warp];
  // this lane's words of the interleaved pair: element lane + 32 i
  const int word0 = ((lane & 7) >> 2) * L::kRegion + (lane >> 3) * 4 + (lane & 3);  // + 16 i

  for (int pr = warp; pr < pairs; pr += warps) {
    // 1. both rows, interleaved, into shared memory; then the next pair's rows are asked for
#pragma unroll
    for (int v = 0; v < kVecs; ++v) {
      const int pv = lane + 32 * v;
      reinterpret_cast<uint4 *>(mine)[pv] =
          make_uint4(prmt(pa[v].x, pb[v].x, 0x5410u), prmt(pa[v].x, pb[v].x, 0x7632u),
                     prmt(pa[v].y, pb[v].y, 0x5410u), prmt(pa[v].y, pb[v].y, 0x7632u));
      reinterpret_cast<uint4 *>(mine + L::kRegion)[pv] =
          make_uint4(prmt(pa[v].z, pb[v].z, 0x5410u), prmt(pa[v].z, pb[v].z, 0x7632u),
                     prmt(pa[v].w, pb[v].w, 0x5410u), prmt(pa[v].w, pb[v].w, 0x7632u));
    }
    const PrepPair now = cur;
    if (pr + warps < pairs) {
      cur = prep_pair_of<D>(a, row, pr + warps, pq, pk);
      fetch(cur);
    }
    // the norm weights of this lane's elements (query and K rows)
    float w[E];
    if (now.kind != 2) {
      const __nv_bfloat16 *weight = now.kind == 0 ? a.q_norm_weight : a.k_norm_weight;
#pragma unroll
      for (int i = 0; i < E; ++i) w[i] = __bfloat162float(__ldg(weight + lane + i * 32));
    }
    __syncwarp();
    // 2. this lane's elements of both rows; sums of squares in the reference's order
    f32x2 x[E];
    f32x2 ss = pack2(0.0f, 0.0f);
#pragma unroll
    for (int i = 0; i < E; ++i) {
      const uint32_t wd = mine[word0 + 16 * i];
      x[i] = pack2(__uint_as_float(wd << 16), __uint_as_float(wd & 0xffff0000u));
      ss = fma2_rn(x[i], x[i], ss);
    }
    float ss_a, ss_b;
    unpack2(ss, ss_a, ss_b);
#pragma unroll
    for (int offset = 16; offset > 0; offset /= 2) {
      ss_a = __fadd_rn(ss_a, __shfl_xor_sync(0xffffffffu, ss_a, offset));
      ss_b = __fadd_rn(ss_b, __shfl_xor_sync(0xffffffffu, ss_b, offset));
    }
    const f32x2 scale2 = pack2(rms_scale_of<D, kIeee>(ss_a), rms_scale_of<D, kIeee>(ss_b));
    // 3. norm (+ weight, + rotation), rounded and packed per element of the pair;
    // a lane's words are its own: they take the results
    if (now.kind == 2) {
#pragma unroll
      for (int i = 0; i < E; ++i) {
        float ya, yb;
        unpack2(mul2_prep<kIeee>(x[i], scale2), ya, yb);
        mine[word0 + 16 * i] = cvt_bf16x2(ya, yb);
      }
    } else {
#pragma unroll
      for (int i = 0; i < E; ++i) {
        x[i] = mul2_prep<kIeee>(mul2_prep<kIeee>(x[i], scale2), pack2(w[i], w[i]));
      }
#pragma unroll
      for (int i = 0; i < kPairs; ++i) {  // lo' = lo c - hi s, hi' = hi c + lo s
        const f32x2 lo = x[i];
        const f32x2 hi = x[i + kPairs];
        const f32x2 c2 = pack2(rc[i], rc[i]);
        x[i] = fma2_rn(hi, pack2(-rs[i], -rs[i]), mul2_rn(lo, c2));
        x[i + kPairs] = fma2_rn(lo, pack2(rs[i], rs[i]), mul2_rn(hi, c2));
      }
#pragma unroll
      for (int i = 0; i < E; ++i) {
        float ya, yb;
        unpack2(x[i], ya, yb);
        mine[word0 + 16 * i] = cvt_bf16x2(ya, yb);
      }
    }
    __syncwarp();
    // 4. de-interleave and out
#pragma unroll
    for (int v = 0; v < kVecs; ++v) {
      const int pv = lane + 32 * v;
      const uint4 w0 = reinterpret_cast<const uint4 *>(mine)[pv];
      const uint4 w1 = reinterpret_cast<const uint4 *>(mine + L::kRegion)[pv];
      reinterpret_cast<uint4 *>(now.dst)[pv] =
          make_uint4(prmt(w0.x, w0.y, 0x5410u), prmt(w0.z, w0.w, 0x5410u),
                     prmt(w1.x, w1.y, 0x5410u), prmt(w1.z, w1.w, 0x5410u));
      if (now.second) {
        reinterpret_cast<uint4 *>(now.dst + D)[pv] =
            make_uint4(prmt(w0.x, w0.y, 0x7632u), prmt(w0.z, w0.w, 0x7632u),
                       prmt(w1.x, w1.y, 0x7632u), prmt(w1.z, w1.w, 0x7632u));
      }
    }
    __syncwarp();  // the next pair's packs overwrite the words
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
  // pairs of head rows per token; two pairs per warp where there are that many
  const int pairs = (a.q_heads + 1) / 2 + 2 * ((a.kv_heads + 1) / 2);
  const int warps = std::max(1, std::min(kPrepWarps, (pairs + 1) / 2));
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

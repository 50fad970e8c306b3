// Split-KV flash-decode with evenly balanced key ranges.
//
// The reference (and decode_attention.cu) cut every sequence into splits of a
// fixed size and give each split a CTA; with ragged batches the CTA count is
// whatever the lengths make it, so the last wave is partly empty and every CTA
// pays its own pipeline fill and drain. Here the live keys of the whole batch
// are laid end to end and divided into one contiguous range per CTA, the same
// number of keys each. The grid is a fixed number of CTAs (two per SM), every
// CTA streams the same amount of HBM, the producer's ring never drains at a
// split boundary, and a sequence produces at most one partial per CTA that
// touches it (a sequence that falls entirely inside one range is finished by
// that CTA and never goes through scratch). The CTA walks the sequences of
// its range in order; a query head's (m, l, acc) is flushed when the walk
// leaves the sequence.
//
// Same math per stage as the fixed-split kernel (decode_common.cuh); same
// results within fp32 summation order. Partials live in the caller's scratch:
// the partial of CTA c for sequence b sits in slot c + b, which is unique
// because ranges and sequences advance together.
#include <cstring>
#include <type_traits>

#include "decode_common.cuh"
#include "decode_fp8.cuh"
#include "balanced_partition.cuh"
#include "kernels.cuh"
#include "prep_common.cuh"

namespace b200kv {

namespace {

// ---- in-kernel append (fused kernels) ---------------------------------------
// One consumer warp = one KV head. The arithmetic and the lane ownership are
// the append kernel's (prep_common.cuh), so the rows are the same bits; the
// per-warp 1 KiB buffer turns "lane l holds elements l + 32 i" into rows in
// memory order.

// Prepared query rows of heads 2 * head, 2 * head + 1 of sequence b, returned
// as the 16 bytes per lane the attention wants (dims 8 * lane .. + 7). When
// `with_kv`, also leaves the prepared K row at wbuf[0, 512) and the V row at
// wbuf[512, 1024).
template <bool kIeee>
__device__ __forceinline__ void prepare_rows(uint4 (&qpack)[2],
                                             const BalancedParams &p, int b,
                                             int head, int pos, bool with_kv,
                                             uint8_t *wbuf, int lane) {
  constexpr int D = 256;
  const float *cos_row = p.cos + int64_t(pos) * (D / 2);
  const float *sin_row = p.sin + int64_t(pos) * (D / 2);
  const int64_t kv_src = (int64_t(b) * p.cfg.num_heads + head) * D;
  float xq[2][D / 32], xk[D / 32], xv[D / 32];
#pragma unroll
  for (int g = 0; g < 2; ++g) {
    load_head<D>(p.raw_q + (int64_t(b) * p.q_heads + head * 2 + g) * D, lane,
                 xq[g]);
  }
  const bool has_v = p.raw_v != nullptr;
  if (with_kv) {
    load_head<D>(p.raw_k + kv_src, lane, xk);
    if (has_v) load_head<D>(p.raw_v + kv_src, lane, xv);
  }
  __nv_bfloat16 *rows = reinterpret_cast<__nv_bfloat16 *>(wbuf);
  __nv_bfloat16 y[D / 32];
#pragma unroll
  for (int g = 0; g < 2; ++g) {
    prep_weighted_rope_values<D, D, kIeee>(y, xq[g], p.q_norm_weight, cos_row,
                                           sin_row, lane);
    store_head<D>(rows + g * D, y, lane);
  }
  __syncwarp();
#pragma unroll
  for (int g = 0; g < 2; ++g) {
    qpack[g] = reinterpret_cast<const uint4 *>(wbuf)[g * 32 + lane];
  }
  __syncwarp();
  if (with_kv) {
    prep_weighted_rope_values<D, D, kIeee>(y, xk, p.k_norm_weight, cos_row,
                                           sin_row, lane);
    store_head<D>(rows, y, lane);
    if (has_v) {
      prep_scale_free_values<D, kIeee>(y, xv);
    } else {
      prep_scale_free_values<D, kIeee>(y, xk);
    }
    store_head<D>(rows + D, y, lane);
    __syncwarp();
  }
}

// Physical page of position pos of sequence b, or -1 (unmapped: nothing is
// appended, src/gemma4_flash_attention_decode.cu:333-338).
__device__ __forceinline__ int append_page(const BalancedParams &p, int b,
                                           int pos) {
  const Gemma4KvCacheConfig &c = p.cfg;
  const int slot = (pos / c.page_size) % c.max_pages_per_seq;
  const int e = __ldg(p.page_table + int64_t(b) * c.max_pages_per_seq + slot);
  return (e >= 0 && e < c.num_pages) ? e : -1;
}

// What the append leaves in global memory for one (sequence, KV head): the two
// prepared query rows and, if the page is mapped, the new K and V rows (from
// wbuf). Call only after pdl_wait_for_predecessor().
__device__ __forceinline__ void store_appended_rows(const BalancedParams &p,
                                                    const uint4 (&qpack)[2],
                                                    int b, int head, int pos,
                                                    int physical,
                                                    const uint8_t *wbuf,
                                                    int lane) {
  constexpr int D = 256;
#pragma unroll
  for (int g = 0; g < 2; ++g) {
    reinterpret_cast<uint4 *>(p.q_prepared +
                              (int64_t(b) * p.q_heads + head * 2 + g) * D)[lane] =
        qpack[g];
  }
  if (physical >= 0) {
    const Gemma4KvCacheConfig &c = p.cfg;
    const int64_t off = cache_offset(
        c, p.layer, physical, pos - (pos / c.page_size) * c.page_size, head, 0);
    const uint4 *rows = reinterpret_cast<const uint4 *>(wbuf);
    // the fused kernels are handed the caches they may write
    uint4 *dst_k = reinterpret_cast<uint4 *>(
        static_cast<__nv_bfloat16 *>(const_cast<void *>(p.cache_k)) + off);
    uint4 *dst_v = reinterpret_cast<uint4 *>(
        static_cast<__nv_bfloat16 *>(const_cast<void *>(p.cache_v)) + off);
    dst_k[lane] = rows[lane];
    dst_v[lane] = rows[32 + lane];
  }
}

// Appends of sequences whose new position is not a live key of the attention
// (lengths and positions that do not belong together): no CTA meets the row
// while streaming, so CTA (b mod grid) does it here. All lanes of a consumer
// warp call it, after the warp's last use of wbuf.
template <bool kIeee>
__device__ __forceinline__ void append_unstreamed_rows(const BalancedParams &p,
                                                       const int *s_prefix,
                                                       const int *s_first,
                                                       int head, uint8_t *wbuf,
                                                       int lane) {
  for (int b = int(blockIdx.x); b < p.batch_count; b += int(gridDim.x)) {
    const int pos = __ldg(p.token_position + b);
    if (pos < 0) continue;
    const int first = s_first[b];
    const int count = s_prefix[b + 1] - s_prefix[b];
    if (pos >= first && pos < first + count) continue;  // its streamer does it
    uint4 qpack[2];
    if (p.raw_from_predecessor) pdl_wait_for_predecessor();
    prepare_rows<kIeee>(qpack, p, b, head, pos, true, wbuf, lane);
    pdl_wait_for_predecessor();
    store_appended_rows(p, qpack, b, head, pos, append_page(p, b, pos), wbuf,
                        lane);
    __syncwarp();
  }
}

// kMode: kAttentionOnly reads the prepared q and expects the step's rows in
// the cache (a preceding append launch); the fused modes take the step's raw
// projections, prepare q in the consumer warps, and the CTA whose range holds a
// sequence's new key prepares that row, uses it from shared memory and writes
// it to the cache: one launch per layer-step instead of two, and nothing the
// attention streams early depends on a preceding kernel.
template <class T, int kMode, int kMaxBatch>
__global__ __launch_bounds__(T::kThreads, T::kCtasPerSm) void decode_balanced_kernel(
    BalancedParams p) {
  constexpr int G = T::G;
  constexpr int ST = T::kStageTokens;
  constexpr bool kFused = kMode != kAttentionOnly;
  constexpr bool kIeee = kMode == kFusedIeee;
  static_assert(T::kWarpsPerHead == 1, "one warp per KV head: no merge step");
  static_assert(!kFused || !T::kFp8, "the fused append is bf16 only");
  extern __shared__ __align__(128) uint8_t smem[];
  constexpr int kAppendBytes =
      kFused ? T::kConsumerWarps * kAppendBufferBytesPerWarp : 0;
  int *s_prefix = reinterpret_cast<int *>(smem + T::kRingBytes + kAppendBytes);
  int *s_first = s_prefix + kMaxBatch + 1;
  __shared__ int s_warp_sums[32];

  const int warp = int(threadIdx.x) >> 5;
  const int lane = int(threadIdx.x) & 31;
  const Gemma4KvCacheConfig &cfg = p.cfg;
  [[maybe_unused]] uint8_t *wbuf =
      smem + T::kRingBytes + (warp & 7) * kAppendBufferBytesPerWarp;

  // Programmatic dependent launch. What this kernel reads before its
  // pdl_wait_for_predecessor() must have been complete before the preceding
  // kernel started:
  //  * attention only: the preceding kernel is this layer-step's append;
  //    lengths, page table and every cache row except those of the page that
  //    holds each sequence's newest key (the fp8 append may re-encode that
  //    whole page) qualify; the prepared q does not.
  //  * fused: the preceding kernel is the previous layer-step's combine, which
  //    started only after every CTA of that step's fused kernel had passed its
  //    own wait (the release below comes after the wait), so two kernels back
  //    everything is complete; one kernel back a cache row may still be in
  //    flight -- the previous step's newest key -- and the scratch may still be
  //    read. Pages from that key's page on are loaded after the wait; scratch,
  //    outputs and cache rows are written after the wait.
  // Every CTA waits before it exits, so "this grid is complete" still implies
  // "everything before it is complete".
  if constexpr (!kFused) pdl_release_successor();

  // The barriers are initialised under the scan's first load; its barriers
  // make them visible to the CTA.
  const Ring<T> ring(smem);
  if (threadIdx.x == 0) ring.init_barriers();
  scan_live_keys<kMaxBatch>(p, s_prefix, s_first, s_warp_sums);
  const int total = s_prefix[p.batch_count];
  const int width = range_width(max(total, 1), p.num_ctas, ST);
  const int r0 = int(blockIdx.x) * width;
  if (total == 0 || r0 >= total) {  // nothing to stream; the combine zeroes empty rows
    if constexpr (kFused) {
      if (warp < T::kConsumerWarps) {
        append_unstreamed_rows<kIeee>(p, s_prefix, s_first, warp, wbuf, lane);
      }
      // An idle CTA has touched nothing a predecessor owns (or has waited in
      // the append above) and leaves at once: small batches keep most of the
      // grid idle, and the next layer-step's CTAs need the room to start under
      // this one. CTA 0 keeps the "complete implies predecessors complete"
      // chain when no CTA has keys (a CTA with keys always waits).
      if (blockIdx.x != 0) return;
    }
    pdl_wait_for_predecessor();
    if constexpr (kFused) pdl_release_successor();
    return;
  }
  const int r1 = min(total, r0 + width);
  int b_start = 0;
  {
    int lo = 0, hi = p.batch_count - 1;  // last b with prefix[b] <= r0
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (s_prefix[mid] <= r0) lo = mid; else hi = mid - 1;
    }
    b_start = lo;
  }

  if (warp == T::kConsumerWarps) {
    // ------------------------------ producer ------------------------------
    const uint64_t policy = l2_policy_evict_first();
    const KvSource src = {static_cast<const uint8_t *>(p.cache_k),
                          static_cast<const uint8_t *>(p.cache_v),
                          p.page_table, p.layer};
    bool ok = true;
    bool waited = false;
    PageEntryCache page_cache;
    int it = 0;  // stages armed so far, across all pieces of the range
    int b = b_start, flat = r0;
    Segment seg;
    while (ok && next_segment(b, flat, r1, s_prefix, s_first, seg)) {
      const int a0 = (seg.pos0 / ST) * ST;
      const int nchunks = div_up(seg.pos1 - a0, ST);
      // first position of the first page the preceding kernels may have touched
      const int seq_len = s_first[seg.b] + s_prefix[seg.b + 1] - s_prefix[seg.b];
      const int newest = max(seq_len - (kFused ? 2 : 1), 0);
      const int fresh = (newest / cfg.page_size) * cfg.page_size;
      for (int c = 0; c < nchunks; ++c, ++it) {
        if (!waited && min(seg.pos1, a0 + (c + 1) * ST) > fresh) {
          pdl_wait_for_predecessor();
          waited = true;
        }
        const int stage = it % kStages;
        const int fill = it / kStages;
        if (fill > 0 &&
            !mbar_wait_bounded(ring.empty_bar(stage), uint32_t(fill - 1) & 1u)) {
          ok = false;
          break;
        }
        const int base = a0 + c * ST;
        if constexpr (T::kFp8) {
          const Fp8Scales scales = {p.scale_k, p.scale_v, p.scale_log2};
          producer_fill_stage_fp8(ring, src, scales, cfg, seg.b, base,
                                  max(seg.pos0, base), min(seg.pos1, base + ST),
                                  stage, policy, lane);
        } else {
          producer_fill_stage<T>(ring, src, cfg, seg.b, base, max(seg.pos0, base),
                                 min(seg.pos1, base + ST), stage, policy, lane,
                                 &page_cache);
        }
      }
    }
    for (int s = 0; s < kStages && s < it; ++s) {
      const int fill = (it - 1 - s) / kStages;
      if (!mbar_wait_bounded(ring.full_bar(s), uint32_t(fill) & 1u)) ok = false;
    }
    if (!waited) pdl_wait_for_predecessor();
    if constexpr (kFused) pdl_release_successor();
    if (!ok && lane == 0) set_status(p.status, B200KV_STATUS_WAIT_TIMEOUT);
    return;
  }

  // -------------------------------- consumers --------------------------------
  if constexpr (!kFused) {
    pdl_wait_for_predecessor();  // q comes from the append
  } else {
    if (p.raw_from_predecessor) pdl_wait_for_predecessor();
  }
  const int head = warp;  // kWarpsPerHead == 1
  std::conditional_t<T::kFp8, Fp8WarpState, WarpState<T>> st;
  int b = b_start, flat = r0;
  Segment seg, next;
  bool have = next_segment(b, flat, r1, s_prefix, s_first, seg);
  [[maybe_unused]] uint4 raw[G];
  if constexpr (!T::kFp8 && !kFused) {
    load_q_raw<T>(raw, p.q, int64_t(seg.b) * p.q_heads + head * G, lane);
  }
  int it = 0;
  while (have) {
    // fused: position of the sequence's new row, and whether this piece of the
    // sequence contains it (then this warp prepares, uses and stores the row)
    [[maybe_unused]] int new_pos = -1;
    [[maybe_unused]] int new_page = -1;
    [[maybe_unused]] bool owns_new = false;
    if constexpr (T::kFp8) {
      st.load_q(p.q + (int64_t(seg.b) * p.q_heads + head * G) * T::D, lane);
    } else if constexpr (kFused) {
      new_pos = __ldg(p.token_position + seg.b);
      owns_new = new_pos >= seg.pos0 && new_pos < seg.pos1;
      if (owns_new) new_page = append_page(p, seg.b, new_pos);  // in flight early
      if (new_pos >= 0) {
        prepare_rows<kIeee>(raw, p, seg.b, head, new_pos, owns_new, wbuf, lane);
      } else {  // no append for this sequence: q is what the caller left there
        load_q_raw<T>(raw, p.q_prepared, int64_t(seg.b) * p.q_heads + head * G,
                      lane);
      }
      st.set_q(raw, p.scale_log2);
    } else {
      st.set_q(raw, p.scale_log2);
    }
    st.reset();
    // Fetch the next sequence's query rows while this one streams.
    const bool have_next = next_segment(b, flat, r1, s_prefix, s_first, next);
    if constexpr (!T::kFp8 && !kFused) {
      if (have_next) {
        load_q_raw<T>(raw, p.q, int64_t(next.b) * p.q_heads + head * G, lane);
      }
    }
    const int a0 = (seg.pos0 / ST) * ST;
    const int nchunks = div_up(seg.pos1 - a0, ST);
    for (int c = 0; c < nchunks; ++c, ++it) {
      const int stage = it % kStages;
      const int fill = it / kStages;
      if (!mbar_wait_bounded(ring.full_bar(stage), uint32_t(fill) & 1u)) {
        if (lane == 0) set_status(p.status, B200KV_STATUS_WAIT_TIMEOUT);
        return;  // every other wait in this CTA is bounded as well
      }
      if constexpr (T::kFp8) {
        consume_stage_fp8(st, ring, stage, head, lane);
      } else {
        if constexpr (kFused) {
          // The stage that holds the new key: the copy brought whatever the
          // cache had there; this head's slice of the row is replaced by the
          // prepared one (only this warp reads the slice). The slot's mask bit
          // is set exactly when its page is mapped.
          const int slot = new_pos - (a0 + c * ST);
          if (owns_new && slot >= 0 && slot < ST &&
              ((ring.masks()[stage] >> slot) & 1ull) != 0ull) {
            uint8_t *k_row = smem + stage * T::kStageBytes +
                             slot * T::kRowBytes + head * T::D * 2;
            const uint4 *rows = reinterpret_cast<const uint4 *>(wbuf);
            reinterpret_cast<uint4 *>(k_row)[lane] = rows[lane];
            reinterpret_cast<uint4 *>(k_row + T::kStageTensorBytes)[lane] =
                rows[32 + lane];
            fence_proxy_async_shared();  // the next fill of the stage is a bulk copy
            __syncwarp();
          }
        }
        consume_stage<T>(st, ring, stage, head, 0, lane);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(ring.empty_bar(stage));
    }
    float l[G];
    st.denominators(l, lane);
    if constexpr (kFused) {
      pdl_wait_for_predecessor();
      pdl_release_successor();
      if (owns_new) {
        store_appended_rows(p, raw, seg.b, head, new_pos, new_page, wbuf, lane);
        __syncwarp();
      }
    }
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const int q_head = head * G + g;
      if (seg.whole) {
        write_output_row<T>(p.out, p.lse, int64_t(seg.b) * p.q_heads + q_head,
                            st.acc[g], st.m[g], l[g], lane);
      } else {
        const int64_t slot = int64_t(int(blockIdx.x) + seg.b) * p.q_heads + q_head;
        write_partial_row<T>(p.partial_m, p.partial_l, p.partial_acc, slot,
                             st.acc[g], st.m[g], l[g], lane);
      }
    }
    seg = next;
    have = have_next;
  }
  if constexpr (kFused) {
    append_unstreamed_rows<kIeee>(p, s_prefix, s_first, head, wbuf, lane);
  }
}

// One CTA per (sequence, q_head) row. Recomputes which CTAs touched the
// sequence from the same prefix sums and combines their partials; rows that
// one CTA finished alone are left as they are; empty rows are zeroed.
}  // namespace

bool decode_balanced_supported(const Gemma4KvCacheConfig &c, int q_heads,
                               int batch_count) {
  return c.head_dim == 256 && c.num_heads == 8 && q_heads == 16 &&
         batch_count <= kMaxBalancedBatch;
}

namespace {

template <class T, int kMode = kAttentionOnly, int kMaxBatch = kMaxBalancedBatch>
cudaError_t launch_balanced(BalancedParams p, int64_t scratch_slots,
                            cudaStream_t stream) {
  constexpr int kSmem =
      T::kRingBytes + (2 * kMaxBatch + 1) * 4 +
      (kMode != kAttentionOnly ? T::kConsumerWarps * kAppendBufferBytesPerWarp : 0);
  static_assert(T::kRingBytes % 16 == 0, "the append buffers hold 16-byte rows");
  // per SM: two CTAs, each with 1 KiB the system reserves and the static arrays
  static_assert(2 * (kSmem + 1024 + 256) <= 228 * 1024, "two CTAs per SM");
  int device = 0, sm_count = 0;
  cudaError_t st = cudaGetDevice(&device);
  if (st != cudaSuccess) return st;
  st = cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device);
  if (st != cudaSuccess) return st;
  // Slot c + b needs num_ctas + batch - 1 slots per head.
  const int64_t num_ctas = std::min<int64_t>(int64_t(sm_count) * T::kCtasPerSm,
                                             scratch_slots - p.batch_count);
  if (num_ctas < 1 || p.partial_m == nullptr || p.partial_l == nullptr ||
      p.partial_acc == nullptr) {
    return cudaErrorInvalidValue;
  }
  p.num_ctas = int32_t(num_ctas);
  if (p.batch_count > kMaxBatch) return cudaErrorInvalidValue;
  st = cudaFuncSetAttribute(decode_balanced_kernel<T, kMode, kMaxBatch>,
                            cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);
  if (st != cudaSuccess) return st;
  st = launch_pdl(decode_balanced_kernel<T, kMode, kMaxBatch>,
                  dim3(unsigned(num_ctas)), dim3(T::kThreads), kSmem, stream, p);
  if (st != cudaSuccess) return st;
  return launch_balanced_combine<T::D>(p, int(T::kStageTokens), stream);
}

BalancedParams balanced_params(const DecodeArgs &a) {
  BalancedParams p = {};
  p.out = a.out;
  p.lse = a.lse;
  p.q = a.q;
  p.cache_k = a.cache_k;
  p.cache_v = a.cache_v;
  p.cfg = a.cfg;
  p.page_table = a.page_table;
  p.seq_lengths = a.seq_lengths;
  p.layer = a.layer;
  p.scale_log2 = a.softmax_scale * 1.4426950408889634f;
  p.batch_count = a.batch_count;
  p.q_heads = a.q_heads;
  p.partial_m = a.partial_m;
  p.partial_l = a.partial_l;
  p.partial_acc = a.partial_acc;
  p.status = a.status;
  return p;
}

}  // namespace

cudaError_t decode_attention_balanced_bf16(const DecodeArgs &a,
                                           cudaStream_t stream) {
  if (decode_gqa16_supported(a.cfg, a.q_heads, a.batch_count)) {
    return decode_attention_gqa16_bf16(a, stream);
  }
  if (!decode_balanced_supported(a.cfg, a.q_heads, a.batch_count)) {
    return cudaErrorInvalidValue;
  }
  return launch_balanced<DecodeTraits<256, 8, 2, 8>>(
      balanced_params(a), int64_t(a.batch_count) * a.num_splits, stream);
}

cudaError_t decode_attention_fp8(const DecodeArgs &a, const void *cache_k,
                                 const void *cache_v, const float *scale_k,
                                 const float *scale_v, cudaStream_t stream) {
  const Gemma4KvCacheConfig &c = a.cfg;
  if (a.out == nullptr || a.q == nullptr || cache_k == nullptr ||
      cache_v == nullptr || scale_k == nullptr || scale_v == nullptr ||
      a.page_table == nullptr || a.seq_lengths == nullptr ||
      a.batch_count <= 0 || a.layer < 0 || a.layer >= c.num_layers ||
      c.num_pages <= 0 || c.page_size <= 0 || c.max_pages_per_seq <= 0 ||
      c.window_size < 0 || a.num_splits <= 0 || !(a.softmax_scale > 0.0f) ||
      c.page_size % Fp8DecodeTraits::kStageTokens != 0 ||
      !decode_balanced_supported(c, a.q_heads, a.batch_count)) {
    return cudaErrorInvalidValue;
  }
  if (c.window_size > 0 &&
      int64_t(c.max_pages_per_seq) * c.page_size < c.window_size) {
    return cudaErrorInvalidValue;
  }
  const uintptr_t align = reinterpret_cast<uintptr_t>(cache_k) |
                          reinterpret_cast<uintptr_t>(cache_v) |
                          reinterpret_cast<uintptr_t>(a.q) |
                          reinterpret_cast<uintptr_t>(a.out) |
                          reinterpret_cast<uintptr_t>(a.partial_acc);
  if ((align & 15u) != 0) return cudaErrorInvalidValue;
  BalancedParams p = balanced_params(a);
  p.cache_k = cache_k;
  p.cache_v = cache_v;
  p.scale_k = scale_k;
  p.scale_v = scale_v;
  return launch_balanced<Fp8DecodeTraits>(
      p, int64_t(a.batch_count) * a.num_splits, stream);
}

bool decode_fused_supported(const AppendArgs &ap, const DecodeArgs &a) {
  const Gemma4KvCacheConfig &c = a.cfg;
  return a.split_size == 0 &&
         decode_balanced_supported(c, a.q_heads, a.batch_count) &&
         ap.rotary_dim == 256 && ap.q_heads == a.q_heads &&
         ap.batch_count == a.batch_count && ap.cache_layer == a.layer &&
         ap.page_table == a.page_table && ap.q_prepared == a.q &&
         ap.cache_k == a.cache_k && ap.cache_v == a.cache_v &&
         memcmp(&ap.cfg, &c, sizeof(c)) == 0;
}

cudaError_t decode_layer_step_fused_bf16(const AppendArgs &ap,
                                         const DecodeArgs &a,
                                         cudaStream_t stream) {
  cudaError_t st = validate_append_args(ap);
  if (st != cudaSuccess) return st;
  st = validate_decode_args(a);
  if (st != cudaSuccess) return st;
  if (!decode_fused_supported(ap, a)) return cudaErrorInvalidValue;
  if ((reinterpret_cast<uintptr_t>(ap.q_prepared) & 15u) != 0) {
    return cudaErrorInvalidValue;
  }
  BalancedParams p = balanced_params(a);
  p.raw_q = ap.q;
  p.raw_k = ap.k;
  p.raw_v = ap.v;
  p.q_norm_weight = ap.q_norm_weight;
  p.k_norm_weight = ap.k_norm_weight;
  p.cos = ap.cos;
  p.sin = ap.sin;
  p.token_position = ap.token_position;
  p.q_prepared = ap.q_prepared;
  p.raw_from_predecessor = ap.raw_from_predecessor ? 1 : 0;
  using T = DecodeTraits<256, 8, 2, 8>;
  const int64_t slots = int64_t(a.batch_count) * a.num_splits;
  const bool small = a.batch_count <= kSmallBalancedBatch;
  if (ap.norm_mode == B200KV_NORM_IEEE) {
    return small ? launch_balanced<T, kFusedIeee, kSmallBalancedBatch>(p, slots, stream)
                 : launch_balanced<T, kFusedIeee>(p, slots, stream);
  }
  return small ? launch_balanced<T, kFusedApprox, kSmallBalancedBatch>(p, slots, stream)
               : launch_balanced<T, kFusedApprox>(p, slots, stream);
}

int decode_balanced_num_splits(int batch_count, int sm_count) {
  const int ctas = std::max(sm_count, 1) * 2;
  return div_up(ctas, std::max(batch_count, 1)) + 1;
}

}  // namespace b200kv

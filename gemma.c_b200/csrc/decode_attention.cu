// Split-KV flash-decode over the paged KV cache, plus the combine.
//
// Replaces phase_decode_paged_grouped_split, phase_decode_global_q_head_direct
// and phase_decode_paged_reduce of the reference
// (src/gemma4_flash_attention_decode.cu:613-977). Same task meaning
// (batch row, split of split_size keys starting at first_key), same partial
// scratch layout, same edge behaviour (empty rows give zeros, over-provisioned
// splits leave the scratch untouched, unmapped pages contribute nothing).
//
// Design (B200): the reference makes one 512-thread CTA do G block-wide
// reductions per key. Here a CTA owns one (sequence, split) for ALL KV heads,
// because in the cache layout [page, offset, head, dim] the rows of all heads
// for consecutive tokens of a page are one contiguous byte range. A producer
// warp streams those ranges into a 3-stage shared-memory ring with
// bulk-async copies completing on mbarriers (64 KiB per stage: K and V for
// kStageTokens tokens); 16 consumer warps each own one KV head and four of a
// stage's tokens. A lane holds 8 of the 256 head dims, so one key's row is a
// single conflict-free 128-bit shared load per lane; the G*4 partial dot
// products of a warp are finished with one shuffle reduce-scatter (9
// shuffles for 8 scores) instead of a reduction per key. Softmax is fp32
// online in the exp2 domain; P*V reuses the same lane<->dim mapping.
#include "decode_common.cuh"
#include "kernels.cuh"

#include <cstdlib>

namespace b200kv {

namespace {

struct DecodeParams {
  __nv_bfloat16 *out;
  float *lse;
  const __nv_bfloat16 *q;
  const __nv_bfloat16 *cache_k;
  const __nv_bfloat16 *cache_v;
  Gemma4KvCacheConfig cfg;
  const int32_t *page_table;
  const int32_t *seq_lengths;
  int32_t layer;
  float scale_log2;  // softmax_scale * log2(e)
  int32_t split_size;
  int32_t num_splits;
  int32_t q_heads;
  float *partial_m;
  float *partial_l;
  float *partial_acc;
  int32_t *status;
};

template <class T>
__global__ __launch_bounds__(T::kThreads, T::kCtasPerSm) void decode_split_kernel(
    DecodeParams p) {
  constexpr int D = T::D;
  constexpr int HKV = T::HKV;
  constexpr int G = T::G;
  constexpr int ST = T::kStageTokens;
  constexpr int kConsumerWarps = T::kConsumerWarps;
  extern __shared__ __align__(128) uint8_t smem[];

  const int split = int(blockIdx.x);
  const int batch = int(blockIdx.y);
  const int warp = int(threadIdx.x) >> 5;
  const int lane = int(threadIdx.x) & 31;
  const Gemma4KvCacheConfig &cfg = p.cfg;

  // Everything this kernel reads may have been written by the launch before it
  // (the appended row, the prepared q, this step's lengths).
  pdl_wait_for_predecessor();
  pdl_release_successor();

  const int seq_len = __ldg(p.seq_lengths + batch);
  const LiveRange lr = live_range(cfg, seq_len, p.split_size);
  const bool write_direct = p.num_splits == 1;
  if (lr.key_count == 0 && write_direct) {
    // src/gemma4_flash_attention_decode.cu:735-745: no live key, zero rows.
    const int64_t row0 = int64_t(batch) * p.q_heads;
    for (int i = int(threadIdx.x); i < p.q_heads * D / 8; i += T::kThreads) {
      reinterpret_cast<uint4 *>(p.out + row0 * D)[i] = make_uint4(0, 0, 0, 0);
    }
    if (p.lse != nullptr && int(threadIdx.x) < p.q_heads) {
      p.lse[row0 + threadIdx.x] = -INFINITY;
    }
    return;
  }
  if (split >= lr.actual_splits) return;  // :746-748

  const int split_begin = lr.first_key + split * p.split_size;
  const int split_end = min(seq_len, split_begin + p.split_size);
  // Stage c holds positions [base_c, base_c + ST) ∩ [split_begin, split_end),
  // base_c = a0 + c * ST, so a token's slot in a stage is position % ST.
  const int a0 = (split_begin / ST) * ST;
  const int nchunks = div_up(split_end - a0, ST);

  const Ring<T> ring(smem);
  if (threadIdx.x == 0) ring.init_barriers();
  __syncthreads();

  if (warp == kConsumerWarps) {
    // ------------------------------ producer ------------------------------
    const uint64_t policy = l2_policy_evict_first();
    const KvSource src = {reinterpret_cast<const uint8_t *>(p.cache_k),
                          reinterpret_cast<const uint8_t *>(p.cache_v),
                          p.page_table, p.layer};
    bool ok = true;
    PageEntryCache page_cache;
    int issued = 0;  // chunks whose full barrier has been armed
    for (int c = 0; c < nchunks; ++c) {
      const int stage = c % kStages;
      const int fill = c / kStages;
      if (fill > 0) {
        ok = mbar_wait_bounded(ring.empty_bar(stage), uint32_t(fill - 1) & 1u);
        if (!ok) break;
      }
      const int base = a0 + c * ST;
      producer_fill_stage<T>(ring, src, cfg, batch, base, max(split_begin, base),
                             min(split_end, base + ST), stage, policy, lane,
                             &page_cache);
      issued = c + 1;
    }
    // Hold the CTA until every copy this warp issued has landed.
    for (int s = 0; s < kStages && s < issued; ++s) {
      const int fill = (issued - 1 - s) / kStages;  // last fill of stage s
      if (!mbar_wait_bounded(ring.full_bar(s), uint32_t(fill) & 1u)) ok = false;
    }
    if (!ok && lane == 0) set_status(p.status, B200KV_STATUS_WAIT_TIMEOUT);
    return;
  }

  // -------------------------------- consumers --------------------------------
  const int head = warp % HKV;
  const int sub = warp / HKV;
  WarpState<T> st;
  {
    uint4 raw[G];
    load_q_raw<T>(raw, p.q, int64_t(batch) * p.q_heads + head * G, lane);
    st.set_q(raw, p.scale_log2);
  }
  st.reset();

  bool ok = true;
  for (int c = 0; c < nchunks; ++c) {
    const int stage = c % kStages;
    const int fill = c / kStages;
    if (!mbar_wait_bounded(ring.full_bar(stage), uint32_t(fill) & 1u)) {
      ok = false;
      break;
    }
    consume_stage<T>(st, ring, stage, head, sub, lane);
    __syncwarp();
    if (lane == 0) mbar_arrive(ring.empty_bar(stage));
  }
  if (!ok) {
    if (lane == 0) set_status(p.status, B200KV_STATUS_WAIT_TIMEOUT);
    return;  // every other wait in this CTA is bounded as well
  }

  float l[G];
  st.denominators(l, lane);
  float (&m)[G] = st.m;
  float (&acc)[G][8] = st.acc;

  // Merge the kWarpsPerHead warps of one head through the (now idle) ring.
  if constexpr (T::kWarpsPerHead > 1) {
    constexpr int kFields = 2 * G + 8 * G;  // m, l, acc per lane
    float *xchg = reinterpret_cast<float *>(smem);
    named_barrier_sync(1, kConsumerWarps * kWarpSize);
    if (sub > 0) {
      float *dst = xchg + (size_t(warp) * kFields) * kWarpSize + lane;
#pragma unroll
      for (int g = 0; g < G; ++g) {
        dst[(g)*kWarpSize] = m[g];
        dst[(G + g) * kWarpSize] = l[g];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          dst[(2 * G + g * 8 + i) * kWarpSize] = acc[g][i];
        }
      }
    }
    named_barrier_sync(1, kConsumerWarps * kWarpSize);
    if (sub > 0) return;
    for (int other = 1; other < T::kWarpsPerHead; ++other) {
      const float *src =
          xchg + (size_t(other * HKV + head) * kFields) * kWarpSize + lane;
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const float om = src[(g)*kWarpSize];
        const float ol = src[(G + g) * kWarpSize];
        if (om == -INFINITY) continue;  // that warp saw no key
        const float nm = fmaxf(m[g], om);
        const float a = ex2_approx(m[g] - nm);  // 0 when m[g] is -inf
        const float b = ex2_approx(om - nm);
        l[g] = l[g] * a + ol * b;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          acc[g][i] = acc[g][i] * a + src[(2 * G + g * 8 + i) * kWarpSize] * b;
        }
        m[g] = nm;
      }
    }
  }

#pragma unroll
  for (int g = 0; g < G; ++g) {
    const int64_t row = int64_t(batch) * p.q_heads + head * G + g;
    if (write_direct) {
      // :849-863 -- a single split writes the bf16 row itself.
      write_output_row<T>(p.out, p.lse, row, acc[g], m[g], l[g], lane);
    } else {
      // :865-877 -- partials, stride num_splits per row. m is kept in the
      // exp2 domain (scaled score * log2 e); the combine below knows.
      write_partial_row<T>(p.partial_m, p.partial_l, p.partial_acc,
                           row * p.num_splits + split, acc[g], m[g], l[g], lane);
    }
  }
}

// One CTA per (batch, q_head) row and dim slice: combine of that row's live
// splits.
template <int D, int kSlices, int kThreads>
__global__ __launch_bounds__(kThreads) void decode_combine_kernel(
    DecodeParams p) {
  __shared__ float s_w[kCombineChunk];
  __shared__ float s_red[kThreads / 32];
  __shared__ float4 s_val[kThreads];
  const int row = int(blockIdx.x);
  const int slice = int(blockIdx.y);
  const int batch = row / p.q_heads;

  pdl_wait_for_predecessor();
  pdl_release_successor();

  // The live split count is recomputed from the lengths so that slots of
  // over-provisioned splits, which nobody wrote, are never read (:903-916).
  const int seq_len = __ldg(p.seq_lengths + batch);
  const LiveRange lr = live_range(p.cfg, seq_len, p.split_size);
  const int n = min(lr.actual_splits, p.num_splits);
  __nv_bfloat16 *out_row = p.out + int64_t(row) * D;
  float *lse_row = p.lse != nullptr ? p.lse + row : nullptr;
  if (n == 0) {
    combine_empty_row<D, kSlices>(out_row, lse_row, slice);
    return;
  }
  combine_row<D, kSlices, kThreads>(out_row, lse_row, p.partial_m, p.partial_l,
                          p.partial_acc, int64_t(row) * p.num_splits, 1, n, slice,
                          s_w, s_red, s_val);
}

template <class T>
cudaError_t launch_split(const DecodeParams &p, int batch_count,
                         cudaStream_t stream) {
  static_assert(T::kRingBytes <= 227 * 1024, "ring must fit one SM");
  // Per-device opt-in for the large dynamic shared-memory carve-out; the
  // attribute is sticky, setting it again is cheap and thread-safe.
  cudaError_t st = cudaFuncSetAttribute(
      decode_split_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
      T::kRingBytes);
  if (st != cudaSuccess) return st;
  const dim3 grid(p.num_splits, batch_count);
  return launch_pdl(decode_split_kernel<T>, grid, dim3(T::kThreads),
                    T::kRingBytes, stream, p);
}

}  // namespace

int decode_stage_tokens(int kv_heads) {
  if (kv_heads <= 0 || 16 % kv_heads != 0) return kTokPerWarp;
  return (16 / kv_heads) * kTokPerWarp;
}

namespace {
// Tuning hook: B200KV_DECODE_CW=8|16 forces the consumer-warp variant.
int forced_consumer_warps() {
  const char *v = std::getenv("B200KV_DECODE_CW");
  return v == nullptr ? 0 : std::atoi(v);
}
}  // namespace

cudaError_t validate_decode_args(const DecodeArgs &a) {
  const Gemma4KvCacheConfig &c = a.cfg;
  // Validation mirrors gemma4_fa_valid_cache_config and the launcher checks
  // (src/gemma4_flash_attention_decode.cu:377-392,1129-1134).
  if (a.out == nullptr || a.q == nullptr || a.cache_k == nullptr ||
      a.cache_v == nullptr || a.page_table == nullptr ||
      a.seq_lengths == nullptr || a.batch_count <= 0 || a.layer < 0 ||
      a.layer >= c.num_layers || c.num_pages <= 0 || c.page_size <= 0 ||
      c.max_pages_per_seq <= 0 || c.batch_size <= 0 || c.window_size < 0 ||
      a.split_size < 0 || a.num_splits <= 0 || !(a.softmax_scale > 0.0f) ||
      a.q_heads <= 0 || c.num_heads <= 0 || a.q_heads % c.num_heads != 0) {
    return cudaErrorInvalidValue;
  }
  if (c.window_size > 0 &&
      int64_t(c.max_pages_per_seq) * c.page_size < c.window_size) {
    return cudaErrorInvalidValue;  // ring smaller than the window (:389-391)
  }
  const bool balanced = a.split_size == 0;
  if ((a.num_splits > 1 || balanced) &&
      (a.partial_m == nullptr || a.partial_l == nullptr ||
       a.partial_acc == nullptr)) {
    return cudaErrorInvalidValue;
  }
  if (a.batch_count > 65535) return cudaErrorInvalidValue;  // grid.y limit
  const uintptr_t align = reinterpret_cast<uintptr_t>(a.cache_k) |
                          reinterpret_cast<uintptr_t>(a.cache_v) |
                          reinterpret_cast<uintptr_t>(a.q) |
                          reinterpret_cast<uintptr_t>(a.out) |
                          reinterpret_cast<uintptr_t>(a.partial_acc);
  if ((align & 15u) != 0) return cudaErrorInvalidValue;
  return cudaSuccess;
}

cudaError_t decode_attention_bf16(const DecodeArgs &a, cudaStream_t stream) {
  const Gemma4KvCacheConfig &c = a.cfg;
  const cudaError_t valid = validate_decode_args(a);
  if (valid != cudaSuccess) return valid;
  const bool balanced = a.split_size == 0;
  if (balanced) return decode_attention_balanced_bf16(a, stream);

  DecodeParams p;
  p.out = a.out;
  p.lse = a.lse;
  p.q = a.q;
  p.cache_k = a.cache_k;
  p.cache_v = a.cache_v;
  p.cfg = c;
  p.page_table = a.page_table;
  p.seq_lengths = a.seq_lengths;
  p.layer = a.layer;
  p.scale_log2 = a.softmax_scale * 1.4426950408889634f;
  p.split_size = a.split_size;
  p.num_splits = a.num_splits;
  p.q_heads = a.q_heads;
  p.partial_m = a.partial_m;
  p.partial_l = a.partial_l;
  p.partial_acc = a.partial_acc;
  p.status = a.status;

  const int G = a.q_heads / c.num_heads;
  cudaError_t st = cudaErrorInvalidValue;  // unknown geometry (:1156)
  if (c.head_dim == 256 && G == 2) {
    const int forced = forced_consumer_warps();
    switch (c.num_heads) {
      case 8:
        if (forced == 16) {
          st = launch_split<DecodeTraits<256, 8, 2, 16>>(p, a.batch_count, stream);
        } else {
          st = launch_split<DecodeTraits<256, 8, 2, 8>>(p, a.batch_count, stream);
        }
        break;
      case 4: st = launch_split<DecodeTraits<256, 4, 2, 16>>(p, a.batch_count, stream); break;
      case 2: st = launch_split<DecodeTraits<256, 2, 2, 16>>(p, a.batch_count, stream); break;
      case 1: st = launch_split<DecodeTraits<256, 1, 2, 16>>(p, a.batch_count, stream); break;
      default: break;
    }
  }
  if (st != cudaSuccess) return st;
  if (a.num_splits > 1) {
    const int64_t rows = int64_t(a.batch_count) * a.q_heads;
    st = B200KV_LAUNCH_COMBINE(decode_combine_kernel, rows, stream, p);
  }
  return st;
}

}  // namespace b200kv

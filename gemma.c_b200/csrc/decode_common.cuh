// Building blocks shared by the two split-KV decode kernels (fixed splits in
// decode_attention.cu, evenly balanced key ranges in decode_balanced.cu): the
// shared-memory ring a producer warp fills with bulk-async copies, and the
// per-warp online-softmax step over one ring stage.
#pragma once

#include "common.cuh"

namespace b200kv {

constexpr int kTokPerWarp = 4;
constexpr int kStages = 3;

// CW consumer warps per CTA: 16 gives one CTA per SM with 64 KiB stages, 8
// gives two CTAs per SM with 32 KiB stages (same bytes in flight per SM, but
// one CTA's pipeline fill and epilogue overlap the other's streaming).
template <int D_, int HKV_, int G_, int CW_>
struct DecodeTraits {
  static constexpr int D = D_;
  static constexpr int HKV = HKV_;
  static constexpr int G = G_;
  static constexpr int kConsumerWarps = CW_;
  static constexpr int kCtasPerSm = CW_ <= 8 ? 2 : 1;
  static constexpr int kWarpsPerHead = kConsumerWarps / HKV;
  static constexpr int kStageTokens = kWarpsPerHead * kTokPerWarp;
  static constexpr bool kFp8 = false;
  static constexpr int kElemBytes = 2;
  static constexpr int kRowBytes = HKV * D * 2;  // one token, all heads
  static constexpr int kStageTensorBytes = kStageTokens * kRowBytes;
  static constexpr int kStageBytes = 2 * kStageTensorBytes;  // K then V
  static constexpr int kThreads = (kConsumerWarps + 1) * kWarpSize;
  static constexpr int kMetaBytes = 256;  // barriers + per-stage token masks
  static constexpr int kRingBytes = kStages * kStageBytes + kMetaBytes;
  static_assert(kConsumerWarps % HKV == 0, "warps must tile the KV heads");
  static_assert(D == 256, "a lane owns 8 dims = one 128-bit load per row");
  static_assert(G == 2, "score reduce-scatter is written for G * 4 == 8");
  static_assert(kStageTokens <= 64, "token mask is 64 bits");
};

struct LiveRange {
  int first_key;
  int key_count;
  int actual_splits;
};

__device__ __forceinline__ LiveRange live_range(const Gemma4KvCacheConfig &c,
                                                int seq_len, int split_size) {
  // src/gemma4_flash_attention_decode.cu:728-733
  LiveRange r;
  r.first_key = c.window_size > 0 ? max(0, seq_len - c.window_size) : 0;
  r.key_count = max(0, seq_len - r.first_key);
  r.actual_splits = div_up(r.key_count, split_size);
  return r;
}

// Sum 8 per-lane partials across the warp so that lane l ends with the
// complete value of index (l >> 2) & 7 (lanes that share l >> 2 hold copies).
__device__ __forceinline__ float reduce_scatter8(float (&v)[8], int lane) {
  const bool up16 = (lane & 16) != 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float send = up16 ? v[i] : v[i + 4];
    const float keep = up16 ? v[i + 4] : v[i];
    v[i] = keep + __shfl_xor_sync(0xffffffffu, send, 16);
  }
  const bool up8 = (lane & 8) != 0;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const float send = up8 ? v[i] : v[i + 2];
    const float keep = up8 ? v[i + 2] : v[i];
    v[i] = keep + __shfl_xor_sync(0xffffffffu, send, 8);
  }
  const bool up4 = (lane & 4) != 0;
  {
    const float send = up4 ? v[0] : v[1];
    const float keep = up4 ? v[1] : v[0];
    v[0] = keep + __shfl_xor_sync(0xffffffffu, send, 4);
  }
  float r = v[0];
  r += __shfl_xor_sync(0xffffffffu, r, 2);
  r += __shfl_xor_sync(0xffffffffu, r, 1);
  return r;
}

// The ring in dynamic shared memory: kStages stages of (K rows, V rows), then
// full[kStages] and empty[kStages] mbarriers and one 64-bit token mask per
// stage (bit i set = slot i of the stage holds a live, mapped token).
template <class T>
struct Ring {
  uint8_t *smem;
  uint32_t base;
  __device__ explicit Ring(uint8_t *p) : smem(p), base(smem_u32(p)) {}
  __device__ uint32_t full_bar(int s) const {
    return base + kStages * T::kStageBytes + 8u * uint32_t(s);
  }
  __device__ uint32_t empty_bar(int s) const {
    return base + kStages * T::kStageBytes + 8u * uint32_t(kStages + s);
  }
  __device__ unsigned long long *masks() const {
    return reinterpret_cast<unsigned long long *>(
        smem + kStages * T::kStageBytes + 16 * kStages);
  }
  __device__ uint32_t k_stage(int s) const {
    return base + uint32_t(s) * T::kStageBytes;
  }
  __device__ void init_barriers() const {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), T::kConsumerWarps);
    }
    mbar_fence_init();
  }
};

struct KvSource {
  const uint8_t *cache_k;  // byte pointers: elements are bf16 or e4m3
  const uint8_t *cache_v;
  const int32_t *page_table;
  int32_t layer;
};

// Producer warp: fill one stage with the keys [c0, c1) of sequence `batch`
// (all inside [base, base + kStageTokens)); a token sits in slot position -
// base. One lane per page segment resolves the page table and issues the two
// bulk copies; lane 0 publishes the token mask and arms the full barrier.
// The page-table entry a lane resolved last. A stage is shorter than a page,
// so consecutive stages mostly need the same entry; without this every stage
// starts with a dependent global load (about a microsecond on a miss), which
// is what bounded a CTA that streams only a few stages.
struct PageEntryCache {
  int batch = -1;
  int logical_page = -1;
  int physical = -1;
};

template <class T>
__device__ __forceinline__ void producer_fill_stage(
    const Ring<T> &ring, const KvSource &src, const Gemma4KvCacheConfig &cfg,
    int batch, int base, int c0, int c1, int stage, uint64_t policy, int lane,
    PageEntryCache *cache = nullptr) {
  const int ps = cfg.page_size;
  auto resolve = [&](int lp) {
    if (cache != nullptr && cache->batch == batch && cache->logical_page == lp) {
      return cache->physical;
    }
    const int slot = lp % cfg.max_pages_per_seq;
    const int phys =
        __ldg(src.page_table + int64_t(batch) * cfg.max_pages_per_seq + slot);
    if (cache != nullptr) {
      cache->batch = batch;
      cache->logical_page = lp;
      cache->physical = phys;
    }
    return phys;
  };
  const uint32_t k_dst = ring.k_stage(stage);
  const uint32_t v_dst = k_dst + T::kStageTensorBytes;

  if constexpr (T::kRowBytes >= 4096 && T::kStageTokens <= kWarpSize) {
    // Wide rows (all 8 KV heads: 4 KiB per token and tensor): one lane per
    // token, one copy per token and tensor. A CTA that streams only a few
    // stages is bound by how fast its copies come in, and that grows with the
    // number of copies in flight, not with their size.
    const int pos = c0 + lane;
    const bool mine = pos < c1;
    const int lp = mine ? pos / ps : 0;
    const int phys = mine ? resolve(lp) : -1;
    const bool valid = mine && phys >= 0 && phys < cfg.num_pages;
    const uint32_t live = __ballot_sync(0xffffffffu, valid);
    if (lane == 0) {
      ring.masks()[stage] = static_cast<unsigned long long>(live) << (c0 - base);
      if (live != 0u) {
        mbar_arrive_expect_tx(ring.full_bar(stage),
                              2u * uint32_t(__popc(live)) * T::kRowBytes);
      } else {
        mbar_arrive(ring.full_bar(stage));
      }
    }
    __syncwarp();
    if (valid) {
      const int64_t off = cache_offset(cfg, src.layer, phys, pos - lp * ps, 0, 0);
      const uint32_t dst_off = uint32_t(pos - base) * T::kRowBytes;
      bulk_load_hint(k_dst + dst_off, src.cache_k + off * T::kElemBytes,
                     T::kRowBytes, ring.full_bar(stage), policy);
      bulk_load_hint(v_dst + dst_off, src.cache_v + off * T::kElemBytes,
                     T::kRowBytes, ring.full_bar(stage), policy);
    }
    return;
  }

  const int first_page = c0 / ps;
  const int nseg = (c1 - 1) / ps - first_page + 1;

  unsigned long long my_mask = 0;
  uint32_t my_bytes = 0;
  for (int seg0 = 0; seg0 < nseg; seg0 += kWarpSize) {
    const int seg = seg0 + lane;
    if (seg < nseg) {
      const int lp = first_page + seg;
      const int s0 = max(c0, lp * ps);
      const int s1 = min(c1, (lp + 1) * ps);
      const int phys = resolve(lp);
      if (phys >= 0 && phys < cfg.num_pages) {
        const int n = s1 - s0;
        my_bytes += uint32_t(n) * T::kRowBytes;
        my_mask |= ((n >= 64 ? ~0ull : ((1ull << n) - 1ull)) << (s0 - base));
      }
    }
  }
  const uint32_t bytes = __reduce_add_sync(0xffffffffu, my_bytes);
  const uint32_t mask_lo = __reduce_or_sync(0xffffffffu, uint32_t(my_mask));
  const uint32_t mask_hi =
      __reduce_or_sync(0xffffffffu, uint32_t(my_mask >> 32));
  if (lane == 0) {
    ring.masks()[stage] =
        (static_cast<unsigned long long>(mask_hi) << 32) | mask_lo;
    if (bytes > 0) {
      mbar_arrive_expect_tx(ring.full_bar(stage), 2u * bytes);
    } else {
      mbar_arrive(ring.full_bar(stage));
    }
  }
  __syncwarp();
  for (int seg0 = 0; seg0 < nseg; seg0 += kWarpSize) {
    const int seg = seg0 + lane;
    if (seg < nseg) {
      const int lp = first_page + seg;
      const int s0 = max(c0, lp * ps);
      const int s1 = min(c1, (lp + 1) * ps);
      const int phys = resolve(lp);
      if (phys >= 0 && phys < cfg.num_pages) {
        const int64_t off =
            cache_offset(cfg, src.layer, phys, s0 - lp * ps, 0, 0);
        const uint32_t dst_off = uint32_t(s0 - base) * T::kRowBytes;
        const uint32_t nbytes = uint32_t(s1 - s0) * T::kRowBytes;
        bulk_load_hint(k_dst + dst_off, src.cache_k + off * T::kElemBytes,
                       nbytes, ring.full_bar(stage), policy);
        bulk_load_hint(v_dst + dst_off, src.cache_v + off * T::kElemBytes,
                       nbytes, ring.full_bar(stage), policy);
      }
    }
  }
}

// Running state of one consumer warp: its KV head's two query heads, 8 of the
// 256 dims per lane.
template <class T>
struct WarpState {
  float qf[T::G][8];  // q * softmax_scale * log2(e)
  float acc[T::G][8];
  float m[T::G];      // running maxima, exp2 domain
  float l_lane;       // running sum of this lane's own (g, t) weights

  __device__ __forceinline__ void reset() {
#pragma unroll
    for (int g = 0; g < T::G; ++g) {
      m[g] = -INFINITY;
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[g][i] = 0.0f;
    }
    l_lane = 0.0f;
  }

  __device__ __forceinline__ void set_q(const uint4 (&raw)[T::G],
                                        float scale_log2) {
#pragma unroll
    for (int g = 0; g < T::G; ++g) {
      const uint32_t w[4] = {raw[g].x, raw[g].y, raw[g].z, raw[g].w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        qf[g][2 * i] = bf16_lo(w[i]) * scale_log2;
        qf[g][2 * i + 1] = bf16_hi(w[i]) * scale_log2;
      }
    }
  }

  // Per-head denominators from the per-lane sums: add the four token lanes
  // (copies in lanes that share lane >> 2 are not added), then fetch the
  // other head's value.
  __device__ __forceinline__ void denominators(float (&l)[T::G], int lane) const {
    const int my_g = lane >> 4;
    float l_mine = l_lane + __shfl_xor_sync(0xffffffffu, l_lane, 8);
    l_mine += __shfl_xor_sync(0xffffffffu, l_mine, 4);
    const float l_other = __shfl_xor_sync(0xffffffffu, l_mine, 16);
    l[0] = my_g == 0 ? l_mine : l_other;
    l[1] = my_g == 0 ? l_other : l_mine;
  }
};

template <class T>
__device__ __forceinline__ void load_q_raw(uint4 (&raw)[T::G],
                                           const __nv_bfloat16 *q,
                                           int64_t first_row, int lane) {
#pragma unroll
  for (int g = 0; g < T::G; ++g) {
    raw[g] = __ldg(reinterpret_cast<const uint4 *>(q + (first_row + g) * T::D) +
                   lane);
  }
}

// One stage of the ring for one consumer warp (KV head `head`, token group
// `sub`): scores for its four tokens, online-softmax update, P*V.
template <class T>
__device__ __forceinline__ void consume_stage(WarpState<T> &st,
                                              const Ring<T> &ring, int stage,
                                              int head, int sub, int lane) {
  constexpr int G = T::G;
  const int my_g = lane >> 4;        // which of the G q heads this lane scores
  const int my_t = (lane >> 2) & 3;  // which of the warp's 4 tokens
  const unsigned long long mask = ring.masks()[stage];
  const uint32_t mine = uint32_t(mask >> (sub * kTokPerWarp)) & 0xfu;
  if (mine == 0u) return;
  const uint32_t k_base = ring.k_stage(stage) +
                          uint32_t(sub * kTokPerWarp) * T::kRowBytes +
                          uint32_t(head * T::D + lane * 8) * 2u;
  const uint32_t v_base = k_base + T::kStageTensorBytes;

  float s[G * kTokPerWarp];
#pragma unroll
  for (int i = 0; i < G * kTokPerWarp; ++i) s[i] = 0.0f;
#pragma unroll
  for (int t = 0; t < kTokPerWarp; ++t) {
    if ((mine >> t) & 1u) {
      const uint4 kk = lds128(k_base + uint32_t(t) * T::kRowBytes);
      const uint32_t w[4] = {kk.x, kk.y, kk.z, kk.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float lo = bf16_lo(w[i]);
        const float hi = bf16_hi(w[i]);
#pragma unroll
        for (int g = 0; g < G; ++g) {
          s[g * kTokPerWarp + t] =
              fmaf(st.qf[g][2 * i], lo, s[g * kTokPerWarp + t]);
          s[g * kTokPerWarp + t] =
              fmaf(st.qf[g][2 * i + 1], hi, s[g * kTokPerWarp + t]);
        }
      }
    }
  }
  float my_s = reduce_scatter8(s, lane);
  if (((mine >> my_t) & 1u) == 0u) my_s = -INFINITY;

  float tile_max = fmaxf(my_s, __shfl_xor_sync(0xffffffffu, my_s, 8));
  tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, 4));
  const float other_max = __shfl_xor_sync(0xffffffffu, tile_max, 16);
  const float new_m0 = fmaxf(st.m[0], my_g == 0 ? tile_max : other_max);
  const float new_m1 = fmaxf(st.m[1], my_g == 0 ? other_max : tile_max);
  if (new_m0 > st.m[0] || new_m1 > st.m[1]) {
    const float corr0 = ex2_approx(st.m[0] - new_m0);
    const float corr1 = ex2_approx(st.m[1] - new_m1);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      st.acc[0][i] *= corr0;
      st.acc[1][i] *= corr1;
    }
    st.l_lane *= (my_g == 0 ? corr0 : corr1);
    st.m[0] = new_m0;
    st.m[1] = new_m1;
  }
  const float pr = ex2_approx(my_s - (my_g == 0 ? st.m[0] : st.m[1]));
  st.l_lane += pr;

#pragma unroll
  for (int t = 0; t < kTokPerWarp; ++t) {
    if ((mine >> t) & 1u) {
      const float p0 = __shfl_sync(0xffffffffu, pr, t << 2);
      const float p1 = __shfl_sync(0xffffffffu, pr, 16 | (t << 2));
      const uint4 vv = lds128(v_base + uint32_t(t) * T::kRowBytes);
      const uint32_t w[4] = {vv.x, vv.y, vv.z, vv.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float lo = bf16_lo(w[i]);
        const float hi = bf16_hi(w[i]);
        st.acc[0][2 * i] = fmaf(p0, lo, st.acc[0][2 * i]);
        st.acc[0][2 * i + 1] = fmaf(p0, hi, st.acc[0][2 * i + 1]);
        st.acc[1][2 * i] = fmaf(p1, lo, st.acc[1][2 * i]);
        st.acc[1][2 * i + 1] = fmaf(p1, hi, st.acc[1][2 * i + 1]);
      }
    }
  }
}

// Final bf16 row (and LSE) of one query head from a complete (m, l, acc).
template <class T>
__device__ __forceinline__ void write_output_row(__nv_bfloat16 *out, float *lse,
                                                 int64_t row,
                                                 const float (&acc)[8], float m,
                                                 float l, int lane) {
  const float inv = l > 0.0f ? 1.0f / l : 0.0f;
  uint32_t packed[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __nv_bfloat162 h2 =
        __floats2bfloat162_rn(acc[2 * i] * inv, acc[2 * i + 1] * inv);
    packed[i] = *reinterpret_cast<const uint32_t *>(&h2);
  }
  reinterpret_cast<uint4 *>(out + row * T::D)[lane] =
      make_uint4(packed[0], packed[1], packed[2], packed[3]);
  if (lse != nullptr && lane == 0) {
    lse[row] = l > 0.0f ? (m + lg2_approx(l)) * 0.6931471805599453f : -INFINITY;
  }
}

// Unnormalised partial of one query head into scratch slot `slot`.
template <class T>
__device__ __forceinline__ void write_partial_row(float *partial_m,
                                                  float *partial_l,
                                                  float *partial_acc,
                                                  int64_t slot,
                                                  const float (&acc)[8], float m,
                                                  float l, int lane) {
  if (lane == 0) {
    partial_m[slot] = m;
    partial_l[slot] = l;
  }
  float4 *dst = reinterpret_cast<float4 *>(partial_acc + slot * T::D) + lane * 2;
  dst[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
  dst[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
}

// LSE-style combine of n partials of one (sequence, query head) row; partial i
// lives at scratch index first + i * stride
// (src/gemma4_flash_attention_decode.cu:881-977 does the same sums serially).
// A CTA of kThreads threads handles slice `slice` of kSlices equal slices of
// the row's D dims: the threads form kGroups groups of kCols (one float4
// column each); a group owns every kGroups-th partial and keeps four loads in
// flight, so 4 * kGroups partials are read per round trip. Three shapes are
// used (combine_shape): one slice of 256 threads for many rows with few
// partials each; with few rows and many partials (small batches) the combine
// is a chain of load round trips on a handful of SMs, and four slices put four
// times the SMs on it; in between, four slices of 128 threads: the combine's
// CTAs are resident, waiting for the attention kernel to finish, while the next
// layer-step's attention CTAs look for room to start, and half the threads
// leave room for one of those per SM. (A second one does not fit beside a
// combine CTA: two attention CTAs put five 96-register warps on two of the
// SM's four register-file partitions, 15 360 of 16 384 registers.)
constexpr int kCombineChunk = 512;  // partials whose weights fit the table

template <int D, int kSlices, int kThreads>
struct CombineShape {
  static constexpr int kCols = D / 4 / kSlices;
  static constexpr int kGroups = kThreads / kCols;
  static constexpr int kWarps = kThreads / 32;
  static_assert(kCols * kSlices * 4 == D && kCols * kGroups == kThreads,
                "thread mapping");
};

template <int D, int kSlices, int kThreads>
__device__ __forceinline__ void combine_row(__nv_bfloat16 *out_row, float *lse_row,
                                            const float *partial_m,
                                            const float *partial_l,
                                            const float *partial_acc,
                                            int64_t first, int64_t stride, int n,
                                            int slice, float *s_w, float *s_red,
                                            float4 *s_val) {
  using Shape = CombineShape<D, kSlices, kThreads>;
  constexpr int kWarps = Shape::kWarps;
  constexpr int kCols = Shape::kCols;
  constexpr int kGroups = Shape::kGroups;
  const int tid = int(threadIdx.x);
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int group = tid / kCols;
  const int col = slice * kCols + tid % kCols;
  const float *pm = partial_m + first;
  const float *pl = partial_l + first;
  const float4 *acc =
      reinterpret_cast<const float4 *>(partial_acc + first * D) + col;
  const size_t acc_stride = size_t(stride) * (D / 4);

  // The first round of accumulator loads does not depend on the weights: it
  // is issued before the maxima are known and lands while they are reduced.
  float4 pre[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int s = group + j * kGroups;
    pre[j] = s < n ? __ldg(acc + size_t(s) * acc_stride)
                   : make_float4(0.f, 0.f, 0.f, 0.f);
  }

  // Pass 1: the row maximum over the partials.
  float M = -INFINITY;
  for (int s = tid; s < n; s += kThreads) {
    M = fmaxf(M, __ldg(pm + s * stride));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
  if (lane == 0) s_red[warp] = M;
  __syncthreads();
  M = s_red[0];
#pragma unroll
  for (int w = 1; w < kWarps; ++w) M = fmaxf(M, s_red[w]);
  __syncthreads();

  // Pass 2: weights 2^(m_i - M) (0 for partials without mass, :953-956), the
  // denominator, and the weighted sum of the accumulators. A weight of 0 must
  // drop its partial whatever the scratch holds.
  float L = 0.0f;
  float4 value = make_float4(0.f, 0.f, 0.f, 0.f);
  auto add = [&value](const float4 &a, float w) {
    if (w > 0.0f) {
      value.x = fmaf(a.x, w, value.x);
      value.y = fmaf(a.y, w, value.y);
      value.z = fmaf(a.z, w, value.z);
      value.w = fmaf(a.w, w, value.w);
    }
  };
  for (int base = 0; base < n; base += kCombineChunk) {
    const int cnt = min(kCombineChunk, n - base);
    for (int s = tid; s < cnt; s += kThreads) {
      const float sl = __ldg(pl + (base + s) * stride);
      const float w =
          sl > 0.0f ? ex2_approx(__ldg(pm + (base + s) * stride) - M) : 0.0f;
      s_w[s] = w;
      L = fmaf(sl, w, L);
    }
    __syncthreads();
    int s = group;
    if (base == 0) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (s + j * kGroups < cnt) add(pre[j], s_w[s + j * kGroups]);
      }
      s += 4 * kGroups;
    }
    for (; s + 3 * kGroups < cnt; s += 4 * kGroups) {
      const float4 a0 = __ldg(acc + size_t(base + s) * acc_stride);
      const float4 a1 = __ldg(acc + size_t(base + s + kGroups) * acc_stride);
      const float4 a2 = __ldg(acc + size_t(base + s + 2 * kGroups) * acc_stride);
      const float4 a3 = __ldg(acc + size_t(base + s + 3 * kGroups) * acc_stride);
      add(a0, s_w[s]);
      add(a1, s_w[s + kGroups]);
      add(a2, s_w[s + 2 * kGroups]);
      add(a3, s_w[s + 3 * kGroups]);
    }
    for (; s < cnt; s += kGroups) {
      const float w = s_w[s];
      if (w > 0.0f) add(__ldg(acc + size_t(base + s) * acc_stride), w);
    }
    __syncthreads();
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) L += __shfl_xor_sync(0xffffffffu, L, o);
  if (lane == 0) s_red[warp] = L;
  s_val[tid] = value;  // [group][column of the slice]
  __syncthreads();
  if (group == 0) {
    L = 0.0f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) L += s_red[w];
#pragma unroll 4
    for (int g = 1; g < kGroups; ++g) {
      const float4 o = s_val[g * kCols + tid];
      value.x += o.x;
      value.y += o.y;
      value.z += o.z;
      value.w += o.w;
    }
    const float inv = L > 0.0f ? 1.0f / L : 0.0f;
    const __nv_bfloat162 lo = __floats2bfloat162_rn(value.x * inv, value.y * inv);
    const __nv_bfloat162 hi = __floats2bfloat162_rn(value.z * inv, value.w * inv);
    reinterpret_cast<uint2 *>(out_row)[col] =
        make_uint2(*reinterpret_cast<const uint32_t *>(&lo),
                   *reinterpret_cast<const uint32_t *>(&hi));
    if (lse_row != nullptr && tid == 0 && slice == 0) {
      *lse_row = L > 0.0f ? (M + lg2_approx(L)) * 0.6931471805599453f : -INFINITY;
    }
  }
  __syncthreads();  // the shared arrays are free for the caller's next row
}

// Shape of the combine launch for `rows` output rows: 0 = four slices of 256
// threads, 1 = four slices of 128 threads, 2 = one slice of 256 threads.
inline int combine_shape(int64_t rows) {
  return rows <= 32 ? 0 : (rows <= 512 ? 1 : 2);
}

// Launches kernel<D, slices, threads> for the shape of `rows`.
#define B200KV_LAUNCH_COMBINE(kernel, rows, stream, ...)                       \
  (combine_shape(rows) == 0                                                    \
       ? launch_pdl(kernel<256, 4, 256>, dim3(unsigned(rows), 4), dim3(256), 0,  \
                    stream, __VA_ARGS__)                                       \
       : combine_shape(rows) == 1                                              \
             ? launch_pdl(kernel<256, 4, 128>, dim3(unsigned(rows), 4),          \
                          dim3(128), 0, stream, __VA_ARGS__)                   \
             : launch_pdl(kernel<256, 1, 256>, dim3(unsigned(rows)), dim3(256),  \
                          0, stream, __VA_ARGS__))

// Row of zeros and LSE = -inf for a (sequence, head) without live keys
// (src/gemma4_flash_attention_decode.cu:920-926).
template <int D, int kSlices>
__device__ __forceinline__ void combine_empty_row(__nv_bfloat16 *out_row,
                                                  float *lse_row, int slice) {
  constexpr int kCols = D / 4 / kSlices;  // <= 64: every shape has the threads
  const int tid = int(threadIdx.x);
  if (tid < kCols) {
    reinterpret_cast<uint2 *>(out_row)[slice * kCols + tid] = make_uint2(0, 0);
  }
  if (lse_row != nullptr && tid == 0 && slice == 0) *lse_row = -INFINITY;
}

}  // namespace b200kv

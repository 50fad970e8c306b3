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
#include "common.cuh"
#include "kernels.cuh"

namespace b200kv {

namespace {

constexpr int kConsumerWarps = 16;
constexpr int kTokPerWarp = 4;
constexpr int kStages = 3;

template <int D_, int HKV_, int G_>
struct DecodeTraits {
  static constexpr int D = D_;
  static constexpr int HKV = HKV_;
  static constexpr int G = G_;
  static constexpr int kWarpsPerHead = kConsumerWarps / HKV;
  static constexpr int kStageTokens = kWarpsPerHead * kTokPerWarp;
  static constexpr int kRowBytes = HKV * D * 2;  // one token, all heads
  static constexpr int kStageTensorBytes = kStageTokens * kRowBytes;
  static constexpr int kStageBytes = 2 * kStageTensorBytes;  // K then V
  static constexpr int kThreads = (kConsumerWarps + 1) * kWarpSize;
  static constexpr int kMetaBytes = 256;  // barriers + per-stage token masks
  static constexpr int kSmemBytes = kStages * kStageBytes + kMetaBytes;
  static_assert(kConsumerWarps % HKV == 0, "warps must tile the KV heads");
  static_assert(D == 256, "a lane owns 8 dims = one 128-bit load per row");
  static_assert(G == 2, "score reduce-scatter is written for G * 4 == 8");
  static_assert(kStageTokens <= 64, "token mask is 64 bits");
};

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

template <class T>
__global__ __launch_bounds__(T::kThreads, 1) void decode_split_kernel(
    DecodeParams p) {
  constexpr int D = T::D;
  constexpr int HKV = T::HKV;
  constexpr int G = T::G;
  constexpr int ST = T::kStageTokens;
  extern __shared__ __align__(128) uint8_t smem[];

  const int split = int(blockIdx.x);
  const int batch = int(blockIdx.y);
  const int warp = int(threadIdx.x) >> 5;
  const int lane = int(threadIdx.x) & 31;
  const Gemma4KvCacheConfig &cfg = p.cfg;

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

  const uint32_t smem_base = smem_u32(smem);
  const uint32_t meta = smem_base + kStages * T::kStageBytes;
  // meta: full[kStages] u64, empty[kStages] u64, then masks (u64 per stage)
  auto full_bar = [&](int s) { return meta + 8u * uint32_t(s); };
  auto empty_bar = [&](int s) { return meta + 8u * uint32_t(kStages + s); };
  unsigned long long *masks = reinterpret_cast<unsigned long long *>(
      smem + kStages * T::kStageBytes + 16 * kStages);

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), kConsumerWarps);
    }
    mbar_fence_init();
  }
  __syncthreads();

  if (warp == kConsumerWarps) {
    // ------------------------------ producer ------------------------------
    const uint64_t policy = l2_policy_evict_first();
    const int ps = cfg.page_size;
    const int64_t table_row = int64_t(batch) * cfg.max_pages_per_seq;
    bool ok = true;
    int issued = 0;  // chunks whose full barrier has been armed
    for (int c = 0; c < nchunks; ++c) {
      const int stage = c % kStages;
      const int fill = c / kStages;
      if (fill > 0) {
        ok = mbar_wait_bounded(empty_bar(stage), uint32_t(fill - 1) & 1u);
        if (!ok) break;
      }
      const int base = a0 + c * ST;
      const int c0 = max(split_begin, base);
      const int c1 = min(split_end, base + ST);
      const int first_page = c0 / ps;
      const int nseg = (c1 - 1) / ps - first_page + 1;
      const uint32_t k_dst = smem_base + uint32_t(stage) * T::kStageBytes;
      const uint32_t v_dst = k_dst + T::kStageTensorBytes;

      unsigned long long my_mask = 0;
      uint32_t my_bytes = 0;
      for (int seg0 = 0; seg0 < nseg; seg0 += kWarpSize) {
        const int seg = seg0 + lane;
        if (seg < nseg) {
          const int lp = first_page + seg;
          const int s0 = max(c0, lp * ps);
          const int s1 = min(c1, (lp + 1) * ps);
          const int slot = lp % cfg.max_pages_per_seq;
          const int phys = __ldg(p.page_table + table_row + slot);
          if (phys >= 0 && phys < cfg.num_pages) {
            const int n = s1 - s0;
            my_bytes += uint32_t(n) * T::kRowBytes;
            my_mask |= ((n >= 64 ? ~0ull : ((1ull << n) - 1ull)) << (s0 - base));
          }
        }
      }
      const uint32_t bytes = __reduce_add_sync(0xffffffffu, my_bytes);
      const uint32_t mask_lo =
          __reduce_or_sync(0xffffffffu, uint32_t(my_mask));
      const uint32_t mask_hi =
          __reduce_or_sync(0xffffffffu, uint32_t(my_mask >> 32));
      if (lane == 0) {
        masks[stage] = (static_cast<unsigned long long>(mask_hi) << 32) | mask_lo;
        if (bytes > 0) {
          mbar_arrive_expect_tx(full_bar(stage), 2u * bytes);
        } else {
          mbar_arrive(full_bar(stage));
        }
      }
      __syncwarp();
      for (int seg0 = 0; seg0 < nseg; seg0 += kWarpSize) {
        const int seg = seg0 + lane;
        if (seg < nseg) {
          const int lp = first_page + seg;
          const int s0 = max(c0, lp * ps);
          const int s1 = min(c1, (lp + 1) * ps);
          const int slot = lp % cfg.max_pages_per_seq;
          const int phys = __ldg(p.page_table + table_row + slot);
          if (phys >= 0 && phys < cfg.num_pages) {
            const int64_t src =
                cache_offset(cfg, p.layer, phys, s0 - lp * ps, 0, 0);
            const uint32_t dst_off = uint32_t(s0 - base) * T::kRowBytes;
            const uint32_t nbytes = uint32_t(s1 - s0) * T::kRowBytes;
            bulk_load_hint(k_dst + dst_off, p.cache_k + src, nbytes,
                           full_bar(stage), policy);
            bulk_load_hint(v_dst + dst_off, p.cache_v + src, nbytes,
                           full_bar(stage), policy);
          }
        }
      }
      issued = c + 1;
    }
    // Hold the CTA until every copy this warp issued has landed.
    for (int s = 0; s < kStages && s < issued; ++s) {
      // last fill of stage s among chunks [0, issued)
      const int fill = (issued - 1 - s) / kStages;
      if (!mbar_wait_bounded(full_bar(s), uint32_t(fill) & 1u)) ok = false;
    }
    if (!ok && lane == 0) set_status(p.status, B200KV_STATUS_WAIT_TIMEOUT);
    return;
  }

  // -------------------------------- consumers --------------------------------
  const int head = warp % HKV;
  const int sub = warp / HKV;
  const int my_g = lane >> 4;        // which of the G q heads this lane scores
  const int my_t = (lane >> 2) & 3;  // which of the warp's 4 tokens

  float qf[G][8];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    const int64_t row = int64_t(batch) * p.q_heads + head * G + g;
    const uint4 raw =
        __ldg(reinterpret_cast<const uint4 *>(p.q + row * D) + lane);
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      qf[g][2 * i] = bf16_lo(w[i]) * p.scale_log2;
      qf[g][2 * i + 1] = bf16_hi(w[i]) * p.scale_log2;
    }
  }

  float acc[G][8];
  float m[G];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    m[g] = -INFINITY;
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[g][i] = 0.0f;
  }
  float l_lane = 0.0f;  // running sum of this lane's own (g, t) weights

  const uint32_t lane_off = uint32_t(head * D + lane * 8) * 2u;
  bool ok = true;
  for (int c = 0; c < nchunks; ++c) {
    const int stage = c % kStages;
    const int fill = c / kStages;
    if (!mbar_wait_bounded(full_bar(stage), uint32_t(fill) & 1u)) {
      ok = false;
      break;
    }
    const unsigned long long mask = masks[stage];
    const uint32_t mine = uint32_t(mask >> (sub * kTokPerWarp)) & 0xfu;
    if (mine != 0u) {
      const uint32_t k_base = smem_base + uint32_t(stage) * T::kStageBytes +
                              uint32_t(sub * kTokPerWarp) * T::kRowBytes +
                              lane_off;
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
                  fmaf(qf[g][2 * i], lo, s[g * kTokPerWarp + t]);
              s[g * kTokPerWarp + t] =
                  fmaf(qf[g][2 * i + 1], hi, s[g * kTokPerWarp + t]);
            }
          }
        }
      }
      float my_s = reduce_scatter8(s, lane);
      if (((mine >> my_t) & 1u) == 0u) my_s = -INFINITY;

      float tile_max = fmaxf(my_s, __shfl_xor_sync(0xffffffffu, my_s, 8));
      tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, 4));
      const float other_max = __shfl_xor_sync(0xffffffffu, tile_max, 16);
      const float new_m0 = fmaxf(m[0], my_g == 0 ? tile_max : other_max);
      const float new_m1 = fmaxf(m[1], my_g == 0 ? other_max : tile_max);
      if (new_m0 > m[0] || new_m1 > m[1]) {
        const float corr0 = ex2_approx(m[0] - new_m0);
        const float corr1 = ex2_approx(m[1] - new_m1);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          acc[0][i] *= corr0;
          acc[1][i] *= corr1;
        }
        l_lane *= (my_g == 0 ? corr0 : corr1);
        m[0] = new_m0;
        m[1] = new_m1;
      }
      const float pr = ex2_approx(my_s - (my_g == 0 ? m[0] : m[1]));
      l_lane += pr;

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
            acc[0][2 * i] = fmaf(p0, lo, acc[0][2 * i]);
            acc[0][2 * i + 1] = fmaf(p0, hi, acc[0][2 * i + 1]);
            acc[1][2 * i] = fmaf(p1, lo, acc[1][2 * i]);
            acc[1][2 * i + 1] = fmaf(p1, hi, acc[1][2 * i + 1]);
          }
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(empty_bar(stage));
  }
  if (!ok) {
    if (lane == 0) set_status(p.status, B200KV_STATUS_WAIT_TIMEOUT);
    return;  // every other wait in this CTA is bounded as well
  }

  // Denominator per head: sum the four token lanes (copies in lanes that
  // share lane >> 2 are not added), then fetch the other head's value.
  float l_mine = l_lane + __shfl_xor_sync(0xffffffffu, l_lane, 8);
  l_mine += __shfl_xor_sync(0xffffffffu, l_mine, 4);
  const float l_other = __shfl_xor_sync(0xffffffffu, l_mine, 16);
  float l[G];
  l[0] = my_g == 0 ? l_mine : l_other;
  l[1] = my_g == 0 ? l_other : l_mine;

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
      const float inv = l[g] > 0.0f ? 1.0f / l[g] : 0.0f;
      uint32_t packed[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const __nv_bfloat162 h2 = __floats2bfloat162_rn(
            acc[g][2 * i] * inv, acc[g][2 * i + 1] * inv);
        packed[i] = *reinterpret_cast<const uint32_t *>(&h2);
      }
      reinterpret_cast<uint4 *>(p.out + row * D)[lane] =
          make_uint4(packed[0], packed[1], packed[2], packed[3]);
      if (p.lse != nullptr && lane == 0) {
        p.lse[row] = l[g] > 0.0f
                         ? (m[g] + lg2_approx(l[g])) * 0.6931471805599453f
                         : -INFINITY;
      }
    } else {
      // :865-877 -- partials, stride num_splits per row. m is kept in the
      // exp2 domain (scaled score * log2 e); the combine below knows.
      const int64_t slot = row * p.num_splits + split;
      if (lane == 0) {
        p.partial_m[slot] = m[g];
        p.partial_l[slot] = l[g];
      }
      float4 *dst = reinterpret_cast<float4 *>(p.partial_acc + slot * D) +
                    lane * 2;
      dst[0] = make_float4(acc[g][0], acc[g][1], acc[g][2], acc[g][3]);
      dst[1] = make_float4(acc[g][4], acc[g][5], acc[g][6], acc[g][7]);
    }
  }
}

// One CTA per (batch, q_head) row: LSE-style combine of the live splits
// (src/gemma4_flash_attention_decode.cu:881-977).
template <int D>
__global__ __launch_bounds__(D / 4) void decode_combine_kernel(DecodeParams p) {
  const int row = int(blockIdx.x);
  const int batch = row / p.q_heads;
  const int tid = int(threadIdx.x);
  const int seq_len = __ldg(p.seq_lengths + batch);
  const LiveRange lr = live_range(p.cfg, seq_len, p.split_size);
  const int reduce_splits = min(lr.actual_splits, p.num_splits);
  uint2 *out = reinterpret_cast<uint2 *>(p.out + int64_t(row) * D) + tid;
  if (reduce_splits == 0) {  // :920-926
    *out = make_uint2(0, 0);
    if (p.lse != nullptr && tid == 0) p.lse[row] = -INFINITY;
    return;
  }
  const float *pm = p.partial_m + int64_t(row) * p.num_splits;
  const float *pl = p.partial_l + int64_t(row) * p.num_splits;
  float M = -INFINITY;
  for (int s = 0; s < reduce_splits; ++s) M = fmaxf(M, __ldg(pm + s));
  float L = 0.0f;
  float4 value = make_float4(0.f, 0.f, 0.f, 0.f);
  const float4 *acc = reinterpret_cast<const float4 *>(
                          p.partial_acc + int64_t(row) * p.num_splits * D) +
                      tid;
  for (int s = 0; s < reduce_splits; ++s) {
    const float sl = __ldg(pl + s);
    if (sl > 0.0f) {  // :953-956 skips empty splits
      const float w = ex2_approx(__ldg(pm + s) - M);
      L = fmaf(sl, w, L);
      const float4 a = __ldg(acc + size_t(s) * (D / 4));
      value.x = fmaf(a.x, w, value.x);
      value.y = fmaf(a.y, w, value.y);
      value.z = fmaf(a.z, w, value.z);
      value.w = fmaf(a.w, w, value.w);
    }
  }
  const float inv = L > 0.0f ? 1.0f / L : 0.0f;
  const __nv_bfloat162 lo = __floats2bfloat162_rn(value.x * inv, value.y * inv);
  const __nv_bfloat162 hi = __floats2bfloat162_rn(value.z * inv, value.w * inv);
  *out = make_uint2(*reinterpret_cast<const uint32_t *>(&lo),
                    *reinterpret_cast<const uint32_t *>(&hi));
  if (p.lse != nullptr && tid == 0) {
    p.lse[row] =
        L > 0.0f ? (M + lg2_approx(L)) * 0.6931471805599453f : -INFINITY;
  }
}

template <class T>
cudaError_t launch_split(const DecodeParams &p, int batch_count,
                         cudaStream_t stream) {
  static_assert(T::kSmemBytes <= 227 * 1024, "ring must fit one SM");
  // Per-device opt-in for the large dynamic shared-memory carve-out; the
  // attribute is sticky, setting it again is cheap and thread-safe.
  cudaError_t st = cudaFuncSetAttribute(
      decode_split_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
      T::kSmemBytes);
  if (st != cudaSuccess) return st;
  const dim3 grid(p.num_splits, batch_count);
  decode_split_kernel<T><<<grid, T::kThreads, T::kSmemBytes, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace

int decode_stage_tokens(int kv_heads) {
  if (kv_heads <= 0 || kConsumerWarps % kv_heads != 0) return kTokPerWarp;
  return (kConsumerWarps / kv_heads) * kTokPerWarp;
}

cudaError_t decode_attention_bf16(const DecodeArgs &a, cudaStream_t stream) {
  const Gemma4KvCacheConfig &c = a.cfg;
  // Validation mirrors gemma4_fa_valid_cache_config and the launcher checks
  // (src/gemma4_flash_attention_decode.cu:377-392,1129-1134).
  if (a.out == nullptr || a.q == nullptr || a.cache_k == nullptr ||
      a.cache_v == nullptr || a.page_table == nullptr ||
      a.seq_lengths == nullptr || a.batch_count <= 0 || a.layer < 0 ||
      a.layer >= c.num_layers || c.num_pages <= 0 || c.page_size <= 0 ||
      c.max_pages_per_seq <= 0 || c.batch_size <= 0 || c.window_size < 0 ||
      a.split_size <= 0 || a.num_splits <= 0 || !(a.softmax_scale > 0.0f) ||
      a.q_heads <= 0 || c.num_heads <= 0 || a.q_heads % c.num_heads != 0) {
    return cudaErrorInvalidValue;
  }
  if (c.window_size > 0 &&
      int64_t(c.max_pages_per_seq) * c.page_size < c.window_size) {
    return cudaErrorInvalidValue;  // ring smaller than the window (:389-391)
  }
  if (a.num_splits > 1 && (a.partial_m == nullptr || a.partial_l == nullptr ||
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
    switch (c.num_heads) {
      case 8: st = launch_split<DecodeTraits<256, 8, 2>>(p, a.batch_count, stream); break;
      case 4: st = launch_split<DecodeTraits<256, 4, 2>>(p, a.batch_count, stream); break;
      case 2: st = launch_split<DecodeTraits<256, 2, 2>>(p, a.batch_count, stream); break;
      case 1: st = launch_split<DecodeTraits<256, 1, 2>>(p, a.batch_count, stream); break;
      default: break;
    }
  }
  if (st != cudaSuccess) return st;
  if (a.num_splits > 1) {
    decode_combine_kernel<256>
        <<<a.batch_count * a.q_heads, 64, 0, stream>>>(p);
    st = cudaGetLastError();
  }
  return st;
}

}  // namespace b200kv

// FP8 e4m3 variant of the decode ring: K/V rows are one byte per element with
// one fp32 scale per (page, KV head) and tensor. No counterpart in the
// reference (its caches are bf16 only); the quantisation rule is stated in
// fp8_cache.cu. Dequantisation is fused into the attention: the K scale is
// applied to the reduced score, the V scale is folded into the softmax weight,
// so the only extra work per element is the e4m3 -> fp32 conversion.
#pragma once

#include <cuda_fp8.h>

#include "decode_common.cuh"

namespace b200kv {

// 8 KV heads x 256 dims, 2 query heads per KV head, 8 consumer warps (one per
// KV head), two CTAs per SM. A stage holds 8 tokens (two groups of four per
// warp): 16 KiB of K + 16 KiB of V.
struct Fp8DecodeTraits {
  static constexpr int D = 256;
  static constexpr int HKV = 8;
  static constexpr int G = 2;
  static constexpr int kConsumerWarps = 8;
  static constexpr int kCtasPerSm = 2;
  static constexpr int kWarpsPerHead = 1;
  static constexpr bool kFp8 = true;
  static constexpr int kElemBytes = 1;
  static constexpr int kGroups = 2;
  static constexpr int kStageTokens = kGroups * kTokPerWarp;
  static constexpr int kRowBytes = HKV * D;
  static constexpr int kStageTensorBytes = kStageTokens * kRowBytes;
  static constexpr int kStageBytes = 2 * kStageTensorBytes;
  static constexpr int kThreads = (kConsumerWarps + 1) * kWarpSize;
  static constexpr int kMetaBytes = 256;
  static constexpr int kMaxSegs = kStageTokens;  // page_size 1 at worst
  // per stage: [segment][tensor][head] fp32
  static constexpr int kScaleFloatsPerStage = kMaxSegs * 2 * HKV;
  static constexpr int kScaleBytes = kStages * kScaleFloatsPerStage * 4;
  static constexpr int kRingBytes = kStages * kStageBytes + kMetaBytes + kScaleBytes;
};

struct Fp8Scales {
  const float *scale_k;  // [layer, page, head]
  const float *scale_v;
};

__device__ __forceinline__ float *fp8_scale_table(const Ring<Fp8DecodeTraits> &ring,
                                                  int stage) {
  using T = Fp8DecodeTraits;
  return reinterpret_cast<float *>(ring.smem + kStages * T::kStageBytes +
                                   T::kMetaBytes) +
         stage * T::kScaleFloatsPerStage;
}

__device__ __forceinline__ uint2 lds64(uint32_t addr) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];"
               : "=r"(v.x), "=r"(v.y)
               : "r"(addr));
  return v;
}

__device__ __forceinline__ float2 e4m3x2_to_float2(uint32_t two_bytes) {
  const __half2_raw h = __nv_cvt_fp8x2_to_halfraw2(
      static_cast<__nv_fp8x2_storage_t>(two_bytes & 0xffffu), __NV_E4M3);
  return __half22float2(*reinterpret_cast<const __half2 *>(&h));
}

// Producer warp, fp8: as producer_fill_stage, plus the per-page scales of the
// stage's segments into shared memory. The copies are issued first so that the
// scale loads overlap them; the full barrier is armed last (its one pending
// arrival keeps the phase open until then).
__device__ __forceinline__ void producer_fill_stage_fp8(
    const Ring<Fp8DecodeTraits> &ring, const KvSource &src,
    const Fp8Scales &scales, const Gemma4KvCacheConfig &cfg, int batch, int base,
    int c0, int c1, int stage, uint64_t policy, int lane) {
  using T = Fp8DecodeTraits;
  const int ps = cfg.page_size;
  const int64_t table_row = int64_t(batch) * cfg.max_pages_per_seq;
  const int first_page = c0 / ps;
  const int nseg = (c1 - 1) / ps - first_page + 1;  // <= kStageTokens
  const uint32_t k_dst = ring.k_stage(stage);
  const uint32_t v_dst = k_dst + T::kStageTensorBytes;

  int phys = -1;
  unsigned long long my_mask = 0;
  uint32_t my_bytes = 0;
  if (lane < nseg) {
    const int lp = first_page + lane;
    const int s0 = max(c0, lp * ps);
    const int s1 = min(c1, (lp + 1) * ps);
    const int slot = lp % cfg.max_pages_per_seq;
    const int entry = __ldg(src.page_table + table_row + slot);
    if (entry >= 0 && entry < cfg.num_pages) {
      phys = entry;
      const int n = s1 - s0;
      my_bytes = uint32_t(n) * T::kRowBytes;
      my_mask = ((1ull << n) - 1ull) << (s0 - base);
      const int64_t off = cache_offset(cfg, src.layer, phys, s0 - lp * ps, 0, 0);
      const uint32_t dst_off = uint32_t(s0 - base) * T::kRowBytes;
      bulk_load_hint(k_dst + dst_off, src.cache_k + off, my_bytes,
                     ring.full_bar(stage), policy);
      bulk_load_hint(v_dst + dst_off, src.cache_v + off, my_bytes,
                     ring.full_bar(stage), policy);
    }
  }
  float *table = fp8_scale_table(ring, stage);
#pragma unroll
  for (int e0 = 0; e0 < T::kMaxSegs * T::HKV; e0 += kWarpSize) {
    const int e = e0 + lane;
    const int seg = e / T::HKV;
    const int head = e % T::HKV;
    const int seg_phys = __shfl_sync(0xffffffffu, phys, seg & 31);
    float sk = 0.0f, sv = 0.0f;
    if (seg < nseg && seg_phys >= 0) {
      const int64_t idx =
          (int64_t(src.layer) * cfg.num_pages + seg_phys) * T::HKV + head;
      sk = __ldg(scales.scale_k + idx);
      sv = __ldg(scales.scale_v + idx);
    }
    table[(seg * 2 + 0) * T::HKV + head] = sk;
    table[(seg * 2 + 1) * T::HKV + head] = sv;
  }
  const uint32_t bytes = __reduce_add_sync(0xffffffffu, my_bytes);
  const uint32_t mask_lo = __reduce_or_sync(0xffffffffu, uint32_t(my_mask));
  __syncwarp();
  if (lane == 0) {
    ring.masks()[stage] = mask_lo;
    if (bytes > 0) {
      mbar_arrive_expect_tx(ring.full_bar(stage), 2u * bytes);
    } else {
      mbar_arrive(ring.full_bar(stage));
    }
  }
}

// One stage for one consumer warp (= KV head `head`), fp8 rows.
__device__ __forceinline__ void consume_stage_fp8(
    WarpState<Fp8DecodeTraits> &st, const Ring<Fp8DecodeTraits> &ring, int stage,
    int head, int lane, int base, int c0, int page_size) {
  using T = Fp8DecodeTraits;
  constexpr int G = T::G;
  const int my_g = lane >> 4;
  const int my_t = (lane >> 2) & 3;
  const uint32_t mask = uint32_t(ring.masks()[stage]);
  const float *table = fp8_scale_table(ring, stage);
  const int first_page = c0 / page_size;
#pragma unroll
  for (int grp = 0; grp < T::kGroups; ++grp) {
    const uint32_t mine = (mask >> (grp * kTokPerWarp)) & 0xfu;
    if (mine == 0u) continue;
    const uint32_t k_base = ring.k_stage(stage) +
                            uint32_t(grp * kTokPerWarp) * T::kRowBytes +
                            uint32_t(head * T::D + lane * 8);
    const uint32_t v_base = k_base + T::kStageTensorBytes;

    float s[G * kTokPerWarp];
#pragma unroll
    for (int i = 0; i < G * kTokPerWarp; ++i) s[i] = 0.0f;
#pragma unroll
    for (int t = 0; t < kTokPerWarp; ++t) {
      if ((mine >> t) & 1u) {
        const uint2 kk = lds64(k_base + uint32_t(t) * T::kRowBytes);
        const uint32_t w[2] = {kk.x, kk.y};
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const float2 a = e4m3x2_to_float2(w[i]);
          const float2 b = e4m3x2_to_float2(w[i] >> 16);
#pragma unroll
          for (int g = 0; g < G; ++g) {
            float acc = s[g * kTokPerWarp + t];
            acc = fmaf(st.qf[g][4 * i + 0], a.x, acc);
            acc = fmaf(st.qf[g][4 * i + 1], a.y, acc);
            acc = fmaf(st.qf[g][4 * i + 2], b.x, acc);
            acc = fmaf(st.qf[g][4 * i + 3], b.y, acc);
            s[g * kTokPerWarp + t] = acc;
          }
        }
      }
    }
    float my_s = reduce_scatter8(s, lane);
    float my_sv = 0.0f;
    if ((mine >> my_t) & 1u) {
      const int token = grp * kTokPerWarp + my_t;
      const int seg = (base + token) / page_size - first_page;
      my_s *= table[(seg * 2 + 0) * T::HKV + head];
      my_sv = table[(seg * 2 + 1) * T::HKV + head];
    } else {
      my_s = -INFINITY;
    }

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
    const float pv = pr * my_sv;  // softmax weight times the V scale of its page

#pragma unroll
    for (int t = 0; t < kTokPerWarp; ++t) {
      if ((mine >> t) & 1u) {
        const float p0 = __shfl_sync(0xffffffffu, pv, t << 2);
        const float p1 = __shfl_sync(0xffffffffu, pv, 16 | (t << 2));
        const uint2 vv = lds64(v_base + uint32_t(t) * T::kRowBytes);
        const uint32_t w[2] = {vv.x, vv.y};
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const float2 a = e4m3x2_to_float2(w[i]);
          const float2 b = e4m3x2_to_float2(w[i] >> 16);
          st.acc[0][4 * i + 0] = fmaf(p0, a.x, st.acc[0][4 * i + 0]);
          st.acc[0][4 * i + 1] = fmaf(p0, a.y, st.acc[0][4 * i + 1]);
          st.acc[0][4 * i + 2] = fmaf(p0, b.x, st.acc[0][4 * i + 2]);
          st.acc[0][4 * i + 3] = fmaf(p0, b.y, st.acc[0][4 * i + 3]);
          st.acc[1][4 * i + 0] = fmaf(p1, a.x, st.acc[1][4 * i + 0]);
          st.acc[1][4 * i + 1] = fmaf(p1, a.y, st.acc[1][4 * i + 1]);
          st.acc[1][4 * i + 2] = fmaf(p1, b.x, st.acc[1][4 * i + 2]);
          st.acc[1][4 * i + 3] = fmaf(p1, b.y, st.acc[1][4 * i + 3]);
        }
      }
    }
  }
}

}  // namespace b200kv

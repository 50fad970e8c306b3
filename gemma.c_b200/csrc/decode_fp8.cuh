// FP8 e4m3 variant of the decode ring: K/V rows are one byte per element with
// one fp32 scale per (page, KV head) and tensor. No counterpart in the
// reference (its caches are bf16 only); the quantisation rule and the cache
// layout are stated in fp8_cache.cu.
//
// At one byte per element the fp32 lane-per-8-dims arithmetic of the bf16
// kernel issues more instructions per byte than HBM delivers bytes, so the two
// contractions are done differently here:
//   * scores: one tensor-core chain per stage. A = the 8 key rows of the stage
//     (e4m3 as stored, rows 8..15 of the tile zero), B = the query, split into
//     two e4m3 terms hi + lo per head (columns h0.hi h0.lo h1.hi h1.lo, the
//     other four zero), fp32 accumulate: 8 x mma.m16n8k32 per 8 keys. hi + lo
//     carries the query to about 2^-8 relative, the precision bf16 gives it;
//     the K scale of the page and the power of two that normalised the query
//     multiply the finished score.
//   * P*V: packed half2 FMAs on the e4m3 codes of V (exact in fp16) with the
//     softmax weights rounded to fp16, accumulated in fp16 over the 8 keys of
//     the stage only (|sum| <= 8 * 448), then folded into the fp32 accumulator
//     with the V scale of the page.
#pragma once

#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include "decode_common.cuh"

namespace b200kv {

// 8 KV heads x 256 dims, 2 query heads per KV head, 8 consumer warps (one per
// KV head), two CTAs per SM. A stage is one aligned block of 8 tokens of one
// page: 16 KiB of K + 16 KiB of V, each contiguous in the cache.
struct Fp8DecodeTraits {
  static constexpr int D = 256;
  static constexpr int HKV = 8;
  static constexpr int G = 2;
  static constexpr int kConsumerWarps = 8;
  static constexpr int kCtasPerSm = 2;
  static constexpr int kWarpsPerHead = 1;
  static constexpr bool kFp8 = true;
  static constexpr int kElemBytes = 1;
  static constexpr int kStageTokens = 8;
  static constexpr int kRowBytes = HKV * D;
  static constexpr int kStageTensorBytes = kStageTokens * kRowBytes;
  static constexpr int kStageBytes = 2 * kStageTensorBytes;
  static constexpr int kThreads = (kConsumerWarps + 1) * kWarpSize;
  static constexpr int kMetaBytes = 256;
  // per stage: K multipliers of the 8 heads, then V scales of the 8 heads
  static constexpr int kScaleFloatsPerStage = 2 * HKV;
  static constexpr int kScaleBytes = kStages * kScaleFloatsPerStage * 4;
  // per consumer warp: the stage's 8 x 2 softmax weights as (p, p) half2 pairs
  static constexpr int kWeightBytesPerWarp = kStageTokens * G * 4;
  static constexpr int kWeightBytes = kConsumerWarps * kWeightBytesPerWarp;
  static constexpr int kRingBytes =
      kStages * kStageBytes + kMetaBytes + kScaleBytes + kWeightBytes;
};

struct Fp8Scales {
  const float *scale_k;  // [layer, page, head]
  const float *scale_v;
  float scale_log2;      // softmax scale * log2(e), folded into the K multiplier
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

__device__ __forceinline__ __half2 e4m3x2_to_half2(uint32_t two_bytes) {
  const __half2_raw h = __nv_cvt_fp8x2_to_halfraw2(
      static_cast<__nv_fp8x2_storage_t>(two_bytes & 0xffffu), __NV_E4M3);
  return *reinterpret_cast<const __half2 *>(&h);
}

// D (16x8, fp32) += A (16x32 e4m3, row) * B (32x8 e4m3, col); rows 8..15 of A
// are zero here, so a1 = a3 = 0 and d2, d3 are never read.
__device__ __forceinline__ void mma_e4m3_m16n8k32(float (&d)[4], uint32_t a0,
                                                  uint32_t a2, uint32_t b0,
                                                  uint32_t b1) {
  const uint32_t zero = 0u;
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 "
      "{%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(zero), "r"(a2), "r"(zero), "r"(b0), "r"(b1));
}

// Producer warp, fp8: the stage [base, base + 8) is one 8-token block of one
// page; its K block and its V rows are each 16 KiB contiguous and are copied
// whole (positions outside [c0, c1) are masked off by the consumers). The
// copies are issued first so that the scale loads overlap them; the full
// barrier is armed last (its one pending arrival keeps the phase open).
__device__ __forceinline__ void producer_fill_stage_fp8(
    const Ring<Fp8DecodeTraits> &ring, const KvSource &src,
    const Fp8Scales &scales, const Gemma4KvCacheConfig &cfg, int batch, int base,
    int c0, int c1, int stage, uint64_t policy, int lane) {
  using T = Fp8DecodeTraits;
  const int ps = cfg.page_size;
  const int lp = base / ps;
  const int slot = lp % cfg.max_pages_per_seq;
  const int entry =
      __ldg(src.page_table + int64_t(batch) * cfg.max_pages_per_seq + slot);
  const bool mapped = entry >= 0 && entry < cfg.num_pages;
  if (mapped) {
    const int64_t off =
        ((int64_t(src.layer) * cfg.num_pages + entry) * ps + (base - lp * ps)) *
        T::kRowBytes;
    const uint32_t k_dst = ring.k_stage(stage);
    if (lane == 0) {
      bulk_load_hint(k_dst, src.cache_k + off, T::kStageTensorBytes,
                     ring.full_bar(stage), policy);
    } else if (lane == 1) {
      bulk_load_hint(k_dst + T::kStageTensorBytes, src.cache_v + off,
                     T::kStageTensorBytes, ring.full_bar(stage), policy);
    }
    if (lane < 2 * T::HKV) {
      const int64_t idx =
          (int64_t(src.layer) * cfg.num_pages + entry) * T::HKV + (lane & 7);
      fp8_scale_table(ring, stage)[lane] =
          lane < T::HKV ? __ldg(scales.scale_k + idx) * scales.scale_log2
                        : __ldg(scales.scale_v + idx);
    }
  }
  __syncwarp();
  if (lane == 0) {
    const uint32_t mask = mapped ? ((1u << (c1 - c0)) - 1u) << (c0 - base) : 0u;
    ring.masks()[stage] = mask;
    if (mapped) {
      mbar_arrive_expect_tx(ring.full_bar(stage), 2u * T::kStageTensorBytes);
    } else {
      mbar_arrive(ring.full_bar(stage));
    }
  }
}

// Running state of one consumer warp (= one KV head, two query heads). For the
// score MMA lane = 4 * g + t holds row g (a key of the stage) of A and column g
// of B; for P*V a lane owns dims 8 * lane .. + 7 of both heads, as in the bf16
// kernel.
struct Fp8WarpState {
  uint32_t qb[16];  // B fragments: MMA j uses qb[2 * j], qb[2 * j + 1]
  float qmul;       // undoes the query normalisation of head (lane & 1)
  float acc[2][8];
  float m[2];       // running maxima, exp2 domain
  float l_lane;     // running sum of the weights of (key lane >> 2, head lane & 1)

  __device__ __forceinline__ void reset() {
#pragma unroll
    for (int g = 0; g < 2; ++g) {
      m[g] = -INFINITY;
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[g][i] = 0.0f;
    }
    l_lane = 0.0f;
  }

  // Loads the two prepared query rows of this warp's KV head (q_rows points at
  // the first of them) and builds the B fragments. Column n = lane >> 2 is
  // head n / 2, term n % 2 (0 = hi, 1 = lo) for n < 4 and zero otherwise. MMA
  // j = 2c + u contracts dims 16 (t + 4c) + 8u + {0..7}, t = lane & 3, which is
  // the order the K rows are fetched in (consume_stage_fp8). Each head is
  // scaled by the power of two that puts its largest magnitude in [128, 256)
  // before the split, so neither term leaves the e4m3 range.
  __device__ __forceinline__ void load_q(const __nv_bfloat16 *q_rows, int lane) {
    const int n = lane >> 2;
    const int t = lane & 3;
    const uint4 *row =
        reinterpret_cast<const uint4 *>(q_rows + ((n >> 1) & 1) * Fp8DecodeTraits::D);
    // two passes over the same 8 loads (the second hits L1): holding them
    // across the reduction costs registers the streaming loop needs
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint4 raw = __ldg(row + 2 * (t + 4 * (i >> 1)) + (i & 1));
      const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        amax = fmaxf(amax, fmaxf(fabsf(bf16_lo(w[k])), fabsf(bf16_hi(w[k]))));
      }
    }
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    // amax = 2^(ex - 127) * [1, 2): scale by 2^(134 - ex), undo with 2^(ex - 134)
    const int ex = min(max((__float_as_int(amax) >> 23) & 0xff, 8), 253);
    const float up = __int_as_float((261 - ex) << 23);
    const float down = __int_as_float((ex - 7) << 23);
    const bool lo_term = (n & 1) != 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint4 raw = __ldg(row + 2 * (t + 4 * (i >> 1)) + (i & 1));
      const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
      uint32_t packed[2];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        float2 x = make_float2(bf16_lo(w[k]) * up, bf16_hi(w[k]) * up);
        uint32_t code = __nv_cvt_float2_to_fp8x2(x, __NV_SATFINITE, __NV_E4M3);
        if (lo_term) {
          const float2 hi = __half22float2(e4m3x2_to_half2(code));
          x = make_float2(x.x - hi.x, x.y - hi.y);
          code = __nv_cvt_float2_to_fp8x2(x, __NV_SATFINITE, __NV_E4M3);
        }
        if ((k & 1) == 0) {
          packed[k >> 1] = code & 0xffffu;
        } else {
          packed[k >> 1] |= code << 16;
        }
      }
      // load i = 2c + u covers dims 16 (t + 4c) + 8u + {0..7}: MMA j = 2c + u = i
      qb[2 * i] = n < 4 ? packed[0] : 0u;
      qb[2 * i + 1] = n < 4 ? packed[1] : 0u;
    }
    // the score of head h is finished in lanes with t == h; head h's factor
    // was computed in the lanes with n == 2h (and 2h + 1)
    qmul = __shfl_sync(0xffffffffu, down, (t & 1) << 3);
  }

  __device__ __forceinline__ void denominators(float (&l)[2], int lane) const {
    float x = l_lane + __shfl_xor_sync(0xffffffffu, l_lane, 4);
    x += __shfl_xor_sync(0xffffffffu, x, 8);
    x += __shfl_xor_sync(0xffffffffu, x, 16);
    l[0] = __shfl_sync(0xffffffffu, x, 0);
    l[1] = __shfl_sync(0xffffffffu, x, 1);
  }
};

// One stage for one consumer warp (= KV head `head`).
__device__ __forceinline__ void consume_stage_fp8(Fp8WarpState &st,
                                                  const Ring<Fp8DecodeTraits> &ring,
                                                  int stage, int head, int lane) {
  using T = Fp8DecodeTraits;
  const uint32_t mask = uint32_t(ring.masks()[stage]);
  if (mask == 0u) return;
  const int g = lane >> 2;
  const int t = lane & 3;
  const float *table = fp8_scale_table(ring, stage);
  const float k_mul = table[head];
  const float v_scale = table[T::HKV + head];

  // ---- scores: row g of the tile is key g; the lane fetches granules t + 4c
  // of that row (stored permuted, fp8_cache.cu) and each 128-bit load feeds two
  // MMAs. Two accumulator chains halve the dependent latency.
  const uint32_t k_row = ring.k_stage(stage) + uint32_t(head) * (8u * T::D) +
                         uint32_t(g) * T::D;
  const uint32_t swz = uint32_t(g & 1) << 2;
  float d_even[4] = {0.f, 0.f, 0.f, 0.f};
  float d_odd[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const uint4 kk = lds128(k_row + ((uint32_t(t + 4 * c) ^ swz) << 4));
    mma_e4m3_m16n8k32(d_even, kk.x, kk.y, st.qb[4 * c], st.qb[4 * c + 1]);
    mma_e4m3_m16n8k32(d_odd, kk.z, kk.w, st.qb[4 * c + 2], st.qb[4 * c + 3]);
  }
  // columns 2t, 2t + 1 of row g: hi and lo term of head t (t < 2)
  const bool live = t < 2 && ((mask >> g) & 1u) != 0u;
  const float my_s =
      live ? ((d_even[0] + d_odd[0]) + (d_even[1] + d_odd[1])) * (st.qmul * k_mul)
           : -INFINITY;

  // ---- online softmax: maxima over the keys (lanes that share t)
  float tile_max = fmaxf(my_s, __shfl_xor_sync(0xffffffffu, my_s, 4));
  tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, 8));
  tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, 16));
  const float new_m0 = fmaxf(st.m[0], __shfl_sync(0xffffffffu, tile_max, 0));
  const float new_m1 = fmaxf(st.m[1], __shfl_sync(0xffffffffu, tile_max, 1));
  if (new_m0 > st.m[0] || new_m1 > st.m[1]) {
    const float corr0 = ex2_approx(st.m[0] - new_m0);
    const float corr1 = ex2_approx(st.m[1] - new_m1);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      st.acc[0][i] *= corr0;
      st.acc[1][i] *= corr1;
    }
    st.l_lane *= ((t & 1) == 0 ? corr0 : corr1);
    st.m[0] = new_m0;
    st.m[1] = new_m1;
  }
  const float pr = ex2_approx(my_s - ((t & 1) == 0 ? st.m[0] : st.m[1]));
  st.l_lane += pr;
  // Every lane needs every key's two weights, duplicated into both halves of a
  // half2: exchanged through 64 bytes of shared memory per warp (the previous
  // stage's reads are behind the __syncwarp that ends a stage).
  constexpr uint32_t kWeightOffset =
      kStages * T::kStageBytes + T::kMetaBytes + T::kScaleBytes;
  const uint32_t w_off = kWeightOffset + uint32_t(head) * T::kWeightBytesPerWarp;
  if (t < 2) {
    const __half2 pp = __float2half2_rn(pr);
    reinterpret_cast<uint32_t *>(ring.smem + w_off)[g * 2 + t] =
        *reinterpret_cast<const uint32_t *>(&pp);
  }
  __syncwarp();

  // ---- P*V on the codes, fp16 over the stage, then one scaled fp32 update
  const uint32_t v_base = ring.k_stage(stage) + T::kStageTensorBytes +
                          uint32_t(head * T::D + lane * 8);
  __half2 part[2][4];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
#pragma unroll
    for (int i = 0; i < 4; ++i) part[h][i] = __float2half2_rn(0.0f);
  }
  auto add_key = [&](int tk, uint32_t p0_bits, uint32_t p1_bits) {
    const __half2 p0 = *reinterpret_cast<const __half2 *>(&p0_bits);
    const __half2 p1 = *reinterpret_cast<const __half2 *>(&p1_bits);
    const uint2 vv = lds64(v_base + uint32_t(tk) * T::kRowBytes);
    const __half2 v[4] = {e4m3x2_to_half2(vv.x), e4m3x2_to_half2(vv.x >> 16),
                          e4m3x2_to_half2(vv.y), e4m3x2_to_half2(vv.y >> 16)};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      part[0][i] = __hfma2(p0, v[i], part[0][i]);
      part[1][i] = __hfma2(p1, v[i], part[1][i]);
    }
  };
  if (mask == 0xffu) {
#pragma unroll
    for (int pair = 0; pair < T::kStageTokens / 2; ++pair) {
      const uint4 w = lds128(ring.base + w_off + uint32_t(pair) * 16u);
      add_key(2 * pair, w.x, w.y);
      add_key(2 * pair + 1, w.z, w.w);
    }
  } else {
    // rows outside the range may hold anything (a NaN code times a zero weight
    // is still a NaN): they are skipped, not weighted by zero
#pragma unroll
    for (int pair = 0; pair < T::kStageTokens / 2; ++pair) {
      const uint4 w = lds128(ring.base + w_off + uint32_t(pair) * 16u);
      if ((mask >> (2 * pair)) & 1u) add_key(2 * pair, w.x, w.y);
      if ((mask >> (2 * pair + 1)) & 1u) add_key(2 * pair + 1, w.z, w.w);
    }
  }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __half22float2(part[h][i]);
      st.acc[h][2 * i] = fmaf(v_scale, f.x, st.acc[h][2 * i]);
      st.acc[h][2 * i + 1] = fmaf(v_scale, f.y, st.acc[h][2 * i + 1]);
    }
  }
}

}  // namespace b200kv

/* Device-side form of the KV path: CTA-cooperative __device__ phases that a
 * persistent / cooperative kernel (gemma.c's decode megakernel) can call between
 * its own grid-wide barriers, in place of the reference's phases
 *
 *   phase_decode_q_paged_kv_norm_rope   src/gemma4_flash_attention_decode.cu:305-375
 *   phase_decode_paged_grouped_split    src/gemma4_flash_attention_decode.cu:692-878
 *   phase_decode_paged_reduce           src/gemma4_flash_attention_decode.cu:881-977
 *
 * with the reference's conventions: a phase never reads threadIdx / blockIdx
 * -- the caller passes thread_idx / thread_count (all threads of the CTA, a
 * multiple of 32) and the task (batch, kv_head, split / q_head) -- it allocates
 * nothing, invalid rows and unmapped pages are skipped silently, and every
 * buffer has the layout of the host entry points in gemma4_b200kv.h (caches
 * [layer, page, offset, head, dim], partials [row * num_splits + split]).
 *
 * These are the portable form: plain 128-bit loads, no TMA, no programmatic
 * dependent launch, so they work under any synchronisation the caller uses
 * (rows and partials written earlier in the same kernel are read past L1).
 * The library's own kernels (b200kv_decode_layer_step_bf16) are the fast form
 * and what the measurements refer to. Same arithmetic as those kernels: the
 * append's bits are the reference GPU code's (rsqrt.approx, flush-to-zero prep
 * multiplies), attention accumulates in fp32 in the exp2 domain.
 *
 * Geometry: head_dim 256, rotary_dim 256, two query heads per KV head.
 * A phase that uses shared memory says how much; phases end with all their
 * global writes issued, the caller's barrier (grid.sync) publishes them.
 */
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "gemma4_b200kv.hpp"

namespace b200kv_device {

constexpr int kDim = 256;
constexpr int kGroup = 2;  // query heads per KV head
constexpr float kRmsEps = 1.0e-6f;  // GEMMA4_RMS_NORM_EPS, src/gemma4.h:29
// floats of shared memory split_phase needs per warp of the CTA
constexpr int kSplitSmemFloatsPerWarp = kGroup * kDim + 2 * kGroup;

namespace detail {

__device__ __forceinline__ float mul_ftz(float a, float b) {
  float r;
  asm("mul.ftz.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float lg2(float x) {
  float y;
  asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

// One warp, one head row: lane l owns elements l + 32 i; sum of squares as an
// fma chain per lane, then the xor butterfly 16, 8, 4, 2, 1
// (src/gemma4_rmsnorm.cu:90-101, src/gemma4_cuda_utils.cuh:165-170).
__device__ __forceinline__ float rms_scale(const float (&x)[8]) {
  float ss = 0.0f;
#pragma unroll
  for (int i = 0; i < 8; ++i) ss = __fmaf_rn(x[i], x[i], ss);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss = __fadd_rn(ss, __shfl_xor_sync(0xffffffffu, ss, o));
  return rsqrtf(__fadd_rn(__fdiv_rn(ss, float(kDim)), kRmsEps));
}

// Weighted RMSNorm + split-half RoPE of one head row into `out`
// (prep_weighted_rope_head_values, src/gemma4_flash_attention_decode.cu:231-264).
__device__ __forceinline__ void prep_weighted_rope(__nv_bfloat16 *out, const __nv_bfloat16 *in,
                                                   const __nv_bfloat16 *weight,
                                                   const float *cos_row, const float *sin_row,
                                                   int lane) {
  float x[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) x[i] = __bfloat162float(in[lane + 32 * i]);
  const float scale = rms_scale(x);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float lo = mul_ftz(mul_ftz(x[i], scale), __bfloat162float(weight[lane + 32 * i]));
    const float hi =
        mul_ftz(mul_ftz(x[i + 4], scale), __bfloat162float(weight[lane + 32 * (i + 4)]));
    const float c = cos_row[lane + 32 * i];
    const float s = sin_row[lane + 32 * i];
    out[lane + 32 * i] = __float2bfloat16_rn(__fmaf_rn(-hi, s, __fmul_rn(lo, c)));
    out[lane + 32 * (i + 4)] = __float2bfloat16_rn(__fmaf_rn(lo, s, __fmul_rn(hi, c)));
  }
}

// Scale-free RMSNorm of one head row (V rows; src/...decode.cu:268-280).
__device__ __forceinline__ void prep_scale_free(__nv_bfloat16 *out, const __nv_bfloat16 *in,
                                                int lane) {
  float x[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) x[i] = __bfloat162float(in[lane + 32 * i]);
  const float scale = rms_scale(x);
#pragma unroll
  for (int i = 0; i < 8; ++i) out[lane + 32 * i] = __float2bfloat16_rn(mul_ftz(x[i], scale));
}

// Physical page of `position` for sequence `batch`, -1 if unmapped or out of
// the table (decode_cache_head_offset, src/...decode.cu:285-303).
__device__ __forceinline__ int physical_page(const Gemma4KvCacheConfig &c,
                                             const int32_t *page_table, int batch,
                                             int position) {
  const int lp = position / c.page_size;
  if (c.window_size == 0 && lp >= c.max_pages_per_seq) return -1;
  const int e = __ldcg(page_table + int64_t(batch) * c.max_pages_per_seq + lp % c.max_pages_per_seq);
  return (e >= 0 && e < c.num_pages) ? e : -1;
}

}  // namespace detail

/* The fused append for one (batch, kv_head): the two query heads of the group
 * into q_prepared [batch, q_heads, 256], the K row and the V row (from raw V, or
 * from raw K when v == nullptr) into the cache at token_position[batch]. A
 * negative position, a batch outside the cache's batch_size, or an unmapped
 * page skips the sequence / the cache write. One warp per row (four rows), the
 * CTA's warps take them in turn. No shared memory, no barrier inside. */
__device__ inline void append_phase(__nv_bfloat16 *q_prepared, __nv_bfloat16 *cache_k,
                                    __nv_bfloat16 *cache_v, const Gemma4KvCacheConfig &cfg,
                                    const int32_t *page_table, const int32_t *token_position,
                                    int32_t cache_layer, const __nv_bfloat16 *q,
                                    const __nv_bfloat16 *k, const __nv_bfloat16 *v,
                                    const __nv_bfloat16 *q_norm_weight,
                                    const __nv_bfloat16 *k_norm_weight, const float *cos,
                                    const float *sin, int32_t q_heads, int batch, int kv_head,
                                    int thread_idx, int thread_count) {
  const int warp = thread_idx >> 5;
  const int lane = thread_idx & 31;
  const int warps = thread_count >> 5;
  const int position = token_position[batch];
  if (position < 0 || batch < 0 || batch >= cfg.batch_size) return;
  const float *cos_row = cos + int64_t(position) * (kDim / 2);
  const float *sin_row = sin + int64_t(position) * (kDim / 2);
  for (int role = warp; role < kGroup + 2; role += warps) {
    if (role < kGroup) {
      const int64_t row = (int64_t(batch) * q_heads + kv_head * kGroup + role) * kDim;
      detail::prep_weighted_rope(q_prepared + row, q + row, q_norm_weight, cos_row, sin_row, lane);
      continue;
    }
    const int page = detail::physical_page(cfg, page_table, batch, position);
    if (page < 0) continue;
    const int64_t src = (int64_t(batch) * cfg.num_heads + kv_head) * kDim;
    const int64_t dst = gemma4_kv_cache_offset(
        cfg, cache_layer, page, position - (position / cfg.page_size) * cfg.page_size, kv_head, 0);
    if (role == kGroup) {
      detail::prep_weighted_rope(cache_k + dst, k + src, k_norm_weight, cos_row, sin_row, lane);
    } else {
      detail::prep_scale_free(cache_v + dst, (v != nullptr ? v : k) + src, lane);
    }
  }
}

/* Split-KV flash-decode for one task (batch, kv_head, split): the two query
 * heads of the KV head over the keys [first + split * split_size, ... +
 * split_size) of the live range (first = max(0, len - window) for a sliding
 * cache, 0 otherwise). With num_splits == 1 the normalised rows go to `out`
 * (and the log-sum-exp to `lse` if not null); otherwise the unnormalised partial
 * goes to partial_m / partial_l / partial_acc at [row * num_splits + split]
 * with m in the exp2 domain (what reduce_phase and the library's combine
 * expect). A split beyond the live keys returns without touching the scratch,
 * like the reference's (src/...decode.cu:746-748); with num_splits == 1 an empty
 * sequence writes zero rows. Warps take groups of four keys in turn; `smem`
 * holds kSplitSmemFloatsPerWarp floats per warp; all threads of the CTA must
 * call (two __syncthreads inside). */
__device__ inline void split_phase(float *partial_m, float *partial_l, float *partial_acc,
                                   __nv_bfloat16 *out, float *lse,
                                   const __nv_bfloat16 *q_prepared, const __nv_bfloat16 *cache_k,
                                   const __nv_bfloat16 *cache_v, const Gemma4KvCacheConfig &cfg,
                                   const int32_t *page_table, const int32_t *seq_lengths,
                                   int32_t cache_layer, float softmax_scale, int32_t split_size,
                                   int32_t num_splits, int32_t q_heads, int batch, int kv_head,
                                   int split, float *smem, int thread_idx, int thread_count) {
  const int warp = thread_idx >> 5;
  const int lane = thread_idx & 31;
  const int warps = thread_count >> 5;
  const int len = seq_lengths[batch];
  const int first = cfg.window_size > 0 ? max(0, len - cfg.window_size) : 0;
  const int count = max(0, len - first);
  const int actual_splits = (count + split_size - 1) / split_size;
  if (split >= actual_splits && !(num_splits == 1 && split == 0)) return;
  const int k0 = first + split * split_size;
  const int k1 = min(len, k0 + split_size);

  // q of the two heads, 8 dims per lane, scaled into the exp2 domain
  float qf[kGroup][8];
  const float scale_log2 = softmax_scale * 1.4426950408889634f;
#pragma unroll
  for (int g = 0; g < kGroup; ++g) {
    const uint4 raw = __ldcg(reinterpret_cast<const uint4 *>(
                                 q_prepared + (int64_t(batch) * q_heads + kv_head * kGroup + g) * kDim) +
                             lane);
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      qf[g][2 * i] = detail::bf16_lo(w[i]) * scale_log2;
      qf[g][2 * i + 1] = detail::bf16_hi(w[i]) * scale_log2;
    }
  }
  float m[kGroup] = {-INFINITY, -INFINITY};
  float l[kGroup] = {0.0f, 0.0f};
  float acc[kGroup][8];
#pragma unroll
  for (int g = 0; g < kGroup; ++g) {
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[g][i] = 0.0f;
  }
  // Groups of four keys per warp step: the eight row loads of a step are in
  // flight together; a key of an unmapped page is skipped.
  for (int base = k0 + warp * 4; base < k1; base += warps * 4) {
    uint4 kk[4], vv[4];
    bool live[4];
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const int pos = base + t;
      live[t] = false;
      if (pos < k1) {
        const int page = detail::physical_page(cfg, page_table, batch, pos);
        if (page >= 0) {
          const int64_t off = gemma4_kv_cache_offset(
              cfg, cache_layer, page, pos - (pos / cfg.page_size) * cfg.page_size, kv_head, 0);
          kk[t] = __ldcg(reinterpret_cast<const uint4 *>(cache_k + off) + lane);
          vv[t] = __ldcg(reinterpret_cast<const uint4 *>(cache_v + off) + lane);
          live[t] = true;
        }
      }
    }
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      if (!live[t]) continue;  // uniform across the warp
      const uint32_t kw[4] = {kk[t].x, kk[t].y, kk[t].z, kk[t].w};
      float s[kGroup] = {0.0f, 0.0f};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float lo = detail::bf16_lo(kw[i]);
        const float hi = detail::bf16_hi(kw[i]);
#pragma unroll
        for (int g = 0; g < kGroup; ++g) {
          s[g] = fmaf(qf[g][2 * i], lo, s[g]);
          s[g] = fmaf(qf[g][2 * i + 1], hi, s[g]);
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        s[0] += __shfl_xor_sync(0xffffffffu, s[0], o);
        s[1] += __shfl_xor_sync(0xffffffffu, s[1], o);
      }
      const uint32_t vw[4] = {vv[t].x, vv[t].y, vv[t].z, vv[t].w};
#pragma unroll
      for (int g = 0; g < kGroup; ++g) {
        const float top = fmaxf(m[g], s[g]);
        const float corr = detail::ex2(m[g] - top);  // 0 for the first key
        const float p = detail::ex2(s[g] - top);
        l[g] = fmaf(l[g], corr, p);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          acc[g][2 * i] = fmaf(p, detail::bf16_lo(vw[i]), acc[g][2 * i] * corr);
          acc[g][2 * i + 1] = fmaf(p, detail::bf16_hi(vw[i]), acc[g][2 * i + 1] * corr);
        }
        m[g] = top;
      }
    }
  }
  // The warps' states meet in shared memory; thread t finishes dims t, t + thread_count, ...
  float *w_acc = smem + warp * kSplitSmemFloatsPerWarp;
#pragma unroll
  for (int g = 0; g < kGroup; ++g) {
#pragma unroll
    for (int i = 0; i < 8; ++i) w_acc[g * kDim + lane * 8 + i] = acc[g][i];
    if (lane == 0) {
      w_acc[kGroup * kDim + g] = m[g];
      w_acc[kGroup * kDim + kGroup + g] = l[g];
    }
  }
  __syncthreads();
  for (int e = thread_idx; e < kGroup * kDim; e += thread_count) {
    const int g = e / kDim;
    const int d = e - g * kDim;
    float top = -INFINITY;
    for (int w = 0; w < warps; ++w) {
      top = fmaxf(top, smem[w * kSplitSmemFloatsPerWarp + kGroup * kDim + g]);
    }
    float sum = 0.0f, value = 0.0f;
    for (int w = 0; w < warps; ++w) {
      const float *ws = smem + w * kSplitSmemFloatsPerWarp;
      const float mw = ws[kGroup * kDim + g];
      const float wt = mw == -INFINITY ? 0.0f : detail::ex2(mw - top);
      sum = fmaf(ws[kGroup * kDim + kGroup + g], wt, sum);
      value = fmaf(ws[g * kDim + d], wt, value);
    }
    const int64_t row = int64_t(batch) * q_heads + kv_head * kGroup + g;
    if (num_splits == 1) {
      out[row * kDim + d] = __float2bfloat16_rn(sum > 0.0f ? value / sum : 0.0f);
      if (lse != nullptr && d == 0) {
        lse[row] = sum > 0.0f ? (top + detail::lg2(sum)) * 0.6931471805599453f : -INFINITY;
      }
    } else {
      const int64_t slot = row * num_splits + split;
      partial_acc[slot * kDim + d] = value;
      if (d == 0) {
        partial_m[slot] = top;
        partial_l[slot] = sum;
      }
    }
  }
  __syncthreads();  // smem may be reused by the caller's next task
}

/* Combine of the splits of one output row (batch, q_head): M = max m_s,
 * L = sum l_s 2^(m_s - M) over the live splits (recomputed from seq_lengths as
 * the reference does, src/...decode.cu:910-916), out = sum acc_s 2^(m_s - M) / L
 * as bf16, zero rows without a live split; lse (natural log) if not null. With
 * num_splits == 1 the split phase has written the row already and this returns.
 * No shared memory, no barrier. */
__device__ inline void reduce_phase(__nv_bfloat16 *out, float *lse, const float *partial_m,
                                    const float *partial_l, const float *partial_acc,
                                    const Gemma4KvCacheConfig &cfg, const int32_t *seq_lengths,
                                    int32_t split_size, int32_t num_splits, int32_t q_heads,
                                    int batch, int q_head, int thread_idx, int thread_count) {
  if (num_splits == 1) return;
  const int len = seq_lengths[batch];
  const int first = cfg.window_size > 0 ? max(0, len - cfg.window_size) : 0;
  const int count = max(0, len - first);
  const int live = min((count + split_size - 1) / split_size, num_splits);
  const int64_t row = int64_t(batch) * q_heads + q_head;
  float top = -INFINITY;
  for (int s = 0; s < live; ++s) {
    if (__ldcg(partial_l + row * num_splits + s) > 0.0f) {
      top = fmaxf(top, __ldcg(partial_m + row * num_splits + s));
    }
  }
  float sum = 0.0f;
  for (int s = 0; s < live; ++s) {
    const float ls = __ldcg(partial_l + row * num_splits + s);
    if (ls > 0.0f) sum = fmaf(ls, detail::ex2(__ldcg(partial_m + row * num_splits + s) - top), sum);
  }
  for (int d = thread_idx; d < kDim; d += thread_count) {
    float value = 0.0f;
    for (int s = 0; s < live; ++s) {
      const int64_t slot = row * num_splits + s;
      if (__ldcg(partial_l + slot) > 0.0f) {
        value = fmaf(__ldcg(partial_acc + slot * kDim + d),
                     detail::ex2(__ldcg(partial_m + slot) - top), value);
      }
    }
    out[row * kDim + d] = __float2bfloat16_rn(sum > 0.0f ? value / sum : 0.0f);
  }
  if (lse != nullptr && thread_idx == 0) {
    lse[row] = sum > 0.0f ? (top + detail::lg2(sum)) * 0.6931471805599453f : -INFINITY;
  }
}

}  // namespace b200kv_device

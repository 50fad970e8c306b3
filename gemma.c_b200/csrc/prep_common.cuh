// Per-head prep arithmetic (RMSNorm + split-half RoPE) shared by the bf16 and
// fp8 append kernels. One warp owns one head; lane l holds elements l + 32*i
// (the reference's ownership, src/gemma4_flash_attention_decode.cu:216-227),
// the sum of squares is an fma chain per lane followed by the xor butterfly
// 16,8,4,2,1 (src/gemma4_rmsnorm.cu:90-101, src/gemma4_cuda_utils.cuh:165-170)
// -- that order defines the bit pattern of the scale.
#pragma once

#include "common.cuh"

namespace b200kv {

constexpr float kRmsEps = 1.0e-6f;  // GEMMA4_RMS_NORM_EPS, src/gemma4.h:29

// The reference compiles its prep call sites with flush-to-zero multiplies
// and the shared norm/rope helpers without; the approx mode reproduces that
// split, the IEEE mode uses plain round-to-nearest everywhere.
template <bool kIeee>
__device__ __forceinline__ float mul_prep(float a, float b) {
  if constexpr (kIeee) {
    return __fmul_rn(a, b);
  } else {
    float r;
    asm("mul.ftz.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
    return r;
  }
}

template <int D, bool kIeee>
__device__ __forceinline__ float warp_rms_scale(const float (&x)[D / 32]) {
  float ss = 0.0f;
#pragma unroll
  for (int i = 0; i < D / 32; ++i) ss = __fmaf_rn(x[i], x[i], ss);
#pragma unroll
  for (int offset = 16; offset > 0; offset /= 2) {
    ss = __fadd_rn(ss, __shfl_xor_sync(0xffffffffu, ss, offset));
  }
  const float t = __fadd_rn(__fdiv_rn(ss, float(D)), kRmsEps);
  if constexpr (kIeee) {
    return __fdiv_rn(1.0f, __fsqrt_rn(t));
  } else {
    return rsqrtf(t);
  }
}

template <int D>
__device__ __forceinline__ void load_head(const __nv_bfloat16 *in, int lane,
                                          float (&x)[D / 32]) {
#pragma unroll
  for (int i = 0; i < D / 32; ++i) {
    x[i] = __bfloat162float(in[lane + i * 32]);
  }
}

// This lane's norm weights (elements lane + 32 i) and RoPE factors (dims
// lane + 32 i of the first ROT / 2) in registers.
template <int D, int ROT>
struct PrepTables {
  float w[D / 32];
  float c[ROT / 64];
  float s[ROT / 64];

  __device__ __forceinline__ void load_weight(const __nv_bfloat16 *weight,
                                              int lane) {
#pragma unroll
    for (int i = 0; i < D / 32; ++i) {
      w[i] = __bfloat162float(__ldg(weight + lane + i * 32));
    }
  }
  __device__ __forceinline__ void load_rope(const float *cos_row,
                                            const float *sin_row, int lane) {
#pragma unroll
    for (int i = 0; i < ROT / 64; ++i) {
      c[i] = __ldg(cos_row + lane + i * 32);
      s[i] = __ldg(sin_row + lane + i * 32);
    }
  }
};

// Learned-weight RMSNorm, then split-half RoPE on the first ROT dims; the
// bf16 results stay in registers, y[j] being element lane + 32*j.
template <int D, int ROT, bool kIeee>
__device__ __forceinline__ void prep_weighted_rope_tables(
    __nv_bfloat16 (&y)[D / 32], const float (&x)[D / 32],
    const PrepTables<D, ROT> &t) {
  constexpr int kPairs = ROT / 64;
  const float scale = warp_rms_scale<D, kIeee>(x);
#pragma unroll
  for (int i = 0; i < kPairs; ++i) {
    const float lo = mul_prep<kIeee>(mul_prep<kIeee>(x[i], scale), t.w[i]);
    const float hi =
        mul_prep<kIeee>(mul_prep<kIeee>(x[i + kPairs], scale), t.w[i + kPairs]);
    y[i] = __float2bfloat16_rn(__fmaf_rn(-hi, t.s[i], __fmul_rn(lo, t.c[i])));
    y[i + kPairs] = __float2bfloat16_rn(__fmaf_rn(lo, t.s[i], __fmul_rn(hi, t.c[i])));
  }
#pragma unroll
  for (int i = 2 * kPairs; i < D / 32; ++i) {  // dims >= ROT: no rotation
    y[i] = __float2bfloat16_rn(mul_prep<kIeee>(mul_prep<kIeee>(x[i], scale), t.w[i]));
  }
}

template <int D, int ROT, bool kIeee>
__device__ __forceinline__ void prep_weighted_rope_values(
    __nv_bfloat16 (&y)[D / 32], const float (&x)[D / 32],
    const __nv_bfloat16 *weight, const float *cos_row, const float *sin_row,
    int lane) {
  PrepTables<D, ROT> t;
  t.load_weight(weight, lane);
  t.load_rope(cos_row, sin_row, lane);
  prep_weighted_rope_tables<D, ROT, kIeee>(y, x, t);
}

template <int D>
__device__ __forceinline__ void store_head(__nv_bfloat16 *out,
                                           const __nv_bfloat16 (&y)[D / 32],
                                           int lane) {
#pragma unroll
  for (int i = 0; i < D / 32; ++i) out[lane + i * 32] = y[i];
}

template <int D, int ROT, bool kIeee>
__device__ __forceinline__ void prep_weighted_rope(
    __nv_bfloat16 *out, const float (&x)[D / 32], const __nv_bfloat16 *weight,
    const float *cos_row, const float *sin_row, int lane) {
  __nv_bfloat16 y[D / 32];
  prep_weighted_rope_values<D, ROT, kIeee>(y, x, weight, cos_row, sin_row, lane);
  store_head<D>(out, y, lane);
}

// Scale-free RMSNorm (V rows): no weight, no rotation.
template <int D, bool kIeee>
__device__ __forceinline__ void prep_scale_free_values(
    __nv_bfloat16 (&y)[D / 32], const float (&x)[D / 32]) {
  const float scale = warp_rms_scale<D, kIeee>(x);
#pragma unroll
  for (int i = 0; i < D / 32; ++i) {
    y[i] = __float2bfloat16_rn(mul_prep<kIeee>(x[i], scale));
  }
}

template <int D, bool kIeee>
__device__ __forceinline__ void prep_scale_free(__nv_bfloat16 *out,
                                                const float (&x)[D / 32],
                                                int lane) {
  __nv_bfloat16 y[D / 32];
  prep_scale_free_values<D, kIeee>(y, x);
  store_head<D>(out, y, lane);
}

}  // namespace b200kv

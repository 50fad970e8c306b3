// Decode projections either side of the KV path (batch rows of one token):
//
//   ingress  raw[q|k|v] = bf16( RMSNorm(x, w_in) . W_qkv[col] )   per column
//            (phase_decode_rmsnorm_project_bf16,
//             src/gemma4_flash_attention_decode.cu:447-496)
//   egress   o = bf16( attention_out . W_o[col] ), then by the last CTA
//            normed = RMSNorm(o, w_post), ffn_residual = x + normed,
//            ffn_x = RMSNorm(ffn_residual, w_pre_ffn)
//            (project_attention_out_post_attention, :35-129; the pre-FFN norm
//             of decode_megakernel_fused_layer_kernel, :1049-1058)
//
// Both are a row vector times a column-major bf16 matrix: every weight byte is
// read once, 2 flop per byte, so the bound is HBM bandwidth. One kernel serves
// both. A CTA owns a contiguous range of columns (= one contiguous byte range
// of the matrix); a producer warp streams it through a six-stage ring of
// shared memory with one bulk copy per column (cp.async.bulk, completion
// counted on an mbarrier, evict-first in L2, nothing multicast), starting
// before the preceding kernel has finished (the weights do not depend on it).
// Sixteen consumer warps each take one column of a stage.
//
// The sums are rounded to bf16, so the order of the fp32 additions decides
// bits. The reference adds in the order of its 512-thread block: thread t
// chains fmaf over the 8 elements of pack t (and t + 512, ...), each warp
// folds with __shfl_down 16..1, warp 0 folds the 16 warp sums the same way.
// Here one warp owns a column: lane l computes the chains of threads
// 32 v + l for all 16 "virtual warps" v, the 16 folds run together as a
// reduce-scatter with the same pairings (20 shuffles instead of 80), and the
// fold over v is four more xor steps. The results are the reference kernels'
// bits (checked against the reference's own code compiled for the same GPU).
#include <algorithm>

#include "common.cuh"
#include "kernels.cuh"
#include "prep_common.cuh"

namespace b200kv {
namespace {

constexpr int kProjConsumerWarps = 16;
constexpr int kProjConsumerThreads = kProjConsumerWarps * kWarpSize;  // 512
constexpr int kProjThreads = kProjConsumerThreads + kWarpSize;
constexpr int kProjStages = 6;
constexpr int kProjHidden = 3840;  // GEMMA4_HIDDEN_SIZE, src/gemma4.h:6
constexpr int kProjHiddenPacks = kProjHidden / 8;
constexpr uint32_t kFullMask = 0xffffffffu;

// NV: virtual warps that hold data (width / 256 per chain step);
// CH: packs chained per virtual thread (width 8192: packs t and t + 512).
template <int NV_, int CH_>
struct ProjTraits {
  static constexpr int NV = NV_;
  static constexpr int CH = CH_;
  static constexpr int kWidth = 256 * NV * CH;
  static constexpr int kColBytes = kWidth * 2;
  static constexpr int kStageCols = 4 / CH;  // 30 KB or 32 KB per stage
  static constexpr int kStageBytes = kStageCols * kColBytes;
  static constexpr int kGroups = kProjConsumerWarps / kStageCols;
  static constexpr int kRingBytes = kProjStages * kStageBytes;
  static constexpr int kXBytes = kWidth * 2;
  static constexpr int kSmem = kRingBytes + kXBytes;
  static_assert(kSmem + 2048 <= 227 * 1024, "one CTA per SM");
};

struct ProjParams {
  const __nv_bfloat16 *w = nullptr;   // [cols][width]
  const __nv_bfloat16 *x = nullptr;   // [rows][x_stride]
  int64_t x_stride = 0;
  const __nv_bfloat16 *input_norm_weight = nullptr;  // ingress only
  // Output: up to three tensors one after the other, [rows][seg0],
  // [rows][seg1 - seg0], [rows][cols - seg1] (the raw q, k and v rows; for one
  // row this is the reference's [q|k|v] scratch). seg0 = seg1 = cols: one tensor.
  __nv_bfloat16 *out = nullptr;
  int32_t seg0 = 0, seg1 = 0;
  int32_t rows = 0;
  int32_t cols = 0;
  int32_t norm_mode = 0;
  // egress tail, run by the CTA that finishes a row last
  const __nv_bfloat16 *residual_in = nullptr;  // [rows][hidden]
  const __nv_bfloat16 *post_norm_weight = nullptr;
  const __nv_bfloat16 *pre_ffn_norm_weight = nullptr;
  __nv_bfloat16 *normed_out = nullptr;
  __nv_bfloat16 *ffn_residual = nullptr;
  __nv_bfloat16 *ffn_x = nullptr;
  unsigned int *ticket = nullptr;  // [rows], zero between calls
  int32_t *status = nullptr;
};

__device__ __forceinline__ int64_t out_index(const ProjParams &p, int row,
                                             int col) {
  if (col < p.seg0) return int64_t(row) * p.seg0 + col;
  if (col < p.seg1) {
    return int64_t(p.rows) * p.seg0 + int64_t(row) * (p.seg1 - p.seg0) + (col - p.seg0);
  }
  return int64_t(p.rows) * p.seg1 + int64_t(row) * (p.cols - p.seg1) + (col - p.seg1);
}

__device__ __forceinline__ float xor_fold(float v) {
#pragma unroll
  for (int offset = 16; offset > 0; offset /= 2) {
    v = __fadd_rn(v, __shfl_xor_sync(kFullMask, v, offset));
  }
  return v;
}

__device__ __forceinline__ float pack_sum_sq(const uint4 &p, float ss) {
  const uint32_t w[4] = {p.x, p.y, p.z, p.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float lo = bf16_lo(w[i]), hi = bf16_hi(w[i]);
    ss = __fmaf_rn(lo, lo, ss);
    ss = __fmaf_rn(hi, hi, ss);
  }
  return ss;
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t *>(&v);
}

// Learned-weight RMSNorm of one hidden row held as one pack per thread
// (threads >= 480 hold nothing), in the order of gemma4_rmsnorm_row_bf16 run
// by 512 threads (src/gemma4_rmsnorm.cu:27-87): fma chain per pack, xor fold
// per warp, xor fold of the 16 warp sums with zeros in lanes 16..31.
// `red` is 16 floats of shared memory not used by anything else until the
// barrier inside has been passed by all 512 threads. `g` is this thread's pack
// of the weight (loaded by the caller ahead of the values: it never depends on
// a preceding kernel).
__device__ __forceinline__ uint4 hidden_rmsnorm_pack(
    const uint4 &values, const uint4 &g, float *red, int thread,
    int norm_mode) {
  const int lane = thread & 31, warp = thread >> 5;
  float ss = 0.0f;
  if (thread < kProjHiddenPacks) ss = pack_sum_sq(values, ss);
  ss = xor_fold(ss);
  if (lane == 0) red[warp] = ss;
  named_barrier_sync(1, kProjConsumerThreads);
  float total = lane < kProjConsumerWarps ? red[lane] : 0.0f;
  total = xor_fold(total);
  const float t = __fadd_rn(__fdiv_rn(total, float(kProjHidden)), kRmsEps);
  const float scale = norm_mode == B200KV_NORM_IEEE
                          ? __fdiv_rn(1.0f, __fsqrt_rn(t))
                          : rsqrtf(t);
  uint4 result = make_uint4(0, 0, 0, 0);
  if (thread < kProjHiddenPacks) {
    const uint32_t v[4] = {values.x, values.y, values.z, values.w};
    const uint32_t gw[4] = {g.x, g.y, g.z, g.w};
    uint32_t r[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float lo = __fmul_rn(__fmul_rn(bf16_lo(v[i]), scale), bf16_lo(gw[i]));
      const float hi = __fmul_rn(__fmul_rn(bf16_hi(v[i]), scale), bf16_hi(gw[i]));
      r[i] = pack_bf16x2(lo, hi);
    }
    result = make_uint4(r[0], r[1], r[2], r[3]);
  }
  return result;
}

__device__ __forceinline__ uint4 load_hidden_pack(const __nv_bfloat16 *row,
                                                  int thread) {
  return thread < kProjHiddenPacks
             ? __ldg(reinterpret_cast<const uint4 *>(row) + thread)
             : make_uint4(0, 0, 0, 0);
}

// One column: this lane's 16 chain sums, folded in the block's order.
template <class T>
__device__ __forceinline__ float column_dot(uint32_t w_smem, uint32_t x_smem,
                                            int lane) {
  float p[16];
#pragma unroll
  for (int v = 0; v < 16; ++v) {
    float s = 0.0f;
    if (v < T::NV) {
#pragma unroll
      for (int j = 0; j < T::CH; ++j) {
        const uint32_t off = uint32_t((j * 512 + v * 32 + lane) * 16);
        const uint4 xv = lds128(x_smem + off);
        const uint4 wv = lds128(w_smem + off);
        const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
        const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          s = __fmaf_rn(bf16_lo(xw[i]), bf16_lo(ww[i]), s);
          s = __fmaf_rn(bf16_hi(xw[i]), bf16_hi(ww[i]), s);
        }
      }
    }
    p[v] = s;
  }
  // The 16 __shfl_down folds at once: at the step with offset o the pairing is
  // (lane, lane + o) as in the reference; which half of the values a lane
  // keeps is chosen by that lane bit, so afterwards lane l holds the sum of
  // virtual warp v = l / 2.
  const bool b4 = lane & 16, b3 = lane & 8, b2 = lane & 4, b1 = lane & 2;
  float y[8], z[4], u[2];
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const float send = b4 ? p[k] : p[k + 8];
    const float keep = b4 ? p[k + 8] : p[k];
    y[k] = __fadd_rn(keep, __shfl_xor_sync(kFullMask, send, 16));
  }
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float send = b3 ? y[k] : y[k + 4];
    const float keep = b3 ? y[k + 4] : y[k];
    z[k] = __fadd_rn(keep, __shfl_xor_sync(kFullMask, send, 8));
  }
#pragma unroll
  for (int k = 0; k < 2; ++k) {
    const float send = b2 ? z[k] : z[k + 2];
    const float keep = b2 ? z[k + 2] : z[k];
    u[k] = __fadd_rn(keep, __shfl_xor_sync(kFullMask, send, 4));
  }
  float s = __fadd_rn(b1 ? u[1] : u[0],
                      __shfl_xor_sync(kFullMask, b1 ? u[0] : u[1], 2));
  s = __fadd_rn(s, __shfl_xor_sync(kFullMask, s, 1));
  // Warp 0 of the reference: warp sums in lanes 0..15, zeros above, folded
  // with offsets 16 (adds the zero), 8, 4, 2, 1; v sits in lane bits 4..1.
  s = __fadd_rn(s, 0.0f);
#pragma unroll
  for (int offset = 16; offset > 1; offset /= 2) {
    s = __fadd_rn(s, __shfl_xor_sync(kFullMask, s, offset));
  }
  return s;
}

template <class T, bool kEgress>
__global__ void __launch_bounds__(kProjThreads, 1)
decode_projection_kernel(const ProjParams p) {
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ __align__(8) uint64_t full_bar[kProjStages];
  __shared__ __align__(8) uint64_t empty_bar[kProjStages];
  __shared__ float red[3][kProjConsumerWarps];
  __shared__ unsigned int last_flag;
  // Stages the producer has armed so far. A parity wait cannot tell phase k
  // from phase k - 2, and a consumer group may reach "stage n" before the data
  // of stage n - kProjStages (same slot, consumed by another group) has landed;
  // it therefore waits for the producer to have armed stage n first -- which
  // the producer does only after that earlier stage was consumed.
  __shared__ volatile int armed;

  const int thread = int(threadIdx.x);
  const int lane = thread & 31, warp = thread >> 5;
  const int row = int(blockIdx.y);
  const uint32_t ring = smem_u32(smem);
  const uint32_t x_smem = ring + T::kRingBytes;

  const int col_begin = int(int64_t(p.cols) * blockIdx.x / gridDim.x);
  const int col_end = int(int64_t(p.cols) * (blockIdx.x + 1) / gridDim.x);
  const int stages = div_up(col_end - col_begin, T::kStageCols);

  if (thread == 0) {
    armed = 0;
    for (int s = 0; s < kProjStages; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), T::kStageCols);
    }
    mbar_fence_init();
  }
  __syncthreads();

  if (warp == kProjConsumerWarps) {
    // Producer: the matrix does not depend on the preceding kernel.
    if (lane == 0) {
      const uint64_t policy = l2_policy_evict_first();
      for (int n = 0; n < stages; ++n) {
        const int slot = n % kProjStages;
        if (n >= kProjStages &&
            !mbar_wait_bounded(smem_u32(&empty_bar[slot]),
                               uint32_t(n / kProjStages - 1) & 1u)) {
          set_status(p.status, B200KV_STATUS_WAIT_TIMEOUT);
          break;
        }
        const int col = col_begin + n * T::kStageCols;
        const int count = min(T::kStageCols, col_end - col);
        const uint32_t bar = smem_u32(&full_bar[slot]);
        mbar_arrive_expect_tx(bar, uint32_t(count * T::kColBytes));
        for (int c = 0; c < count; ++c) {
          bulk_load_hint(ring + uint32_t(slot * T::kStageBytes + c * T::kColBytes),
                         p.w + int64_t(col + c) * T::kWidth,
                         uint32_t(T::kColBytes), bar, policy);
        }
        __threadfence_block();
        armed = n + 1;
      }
      // Leave only when every copy this thread issued has landed: a CTA must
      // not exit (a consumer may have given up on a wait) with bulk copies
      // still writing into its shared memory. The last kProjStages stages are
      // the ones that can still be in flight; nothing re-arms their barriers.
      const int issued = armed;
      for (int n = max(0, issued - kProjStages); n < issued; ++n) {
        if (!mbar_wait_bounded(smem_u32(&full_bar[n % kProjStages]),
                               uint32_t(n / kProjStages) & 1u)) {
          set_status(p.status, B200KV_STATUS_WAIT_TIMEOUT);
          break;
        }
      }
    }
    return;
  }

  // Consumers: the input row is the preceding kernel's output; the norm
  // weights and the layer input (the residual) are older than that.
  uint4 gamma0 = make_uint4(0, 0, 0, 0), gamma1 = gamma0, gamma2 = gamma0,
        resid = gamma0;
  if constexpr (!kEgress) {
    gamma0 = load_hidden_pack(p.input_norm_weight, thread);
  } else {
    gamma1 = load_hidden_pack(p.post_norm_weight, thread);
    if (p.ffn_x != nullptr) gamma2 = load_hidden_pack(p.pre_ffn_norm_weight, thread);
    resid = load_hidden_pack(p.residual_in + int64_t(row) * kProjHidden, thread);
  }
  pdl_wait_for_predecessor();
  pdl_release_successor();
  {
    const __nv_bfloat16 *x_row = p.x + int64_t(row) * p.x_stride;
    uint4 *x_rows = reinterpret_cast<uint4 *>(smem + T::kRingBytes);
    if constexpr (!kEgress) {
      uint4 values = make_uint4(0, 0, 0, 0);
      if (thread < kProjHiddenPacks) {
        values = *(reinterpret_cast<const uint4 *>(x_row) + thread);
      }
      const uint4 normed =
          hidden_rmsnorm_pack(values, gamma0, red[0], thread, p.norm_mode);
      if (thread < kProjHiddenPacks) x_rows[thread] = normed;
    } else {
      for (int pack = thread; pack < T::kWidth / 8; pack += kProjConsumerThreads) {
        x_rows[pack] = *(reinterpret_cast<const uint4 *>(x_row) + pack);
      }
    }
    named_barrier_sync(1, kProjConsumerThreads);
  }

  const int group = warp / T::kStageCols;
  const int cidx = warp % T::kStageCols;
  for (int n = group; n < stages; n += T::kGroups) {
    const int slot = n % kProjStages;
    bool ok = true;
    if (n >= kProjStages && armed <= n) {
      const long long start = clock64();
      while (armed <= n) {
        if (clock64() - start > kWaitClockLimit) {
          ok = false;
          break;
        }
        __nanosleep(32);
      }
    }
    __threadfence_block();
    if (!ok || !mbar_wait_bounded(smem_u32(&full_bar[slot]),
                                  uint32_t(n / kProjStages) & 1u)) {
      if (lane == 0) set_status(p.status, B200KV_STATUS_WAIT_TIMEOUT);
      break;
    }
    const int col = col_begin + n * T::kStageCols + cidx;
    if (col < col_end) {
      const float s = column_dot<T>(
          ring + uint32_t(slot * T::kStageBytes + cidx * T::kColBytes), x_smem,
          lane);
      if (lane == 0) p.out[out_index(p, row, col)] = __float2bfloat16_rn(s);
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(smem_u32(&empty_bar[slot]));
  }

  if constexpr (kEgress) {
    // The CTA that finishes a row last norms it and adds the residual. One
    // acquire-release ticket at device scope: the barrier before it orders the
    // CTA's column stores ahead of the release, the barrier after it orders the
    // acquire ahead of the last CTA's loads of everyone's columns.
    named_barrier_sync(1, kProjConsumerThreads);
    if (thread == 0) {
      unsigned int done;
      asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;"
                   : "=r"(done)
                   : "l"(p.ticket + row)
                   : "memory");
      last_flag = (done == gridDim.x - 1) ? 1u : 0u;
    }
    named_barrier_sync(1, kProjConsumerThreads);
    if (last_flag == 0u) return;
    uint4 o = make_uint4(0, 0, 0, 0);
    const int64_t base = int64_t(row) * kProjHidden;
    if (thread < kProjHiddenPacks) {
      o = __ldcg(reinterpret_cast<const uint4 *>(p.out + base) + thread);
    }
    const uint4 normed =
        hidden_rmsnorm_pack(o, gamma1, red[1], thread, p.norm_mode);
    uint4 sum = make_uint4(0, 0, 0, 0);
    if (thread < kProjHiddenPacks) {
      const uint32_t a[4] = {resid.x, resid.y, resid.z, resid.w};
      const uint32_t b[4] = {normed.x, normed.y, normed.z, normed.w};
      uint32_t r[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {  // gemma4_bf16_pack_add, cuda_utils.cuh:105-122
        r[i] = pack_bf16x2(__fadd_rn(bf16_lo(a[i]), bf16_lo(b[i])),
                           __fadd_rn(bf16_hi(a[i]), bf16_hi(b[i])));
      }
      sum = make_uint4(r[0], r[1], r[2], r[3]);
      *(reinterpret_cast<uint4 *>(p.normed_out + base) + thread) = normed;
      *(reinterpret_cast<uint4 *>(p.ffn_residual + base) + thread) = sum;
    }
    if (p.ffn_x != nullptr) {
      const uint4 fx =
          hidden_rmsnorm_pack(sum, gamma2, red[2], thread, p.norm_mode);
      if (thread < kProjHiddenPacks) {
        *(reinterpret_cast<uint4 *>(p.ffn_x + base) + thread) = fx;
      }
    }
    if (thread == 0) p.ticket[row] = 0u;  // ready for the next call
  }
}

template <class T, bool kEgress>
cudaError_t launch_projection(const ProjParams &p, int rows,
                              cudaStream_t stream) {
  int device = 0, sm_count = 0;
  cudaError_t st = cudaGetDevice(&device);
  if (st != cudaSuccess) return st;
  st = cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device);
  if (st != cudaSuccess) return st;
  const int ctas = std::max(1, std::min(sm_count, p.cols / T::kStageCols));
  st = cudaFuncSetAttribute(decode_projection_kernel<T, kEgress>,
                            cudaFuncAttributeMaxDynamicSharedMemorySize, T::kSmem);
  if (st != cudaSuccess) return st;
  return launch_pdl(decode_projection_kernel<T, kEgress>,
                    dim3(unsigned(ctas), unsigned(rows)), dim3(kProjThreads),
                    size_t(T::kSmem), stream, p);
}

bool aligned16(const void *ptr) {
  return (reinterpret_cast<uintptr_t>(ptr) & 15u) == 0;
}

}  // namespace

cudaError_t decode_ingress_bf16(const IngressArgs &a, cudaStream_t stream) {
  if (a.rows == 0) return cudaSuccess;
  if (a.rows < 0 || a.raw_qkv == nullptr || a.x == nullptr ||
      a.input_norm_weight == nullptr || a.qkv_proj_col_major == nullptr ||
      a.hidden != kProjHidden || a.cols <= 0 || a.cols % 8 != 0 ||
      a.q_width <= 0 || a.k_width < 0 || a.q_width + a.k_width > a.cols ||
      a.q_width % 8 != 0 || a.k_width % 8 != 0 ||
      !aligned16(a.raw_qkv) || !aligned16(a.x) || !aligned16(a.input_norm_weight) ||
      !aligned16(a.qkv_proj_col_major) ||
      (a.norm_mode != B200KV_NORM_RSQRT_APPROX && a.norm_mode != B200KV_NORM_IEEE)) {
    return cudaErrorInvalidValue;
  }
  ProjParams p;
  p.w = a.qkv_proj_col_major;
  p.x = a.x;
  p.x_stride = kProjHidden;
  p.input_norm_weight = a.input_norm_weight;
  p.out = a.raw_qkv;
  p.seg0 = a.q_width;
  p.seg1 = a.q_width + a.k_width;
  p.rows = a.rows;
  p.cols = a.cols;
  p.norm_mode = a.norm_mode;
  p.status = a.status;
  return launch_projection<ProjTraits<15, 1>, false>(p, a.rows, stream);
}

cudaError_t decode_egress_bf16(const EgressArgs &a, cudaStream_t stream) {
  if (a.rows == 0) return cudaSuccess;
  if (a.rows < 0 || a.residual_out == nullptr || a.normed_out == nullptr ||
      a.ffn_residual == nullptr || a.attention_out == nullptr ||
      a.o_proj_col_major == nullptr || a.post_norm_weight == nullptr ||
      a.x == nullptr || a.ticket == nullptr || a.hidden != kProjHidden ||
      (a.ffn_x != nullptr && a.pre_ffn_norm_weight == nullptr) ||
      (a.attention_width != 4096 && a.attention_width != 8192) ||
      !aligned16(a.residual_out) || !aligned16(a.normed_out) ||
      !aligned16(a.ffn_residual) || !aligned16(a.ffn_x) ||
      !aligned16(a.attention_out) || !aligned16(a.o_proj_col_major) ||
      !aligned16(a.post_norm_weight) || !aligned16(a.pre_ffn_norm_weight) ||
      !aligned16(a.x) ||
      (a.norm_mode != B200KV_NORM_RSQRT_APPROX && a.norm_mode != B200KV_NORM_IEEE)) {
    return cudaErrorInvalidValue;
  }
  ProjParams p;
  p.w = a.o_proj_col_major;
  p.x = a.attention_out;
  p.x_stride = a.attention_width;
  p.out = a.residual_out;
  p.seg0 = p.seg1 = kProjHidden;
  p.rows = a.rows;
  p.cols = kProjHidden;
  p.norm_mode = a.norm_mode;
  p.residual_in = a.x;
  p.post_norm_weight = a.post_norm_weight;
  p.pre_ffn_norm_weight = a.pre_ffn_norm_weight;
  p.normed_out = a.normed_out;
  p.ffn_residual = a.ffn_residual;
  p.ffn_x = a.ffn_x;
  p.ticket = a.ticket;
  p.status = a.status;
  if (a.attention_width == 4096) {
    return launch_projection<ProjTraits<16, 1>, true>(p, a.rows, stream);
  }
  return launch_projection<ProjTraits<16, 2>, true>(p, a.rows, stream);
}

}  // namespace b200kv

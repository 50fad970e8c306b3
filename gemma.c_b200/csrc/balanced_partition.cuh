// What the kernels with the evenly balanced key partition share: the launch
// parameters, the partition itself (prefix sums of the live keys, one contiguous
// range of the flattened keys per CTA, the walk over the pieces of a range) and
// the combine kernel that merges the partials of the CTAs that touched a
// sequence. Used by decode_balanced.cu (8 KV heads x 256, bf16 and fp8) and
// decode_gqa16.cu (1 KV head x 512, 16 query heads).
#pragma once

#include <algorithm>

#include "decode_common.cuh"
#include "kernels.cuh"

namespace b200kv {

constexpr int kMaxBalancedBatch = 1024;  // live-key prefix sums live in smem
// Second instantiation of the fused kernel for small batches: 8 KiB less
// shared memory, which is what lets a CTA of the next layer-step's kernel (and
// a waiting combine CTA) share an SM with a CTA of this one.
constexpr int kSmallBalancedBatch = 64;
constexpr int kMinKeysPerCta = 8;        // below this a CTA is all latency

struct BalancedParams {
  __nv_bfloat16 *out;
  float *lse;
  const __nv_bfloat16 *q;
  const void *cache_k;     // bf16 or e4m3 rows, Layout-A
  const void *cache_v;
  const float *scale_k;    // fp8 only: [layer, page, head]
  const float *scale_v;
  Gemma4KvCacheConfig cfg;
  const int32_t *page_table;
  const int32_t *seq_lengths;
  int32_t layer;
  float scale_log2;
  int32_t batch_count;
  int32_t q_heads;
  float *partial_m;
  float *partial_l;
  float *partial_acc;
  int32_t num_ctas;  // CTAs of the split kernel (the combine recomputes ranges)
  int32_t *status;
  // Fused kernels only: this step's projections and what the append needs to
  // prepare them; the kernel writes the new cache rows and the prepared q.
  const __nv_bfloat16 *raw_q;
  const __nv_bfloat16 *raw_k;
  const __nv_bfloat16 *raw_v;  // nullptr: V is derived from raw K
  const __nv_bfloat16 *q_norm_weight;
  const __nv_bfloat16 *k_norm_weight;
  const float *cos;
  const float *sin;
  const int32_t *token_position;
  __nv_bfloat16 *q_prepared;
  // Non-zero: raw_q / raw_k / raw_v are written by the kernel launched just
  // before this one (the QKV projection), so the consumer warps wait for it
  // before they read a raw row; the key stream of the producer warp is not held.
  int32_t raw_from_predecessor;
};

enum : int { kAttentionOnly = 0, kFusedApprox = 1, kFusedIeee = 2 };
constexpr int kAppendBufferBytesPerWarp = 1024;

__device__ __forceinline__ int range_width(int total, int num_ctas, int tile) {
  const int even = div_up(div_up(total, num_ctas), tile) * tile;
  return max(kMinKeysPerCta, even);
}

// Exclusive prefix sums of the live key counts into s_prefix[0..batch] and the
// first live position of each sequence into s_first[0..batch). All threads of
// the CTA call it; returns after a barrier.
template <int kMaxBatch>
__device__ void scan_live_keys(const BalancedParams &p, int *s_prefix,
                               int *s_first, int *s_warp_sums) {
  const int tid = int(threadIdx.x);
  const int nthreads = int(blockDim.x);
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int per_thread = div_up(p.batch_count, nthreads);
  const int b0 = tid * per_thread;
  int counts[kMaxBatch / 256 + 1];
  int sum = 0;
  for (int i = 0; i < per_thread && i < int(sizeof(counts) / sizeof(int)); ++i) {
    const int b = b0 + i;
    int n = 0;
    if (b < p.batch_count) {
      const int len = __ldg(p.seq_lengths + b);
      const int first = p.cfg.window_size > 0 ? max(0, len - p.cfg.window_size) : 0;
      n = max(0, len - first);
      s_first[b] = first;
    }
    counts[i] = n;
    sum += n;
  }
  int incl = sum;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int t = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += t;
  }
  if (lane == 31) s_warp_sums[warp] = incl;
  __syncthreads();
  int offset = incl - sum;
  for (int w = 0; w < warp; ++w) offset += s_warp_sums[w];
  for (int i = 0; i < per_thread && i < int(sizeof(counts) / sizeof(int)); ++i) {
    const int b = b0 + i;
    if (b < p.batch_count) s_prefix[b] = offset;
    offset += counts[i];
  }
  if (tid == nthreads - 1) s_prefix[p.batch_count] = offset;
  __syncthreads();
}

struct Segment {
  int b;      // sequence
  int pos0;   // first key position of the piece
  int pos1;   // one past the last
  bool whole; // the piece is the sequence's entire live range
};

// Next piece of the flattened range [flat, r1): the part of one sequence.
__device__ __forceinline__ bool next_segment(int &b, int &flat, int r1,
                                             const int *s_prefix,
                                             const int *s_first, Segment &seg) {
  if (flat >= r1) return false;
  while (s_prefix[b + 1] <= flat) ++b;  // sequences already done or empty
  const int end = min(r1, s_prefix[b + 1]);
  seg.b = b;
  seg.pos0 = s_first[b] + (flat - s_prefix[b]);
  seg.pos1 = s_first[b] + (end - s_prefix[b]);
  seg.whole = flat == s_prefix[b] && end == s_prefix[b + 1];
  flat = end;
  return true;
}

// Combine of the balanced kernels: a CTA takes (row, slice) items -- one when
// the grid has a CTA per item, several in turn when it does not -- recomputes
// which CTAs touched the row's sequence from the same prefix sums and combines
// their partials; rows that one CTA finished alone are left as they are; empty
// rows are zeroed.
template <int D, int kSlices, int kThreads>
__global__ __launch_bounds__(kThreads) void balanced_combine_kernel(
    BalancedParams p, int tile) {
  __shared__ float s_w[kCombineChunk];
  __shared__ float s_red[kThreads / 32];
  __shared__ float4 s_val[kThreads];
  __shared__ int s_sum[3][kThreads / 32];
  const int tid = int(threadIdx.x);
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int items = p.batch_count * p.q_heads * kSlices;

  pdl_release_successor();

  for (int item = int(blockIdx.x); item < items; item += int(gridDim.x)) {
    const int row = item / kSlices;
    const int slice = item - row * kSlices;
    const int b = row / p.q_heads;
    const int q_head = row - b * p.q_heads;
    int before = 0, all = 0, mine = 0;
    for (int i = tid; i < p.batch_count; i += kThreads) {
      const int len = __ldg(p.seq_lengths + i);
      const int first = p.cfg.window_size > 0 ? max(0, len - p.cfg.window_size) : 0;
      const int n = max(0, len - first);
      all += n;
      if (i < b) before += n;
      if (i == b) mine = n;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      before += __shfl_xor_sync(0xffffffffu, before, o);
      all += __shfl_xor_sync(0xffffffffu, all, o);
      mine += __shfl_xor_sync(0xffffffffu, mine, o);
    }
    if (lane == 0) {
      s_sum[0][warp] = before;
      s_sum[1][warp] = all;
      s_sum[2][warp] = mine;
    }
    __syncthreads();
    before = all = mine = 0;
#pragma unroll
    for (int w = 0; w < kThreads / 32; ++w) {
      before += s_sum[0][w];
      all += s_sum[1][w];
      mine += s_sum[2][w];
    }
    __syncthreads();  // s_sum is rewritten by the next item

    // The lengths were final before the attention kernel started; its
    // partials and directly written rows are not.
    pdl_wait_for_predecessor();
    __nv_bfloat16 *out_row = p.out + int64_t(row) * D;
    float *lse_row = p.lse != nullptr ? p.lse + row : nullptr;
    if (mine == 0) {
      combine_empty_row<D, kSlices>(out_row, lse_row, slice);
      continue;
    }
    const int width = range_width(all, p.num_ctas, tile);
    const int c_first = before / width;
    const int c_last = (before + mine - 1) / width;
    if (c_first == c_last) continue;  // finished by that CTA
    combine_row<D, kSlices, kThreads>(
        out_row, lse_row, p.partial_m, p.partial_l, p.partial_acc,
        int64_t(c_first + b) * p.q_heads + q_head, p.q_heads,
        c_last - c_first + 1, slice, s_w, s_red, s_val);
  }
}

// Launch of the combine for `p` (after the attention kernel, same stream).
template <int D>
cudaError_t launch_balanced_combine(const BalancedParams &p, int tile,
                                    cudaStream_t stream) {
  const int64_t rows = int64_t(p.batch_count) * p.q_heads;
  switch (combine_shape(rows)) {
    case 0:
      return launch_pdl(balanced_combine_kernel<D, 4, 256>,
                        dim3(unsigned(rows * 4)), dim3(256), 0, stream, p, tile);
    case 1:
      return launch_pdl(balanced_combine_kernel<D, 4, 128>,
                        dim3(unsigned(rows * 4)), dim3(128), 0, stream, p, tile);
    default:
      return launch_pdl(balanced_combine_kernel<D, 1, 256>,
                        dim3(unsigned(rows)), dim3(256), 0, stream, p, tile);
  }
}

}  // namespace b200kv

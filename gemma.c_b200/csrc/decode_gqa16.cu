// Decode attention for the reference's native global-layer geometry: 16 query
// heads on ONE KV head of 512 dims (src/gemma4.h:19-21, Traits at
// src/gemma4_flash_attention_decode.cu:150-157). Every key row is shared by 16
// query rows, so QK^T and P*V are real 16-row tiles and run on the tensor
// cores (bf16 mma.sync m16n8k16, fp32 accumulate); with two query heads per KV
// head (the other geometry) they are not, and decode_balanced.cu keeps them on
// the CUDA cores. The kernel is still HBM-bound: 2 KiB per key against
// 32 KFLOP.
//
// Same partition, scratch layout, combine and programmatic-launch rules as
// decode_balanced.cu (balanced_partition.cuh). Per CTA: one producer warp and
// four consumer warps; a stage is 16 keys (K rows then V rows, 1 KiB each,
// copied in pairs of rows with 16 bytes of padding after each pair, see
// Gqa16Traits).
//   scores: warp w contracts dims [128 w, 128 w + 128) for all 16 keys (16
//           MMAs), the four partial 16 x 16 tiles are summed through shared
//           memory (one named barrier per stage, double-buffered);
//   softmax: every warp holds the full tile and does the same fp32 online
//           update (exp2 domain), P rounded to bf16 is the A operand of
//   P*V:    warp w owns output dims [128 w, 128 w + 128): 16 MMAs with V
//           fragments from ldmatrix.trans.
#include <cstring>

#include "balanced_partition.cuh"
#include "kernels.cuh"
#include "mma_common.cuh"

namespace b200kv {

namespace {

struct Gqa16Traits {
  static constexpr int D = 512;
  static constexpr int HQ = 16;
  static constexpr int kConsumerWarps = 4;
  static constexpr int kThreads = (kConsumerWarps + 1) * kWarpSize;
  static constexpr int kCtasPerSm = 2;
  static constexpr int kStageTokens = 16;
  static constexpr int kRowBytes = D * 2;             // one key, the one head
  // Rows sit in the stage in pairs: 2 KiB contiguous (one bulk copy when both
  // rows are wanted), then 16 bytes of padding. The 8 rows of an ldmatrix tile
  // then fall into 4 bank groups (2-way conflict) instead of 1 (8-way); single
  // padded rows would be conflict-free but need twice the bulk copies, and the
  // copy engine's rate per copy, not the banks, is what limits this kernel.
  static constexpr int kPairStride = 2 * kRowBytes + 16;
  static constexpr int kStageTensorBytes = (kStageTokens / 2) * kPairStride;
  static constexpr int kStageBytes = 2 * kStageTensorBytes;  // K then V
  static constexpr int kMetaBytes = 256;
  static constexpr int kRingBytes = kStages * kStageBytes + kMetaBytes;
  // partial score tiles: [buffer][warp][key half][lane][4 floats]
  static constexpr int kExchangeBytes = 2 * kConsumerWarps * 32 * 8 * 4;
  static constexpr int kMaxBatch = 256;
  static constexpr int kSmem =
      kRingBytes + kExchangeBytes + (2 * kMaxBatch + 1) * 4 + 16;
  static constexpr int kDimsPerWarp = D / kConsumerWarps;  // 128
};

// Byte offset of key row `key` inside a stage's K (or V) rows.
__device__ __forceinline__ uint32_t gqa16_row_offset(int key) {
  return uint32_t(key >> 1) * Gqa16Traits::kPairStride +
         uint32_t(key & 1) * Gqa16Traits::kRowBytes;
}

__device__ __forceinline__ void consumer_barrier() {
  asm volatile("bar.sync 1, %0;" ::"n"(Gqa16Traits::kConsumerWarps * 32)
               : "memory");
}

struct Gqa16Ring {
  using T = Gqa16Traits;
  uint8_t *smem;
  uint32_t base;
  __device__ explicit Gqa16Ring(uint8_t *p) : smem(p), base(smem_u32(p)) {}
  __device__ uint32_t full_bar(int s) const {
    return base + kStages * T::kStageBytes + 8u * uint32_t(s);
  }
  __device__ uint32_t empty_bar(int s) const {
    return base + kStages * T::kStageBytes + 8u * uint32_t(kStages + s);
  }
  __device__ uint32_t *masks() const {
    return reinterpret_cast<uint32_t *>(smem + kStages * T::kStageBytes +
                                        16 * kStages);
  }
  __device__ int *abort_flag() const {
    return reinterpret_cast<int *>(smem + kStages * T::kStageBytes +
                                   16 * kStages + 4 * kStages);
  }
  __device__ uint32_t k_stage(int s) const {
    return base + uint32_t(s) * T::kStageBytes;
  }
  __device__ void init() const {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), T::kConsumerWarps);
    }
    *abort_flag() = 0;
    mbar_fence_init();
  }
};

// Producer warp: lane i < 16 resolves the page of key base + i of the stage;
// an even lane whose neighbour's row is wanted too and follows it in memory
// copies both rows (K and V, 2 KiB each) at once, otherwise every wanted row
// is copied by its own lane (1 KiB each).
__device__ __forceinline__ void gqa16_fill_stage(const Gqa16Ring &ring,
                                                 const BalancedParams &p,
                                                 int batch, int base, int c0,
                                                 int c1, int stage,
                                                 uint64_t policy, int lane) {
  using T = Gqa16Traits;
  const Gemma4KvCacheConfig &cfg = p.cfg;
  const int pos = base + lane;
  long long off = -1;
  if (lane < T::kStageTokens && pos >= c0 && pos < c1) {
    const int lp = pos / cfg.page_size;
    const int slot = lp % cfg.max_pages_per_seq;
    const int phys =
        __ldg(p.page_table + int64_t(batch) * cfg.max_pages_per_seq + slot);
    if (phys >= 0 && phys < cfg.num_pages) {
      off = cache_offset(cfg, p.layer, phys, pos - lp * cfg.page_size, 0, 0);
    }
  }
  const uint32_t mask = __ballot_sync(0xffffffffu, off >= 0);
  const long long next_off = __shfl_down_sync(0xffffffffu, off, 1);
  const long long prev_off = __shfl_up_sync(0xffffffffu, off, 1);
  const bool pair_head =
      (lane & 1) == 0 && off >= 0 && next_off == off + T::D;
  const bool pair_tail = (lane & 1) == 1 && off >= 0 && prev_off == off - T::D;
  if (lane == 0) {
    ring.masks()[stage] = mask;
    if (mask != 0u) {
      mbar_arrive_expect_tx(ring.full_bar(stage),
                            uint32_t(__popc(mask)) * 2u * T::kRowBytes);
    } else {
      mbar_arrive(ring.full_bar(stage));
    }
  }
  __syncwarp();
  if (off >= 0 && !pair_tail) {
    const uint32_t bytes = pair_head ? 2u * T::kRowBytes : uint32_t(T::kRowBytes);
    const uint32_t dst = ring.k_stage(stage) + gqa16_row_offset(lane);
    bulk_load_hint(dst, static_cast<const __nv_bfloat16 *>(p.cache_k) + off,
                   bytes, ring.full_bar(stage), policy);
    bulk_load_hint(dst + T::kStageTensorBytes,
                   static_cast<const __nv_bfloat16 *>(p.cache_v) + off, bytes,
                   ring.full_bar(stage), policy);
  }
}

__global__ __launch_bounds__(Gqa16Traits::kThreads, Gqa16Traits::kCtasPerSm) void
decode_gqa16_kernel(BalancedParams p) {
  using T = Gqa16Traits;
  constexpr int ST = T::kStageTokens;
  extern __shared__ __align__(128) uint8_t smem[];
  float *exchange = reinterpret_cast<float *>(smem + T::kRingBytes);
  int *s_prefix =
      reinterpret_cast<int *>(smem + T::kRingBytes + T::kExchangeBytes);
  int *s_first = s_prefix + T::kMaxBatch + 1;
  __shared__ int s_warp_sums[32];

  const int warp = int(threadIdx.x) >> 5;
  const int lane = int(threadIdx.x) & 31;
  const Gemma4KvCacheConfig &cfg = p.cfg;

  // As the attention-only mode of decode_balanced_kernel: the preceding kernel
  // is this layer-step's append; lengths, page table and all cache rows but
  // those of the page with each sequence's newest key were complete before it
  // started. The prepared q and that page are touched after the wait; every
  // CTA waits before it exits.
  pdl_release_successor();

  // initialised under the scan's first load; its barriers publish them
  const Gqa16Ring ring(smem);
  if (threadIdx.x == 0) ring.init();
  scan_live_keys<T::kMaxBatch>(p, s_prefix, s_first, s_warp_sums);
  const int total = s_prefix[p.batch_count];
  const int width = range_width(max(total, 1), p.num_ctas, ST);
  const int r0 = int(blockIdx.x) * width;
  if (total == 0 || r0 >= total) {
    pdl_wait_for_predecessor();
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
    bool ok = true;
    bool waited = false;
    int it = 0;
    int b = b_start, flat = r0;
    Segment seg;
    while (ok && next_segment(b, flat, r1, s_prefix, s_first, seg)) {
      const int a0 = (seg.pos0 / ST) * ST;
      const int nchunks = div_up(seg.pos1 - a0, ST);
      const int seq_len = s_first[seg.b] + s_prefix[seg.b + 1] - s_prefix[seg.b];
      const int fresh = (max(seq_len - 1, 0) / cfg.page_size) * cfg.page_size;
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
        gqa16_fill_stage(ring, p, seg.b, base, max(seg.pos0, base),
                         min(seg.pos1, base + ST), stage, policy, lane);
      }
    }
    for (int s = 0; s < kStages && s < it; ++s) {
      const int fill = (it - 1 - s) / kStages;
      if (!mbar_wait_bounded(ring.full_bar(s), uint32_t(fill) & 1u)) ok = false;
    }
    if (!waited) pdl_wait_for_predecessor();
    if (!ok && lane == 0) set_status(p.status, B200KV_STATUS_WAIT_TIMEOUT);
    return;
  }

  // -------------------------------- consumers --------------------------------
  pdl_wait_for_predecessor();  // the prepared q comes from the append
  const int g = lane >> 2;     // fragment row (query heads g and g + 8)
  const int t = lane & 3;
  const int dim0 = warp * T::kDimsPerWarp;
  // ldmatrix row addresses of this lane, relative to a stage's K (V) rows
  const uint32_t k_lane_off =
      gqa16_row_offset(lane & 7) + uint32_t(dim0 + 8 * (lane >> 3)) * 2u;
  const uint32_t v_lane_off =
      gqa16_row_offset((lane & 7) + 8 * ((lane >> 3) & 1)) +
      uint32_t(dim0 + 8 * (lane >> 4)) * 2u;

  int b = b_start, flat = r0;
  Segment seg;
  int it = 0;
  int exchanges = 0;  // stages that went through the exchange (its buffer parity)
  while (next_segment(b, flat, r1, s_prefix, s_first, seg)) {
    // A fragments of q for this warp's 128 dims: 8 k-steps x 4 registers
    uint32_t qa[8][4];
    {
      const __nv_bfloat16 *q0 =
          p.q + (int64_t(seg.b) * T::HQ + g) * T::D + dim0 + 2 * t;
      const __nv_bfloat16 *q1 = q0 + 8 * T::D;
#pragma unroll
      for (int s = 0; s < 8; ++s) {
        qa[s][0] = *reinterpret_cast<const uint32_t *>(q0 + 16 * s);
        qa[s][1] = *reinterpret_cast<const uint32_t *>(q1 + 16 * s);
        qa[s][2] = *reinterpret_cast<const uint32_t *>(q0 + 16 * s + 8);
        qa[s][3] = *reinterpret_cast<const uint32_t *>(q1 + 16 * s + 8);
      }
    }
    float o[16][4];  // output tile: n-tile x (row g: 2 dims, row g + 8: 2 dims)
#pragma unroll
    for (int n = 0; n < 16; ++n) {
#pragma unroll
      for (int i = 0; i < 4; ++i) o[n][i] = 0.0f;
    }
    float m_run[2] = {-INFINITY, -INFINITY};  // rows g, g + 8 (exp2 domain)
    float l_run[2] = {0.0f, 0.0f};            // this lane's columns only

    const int a0 = (seg.pos0 / ST) * ST;
    const int nchunks = div_up(seg.pos1 - a0, ST);
    for (int c = 0; c < nchunks; ++c, ++it) {
      const int stage = it % kStages;
      const int fill = it / kStages;
      if (!mbar_wait_bounded(ring.full_bar(stage), uint32_t(fill) & 1u)) {
        *ring.abort_flag() = 1;  // the others learn of it at their next barrier
      }
      const uint32_t mask = ring.masks()[stage];
      if (mask != 0u) {
        const uint32_t k_base = ring.k_stage(stage);
        const uint32_t v_base = k_base + T::kStageTensorBytes;
        // ---- partial scores over this warp's dims
        float sc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
        for (int j = 0; j < 2; ++j) {
#pragma unroll
          for (int s2 = 0; s2 < 4; ++s2) {
            uint32_t kb[4];
            ldmatrix_x4(kb, k_base + gqa16_row_offset(8 * j) + k_lane_off +
                                uint32_t(32 * s2) * 2u);
            mma_bf16_m16n8k16(sc[j], qa[2 * s2][0], qa[2 * s2][1],
                              qa[2 * s2][2], qa[2 * s2][3], kb[0], kb[1]);
            mma_bf16_m16n8k16(sc[j], qa[2 * s2 + 1][0], qa[2 * s2 + 1][1],
                              qa[2 * s2 + 1][2], qa[2 * s2 + 1][3], kb[2],
                              kb[3]);
          }
        }
        // ---- sum of the four warps' partial tiles
        // (a write to a buffer comes after the barrier of the previous
        // exchange, which no warp passes before it has read this buffer's
        // previous contents)
        float *xw = exchange + ((exchanges & 1) * T::kConsumerWarps) * 256;
        ++exchanges;
        reinterpret_cast<float4 *>(xw + warp * 256)[lane] =
            make_float4(sc[0][0], sc[0][1], sc[0][2], sc[0][3]);
        reinterpret_cast<float4 *>(xw + warp * 256)[32 + lane] =
            make_float4(sc[1][0], sc[1][1], sc[1][2], sc[1][3]);
        consumer_barrier();
        if (*ring.abort_flag() != 0) {
          if (warp == 0 && lane == 0) {
            set_status(p.status, B200KV_STATUS_WAIT_TIMEOUT);
          }
          return;  // all four warps read the flag after the same barrier
        }
#pragma unroll
        for (int j = 0; j < 2; ++j) {
#pragma unroll
          for (int i = 0; i < 4; ++i) sc[j][i] = 0.0f;
        }
#pragma unroll
        for (int w = 0; w < T::kConsumerWarps; ++w) {
          const float4 u0 = reinterpret_cast<const float4 *>(xw + w * 256)[lane];
          const float4 u1 =
              reinterpret_cast<const float4 *>(xw + w * 256)[32 + lane];
          sc[0][0] += u0.x; sc[0][1] += u0.y; sc[0][2] += u0.z; sc[0][3] += u0.w;
          sc[1][0] += u1.x; sc[1][1] += u1.y; sc[1][2] += u1.z; sc[1][3] += u1.w;
        }
        // ---- online softmax; sc[j][0..1] are row g, sc[j][2..3] row g + 8,
        // keys 8 j + 2 t and 8 j + 2 t + 1
        float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int j = 0; j < 2; ++j) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int key = 8 * j + 2 * t + (i & 1);
            const bool live = ((mask >> key) & 1u) != 0u;
            sc[j][i] = live ? sc[j][i] * p.scale_log2 : -INFINITY;
            tile_max[i >> 1] = fmaxf(tile_max[i >> 1], sc[j][i]);
          }
        }
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(0xffffffffu, tile_max[r], 1));
          tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(0xffffffffu, tile_max[r], 2));
        }
        const float m_new[2] = {fmaxf(m_run[0], tile_max[0]),
                                fmaxf(m_run[1], tile_max[1])};
        if (m_new[0] > m_run[0] || m_new[1] > m_run[1]) {
          const float corr0 = ex2_approx(m_run[0] - m_new[0]);
          const float corr1 = ex2_approx(m_run[1] - m_new[1]);
#pragma unroll
          for (int n = 0; n < 16; ++n) {
            o[n][0] *= corr0;
            o[n][1] *= corr0;
            o[n][2] *= corr1;
            o[n][3] *= corr1;
          }
          l_run[0] *= corr0;
          l_run[1] *= corr1;
          m_run[0] = m_new[0];
          m_run[1] = m_new[1];
        }
        uint32_t pa[4];  // P as the A operand: keys 0..7 | 8..15, rows g | g + 8
        {
          const float p00 = ex2_approx(sc[0][0] - m_run[0]);
          const float p01 = ex2_approx(sc[0][1] - m_run[0]);
          const float p02 = ex2_approx(sc[0][2] - m_run[1]);
          const float p03 = ex2_approx(sc[0][3] - m_run[1]);
          const float p10 = ex2_approx(sc[1][0] - m_run[0]);
          const float p11 = ex2_approx(sc[1][1] - m_run[0]);
          const float p12 = ex2_approx(sc[1][2] - m_run[1]);
          const float p13 = ex2_approx(sc[1][3] - m_run[1]);
          l_run[0] += (p00 + p01) + (p10 + p11);
          l_run[1] += (p02 + p03) + (p12 + p13);
          pa[0] = pack_bf16x2(p00, p01);
          pa[1] = pack_bf16x2(p02, p03);
          pa[2] = pack_bf16x2(p10, p11);
          pa[3] = pack_bf16x2(p12, p13);
        }
        // ---- rows the copy did not bring may hold anything (0 x NaN is NaN):
        // this warp's slice of them is zeroed before it is multiplied
        if (mask != 0xffffu) {
          for (int key = 0; key < ST; ++key) {
            if (((mask >> key) & 1u) == 0u && lane < 16) {
              reinterpret_cast<uint4 *>(smem + stage * T::kStageBytes +
                                        T::kStageTensorBytes +
                                        gqa16_row_offset(key) + dim0 * 2)[lane] =
                  make_uint4(0u, 0u, 0u, 0u);
            }
          }
          fence_proxy_async_shared();  // the stage's next fill is a bulk copy
          __syncwarp();
        }
        // ---- P*V for this warp's 128 output dims
#pragma unroll
        for (int np = 0; np < 8; ++np) {
          uint32_t vb[4];
          ldmatrix_x4_trans(vb, v_base + v_lane_off + uint32_t(16 * np) * 2u);
          mma_bf16_m16n8k16(o[2 * np], pa[0], pa[1], pa[2], pa[3], vb[0], vb[1]);
          mma_bf16_m16n8k16(o[2 * np + 1], pa[0], pa[1], pa[2], pa[3], vb[2],
                            vb[3]);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(ring.empty_bar(stage));
    }

    // ---- the sequence's piece is done: final rows or a partial
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
      l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int head = g + 8 * r;
      const int64_t row = int64_t(seg.b) * T::HQ + head;
      if (seg.whole) {
        const float inv = l_run[r] > 0.0f ? 1.0f / l_run[r] : 0.0f;
        __nv_bfloat16 *dst = p.out + row * T::D + dim0 + 2 * t;
#pragma unroll
        for (int n = 0; n < 16; ++n) {
          *reinterpret_cast<uint32_t *>(dst + 8 * n) =
              pack_bf16x2(o[n][2 * r] * inv, o[n][2 * r + 1] * inv);
        }
        if (p.lse != nullptr && warp == 0 && t == 0) {
          p.lse[row] = l_run[r] > 0.0f
                           ? (m_run[r] + lg2_approx(l_run[r])) * 0.6931471805599453f
                           : -INFINITY;
        }
      } else {
        const int64_t slot = int64_t(int(blockIdx.x) + seg.b) * T::HQ + head;
        float *dst = p.partial_acc + slot * T::D + dim0 + 2 * t;
#pragma unroll
        for (int n = 0; n < 16; ++n) {
          *reinterpret_cast<float2 *>(dst + 8 * n) =
              make_float2(o[n][2 * r], o[n][2 * r + 1]);
        }
        if (warp == 0 && t == 0) {
          p.partial_m[slot] = m_run[r];
          p.partial_l[slot] = l_run[r];
        }
      }
    }
  }
}

}  // namespace

bool decode_gqa16_supported(const Gemma4KvCacheConfig &c, int q_heads,
                            int batch_count) {
  return c.head_dim == 512 && c.num_heads == 1 && q_heads == 16 &&
         batch_count <= Gqa16Traits::kMaxBatch;
}

cudaError_t decode_attention_gqa16_bf16(const DecodeArgs &a,
                                        cudaStream_t stream) {
  using T = Gqa16Traits;
  if (!decode_gqa16_supported(a.cfg, a.q_heads, a.batch_count)) {
    return cudaErrorInvalidValue;
  }
  static_assert(2 * (T::kSmem + 1024 + 256) <= 228 * 1024, "two CTAs per SM");
  static_assert(T::kRingBytes % 16 == 0 && T::kPairStride % 16 == 0, "alignment");
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
  int device = 0, sm_count = 0;
  cudaError_t st = cudaGetDevice(&device);
  if (st != cudaSuccess) return st;
  st = cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device);
  if (st != cudaSuccess) return st;
  const int64_t slots = int64_t(a.batch_count) * a.num_splits;
  const int64_t num_ctas = std::min<int64_t>(int64_t(sm_count) * T::kCtasPerSm,
                                             slots - a.batch_count);
  if (num_ctas < 1 || p.partial_m == nullptr || p.partial_l == nullptr ||
      p.partial_acc == nullptr) {
    return cudaErrorInvalidValue;
  }
  p.num_ctas = int32_t(num_ctas);
  st = cudaFuncSetAttribute(decode_gqa16_kernel,
                            cudaFuncAttributeMaxDynamicSharedMemorySize,
                            T::kSmem);
  if (st != cudaSuccess) return st;
  st = launch_pdl(decode_gqa16_kernel, dim3(unsigned(num_ctas)),
                  dim3(T::kThreads), T::kSmem, stream, p);
  if (st != cudaSuccess) return st;
  return launch_balanced_combine<T::D>(p, T::kStageTokens, stream);
}

}  // namespace b200kv

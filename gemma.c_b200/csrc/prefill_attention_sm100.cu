// Prompt attention on the fifth-generation tensor cores: tcgen05.mma with the
// accumulators (and the softmax weights) in tensor memory, tiles brought in by
// TMA. Same contract as prefill_attention.cu (which keeps the mma.sync path as
// the comparison arm): each sequence's query row r sees its own keys c <= r and,
// with a window, c >= r - window + 1 (src/gemma4_flash_attention_prefill.cu:502-540).
//
// Two geometries share one kernel template:
//   head_dim 256 (sliding layers): one CTA = 128 query rows of one query head,
//     key tiles of 128.
//   head_dim 512 (global layers): the 512 output dims do not fit tensor memory
//     beside the scores, so one CTA = 128 query rows of one query head and ONE
//     HALF of the output dims (256 of V's 512); the two CTAs of a head each
//     compute the full scores (Q K^T over 512 dims) and the same softmax, and
//     multiply by their own half of V. Key tiles of 64.
// Nineteen warps:
//   warps 0-15 softmax: four threads per query row, a quarter of the tile's key
//              columns each (the softmax is latency-bound per warp; 16 warps
//              hide it)
//   warp 16    one thread issues the TMA loads of Q (once) and of the K tiles
//   warp 17    one thread issues the MMAs and commits them to mbarriers
//   warp 18    one thread issues the TMA loads of the V tiles
// shared memory: Q (128 x head_dim), one K tile (keys x head_dim) and one V tile
//   (keys x 256), all bf16, all as column blocks of 64 elements (128 bytes per
//   row) in the 128-byte swizzle that both the tensor maps and the tcgen05 smem
//   descriptors name; K-major for Q and K, MN-major for V.
// tensor memory (512 columns): S[2] (128 lanes x tile keys fp32, double-buffered)
//   and O (128 x 256 fp32); lane = query row.
// per key tile: head_dim / 16 MMAs (M 128, N = tile keys, K 16) give S = Q K^T;
//   the softmax threads read their part of their row of S with tcgen05.ld, do the
//   online softmax without a shuffle (the four threads of a row exchange their
//   maxima through shared memory) and write the bf16 weights back over the
//   scores they read (two per 32-bit column); tile keys / 16 MMAs (M 128, N 256,
//   K 16) with P as the tensor-memory A operand add P V to O. K of the next tile
//   is loaded as soon as Q K^T of this one is done, and its scores are computed
//   while the threads do this tile's softmax; V of the next tile is loaded as
//   soon as P V of this one is done.
// The running maximum a row scales by is only raised when the tile's maximum
// exceeds it by more than 2^8 (the weights then stay below 256, exact enough in
// bf16 and fp32), so the rescaling of O in tensor memory is rare. The denominator
// sums the weights as rounded to bf16, the numbers P V uses.
//
// Every wait is bounded (tens of milliseconds: a tile takes microseconds). A
// wait that runs out records which one in a device-side fault word and raises
// the CTA's abort flag, which every other wait polls; all roles then fall
// through to the common exit, which waits (bounded) for the loads in flight and
// frees the tensor memory. CTAs that start later return at once. The host clears
// the word before each launch and reads it through prefill_attention_sm100_fault().
#include <cuda.h>

#include "common.cuh"
#include "kernels.cuh"

namespace b200kv {

namespace {

constexpr int kBlockM = 128;
constexpr int kDv = 256;                                // output dims per CTA
constexpr int kSoftmaxThreads = 512;
constexpr int kSoftmaxWarps = kSoftmaxThreads / 32;
constexpr int kThreads = kSoftmaxThreads + 96;
constexpr uint32_t kTmemColumns = 512;
constexpr float kRescaleSlack = 8.0f;                   // log2 units
constexpr long long kTileWaitClocks = 1ll << 26;        // ~35 ms

template <int kHeadDim_, int kBlockN_>
struct Sm100Traits {
  static constexpr int kHeadDim = kHeadDim_;            // contraction dims of Q K^T
  static constexpr int kBlockN = kBlockN_;              // keys per tile
  static constexpr int kQuarterN = kBlockN / 4;         // score columns per softmax thread
  static constexpr int kVSplits = kHeadDim / kDv;       // CTAs that share a head's scores
  static constexpr int kQBlockBytes = kBlockM * 128;    // 128 rows x 64 elements
  static constexpr int kKBlockBytes = kBlockN * 128;    // keys x 64 elements
  static constexpr int kQBytes = kBlockM * kHeadDim * 2;
  static constexpr int kKBytes = kBlockN * kHeadDim * 2;
  static constexpr int kVBytes = kBlockN * kDv * 2;
  static constexpr int kTileBytes = kQBytes + kKBytes + kVBytes;
  static constexpr uint32_t kTmemO = 2 * kBlockN;       // S[2] at 0 and kBlockN, O behind
  static_assert(kQuarterN == 32 || kQuarterN == 16, "tensor-memory access shapes");
  static_assert(kTmemO + kDv <= kTmemColumns, "tensor memory");
};

// 0, or which wait ran out: 1 softmax on scores, 2 softmax on P V, 3 loader,
// 4 MMA issuer, 5 last P V; 6: the shared-memory window was not 1024-byte aligned
__device__ int g_prefill_sm100_fault;

struct Sm100PrefillParams {
  __nv_bfloat16 *out;
  int32_t seq_len;
  int32_t q_heads;
  int32_t kv_heads;
  int32_t window;
  float scale_log2;
};

// Shared-memory matrix descriptor for a 128-byte-swizzled tile: start address
// and the two strides in 16-byte units, descriptor version 1, layout type 2.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr,
                                              uint32_t leading_units,
                                              uint32_t stride_units) {
  const uint32_t lo = ((smem_addr >> 4) & 0x3fffu) | (leading_units << 16);
  const uint32_t hi = (stride_units & 0x3fffu) | (1u << 14) | (2u << 29);
  return (uint64_t(hi) << 32) | lo;
}

// Instruction descriptor: fp32 accumulate, bf16 x bf16, M = 128.
__host__ __device__ constexpr uint32_t umma_idesc(uint32_t n, bool b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (b_mn_major ? (1u << 16) : 0u) |
         ((n >> 3) << 17) | ((128u >> 4) << 24);
}

__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc,
                                          uint64_t b_desc, uint32_t idesc,
                                          bool accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(uint32_t(accumulate))
      : "memory");
}
// The same with the A operand in tensor memory: lane = row, each 32-bit column
// two consecutive bf16 of the contraction dimension (8 columns per K = 16).
__device__ __forceinline__ void umma_bf16_a_tmem(uint32_t d_tmem, uint32_t a_tmem,
                                                 uint64_t b_desc, uint32_t idesc,
                                                 bool accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}\n" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(uint32_t(accumulate))
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile(
      "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
      : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float *r) {
  uint32_t u[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,"
      "%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(u[0]), "=r"(u[1]), "=r"(u[2]), "=r"(u[3]), "=r"(u[4]), "=r"(u[5]),
        "=r"(u[6]), "=r"(u[7]), "=r"(u[8]), "=r"(u[9]), "=r"(u[10]), "=r"(u[11]),
        "=r"(u[12]), "=r"(u[13]), "=r"(u[14]), "=r"(u[15]), "=r"(u[16]),
        "=r"(u[17]), "=r"(u[18]), "=r"(u[19]), "=r"(u[20]), "=r"(u[21]),
        "=r"(u[22]), "=r"(u[23]), "=r"(u[24]), "=r"(u[25]), "=r"(u[26]),
        "=r"(u[27]), "=r"(u[28]), "=r"(u[29]), "=r"(u[30]), "=r"(u[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) r[i] = __uint_as_float(u[i]);
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float *r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,"
      "%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};" ::"r"(taddr),
      "r"(__float_as_uint(r[0])), "r"(__float_as_uint(r[1])),
      "r"(__float_as_uint(r[2])), "r"(__float_as_uint(r[3])),
      "r"(__float_as_uint(r[4])), "r"(__float_as_uint(r[5])),
      "r"(__float_as_uint(r[6])), "r"(__float_as_uint(r[7])),
      "r"(__float_as_uint(r[8])), "r"(__float_as_uint(r[9])),
      "r"(__float_as_uint(r[10])), "r"(__float_as_uint(r[11])),
      "r"(__float_as_uint(r[12])), "r"(__float_as_uint(r[13])),
      "r"(__float_as_uint(r[14])), "r"(__float_as_uint(r[15])),
      "r"(__float_as_uint(r[16])), "r"(__float_as_uint(r[17])),
      "r"(__float_as_uint(r[18])), "r"(__float_as_uint(r[19])),
      "r"(__float_as_uint(r[20])), "r"(__float_as_uint(r[21])),
      "r"(__float_as_uint(r[22])), "r"(__float_as_uint(r[23])),
      "r"(__float_as_uint(r[24])), "r"(__float_as_uint(r[25])),
      "r"(__float_as_uint(r[26])), "r"(__float_as_uint(r[27])),
      "r"(__float_as_uint(r[28])), "r"(__float_as_uint(r[29])),
      "r"(__float_as_uint(r[30])), "r"(__float_as_uint(r[31]))
      : "memory");
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t *r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
      "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]),
      "r"(r[14]), "r"(r[15])
      : "memory");
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// One box of 128 rows x 64 elements of a [batch][token][elements] tensor into a
// swizzled column block; bytes counted on the mbarrier (rows past the sequence
// arrive as zeros and count all the same).
__device__ __forceinline__ void tma_load_block(uint32_t dst, const CUtensorMap *map,
                                               int x, int y, int z, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3, %4}], [%5];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(z), "r"(bar)
      : "memory");
}

// kCount fp32 columns of this thread's lane (kCount = 32 or 16)
template <int kCount>
__device__ __forceinline__ void tmem_ld(uint32_t taddr, float *r) {
  if constexpr (kCount == 32) {
    tmem_ld32(taddr, r);
  } else {
    uint32_t u[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(u[0]), "=r"(u[1]), "=r"(u[2]), "=r"(u[3]), "=r"(u[4]), "=r"(u[5]),
          "=r"(u[6]), "=r"(u[7]), "=r"(u[8]), "=r"(u[9]), "=r"(u[10]), "=r"(u[11]),
          "=r"(u[12]), "=r"(u[13]), "=r"(u[14]), "=r"(u[15])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) r[i] = __uint_as_float(u[i]);
  }
}
// kCount packed bf16 pairs into this thread's lane (kCount = 16 or 8)
template <int kCount>
__device__ __forceinline__ void tmem_st_packed(uint32_t taddr, const uint32_t *r) {
  if constexpr (kCount == 16) {
    tmem_st16(taddr, r);
  } else {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
        "r"(r[7])
        : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
  }
}

struct Barriers {
  uint64_t q_full;
  uint64_t k_full;
  uint64_t v_full;
  uint64_t s_full[2];   // Q K^T into S[b] done (also: the K tile is free)
  // The softmax warps have written P over their scores in S[b]. One barrier per
  // buffer: the softmax may finish tile it + 1 before the MMA thread has looked
  // at tile it (it waits for V as well), and a single barrier would then be two
  // phases ahead of its reader.
  uint64_t p_full[2];
  // P V of the tile in S[b] done: S[b] (the weights) and the V tile are free, O is
  // stable. One barrier per buffer, like p_full: each then completes once per
  // two tiles, so a waiter that has seen tile t - 2 (same buffer) complete is
  // exactly one phase behind tile t and a parity wait cannot alias.
  uint64_t pv_done[2];
};

struct SmallState {
  Barriers bars;
  uint32_t tmem_base;
  int abort;
  __nv_bfloat16 row_max[2][4][kBlockM];  // [tile parity][column quarter][row]
};

template <class T>
__global__ __launch_bounds__(kThreads, 1) void prefill_attention_sm100_kernel(
    Sm100PrefillParams p, const __grid_constant__ CUtensorMap map_q,
    const __grid_constant__ CUtensorMap map_k,
    const __grid_constant__ CUtensorMap map_v) {
  constexpr int kHeadDim = T::kHeadDim;
  constexpr int kBlockN = T::kBlockN;
  constexpr int kQuarterN = T::kQuarterN;
  // All shared memory is dynamic: the three tiles, 1024-byte aligned as their
  // 128-byte swizzle wants (the window of a kernel without static shared memory
  // starts on such a boundary; checked below), then the small state.
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  SmallState &small = *reinterpret_cast<SmallState *>(smem_raw + T::kTileBytes);
  Barriers &s_bars = small.bars;
  __nv_bfloat16(&s_max)[2][4][kBlockM] = small.row_max;
  const uint32_t s_q = smem_u32(smem_raw);
  const uint32_t s_k = s_q + T::kQBytes;
  const uint32_t s_v = s_k + T::kKBytes;
  if ((s_q & 1023u) != 0) {
    if (threadIdx.x == 0) atomicCAS(&g_prefill_sm100_fault, 0, 6);
    return;
  }

  // an earlier CTA gave up: the whole CTA returns, on one common reading
  if (__syncthreads_or(*reinterpret_cast<volatile int *>(&g_prefill_sm100_fault) != 0)) {
    return;
  }
  const int tid = int(threadIdx.x);
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int S = p.seq_len;
  const int m_block = int(gridDim.x) - 1 - int(blockIdx.x);  // longest first
  const int batch = int(blockIdx.y);
  const int head = int(blockIdx.z) / T::kVSplits;
  const int v_part = int(blockIdx.z) % T::kVSplits;  // which 256 of V's dims
  const int kv_head = head / (p.q_heads / p.kv_heads);
  const int m0 = m_block * kBlockM;
  const int last_row = min(m0 + kBlockM, S) - 1;
  const int tile_hi = last_row / kBlockN;
  const int tile_lo = p.window > 0 ? max(0, m0 - p.window + 1) / kBlockN : 0;
  const int tiles = tile_hi - tile_lo + 1;

  const uint32_t bar_q_full = smem_u32(&s_bars.q_full);
  const uint32_t bar_k_full = smem_u32(&s_bars.k_full);
  const uint32_t bar_v_full = smem_u32(&s_bars.v_full);
  const uint32_t bar_s_full = smem_u32(&s_bars.s_full[0]);    // + 8 b
  const uint32_t bar_p_full = smem_u32(&s_bars.p_full[0]);    // + 8 b
  const uint32_t bar_pv_done = smem_u32(&s_bars.pv_done[0]);  // + 8 b
  if (tid == 0) {
    mbar_init(bar_q_full, 1);
    mbar_init(bar_k_full, 1);
    mbar_init(bar_v_full, 1);
    mbar_init(bar_s_full, 1);
    mbar_init(bar_s_full + 8, 1);
    mbar_init(bar_p_full, kSoftmaxWarps);
    mbar_init(bar_p_full + 8, kSoftmaxWarps);
    mbar_init(bar_pv_done, 1);
    mbar_init(bar_pv_done + 8, 1);
    small.abort = 0;
    mbar_fence_init();
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(&small.tmem_base)),
                 "r"(kTmemColumns)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::
                     : "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = small.tmem_base;
  volatile int *abort_flag = &small.abort;

  // Bounded wait that also gives up when another role has; false = give up.
  auto wait = [&](uint32_t bar, uint32_t parity, int code) -> bool {
    if (mbar_try_wait(bar, parity)) return true;
    const long long start = clock64();
    for (uint32_t poll = 0;; ++poll) {
      if (mbar_try_wait(bar, parity)) return true;
      if ((poll & 31u) == 31u) {
        if (*abort_flag != 0) return false;
        if (clock64() - start > kTileWaitClocks) {
          atomicCAS(&g_prefill_sm100_fault, 0, code);
          *abort_flag = 1;
          return false;
        }
      }
    }
  };

  if (warp == kSoftmaxWarps) {
    // ------------------------------------------------------------ Q and K loader
    if (lane == 0) {
      mbar_arrive_expect_tx(bar_q_full, T::kQBytes);
#pragma unroll
      for (int blk = 0; blk < kHeadDim / 64; ++blk) {
        tma_load_block(s_q + blk * T::kQBlockBytes, &map_q, head * kHeadDim + blk * 64, m0,
                       batch, bar_q_full);
      }
      int issued = 0;
      for (int it = 0; it < tiles; ++it) {
        // K tile free: Q K^T of the previous tile done
        if (it > 0 && !wait(bar_s_full + 8u * uint32_t((it - 1) & 1),
                            uint32_t((it - 1) >> 1) & 1u, 3)) {
          break;
        }
        mbar_arrive_expect_tx(bar_k_full, T::kKBytes);
#pragma unroll
        for (int blk = 0; blk < kHeadDim / 64; ++blk) {
          tma_load_block(s_k + blk * T::kKBlockBytes, &map_k, kv_head * kHeadDim + blk * 64,
                         (tile_lo + it) * kBlockN, batch, bar_k_full);
        }
        ++issued;
      }
      if (*abort_flag != 0) {
        // nobody may be waiting for the last loads any more: see them land
        // before the CTA gives its shared memory back
        mbar_wait_bounded(bar_q_full, 0, kTileWaitClocks);
        if (issued > 0) {
          mbar_wait_bounded(bar_k_full, uint32_t(issued - 1) & 1u, kTileWaitClocks);
        }
      }
    }
  } else if (warp == kSoftmaxWarps + 2) {
    // ------------------------------------------------------------ V loader
    // (its own thread: a V tile waits for P V of the previous tile, a K tile for
    // Q K^T of the previous tile, and neither should queue behind the other)
    if (lane == 0) {
      int issued = 0;
      for (int it = 0; it < tiles; ++it) {
        if (it > 0 && !wait(bar_pv_done + 8u * uint32_t((it - 1) & 1),
                            uint32_t((it - 1) >> 1) & 1u, 3)) {
          break;
        }
        mbar_arrive_expect_tx(bar_v_full, T::kVBytes);
#pragma unroll
        for (int blk = 0; blk < kDv / 64; ++blk) {
          tma_load_block(s_v + blk * T::kKBlockBytes, &map_v,
                         kv_head * kHeadDim + v_part * kDv + blk * 64,
                         (tile_lo + it) * kBlockN, batch, bar_v_full);
        }
        ++issued;
      }
      if (*abort_flag != 0 && issued > 0) {
        mbar_wait_bounded(bar_v_full, uint32_t(issued - 1) & 1u, kTileWaitClocks);
      }
    }
  } else if (warp == kSoftmaxWarps + 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t kIdescQK = umma_idesc(kBlockN, false);
      constexpr uint32_t kIdescPV = umma_idesc(kDv, true);
      // S[buf] = Q K^T: steps of 16 dims; a step moves 32 bytes inside a column
      // block, four steps move to the next block
      auto issue_qk = [&](int buf) {
#pragma unroll
        for (int ks = 0; ks < kHeadDim / 16; ++ks) {
          const uint32_t in = uint32_t(ks & 3) * 32u;
          umma_bf16(tmem + uint32_t(buf) * kBlockN,
                    umma_desc(s_q + uint32_t(ks >> 2) * T::kQBlockBytes + in, 1, 64),
                    umma_desc(s_k + uint32_t(ks >> 2) * T::kKBlockBytes + in, 1, 64),
                    kIdescQK, ks > 0);
        }
        umma_commit(bar_s_full + 8u * uint32_t(buf));
      };
      // O (+)= P V: steps of 16 keys. P sits in tensor memory where the scores
      // were: the thread that read a quarter of the columns of S[buf] left its
      // weights, two per column, in the first half of them. V is MN-major:
      // 8-key groups 1024 bytes apart, 64-dim blocks one column block apart
      auto issue_pv = [&](int buf, bool accumulate) {
#pragma unroll
        for (int j = 0; j < kBlockN / 16; ++j) {
          const uint32_t key = 16u * uint32_t(j);
          const uint32_t p_at = tmem + uint32_t(buf) * kBlockN + (key / kQuarterN) * kQuarterN +
                                (key % kQuarterN) / 2u;
          umma_bf16_a_tmem(tmem + T::kTmemO, p_at,
                           umma_desc(s_v + uint32_t(j) * 2048u, T::kKBlockBytes >> 4, 64),
                           kIdescPV, accumulate || j > 0);
        }
        umma_commit(bar_pv_done + 8u * uint32_t(buf));
      };
      bool ok = wait(bar_q_full, 0, 4) && wait(bar_k_full, 0, 4);
      if (ok) {
        tc_fence_after();
        issue_qk(0);
      }
      for (int it = 0; it < tiles && ok; ++it) {
        if (it + 1 < tiles) {
          // next tile's scores: its K has landed and S[(it + 1) & 1], which held
          // the weights of tile it - 1, is no longer read
          const int n = it + 1;
          ok = wait(bar_k_full, uint32_t(n) & 1u, 4);
          if (ok && n >= 2) {
            ok = wait(bar_pv_done + 8u * uint32_t(n & 1), uint32_t((n - 2) >> 1) & 1u, 4);
          }
          if (!ok) break;
          tc_fence_after();
          issue_qk(n & 1);
        }
        ok = wait(bar_v_full, uint32_t(it) & 1u, 4) &&
             wait(bar_p_full + 8u * uint32_t(it & 1), uint32_t(it >> 1) & 1u, 4);
        if (!ok) break;
        tc_fence_after();
        issue_pv(it & 1, it > 0);
      }
    }
  } else {
    // ------------------------------------------------------------ softmax
    const int quarter = warp >> 2;  // which quarter of a tile's key columns
    const int row_in = tid & (kBlockM - 1);
    const int row = m0 + row_in;
    const uint32_t lane_base = uint32_t(32 * (warp & 3)) << 16;
    const int row_barrier = 1 + (warp & 3);  // the four warps that share 32 rows
    const float scale = p.scale_log2;
    float m_ref = -INFINITY;  // the maximum this row's weights are scaled by
    float l_run = 0.0f;       // this thread's quarter of the row's denominator
    bool ok = true;
    // The four warps that share 32 rows meet at a named barrier once per tile and
    // once at the end. Each decides for itself when to give up a wait, so one may
    // leave the loop while a sibling still passes the same wait; a warp that has
    // given up therefore makes up the arrivals it skipped (below), and no sibling
    // is left alone at the barrier on its way to the common exit.
    int row_syncs = 0;
    for (int it = 0; it < tiles; ++it) {
      const int tile = tile_lo + it;
      const int buf = it & 1;
      const int k0 = tile * kBlockN + quarter * kQuarterN;
      ok = wait(bar_s_full + 8u * uint32_t(buf), uint32_t(it >> 1) & 1u, 1);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      float s[kQuarterN];
      const uint32_t s_at =
          tmem + lane_base + uint32_t(buf) * kBlockN + uint32_t(quarter) * kQuarterN;
      tmem_ld<kQuarterN>(s_at, s);

      const bool edge = tile * kBlockN + kBlockN - 1 > m0 ||
                        (p.window > 0 && tile * kBlockN < last_row - p.window + 1);
      if (edge) {
#pragma unroll
        for (int c = 0; c < kQuarterN; ++c) {
          const int col = k0 + c;
          if (col > row || (p.window > 0 && col < row - p.window + 1)) s[c] = -INFINITY;
        }
      }
      // maximum of the raw scores in four independent chains (the scale is positive)
      float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int c = 0; c < kQuarterN; c += 4) {
#pragma unroll
        for (int u = 0; u < 4; ++u) mx[u] = fmaxf(mx[u], s[c + u]);
      }
      // The four threads of a row publish their maxima rounded to bf16 and all
      // use the largest published value: the same number in every thread, and
      // close enough to the true maximum for a scaling reference.
      const __nv_bfloat16 m_mine =
          __float2bfloat16_rn(fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * scale);
      s_max[buf][quarter][row_in] = m_mine;
      named_barrier_sync(row_barrier, 128);
      ++row_syncs;
      const float m_tile = fmaxf(fmaxf(__bfloat162float(s_max[buf][0][row_in]),
                                       __bfloat162float(s_max[buf][1][row_in])),
                                 fmaxf(__bfloat162float(s_max[buf][2][row_in]),
                                       __bfloat162float(s_max[buf][3][row_in])));
      float factor = 1.0f;
      if (m_tile > m_ref + kRescaleSlack || m_ref == -INFINITY) {
        if (m_tile > -INFINITY) {
          factor = m_ref == -INFINITY ? 1.0f : ex2_approx(m_ref - m_tile);
          m_ref = m_tile;
        }
      }
      const float neg_m = m_ref == -INFINITY ? 0.0f : -m_ref;
      float sum[4] = {0.0f, 0.0f, 0.0f, 0.0f};
      uint32_t packed[kQuarterN / 2];
#pragma unroll
      for (int i = 0; i < kQuarterN / 2; ++i) {
        const float e0 = ex2_approx(fmaf(s[2 * i], scale, neg_m));
        const float e1 = ex2_approx(fmaf(s[2 * i + 1], scale, neg_m));
        const __nv_bfloat162 h = __floats2bfloat162_rn(e0, e1);
        const uint32_t u = *reinterpret_cast<const uint32_t *>(&h);
        packed[i] = u;
        // the denominator sums the weights as rounded, the ones P V uses
        sum[i & 3] += __uint_as_float(u << 16) + __uint_as_float(u & 0xffff0000u);
      }
      l_run = l_run * factor + ((sum[0] + sum[1]) + (sum[2] + sum[3]));
      // tensor-memory accesses are warp-wide: the warp rescales its quarter of
      // the columns of O if any of its rows must, once P V of the previous tile
      // no longer adds to them
      if (it > 0 && __any_sync(0xffffffffu, factor != 1.0f)) {
        ok = wait(bar_pv_done + 8u * uint32_t((it - 1) & 1), uint32_t((it - 1) >> 1) & 1u, 2);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
#pragma unroll 1
        for (int c = 0; c < kDv / 4; c += 32) {
          float o[32];
          const uint32_t at = tmem + lane_base + T::kTmemO + uint32_t(quarter * (kDv / 4) + c);
          tmem_ld32(at, o);
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] *= factor;
          tmem_st32(at, o);
        }
      }
      // this thread's weights go where it read its scores from
      tmem_st_packed<kQuarterN / 2>(s_at, packed);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_p_full + 8u * uint32_t(buf));
    }

    // ---- the last P V, then O / l as bf16
    // P V of the last two tiles may both still be running: wait for each on its
    // own buffer's barrier. The warp has seen tile tiles - 3 complete (the last
    // tile's scores were issued after it) and P V products complete in order, so
    // on either barrier the awaited phase is the one right after a phase the
    // warp knows to be complete.
    if (ok && tiles >= 2) {
      ok = wait(bar_pv_done + 8u * uint32_t((tiles - 2) & 1), uint32_t((tiles - 2) >> 1) & 1u, 5);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      ok = wait(bar_pv_done + 8u * uint32_t((tiles - 1) & 1), uint32_t((tiles - 1) >> 1) & 1u, 5);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      tc_fence_after();
      // the V tile is no longer read: its first bytes carry the four partial
      // denominators of every row
      float *row_sum = reinterpret_cast<float *>(smem_raw + T::kQBytes + T::kKBytes);
      row_sum[quarter * kBlockM + row_in] = l_run;
      named_barrier_sync(row_barrier, 128);
      ++row_syncs;
      const float l_row = (row_sum[row_in] + row_sum[kBlockM + row_in]) +
                          (row_sum[2 * kBlockM + row_in] + row_sum[3 * kBlockM + row_in]);
      const float inv = l_row > 0.0f ? 1.0f / l_row : 0.0f;
      __nv_bfloat16 *dst = p.out + ((int64_t(batch) * S + row) * p.q_heads + head) * kHeadDim +
                           v_part * kDv + quarter * (kDv / 4);
      // tensor-memory loads are warp-wide: rows past the sequence take part in
      // them and only skip the stores
#pragma unroll 1
      for (int c = 0; c < kDv / 4; c += 32) {
        float o[32];
        tmem_ld32(tmem + lane_base + T::kTmemO + uint32_t(quarter * (kDv / 4) + c), o);
        if (row < S) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint32_t w[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const __nv_bfloat162 h = __floats2bfloat162_rn(o[8 * i + 2 * j] * inv,
                                                             o[8 * i + 2 * j + 1] * inv);
              w[j] = *reinterpret_cast<const uint32_t *>(&h);
            }
            reinterpret_cast<uint4 *>(dst + c)[i] = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      }
    }
    // gave up somewhere above (ok is warp-uniform): the arrivals still owed
    for (; row_syncs < tiles + 1; ++row_syncs) named_barrier_sync(row_barrier, 128);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem),
                 "r"(kTmemColumns)
                 : "memory");
  }
}

using EncodeTiledFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                   const cuuint64_t *, const cuuint64_t *,
                                   const cuuint32_t *, const cuuint32_t *,
                                   CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = [] {
    void *ptr = nullptr;
    cudaDriverEntryPointQueryResult result;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault,
                                &result) != cudaSuccess ||
        result != cudaDriverEntryPointSuccess) {
      return EncodeTiledFn(nullptr);
    }
    return reinterpret_cast<EncodeTiledFn>(ptr);
  }();
  return fn;
}

// [batch][token][heads * head_dim] bf16, boxes of box_rows tokens x 64 elements,
// 128-byte swizzle; tokens past the sequence read as zeros.
bool make_rows_map(CUtensorMap *map, const __nv_bfloat16 *base, int batch, int seq_len,
                   int row_elems, int box_rows) {
  EncodeTiledFn encode = encode_tiled_fn();
  if (encode == nullptr) return false;
  const cuuint64_t dims[3] = {cuuint64_t(row_elems), cuuint64_t(seq_len), cuuint64_t(batch)};
  const cuuint64_t strides[2] = {cuuint64_t(row_elems) * 2,
                                 cuuint64_t(seq_len) * row_elems * 2};
  const cuuint32_t box[3] = {64, cuuint32_t(box_rows), 1};
  const cuuint32_t elem_strides[3] = {1, 1, 1};
  return encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3,
                const_cast<__nv_bfloat16 *>(base), dims, strides, box, elem_strides,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <class T>
cudaError_t launch_sm100(__nv_bfloat16 *out, const __nv_bfloat16 *q, const __nv_bfloat16 *k,
                         const __nv_bfloat16 *v, int batch, int seq_len, int q_heads,
                         int kv_heads, int window, float softmax_scale,
                         cudaStream_t stream) {
  constexpr int kSmemBytes = T::kTileBytes + int(sizeof(SmallState));
  static_assert(kSmemBytes <= 227 * 1024, "tiles must fit one SM");
  CUtensorMap map_q, map_k, map_v;
  if (!make_rows_map(&map_q, q, batch, seq_len, q_heads * T::kHeadDim, kBlockM) ||
      !make_rows_map(&map_k, k, batch, seq_len, kv_heads * T::kHeadDim, T::kBlockN) ||
      !make_rows_map(&map_v, v, batch, seq_len, kv_heads * T::kHeadDim, T::kBlockN)) {
    return cudaErrorInvalidValue;
  }
  Sm100PrefillParams p = {out,    seq_len, q_heads, kv_heads,
                          window, softmax_scale * 1.4426950408889634f};
  cudaError_t st = cudaFuncSetAttribute(prefill_attention_sm100_kernel<T>,
                                        cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        kSmemBytes);
  if (st != cudaSuccess) return st;
  void *fault_word = nullptr;
  st = cudaGetSymbolAddress(&fault_word, g_prefill_sm100_fault);
  if (st != cudaSuccess) return st;
  st = cudaMemsetAsync(fault_word, 0, sizeof(int), stream);
  if (st != cudaSuccess) return st;
  const dim3 grid(unsigned(div_up(seq_len, kBlockM)), unsigned(batch),
                  unsigned(q_heads * T::kVSplits));
  prefill_attention_sm100_kernel<T><<<grid, kThreads, kSmemBytes, stream>>>(p, map_q, map_k,
                                                                            map_v);
  return cudaGetLastError();
}

}  // namespace

cudaError_t prefill_attention_sm100_bf16(__nv_bfloat16 *out,
                                         const __nv_bfloat16 *q,
                                         const __nv_bfloat16 *k,
                                         const __nv_bfloat16 *v, int batch,
                                         int seq_len, int q_heads, int kv_heads,
                                         int head_dim, int window, float softmax_scale,
                                         cudaStream_t stream) {
  if (q_heads * (head_dim / kDv) > 65535) return cudaErrorInvalidValue;
  if (head_dim == 256) {
    return launch_sm100<Sm100Traits<256, 128>>(out, q, k, v, batch, seq_len, q_heads,
                                               kv_heads, window, softmax_scale, stream);
  }
  if (head_dim == 512) {
    return launch_sm100<Sm100Traits<512, 64>>(out, q, k, v, batch, seq_len, q_heads,
                                              kv_heads, window, softmax_scale, stream);
  }
  return cudaErrorInvalidValue;
}

int prefill_attention_sm100_fault() {
  int fault = -1;
  if (cudaMemcpyFromSymbol(&fault, g_prefill_sm100_fault, sizeof(int)) !=
      cudaSuccess) {
    return -1;
  }
  return fault;
}

}  // namespace b200kv

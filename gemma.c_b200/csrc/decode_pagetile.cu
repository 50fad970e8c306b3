// Decode layer-step by (sequence, KV head, range of key tiles), in ONE launch.
//
// The balanced kernel (decode_balanced.cu) gives every CTA the rows of all
// eight KV heads of its keys and leaves the merge of the CTAs' partials to a
// second launch. That is the right shape when a launch streams hundreds of MB.
// For small jobs -- a sliding-window layer of a few sequences, a batch-1 layer,
// the share of one rank of a sharded batch -- the fixed costs decide: sixteen
// partial rows per CTA (16 KiB against the 32 KiB of keys a small CTA streams),
// a second kernel that waits for the first, and query rows prepared again for
// every sequence a range touches. Here:
//
//  * A CTA owns one KV head of one sequence over a contiguous range of its live
//    keys. Its two query rows are prepared once. The head's rows are 512-byte
//    slices of the cache's 4 KiB token rows; a TMA tensor map over
//    [dim][head][page offset][page] fetches the slices of up to 16 tokens of a
//    page as one tile (cp.async.bulk.tensor.4d, completion on an mbarrier, no
//    multicast), two tiles per 32-token stage and tensor, three stages.
//  * Pages of 8 tokens or more: the stage's arithmetic runs on the tensor cores
//    (bf16 mma.sync m16n8k16; see consume_half_mma). The tiles come in through a
//    five-dimensional view of the cache that lays a tile down as four blocks of
//    64 dims with the 128-byte swizzle, so that ldmatrix reads them without bank
//    conflicts; stages alternate between two groups of four warps, a warp per
//    (key half, output-dim half). Smaller pages: eight consumer warps take four
//    tokens of a stage each (the scalar arithmetic of decode_common.cuh).
//    Either way the warps merge their running (m, l, acc) through the idle ring
//    at the end, and the CTA leaves ONE partial of two rows (2 KiB).
//  * The last CTA of a (sequence, head) to arrive -- a ticket per pair, taken
//    with a fence on either side -- merges that pair's partials and writes the
//    two output rows and their log-sum-exp: what phase_decode_paged_reduce does
//    behind a grid-wide barrier (src/gemma4_flash_attention_decode.cu:881-977),
//    without a second launch. A pair with a single range writes its rows
//    directly.
//  * The step's append is fused as in the balanced kernel: warps 0..3 prepare
//    the two query rows and, in the CTA whose range holds the new position,
//    the K and V row (prep_common.cuh: the append kernel's arithmetic, so the
//    same bits); the new row is patched into the stage the tile arrived in and
//    written to the cache after the wait for the preceding kernel.
//
// Works for any number of KV heads (the caches of KV-head-sharded ranks
// included). Ranges are cut per sequence, so it is chosen when the live keys of
// the sequences are equal by construction (sliding windows) or there is one
// sequence; ragged batches stay on the balanced partition.
//
// Programmatic dependent launch follows decode_balanced.cu: before its
// griddepcontrol.wait a CTA reads lengths, positions, page-table entries, raw
// projections (unless they come from the preceding kernel) and key tiles older
// than the page of the previous step's newest key; everything it writes
// (prepared q, cache rows, partials, tickets, outputs) and the newest tiles
// come after. By default the dependent launch is released by a warp that has
// itself waited for the preceding kernel, so at most two kernels are in flight.
//
// Runs (b200kv_decode_step_bf16 decides, see host_api.cu): a kernel may be told
// to release the next launch at once (release_early), and is told how many of
// the launches it can then meet are earlier decode steps of its own cache layer
// (steps_in_flight; 0 = layer-steps of other layers only, no tile waits). The
// rows those steps append are not in the cache yet: the kernel either gets their
// raw K / V rows and positions and prepares them itself (fwd_*, patched into the
// stages like its own new row), or holds back the tiles of those positions
// until the preceding kernel is complete. Completion stays a chain -- every CTA
// waits for the preceding kernel before it writes or leaves -- which is what
// scratch, tickets, outputs and the slots of a tight ring rely on.
#include <cuda.h>

#include <algorithm>
#include <cstdlib>
#include <cstring>

#include "balanced_partition.cuh"
#include "decode_common.cuh"
#include "kernels.cuh"
#include "mma_common.cuh"
#include "prep_common.cuh"

namespace b200kv {

namespace {

using TileTraits = DecodeTraits<256, 1, 2, 8>;  // one head: 8 warps x 4 tokens
constexpr int kTileStage = TileTraits::kStageTokens;  // 32 tokens
constexpr int kMaxTileTokens = 16;                    // tokens of one TMA tile
constexpr int kMergeGroup = 32;      // partials one CTA merges in one round of loads
constexpr int kMaxMergeGroups = B200KV_TICKETS_PER_HEAD - 1;  // groups per (sequence, head)
constexpr int kMaxRanges = kMergeGroup * kMaxMergeGroups;  // key ranges per (sequence, head)
// Above this many sequences a sliding-window layer is a bandwidth job and stays
// on the balanced partition (see decode_pagetile_preferred).
constexpr int kPagetileMaxBatch = 32;
constexpr int kPagetileMaxLinearKeys = 32768;
constexpr int kTileConsumerThreads = TileTraits::kConsumerWarps * kWarpSize;
// 8 consumer warps, the producer warp, and a warp that does nothing but wait
// for the preceding kernel and then release the next one (see the kernel).
constexpr int kTileThreads = TileTraits::kThreads + kWarpSize;
// The tensor-core variant keeps its two q rows 16 bytes further apart than a
// row is long, so that the ldmatrix that replicates them over eight matrix rows
// reads two bank groups instead of one.
constexpr int kQStrideMma = 256 + 8;
// Rows of unfinished earlier steps of the same cache layer that a step prepares
// itself instead of waiting for them to reach the cache (TileParams::fwd_*).
constexpr int kMaxForward = AppendArgs::kMaxForward;
// q rows, new K/V rows, flags, forwarded K/V rows and their positions
constexpr int kTileExtraBytes = 2 * kQStrideMma * 2 + 2 * 512 + 64 + kMaxForward * 1024 + 32;
// Shared-memory layout of a TMA tile (tile_tokens tokens of one head, K or V) in
// the tensor-core variant: four blocks of 64 dims, each [tile_tokens][128 bytes],
// written by one TMA copy with the 128-byte swizzle (the 16-byte chunk c of
// token row r lands at chunk c ^ (r % 8)), so that the eight rows of an ldmatrix
// tile fall into eight different bank groups. The tiles of a stage follow one
// another as in the scalar variant (tile_tokens * 512 bytes each).
constexpr int kMmaMinTileTokens = 8;  // a block is then a whole number of swizzle atoms
constexpr int kTileSmemBytes = TileTraits::kRingBytes + kTileExtraBytes;
static_assert(TileTraits::kRingBytes % 128 == 0, "rows behind the ring stay aligned");
static_assert(2 * (kTileSmemBytes + 1024) <= 228 * 1024, "two CTAs per SM");

struct TileParams {
  __nv_bfloat16 *out;
  float *lse;
  const __nv_bfloat16 *q;  // attention only: the prepared q
  __nv_bfloat16 *cache_k;  // fused: the new rows are written here
  __nv_bfloat16 *cache_v;
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
  uint32_t *ticket;     // [batch * kv_heads * B200KV_TICKETS_PER_HEAD], zero between launches
  int32_t ranges;       // key ranges (CTAs) per sequence and head
  int32_t tile_tokens;  // tokens of one TMA tile: min(page_size, 16)
  int32_t *status;
  // fused modes
  const __nv_bfloat16 *raw_q;
  const __nv_bfloat16 *raw_k;
  const __nv_bfloat16 *raw_v;
  const __nv_bfloat16 *q_norm_weight;
  const __nv_bfloat16 *k_norm_weight;
  const float *cos;
  const float *sin;
  const int32_t *token_position;
  __nv_bfloat16 *q_prepared;
  int32_t raw_from_predecessor;
  // How many of the kernels that may still be in flight when this one starts
  // are decode steps of this cache layer (each appends the position before the
  // next one's): the tiles of that many positions before the new one wait for
  // the preceding kernel. 0: none writes this layer's cache, no tile waits.
  int32_t steps_in_flight;
  // With fwd_count == steps_in_flight no tile waits either: the K / V rows those
  // steps append are prepared here from their raw rows (fwd_k, fwd_v; V from K
  // where fwd_v is null) at their positions (fwd_pos, per sequence; negative: the
  // step did not append for that sequence), nearest step first.
  int32_t fwd_count;
  const __nv_bfloat16 *fwd_k[kMaxForward];
  const __nv_bfloat16 *fwd_v[kMaxForward];
  const int32_t *fwd_pos[kMaxForward];
  // Non-zero: the next kernel may start as soon as this one runs (the caller has
  // checked that what the next kernel reads before its own wait is written by
  // none of the kernels that can then be in flight).
  int32_t release_early;
  // The all-gather of the output rows over peer memory, finished by this kernel
  // (world == 0: none). The rows of this rank are [batch, q_heads, 256] bf16.
  PeerEpilogue peer;
};

// One tile: the 512-byte slices of head `head` for `tile_tokens` tokens of a
// page, starting at offset `offset` (a multiple of the tile size). The inner
// coordinate is 0, so the 16-byte rule of TMA starts holds by construction.
__device__ __forceinline__ void tma_load_tile(uint32_t dst, const CUtensorMap *map,
                                              int head, int offset, int page,
                                              uint32_t bar, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      ".L2::cache_hint [%0], [%1, {%2, %3, %4, %5}], [%6], %7;" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(0), "r"(head), "r"(offset), "r"(page),
      "r"(bar), "l"(policy)
      : "memory");
}

// The same tile through the five-dimensional view [64 dims][page offset]
// [block of 64 dims][head][page] (tensor-core variant): the copy lays the four
// blocks of the tile down one after the other, 128-byte rows, swizzled.
__device__ __forceinline__ void tma_load_tile_blocked(uint32_t dst, const CUtensorMap *map,
                                                      int head, int offset, int page,
                                                      uint32_t bar, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      ".L2::cache_hint [%0], [%1, {%2, %3, %4, %5, %6}], [%7], %8;" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(0), "r"(offset), "r"(0), "r"(head), "r"(page),
      "r"(bar), "l"(policy)
      : "memory");
}

// The descriptor of a tensor map is fetched on first use; asking for it at the
// start of the kernel takes that round trip off the first tile.
__device__ __forceinline__ void prefetch_tensor_map(const CUtensorMap *map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

__device__ __forceinline__ void st_release_sys(uint32_t *addr, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t *addr) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}

// ---------------------------------------------------------------------------
// Tensor-core arithmetic of one stage (kMma). Four warps share a stage: warp
// (kh, dh) scores the 16 keys of half kh against the two query rows and
// accumulates P * V for the 128 dims of half dh. Both contractions are written
// so that nothing has to move between lanes in between:
//
//   S [16 x 16] = Q8 [16 x 256] * K^T: the 16 rows of the A operand are the two
//     query rows over and over (row i is query i % 2), the B operand comes
//     straight from the K rows by ldmatrix. Thread (g, t) then holds the scores
//     of query g % 2 against keys 2t, 2t + 1, 2t + 8, 2t + 9 -- which is exactly
//     the B fragment of
//   O^T [128 x 8] += V^T [128 x 16] * P^T [16 x 8]: column n of P^T is query
//     n % 2; V^T comes from the V rows by ldmatrix.trans; thread (g, t) ends
//     with dims g, g + 8 (of each 16-dim tile) of both queries.
//
// The running maximum and sum are per query as in decode_common.cuh (exp2
// domain); P is rounded to bf16 for the second contraction, the sum adds the
// unrounded weights.
// ---------------------------------------------------------------------------
struct MmaLane {
  uint32_t row;     // byte offset of this lane's ldmatrix row (block 0) inside a stage's K rows,
                    // with the swizzle term of the lane's chunk already applied
  uint32_t block;   // bytes from one 64-dim block of a tile to the next
  uint32_t q_addr;  // its row of the q matrices: query lane % 2, chunk lane / 8
  int key0;         // first of its four keys within the half: 2 (lane % 4)
  int own;          // the query its scores belong to: (lane / 4) % 2
  // Address of the lane's row for the 16-dim step `step` (0..3) of block `blk`:
  // chunk 2 step + sel lands at chunk (2 step + sel) ^ (token % 8), and since
  // 2 step and sel share no bit, that is (2 step) ^ (sel ^ token % 8).
  __device__ __forceinline__ uint32_t at(uint32_t tensor, int blk, int step) const {
    return (tensor + uint32_t(blk) * block + row) ^ uint32_t(step << 5);
  }
  __device__ MmaLane(int lane, int kh, int tile_tokens, uint32_t q_base) {
    const int key = kh * 16 + ((lane >> 4) << 3) + (lane & 7);
    const uint32_t sel = uint32_t(lane >> 3) & 1u;
    block = uint32_t(tile_tokens) * 128u;
    row = uint32_t(key / tile_tokens) * uint32_t(tile_tokens) * 512u +
          uint32_t(key % tile_tokens) * 128u + ((sel ^ uint32_t(key & 7)) << 4);
    q_addr = q_base + uint32_t(lane & 1) * uint32_t(kQStrideMma * 2) +
             uint32_t(lane >> 3) * 16u;
    key0 = (lane & 3) * 2;
    own = (lane >> 2) & 1;
  }
};

struct MmaState {
  float acc[8][4];  // tile j: dims 16 j + g (queries 0, 1), 16 j + g + 8 (queries 0, 1)
  float m[2];       // running maxima of the two queries, exp2 domain
  float l_lane;     // running sum of this lane's own weights (query `own`)
  __device__ __forceinline__ void reset() {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[j][i] = 0.0f;
    }
    m[0] = m[1] = -INFINITY;
    l_lane = 0.0f;
  }
};

// k_tensor: shared address of the stage's K rows (V rows follow at
// kStageTensorBytes), 1024-byte aligned; mask16: live keys of the half (not
// zero). Fragments are fetched one round ahead of the MMAs that use them: the
// asm statements are volatile, so the order written here is the order issued.
__device__ __forceinline__ void consume_half_mma(MmaState &st, const MmaLane &ln,
                                                 uint32_t k_tensor, uint32_t mask16,
                                                 int dh, float scale_log2) {
  float s[2][2][4];  // [parity of the 16-dim step][8-key tile][fragment]
#pragma unroll
  for (int a = 0; a < 2; ++a) {
#pragma unroll
    for (int b = 0; b < 2; ++b) {
#pragma unroll
      for (int i = 0; i < 4; ++i) s[a][b][i] = 0.0f;
    }
  }
  uint32_t qa[2][4], kb[2][2][4];
  auto fetch_round = [&](int kp, int buf) {  // the 16-dim steps 2 kp, 2 kp + 1
    ldmatrix_x4(qa[buf], ln.q_addr + uint32_t(kp) * 64u);
    ldmatrix_x4(kb[buf][0], ln.at(k_tensor, kp >> 1, (2 * kp) & 3));
    ldmatrix_x4(kb[buf][1], ln.at(k_tensor, kp >> 1, (2 * kp + 1) & 3));
  };
  fetch_round(0, 0);
#pragma unroll
  for (int kp = 0; kp < 8; ++kp) {
    const int cur = kp & 1;
    if (kp + 1 < 8) fetch_round(kp + 1, cur ^ 1);
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      mma_bf16_m16n8k16(s[j][0], qa[cur][2 * j], qa[cur][2 * j], qa[cur][2 * j + 1],
                        qa[cur][2 * j + 1], kb[cur][j][0], kb[cur][j][1]);
      mma_bf16_m16n8k16(s[j][1], qa[cur][2 * j], qa[cur][2 * j], qa[cur][2 * j + 1],
                        qa[cur][2 * j + 1], kb[cur][j][2], kb[cur][j][3]);
    }
  }
  // the first V fragments travel under the softmax
  const uint32_t v_tensor = k_tensor + TileTraits::kStageTensorBytes;
  uint32_t va[2][4];
  ldmatrix_x4_trans(va[0], ln.at(v_tensor, dh * 2, 0));
  ldmatrix_x4_trans(va[1], ln.at(v_tensor, dh * 2, 1));

  float sc[4];
  sc[0] = (s[0][0][0] + s[1][0][0]) * scale_log2;  // key key0
  sc[1] = (s[0][0][1] + s[1][0][1]) * scale_log2;  // key key0 + 1
  sc[2] = (s[0][1][0] + s[1][1][0]) * scale_log2;  // key key0 + 8
  sc[3] = (s[0][1][1] + s[1][1][1]) * scale_log2;  // key key0 + 9
  const uint32_t mine = mask16 >> ln.key0;  // bits 0, 1, 8, 9: this lane's keys
  if ((mine & 0x001u) == 0u) sc[0] = -INFINITY;
  if ((mine & 0x002u) == 0u) sc[1] = -INFINITY;
  if ((mine & 0x100u) == 0u) sc[2] = -INFINITY;
  if ((mine & 0x200u) == 0u) sc[3] = -INFINITY;
  float tile_max = fmaxf(fmaxf(sc[0], sc[1]), fmaxf(sc[2], sc[3]));
  tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, 1));
  tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, 2));
  const float other_max = __shfl_xor_sync(0xffffffffu, tile_max, 4);
  const float new_m0 = fmaxf(st.m[0], ln.own == 0 ? tile_max : other_max);
  const float new_m1 = fmaxf(st.m[1], ln.own == 0 ? other_max : tile_max);
  if (new_m0 > st.m[0] || new_m1 > st.m[1]) {
    const float corr0 = ex2_approx(st.m[0] - new_m0);
    const float corr1 = ex2_approx(st.m[1] - new_m1);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      st.acc[j][0] *= corr0;
      st.acc[j][1] *= corr1;
      st.acc[j][2] *= corr0;
      st.acc[j][3] *= corr1;
    }
    st.l_lane *= (ln.own == 0 ? corr0 : corr1);
    st.m[0] = new_m0;
    st.m[1] = new_m1;
  }
  const float m_own = ln.own == 0 ? st.m[0] : st.m[1];
  float pr[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) pr[i] = ex2_approx(sc[i] - m_own);
  st.l_lane += (pr[0] + pr[1]) + (pr[2] + pr[3]);
  const uint32_t pb0 = pack_bf16x2(pr[0], pr[1]);
  const uint32_t pb1 = pack_bf16x2(pr[2], pr[3]);

  // A dead key's V row may hold anything (0 * NaN would poison the sums): its
  // elements are cleared where the half is not complete.
  const bool partial = mask16 != 0xffffu;
  const uint32_t keep0 = ((mine & 0x001u) ? 0x0000ffffu : 0u) | ((mine & 0x002u) ? 0xffff0000u : 0u);
  const uint32_t keep1 = ((mine & 0x100u) ? 0x0000ffffu : 0u) | ((mine & 0x200u) ? 0xffff0000u : 0u);
#pragma unroll
  for (int j = 0; j < 8; ++j) {  // dims dh * 128 + 16 j ...
    const int cur = j & 1;
    uint32_t a0 = va[cur][0], a1 = va[cur][1], a2 = va[cur][2], a3 = va[cur][3];
    if (j + 2 < 8) ldmatrix_x4_trans(va[cur], ln.at(v_tensor, dh * 2 + ((j + 2) >> 2), (j + 2) & 3));
    if (partial) {
      a0 &= keep0;
      a1 &= keep0;
      a2 &= keep1;
      a3 &= keep1;
    }
    mma_bf16_m16n8k16(st.acc[j], a0, a1, a2, a3, pb0, pb1);
  }
}

template <int kMode, bool kMma>
__global__ __launch_bounds__(kTileThreads, 2) void decode_pagetile_kernel(
    TileParams p, const __grid_constant__ CUtensorMap map_k,
    const __grid_constant__ CUtensorMap map_v) {
  using T = TileTraits;
  constexpr int D = 256;
  constexpr int ST = kTileStage;
  constexpr bool kFused = kMode != kAttentionOnly;
  constexpr bool kIeee = kMode == kFusedIeee;
  constexpr int kQStride = kMma ? kQStrideMma : D;  // elements between the two q rows
  // partial states the CTA's warps leave for the merge: one per warp, or one per
  // (group of four warps, key half)
  constexpr int kStates = kMma ? 4 : T::kConsumerWarps;
  extern __shared__ __align__(1024) uint8_t smem[];
  __nv_bfloat16 *s_q = reinterpret_cast<__nv_bfloat16 *>(smem + T::kRingBytes);  // [2][kQStride]
  __nv_bfloat16 *s_new = s_q + 2 * kQStride;  // [2][256]: the new K row, the new V row
  volatile int *s_flag = reinterpret_cast<volatile int *>(s_new + 2 * D);  // abort, last
  // forwarded rows [step][K row, V row][256] and the position of each (-1: not in this CTA's range)
  __nv_bfloat16 *s_fwd = s_new + 2 * D + 32;
  volatile int *s_fwd_pos = reinterpret_cast<volatile int *>(s_fwd + kMaxForward * 2 * D);

  const int warp = int(threadIdx.x) >> 5;
  const int lane = int(threadIdx.x) & 31;
  const Gemma4KvCacheConfig &cfg = p.cfg;
  const int H = cfg.num_heads;
  const int bid = int(blockIdx.x);
  const int h = bid % H;
  const int r = (bid / H) % p.ranges;
  const int b = bid / (H * p.ranges);

  // Attention only: the successor (the next step's append, or anything else)
  // waits for this whole grid before it touches a thing.
  if constexpr (!kFused) pdl_release_successor();

  const Ring<T> ring(smem);
  if (threadIdx.x == 0) {
    ring.init_barriers();
    s_flag[0] = 0;
    s_flag[1] = 0;
  }
  // The raw row a prep warp works on depends on nothing but (b, h): fetched
  // first, so that it lands under the length and position loads.
  [[maybe_unused]] float x[D / 32];
  [[maybe_unused]] const __nv_bfloat16 *raw_row = nullptr;
  if constexpr (kFused) {
    if (warp < 4) {
      const int64_t kv_src = (int64_t(b) * H + h) * D;
      raw_row = warp < 2 ? p.raw_q + (int64_t(b) * p.q_heads + h * 2 + warp) * D
                         : (warp == 2 || p.raw_v == nullptr ? p.raw_k + kv_src
                                                            : p.raw_v + kv_src);
      if (!p.raw_from_predecessor) load_head<D>(raw_row, lane, x);
    }
  }
  if (warp == T::kConsumerWarps && lane == 0) {
    prefetch_tensor_map(&map_k);
    prefetch_tensor_map(&map_v);
  }
  // A short page-table row (a sliding-window ring) is fetched whole by the
  // producer warp before the length is known, four entries per lane: one
  // dependent round trip less before the first tile can be asked for.
  const int mpps = cfg.max_pages_per_seq;
  const bool small_table = mpps <= 4 * kWarpSize;
  int table_regs[4] = {-1, -1, -1, -1};
  if (warp == T::kConsumerWarps && small_table) {
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      if (lane * 4 + k < mpps) {
        table_regs[k] = __ldg(p.page_table + int64_t(b) * mpps + lane * 4 + k);
      }
    }
  }
  const int len = __ldg(p.seq_lengths + b);
  int new_pos = -1;
  if constexpr (kFused) new_pos = __ldg(p.token_position + b);
  __syncthreads();  // barriers and flags are set

  // The live keys and this CTA's share of them, in chunks of one stage (32
  // positions, aligned in position space).
  const int first = cfg.window_size > 0 ? max(0, len - cfg.window_size) : 0;
  const int count = max(0, len - first);
  const int chunk_lo = first / ST;
  const int chunks_total = count > 0 ? (len - 1) / ST - chunk_lo + 1 : 0;
  const int r_eff = min(p.ranges, chunks_total);
  // Ranges beyond the live chunks have nothing to do. Range 0 always stays: it
  // writes the rows of an empty sequence and keeps "this grid is complete
  // implies its predecessors are" (every CTA that stays waits before it exits).
  if (r >= max(r_eff, 1)) return;
  const int c0 = r_eff > 0 ? chunk_lo + int(int64_t(r) * chunks_total / r_eff) : 0;
  const int c1 = r_eff > 0 ? chunk_lo + int(int64_t(r + 1) * chunks_total / r_eff) : 0;
  const int nchunks = c1 - c0;
  const bool new_live = kFused && new_pos >= first && new_pos < len;
  const bool owns_new = new_live && new_pos / ST >= c0 && new_pos / ST < c1;
  // a new position that is not a live key of the attention (lengths and
  // positions that do not belong together): range 0 appends it all the same
  const bool preps_kv = owns_new || (kFused && new_pos >= 0 && !new_live && r == 0);

  if (warp == T::kConsumerWarps + 1) {
    // ------------------------------ sentinel ------------------------------
    // The next kernel may start once the kernel BEFORE this one is complete:
    // then only this kernel's writes are still in flight, which is what the
    // next kernel's early reads allow for (it leaves the page of this step's
    // new key, and everything it writes, for after its own wait). A warp of its
    // own passes that on as soon as it is true, however far this CTA's stream is.
    // (With release_early the caller has made sure that the next kernel's early
    // reads allow for deeper overlap, and the release comes at once. The order
    // of completion stays a chain either way: every CTA waits before it exits.)
    if constexpr (kFused) {
      if (p.release_early == 0) pdl_wait_for_predecessor();
      pdl_release_successor();
    }
    return;
  }
  if (warp == T::kConsumerWarps) {
    // ------------------------------ producer ------------------------------
    const uint64_t policy = l2_policy_evict_first();
    const int tb = p.tile_tokens;
    const int tiles = ST / tb;
    const int ps = cfg.page_size;
    // first position of the first page the preceding kernels may have written
    // (fused: the steps in flight wrote the positions len - 2 down to
    // len - 1 - steps_in_flight; attention only: the append before wrote len - 1)
    const int newest = max(len - 1 - (kFused ? p.steps_in_flight : 0), 0);
    const int fresh = (kFused && (p.steps_in_flight == 0 || p.fwd_count >= p.steps_in_flight))
                          ? len
                          : (newest / ps) * ps;
    bool ok = true;
    bool waited = false;
    int cached_lp = -1, cached_phys = -1;
    int issued = 0;
    for (int c = 0; c < nchunks; ++c) {
      const int base = (c0 + c) * ST;
      if (!waited && min(len, base + ST) > fresh) {
        pdl_wait_for_predecessor();
        waited = true;
      }
      const int stage = c % kStages;
      const int fill = c / kStages;
      if (fill > 0 &&
          !mbar_wait_bounded(ring.empty_bar(stage), uint32_t(fill - 1) & 1u)) {
        ok = false;
        break;
      }
      const int pos0 = base + lane * tb;
      const int live0 = max(pos0, first);
      const int live1 = min(pos0 + tb, len);
      const bool mine = lane < tiles && live0 < live1;
      int phys = -1;
      if (small_table) {
        const int slot = mine ? (pos0 / ps) % mpps : 0;
        const int e0 = __shfl_sync(0xffffffffu, table_regs[0], slot >> 2);
        const int e1 = __shfl_sync(0xffffffffu, table_regs[1], slot >> 2);
        const int e2 = __shfl_sync(0xffffffffu, table_regs[2], slot >> 2);
        const int e3 = __shfl_sync(0xffffffffu, table_regs[3], slot >> 2);
        const int e = (slot & 2) ? ((slot & 1) ? e3 : e2) : ((slot & 1) ? e1 : e0);
        phys = mine ? e : -1;
      } else if (mine) {
        const int lp = pos0 / ps;
        if (lp != cached_lp) {
          cached_phys = __ldg(p.page_table + int64_t(b) * mpps + lp % mpps);
          cached_lp = lp;
        }
        phys = cached_phys;
      }
      const bool valid = mine && phys >= 0 && phys < cfg.num_pages;
      const uint32_t bits =
          valid ? ((1u << (live1 - live0)) - 1u) << (live0 - base) : 0u;
      const uint32_t mask = __reduce_or_sync(0xffffffffu, bits);
      const int nvalid = __popc(__ballot_sync(0xffffffffu, valid));
      if (lane == 0) {
        ring.masks()[stage] = mask;
        if (nvalid > 0) {
          mbar_arrive_expect_tx(ring.full_bar(stage),
                                uint32_t(nvalid) * 2u * uint32_t(tb) * T::kRowBytes);
        } else {
          mbar_arrive(ring.full_bar(stage));
        }
      }
      __syncwarp();
      if (valid) {
        const int page = p.layer * cfg.num_pages + phys;
        const uint32_t dst = ring.k_stage(stage) + uint32_t(lane * tb) * T::kRowBytes;
        if constexpr (kMma) {
          tma_load_tile_blocked(dst, &map_k, h, pos0 % ps, page, ring.full_bar(stage), policy);
          tma_load_tile_blocked(dst + T::kStageTensorBytes, &map_v, h, pos0 % ps, page,
                                ring.full_bar(stage), policy);
        } else {
          tma_load_tile(dst, &map_k, h, pos0 % ps, page, ring.full_bar(stage), policy);
          tma_load_tile(dst + T::kStageTensorBytes, &map_v, h, pos0 % ps, page,
                        ring.full_bar(stage), policy);
        }
      }
      issued = c + 1;
    }
    // hold the CTA until every copy this warp issued has landed
    for (int s = 0; s < kStages && s < issued; ++s) {
      const int fill = (issued - 1 - s) / kStages;
      if (!mbar_wait_bounded(ring.full_bar(s), uint32_t(fill) & 1u)) ok = false;
    }
    if (!waited) pdl_wait_for_predecessor();
    if (!ok && lane == 0) set_status(p.status, B200KV_STATUS_WAIT_TIMEOUT);
    return;
  }

  // -------------------------------- consumers --------------------------------
  // Prologue: the two query rows of this head (and, where this CTA appends, the
  // new K and V row) into shared memory; warps 0..3 work in parallel.
  [[maybe_unused]] int new_page = -1;
  if constexpr (kFused) {
    if (warp < 4) {
      if (p.raw_from_predecessor) {
        pdl_wait_for_predecessor();
        load_head<D>(raw_row, lane, x);
      }
      __nv_bfloat16 y[D / 32];
      if (warp < 2) {
        if (new_pos >= 0) {
          prep_weighted_rope_values<D, D, kIeee>(y, x, p.q_norm_weight,
                                                 p.cos + int64_t(new_pos) * (D / 2),
                                                 p.sin + int64_t(new_pos) * (D / 2), lane);
          store_head<D>(s_q + warp * kQStride, y, lane);
        } else {  // no append for this sequence: q is what the caller left there
          reinterpret_cast<uint4 *>(s_q + warp * kQStride)[lane] = __ldg(
              reinterpret_cast<const uint4 *>(
                  p.q_prepared + (int64_t(b) * p.q_heads + h * 2 + warp) * D) +
              lane);
        }
      } else if (preps_kv) {
        // the row's page: unmapped means nothing is appended
        // (src/gemma4_flash_attention_decode.cu:333-338)
        const int e = __ldg(p.page_table + int64_t(b) * cfg.max_pages_per_seq +
                            (new_pos / cfg.page_size) % cfg.max_pages_per_seq);
        new_page = (e >= 0 && e < cfg.num_pages) ? e : -1;
        if (warp == 2) {
          prep_weighted_rope_values<D, D, kIeee>(y, x, p.k_norm_weight,
                                                 p.cos + int64_t(new_pos) * (D / 2),
                                                 p.sin + int64_t(new_pos) * (D / 2), lane);
        } else {
          prep_scale_free_values<D, kIeee>(y, x);
        }
        store_head<D>(s_new + (warp - 2) * D, y, lane);
      }
    }
    // Rows of the unfinished steps before this one that fall into this CTA's
    // range: prepared here like the new row (task 2 j is step j's K row, 2 j + 1
    // its V row; warps 4..7 start on them while warps 0..3 prepare q, K and V).
    if (p.fwd_count > 0) {
#pragma unroll
      for (int j = 0; j < kMaxForward; ++j) {
        if (j >= p.fwd_count) break;
#pragma unroll
        for (int kind = 0; kind < 2; ++kind) {
          if (((2 * j + kind + 4) & 7) != warp) continue;
          const int pos = __ldg(p.fwd_pos[j] + b);
          const bool here = pos >= first && pos < len && pos / ST >= c0 && pos / ST < c1;
          if (kind == 0 && lane == 0) s_fwd_pos[j] = here ? pos : -1;
          if (!here) continue;
          const __nv_bfloat16 *src =
              (kind == 0 || p.fwd_v[j] == nullptr ? p.fwd_k[j] : p.fwd_v[j]) +
              (int64_t(b) * H + h) * D;
          float xf[D / 32];
          load_head<D>(src, lane, xf);
          __nv_bfloat16 yf[D / 32];
          if (kind == 0) {
            prep_weighted_rope_values<D, D, kIeee>(yf, xf, p.k_norm_weight,
                                                   p.cos + int64_t(pos) * (D / 2),
                                                   p.sin + int64_t(pos) * (D / 2), lane);
          } else {
            prep_scale_free_values<D, kIeee>(yf, xf);
          }
          store_head<D>(s_fwd + (2 * j + kind) * D, yf, lane);
        }
      }
    }
  } else {
    pdl_wait_for_predecessor();  // q comes from the append
    if (warp < 2) {
      reinterpret_cast<uint4 *>(s_q + warp * kQStride)[lane] = __ldg(
          reinterpret_cast<const uint4 *>(
              p.q + (int64_t(b) * p.q_heads + h * 2 + warp) * D) +
          lane);
    }
  }
  named_barrier_sync(1, kTileConsumerThreads);

  bool ok = true;
  float *x_acc = reinterpret_cast<float *>(smem);  // [kStates][2][256], in the idle ring
  float *x_m = x_acc + kStates * 2 * D;            // [kStates][2]
  float *x_l = x_m + kStates * 2;                  // [kStates][2]
  if constexpr (kMma) {
    // Chunks alternate between the two groups of four warps; within a group,
    // warp (kh, dh) takes key half kh and output-dim half dh of the stage. Every
    // warp waits for and releases every stage, its group's or not: a warp that
    // skipped the other group's stages could meet a barrier two phases on, and a
    // parity wait cannot tell that from the phase it is waiting for.
    const int qd = warp >> 2;
    const int kh = (warp >> 1) & 1;
    const int dh = warp & 1;
    const MmaLane ln(lane, kh, p.tile_tokens, smem_u32(s_q));
    MmaState st;
    st.reset();
    if ((ring.base & 1023u) != 0u) {  // the swizzle is a function of the address
      ok = false;
    }
    for (int c = 0; ok && c < nchunks; ++c) {
      const int stage = c % kStages;
      if (!mbar_wait_bounded(ring.full_bar(stage), uint32_t(c / kStages) & 1u)) {
        ok = false;
        break;
      }
      if ((c & 1) != qd) {  // the other group's stage
        if (lane == 0) mbar_arrive(ring.empty_bar(stage));
        continue;
      }
      const uint32_t mask = uint32_t(ring.masks()[stage]);
      if constexpr (kFused) {
        // The stage that holds the new key: the tile brought whatever the cache
        // had there. Both warps that read the key's half replace the row by the
        // prepared one before they read it -- the same bytes twice, so neither
        // has to wait for the other. The slot's mask bit is set exactly when its
        // page is mapped.
        auto patch = [&](int pos, const __nv_bfloat16 *kv_rows) {
          const int slot = pos % ST;
          if (kh == slot / 16 && ((mask >> slot) & 1u) != 0u) {
            const uint4 *rows = reinterpret_cast<const uint4 *>(kv_rows);
            const int tb = p.tile_tokens;  // chunk lane of the row: block lane / 8, swizzled
            uint8_t *k_row = smem + stage * T::kStageBytes + (slot / tb) * tb * T::kRowBytes +
                             (lane >> 3) * tb * 128 + (slot % tb) * 128 +
                             (((lane & 7) ^ (slot & 7)) << 4);
            *reinterpret_cast<uint4 *>(k_row) = rows[lane];
            *reinterpret_cast<uint4 *>(k_row + T::kStageTensorBytes) = rows[32 + lane];
            fence_proxy_async_shared();  // the next fill of the stage is a bulk copy
            __syncwarp();
          }
        };
        if (owns_new && c0 + c == new_pos / ST) patch(new_pos, s_new);
        // ... and so do the rows the unfinished steps before this one append
        for (int j = 0; j < p.fwd_count; ++j) {
          const int pos = s_fwd_pos[j];
          if (pos >= 0 && pos / ST == c0 + c) patch(pos, s_fwd + 2 * j * D);
        }
      }
      const uint32_t mask16 = (mask >> (kh * 16)) & 0xffffu;
      if (mask16 != 0u) {
        consume_half_mma(st, ln, ring.k_stage(stage), mask16, dh, p.scale_log2);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(ring.empty_bar(stage));
    }
    if (!ok && lane == 0) {
      set_status(p.status, B200KV_STATUS_WAIT_TIMEOUT);
      s_flag[0] = 1;
    }
    // The warp's state into the exchange area: the two dim halves of a (group,
    // key half) make one partial state.
    float l = st.l_lane + __shfl_xor_sync(0xffffffffu, st.l_lane, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    named_barrier_sync(1, kTileConsumerThreads);  // every warp is past its last stage
    const int state = qd * 2 + kh;
    const int g8 = lane >> 2;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if ((j & 3) == (lane & 3)) {  // the four lanes of a row hold copies: one tile each
        const int dim = dh * 128 + 16 * j + g8;
        x_acc[(state * 2 + 0) * D + dim] = st.acc[j][0];
        x_acc[(state * 2 + 1) * D + dim] = st.acc[j][1];
        x_acc[(state * 2 + 0) * D + dim + 8] = st.acc[j][2];
        x_acc[(state * 2 + 1) * D + dim + 8] = st.acc[j][3];
      }
    }
    if (dh == 0 && (lane == 0 || lane == 4)) {  // lane 4 g scores query g
      x_m[state * 2 + g8] = g8 == 0 ? st.m[0] : st.m[1];
      x_l[state * 2 + g8] = l;
    }
  } else {
    WarpState<T> st;
    {
      uint4 raw[2];
      raw[0] = reinterpret_cast<const uint4 *>(s_q)[lane];
      raw[1] = reinterpret_cast<const uint4 *>(s_q + D)[lane];
      st.set_q(raw, p.scale_log2);
    }
    st.reset();
    // The stage that holds the new key: the tile brought whatever the cache had
    // there; the warp that owns the token's slot replaces the row by the prepared
    // one (no other warp reads that slot). The slot's mask bit is set exactly when
    // its page is mapped.
    auto patch_new_row = [&](int c, int stage) {
      if constexpr (kFused) {
        auto patch = [&](int pos, const __nv_bfloat16 *kv_rows) {
          const int slot = pos % ST;
          if (warp == slot / kTokPerWarp && ((ring.masks()[stage] >> slot) & 1ull) != 0ull) {
            uint8_t *k_row = smem + stage * T::kStageBytes + slot * T::kRowBytes;
            const uint4 *rows = reinterpret_cast<const uint4 *>(kv_rows);
            reinterpret_cast<uint4 *>(k_row)[lane] = rows[lane];
            reinterpret_cast<uint4 *>(k_row + T::kStageTensorBytes)[lane] = rows[32 + lane];
            fence_proxy_async_shared();  // the next fill of the stage is a bulk copy
            __syncwarp();
          }
        };
        if (owns_new && c0 + c == new_pos / ST) patch(new_pos, s_new);
        for (int j = 0; j < p.fwd_count; ++j) {  // rows of the unfinished steps before this one
          const int pos = s_fwd_pos[j];
          if (pos >= 0 && pos / ST == c0 + c) patch(pos, s_fwd + 2 * j * D);
        }
      }
    };
    for (int c = 0; c < nchunks; ++c) {
      const int stage = c % kStages;
      if (!mbar_wait_bounded(ring.full_bar(stage), uint32_t(c / kStages) & 1u)) {
        ok = false;
        break;
      }
      patch_new_row(c, stage);
      consume_stage<T>(st, ring, stage, 0, warp, lane);
      __syncwarp();
      if (lane == 0) mbar_arrive(ring.empty_bar(stage));
    }
    if (!ok && lane == 0) {
      set_status(p.status, B200KV_STATUS_WAIT_TIMEOUT);
      s_flag[0] = 1;
    }
    // The warps' states into the ring (idle once every warp is past its last
    // stage).
    float l[2];
    st.denominators(l, lane);
    named_barrier_sync(1, kTileConsumerThreads);
#pragma unroll
    for (int g = 0; g < 2; ++g) {
      float4 *dst = reinterpret_cast<float4 *>(x_acc + (warp * 2 + g) * D) + lane * 2;
      dst[0] = make_float4(st.acc[g][0], st.acc[g][1], st.acc[g][2], st.acc[g][3]);
      dst[1] = make_float4(st.acc[g][4], st.acc[g][5], st.acc[g][6], st.acc[g][7]);
      if (lane == 0) {
        x_m[warp * 2 + g] = st.m[g];
        x_l[warp * 2 + g] = l[g];
      }
    }
  }
  // Merge of the states: thread t ends with dim t of both rows.
  named_barrier_sync(1, kTileConsumerThreads);
  const int t = int(threadIdx.x);  // 0..255: the dim this thread finishes
  float M[2], L[2], A[2];
#pragma unroll
  for (int g = 0; g < 2; ++g) {
    M[g] = -INFINITY;
#pragma unroll
    for (int w = 0; w < kStates; ++w) M[g] = fmaxf(M[g], x_m[w * 2 + g]);
    L[g] = 0.0f;
    A[g] = 0.0f;
#pragma unroll
    for (int w = 0; w < kStates; ++w) {
      const float mw = x_m[w * 2 + g];
      const float wt = mw == -INFINITY ? 0.0f : ex2_approx(mw - M[g]);
      L[g] = fmaf(x_l[w * 2 + g], wt, L[g]);
      A[g] = fmaf(x_acc[(w * 2 + g) * D + t], wt, A[g]);
    }
  }

  // Everything below writes memory the preceding kernel may still use.
  pdl_wait_for_predecessor();
  if (s_flag[0] != 0) return;  // a wait ran out in this CTA: the status word says so

  if constexpr (kFused) {
    if (warp < 2 && r == 0 && new_pos >= 0) {
      reinterpret_cast<uint4 *>(p.q_prepared +
                                (int64_t(b) * p.q_heads + h * 2 + warp) * D)[lane] =
          reinterpret_cast<const uint4 *>(s_q + warp * kQStride)[lane];
    } else if ((warp == 2 || warp == 3) && preps_kv && new_page >= 0) {
      const int64_t off =
          cache_offset(cfg, p.layer, new_page,
                       new_pos - (new_pos / cfg.page_size) * cfg.page_size, h, 0);
      __nv_bfloat16 *dst = (warp == 2 ? p.cache_k : p.cache_v) + off;
      reinterpret_cast<uint4 *>(dst)[lane] =
          reinterpret_cast<const uint4 *>(s_new + (warp - 2) * D)[lane];
    }
  }

  // A ticket: the CTA's writes are complete in every thread's view after the
  // barrier; one acq_rel atomic at GPU scope then publishes them (release: the
  // writes the barrier ordered before it) and, for the CTA that arrives last,
  // makes the other CTAs' writes visible (acquire). True in the last arriver.
  auto last_to_arrive = [&](uint32_t *counter, int expected) {
    named_barrier_sync(1, kTileConsumerThreads);
    if (t == 0) {
      uint32_t before;
      asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], %2;"
                   : "=r"(before)
                   : "l"(counter), "r"(1u)
                   : "memory");
      s_flag[1] = before == uint32_t(expected - 1) ? 1 : 0;
    }
    named_barrier_sync(1, kTileConsumerThreads);
    return s_flag[1] != 0;
  };
  auto write_rows = [&]() {
#pragma unroll
    for (int g = 0; g < 2; ++g) {
      const int64_t row = int64_t(b) * p.q_heads + h * 2 + g;
      const float inv = L[g] > 0.0f ? 1.0f / L[g] : 0.0f;
      p.out[row * D + t] = __float2bfloat16_rn(A[g] * inv);
      if (p.lse != nullptr && t == 0) {
        p.lse[row] = L[g] > 0.0f ? (M[g] + lg2_approx(L[g])) * 0.6931471805599453f
                                 : -INFINITY;
      }
    }
  };
  // The exchange that may follow: a final CTA stores its two rows into this
  // rank's slot of every rank's gather buffer (plain peer stores over NVLink, no
  // multicast); the last final CTA on this GPU -- a counter next to the flags --
  // fences, publishes the call's epoch to every peer and waits, bounded, until
  // every peer's epoch has arrived here. "This kernel is complete" then means
  // "every rank's rows are in this GPU's buffer", without another launch.
  const PeerEpilogue &peer = p.peer;
  const uint32_t epoch = peer.world > 0 ? *peer.epoch + 1u : 0u;
  const int64_t half = int64_t(epoch & 1u) * peer.world;
  auto peer_store = [&](int64_t row, int word, uint2 v) {  // 8 bytes of a row of this rank
    for (int rk = 0; rk < peer.world; ++rk) {
      uint2 *dst = reinterpret_cast<uint2 *>(peer.data[rk] + (half + peer.rank) * peer.slot_packs);
      dst[row * (D / 4) + word] = v;
    }
  };
  auto peer_finish = [&]() {  // all threads of the consumer warps call it
    if (peer.world <= 0) return;
    __threadfence_system();
    if (!last_to_arrive(peer.done, p.batch_count * H)) return;
    if (t < peer.world) {
      __threadfence_system();
      st_release_sys(peer.flags[t] + half + peer.rank, epoch);
      const uint32_t *mine = peer.flags[peer.rank] + half + t;
      const long long start = clock64();
      while (int32_t(ld_acquire_sys(mine) - epoch) < 0) {
        if (clock64() - start > peer.wait_clocks) {
          set_status(p.status, B200KV_STATUS_WAIT_TIMEOUT);
          break;
        }
        __nanosleep(100);
      }
    }
    named_barrier_sync(1, kTileConsumerThreads);
    if (t == 0) {
      *peer.epoch = epoch;
      *peer.done = 0u;
    }
  };
  if (r_eff <= 1) {  // the only range of its (sequence, head), or no live key
    write_rows();
    for (int rk = 0; rk < peer.world; ++rk) {  // the same two rows for the peers, a dim per thread
      __nv_bfloat16 *dst = reinterpret_cast<__nv_bfloat16 *>(
          peer.data[rk] + (half + peer.rank) * peer.slot_packs);
#pragma unroll
      for (int g = 0; g < 2; ++g) {
        const float inv = L[g] > 0.0f ? 1.0f / L[g] : 0.0f;
        dst[(int64_t(b) * p.q_heads + h * 2 + g) * D + t] = __float2bfloat16_rn(A[g] * inv);
      }
    }
    peer_finish();
    return;
  }

  // One partial of two rows, then the ticket: the last CTA of the pair merges.
  const int64_t pair = (int64_t(b) * H + h) * p.ranges;  // first slot of the pair
#pragma unroll
  for (int g = 0; g < 2; ++g) {
    const int64_t slot = (pair + r) * 2 + g;
    p.partial_acc[slot * D + t] = A[g];
    if (t == 0) {
      p.partial_m[slot] = M[g];
      p.partial_l[slot] = L[g];
    }
  }
  // Merge of up to 32 partials at slots first, first + stride, ... Thread t owns
  // four dims (t % 64) of row (t / 64) % 2 and every second partial, parity
  // t / 128: all its loads are independent and go out together, before the
  // weights are known. Lane i of every warp holds partial i's (m, l) of the
  // warp's row: maximum, weights and denominator by shuffles. The partials were
  // written by other SMs: read them past L1 (a line of the same scratch may sit
  // there from an earlier launch). Afterwards the threads of parity 0 hold the
  // merged (top, sum, value) of their row and dims.
  constexpr int kPre = kMergeGroup / 2;
  const int col = t & 63;
  const int g = (t >> 6) & 1;
  const int parity = t >> 7;
  float top = -INFINITY;
  float sum = 0.0f;
  float4 value = make_float4(0.f, 0.f, 0.f, 0.f);
  float4 *x_sum = reinterpret_cast<float4 *>(x_acc);  // the warps' exchange area is idle
  auto merge = [&](int64_t first, int stride, int count) {
    const float4 *mine = reinterpret_cast<const float4 *>(p.partial_acc) + col;
    float4 pre[kPre];
#pragma unroll
    for (int j = 0; j < kPre; ++j) {
      const int i = parity + 2 * j;
      pre[j] = i < count ? __ldcg(mine + ((first + int64_t(i) * stride) * 2 + g) * (D / 4))
                         : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    const int64_t ml = (first + int64_t(lane) * stride) * 2 + g;
    const float mi = lane < count ? __ldcg(p.partial_m + ml) : -INFINITY;
    const float li = lane < count ? __ldcg(p.partial_l + ml) : 0.0f;
    top = mi;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, o));
    const float wi = li > 0.0f ? ex2_approx(mi - top) : 0.0f;
    sum = li * wi;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    value = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int j = 0; j < kPre; ++j) {
      const float w = __shfl_sync(0xffffffffu, wi, (parity + 2 * j) & 31);
      if (parity + 2 * j < count && w > 0.0f) {  // a partial without mass is dropped
        value.x = fmaf(pre[j].x, w, value.x);
        value.y = fmaf(pre[j].y, w, value.y);
        value.z = fmaf(pre[j].z, w, value.z);
        value.w = fmaf(pre[j].w, w, value.w);
      }
    }
    named_barrier_sync(1, kTileConsumerThreads);  // x_sum is free (a merge before this one)
    if (parity == 1) x_sum[t - 128] = value;
    named_barrier_sync(1, kTileConsumerThreads);
    if (parity == 0) {
      const float4 o = x_sum[t];
      value.x += o.x;
      value.y += o.y;
      value.z += o.z;
      value.w += o.w;
    }
  };
  auto write_merged_rows = [&]() {
    if (parity == 0) {
      const float inv = sum > 0.0f ? 1.0f / sum : 0.0f;
      const int64_t row = int64_t(b) * p.q_heads + h * 2 + g;
      const __nv_bfloat162 lo = __floats2bfloat162_rn(value.x * inv, value.y * inv);
      const __nv_bfloat162 hi = __floats2bfloat162_rn(value.z * inv, value.w * inv);
      const uint2 packed = make_uint2(*reinterpret_cast<const uint32_t *>(&lo),
                                      *reinterpret_cast<const uint32_t *>(&hi));
      reinterpret_cast<uint2 *>(p.out + row * D)[col] = packed;
      peer_store(row, col, packed);
      if (p.lse != nullptr && col == 0) {
        p.lse[row] = sum > 0.0f ? (top + lg2_approx(sum)) * 0.6931471805599453f : -INFINITY;
      }
    }
  };
  // Tickets: one word per (sequence, head) for the pair, then kMaxMergeGroups
  // words per pair for its groups of kMergeGroup ranges.
  uint32_t *pair_ticket = p.ticket + (int64_t(b) * H + h);
  const int groups = div_up(r_eff, kMergeGroup);
  if (groups == 1) {
    if (!last_to_arrive(pair_ticket, r_eff)) return;
    merge(pair, 1, r_eff);
    write_merged_rows();
    if (t == 0) *pair_ticket = 0u;  // ready for the next launch
    peer_finish();
    return;
  }
  // More than 32 ranges (long contexts on few heads): the last CTA of each group
  // of 32 merges the group into the group's first slot, the last group to finish
  // merges the groups. One CTA never reads more than 32 + groups partials.
  const int group = r / kMergeGroup;
  const int group_size = min(kMergeGroup, r_eff - group * kMergeGroup);
  uint32_t *group_ticket = p.ticket + int64_t(p.batch_count) * H +
                           (int64_t(b) * H + h) * kMaxMergeGroups + group;
  if (!last_to_arrive(group_ticket, group_size)) return;
  const int64_t group_slot = pair + int64_t(group) * kMergeGroup;
  merge(group_slot, 1, group_size);
  if (parity == 0) {  // every partial of the group has been read: its first slot takes the sum
    reinterpret_cast<float4 *>(p.partial_acc)[(group_slot * 2 + g) * (D / 4) + col] = value;
    if (col == 0) {
      p.partial_m[group_slot * 2 + g] = top;
      p.partial_l[group_slot * 2 + g] = sum;
    }
  }
  if (t == 0) *group_ticket = 0u;
  if (!last_to_arrive(pair_ticket, groups)) return;
  merge(pair, kMergeGroup, groups);
  write_merged_rows();
  if (t == 0) *pair_ticket = 0u;
  peer_finish();
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

// The cache as [dim][head][page offset][layer * pages + page] bf16 with tiles of
// (256 dims, one head, tile_tokens offsets, one page): 512-byte rows, dense in
// shared memory. Swizzled (the tensor-core variant): boxes of 64 dims, 128-byte
// rows with the 128-byte swizzle.
bool make_cache_map(CUtensorMap *map, const __nv_bfloat16 *base,
                    const Gemma4KvCacheConfig &c, int tile_tokens, bool swizzled) {
  EncodeTiledFn encode = encode_tiled_fn();
  if (encode == nullptr) return false;
  const cuuint64_t row = cuuint64_t(c.head_dim) * 2;
  if (swizzled) {
    // [64 dims][page offset][block of 64 dims][head][layer * pages + page]: a box of
    // (64, tile_tokens, 4, 1, 1) is the tile as four blocks of 128-byte rows.
    const cuuint64_t dims[5] = {64, cuuint64_t(c.page_size), cuuint64_t(c.head_dim) / 64,
                                cuuint64_t(c.num_heads),
                                cuuint64_t(c.num_layers) * cuuint64_t(c.num_pages)};
    const cuuint64_t strides[4] = {row * c.num_heads, 128, row,
                                   row * c.num_heads * c.page_size};
    const cuuint32_t box[5] = {64, cuuint32_t(tile_tokens), cuuint32_t(c.head_dim) / 64, 1, 1};
    const cuuint32_t elem_strides[5] = {1, 1, 1, 1, 1};
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5,
                  const_cast<__nv_bfloat16 *>(base), dims, strides, box, elem_strides,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
  }
  const cuuint64_t dims[4] = {cuuint64_t(c.head_dim), cuuint64_t(c.num_heads),
                              cuuint64_t(c.page_size),
                              cuuint64_t(c.num_layers) * cuuint64_t(c.num_pages)};
  const cuuint64_t strides[3] = {row, row * c.num_heads, row * c.num_heads * c.page_size};
  const cuuint32_t box[4] = {cuuint32_t(c.head_dim), 1, cuuint32_t(tile_tokens), 1};
  const cuuint32_t elem_strides[4] = {1, 1, 1, 1};
  return encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4,
                const_cast<__nv_bfloat16 *>(base), dims, strides, box, elem_strides,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int tile_tokens_of(int page_size) {
  const int tb = std::min(page_size, kMaxTileTokens);
  // tiles tile a page and a stage: 32 % tb == 0 and page_size % tb == 0
  if (tb < 2 || kTileStage % tb != 0 || page_size % tb != 0) return 0;
  return tb;
}

// B200KV_PAGETILE: "0" never, "1" wherever the geometry allows, unset: the
// built-in choice (pagetile_preferred).
int pagetile_override() {
  static const int mode = [] {
    const char *v = std::getenv("B200KV_PAGETILE");
    if (v == nullptr) return -1;
    return std::strcmp(v, "0") == 0 ? 0 : 1;
  }();
  return mode;
}

// B200KV_PAGETILE_RANGES=n: tuning aid, n key ranges per (sequence, head).
int pagetile_ranges_override() {
  static const int n = [] {
    const char *v = std::getenv("B200KV_PAGETILE_RANGES");
    return v == nullptr ? 0 : std::atoi(v);
  }();
  return n;
}

// B200KV_PAGETILE_MMA=0: tuning aid, the scalar arithmetic for every page size.
bool pagetile_mma_allowed() {
  static const bool allowed = [] {
    const char *v = std::getenv("B200KV_PAGETILE_MMA");
    return v == nullptr || std::strcmp(v, "0") != 0;
  }();
  return allowed;
}

template <int kMode, bool kMma>
cudaError_t launch_pagetile_variant(const TileParams &p, const CUtensorMap &map_k,
                                    const CUtensorMap &map_v, cudaStream_t stream) {
  cudaError_t st = cudaFuncSetAttribute(decode_pagetile_kernel<kMode, kMma>,
                                        cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        kTileSmemBytes);
  if (st != cudaSuccess) return st;
  const int64_t ctas = int64_t(p.batch_count) * p.ranges * p.cfg.num_heads;
  return launch_pdl(decode_pagetile_kernel<kMode, kMma>, dim3(unsigned(ctas)),
                    dim3(kTileThreads), kTileSmemBytes, stream, p, map_k, map_v);
}

template <int kMode>
cudaError_t launch_pagetile(const TileParams &p, bool mma, const CUtensorMap &map_k,
                            const CUtensorMap &map_v, cudaStream_t stream) {
  return mma ? launch_pagetile_variant<kMode, true>(p, map_k, map_v, stream)
             : launch_pagetile_variant<kMode, false>(p, map_k, map_v, stream);
}

}  // namespace

bool decode_pagetile_supported(const Gemma4KvCacheConfig &c, int q_heads,
                               int batch_count) {
  return c.head_dim == 256 && c.num_heads >= 1 && c.num_heads <= 64 &&
         q_heads == 2 * c.num_heads && tile_tokens_of(c.page_size) > 0 &&
         batch_count >= 1 && int64_t(batch_count) * c.num_heads <= (1 << 20);
}

bool decode_pagetile_preferred(const Gemma4KvCacheConfig &c, int q_heads,
                               int batch_count, bool has_ticket) {
  if (!has_ticket || !decode_pagetile_supported(c, q_heads, batch_count)) return false;
  const int forced = pagetile_override();
  if (forced >= 0) return forced == 1;
  // Ranges are cut per sequence: chosen where the sequences' live keys are equal
  // by construction (a sliding window) or there is one sequence; small jobs only
  // -- a big batch is bandwidth-bound and streams best through the balanced
  // partition.
  if (c.window_size > 0) return batch_count <= kPagetileMaxBatch;
  if (batch_count != 1) return false;
  // One sequence on a linear cache. Fewer than 8 KV heads (the cache of a
  // KV-head-sharded rank): the alternative is three launches of the fixed-split
  // kernels. 8 heads: up to kPagetileMaxLinearKeys of capacity; a longer context
  // is a bandwidth job again (131072 keys: 169 us balanced, 171 here).
  return c.num_heads < 8 ||
         int64_t(c.max_pages_per_seq) * c.page_size <= kPagetileMaxLinearKeys;
}

cudaError_t decode_layer_step_pagetile_bf16(const AppendArgs *ap, const DecodeArgs &a,
                                            uint32_t *ticket, cudaStream_t stream,
                                            const PeerEpilogue *peer) {
  const Gemma4KvCacheConfig &c = a.cfg;
  cudaError_t st = validate_decode_args(a);
  if (st != cudaSuccess) return st;
  if (ap != nullptr) {
    st = validate_append_args(*ap);
    if (st != cudaSuccess) return st;
    if (ap->rotary_dim != 256 || ap->q_heads != a.q_heads ||
        ap->batch_count != a.batch_count || ap->cache_layer != a.layer ||
        ap->page_table != a.page_table || ap->q_prepared != a.q ||
        ap->cache_k != a.cache_k || ap->cache_v != a.cache_v ||
        std::memcmp(&ap->cfg, &c, sizeof(c)) != 0 ||
        (reinterpret_cast<uintptr_t>(ap->q_prepared) & 15u) != 0) {
      return cudaErrorInvalidValue;
    }
  }
  if (ticket == nullptr || !decode_pagetile_supported(c, a.q_heads, a.batch_count)) {
    return cudaErrorInvalidValue;
  }
  int device = 0, sm_count = 0;
  st = cudaGetDevice(&device);
  if (st != cudaSuccess) return st;
  st = cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device);
  if (st != cudaSuccess) return st;

  TileParams p = {};
  p.out = a.out;
  p.lse = a.lse;
  p.q = a.q;
  p.cache_k = const_cast<__nv_bfloat16 *>(a.cache_k);
  p.cache_v = const_cast<__nv_bfloat16 *>(a.cache_v);
  p.cfg = c;
  p.page_table = a.page_table;
  p.seq_lengths = a.seq_lengths;
  p.layer = a.layer;
  p.scale_log2 = a.softmax_scale * 1.4426950408889634f;
  p.batch_count = a.batch_count;
  p.q_heads = a.q_heads;
  p.partial_m = a.partial_m;
  p.partial_l = a.partial_l;
  p.partial_acc = a.partial_acc;
  p.ticket = ticket;
  p.status = a.status;
  p.tile_tokens = tile_tokens_of(c.page_size);
  if (peer != nullptr) p.peer = *peer;
  // Ranges per (sequence, head): enough CTAs for two per SM, no more than the
  // scratch holds (batch * q_heads * num_splits rows = two rows per range) or
  // the chunks a sequence can have.
  const int64_t pairs = int64_t(a.batch_count) * c.num_heads;
  const int64_t span = c.window_size > 0 ? int64_t(c.window_size)
                                         : int64_t(c.max_pages_per_seq) * c.page_size;
  const int64_t max_chunks = span / kTileStage + 2;
  // ... and at least two chunks per CTA where a sequence is that long: a CTA's
  // fixed cost (prologue, merge of its warps, its partial) is that of a chunk or
  // two, and every further partial lengthens the last CTA's merge.
  // (a launch of a run of overlapping launches: one CTA per SM, so that the next
  // launch of the run streams beside this one instead of waiting for its CTAs
  // to leave -- a CTA stays until the launch before its own is complete)
  const int64_t grid_target = (ap != nullptr && ap->chained ? 1 : 2) * int64_t(sm_count);
  int64_t ranges = std::max<int64_t>(1, grid_target / pairs);
  ranges = std::min<int64_t>({ranges, int64_t(kMaxRanges), std::max<int64_t>(1, max_chunks / 2),
                              std::max<int64_t>(1, a.num_splits)});
  // up to 32 partials per pair are merged in one round of loads; a few more
  // ranges than that do not pay for the second round
  if (ranges > 32 && ranges < 48) ranges = 32;
  if (pagetile_ranges_override() > 0) {
    ranges = std::min<int64_t>({int64_t(pagetile_ranges_override()), int64_t(kMaxRanges),
                                std::max<int64_t>(1, a.num_splits)});
  }
  if (ranges > 1 && (a.partial_m == nullptr || a.partial_l == nullptr ||
                     a.partial_acc == nullptr)) {
    return cudaErrorInvalidValue;
  }
  p.ranges = int32_t(ranges);
  // Tiles of at least 8 tokens go through the tensor cores (swizzled rows);
  // smaller pages keep the scalar arithmetic.
  const bool mma = p.tile_tokens >= kMmaMinTileTokens && pagetile_mma_allowed();
  CUtensorMap map_k, map_v;
  if (!make_cache_map(&map_k, a.cache_k, c, p.tile_tokens, mma) ||
      !make_cache_map(&map_v, a.cache_v, c, p.tile_tokens, mma)) {
    return cudaErrorInvalidValue;
  }
  if (ap == nullptr) return launch_pagetile<kAttentionOnly>(p, mma, map_k, map_v, stream);
  p.raw_q = ap->q;
  p.raw_k = ap->k;
  p.raw_v = ap->v;
  p.q_norm_weight = ap->q_norm_weight;
  p.k_norm_weight = ap->k_norm_weight;
  p.cos = ap->cos;
  p.sin = ap->sin;
  p.token_position = ap->token_position;
  p.q_prepared = ap->q_prepared;
  p.raw_from_predecessor = ap->raw_from_predecessor ? 1 : 0;
  p.steps_in_flight = std::max(0, ap->steps_in_flight);
  p.fwd_count = std::min<int32_t>(std::max(0, ap->forward_count), kMaxForward);
  for (int j = 0; j < p.fwd_count; ++j) {
    if (ap->forward_k[j] == nullptr || ap->forward_position[j] == nullptr) return cudaErrorInvalidValue;
    p.fwd_k[j] = ap->forward_k[j];
    p.fwd_v[j] = ap->forward_v[j];
    p.fwd_pos[j] = ap->forward_position[j];
  }
  p.release_early = ap->release_early ? 1 : 0;
  return ap->norm_mode == B200KV_NORM_IEEE
             ? launch_pagetile<kFusedIeee>(p, mma, map_k, map_v, stream)
             : launch_pagetile<kFusedApprox>(p, mma, map_k, map_v, stream);
}

}  // namespace b200kv

// Prompt attention for head_dim 256 on the fifth-generation tensor cores:
// tcgen05.mma with both operands in shared memory and the accumulators in
// tensor memory. Same contract as prefill_attention.cu (which keeps the
// mma.sync path for head_dim 512 and as the comparison arm): each sequence's
// query row r sees its own keys c <= r and, with a window, c >= r - window + 1
// (src/gemma4_flash_attention_prefill.cu:502-540).
//
// One CTA = 128 query rows of one query head, 128 threads, thread = row.
//   shared memory: Q (128 x 256), two stages of K and of V (64 keys x 256
//     each), P (128 x 64), all bf16, all stored as column blocks of 64 elements
//     (128 bytes per row) whose 16-byte chunks are XOR-permuted by the row index
//     -- the canonical 128-byte-swizzled layout that tcgen05 smem descriptors
//     name, K-major for Q, K and P, MN-major for V. The tiles are filled with
//     cp.async (16 bytes per thread), so no tensor maps are needed.
//   tensor memory: S[2] (128 lanes x 64 columns fp32, double-buffered) and O
//     (128 x 256 fp32); lane = query row.
//   per 64-key tile: 16 MMAs (M 128, N 64, K 16) give S = Q K^T; every thread
//     reads its row of S with tcgen05.ld, does the online softmax on it without
//     any shuffle, writes the bf16 weights as its row of P; 4 MMAs (M 128,
//     N 256, K 16) add P V to O. One elected thread issues the MMAs and commits
//     them to mbarriers; the scores of the next tile are computed while the
//     threads work on the softmax of this one.
//   The running maximum a row scales by is only raised when the tile's maximum
//     exceeds it by more than 2^8 (the weights then stay below 256, exact enough
//     in bf16 and fp32), so the rescaling of O in tensor memory is rare.
// Every wait is bounded (tens of milliseconds: a tile takes microseconds); a wait
// that runs out records which one in a device-side fault word, makes the CTA
// skip to the exit, which always frees the tensor memory, and makes the CTAs
// that start later return at once. The host clears the word before each launch
// and reads it through prefill_attention_sm100_fault().
#include "common.cuh"
#include "kernels.cuh"

namespace b200kv {

namespace {

constexpr int kD = 256;
constexpr int kBlockM = 128;
constexpr int kBlockN = 64;
constexpr int kThreads = 128;
constexpr int kQBytes = kBlockM * kD * 2;         // 64 KiB: 4 column blocks of 16 KiB
constexpr int kKvTileBytes = kBlockN * kD * 2;    // 32 KiB: 4 column blocks of 8 KiB
constexpr int kPBytes = kBlockM * kBlockN * 2;    // 16 KiB: one column block
constexpr int kSmemBytes = kQBytes + 4 * kKvTileBytes + kPBytes + 1024;  // + alignment slack
constexpr uint32_t kTmemColumns = 512;            // S[2] at 0 and 64, O at 128
constexpr uint32_t kTmemO = 128;
constexpr float kRescaleSlack = 8.0f;             // log2 units
constexpr long long kTileWaitClocks = 1ll << 26;  // ~35 ms

// 0, or which wait ran out: 1 P V of the previous tile, 2 scores, 3 last P V
__device__ int g_prefill_sm100_fault;

struct Sm100PrefillParams {
  __nv_bfloat16 *out;
  const __nv_bfloat16 *q;
  const __nv_bfloat16 *k;
  const __nv_bfloat16 *v;
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
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&r)[32]) {
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
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float (&r)[32]) {
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

__device__ __forceinline__ void cp16(uint32_t dst, const void *src, bool valid) {
  const int bytes = valid ? 16 : 0;  // 0: zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void cp_commit() {
  asm volatile("cp.async.commit_group;" ::: "memory");
}
__device__ __forceinline__ void cp_wait_all() {
  asm volatile("cp.async.wait_group 0;" ::: "memory");
}

// All threads: `rows` rows of 256 elements (row r at src + r * stride elements,
// zero beyond valid_rows) into a tile of four column blocks of `rows` rows.
__device__ __forceinline__ void load_rows(uint32_t dst, const __nv_bfloat16 *src,
                                          int64_t stride, int rows,
                                          int valid_rows) {
  const int chunks = rows * 32;
  for (int i = int(threadIdx.x); i < chunks; i += kThreads) {
    const int r = i >> 5;
    const int c = i & 31;
    const bool valid = r < valid_rows;
    const __nv_bfloat16 *from = src + (valid ? int64_t(r) * stride : 0) + c * 8;
    cp16(dst + uint32_t(c >> 3) * uint32_t(rows) * 128u + uint32_t(r) * 128u +
             (uint32_t((c & 7) ^ (r & 7)) << 4),
         from, valid);
  }
}

__global__ __launch_bounds__(kThreads, 1) void prefill_attention_sm100_kernel(
    Sm100PrefillParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t s_bars[3];  // S[0], S[1] ready; P V done
  __shared__ uint32_t s_tmem_base;
  // 128-byte-swizzled tiles want 1024-byte alignment
  const uint32_t smem0 = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t s_q = smem0;
  const uint32_t s_k = s_q + kQBytes;
  const uint32_t s_v = s_k + 2 * kKvTileBytes;
  const uint32_t s_p = s_v + 2 * kKvTileBytes;
  uint8_t *p_generic = smem_raw + (s_p - smem_u32(smem_raw));

  // an earlier CTA gave up: the whole CTA returns, on one common reading
  if (__syncthreads_or(*reinterpret_cast<volatile int *>(&g_prefill_sm100_fault) != 0)) {
    return;
  }
  const int tid = int(threadIdx.x);
  const int warp = tid >> 5;
  const int S = p.seq_len;
  const int m_block = int(gridDim.x) - 1 - int(blockIdx.x);  // longest first
  const int batch = int(blockIdx.y);
  const int head = int(blockIdx.z);
  const int kv_head = head / (p.q_heads / p.kv_heads);
  const int m0 = m_block * kBlockM;
  const int row = m0 + tid;
  const int64_t seq_row0 = int64_t(batch) * S;
  const int64_t q_stride = int64_t(p.q_heads) * kD;
  const int64_t kv_stride = int64_t(p.kv_heads) * kD;
  const __nv_bfloat16 *q_src = p.q + ((seq_row0 + m0) * p.q_heads + head) * kD;
  const __nv_bfloat16 *k_base = p.k + (seq_row0 * p.kv_heads + kv_head) * kD;
  const __nv_bfloat16 *v_base = p.v + (seq_row0 * p.kv_heads + kv_head) * kD;
  const int last_row = min(m0 + kBlockM, S) - 1;
  const int tile_hi = last_row / kBlockN;
  const int tile_lo = p.window > 0 ? max(0, m0 - p.window + 1) / kBlockN : 0;

  const uint32_t bar_s0 = smem_u32(&s_bars[0]);  // S[b] ready at bar_s0 + 8 b
  const uint32_t bar_o = smem_u32(&s_bars[2]);
  if (tid == 0) {
    mbar_init(bar_s0, 1);
    mbar_init(bar_s0 + 8, 1);
    mbar_init(bar_o, 1);
    mbar_fence_init();
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(&s_tmem_base)),
                 "r"(kTmemColumns)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::
                     : "memory");
  }
  load_rows(s_q, q_src, q_stride, kBlockM, S - m0);
  load_rows(s_k, k_base + int64_t(tile_lo) * kBlockN * kv_stride, kv_stride, kBlockN,
            S - tile_lo * kBlockN);
  load_rows(s_v, v_base + int64_t(tile_lo) * kBlockN * kv_stride, kv_stride, kBlockN,
            S - tile_lo * kBlockN);
  cp_commit();
  cp_wait_all();
  fence_proxy_async_shared();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s_tmem_base;
  const uint32_t lane_base = uint32_t(32 * warp) << 16;

  constexpr uint32_t kIdescQK = umma_idesc(kBlockN, false);
  constexpr uint32_t kIdescPV = umma_idesc(kD, true);
  // S[buf] = Q K(stage)^T: 16 steps of 16 dims; a step moves 32 bytes inside a
  // column block, four steps move to the next block
  auto issue_qk = [&](int stage, int buf) {
    const uint32_t k_tile = s_k + uint32_t(stage) * kKvTileBytes;
#pragma unroll
    for (int ks = 0; ks < kD / 16; ++ks) {
      const uint32_t blk = uint32_t(ks >> 2), in = uint32_t(ks & 3) * 32u;
      umma_bf16(tmem + uint32_t(buf) * kBlockN,
                umma_desc(s_q + blk * (kBlockM * 128u) + in, 1, 64),
                umma_desc(k_tile + blk * (kBlockN * 128u) + in, 1, 64), kIdescQK,
                ks > 0);
    }
    umma_commit(bar_s0 + 8u * uint32_t(buf));
  };
  // O (+)= P V(stage): 4 steps of 16 keys; V is MN-major: 8-key groups 1024
  // bytes apart, 64-dim blocks kBlockN * 128 bytes apart
  auto issue_pv = [&](int stage, bool accumulate) {
    const uint32_t v_tile = s_v + uint32_t(stage) * kKvTileBytes;
#pragma unroll
    for (int j = 0; j < kBlockN / 16; ++j) {
      umma_bf16(tmem + kTmemO, umma_desc(s_p + uint32_t(j) * 32u, 1, 64),
                umma_desc(v_tile + uint32_t(j) * 2048u, (kBlockN * 128u) >> 4, 64),
                kIdescPV, accumulate || j > 0);
    }
    umma_commit(bar_o);
  };

  if (tid == 0) issue_qk(0, 0);

  float m_ref = -INFINITY;  // the maximum this row's weights are scaled by
  float l_run = 0.0f;
  int fault = 0;          // which wait of this thread ran out
  bool ok = true;
  uint32_t s_phase = 0;   // bit b: parity of the next completion of S[b]
  uint32_t o_phase = 0;
  for (int tile = tile_lo; tile <= tile_hi; ++tile) {
    const int it = tile - tile_lo;
    const int stage = it & 1;
    const int buf = it & 1;
    const int k0 = tile * kBlockN;
    // P V of the previous tile done: its V stage and P are free, O is stable
    if (it > 0) {
      if (!mbar_wait_bounded(bar_o, o_phase, kTileWaitClocks)) fault = 1;
      o_phase ^= 1;
    }
    if (tile < tile_hi) {  // the next K / V tile goes into the other stage
      const int nxt = tile + 1;
      load_rows(s_k + uint32_t(stage ^ 1) * kKvTileBytes,
                k_base + int64_t(nxt) * kBlockN * kv_stride, kv_stride, kBlockN,
                S - nxt * kBlockN);
      load_rows(s_v + uint32_t(stage ^ 1) * kKvTileBytes,
                v_base + int64_t(nxt) * kBlockN * kv_stride, kv_stride, kBlockN,
                S - nxt * kBlockN);
      cp_commit();
    }
    // this tile's scores
    if (!mbar_wait_bounded(bar_s0 + 8u * uint32_t(buf), (s_phase >> buf) & 1u,
                           kTileWaitClocks)) {
      fault = 2;
    }
    s_phase ^= 1u << buf;
    tc_fence_after();
    float s[kBlockN];
    {
      float lo[32], hi[32];
      tmem_ld32(tmem + lane_base + uint32_t(buf) * kBlockN, lo);
      tmem_ld32(tmem + lane_base + uint32_t(buf) * kBlockN + 32, hi);
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        s[i] = lo[i];
        s[32 + i] = hi[i];
      }
    }
    // the next tile's keys have landed: its scores run under this softmax
    if (tile < tile_hi) {
      cp_wait_all();
      fence_proxy_async_shared();
    }
    tc_fence_before();
    // every thread has read S[buf]; the next K / V are visible to all; and the
    // CTA agrees on whether any wait ran out
    if (__syncthreads_or(fault != 0)) {
      ok = false;
      break;
    }
    if (tile < tile_hi && tid == 0) {
      tc_fence_after();
      issue_qk(stage ^ 1, buf ^ 1);
    }

    // ---- online softmax on this row
    const bool edge = k0 + kBlockN - 1 > m0 ||
                      (p.window > 0 && k0 < last_row - p.window + 1);
    float m_tile = -INFINITY;
#pragma unroll
    for (int c = 0; c < kBlockN; ++c) {
      float x = s[c] * p.scale_log2;
      if (edge) {
        const int col = k0 + c;
        if (col > row || (p.window > 0 && col < row - p.window + 1)) x = -INFINITY;
      }
      s[c] = x;
      m_tile = fmaxf(m_tile, x);
    }
    float factor = 1.0f;
    if (m_tile > m_ref + kRescaleSlack || m_ref == -INFINITY) {
      if (m_tile > -INFINITY) {
        factor = m_ref == -INFINITY ? 1.0f : ex2_approx(m_ref - m_tile);
        m_ref = m_tile;
      }
    }
    // tensor-memory accesses are warp-wide: the warp rescales if any row must
    if (it > 0 && __any_sync(0xffffffffu, factor != 1.0f)) {
#pragma unroll 1
      for (int c = 0; c < kD; c += 32) {
        float o[32];
        tmem_ld32(tmem + lane_base + kTmemO + uint32_t(c), o);
#pragma unroll
        for (int i = 0; i < 32; ++i) o[i] *= factor;
        tmem_st32(tmem + lane_base + kTmemO + uint32_t(c), o);
      }
    }
    l_run *= factor;
    const float m_use = m_ref == -INFINITY ? 0.0f : m_ref;
    float l_tile = 0.0f;
    uint8_t *p_row = p_generic + tid * 128;
#pragma unroll
    for (int c8 = 0; c8 < kBlockN / 8; ++c8) {
      uint32_t packed[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float e0 = ex2_approx(s[8 * c8 + 2 * i] - m_use);
        const float e1 = ex2_approx(s[8 * c8 + 2 * i + 1] - m_use);
        l_tile += e0 + e1;
        const __nv_bfloat162 h = __floats2bfloat162_rn(e0, e1);
        packed[i] = *reinterpret_cast<const uint32_t *>(&h);
      }
      *reinterpret_cast<uint4 *>(p_row + ((c8 ^ (tid & 7)) << 4)) =
          make_uint4(packed[0], packed[1], packed[2], packed[3]);
    }
    l_run += l_tile;
    fence_proxy_async_shared();  // P is read by the tensor core
    tc_fence_before();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after();
      issue_pv(stage, it > 0);
    }
  }

  // ---- the last P V, then O / l as bf16
  if (ok && !mbar_wait_bounded(bar_o, o_phase, kTileWaitClocks)) fault = 3;
  if (fault != 0) atomicCAS(&g_prefill_sm100_fault, 0, fault);
  ok = !__syncthreads_or(!ok || fault != 0);
  tc_fence_after();
  if (ok) {
    // tensor-memory loads are warp-wide: rows past the sequence take part in
    // them and only skip the stores
    const float inv = l_run > 0.0f ? 1.0f / l_run : 0.0f;
    __nv_bfloat16 *dst = p.out + ((seq_row0 + row) * p.q_heads + head) * kD;
#pragma unroll 1
    for (int c = 0; c < kD; c += 32) {
      float o[32];
      tmem_ld32(tmem + lane_base + kTmemO + uint32_t(c), o);
      if (row < S) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          uint32_t w[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const __nv_bfloat162 h = __floats2bfloat162_rn(
                o[8 * i + 2 * j] * inv, o[8 * i + 2 * j + 1] * inv);
            w[j] = *reinterpret_cast<const uint32_t *>(&h);
          }
          reinterpret_cast<uint4 *>(dst + c)[i] = make_uint4(w[0], w[1], w[2], w[3]);
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem),
                 "r"(kTmemColumns)
                 : "memory");
  }
}

}  // namespace

cudaError_t prefill_attention_sm100_bf16(__nv_bfloat16 *out,
                                         const __nv_bfloat16 *q,
                                         const __nv_bfloat16 *k,
                                         const __nv_bfloat16 *v, int batch,
                                         int seq_len, int q_heads, int kv_heads,
                                         int window, float softmax_scale,
                                         cudaStream_t stream) {
  static_assert(kSmemBytes <= 227 * 1024, "tiles must fit one SM");
  Sm100PrefillParams p = {out,     q,        k,      v,
                          seq_len, q_heads,  kv_heads, window,
                          softmax_scale * 1.4426950408889634f};
  cudaError_t st = cudaFuncSetAttribute(
      prefill_attention_sm100_kernel,
      cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
  if (st != cudaSuccess) return st;
  void *fault_word = nullptr;
  st = cudaGetSymbolAddress(&fault_word, g_prefill_sm100_fault);
  if (st != cudaSuccess) return st;
  st = cudaMemsetAsync(fault_word, 0, sizeof(int), stream);
  if (st != cudaSuccess) return st;
  const dim3 grid(unsigned(div_up(seq_len, kBlockM)), unsigned(batch),
                  unsigned(q_heads));
  prefill_attention_sm100_kernel<<<grid, kThreads, kSmemBytes, stream>>>(p);
  return cudaGetLastError();
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

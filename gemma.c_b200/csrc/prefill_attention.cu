// Prompt ("prefill") attention over contiguous prepared rows: the second stage
// of gemma4_flash_attention_{sliding,global}_fwd_bf16_norm_rope
// (src/gemma4_flash_attention.cuh:9-45; kernel src/gemma4_flash_attention_prefill.cu:48-954).
// The first stage, the per-head norm + RoPE prep, is prefill_prep_kernel in
// append_prep.cu.
//
// Layout as the reference: row = batch * seq_len + t; q and out are
// [row, 16, D], k and v [row, kv_heads, D]. Query row r of a sequence sees keys
// c <= r and, for a sliding layer, c >= max(0, r - window + 1)
// (src/gemma4_flash_attention_prefill.cu:502-540).
//
// One CTA = 64 query rows of one query head: four row-warps of 16 rows each,
// times kDSplit warps along the head dimension (1 for D = 256, 2 for D = 512:
// a warp keeps 256 output dims = 128 accumulator registers). Key/value tiles of
// 32 keys are double-buffered in shared memory with cp.async; all tiles are
// stored with the 16-byte chunks of a row XOR-permuted by the row index, which
// makes every ldmatrix conflict-free. Scores and P*V run on the tensor cores
// (bf16 mma.sync m16n8k16, fp32 accumulate), softmax is fp32 online in the exp2
// domain, the score accumulators are reused as the A operand of P*V. With
// D = 512 the two warps of a row group both compute the full score tile (no
// exchange) and split the output dims.
#include <cstdlib>

#include "common.cuh"
#include "kernels.cuh"

namespace b200kv {

namespace {

template <int D_, int kDSplit_>
struct PrefillTraits {
  static constexpr int D = D_;
  static constexpr int kDSplit = kDSplit_;
  static constexpr int kMWarps = 4;
  static constexpr int kBlockM = 16 * kMWarps;
  static constexpr int kBlockN = 32;
  static constexpr int kWarps = kMWarps * kDSplit;
  static constexpr int kThreads = 32 * kWarps;
  static constexpr int kDimsPerWarp = D / kDSplit;
  static constexpr int kRowBytes = D * 2;
  static constexpr int kChunksPerRow = kRowBytes / 16;
  static constexpr int kQBytes = kBlockM * kRowBytes;
  static constexpr int kTileBytes = kBlockN * kRowBytes;  // one K or V tile
  static constexpr int kSmem = kQBytes + 4 * kTileBytes;  // Q, K[2], V[2]
  static_assert(kDimsPerWarp == 256, "128 accumulator registers per lane");
};

struct PrefillParams {
  __nv_bfloat16 *out;
  const __nv_bfloat16 *q;
  const __nv_bfloat16 *k;
  const __nv_bfloat16 *v;
  int32_t seq_len;
  int32_t q_heads;
  int32_t kv_heads;
  int32_t window;  // 0: causal only
  float scale_log2;
};

__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src,
                                           bool valid) {
  const int bytes = valid ? 16 : 0;  // 0: the 16 bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst),
               "l"(src), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() {
  asm volatile("cp.async.commit_group;" ::: "memory");
}
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4],
                                         uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
      "{%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile(
      "ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
      : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile(
      "ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
      : "r"(addr));
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t *>(&h);
}

// Byte offset of 16-byte chunk `chunk` of row `row` inside a tile whose rows
// are kRowBytes long: the chunk index is XORed with the row's low three bits.
template <class T>
__device__ __forceinline__ uint32_t tile_offset(int row, int chunk) {
  return uint32_t(row) * T::kRowBytes + (uint32_t(chunk ^ (row & 7)) << 4);
}

// All threads: copy `rows` rows of D elements (row r from src + r * stride
// elements; rows at or beyond `valid_rows` are zero-filled) into a tile.
template <class T>
__device__ __forceinline__ void load_tile(uint32_t dst, const __nv_bfloat16 *src,
                                          int64_t stride, int rows,
                                          int valid_rows) {
  const int chunks = rows * T::kChunksPerRow;
  for (int i = int(threadIdx.x); i < chunks; i += T::kThreads) {
    const int r = i / T::kChunksPerRow;
    const int c = i - r * T::kChunksPerRow;
    const bool valid = r < valid_rows;
    const __nv_bfloat16 *from = src + (valid ? int64_t(r) * stride : 0) + c * 8;
    cp_async16(dst + tile_offset<T>(r, c), from, valid);
  }
}

template <class T>
__global__ __launch_bounds__(T::kThreads) void prefill_attention_kernel(
    PrefillParams p) {
  constexpr int D = T::D;
  constexpr int BM = T::kBlockM;
  constexpr int BN = T::kBlockN;
  extern __shared__ __align__(128) uint8_t smem[];
  const uint32_t s_q = smem_u32(smem);
  const uint32_t s_k = s_q + T::kQBytes;
  const uint32_t s_v = s_k + 2 * T::kTileBytes;

  const int warp = int(threadIdx.x) >> 5;
  const int lane = int(threadIdx.x) & 31;
  const int mw = warp % T::kMWarps;          // row group of 16
  const int dw = warp / T::kMWarps;          // slice of the output dims
  const int g = lane >> 2;
  const int t = lane & 3;

  // the last (longest) row blocks first
  const int m_block = int(gridDim.x) - 1 - int(blockIdx.x);
  const int batch = int(blockIdx.y);
  const int head = int(blockIdx.z);
  const int kv_head = head / (p.q_heads / p.kv_heads);
  const int S = p.seq_len;
  const int m0 = m_block * BM;
  const int64_t seq_row0 = int64_t(batch) * S;

  const __nv_bfloat16 *q_src = p.q + ((seq_row0 + m0) * p.q_heads + head) * D;
  const int64_t q_stride = int64_t(p.q_heads) * D;
  const int64_t kv_stride = int64_t(p.kv_heads) * D;
  const __nv_bfloat16 *k_base = p.k + (seq_row0 * p.kv_heads + kv_head) * D;
  const __nv_bfloat16 *v_base = p.v + (seq_row0 * p.kv_heads + kv_head) * D;

  // key tiles [tile_lo, tile_hi]: from the left edge of the window of the
  // block's first row to the diagonal of its last row
  const int last_row = min(m0 + BM, S) - 1;
  const int tile_hi = last_row / BN;
  const int tile_lo = p.window > 0 ? max(0, m0 - p.window + 1) / BN : 0;

  load_tile<T>(s_q, q_src, q_stride, BM, S - m0);
  load_tile<T>(s_k, k_base + int64_t(tile_lo) * BN * kv_stride, kv_stride, BN,
               S - tile_lo * BN);
  load_tile<T>(s_v, v_base + int64_t(tile_lo) * BN * kv_stride, kv_stride, BN,
               S - tile_lo * BN);
  cp_async_commit();

  float o[T::kDimsPerWarp / 8][4];
#pragma unroll
  for (int n = 0; n < T::kDimsPerWarp / 8; ++n) {
#pragma unroll
    for (int i = 0; i < 4; ++i) o[n][i] = 0.0f;
  }
  float m_run[2] = {-INFINITY, -INFINITY};
  float l_run[2] = {0.0f, 0.0f};
  const int row0 = m0 + 16 * mw + g;  // this lane's rows: row0, row0 + 8

  // ldmatrix addressing of this lane
  const int a_row = 16 * mw + (lane & 7) + 8 * ((lane >> 3) & 1);
  const int a_chunk = lane >> 4;                         // + 2 * k-step
  const int kb_row = (lane & 7) + 8 * (lane >> 4);       // + 16 * n-tile pair
  const int kb_chunk = (lane >> 3) & 1;                  // + 2 * k-step
  const int vb_row = (lane & 7) + 8 * ((lane >> 3) & 1); // + 16 * key step
  const int vb_chunk = dw * (T::kDimsPerWarp / 8) + (lane >> 4);  // + 2 * dim pair

  for (int tile = tile_lo; tile <= tile_hi; ++tile) {
    const int buf = (tile - tile_lo) & 1;
    if (tile < tile_hi) {  // the next tile goes into the other buffer
      const int nxt = tile + 1;
      load_tile<T>(s_k + (buf ^ 1) * T::kTileBytes,
                   k_base + int64_t(nxt) * BN * kv_stride, kv_stride, BN,
                   S - nxt * BN);
      load_tile<T>(s_v + (buf ^ 1) * T::kTileBytes,
                   v_base + int64_t(nxt) * BN * kv_stride, kv_stride, BN,
                   S - nxt * BN);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const uint32_t k_tile = s_k + buf * T::kTileBytes;
    const uint32_t v_tile = s_v + buf * T::kTileBytes;
    const int k0 = tile * BN;

    // ---- S = Q K^T for 16 rows x 32 keys
    float sc[4][4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
#pragma unroll
      for (int i = 0; i < 4; ++i) sc[j][i] = 0.0f;
    }
#pragma unroll 4
    for (int ks = 0; ks < D / 16; ++ks) {
      uint32_t a[4];
      ldsm_x4(a, s_q + tile_offset<T>(a_row, 2 * ks + a_chunk));
#pragma unroll
      for (int np = 0; np < 2; ++np) {
        uint32_t b[4];
        ldsm_x4(b, k_tile + tile_offset<T>(16 * np + kb_row, 2 * ks + kb_chunk));
        mma_bf16(sc[2 * np], a, b[0], b[1]);
        mma_bf16(sc[2 * np + 1], a, b[2], b[3]);
      }
    }

    // ---- scale, mask at the causal / window edges, online softmax
    const bool edge = k0 + BN - 1 > m0 ||
                      (p.window > 0 && k0 < last_row - p.window + 1);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float s = sc[j][i] * p.scale_log2;
        if (edge) {
          const int row = row0 + 8 * (i >> 1);
          const int col = k0 + 8 * j + 2 * t + (i & 1);
          const bool masked =
              col > row || (p.window > 0 && col < row - p.window + 1);
          if (masked) s = -INFINITY;
        }
        sc[j][i] = s;
      }
    }
    float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      tile_max[0] = fmaxf(tile_max[0], fmaxf(sc[j][0], sc[j][1]));
      tile_max[1] = fmaxf(tile_max[1], fmaxf(sc[j][2], sc[j][3]));
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(0xffffffffu, tile_max[r], 1));
      tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(0xffffffffu, tile_max[r], 2));
    }
    float m_use[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const float m_new = fmaxf(m_run[r], tile_max[r]);
      // a row that has seen no key yet keeps -inf; exponents then use 0
      m_use[r] = m_new == -INFINITY ? 0.0f : m_new;
      const float corr = ex2_approx(m_run[r] - m_use[r]);
      if (m_new > m_run[r]) {
#pragma unroll
        for (int n = 0; n < T::kDimsPerWarp / 8; ++n) {
          o[n][2 * r] *= corr;
          o[n][2 * r + 1] *= corr;
        }
        l_run[r] *= corr;
        m_run[r] = m_new;
      }
    }
    uint32_t pa[2][4];  // P as the A operand, two steps of 16 keys
#pragma unroll
    for (int kk = 0; kk < 2; ++kk) {
      float e[2][4];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          e[h][i] = ex2_approx(sc[2 * kk + h][i] - m_use[i >> 1]);
        }
      }
      l_run[0] += (e[0][0] + e[0][1]) + (e[1][0] + e[1][1]);
      l_run[1] += (e[0][2] + e[0][3]) + (e[1][2] + e[1][3]);
      pa[kk][0] = pack2(e[0][0], e[0][1]);
      pa[kk][1] = pack2(e[0][2], e[0][3]);
      pa[kk][2] = pack2(e[1][0], e[1][1]);
      pa[kk][3] = pack2(e[1][2], e[1][3]);
    }

    // ---- O += P V for this warp's 256 output dims
#pragma unroll
    for (int kk = 0; kk < 2; ++kk) {
#pragma unroll
      for (int np = 0; np < T::kDimsPerWarp / 16; ++np) {
        uint32_t b[4];
        ldsm_x4_trans(b, v_tile + tile_offset<T>(16 * kk + vb_row, 2 * np + vb_chunk));
        mma_bf16(o[2 * np], pa[kk], b[0], b[1]);
        mma_bf16(o[2 * np + 1], pa[kk], b[2], b[3]);
      }
    }
    __syncthreads();  // the buffer is refilled two iterations from now
  }

  // ---- normalise and store
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = row0 + 8 * r;
    if (row < S) {
      const float inv = l_run[r] > 0.0f ? 1.0f / l_run[r] : 0.0f;
      __nv_bfloat16 *dst = p.out + ((seq_row0 + row) * p.q_heads + head) * D +
                           dw * T::kDimsPerWarp + 2 * t;
#pragma unroll
      for (int n = 0; n < T::kDimsPerWarp / 8; ++n) {
        *reinterpret_cast<uint32_t *>(dst + 8 * n) =
            pack2(o[n][2 * r] * inv, o[n][2 * r + 1] * inv);
      }
    }
  }
}

template <class T>
cudaError_t launch_prefill_attention(const PrefillParams &p, int batch,
                                     cudaStream_t stream) {
  static_assert(T::kSmem <= 227 * 1024, "tiles must fit one SM");
  cudaError_t st = cudaFuncSetAttribute(
      prefill_attention_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
      T::kSmem);
  if (st != cudaSuccess) return st;
  const dim3 grid(unsigned(div_up(p.seq_len, T::kBlockM)), unsigned(batch),
                  unsigned(p.q_heads));
  prefill_attention_kernel<T><<<grid, T::kThreads, T::kSmem, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace

cudaError_t prefill_attention_bf16(__nv_bfloat16 *out, const __nv_bfloat16 *q,
                                   const __nv_bfloat16 *k, const __nv_bfloat16 *v,
                                   int batch, int seq_len, int q_heads,
                                   int kv_heads, int head_dim, int window,
                                   float softmax_scale, cudaStream_t stream) {
  if (out == nullptr || q == nullptr || k == nullptr || v == nullptr ||
      batch <= 0 || seq_len <= 0 || window < 0 || q_heads <= 0 || kv_heads <= 0 ||
      q_heads % kv_heads != 0 || batch > 65535 || q_heads > 65535 ||
      !(softmax_scale > 0.0f)) {
    return cudaErrorInvalidValue;
  }
  const uintptr_t align = reinterpret_cast<uintptr_t>(out) |
                          reinterpret_cast<uintptr_t>(q) |
                          reinterpret_cast<uintptr_t>(k) |
                          reinterpret_cast<uintptr_t>(v);
  if ((align & 15u) != 0) return cudaErrorInvalidValue;
  PrefillParams p = {out,      q,        k,      v,
                     seq_len,  q_heads,  kv_heads, window,
                     softmax_scale * 1.4426950408889634f};
  if (head_dim != 256 && head_dim != 512) return cudaErrorInvalidValue;
  // tcgen05 kernel unless B200KV_PREFILL_MMA_SYNC=1 asks for the mma.sync arm
  static const bool legacy = [] {
    const char *e = std::getenv("B200KV_PREFILL_MMA_SYNC");
    return e != nullptr && e[0] == '1';
  }();
  if (!legacy) {
    return prefill_attention_sm100_bf16(out, q, k, v, batch, seq_len, q_heads, kv_heads,
                                        head_dim, window, softmax_scale, stream);
  }
  if (head_dim == 256) {
    return launch_prefill_attention<PrefillTraits<256, 1>>(p, batch, stream);
  }
  if (head_dim == 512) {
    return launch_prefill_attention<PrefillTraits<512, 2>>(p, batch, stream);
  }
  return cudaErrorInvalidValue;
}

}  // namespace b200kv

// Prefill attention in bfloat16: a flash-style kernel over the paged cache for any mix of
// segments (portions of prompts beside single rows).
//
// Reference: ``prefill_attention_kernel<D>`` (src/ops/attention.hip:136-268): tiles of 16
// queries x 32 keys, a software double buffer, causal mask on absolute positions so that a
// later portion sees the keys of earlier ones, online softmax, never a T x T score matrix.
// Same structure here with tensor cores: a tile is up to 64 consecutive rows of one segment
// and one query head, 16 rows per warp; a CTA runs two tiles one after the other, a heavy one
// (late in a long prompt, many keys) and a light one, so that CTAs are about equally long; keys and values come in blocks
// of 64 through ``cp.async`` into a two-stage shared-memory ring (rows padded by 16 bytes so
// that ``ldmatrix`` is free of bank conflicts); S = Q K^T and O += P V are
// ``mma.sync.m16n8k16`` with float32 accumulators; max, exp and sums are float32 (the
// exponential is ``ex2.approx`` on scores pre-multiplied by log2 e: 2^-22 relative, far below
// the bfloat16 rounding of P that follows).
// Key j is visible to a row at position p iff max(0, p - window + 1) <= j <= p.
// Options: `keep_first` keeps a request's first keys visible when the window has passed them (the
// aligned blocks that hold them are walked first, then the window's); `slopes` takes
// slope_h * (p - j) off head h's score of key j; `gate` multiplies head h's output by
// sigmoid(gate[row, h]).
// Steps of single rows (decode) may split a row's key blocks over several CTAs: the blocks of kept
// first keys are one share, and every aligned group of a few window blocks (four: 256 keys, by
// absolute position) another; each CTA leaves its unnormalised sum, maximum and denominator, and a
// merge kernel adds the shares in ascending order.  Which blocks form a share depends on the row's
// own position only, so the sums do not depend on what else the step holds.
// Key blocks are aligned to multiples of 64 keys, so the order of a row's sums depends on
// its own position only, not on how the prompt was cut.
#include "common.cuh"

namespace nf {

constexpr int kBQ = 64, kBKeys = 64;      // rows per tile (4 warps x 16), keys per block
constexpr int kThreads = 128;
int g_split_blocks = 4;                    // key blocks a share of a split row (aligned groups); nf_set_attention_split_blocks()
constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ void pf_cp_async16(void* smem_dst, const void* gmem_src) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gmem_src));
}
__device__ __forceinline__ void pf_commit() { asm volatile("cp.async.commit_group;"); }
template <int N> __device__ __forceinline__ void pf_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N)); }
__device__ __forceinline__ void pf_ldm4(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
  const unsigned a = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void pf_ldm4t(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
  const unsigned a = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void pf_mma(float* c, unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pf_pack(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}

template <int D>
__global__ void __launch_bounds__(kThreads)
prefill_attention_kernel(const __nv_bfloat16* __restrict__ qkv, int q_row_stride,
                         const __nv_bfloat16* __restrict__ pages, const int* __restrict__ block_table,
                         int bt_width, const int* __restrict__ positions, const int* __restrict__ seg_row0,
                         const int* __restrict__ tiles, __nv_bfloat16* __restrict__ out, int Hq, int Hkv,
                         int page_size, int num_pages, int window, float scale,
                         const float* __restrict__ slopes, int keep_first, const float* __restrict__ gate,
                         int gate_ld, int n_shares, float* __restrict__ part_o, float* __restrict__ part_ml,
                         int kSplitBlocks) {
  constexpr int DS = D + 8;             // padded row stride in elements
  constexpr int LPR = D / 8;            // 16-byte pieces per row
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);        // [64][DS]
  __nv_bfloat16* KVs = Qs + kBQ * DS;                                     // [2 stages][K, V][64][DS]
  const int h = blockIdx.y;
  for (int which = 0; which < 2; ++which) {
  const int seg = tiles[4 * blockIdx.x + 2 * which], row0 = tiles[4 * blockIdx.x + 2 * which + 1];
  if (seg < 0) break;
  const int kvh = h / (Hq / Hkv);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, tq = lane & 3;
  const int n_rows = min(kBQ, seg_row0[seg + 1] - row0);
  const int pos_first = positions[row0];
  const int pos_last = pos_first + n_rows - 1;
  const int* bt = block_table + (size_t)seg * bt_width;
  const size_t head_stride = (size_t)page_size * D;
  const size_t page_stride = (size_t)2 * Hkv * head_stride;
  int lo_tile = 0;
  if (window > 0 && pos_first - window + 1 > 0) lo_tile = pos_first - window + 1;
  const int kb_first = (lo_tile / kBKeys) * kBKeys;
  // blocks of kept first keys that lie wholly before the window's first block, then the window's
  const int n_kept = (min(keep_first, kb_first) + kBKeys - 1) / kBKeys;
  const int n_blocks = n_kept + (pos_last - kb_first) / kBKeys + 1;
  const float slope2 = slopes ? slopes[h] * kLog2e : 0.f;
  auto block_start = [&](int blk) { return blk < n_kept ? blk * kBKeys : kb_first + (blk - n_kept) * kBKeys; };
  // this CTA's blocks: all of them, or (split rows) one share
  int b0 = 0, b1 = n_blocks;
  if (n_shares > 0) {
    const int z = blockIdx.z;
    if (z == 0) {
      b1 = n_kept;
    } else {
      const int first_abs = kb_first / kBKeys;
      const int grp = first_abs / kSplitBlocks + z - 1;                 // absolute group of window blocks
      b0 = n_kept + max(0, grp * kSplitBlocks - first_abs);
      b1 = min(n_blocks, n_kept + (grp + 1) * kSplitBlocks - first_abs);
    }
    if (b0 >= b1) break;                                                // an empty share writes nothing
  }

  // ---- Q tile ------------------------------------------------------------------------------
  for (int c = threadIdx.x; c < kBQ * LPR; c += blockDim.x) {
    const int r = c / LPR, piece = c - r * LPR;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < n_rows)
      v = *reinterpret_cast<const uint4*>(qkv + (size_t)(row0 + r) * q_row_stride + (size_t)h * D + piece * 8);
    *reinterpret_cast<uint4*>(Qs + r * DS + piece * 8) = v;
  }

  auto load_block = [&](int blk, int stage) {
    __nv_bfloat16* Ks = KVs + (size_t)stage * 2 * kBKeys * DS;
    __nv_bfloat16* Vs = Ks + kBKeys * DS;
    const int kb = block_start(blk);
    for (int c = threadIdx.x; c < kBKeys * LPR; c += blockDim.x) {
      const int r = c / LPR, piece = c - r * LPR;
      const int j = kb + r;
      const __nv_bfloat16* src = nullptr;
      if (j <= pos_last) {
        const int lp = j / page_size;
        const int page = lp < bt_width ? bt[lp] : -1;
        if (page >= 0 && page < num_pages)
          src = pages + (size_t)page * page_stride + (size_t)kvh * head_stride + (size_t)(j - lp * page_size) * D + piece * 8;
      }
      if (src) {
        pf_cp_async16(Ks + r * DS + piece * 8, src);
        pf_cp_async16(Vs + r * DS + piece * 8, src + (size_t)Hkv * head_stride);
      } else {
        *reinterpret_cast<uint4*>(Ks + r * DS + piece * 8) = make_uint4(0, 0, 0, 0);
        *reinterpret_cast<uint4*>(Vs + r * DS + piece * 8) = make_uint4(0, 0, 0, 0);
      }
    }
  };

  float o[D / 8][4];
#pragma unroll
  for (int n = 0; n < D / 8; ++n)
#pragma unroll
    for (int i = 0; i < 4; ++i) o[n][i] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  // this thread's two query rows and their positions
  const int r_lo = warp * 16 + g, r_hi = r_lo + 8;
  const int p_lo = pos_first + r_lo, p_hi = pos_first + r_hi;
  const int w_lo = window > 0 ? p_lo - window + 1 : 0, w_hi = window > 0 ? p_hi - window + 1 : 0;

  load_block(b0, 0);
  pf_commit();
  for (int blk = b0; blk < b1; ++blk) {
    if (blk + 1 < b1) load_block(blk + 1, (blk + 1 - b0) & 1);
    pf_commit();
    pf_wait<1>();
    __syncthreads();
    const __nv_bfloat16* Ks = KVs + (size_t)((blk - b0) & 1) * 2 * kBKeys * DS;
    const __nv_bfloat16* Vs = Ks + kBKeys * DS;
    const int kb = block_start(blk);

    // a warp whose 16 rows lie beyond the tile's rows, or wholly before this block's keys,
    // only helps with the copies
    const bool warp_active = warp * 16 < n_rows && kb <= pos_first + warp * 16 + 15;
    if (warp_active) {
    // ---- S = Q K^T for this warp's 16 rows x 64 keys -------------------------------------------
    float s[kBKeys / 8][4];
#pragma unroll
    for (int n = 0; n < kBKeys / 8; ++n)
#pragma unroll
      for (int i = 0; i < 4; ++i) s[n][i] = 0.f;
#pragma unroll
    for (int k0 = 0; k0 < D; k0 += 16) {
      unsigned a0, a1, a2, a3;
      pf_ldm4(a0, a1, a2, a3, Qs + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * DS + k0 + (lane >> 4) * 8);
#pragma unroll
      for (int n0 = 0; n0 < kBKeys; n0 += 16) {
        unsigned b0, b1, b2, b3;
        const int mi = lane >> 3;
        pf_ldm4(b0, b1, b2, b3, Ks + (n0 + (lane & 7) + (mi >> 1) * 8) * DS + k0 + (mi & 1) * 8);
        pf_mma(s[n0 / 8], a0, a1, a2, a3, b0, b1);
        pf_mma(s[n0 / 8 + 1], a0, a1, a2, a3, b2, b3);
      }
    }
    // ---- scale (to base-2 exponent units), mask, online softmax ------------------------------------
    float mx[2] = {-INFINITY, -INFINITY};
    const float sc2 = scale * kLog2e;
    // every key of the block visible to every row of the warp: no mask to apply
    const bool all_visible = warp * 16 + 15 < n_rows && kb + kBKeys - 1 <= pos_first + warp * 16 &&
                             (window <= 0 || kb >= pos_first + warp * 16 + 15 - window + 1);
    if (all_visible && slope2 == 0.f) {
#pragma unroll
      for (int n = 0; n < kBKeys / 8; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          s[n][i] *= sc2;
          mx[i >> 1] = fmaxf(mx[i >> 1], s[n][i]);
        }
    } else {
#pragma unroll
      for (int n = 0; n < kBKeys / 8; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int j = kb + n * 8 + 2 * tq + (i & 1);
          const bool hi_row = i >= 2;
          const int p = hi_row ? p_hi : p_lo;
          const int w = hi_row ? w_hi : w_lo;
          const bool row_ok = (hi_row ? r_hi : r_lo) < n_rows;
          const float v = (row_ok && j <= p && (j >= w || j < keep_first))
                              ? fmaf(-slope2, (float)(p - j), s[n][i] * sc2) : -INFINITY;
          s[n][i] = v;
          mx[i >> 1] = fmaxf(mx[i >> 1], v);
        }
    }
    float alpha[2], m_use[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
      const float m_new = fmaxf(m_run[r], mx[r]);
      m_use[r] = m_new == -INFINITY ? 0.f : m_new;       // a row with nothing visible yet
      alpha[r] = exp2f(m_run[r] - m_use[r]);
      m_run[r] = m_new;
    }
    float sum[2] = {0.f, 0.f};
#pragma unroll
    for (int n = 0; n < kBKeys / 8; ++n)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float p = exp2f(s[n][i] - m_use[i >> 1]);
        s[n][i] = p;
        sum[i >> 1] += p;
      }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], 1);
      sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], 2);
      l_run[r] = l_run[r] * alpha[r] + sum[r];
    }
#pragma unroll
    for (int n = 0; n < D / 8; ++n) {
      o[n][0] *= alpha[0]; o[n][1] *= alpha[0];
      o[n][2] *= alpha[1]; o[n][3] *= alpha[1];
    }
    // ---- O += P V ----------------------------------------------------------------------------------
#pragma unroll
    for (int kk = 0; kk < kBKeys / 16; ++kk) {
      const unsigned a0 = pf_pack(s[2 * kk][0], s[2 * kk][1]);
      const unsigned a1 = pf_pack(s[2 * kk][2], s[2 * kk][3]);
      const unsigned a2 = pf_pack(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      const unsigned a3 = pf_pack(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int d0 = 0; d0 < D; d0 += 16) {
        unsigned b0, b1, b2, b3;
        const int mi = lane >> 3;
        pf_ldm4t(b0, b1, b2, b3, Vs + (kk * 16 + (lane & 7) + (mi & 1) * 8) * DS + d0 + (mi >> 1) * 8);
        pf_mma(o[d0 / 8], a0, a1, a2, a3, b0, b1);
        pf_mma(o[d0 / 8 + 1], a0, a1, a2, a3, b2, b3);
      }
    }
    }  // warp_active
    __syncthreads();      // everyone is done with this stage before the next prefetch overwrites it
  }

  // ---- write O / l -----------------------------------------------------------------------------------
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = r ? r_hi : r_lo;
    if (row >= n_rows) continue;
    if (n_shares > 0) {
      // a share of a split row: the unnormalised sum, the maximum (base-2 units) and the denominator
      const size_t slot = ((size_t)(row0 + row) * Hq + h) * n_shares + blockIdx.z;
#pragma unroll
      for (int n = 0; n < D / 8; ++n) {
        part_o[slot * D + n * 8 + 2 * tq] = o[n][2 * r];
        part_o[slot * D + n * 8 + 2 * tq + 1] = o[n][2 * r + 1];
      }
      if (tq == 0) { part_ml[slot * 2] = m_run[r]; part_ml[slot * 2 + 1] = l_run[r]; }
      continue;
    }
    float inv = l_run[r] > 0.f ? 1.f / l_run[r] : 0.f;
    if (gate) inv *= 1.f / (1.f + expf(-gate[(size_t)(row0 + row) * gate_ld + h]));
    __nv_bfloat16* dst = out + (size_t)(row0 + row) * Hq * D + (size_t)h * D;
#pragma unroll
    for (int n = 0; n < D / 8; ++n) {
      const unsigned v = pf_pack(o[n][2 * r] * inv, o[n][2 * r + 1] * inv);
      *reinterpret_cast<unsigned*>(dst + n * 8 + 2 * tq) = v;
    }
  }
  __syncthreads();      // the next tile reuses the shared memory
  }  // which
}

// One CTA per (row, head) of a step of single rows: the row's shares in ascending order.
__global__ void split_rows_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                        const int* __restrict__ positions, const int* __restrict__ tiles,
                                        __nv_bfloat16* __restrict__ out, int Hq, int D,
                                        int window, int keep_first, int n_shares, const float* __restrict__ gate,
                                        int gate_ld, int kSplitBlocks) {
  const int t = tiles[4 * blockIdx.x + 1], h = blockIdx.y;      // a tile is one row: its first row
  chain_release_if_small();
  const int pos = positions[t];
  chain_wait(part_o, part_ml);
  int lo = 0;
  if (window > 0 && pos - window + 1 > 0) lo = pos - window + 1;
  const int kb_first = (lo / kBKeys) * kBKeys;
  const int n_kept = (min(keep_first, kb_first) + kBKeys - 1) / kBKeys;
  const int first_abs = kb_first / kBKeys, last_abs = pos / kBKeys;
  const int z_last = min(n_shares - 1, last_abs / kSplitBlocks - first_abs / kSplitBlocks + 1);
  const int z_first = n_kept > 0 ? 0 : 1;
  const size_t base = ((size_t)t * Hq + h) * n_shares;
  float m = -INFINITY;
  for (int z = z_first; z <= z_last; ++z) m = fmaxf(m, part_ml[(base + z) * 2]);
  float l = 0.f;
  for (int z = z_first; z <= z_last; ++z) {
    const float mz = part_ml[(base + z) * 2];
    if (mz != -INFINITY) l += part_ml[(base + z) * 2 + 1] * exp2f(mz - m);
  }
  float inv = l > 0.f ? 1.f / l : 0.f;
  if (gate) inv *= 1.f / (1.f + expf(-gate[(size_t)t * gate_ld + h]));
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float acc = 0.f;
    for (int z = z_first; z <= z_last; ++z) {
      const float mz = part_ml[(base + z) * 2];
      if (mz != -INFINITY) acc += part_o[(base + z) * D + d] * exp2f(mz - m);
    }
    out[((size_t)t * Hq + h) * D + d] = __float2bfloat16_rn(acc * inv);
  }
}

template <int D>
static int launch_prefill(const void* qkv, int q_row_stride, const void* pages, const int* block_table,
                          int bt_width, const int* positions, const int* seg_row0, const int* tiles,
                          int n_tiles, void* out, int Hq, int Hkv, int page_size, int num_pages, int window,
                          float scale, const float* slopes, int keep_first, const float* gate, int gate_ld,
                          int n_shares, float* part_o, float* part_ml, cudaStream_t stream) {
  const size_t smem = (size_t)(kBQ + 4 * kBKeys) * (D + 8) * sizeof(__nv_bfloat16);
  static bool set = false;
  if (smem > 48 * 1024 && !set) {
    cudaFuncSetAttribute(prefill_attention_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    set = true;
  }
  dim3 grid(n_tiles, Hq, n_shares > 0 ? n_shares : 1);
  prefill_attention_kernel<D><<<grid, kThreads, smem, stream>>>(
      (const __nv_bfloat16*)qkv, q_row_stride, (const __nv_bfloat16*)pages, block_table, bt_width, positions,
      seg_row0, tiles, (__nv_bfloat16*)out, Hq, Hkv, page_size, num_pages, window, scale, slopes, keep_first, gate,
      gate_ld, n_shares, part_o, part_ml, g_split_blocks);
  if (int rc = check_launch("prefill_attention")) return rc;
  if (n_shares > 0) {
    launch_chained(split_rows_merge_kernel, dim3(n_tiles, Hq), dim3(D >= 64 ? 64 : 32), 0, stream, (const float*)part_o,
                   (const float*)part_ml, positions, tiles, (__nv_bfloat16*)out, Hq, D, window, keep_first, n_shares, gate, gate_ld,
                   g_split_blocks);
    return check_launch("split_rows_merge");
  }
  return 0;
}

}  // namespace nf

using namespace nf;

extern "C" int nf_prefill_attention_tile_rows() { return kBQ; }

// Shares a split row can have: the kept keys' blocks, and the aligned groups of window blocks that the keys of a
// row at a position below `max_context` can touch.
extern "C" int nf_prefill_attention_shares(int window, int max_context) {
  const int span = (window > 0 && window < max_context) ? window : max_context;      // keys a row sees at most
  const int blocks = span / kBKeys + 2;                                             // (ragged at both ends)
  return 1 + (blocks + g_split_blocks - 1) / g_split_blocks + 1;
}

// Key blocks (of 64 keys) a share of a split row holds; a power of two from 1 to 16.  For measurement: the
// shares are aligned groups by absolute position, so a row's sums depend on this number and its position alone.
extern "C" int nf_set_attention_split_blocks(int n) {
  if (n == 1 || n == 2 || n == 4 || n == 8 || n == 16) g_split_blocks = n;
  return g_split_blocks;
}

// bfloat16; head_dim a multiple of 16 up to 128.  `tiles` is int32 [n_ctas, 2, 2]: for every CTA two
// tiles as (segment, first row), each at most 64 consecutive rows of one segment; the second may
// be (-1, -1).  slopes float32 [Hq] or null; keep_first >= 0 (it counts only with a window); gate
// float32 [T, gate_ld] (column h: head h's gate logit) or null.  n_shares > 0: every tile is one row, and a row's key blocks are split into shares (see the top of this file); n_shares must be at least
// nf_prefill_attention_shares(window, longest context); part_o float32 [rows, Hq, n_shares, D], part_ml
// [rows, Hq, n_shares, 2].
extern "C" int nf_prefill_attention_biased(const void* qkv, int q_row_stride, const void* pages,
                                           const int* block_table, int bt_width, const int* positions,
                                           const int* seg_row0, const int* tiles, int n_tiles, void* out, int Hq,
                                           int Hkv, int D, int page_size, int num_pages, int window, float scale,
                                           const float* slopes, int keep_first, const float* gate, int gate_ld,
                                           int n_shares, float* part_o, float* part_ml, cudaStream_t stream) {
  if (n_tiles == 0) return 0;
  NF_REQUIRE(n_shares >= 0 && n_shares <= 65535 && (n_shares == 0 || (part_o && part_ml)),
             "prefill attention: split rows need their workspace");
  NF_REQUIRE(n_tiles > 0 && Hq > 0 && Hkv > 0 && Hq % Hkv == 0 && Hq <= 65535, "prefill attention: bad sizes tiles=%d Hq=%d Hkv=%d", n_tiles, Hq, Hkv);
  NF_REQUIRE(q_row_stride % 8 == 0 && (uintptr_t)qkv % 16 == 0, "prefill attention: query rows must be 16-byte aligned");
  NF_REQUIRE(keep_first >= 0 && (!gate || gate_ld >= Hq), "prefill attention: bad options");
  if (window <= 0) keep_first = 0;
#define NF_PF(DD) case DD: return launch_prefill<DD>(qkv, q_row_stride, pages, block_table, bt_width, positions, seg_row0, tiles, n_tiles, out, Hq, Hkv, page_size, num_pages, window, scale, slopes, keep_first, gate, gate_ld, n_shares, part_o, part_ml, stream);
  switch (D) {
    NF_PF(16) NF_PF(32) NF_PF(48) NF_PF(64) NF_PF(80) NF_PF(96) NF_PF(112) NF_PF(128)
    default:
      set_error("prefill attention: head_dim %d is not a multiple of 16 up to 128", D);
      return 1;
  }
#undef NF_PF
}

extern "C" int nf_prefill_attention(const void* qkv, int q_row_stride, const void* pages,
                                    const int* block_table, int bt_width, const int* positions,
                                    const int* seg_row0, const int* tiles, int n_tiles, void* out, int Hq,
                                    int Hkv, int D, int page_size, int num_pages, int window, float scale,
                                    cudaStream_t stream) {
  return nf_prefill_attention_biased(qkv, q_row_stride, pages, block_table, bt_width, positions, seg_row0, tiles,
                                     n_tiles, out, Hq, Hkv, D, page_size, num_pages, window, scale, nullptr, 0, nullptr,
                                     0, 0, nullptr, nullptr, stream);
}

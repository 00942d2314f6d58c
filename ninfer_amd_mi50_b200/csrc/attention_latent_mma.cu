// Attention over cached latent rows [c | k_rot] on tensor cores (bfloat16), for prompt portions
// and decoded tokens alike.  The mathematics is that of attention_latent.cu: every head's score
// against token j is (q_abs[h] . c_j + q_rot[h] . k_rot_j) * scale, its result sum_j p_j c_j, and
// the softmax's denominator also holds exp(sink[h]).
//
// All heads read the same rows, so the heads are stacked into the M dimension: the M rows of a
// tile are 32 consecutive (token, head) pairs of one request's rows in the step, each with its
// own position for the causal mask.  A CTA (8 warps) walks the keys in aligned blocks of 64,
// which arrive in shared memory through a two-deep cp.async ring (rows of W + 8 elements, so
// that ldmatrix meets no bank conflict):
//   S = Q K^T   [32 x 64]: warp w owns the block's keys 8w .. 8w+7 over all W columns;
//   row maxima and sums meet in shared memory; P is written there as two bfloat16 halves (the
//   rounding and its remainder), so that the weights keep 16 bits of mantissa;
//   O += P C    [32 x R]:  warp w owns R / 8 output columns; C is the block's first R columns,
//               read through ldmatrix.trans as the k-major operand.
// Maxima, exponentials, sums and O are float32.  Long contexts are cut into `nsplit` runs of
// blocks, one CTA each; partial (m, l, O) go to a workspace and a second kernel merges them in
// ascending order, adds the sink to the denominator and writes the head-major output.  Block
// boundaries are absolute key indices, so a row's partial sums depend on its own position and
// on nsplit only.
#define NF_CHAIN_CLASS 8
#include "common.cuh"

namespace nf {

constexpr int kLmRows = 32;        // (token, head) pairs a tile
constexpr int kLmKeys = 64;        // keys a block
constexpr int kLmThreads = 256;
constexpr int kLmPad = 8;          // elements of padding a shared-memory row

__device__ __forceinline__ unsigned lm_smem(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void lm_ldm4(unsigned addr, unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void lm_ldm4t(unsigned addr, unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void lm_mma(float* c, unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void lm_cp16(unsigned dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}

// tiles: int32 [n_tiles, 2] of (segment, first pair of the tile within the segment's pairs); null when
// every segment brings one row: tile i is then segment i / tiles_per_row, pairs from 32 * (i % tiles_per_row)
// ws_o float32 [T * heads, nsplit, R], ws_ml float32 [T * heads, nsplit, 2]
template <int NT>      // n-tiles of 8 output columns a warp owns: R = 64 * NT
__global__ void __launch_bounds__(kLmThreads, 1)
latent_attention_mma_kernel(const __nv_bfloat16* __restrict__ q_abs, const __nv_bfloat16* __restrict__ q, int ldq,
                            int head_stride, int rot_off, const __nv_bfloat16* __restrict__ pages,
                            const int* __restrict__ block_table, int bt_width, const int* __restrict__ positions,
                            const int* __restrict__ seg_row0, const int* __restrict__ tiles,
                            float* __restrict__ ws_o, float* __restrict__ ws_ml, int rows, int heads, int Dr,
                            int page_size, int num_pages, float scale, int nsplit, int blocks_per_split) {
  constexpr int R = 64 * NT;
  extern __shared__ __align__(16) unsigned char lm_raw[];
  const int W = R + Dr, WS = W + kLmPad;
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(lm_raw);              // [32][WS]
  __nv_bfloat16* Ks = Qs + kLmRows * WS;                                      // [2][64][WS]
  __nv_bfloat16* Ps = Ks + 2 * kLmKeys * WS;                                  // [2][32][64 + 8]: leading and trailing half of P
  float* smax = reinterpret_cast<float*>(Ps + 2 * kLmRows * (kLmKeys + kLmPad));  // [8][32]
  float* ssum = smax + 8 * kLmRows;                                           // [8][32]
  int* row_pos = reinterpret_cast<int*>(ssum + 8 * kLmRows);                  // [32]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile = blockIdx.x, split = blockIdx.y;
  const int tiles_per_row = (heads + kLmRows - 1) / kLmRows;
  const int seg = tiles ? tiles[2 * tile] : tile / tiles_per_row;
  const int pair0 = tiles ? tiles[2 * tile + 1] : (tile % tiles_per_row) * kLmRows;
  chain_wait(q_abs, q, pages);
  const int r0 = seg_row0[seg], n_pairs = (seg_row0[seg + 1] - r0) * heads;
  if (threadIdx.x < kLmRows) {
    const int pr = pair0 + threadIdx.x;
    row_pos[threadIdx.x] = pr < n_pairs ? positions[r0 + pr / heads] : -1;
  }
  // the tile's queries: [q_abs | rotated slice], 16 bytes a copy
  const int chunks = W / 8;
  for (int i = threadIdx.x; i < kLmRows * chunks; i += kLmThreads) {
    const int r = i / chunks, c = (i - r * chunks) * 8;
    const int pr = pair0 + r;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (pr < n_pairs) {
      const int t = r0 + pr / heads, h = pr % heads;
      const __nv_bfloat16* src = c < R ? q_abs + ((size_t)h * rows + t) * R + c
                                       : q + (size_t)t * ldq + (size_t)h * head_stride + rot_off + (c - R);
      v = *reinterpret_cast<const uint4*>(src);
    }
    *reinterpret_cast<uint4*>(Qs + r * WS + c) = v;
  }
  __syncthreads();
  int last_pos = -1;
  for (int r = 0; r < kLmRows; ++r) last_pos = max(last_pos, row_pos[r]);
  const int b_begin = split * blocks_per_split;
  const int b_end = min(b_begin + blocks_per_split, last_pos / kLmKeys + 1);      // last_pos >= 0 for a real tile
  const int* bt = block_table + (size_t)seg * bt_width;

  // Four threads a key row: the row's page is looked up once, then 16-byte copies at a stride of four.
  auto fetch = [&](int blk, int buf) {
    const int r = threadIdx.x >> 2;                                  // 256 threads, 64 rows
    const int j = blk * kLmKeys + r;
    const int lp = j / page_size;
    const int page = (j <= last_pos && lp < bt_width) ? bt[lp] : -1;
    __nv_bfloat16* d = Ks + ((size_t)buf * kLmKeys + r) * WS;
    if (page >= 0 && page < num_pages) {
      const __nv_bfloat16* src = pages + ((size_t)page * page_size + (j - lp * page_size)) * W;
      for (int c = (threadIdx.x & 3) * 8; c < W; c += 32) lm_cp16(lm_smem(d + c), src + c);
    } else {
      for (int c = (threadIdx.x & 3) * 8; c < W; c += 32)
        *reinterpret_cast<uint4*>(d + c) = make_uint4(0, 0, 0, 0);   // a masked key's row must still be finite
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };

  // this thread's rows: lane / 4 and lane / 4 + 8 of both 16-row halves
  int my_pos[4];
  float m_run[4], l_run[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    my_pos[i] = row_pos[(i >> 1) * 16 + (i & 1) * 8 + (lane >> 2)];
    m_run[i] = -INFINITY;
    l_run[i] = 0.f;
  }
  float o[2][NT][4];
#pragma unroll
  for (int a = 0; a < 2; ++a)
#pragma unroll
    for (int b = 0; b < NT; ++b)
#pragma unroll
      for (int c = 0; c < 4; ++c) o[a][b][c] = 0.f;

  if (b_begin < b_end) fetch(b_begin, 0);
  for (int blk = b_begin; blk < b_end; ++blk) {
    const int buf = (blk - b_begin) & 1;
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();                                   // the block is in, and everyone is done with the block before
    if (blk + 1 < b_end) fetch(blk + 1, buf ^ 1);      // into the buffer that block used; lands during this one's work
    const __nv_bfloat16* Kb = Ks + (size_t)buf * kLmKeys * WS;
    // ---- S = Q K^T for this warp's 8 keys ----
    // (two sums a 16-row half, over the even and the odd steps of 16 columns: a sum's products wait for
    // one another, and with one sum a half the tensor pipe idled between them)
    float s[2][4], s_odd[2][4];
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
      for (int e = 0; e < 4; ++e) s[mt][e] = s_odd[mt][e] = 0.f;
    {
      const unsigned qa = lm_smem(Qs + (lane & 15) * WS + (lane >> 4) * 8);
      const unsigned ka = lm_smem(Kb + (warp * 8 + (lane & 7)) * WS + (lane >> 3) * 8);
      for (int k0 = 0; k0 < W; k0 += 32) {
        unsigned b0, b1, b2, b3;
        const bool both = k0 + 16 < W;                  // W is a multiple of 16, not always of 32
        if (both) lm_ldm4(ka + k0 * 2, b0, b1, b2, b3);
        else {
          asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(b0), "=r"(b1) : "r"(ka + k0 * 2));
          b2 = b3 = 0;
        }
#pragma unroll
        for (int mt = 0; mt < 2; ++mt) {
          unsigned a0, a1, a2, a3;
          lm_ldm4(qa + (mt * 16 * WS + k0) * 2, a0, a1, a2, a3);
          lm_mma(s[mt], a0, a1, a2, a3, b0, b1);
          if (both) {
            lm_ldm4(qa + (mt * 16 * WS + k0 + 16) * 2, a0, a1, a2, a3);
            lm_mma(s_odd[mt], a0, a1, a2, a3, b2, b3);
          }
        }
      }
#pragma unroll
      for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int e = 0; e < 4; ++e) s[mt][e] += s_odd[mt][e];
    }
    // ---- mask, block maxima ----
    const int key0 = blk * kLmKeys + warp * 8 + (lane & 3) * 2;
    float mx[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int mt = i >> 1, hi = i & 1;
      float v0 = s[mt][hi * 2] * scale, v1 = s[mt][hi * 2 + 1] * scale;
      if (key0 > my_pos[i]) v0 = -INFINITY;
      if (key0 + 1 > my_pos[i]) v1 = -INFINITY;
      s[mt][hi * 2] = v0;
      s[mt][hi * 2 + 1] = v1;
      float m = fmaxf(v0, v1);
      m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
      m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
      mx[i] = m;
    }
    if ((lane & 3) == 0) {
#pragma unroll
      for (int i = 0; i < 4; ++i) smax[warp * kLmRows + (i >> 1) * 16 + (i & 1) * 8 + (lane >> 2)] = mx[i];
    }
    __syncthreads();
    float alpha[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int row = (i >> 1) * 16 + (i & 1) * 8 + (lane >> 2);
      float m = smax[row];
#pragma unroll
      for (int w2 = 1; w2 < 8; ++w2) m = fmaxf(m, smax[w2 * kLmRows + row]);
      const float m_new = fmaxf(m_run[i], m);
      alpha[i] = (m_run[i] == -INFINITY) ? 0.f : __expf(m_run[i] - m_new);
      const int mt = i >> 1, hi = i & 1;
      const float p0 = (s[mt][hi * 2] == -INFINITY) ? 0.f : __expf(s[mt][hi * 2] - m_new);
      const float p1 = (s[mt][hi * 2 + 1] == -INFINITY) ? 0.f : __expf(s[mt][hi * 2 + 1] - m_new);
      m_run[i] = m_new;
      // a weight goes to the tensor cores as two bfloat16 numbers, its rounding and what the rounding
      // left (16 bits of mantissa together): with a single one, a row that rests on one far key
      // carried three times the error of the plain kernel
      const __nv_bfloat162 pb = __floats2bfloat162_rn(p0, p1);
      const __nv_bfloat162 pl = __floats2bfloat162_rn(p0 - __bfloat162float(pb.x), p1 - __bfloat162float(pb.y));
      const int pofs = row * (kLmKeys + kLmPad) + warp * 8 + (lane & 3) * 2;
      *reinterpret_cast<__nv_bfloat162*>(Ps + pofs) = pb;
      *reinterpret_cast<__nv_bfloat162*>(Ps + kLmRows * (kLmKeys + kLmPad) + pofs) = pl;
      float sum = p0 + p1;
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);
      if ((lane & 3) == 0) ssum[warp * kLmRows + row] = sum;
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int row = (i >> 1) * 16 + (i & 1) * 8 + (lane >> 2);
      float sum = 0.f;
#pragma unroll
      for (int w2 = 0; w2 < 8; ++w2) sum += ssum[w2 * kLmRows + row];
      l_run[i] = l_run[i] * alpha[i] + sum;
      const int mt = i >> 1, hi = i & 1;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        o[mt][nt][hi * 2] *= alpha[i];
        o[mt][nt][hi * 2 + 1] *= alpha[i];
      }
    }
    // ---- O += P C for this warp's R / 8 columns ----
    {
      const unsigned pa = lm_smem(Ps + (lane & 15) * (kLmKeys + kLmPad) + (lane >> 4) * 8);
      // trans: lanes 0-7 keys k..k+7 at column n, 8-15 keys k+8..k+15 at n, 16-23 / 24-31 the same at n + 8
      const unsigned ca = lm_smem(Kb + ((lane & 7) + ((lane >> 3) & 1) * 8) * WS + warp * (8 * NT) + (lane >> 4) * 8);
#pragma unroll
      for (int ks = 0; ks < kLmKeys / 16; ++ks) {
        unsigned a[2][4], al[2][4];
#pragma unroll
        for (int mt = 0; mt < 2; ++mt) {
          lm_ldm4(pa + (mt * 16 * (kLmKeys + kLmPad) + ks * 16) * 2, a[mt][0], a[mt][1], a[mt][2], a[mt][3]);
          lm_ldm4(pa + ((kLmRows + mt * 16) * (kLmKeys + kLmPad) + ks * 16) * 2, al[mt][0], al[mt][1], al[mt][2], al[mt][3]);
        }
#pragma unroll
        for (int np = 0; np < NT; np += 2) {
          unsigned b0, b1, b2, b3;
          lm_ldm4t(ca + (ks * 16 * WS + np * 8) * 2, b0, b1, b2, b3);
#pragma unroll
          for (int mt = 0; mt < 2; ++mt) {
            lm_mma(o[mt][np], a[mt][0], a[mt][1], a[mt][2], a[mt][3], b0, b1);
            lm_mma(o[mt][np], al[mt][0], al[mt][1], al[mt][2], al[mt][3], b0, b1);
            if (np + 1 < NT) {
              lm_mma(o[mt][np + 1], a[mt][0], a[mt][1], a[mt][2], a[mt][3], b2, b3);
              lm_mma(o[mt][np + 1], al[mt][0], al[mt][1], al[mt][2], al[mt][3], b2, b3);
            }
          }
        }
      }
    }
  }
  // ---- partial results ----
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int row = (i >> 1) * 16 + (i & 1) * 8 + (lane >> 2);
    const int pr = pair0 + row;
    if (pr >= n_pairs) continue;
    const int t = r0 + pr / heads, h = pr % heads;
    const size_t slot = ((size_t)t * heads + h) * nsplit + split;
    if (warp == 0 && (lane & 3) == 0) {
      ws_ml[slot * 2] = m_run[i];
      ws_ml[slot * 2 + 1] = l_run[i];
    }
    const int mt = i >> 1, hi = i & 1;
    float* dst = ws_o + slot * R + warp * (8 * NT) + (lane & 3) * 2;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
      *reinterpret_cast<float2*>(dst + nt * 8) = make_float2(o[mt][nt][hi * 2], o[mt][nt][hi * 2 + 1]);
  }
}

// out[h, t, :] = (sum_s e^{m_s - M} O_s) / (sum_s e^{m_s - M} l_s + e^{sink_h - M}),  M the maximum of
// the m_s and the sink; splits in ascending order.
__global__ void latent_attention_merge_kernel(const float* __restrict__ ws_o, const float* __restrict__ ws_ml,
                                              const float* __restrict__ sink, __nv_bfloat16* __restrict__ out,
                                              int rows, int heads, int R, int nsplit) {
  const int t = blockIdx.x / heads, h = blockIdx.x % heads;
  chain_wait(ws_o, ws_ml);
  const size_t base = ((size_t)t * heads + h) * nsplit;
  float M = sink ? sink[h] : -INFINITY;
  for (int s = 0; s < nsplit; ++s) M = fmaxf(M, ws_ml[(base + s) * 2]);
  float l = sink ? __expf(sink[h] - M) : 0.f;
  for (int s = 0; s < nsplit; ++s) {
    const float m = ws_ml[(base + s) * 2];
    if (m != -INFINITY) l += __expf(m - M) * ws_ml[(base + s) * 2 + 1];
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
  for (int d = threadIdx.x; d < R; d += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < nsplit; ++s) {
      const float m = ws_ml[(base + s) * 2];
      if (m != -INFINITY) acc += __expf(m - M) * ws_o[(base + s) * R + d];
    }
    out[((size_t)h * rows + t) * R + d] = __float2bfloat16_rn(acc * inv);
  }
}

static size_t lm_smem_bytes(int R, int Dr) {
  const int WS = R + Dr + kLmPad;
  return (size_t)(kLmRows + 2 * kLmKeys) * WS * 2 + (size_t)2 * kLmRows * (kLmKeys + kLmPad) * 2 + 2 * 8 * kLmRows * 4 + kLmRows * 4;
}

}  // namespace nf

using namespace nf;

// Whether the tensor-core kernel takes these sizes (else the plain kernel serves them).
extern "C" int nf_latent_attention_mma_fits(int R, int Dr, int head_stride, int rot_off, int ldq) {
  if (R % 64 != 0 || R < 64 || R > 512 || Dr % 16 != 0 || Dr < 0) return 0;
  if (head_stride % 8 != 0 || rot_off % 8 != 0 || ldq % 8 != 0) return 0;
  return lm_smem_bytes(R, Dr) <= 227 * 1024 ? 1 : 0;
}

extern "C" int nf_latent_attention_mma(const void* q_abs, const void* q, int ldq, int head_stride, int rot_off,
                                       const void* pages, const int* block_table, int bt_width, const int* positions,
                                       const int* seg_row0, const int* tiles, int n_tiles, const float* sink,
                                       void* out, float* ws_o, float* ws_ml, int T, int heads, int R, int Dr,
                                       int page_size, int num_pages, float scale, int nsplit, int blocks_per_split,
                                       cudaStream_t stream) {
  if (T == 0 || n_tiles == 0) return 0;
  NF_REQUIRE(nf_latent_attention_mma_fits(R, Dr, head_stride, rot_off, ldq), "latent attention (tensor cores): sizes R=%d Dr=%d do not fit", R, Dr);
  NF_REQUIRE(nsplit >= 1 && blocks_per_split >= 1, "latent attention: bad split");
  const size_t smem = lm_smem_bytes(R, Dr);
  const dim3 grid(n_tiles, nsplit);
  const __nv_bfloat16* qa = (const __nv_bfloat16*)q_abs;
  const __nv_bfloat16* qq = (const __nv_bfloat16*)q;
  const __nv_bfloat16* pg = (const __nv_bfloat16*)pages;
#define NF_LM(NT)                                                                                                     \
  do {                                                                                                                \
    cudaFuncSetAttribute(latent_attention_mma_kernel<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);    \
    launch_chained(latent_attention_mma_kernel<NT>, grid, dim3(kLmThreads), smem, stream, qa, qq, ldq, head_stride,   \
                   rot_off, pg, block_table, bt_width, positions, seg_row0, tiles, ws_o, ws_ml, T, heads, Dr,         \
                   page_size, num_pages, scale, nsplit, blocks_per_split);                                            \
  } while (0)
  switch (R / 64) {
    case 1: NF_LM(1); break;
    case 2: NF_LM(2); break;
    case 3: NF_LM(3); break;
    case 4: NF_LM(4); break;
    case 5: NF_LM(5); break;
    case 6: NF_LM(6); break;
    case 7: NF_LM(7); break;
    default: NF_LM(8); break;
  }
#undef NF_LM
  launch_chained(latent_attention_merge_kernel, dim3(T * heads), dim3(128), 0, stream, (const float*)ws_o,
                 (const float*)ws_ml, sink, (__nv_bfloat16*)out, T, heads, R, nsplit);
  return check_launch("latent_attention_mma");
}

// Attention over a cache of latent rows: per token the cache keeps one row [c | k_rot], c a
// normalised latent of width R from which every head's keys and values would be projected, and
// k_rot one rotated key part of width Dr that all heads share.  With the key projection folded
// into the query (q_abs[h] = W_uk[h]^T q_plain[h], width R) a head's score against token j is
//     s = (q_abs[h] . c_j + q_rot[h] . k_rot_j) * scale,
// and with the value projection applied after the sum the head's result is the latent
//     o[h] = sum_j p_j c_j            (projected by W_uv[h] afterwards),
// so all heads read the same rows and nothing but the cache row is ever needed.
//
// Softmax with a sink: the denominator holds exp(sink_h) once more; the sink has no key and no
// value and is not scaled.  Scores, maxima, exponentials, sums and the accumulator are float32.
// Keys are visited in blocks of 32 in ascending order from `lo` (0, or pos - window + 1 with a
// window), so a row's result depends on its own position only.
//
// Kernels here: the append (RMS norm of the latent, rotation of the shared key part, write of
// the row into its page), the rotation of the queries' rotated slices, and the plain
// one-warp-per-(row, head) attention that serves every type and size.
#define NF_CHAIN_CLASS 8
#include "common.cuh"

namespace nf {

// src[t, col0 : col0 + R + Dr] -> cache row of (segment, position): [norm(c) * w | rot(k)]
template <typename T>
__global__ void latent_append_kernel(const T* __restrict__ src, int lds, int col0, int R, int Dr,
                                     const float* __restrict__ w, float eps, const float* __restrict__ inv_freq,
                                     int rot_dims, const int* __restrict__ positions,
                                     const int* __restrict__ row_seg, T* __restrict__ pages,
                                     const int* __restrict__ block_table, int bt_width, int page_size,
                                     int num_pages) {
  __shared__ float red[33];
  const int t = blockIdx.x;
  chain_wait(src);
  const T* row = src + (size_t)t * lds + col0;
  float ss = 0.f;
  for (int i = threadIdx.x; i < R; i += blockDim.x) {
    const float v = to_float(row[i]);
    ss += v * v;
  }
  const float inv = rsqrtf(block_sum(ss, red) / (float)R + eps);
  const int pos = positions[t];
  const int lp = pos / page_size;
  const int page = lp < bt_width ? block_table[(size_t)row_seg[t] * bt_width + lp] : -1;
  if (page < 0 || page >= num_pages) return;          // a padding row, or no page: nothing is kept
  T* out = pages + ((size_t)page * page_size + pos % page_size) * (R + Dr);
  for (int i = threadIdx.x; i < R; i += blockDim.x) out[i] = from_float<T>(to_float(row[i]) * inv * w[i]);
  const int half = rot_dims / 2;
  for (int i = threadIdx.x; i < Dr; i += blockDim.x) {
    float v = to_float(row[R + i]);
    if (i < rot_dims) {
      const int f = i < half ? i : i - half;
      float sn, cs;
      sincosf((float)pos * inv_freq[f], &sn, &cs);
      const float other = to_float(row[R + (i < half ? i + half : i - half)]);
      v = i < half ? v * cs - other * sn : v * cs + other * sn;
    }
    out[R + i] = from_float<T>(v);
  }
}

// In place: in every head of q [T, heads, head_stride], the slice [off, off + rot_dims) is turned
// (pair (i, i + rot_dims / 2) by pos * inv_freq[i]).
template <typename T>
__global__ void rope_head_slices_kernel(T* __restrict__ q, int ldq, int heads, int head_stride, int off,
                                        int rot_dims, const float* __restrict__ inv_freq,
                                        const int* __restrict__ positions) {
  const int t = blockIdx.x;
  chain_wait(q);
  const float pos = (float)positions[t];
  const int half = rot_dims / 2;
  for (int i = threadIdx.x; i < heads * half; i += blockDim.x) {
    const int hd = i / half, f = i - hd * half;
    T* p = q + (size_t)t * ldq + (size_t)hd * head_stride + off;
    float sn, cs;
    sincosf(pos * inv_freq[f], &sn, &cs);
    const float a = to_float(p[f]), b = to_float(p[f + half]);
    p[f] = from_float<T>(a * cs - b * sn);
    p[f + half] = from_float<T>(b * cs + a * sn);
  }
}

constexpr int kLatentMaxPerLane = 16;      // R <= 512

// q_abs [heads, T, R] (head-major, what the batched product leaves); q_rot read from q [T, ldq] at
// head * head_stride + rot_off; out [heads, T, R].
template <typename T>
__global__ void __launch_bounds__(128)
latent_attention_generic_kernel(const T* __restrict__ q_abs, const T* __restrict__ q, int ldq, int head_stride,
                                int rot_off, const T* __restrict__ pages, const int* __restrict__ block_table,
                                int bt_width, const int* __restrict__ positions, const int* __restrict__ row_seg,
                                const float* __restrict__ sink, T* __restrict__ out, int rows, int heads, int R,
                                int Dr, int page_size, int num_pages, int window, float scale) {
  extern __shared__ float q_smem[];          // [4 warps][R + Dr]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x;
  const int h = blockIdx.y * 4 + warp;
  if (h >= heads) return;
  chain_wait(q_abs, q, pages);
  const int W = R + Dr;
  float* qv = q_smem + warp * W;
  const T* qa = q_abs + ((size_t)h * rows + t) * R;
  const T* qr = q + (size_t)t * ldq + (size_t)h * head_stride + rot_off;
  for (int d = lane; d < R; d += 32) qv[d] = to_float(qa[d]);
  for (int d = lane; d < Dr; d += 32) qv[R + d] = to_float(qr[d]);
  __syncwarp();
  const int pos = positions[t];
  const int* bt = block_table + (size_t)row_seg[t] * bt_width;
  int lo = 0;
  if (window > 0 && pos - window + 1 > 0) lo = pos - window + 1;
  const bool vec = (W % 8 == 0);

  float m = -INFINITY, l = 0.f;
  float acc[kLatentMaxPerLane];
#pragma unroll
  for (int i = 0; i < kLatentMaxPerLane; ++i) acc[i] = 0.f;

  for (int j0 = lo; j0 <= pos; j0 += 32) {
    const int j = j0 + lane;
    float s = -INFINITY;
    const T* crow = nullptr;
    if (j <= pos) {
      const int lp = j / page_size;
      const int page = lp < bt_width ? bt[lp] : -1;
      if (page >= 0 && page < num_pages) {
        crow = pages + ((size_t)page * page_size + (j % page_size)) * W;
        float dot = 0.f;
        if (vec) {
          for (int d = 0; d < W; d += 8) {
            float kk[8];
            load8(crow + d, kk);
#pragma unroll
            for (int e = 0; e < 8; ++e) dot = fmaf(qv[d + e], kk[e], dot);
          }
        } else {
          for (int d = 0; d < W; ++d) dot = fmaf(qv[d], to_float(crow[d]), dot);
        }
        s = dot * scale;
      }
    }
    const float m_new = fmaxf(m, warp_max(s));
    if (m_new == -INFINITY) continue;
    const float p = (s == -INFINITY) ? 0.f : expf(s - m_new);
    const float alpha = (m == -INFINITY) ? 0.f : expf(m - m_new);
    l = l * alpha + warp_sum(p);
    m = m_new;
#pragma unroll
    for (int i = 0; i < kLatentMaxPerLane; ++i) acc[i] *= alpha;
    const int nkeys = min(32, pos - j0 + 1);
    for (int jj = 0; jj < nkeys; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, p, jj);
      const unsigned long long cp = __shfl_sync(0xffffffffu, (unsigned long long)crow, jj);
      if (cp == 0ull) continue;
      const T* cr = reinterpret_cast<const T*>(cp);
#pragma unroll
      for (int i = 0; i < kLatentMaxPerLane; ++i) {
        const int d = lane + 32 * i;
        if (d < R) acc[i] = fmaf(pj, to_float(cr[d]), acc[i]);
      }
    }
  }
  // the sink joins the denominator: exp(sink) beside the exp(s_j), under a common maximum
  if (sink) {
    const float sk = sink[h];
    const float m_new = fmaxf(m, sk);
    const float alpha = (m == -INFINITY) ? 0.f : expf(m - m_new);
    l = l * alpha + expf(sk - m_new);
#pragma unroll
    for (int i = 0; i < kLatentMaxPerLane; ++i) acc[i] *= alpha;
  }
  const float inv_l = l > 0.f ? 1.f / l : 0.f;
  T* o = out + ((size_t)h * rows + t) * R;
#pragma unroll
  for (int i = 0; i < kLatentMaxPerLane; ++i) {
    const int d = lane + 32 * i;
    if (d < R) o[d] = from_float<T>(acc[i] * inv_l);
  }
}

}  // namespace nf

using namespace nf;

extern "C" int nf_latent_append(const void* src, int lds, int col0, int R, int Dr, const float* w, float eps,
                                const float* inv_freq, int rot_dims, const int* positions, const int* row_seg,
                                void* pages, const int* block_table, int bt_width, int page_size, int num_pages,
                                int T, int dtype, cudaStream_t stream) {
  if (T == 0) return 0;
  NF_REQUIRE(R > 0 && Dr >= 0 && col0 >= 0 && col0 + R + Dr <= lds, "latent_append: bad columns");
  NF_REQUIRE(rot_dims % 2 == 0 && rot_dims >= 0 && rot_dims <= Dr, "latent_append: %d rotated dims of %d", rot_dims, Dr);
  if (dtype == kF32)
    launch_chained(latent_append_kernel<float>, dim3(T), dim3(128), 0, stream, (const float*)src, lds, col0, R, Dr, w, eps, inv_freq, rot_dims, positions, row_seg, (float*)pages, block_table, bt_width, page_size, num_pages);
  else
    launch_chained(latent_append_kernel<__nv_bfloat16>, dim3(T), dim3(128), 0, stream, (const __nv_bfloat16*)src, lds, col0, R, Dr, w, eps, inv_freq, rot_dims, positions, row_seg, (__nv_bfloat16*)pages, block_table, bt_width, page_size, num_pages);
  return check_launch("latent_append");
}

extern "C" int nf_rope_head_slices(void* q, int ldq, int heads, int head_stride, int off, int rot_dims,
                                   const float* inv_freq, const int* positions, int T, int dtype,
                                   cudaStream_t stream) {
  if (T == 0 || rot_dims == 0) return 0;
  NF_REQUIRE(rot_dims % 2 == 0 && off >= 0 && off + rot_dims <= head_stride && heads * head_stride <= ldq,
             "rope_head_slices: bad slice");
  if (dtype == kF32)
    launch_chained(rope_head_slices_kernel<float>, dim3(T), dim3(128), 0, stream, (float*)q, ldq, heads, head_stride, off, rot_dims, inv_freq, positions);
  else
    launch_chained(rope_head_slices_kernel<__nv_bfloat16>, dim3(T), dim3(128), 0, stream, (__nv_bfloat16*)q, ldq, heads, head_stride, off, rot_dims, inv_freq, positions);
  return check_launch("rope_head_slices");
}

extern "C" int nf_latent_attention_generic(const void* q_abs, const void* q, int ldq, int head_stride, int rot_off,
                                           const void* pages, const int* block_table, int bt_width,
                                           const int* positions, const int* row_seg, const float* sink, void* out,
                                           int T, int heads, int R, int Dr, int page_size, int num_pages,
                                           int window, float scale, int dtype, cudaStream_t stream) {
  if (T == 0) return 0;
  NF_REQUIRE(heads > 0 && R > 0 && R <= 32 * kLatentMaxPerLane, "latent attention: latent width %d (1..%d)", R, 32 * kLatentMaxPerLane);
  const dim3 grid(T, (heads + 3) / 4);
  const size_t smem = (size_t)4 * (R + Dr) * sizeof(float);
  if (dtype == kF32)
    launch_chained(latent_attention_generic_kernel<float>, grid, dim3(128), smem, stream, (const float*)q_abs, (const float*)q, ldq, head_stride, rot_off, (const float*)pages, block_table, bt_width, positions, row_seg, sink, (float*)out, T, heads, R, Dr, page_size, num_pages, window, scale);
  else
    launch_chained(latent_attention_generic_kernel<__nv_bfloat16>, grid, dim3(128), smem, stream, (const __nv_bfloat16*)q_abs, (const __nv_bfloat16*)q, ldq, head_stride, rot_off, (const __nv_bfloat16*)pages, block_table, bt_width, positions, row_seg, sink, (__nv_bfloat16*)out, T, heads, R, Dr, page_size, num_pages, window, scale);
  return check_launch("latent_attention_generic");
}

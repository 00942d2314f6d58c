// The stage after the projection of an attention whose values are its keys: add the biases, take
// the queries and the keys each over the root mean square of the WHOLE projection (all heads'
// rows at once, before they are split into heads) times a weight, write the normed keys into the
// key half of the request's cache page and the keys as projected (bias added, not normed) into the
// value half.  Nothing is rotated.  The projection arrives as float32 sums, so a key is rounded
// to the cache's type once.
//
// Cache page layout: [2 (k, v)][kv_heads][page_size][head_dim], as rope_append.cu writes it.
#define NF_CHAIN_CLASS 4
#include "common.cuh"

namespace nf {

template <typename T>
__global__ void __launch_bounds__(256)
qk_whole_norm_append_kernel(const float* __restrict__ proj, int ld, int q_col0, int k_col0,
                            const float* __restrict__ bias_q, const float* __restrict__ bias_k,
                            const float* __restrict__ wq, const float* __restrict__ wk, float eps,
                            const int* __restrict__ positions, const int* __restrict__ row_seg,
                            T* __restrict__ q_out, int Hq, int Hkv, int D, T* __restrict__ pages,
                            const int* __restrict__ block_table, int bt_width, int page_size, int num_pages,
                            int append) {
  __shared__ float red[33];
  const int t = blockIdx.x;
  chain_release_if_small();
  chain_wait(proj);
  const float* row = proj + (size_t)t * ld;
  const int QW = Hq * D, KW = Hkv * D;
  float sq = 0.f, sk = 0.f;
  for (int i = threadIdx.x; i < QW; i += blockDim.x) {
    const float v = row[q_col0 + i] + (bias_q ? bias_q[i] : 0.f);
    sq += v * v;
  }
  for (int i = threadIdx.x; i < KW; i += blockDim.x) {
    const float v = row[k_col0 + i] + (bias_k ? bias_k[i] : 0.f);
    sk += v * v;
  }
  const float inv_q = rsqrtf(block_sum(sq, red) / (float)QW + eps);
  const float inv_k = rsqrtf(block_sum(sk, red) / (float)KW + eps);
  T* qo = q_out + (size_t)t * QW;
  for (int i = threadIdx.x; i < QW; i += blockDim.x) {
    const float v = row[q_col0 + i] + (bias_q ? bias_q[i] : 0.f);
    qo[i] = from_float<T>(v * inv_q * wq[i]);
  }
  if (!append) return;
  const int pos = positions[t], seg = row_seg[t];
  const int lp = pos / page_size;
  const int page = (lp >= 0 && lp < bt_width) ? block_table[(size_t)seg * bt_width + lp] : -1;
  if (page < 0 || page >= num_pages) return;               // no page reserved: never write out of bounds
  T* kdst = pages + ((size_t)page * 2 * Hkv * page_size + (size_t)(pos - lp * page_size)) * D;
  const size_t head_stride = (size_t)page_size * D;
  for (int i = threadIdx.x; i < KW; i += blockDim.x) {
    const int head = i / D, d = i - head * D;
    const float v = row[k_col0 + i] + (bias_k ? bias_k[i] : 0.f);
    kdst[(size_t)head * head_stride + d] = from_float<T>(v * inv_k * wk[i]);
    kdst[(size_t)(Hkv + head) * head_stride + d] = from_float<T>(v);
  }
}

}  // namespace nf

using namespace nf;

extern "C" int nf_qk_whole_norm_append(const float* proj, int ld, int q_col0, int k_col0, const float* bias_q,
                                       const float* bias_k, const float* wq, const float* wk, float eps,
                                       const int* positions, const int* row_seg, void* q_out, int T, int Hq, int Hkv,
                                       int D, void* pages, const int* block_table, int bt_width, int page_size,
                                       int num_pages, int append, int dtype, cudaStream_t stream) {
  if (T == 0) return 0;
  NF_REQUIRE(T > 0 && Hq > 0 && Hkv > 0 && D > 0 && wq && wk, "qk_whole_norm_append: bad arguments");
  NF_REQUIRE(q_col0 >= 0 && k_col0 >= 0 && q_col0 + Hq * D <= ld && k_col0 + Hkv * D <= ld,
             "qk_whole_norm_append: the column ranges leave the projection");
  if (dtype == kF32)
    launch_chained(qk_whole_norm_append_kernel<float>, dim3(T), dim3(256), 0, stream, proj, ld, q_col0, k_col0, bias_q, bias_k, wq, wk, eps, positions, row_seg, (float*)q_out, Hq, Hkv, D, (float*)pages, block_table, bt_width, page_size, num_pages, append);
  else
    launch_chained(qk_whole_norm_append_kernel<__nv_bfloat16>, dim3(T), dim3(256), 0, stream, proj, ld, q_col0, k_col0, bias_q, bias_k, wq, wk, eps, positions, row_seg, (__nv_bfloat16*)q_out, Hq, Hkv, D, (__nv_bfloat16*)pages, block_table, bt_width, page_size, num_pages, append);
  return check_launch("qk_whole_norm_append");
}

// Linear attention with a fixed decay per head: a recurrence over each request's rows, from and
// into the request's state slot.
//
//   S_t = g_h S_{t-1} + k_t v_t^T        (S is D x V per head, float32, zero for a new request)
//   o_t = S_t^T q_t
//
// q, k (heads x D) and v (heads x V) are column ranges of one projection.  Before they enter the
// recurrence they may pass SiLU (all three), a rotation of the first `rot` dimensions of every
// q and k head (pair (i, i + rot/2) by the angle pos * f_i), and k a scale.  Everything after
// the projection is float32: angles, the rotated and scaled vectors, the state, the sums.
//
// One CTA serves 16 value columns of one (request, head) and walks the request's rows of the step
// in order.  A column's D state entries lie in the registers of 8 lanes (entry i with lane i % 8);
// the step's q, k, v are staged 16 tokens at a time in shared memory (activation, rotation and
// scale applied while staging), so the token loop itself has no block-wide barrier.  The sum
// over a column is three shuffles.  A token's result depends on earlier tokens only through S,
// which holds the same bits however the request was cut into steps.
//
// The state of a slot is laid out [head][value column][D]: a column's entries are contiguous, so
// the 8 lanes of a column read and write whole 32-byte sectors.
#define NF_CHAIN_CLASS 2
#include "common.cuh"

namespace nf {

constexpr int kLaLanes = 8;       // lanes that share a value column
constexpr int kLaCols = 16;       // value columns a CTA
constexpr int kLaChunk = 16;      // tokens staged at a time

template <typename T, int EPL>    // EPL: state entries a lane, D <= 8 * EPL
__global__ void __launch_bounds__(kLaLanes* kLaCols)
decay_linear_attention_kernel(const T* __restrict__ src, int ld, int q_col0, int k_col0, int v_col0,
                              const float* __restrict__ decay, const float* __restrict__ inv_freq, int rot,
                              float k_scale, int use_silu, float* __restrict__ state, long slot_stride,
                              const int* __restrict__ seg_row0, const int* __restrict__ seg_slot,
                              const int* __restrict__ seg_pos0, float* __restrict__ out, int H, int D, int V) {
  constexpr int DP = kLaLanes * EPL;                       // padded D
  __shared__ float sq[kLaChunk][DP];
  __shared__ float sk[kLaChunk][DP];
  __shared__ float sv[kLaChunk][kLaCols];
  const int seg = blockIdx.x, head = blockIdx.y, col0 = blockIdx.z * kLaCols;
  const int tid = threadIdx.x, lane = tid % kLaLanes, col = col0 + tid / kLaLanes;
  const bool live = col < V;
  chain_release_if_small();
  chain_wait(src, state);
  const int row0 = seg_row0[seg], rows = seg_row0[seg + 1] - row0;
  const int pos0 = seg_pos0[seg];
  const float g = decay[head];
  float* sp = state + (size_t)seg_slot[seg] * slot_stride + ((size_t)head * V + (live ? col : 0)) * D;
  float s[EPL];
#pragma unroll
  for (int e = 0; e < EPL; ++e) {
    const int i = lane + kLaLanes * e;
    s[e] = (live && i < D) ? sp[i] : 0.f;
  }
  const int half = rot / 2;
  for (int c0 = 0; c0 < rows; c0 += kLaChunk) {
    const int n = min(kLaChunk, rows - c0);
    __syncthreads();                                       // the previous chunk has been read
    // stage q and k: thread per (token, dimension); a rotated pair is handled by its lower index
    for (int x = tid; x < n * DP; x += blockDim.x) {
      const int t = x / DP, i = x - t * DP;
      if (i >= D) { sq[t][i] = 0.f; sk[t][i] = 0.f; continue; }
      if (i >= half && i < rot) continue;                  // written with its partner
      const T* r = src + (size_t)(row0 + c0 + t) * ld + (size_t)head * D;
      float q0 = to_float(r[q_col0 + i]), k0 = to_float(r[k_col0 + i]);
      if (use_silu) { q0 = q0 / (1.f + expf(-q0)); k0 = k0 / (1.f + expf(-k0)); }
      if (i < half) {
        float q1 = to_float(r[q_col0 + i + half]), k1 = to_float(r[k_col0 + i + half]);
        if (use_silu) { q1 = q1 / (1.f + expf(-q1)); k1 = k1 / (1.f + expf(-k1)); }
        const float angle = (float)(pos0 + c0 + t) * inv_freq[i];
        const float cs = cosf(angle), sn = sinf(angle);
        sq[t][i] = q0 * cs - q1 * sn;
        sq[t][i + half] = q1 * cs + q0 * sn;
        sk[t][i] = (k0 * cs - k1 * sn) * k_scale;
        sk[t][i + half] = (k1 * cs + k0 * sn) * k_scale;
      } else {
        sq[t][i] = q0;
        sk[t][i] = k0 * k_scale;
      }
    }
    for (int x = tid; x < n * kLaCols; x += blockDim.x) {
      const int t = x / kLaCols, j = x - t * kLaCols;
      float v = 0.f;
      if (col0 + j < V) {
        v = to_float(src[(size_t)(row0 + c0 + t) * ld + v_col0 + (size_t)head * V + col0 + j]);
        if (use_silu) v = v / (1.f + expf(-v));
      }
      sv[t][j] = v;
    }
    __syncthreads();
    for (int t = 0; t < n; ++t) {
      const float v = sv[t][tid / kLaLanes];
      float o = 0.f;
#pragma unroll
      for (int e = 0; e < EPL; ++e) {
        const int i = lane + kLaLanes * e;
        s[e] = fmaf(g, s[e], sk[t][i] * v);
        o = fmaf(s[e], sq[t][i], o);
      }
      o += __shfl_xor_sync(0xffffffffu, o, 4);
      o += __shfl_xor_sync(0xffffffffu, o, 2);
      o += __shfl_xor_sync(0xffffffffu, o, 1);
      if (live && lane == 0) out[(size_t)(row0 + c0 + t) * H * V + (size_t)head * V + col] = o;
    }
  }
  if (live) {
#pragma unroll
    for (int e = 0; e < EPL; ++e) {
      const int i = lane + kLaLanes * e;
      if (i < D) sp[i] = s[e];
    }
  }
}

template <typename T, int EPL>
static void launch_la(const void* src, int ld, int q0, int k0, int v0, const float* decay, const float* inv_freq,
                      int rot, float k_scale, int use_silu, float* state, long long slot_stride, const int* seg_row0,
                      const int* seg_slot, const int* seg_pos0, float* out, int S, int H, int D, int V,
                      cudaStream_t stream) {
  dim3 grid(S, H, (V + kLaCols - 1) / kLaCols);
  launch_chained(decay_linear_attention_kernel<T, EPL>, grid, dim3(kLaLanes * kLaCols), 0, stream, (const T*)src, ld,
                 q0, k0, v0, decay, inv_freq, rot, k_scale, use_silu, state, (long)slot_stride, seg_row0, seg_slot,
                 seg_pos0, out, H, D, V);
}

template <typename T>
static int dispatch_la(const void* src, int ld, int q0, int k0, int v0, const float* decay, const float* inv_freq,
                       int rot, float k_scale, int use_silu, float* state, long long slot_stride, const int* seg_row0,
                       const int* seg_slot, const int* seg_pos0, float* out, int S, int H, int D, int V,
                       cudaStream_t stream) {
#define NF_LA(E)                                                                                                   \
  launch_la<T, E>(src, ld, q0, k0, v0, decay, inv_freq, rot, k_scale, use_silu, state, slot_stride, seg_row0,      \
                  seg_slot, seg_pos0, out, S, H, D, V, stream)
  if (D <= 8) NF_LA(1);
  else if (D <= 16) NF_LA(2);
  else if (D <= 32) NF_LA(4);
  else if (D <= 64) NF_LA(8);
  else if (D <= 128) NF_LA(16);
  else NF_LA(32);
#undef NF_LA
  return check_launch("decay_linear_attention");
}

}  // namespace nf

using namespace nf;

extern "C" int nf_decay_linear_attention_max_dim() { return 256; }

// src [T, ld] holds q at q_col0 (H x D), k at k_col0 (H x D), v at v_col0 (H x V); decay float32 [H];
// inv_freq float32 [rot / 2] (rot 0: nothing is turned); state float32, slot s at state + s * slot_stride,
// [H][V][D]; out float32 [T, H * V].
extern "C" int nf_decay_linear_attention(const void* src, int ld, int q_col0, int k_col0, int v_col0,
                                         const float* decay, const float* inv_freq, int rot, float k_scale,
                                         int use_silu, float* state, long long slot_stride, const int* seg_row0,
                                         const int* seg_slot, const int* seg_pos0, float* out, int S, int H, int D,
                                         int V, int dtype, cudaStream_t stream) {
  if (S == 0) return 0;
  NF_REQUIRE(S > 0 && H > 0 && D > 0 && V > 0 && D <= 256, "linear attention: bad sizes S=%d H=%d D=%d V=%d", S, H, D, V);
  NF_REQUIRE(rot >= 0 && rot % 2 == 0 && rot <= D && (rot == 0 || inv_freq), "linear attention: rot=%d with D=%d", rot, D);
  NF_REQUIRE(H <= 65535 && (V + kLaCols - 1) / kLaCols <= 65535, "linear attention: too many heads or columns");
  if (dtype == kF32)
    return dispatch_la<float>(src, ld, q_col0, k_col0, v_col0, decay, inv_freq, rot, k_scale, use_silu, state,
                              slot_stride, seg_row0, seg_slot, seg_pos0, out, S, H, D, V, stream);
  return dispatch_la<__nv_bfloat16>(src, ld, q_col0, k_col0, v_col0, decay, inv_freq, rot, k_scale, use_silu, state,
                                    slot_stride, seg_row0, seg_slot, seg_pos0, out, S, H, D, V, stream);
}

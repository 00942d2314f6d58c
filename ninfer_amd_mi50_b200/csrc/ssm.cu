// A state-space mixer's two recurrent pieces, both carried across steps in a request's state slot:
//
//  * a short causal convolution per channel with SiLU.  A request's last taps - 1 inputs live in
//    its slot, so a portion of a prompt (or one decoded token) starts from what the portion
//    before it left; before a sequence's start the inputs are zeros (the slot is zeroed when a
//    request is admitted).  Every output is independent of the others, so all rows of a step
//    run in parallel; a second, small kernel then shifts the step's last inputs into the slot.
//
//  * the selective scan  S_t = exp(-exp(A_log) dt_t) S_{t-1} + dt_t B_t x_t^T,
//    y_t = S_t^T C_t + D x_t  with dt_t = softplus(raw_t + dt_bias), per head; S is [N, P]
//    float32 per head and lives in the slot.  One CTA owns a slice of a head's P columns for one
//    request and walks that request's rows of the step in order; a column's N states are spread
//    over 16 lanes (registers), so y's sum over N is a 16-lane shuffle in a fixed order.  The
//    step's B, C, x and dt are staged through shared memory sixteen tokens at a time.  A token's
//    result depends on the tokens before it only through S, which is the same bits however the
//    request was cut into steps.
//
// Decays, step sizes, the state and the sums are float32; x, B, C come as the activations' type.
#define NF_CHAIN_CLASS 2
#include "common.cuh"

namespace nf {

constexpr int kMaxTaps = 8;

// out[t, c] = silu(bias[c] + sum_j taps[c, j] * u(pos_t - (K - 1 - j)))   u from this step's rows
// of `src` (column col0 + c), from the slot for positions before the step, zero before the start.
template <typename T>
__global__ void causal_conv_silu_kernel(const T* __restrict__ src, int lds, int col0, int C,
                                        const float* __restrict__ taps, const float* __restrict__ bias, int K,
                                        const float* __restrict__ state, long slot_stride,
                                        const int* __restrict__ row_seg, const int* __restrict__ seg_row0,
                                        const int* __restrict__ seg_slot, T* __restrict__ out, int T_rows) {
  const int t = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  chain_wait(src);
  if (c >= C) return;
  const int seg = row_seg[t];
  const int r0 = seg_row0[seg];
  const float* st = state + (size_t)seg_slot[seg] * slot_stride;      // [K - 1][C]
  float acc = bias ? bias[c] : 0.f;
  for (int j = 0; j < K; ++j) {
    const int back = K - 1 - j;          // how many tokens before this one
    const int r = t - back;
    float u;
    if (r >= r0) u = to_float(src[(size_t)r * lds + col0 + c]);
    else {
      const int i = (K - 1) - (r0 - r);  // slot row: K - 2 is the token just before the step
      u = i >= 0 ? st[(size_t)i * C + c] : 0.f;
    }
    acc = fmaf(taps[(size_t)c * K + j], u, acc);
  }
  out[(size_t)t * C + c] = from_float<T>(acc / (1.f + expf(-acc)));
}

// The slot's K - 1 rows become the last K - 1 inputs after this step.
template <typename T>
__global__ void conv_state_shift_kernel(const T* __restrict__ src, int lds, int col0, int C, int K,
                                        float* __restrict__ state, long slot_stride,
                                        const int* __restrict__ seg_row0, const int* __restrict__ seg_slot) {
  const int seg = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  chain_wait(src);
  if (c >= C) return;
  const int r0 = seg_row0[seg], n = seg_row0[seg + 1] - r0;
  float* st = state + (size_t)seg_slot[seg] * slot_stride;
  float keep[kMaxTaps];
  for (int i = 0; i < K - 1; ++i) {
    const int r = n - (K - 1) + i;       // row of the step (relative), negative: from the old slot
    if (r >= 0) keep[i] = to_float(src[(size_t)(r0 + r) * lds + col0 + c]);
    else {
      const int o = i + n;               // old slot row (r + K - 1)
      keep[i] = o < K - 1 ? st[(size_t)o * C + c] : 0.f;
    }
  }
  for (int i = 0; i < K - 1; ++i) st[(size_t)i * C + c] = keep[i];
}

constexpr int kScanLanes = 16;     // lanes that share one column's N states
constexpr int kScanCols = 8;       // columns of P a CTA owns
constexpr int kScanChunk = 16;     // tokens staged at a time
constexpr int kScanMaxPer = 16;    // N <= 256
constexpr int kScanStage = 8;      // 16-byte loads a thread keeps in flight for the next chunk
static_assert(kScanLanes * kScanCols == kScanChunk * kScanCols, "one thread stages one x of a chunk");

template <typename T, int NPER>
__global__ void __launch_bounds__(kScanLanes * kScanCols)
ssd_scan_kernel(const T* __restrict__ xbc, int ldx, int x_col0, int b_col0, int c_col0,
                const T* __restrict__ dt_src, int ld_dt, int dt_col0, const float* __restrict__ dt_bias,
                const float* __restrict__ A_log, const float* __restrict__ Dskip, float* __restrict__ state,
                long slot_stride, const int* __restrict__ seg_row0, const int* __restrict__ seg_slot,
                float* __restrict__ y, int heads, int P, int N, int heads_per_group) {
  extern __shared__ float sm[];
  float* Bs = sm;                                  // [chunk][N]
  float* Cs = Bs + kScanChunk * N;                 // [chunk][N]
  float* xs = Cs + kScanChunk * N;                 // [chunk][cols]
  float* ys = xs + kScanChunk * kScanCols;         // [chunk][cols]
  float* dts = ys + kScanChunk * kScanCols;        // [chunk]
  float* dec = dts + kScanChunk;                   // [chunk]
  const int seg = blockIdx.x;
  const int col_tiles = (P + kScanCols - 1) / kScanCols;
  const int h = blockIdx.y / col_tiles, p0 = (blockIdx.y % col_tiles) * kScanCols;
  const int g = h / heads_per_group;
  const int ln = threadIdx.x % kScanLanes, pl = threadIdx.x / kScanLanes;
  const int p = p0 + pl;
  const bool live = p < P;
  const float rate = expf(A_log[h]), bias = dt_bias[h], skip = Dskip[h];
  chain_wait(xbc, dt_src);
  const int r0 = seg_row0[seg], n_rows = seg_row0[seg + 1] - r0;
  float* S = state + (size_t)seg_slot[seg] * slot_stride + ((size_t)h * P + (live ? p : 0)) * N;
  float s[NPER];
#pragma unroll
  for (int i = 0; i < NPER; ++i) {
    const int n = i * kScanLanes + ln;
    s[i] = (live && n < N) ? S[n] : 0.f;
  }
  // Staging.  When the columns are 16-byte aligned, a chunk's B, C, x and dt are asked for (16 bytes a
  // load, into registers) while the chunk before it is being worked on, and stored to shared memory
  // once that is done; otherwise element by element at the chunk's start.
  constexpr int VE = 16 / (int)sizeof(T);
  const int vpr = N / VE;                                         // 16-byte pieces of one token's B (or C)
  const bool vec = (N % VE == 0) && (ldx % VE == 0) && ((b_col0 + g * N) % VE == 0) && ((c_col0 + g * N) % VE == 0) &&
                   (2 * kScanChunk * vpr <= kScanStage * (int)blockDim.x);
  uint4 pre[kScanStage];
  float pre_x = 0.f, pre_dt = 0.f;
  auto issue = [&](int c0) {
    const int nc = min(kScanChunk, n_rows - c0);
#pragma unroll
    for (int k = 0; k < kScanStage; ++k) {
      const int idx = threadIdx.x + k * blockDim.x;
      const int tt = idx / (2 * vpr), rest = idx - tt * 2 * vpr;
      if (tt < nc) {
        const int col = (rest < vpr ? b_col0 : c_col0) + g * N + (rest < vpr ? rest : rest - vpr) * VE;
        pre[k] = *reinterpret_cast<const uint4*>(xbc + (size_t)(r0 + c0 + tt) * ldx + col);
      }
    }
    {
      const int tt = threadIdx.x / kScanCols, pp = threadIdx.x - tt * kScanCols;
      pre_x = (tt < nc && p0 + pp < P) ? to_float(xbc[(size_t)(r0 + c0 + tt) * ldx + x_col0 + h * P + p0 + pp]) : 0.f;
    }
    if (threadIdx.x < nc) pre_dt = to_float(dt_src[(size_t)(r0 + c0 + threadIdx.x) * ld_dt + dt_col0 + h]);
  };
  if (vec && n_rows > 0) issue(0);
  for (int c0 = 0; c0 < n_rows; c0 += kScanChunk) {
    const int nc = min(kScanChunk, n_rows - c0);
    __syncthreads();
    if (vec) {
#pragma unroll
      for (int k = 0; k < kScanStage; ++k) {
        const int idx = threadIdx.x + k * blockDim.x;
        const int tt = idx / (2 * vpr), rest = idx - tt * 2 * vpr;
        if (tt < nc) {
          float* dst = (rest < vpr ? Bs : Cs) + tt * N + (rest < vpr ? rest : rest - vpr) * VE;
          if (sizeof(T) == 2) {
            float f[8];
            unpack8(pre[k], f);
#pragma unroll
            for (int e = 0; e < 8; ++e) dst[e] = f[e];
          } else {
            *reinterpret_cast<uint4*>(dst) = pre[k];
          }
        }
      }
      xs[threadIdx.x] = pre_x;                                   // blockDim == chunk * cols
      if (threadIdx.x < nc) {
        const float v = pre_dt + bias;
        const float dt = v > 20.f ? v : log1pf(expf(v));
        dts[threadIdx.x] = dt;
        dec[threadIdx.x] = expf(-rate * dt);
      }
    } else {
      for (int i = threadIdx.x; i < nc * N; i += blockDim.x) {
        const int tt = i / N, n = i - tt * N;
        const T* row = xbc + (size_t)(r0 + c0 + tt) * ldx;
        Bs[tt * N + n] = to_float(row[b_col0 + g * N + n]);
        Cs[tt * N + n] = to_float(row[c_col0 + g * N + n]);
      }
      for (int i = threadIdx.x; i < nc * kScanCols; i += blockDim.x) {
        const int tt = i / kScanCols, pp = i - tt * kScanCols;
        xs[i] = p0 + pp < P ? to_float(xbc[(size_t)(r0 + c0 + tt) * ldx + x_col0 + h * P + p0 + pp]) : 0.f;
      }
      if (threadIdx.x < nc) {
        const float v = to_float(dt_src[(size_t)(r0 + c0 + threadIdx.x) * ld_dt + dt_col0 + h]) + bias;
        const float dt = v > 20.f ? v : log1pf(expf(v));
        dts[threadIdx.x] = dt;
        dec[threadIdx.x] = expf(-rate * dt);
      }
    }
    __syncthreads();
    if (vec && c0 + kScanChunk < n_rows) issue(c0 + kScanChunk);   // in flight while this chunk is worked on
    // The recurrence over the chunk's tokens touches only registers and shared memory; each
    // token's sum over N stays a per-lane partial until the chunk is done, so that the sixteen
    // shuffle reductions are independent of one another and of the recurrence.
    float acc[kScanChunk];
#pragma unroll
    for (int tt = 0; tt < kScanChunk; ++tt) {
      acc[tt] = 0.f;
      if (tt < nc) {
        const float a = dec[tt];
        const float dx = dts[tt] * xs[tt * kScanCols + pl];
#pragma unroll
        for (int i = 0; i < NPER; ++i) {
          const int n = i * kScanLanes + ln;
          if (n < N) {
            s[i] = fmaf(a, s[i], dx * Bs[tt * N + n]);
            acc[tt] = fmaf(s[i], Cs[tt * N + n], acc[tt]);
          }
        }
      }
    }
#pragma unroll
    for (int tt = 0; tt < kScanChunk; ++tt) {
#pragma unroll
      for (int o = kScanLanes / 2; o > 0; o >>= 1) acc[tt] += __shfl_xor_sync(0xffffffffu, acc[tt], o);
    }
    if (ln == 0) {
#pragma unroll
      for (int tt = 0; tt < kScanChunk; ++tt)
        if (tt < nc) ys[tt * kScanCols + pl] = acc[tt] + skip * xs[tt * kScanCols + pl];
    }
    __syncthreads();
    for (int i = threadIdx.x; i < nc * kScanCols; i += blockDim.x) {
      const int tt = i / kScanCols, pp = i - tt * kScanCols;
      if (p0 + pp < P) y[(size_t)(r0 + c0 + tt) * heads * P + h * P + p0 + pp] = ys[i];
    }
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < NPER; ++i) {
      const int n = i * kScanLanes + ln;
      if (n < N) S[n] = s[i];
    }
  }
}

template <typename T>
static int launch_scan(const void* xbc, int ldx, int x_col0, int b_col0, int c_col0, const void* dt_src, int ld_dt,
                       int dt_col0, const float* dt_bias, const float* A_log, const float* Dskip, float* state,
                       long slot_stride, const int* seg_row0, const int* seg_slot, float* y, int S, int heads, int P,
                       int N, int groups, cudaStream_t stream) {
  const int nper = (N + kScanLanes - 1) / kScanLanes;
  const dim3 grid(S, heads * ((P + kScanCols - 1) / kScanCols)), block(kScanLanes * kScanCols);
  const size_t smem = (size_t)(2 * kScanChunk * N + 2 * kScanChunk * kScanCols + 2 * kScanChunk) * sizeof(float);
#define NF_SCAN(NP)                                                                                                  \
  launch_chained(ssd_scan_kernel<T, NP>, grid, block, smem, stream, (const T*)xbc, ldx, x_col0, b_col0, c_col0,       \
                 (const T*)dt_src, ld_dt, dt_col0, dt_bias, A_log, Dskip, state, slot_stride, seg_row0, seg_slot, y, \
                 heads, P, N, heads / groups)
  if (nper <= 1) NF_SCAN(1);
  else if (nper <= 2) NF_SCAN(2);
  else if (nper <= 4) NF_SCAN(4);
  else if (nper <= 8) NF_SCAN(8);
  else NF_SCAN(16);
#undef NF_SCAN
  return 0;
}

}  // namespace nf

using namespace nf;

extern "C" int nf_causal_conv_silu(const void* src, int lds, int col0, int C, const float* taps, const float* bias,
                                   int K, float* state, long long slot_stride, const int* row_seg,
                                   const int* seg_row0, const int* seg_slot, void* out, int T, int S, int dtype,
                                   cudaStream_t stream) {
  if (T == 0) return 0;
  NF_REQUIRE(K >= 1 && K <= kMaxTaps, "causal_conv: %d taps (1..%d)", K, kMaxTaps);
  NF_REQUIRE(C > 0 && col0 >= 0 && col0 + C <= lds, "causal_conv: bad columns");
  const dim3 grid(T, (C + 255) / 256), sgrid(S, (C + 255) / 256);
  if (dtype == kF32) {
    launch_chained(causal_conv_silu_kernel<float>, grid, dim3(256), 0, stream, (const float*)src, lds, col0, C, taps, bias, K, (const float*)state, (long)slot_stride, row_seg, seg_row0, seg_slot, (float*)out, T);
    if (K > 1) launch_chained(conv_state_shift_kernel<float>, sgrid, dim3(256), 0, stream, (const float*)src, lds, col0, C, K, state, (long)slot_stride, seg_row0, seg_slot);
  } else {
    launch_chained(causal_conv_silu_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, (const __nv_bfloat16*)src, lds, col0, C, taps, bias, K, (const float*)state, (long)slot_stride, row_seg, seg_row0, seg_slot, (__nv_bfloat16*)out, T);
    if (K > 1) launch_chained(conv_state_shift_kernel<__nv_bfloat16>, sgrid, dim3(256), 0, stream, (const __nv_bfloat16*)src, lds, col0, C, K, state, (long)slot_stride, seg_row0, seg_slot);
  }
  return check_launch("causal_conv_silu");
}

extern "C" int nf_ssd_scan(const void* xbc, int ldx, int x_col0, int b_col0, int c_col0, const void* dt_src,
                           int ld_dt, int dt_col0, const float* dt_bias, const float* A_log, const float* Dskip,
                           float* state, long long slot_stride, const int* seg_row0, const int* seg_slot, float* y,
                           int S, int heads, int P, int N, int groups, int dtype, cudaStream_t stream) {
  if (S == 0) return 0;
  NF_REQUIRE(heads > 0 && groups > 0 && heads % groups == 0, "ssd_scan: %d heads do not split into %d groups", heads, groups);
  NF_REQUIRE(N > 0 && N <= kScanLanes * kScanMaxPer, "ssd_scan: state size %d (1..%d)", N, kScanLanes * kScanMaxPer);
  NF_REQUIRE(P > 0, "ssd_scan: bad head width");
  if (dtype == kF32)
    launch_scan<float>(xbc, ldx, x_col0, b_col0, c_col0, dt_src, ld_dt, dt_col0, dt_bias, A_log, Dskip, state, (long)slot_stride, seg_row0, seg_slot, y, S, heads, P, N, groups, stream);
  else
    launch_scan<__nv_bfloat16>(xbc, ldx, x_col0, b_col0, c_col0, dt_src, ld_dt, dt_col0, dt_bias, A_log, Dskip, state, (long)slot_stride, seg_row0, seg_slot, y, S, heads, P, N, groups, stream);
  return check_launch("ssd_scan");
}

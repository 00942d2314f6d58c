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
//    over a warp's lanes (registers), so y's sum over N is a shuffle reduction in a fixed order.  The
//    step's B, C, x and dt are staged through shared memory sixteen tokens at a time.  A token's
//    result depends on the tokens before it only through S, which is the same bits however the
//    request was cut into steps.
//
// Decays, step sizes, the state and the sums are float32; x, B, C come as the activations' type.
#define NF_CHAIN_CLASS 2
#include "common.cuh"

namespace nf {

constexpr int kMaxTaps = 8;

// out[t, c] = silu(bias[c] + sum_j taps[j, c] * u(pos_t - (K - 1 - j)))   (taps tap-major, [K][C], so that
// neighbouring threads read neighbouring numbers)   u from this step's rows
// of `src` (column col0 + c), from the slot for positions before the step, zero before the start.
// A thread owns VE consecutive channels (VE > 1: 16 bytes a load and a store, columns 16-byte aligned).
template <typename T, int VE>
__global__ void causal_conv_silu_kernel(const T* __restrict__ src, int lds, int col0, int C,
                                        const float* __restrict__ taps, const float* __restrict__ bias, int K,
                                        const float* __restrict__ state, long slot_stride,
                                        const int* __restrict__ row_seg, const int* __restrict__ seg_row0,
                                        const int* __restrict__ seg_slot, T* __restrict__ out, int T_rows) {
  const int t = blockIdx.x;
  const int c = (blockIdx.y * blockDim.x + threadIdx.x) * VE;
  chain_wait(src);
  if (c >= C) return;
  const int seg = row_seg[t];
  const int r0 = seg_row0[seg];
  const float* st = state + (size_t)seg_slot[seg] * slot_stride;      // [K - 1][C]
  float acc[VE];
#pragma unroll
  for (int e = 0; e < VE; ++e) acc[e] = bias ? bias[c + e] : 0.f;
  for (int j = 0; j < K; ++j) {
    const int back = K - 1 - j;          // how many tokens before this one
    const int r = t - back;
    float u[VE];
    if (r >= r0) {
      if (VE == 8) load8(reinterpret_cast<const __nv_bfloat16*>(src) + (size_t)r * lds + col0 + c, u);
      else if (VE == 4) load4(reinterpret_cast<const float*>(src) + (size_t)r * lds + col0 + c, u);
      else u[0] = to_float(src[(size_t)r * lds + col0 + c]);
    } else {
      const int i = (K - 1) - (r0 - r);  // slot row: K - 2 is the token just before the step
#pragma unroll
      for (int e = 0; e < VE; ++e) u[e] = i >= 0 ? st[(size_t)i * C + c + e] : 0.f;
    }
#pragma unroll
    for (int e = 0; e < VE; ++e) acc[e] = fmaf(taps[(size_t)j * C + c + e], u[e], acc[e]);     // taps are [K][C] here
  }
#pragma unroll
  for (int e = 0; e < VE; ++e) acc[e] = acc[e] / (1.f + expf(-acc[e]));
  T* o = out + (size_t)t * C + c;
  if (VE == 8) {
    store4(reinterpret_cast<__nv_bfloat16*>(o), acc);
    store4(reinterpret_cast<__nv_bfloat16*>(o) + 4, acc + 4);
  } else if (VE == 4) {
    store4(reinterpret_cast<float*>(o), acc);
  } else {
    o[0] = from_float<T>(acc[0]);
  }
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

constexpr int kScanLanes = 32;     // lanes that share one column's N states: a warp
constexpr int kScanGroups = 8;     // warps a CTA
constexpr int kScanThreads = kScanLanes * kScanGroups;
constexpr int kScanChunk = 16;     // tokens staged at a time
constexpr int kScanMaxPer = 8;     // N <= 256
constexpr int kScanStage = 4;      // 16-byte loads a thread keeps in flight for the next chunk

// CP: columns of P a thread owns (its warp owns CP columns, the CTA 8 * CP): a token's
// B and C are read from shared memory once for all of them.
template <typename T, int NPER, int CP>
__global__ void __launch_bounds__(kScanThreads)
ssd_scan_kernel(const T* __restrict__ xbc, int ldx, int x_col0, int b_col0, int c_col0,
                const T* __restrict__ dt_src, int ld_dt, int dt_col0, const float* __restrict__ dt_bias,
                const float* __restrict__ A_log, const float* __restrict__ Dskip, float* __restrict__ state,
                long slot_stride, const int* __restrict__ seg_row0, const int* __restrict__ seg_slot,
                float* __restrict__ y, int heads, int P, int N, int heads_per_group) {
  constexpr int kCols = kScanGroups * CP;
  extern __shared__ float sm[];
  float* Bs = sm;                                  // [chunk][N]
  float* Cs = Bs + kScanChunk * N;                 // [chunk][N]
  float* xs = Cs + kScanChunk * N;                 // [chunk][cols]
  float* ys = xs + kScanChunk * kCols;             // [chunk][cols]
  float* dts = ys + kScanChunk * kCols;            // [chunk]
  float* dec = dts + kScanChunk;                   // [chunk]
  const int seg = blockIdx.x;
  const int col_tiles = (P + kCols - 1) / kCols;
  const int h = blockIdx.y / col_tiles, p0 = (blockIdx.y % col_tiles) * kCols;
  const int g = h / heads_per_group;
  const int ln = threadIdx.x % kScanLanes, grp = threadIdx.x / kScanLanes;
  const float rate = expf(A_log[h]), bias = dt_bias[h], skip = Dskip[h];
  chain_wait(xbc, dt_src);
  const int r0 = seg_row0[seg], n_rows = seg_row0[seg + 1] - r0;
  float* S = state + (size_t)seg_slot[seg] * slot_stride + (size_t)h * P * N;
  float s[CP][NPER];
#pragma unroll
  for (int c = 0; c < CP; ++c) {
    const int p = p0 + grp * CP + c;
#pragma unroll
    for (int i = 0; i < NPER; ++i) {
      const int n = i * kScanLanes + ln;
      s[c][i] = (p < P && n < N) ? S[(size_t)p * N + n] : 0.f;
    }
  }
  // Staging.  When the columns are 16-byte aligned, a chunk's B, C, x and dt are asked for (16 bytes a
  // load, into registers) while the chunk before it is being worked on, and stored to shared memory
  // once that is done; otherwise element by element at the chunk's start.
  constexpr int VE = 16 / (int)sizeof(T);
  const int vpr = N / VE;                                         // 16-byte pieces of one token's B (or C)
  const bool vec = (N % VE == 0) && (ldx % VE == 0) && ((b_col0 + g * N) % VE == 0) && ((c_col0 + g * N) % VE == 0) &&
                   (2 * kScanChunk * vpr <= kScanStage * kScanThreads);
  constexpr int XI = (kScanChunk * kCols + kScanThreads - 1) / kScanThreads;     // x values a thread stages
  uint4 pre[kScanStage];
  float pre_x[XI], pre_dt = 0.f;
#pragma unroll
  for (int c = 0; c < XI; ++c) pre_x[c] = 0.f;
  auto issue = [&](int c0) {
    const int nc = min(kScanChunk, n_rows - c0);
#pragma unroll
    for (int k = 0; k < kScanStage; ++k) {
      const int idx = threadIdx.x + k * kScanThreads;
      const int tt = idx / (2 * vpr), rest = idx - tt * 2 * vpr;
      if (tt < nc) {
        const int col = (rest < vpr ? b_col0 : c_col0) + g * N + (rest < vpr ? rest : rest - vpr) * VE;
        pre[k] = *reinterpret_cast<const uint4*>(xbc + (size_t)(r0 + c0 + tt) * ldx + col);
      }
    }
#pragma unroll
    for (int c = 0; c < XI; ++c) {
      const int idx = threadIdx.x + c * kScanThreads;
      const int tt = idx / kCols, pp = idx - tt * kCols;
      pre_x[c] = (tt < nc && p0 + pp < P) ? to_float(xbc[(size_t)(r0 + c0 + tt) * ldx + x_col0 + h * P + p0 + pp]) : 0.f;
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
        const int idx = threadIdx.x + k * kScanThreads;
        const int tt = idx / (2 * vpr), rest = idx - tt * 2 * vpr;
        if (tt < nc) {
          float* dst = (rest < vpr ? Bs : Cs) + tt * N + (rest < vpr ? rest : rest - vpr) * VE;
          if (sizeof(T) == 2) {
            float f[8];
            unpack8(pre[k], f);
            store4(dst, f);                      // (16 bytes a store: eight scalar stores met eight-way bank conflicts)
            store4(dst + 4, f + 4);
          } else {
            *reinterpret_cast<uint4*>(dst) = pre[k];
          }
        }
      }
#pragma unroll
      for (int c = 0; c < XI; ++c)
        if (threadIdx.x + c * kScanThreads < kScanChunk * kCols) xs[threadIdx.x + c * kScanThreads] = pre_x[c];
      if (threadIdx.x < nc) {
        const float v = pre_dt + bias;
        const float dt = v > 20.f ? v : log1pf(expf(v));
        dts[threadIdx.x] = dt;
        dec[threadIdx.x] = expf(-rate * dt);
      }
    } else {
      for (int i = threadIdx.x; i < nc * N; i += kScanThreads) {
        const int tt = i / N, n = i - tt * N;
        const T* row = xbc + (size_t)(r0 + c0 + tt) * ldx;
        Bs[tt * N + n] = to_float(row[b_col0 + g * N + n]);
        Cs[tt * N + n] = to_float(row[c_col0 + g * N + n]);
      }
      for (int i = threadIdx.x; i < nc * kCols; i += kScanThreads) {
        const int tt = i / kCols, pp = i - tt * kCols;
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
    // The recurrence over the chunk's tokens touches only registers and shared memory; a token's sum
    // over N stays a per-lane partial until eight tokens are done, so that their shuffle reductions
    // are independent of one another and of the recurrence.
#pragma unroll
    for (int t0 = 0; t0 < kScanChunk; t0 += 8) {
      if (t0 >= nc) break;
      float acc[8][CP];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int tt = t0 + u;
#pragma unroll
        for (int c = 0; c < CP; ++c) acc[u][c] = 0.f;
        if (tt < nc) {
          const float a = dec[tt], dt = dts[tt];
          float dx[CP];
#pragma unroll
          for (int c = 0; c < CP; ++c) dx[c] = dt * xs[tt * kCols + grp * CP + c];
#pragma unroll
          for (int i = 0; i < NPER; ++i) {
            const int n = i * kScanLanes + ln;
            if (n < N) {
              const float b = Bs[tt * N + n], cc = Cs[tt * N + n];
#pragma unroll
              for (int c = 0; c < CP; ++c) {
                s[c][i] = fmaf(a, s[c][i], dx[c] * b);
                acc[u][c] = fmaf(s[c][i], cc, acc[u][c]);
              }
            }
          }
        }
      }
#pragma unroll
      for (int u = 0; u < 8; ++u)
#pragma unroll
        for (int c = 0; c < CP; ++c) {
#pragma unroll
          for (int o = kScanLanes / 2; o > 0; o >>= 1) acc[u][c] += __shfl_xor_sync(0xffffffffu, acc[u][c], o);
        }
      if (ln == 0) {
#pragma unroll
        for (int u = 0; u < 8; ++u)
          if (t0 + u < nc) {
#pragma unroll
            for (int c = 0; c < CP; ++c) {
              const int col = (t0 + u) * kCols + grp * CP + c;
              ys[col] = acc[u][c] + skip * xs[col];
            }
          }
      }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < nc * kCols; i += kScanThreads) {
      const int tt = i / kCols, pp = i - tt * kCols;
      if (p0 + pp < P) y[(size_t)(r0 + c0 + tt) * heads * P + h * P + p0 + pp] = ys[i];
    }
  }
#pragma unroll
  for (int c = 0; c < CP; ++c) {
    const int p = p0 + grp * CP + c;
#pragma unroll
    for (int i = 0; i < NPER; ++i) {
      const int n = i * kScanLanes + ln;
      if (p < P && n < N) S[(size_t)p * N + n] = s[c][i];
    }
  }
}

template <typename T, int CP>
static void launch_scan_cp(const void* xbc, int ldx, int x_col0, int b_col0, int c_col0, const void* dt_src, int ld_dt,
                           int dt_col0, const float* dt_bias, const float* A_log, const float* Dskip, float* state,
                           long slot_stride, const int* seg_row0, const int* seg_slot, float* y, int S, int heads, int P,
                           int N, int groups, cudaStream_t stream) {
  constexpr int kCols = kScanGroups * CP;
  const int nper = (N + kScanLanes - 1) / kScanLanes;
  const dim3 grid(S, heads * ((P + kCols - 1) / kCols)), block(kScanThreads);
  const size_t smem = (size_t)(2 * kScanChunk * N + 2 * kScanChunk * kCols + 2 * kScanChunk) * sizeof(float);
#define NF_SCAN(NP)                                                                                                  \
  launch_chained(ssd_scan_kernel<T, NP, CP>, grid, block, smem, stream, (const T*)xbc, ldx, x_col0, b_col0, c_col0,   \
                 (const T*)dt_src, ld_dt, dt_col0, dt_bias, A_log, Dskip, state, slot_stride, seg_row0, seg_slot, y, \
                 heads, P, N, heads / groups)
  if (nper <= 1) NF_SCAN(1);
  else if (nper <= 2) NF_SCAN(2);
  else if (nper <= 4) NF_SCAN(4);
  else NF_SCAN(8);
#undef NF_SCAN
}

static int g_scan_columns = 0;      // nf_set_scan_columns(): 1, 2 or 4 forces the choice below (measurement)

// Columns a thread: as many as keep at least one CTA a SM busy and the states in registers.
template <typename T>
static int launch_scan(const void* xbc, int ldx, int x_col0, int b_col0, int c_col0, const void* dt_src, int ld_dt,
                       int dt_col0, const float* dt_bias, const float* A_log, const float* Dskip, float* state,
                       long slot_stride, const int* seg_row0, const int* seg_slot, float* y, int S, int heads, int P,
                       int N, int groups, cudaStream_t stream) {
  const long ctas4 = (long)S * heads * ((P + 31) / 32), ctas2 = (long)S * heads * ((P + 15) / 16);
  const int forced = g_scan_columns;
  if (forced == 4 ? P % 32 == 0 : (forced == 0 && P % 32 == 0 && ctas4 >= 148))
    launch_scan_cp<T, 4>(xbc, ldx, x_col0, b_col0, c_col0, dt_src, ld_dt, dt_col0, dt_bias, A_log, Dskip, state, slot_stride, seg_row0, seg_slot, y, S, heads, P, N, groups, stream);
  else if (forced == 2 ? P % 16 == 0 : (forced == 0 && P % 16 == 0 && ctas2 >= 148))
    launch_scan_cp<T, 2>(xbc, ldx, x_col0, b_col0, c_col0, dt_src, ld_dt, dt_col0, dt_bias, A_log, Dskip, state, slot_stride, seg_row0, seg_slot, y, S, heads, P, N, groups, stream);
  else
    launch_scan_cp<T, 1>(xbc, ldx, x_col0, b_col0, c_col0, dt_src, ld_dt, dt_col0, dt_bias, A_log, Dskip, state, slot_stride, seg_row0, seg_slot, y, S, heads, P, N, groups, stream);
  return 0;
}

}  // namespace nf

using namespace nf;

extern "C" void nf_set_scan_columns(int columns) { g_scan_columns = columns; }

extern "C" int nf_causal_conv_silu(const void* src, int lds, int col0, int C, const float* taps, const float* bias,
                                   int K, float* state, long long slot_stride, const int* row_seg,
                                   const int* seg_row0, const int* seg_slot, void* out, int T, int S, int dtype,
                                   cudaStream_t stream) {
  if (T == 0) return 0;
  NF_REQUIRE(K >= 1 && K <= kMaxTaps, "causal_conv: %d taps (1..%d)", K, kMaxTaps);
  NF_REQUIRE(C > 0 && col0 >= 0 && col0 + C <= lds, "causal_conv: bad columns");
  const dim3 sgrid(S, (C + 255) / 256);
  if (dtype == kF32) {
    if (C % 4 == 0 && lds % 4 == 0 && col0 % 4 == 0)
      launch_chained(causal_conv_silu_kernel<float, 4>, dim3(T, (C / 4 + 127) / 128), dim3(128), 0, stream, (const float*)src, lds, col0, C, taps, bias, K, (const float*)state, (long)slot_stride, row_seg, seg_row0, seg_slot, (float*)out, T);
    else
      launch_chained(causal_conv_silu_kernel<float, 1>, dim3(T, (C + 255) / 256), dim3(256), 0, stream, (const float*)src, lds, col0, C, taps, bias, K, (const float*)state, (long)slot_stride, row_seg, seg_row0, seg_slot, (float*)out, T);
    if (K > 1) launch_chained(conv_state_shift_kernel<float>, sgrid, dim3(256), 0, stream, (const float*)src, lds, col0, C, K, state, (long)slot_stride, seg_row0, seg_slot);
  } else {
    if (C % 8 == 0 && lds % 8 == 0 && col0 % 8 == 0)
      launch_chained(causal_conv_silu_kernel<__nv_bfloat16, 8>, dim3(T, (C / 8 + 127) / 128), dim3(128), 0, stream, (const __nv_bfloat16*)src, lds, col0, C, taps, bias, K, (const float*)state, (long)slot_stride, row_seg, seg_row0, seg_slot, (__nv_bfloat16*)out, T);
    else
      launch_chained(causal_conv_silu_kernel<__nv_bfloat16, 1>, dim3(T, (C + 255) / 256), dim3(256), 0, stream, (const __nv_bfloat16*)src, lds, col0, C, taps, bias, K, (const float*)state, (long)slot_stride, row_seg, seg_row0, seg_slot, (__nv_bfloat16*)out, T);
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

// A state-space mixer's recurrences over the rows of a step, segment by segment (a segment is one request's rows,
// a prompt portion or a single decoded token), from and into the per-request state:
//   * causal_conv_act: a short causal convolution per channel with bias and activation; the inputs before a
//     segment's first row come from the request's state (zeros at a sequence's start);
//   * conv_state_update: the state takes the last taps-1 inputs;
//   * ssm_scan: per head, S <- exp(-exp(A_log) dt) S + dt B x^T, y = S^T C + D x, with dt = softplus(raw + bias);
//     S lives in 32-bit floats, and everything but x, B, C (rounded outputs of the convolution) is 32-bit.
// A segment's rows are walked in order from the state the steps before left, so the result at a position does
// not depend on how the sequence was cut into steps: every sum is taken in the same order.
#include "common.cuh"

namespace cbis {

constexpr int kMaxTaps = 8;
constexpr int kConvRows = 32;      // rows of a segment that one block of the convolution walks

// grid (ceil(C / 128), S, ceil(max rows of a segment / kConvRows)), 128 threads: one channel each.
// u = in[r, c0 + c]; out[r, c] = act(bias[c] + sum_j w[c, j] * u[t - (K-1) + j]), j = 0..K-1.
// state[slot][j][c], j = 0..K-2, holds the input K-1-j rows before the segment's first row.
// The taps sit right-aligned in a window of kMaxTaps (absent taps weigh nothing), so no index depends on K.
template <typename TT>
__global__ void __launch_bounds__(128)
causal_conv_act_kernel(const TT* in, int in_ld, int c0, const float* __restrict__ w, const float* __restrict__ bias,
                       const float* state, long long slot_stride, const int* seg_slot, const int* cu_rows, TT* out,
                       int out_ld, int C, int K, int act) {
  pdl_trigger();
  pdl_wait();
  const int c = blockIdx.x * 128 + threadIdx.x;
  const int s = blockIdx.y;
  const int row0 = cu_rows[s], n = cu_rows[s + 1] - row0;
  const int first = blockIdx.z * kConvRows;
  if (c >= C || first >= n) return;
  const int last = min(n, first + kConvRows);
  const float* st = state + (long long)seg_slot[s] * slot_stride;
  constexpr int M = kMaxTaps;
  float wk[M], hist[M - 1];
#pragma unroll
  for (int j = 0; j < M; ++j) {
    const int tap = j - (M - K);                 // window place j holds tap j - (M - K)
    wk[j] = tap >= 0 ? w[(size_t)c * K + tap] : 0.f;
  }
  const float b = bias ? bias[c] : 0.f;
  // hist[j]: the input (M-1-j) rows before row `first`; only the last K-1 of them are ever weighed
#pragma unroll
  for (int j = 0; j < M - 1; ++j) {
    hist[j] = 0.f;
    const int back = M - 1 - j;                  // rows before `first`
    if (back <= K - 1) {
      const int i = first - back;                // index inside the segment; negative: before this step
      hist[j] = i >= 0 ? to_f32(in[(size_t)(row0 + i) * in_ld + c0 + c]) : st[(size_t)(K - 1 + i) * C + c];
    }
  }
  for (int i0 = first; i0 < last; i0 += 8) {
    float cur[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) cur[u] = i0 + u < last ? to_f32(in[(size_t)(row0 + i0 + u) * in_ld + c0 + c]) : 0.f;
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      if (i0 + u < last) {
        float acc = b;
#pragma unroll
        for (int j = 0; j < M - 1; ++j) acc = fmaf(wk[j], hist[j], acc);
        acc = fmaf(wk[M - 1], cur[u], acc);
        from_f32(out[(size_t)(row0 + i0 + u) * out_ld + c], activate(acc, act));
#pragma unroll
        for (int j = 0; j < M - 2; ++j) hist[j] = hist[j + 1];
        hist[M - 2] = cur[u];
      }
    }
  }
}

// grid (ceil(C / 128), S): state[slot][j][c] <- the input K-1-j rows before the row after the segment's last.
template <typename TT>
__global__ void __launch_bounds__(128)
conv_state_update_kernel(const TT* in, int in_ld, int c0, float* state, long long slot_stride, const int* seg_slot,
                         const int* cu_rows, int C, int K) {
  pdl_trigger();
  pdl_wait();
  const int c = blockIdx.x * 128 + threadIdx.x;
  const int s = blockIdx.y;
  const int row0 = cu_rows[s], n = cu_rows[s + 1] - row0;
  if (c >= C || n <= 0) return;
  float* st = state + (long long)seg_slot[s] * slot_stride;
  float next[kMaxTaps];
#pragma unroll
  for (int j = 0; j < kMaxTaps - 1; ++j) {
    next[j] = 0.f;
    if (j < K - 1) {
      const int i = n - (K - 1) + j;
      next[j] = i >= 0 ? to_f32(in[(size_t)(row0 + i) * in_ld + c0 + c]) : st[(size_t)(K - 1 + i) * C + c];
    }
  }
#pragma unroll
  for (int j = 0; j < kMaxTaps - 1; ++j)
    if (j < K - 1) st[(size_t)j * C + c] = next[j];
}

__device__ __forceinline__ float softplus_f32(float z) { return z > 20.f ? z : log1pf(expf(z)); }

constexpr int kScanTokens = 16;     // rows of a segment staged in shared memory at a time

// grid (ceil(P / 32), H, S), 256 threads: thread t owns column p = 32 * blockIdx.x + t / 8 of the head's state and
// the states n = t % 8 + 8 i, i < NPL, of that column; the eight lanes of a column add their shares of y by shuffles.
// State of a slot: S[h][p][n].  xbc row: x (H*P) | B (G*N) | C (G*N); the raw step sizes are H columns of `proj`.
// The rows are walked 16 at a time: B, C and x of 16 rows wait in shared memory, with the step size dt and
// expm1(-exp(A_log) dt) of each row computed once for the block; the next 16 rows' loads are in flight meanwhile.
template <typename TT, int NPL>
__global__ void __launch_bounds__(256)
ssm_scan_kernel(const TT* xbc, int xbc_ld, const TT* proj, int proj_ld, int dt_off, const float* __restrict__ dt_bias,
                const float* __restrict__ A_log, const float* __restrict__ Dskip, float* state, long long slot_stride,
                const int* seg_slot, const int* cu_rows, float* y, int y_ld, int H, int P, int N, int G) {
  constexpr int NP = 8 * NPL;                       // the state size rounded up
  constexpr int TC = kScanTokens;
  constexpr int BC_PER_THREAD = TC * 2 * NP / 256;  // = NPL
  __shared__ float bc[TC * 2 * NP];                 // [row][B | C][n]
  __shared__ float xs[TC * 32];                     // [row][column of this block]
  __shared__ float dts[TC], dm1s[TC];
  pdl_trigger();
  pdl_wait();
  const int h = blockIdx.y, s = blockIdx.z;
  const int row0 = cu_rows[s], n_rows = cu_rows[s + 1] - row0;
  if (n_rows <= 0) return;
  const int nl = threadIdx.x & 7, pl = threadIdx.x >> 3;
  const int p = blockIdx.x * 32 + pl;
  const bool live = p < P;
  const int g = h / (H / G);
  const int x_col0 = h * P + blockIdx.x * 32;
  const int b_col = H * P + g * N, c_col = H * P + G * N + g * N;
  float* sp = state + (long long)seg_slot[s] * slot_stride + ((size_t)h * P + (live ? p : 0)) * N;
  float S[NPL];
#pragma unroll
  for (int i = 0; i < NPL; ++i) {
    const int n = nl + 8 * i;
    S[i] = (live && n < N) ? sp[n] : 0.f;
  }
  const float neg_a = -expf(A_log[h]), bias = dt_bias[h], dskip = Dskip[h];

  // what this thread fetches of a chunk of rows: NPL values of B | C, two of x, and (the first TC threads) a step size
  float r_bc[BC_PER_THREAD], r_x[2], r_dt = 0.f;
  auto fetch = [&](int first) {
    const int tc = min(TC, n_rows - first);
#pragma unroll
    for (int j = 0; j < BC_PER_THREAD; ++j) {
      const int idx = threadIdx.x + 256 * j, t = idx / (2 * NP), rem = idx % (2 * NP), n = rem % NP;
      r_bc[j] = (t < tc && n < N) ? to_f32(xbc[(size_t)(row0 + first + t) * xbc_ld + (rem < NP ? b_col : c_col) + n]) : 0.f;
    }
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int idx = threadIdx.x + 256 * j, t = idx >> 5, c = idx & 31;
      r_x[j] = (t < tc && blockIdx.x * 32 + c < P) ? to_f32(xbc[(size_t)(row0 + first + t) * xbc_ld + x_col0 + c]) : 0.f;
    }
    if (threadIdx.x < TC)
      r_dt = threadIdx.x < tc ? to_f32(proj[(size_t)(row0 + first + threadIdx.x) * proj_ld + dt_off + h]) : 0.f;
  };
  auto stage = [&]() {
#pragma unroll
    for (int j = 0; j < BC_PER_THREAD; ++j) bc[threadIdx.x + 256 * j] = r_bc[j];
#pragma unroll
    for (int j = 0; j < 2; ++j) xs[threadIdx.x + 256 * j] = r_x[j];
    if (threadIdx.x < TC) {
      const float dt = softplus_f32(r_dt + bias);
      dts[threadIdx.x] = dt;
      // The decay is applied as S += (decay - 1) S with decay - 1 = expm1(-exp(A_log) dt): a decay close to 1 rounded
      // to a float just below 1 loses most of the digits of 1 - decay, the same way at every step when the step size
      // barely changes, and a state that is read a thousand tokens later would carry a thousand times that error.
      dm1s[threadIdx.x] = expm1f(neg_a * dt);
    }
  };
  fetch(0);
  for (int first = 0; first < n_rows; first += TC) {
    __syncthreads();                 // the rows staged before have been used
    stage();
    __syncthreads();
    if (first + TC < n_rows) fetch(first + TC);
    const int tc = min(TC, n_rows - first);
#pragma unroll 4
    for (int t = 0; t < tc; ++t) {
      const float xv = xs[t * 32 + pl];
      const float dx = dts[t] * xv, decay_m1 = dm1s[t];
      const float* Bt = bc + t * 2 * NP + nl;
      float acc = 0.f;
#pragma unroll
      for (int i = 0; i < NPL; ++i) {
        S[i] = fmaf(decay_m1, S[i], fmaf(Bt[8 * i], dx, S[i]));
        acc = fmaf(S[i], Bt[NP + 8 * i], acc);
      }
      acc += __shfl_xor_sync(0xffffffffu, acc, 1);
      acc += __shfl_xor_sync(0xffffffffu, acc, 2);
      acc += __shfl_xor_sync(0xffffffffu, acc, 4);
      if (live && nl == 0) y[(size_t)(row0 + first + t) * y_ld + h * P + p] = fmaf(dskip, xv, acc);
    }
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < NPL; ++i) {
      const int n = nl + 8 * i;
      if (n < N) sp[n] = S[i];
    }
  }
}

template <typename TT>
static int launch_scan(const void* xbc, int xbc_ld, const void* proj, int proj_ld, int dt_off, const float* dt_bias,
                       const float* A_log, const float* D, float* state, long long slot_stride, const int* seg_slot,
                       const int* cu_rows, float* y, int y_ld, int S, int H, int P, int N, int G, cudaStream_t st) {
  const dim3 grid((P + 31) / 32, H, S), block(256);
#define CBIS_SCAN(NPL)                                                                                             \
  return (int)launch_pdl(ssm_scan_kernel<TT, NPL>, grid, block, 0, st, (const TT*)xbc, xbc_ld, (const TT*)proj, proj_ld, \
                         dt_off, dt_bias, A_log, D, state, slot_stride, seg_slot, cu_rows, y, y_ld, H, P, N, G)
  if (N <= 8) CBIS_SCAN(1);
  if (N <= 16) CBIS_SCAN(2);
  if (N <= 32) CBIS_SCAN(4);
  if (N <= 64) CBIS_SCAN(8);
  if (N <= 128) CBIS_SCAN(16);
  if (N <= 256) CBIS_SCAN(32);
#undef CBIS_SCAN
  return CBIS_ERR_TOO_LARGE;
}

}  // namespace cbis

using namespace cbis;

CBIS_EXPORT int cbis_conv_max_taps() { return kMaxTaps; }
CBIS_EXPORT int cbis_scan_max_state() { return 256; }

// in: [T, in_ld] of the compute type, the convolution's channels at columns c0 .. c0 + C - 1; out: [T, out_ld].
// w [C, K] and bias [C] 32-bit; state: 32-bit, (K-1) * C floats at `state + slot * slot_stride`.
CBIS_EXPORT int cbis_causal_conv_act(const void* in, int in_ld, int c0, const float* w, const float* bias,
                                     const float* state, long long slot_stride, const int* seg_slot, const int* cu_rows,
                                     void* out, int out_ld, int C, int K, int act, int n_segments, int max_seg_rows,
                                     int dtype, void* stream) {
  if (n_segments <= 0 || max_seg_rows <= 0) return CBIS_OK;
  if (C <= 0 || K < 1 || K > kMaxTaps) return CBIS_ERR_BAD_SIZE;
  if (n_segments > 65535) return CBIS_ERR_TOO_LARGE;
  const dim3 grid((C + 127) / 128, n_segments, (max_seg_rows + kConvRows - 1) / kConvRows);
  if (grid.z > 65535) return CBIS_ERR_TOO_LARGE;
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == CBIS_F32)
    return (int)launch_pdl(causal_conv_act_kernel<float>, grid, dim3(128), 0, st, (const float*)in, in_ld, c0, w, bias,
                           state, slot_stride, seg_slot, cu_rows, (float*)out, out_ld, C, K, act);
  if (dtype == CBIS_BF16)
    return (int)launch_pdl(causal_conv_act_kernel<__nv_bfloat16>, grid, dim3(128), 0, st, (const __nv_bfloat16*)in, in_ld,
                           c0, w, bias, state, slot_stride, seg_slot, cu_rows, (__nv_bfloat16*)out, out_ld, C, K, act);
  return CBIS_ERR_BAD_DTYPE;
}

CBIS_EXPORT int cbis_conv_state_update(const void* in, int in_ld, int c0, float* state, long long slot_stride,
                                       const int* seg_slot, const int* cu_rows, int C, int K, int n_segments, int dtype,
                                       void* stream) {
  if (n_segments <= 0 || K <= 1) return CBIS_OK;
  if (C <= 0 || K > kMaxTaps) return CBIS_ERR_BAD_SIZE;
  if (n_segments > 65535) return CBIS_ERR_TOO_LARGE;
  const dim3 grid((C + 127) / 128, n_segments);
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == CBIS_F32)
    return (int)launch_pdl(conv_state_update_kernel<float>, grid, dim3(128), 0, st, (const float*)in, in_ld, c0, state,
                           slot_stride, seg_slot, cu_rows, C, K);
  if (dtype == CBIS_BF16)
    return (int)launch_pdl(conv_state_update_kernel<__nv_bfloat16>, grid, dim3(128), 0, st, (const __nv_bfloat16*)in,
                           in_ld, c0, state, slot_stride, seg_slot, cu_rows, C, K);
  return CBIS_ERR_BAD_DTYPE;
}

// xbc [T, xbc_ld]: x | B | C after the convolution (compute type); proj [T, proj_ld] holds the raw step sizes at
// columns dt_off .. dt_off + H - 1; y [T, y_ld] 32-bit; state: H * P * N floats at `state + slot * slot_stride`.
CBIS_EXPORT int cbis_ssm_scan(const void* xbc, int xbc_ld, const void* proj, int proj_ld, int dt_off,
                              const float* dt_bias, const float* A_log, const float* D, float* state,
                              long long slot_stride, const int* seg_slot, const int* cu_rows, float* y, int y_ld,
                              int n_segments, int H, int P, int N, int G, int dtype, void* stream) {
  if (n_segments <= 0) return CBIS_OK;
  if (H <= 0 || P <= 0 || N <= 0 || G <= 0 || H % G) return CBIS_ERR_BAD_SIZE;
  if (n_segments > 65535 || H > 65535) return CBIS_ERR_TOO_LARGE;
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == CBIS_F32)
    return launch_scan<float>(xbc, xbc_ld, proj, proj_ld, dt_off, dt_bias, A_log, D, state, slot_stride, seg_slot,
                              cu_rows, y, y_ld, n_segments, H, P, N, G, st);
  if (dtype == CBIS_BF16)
    return launch_scan<__nv_bfloat16>(xbc, xbc_ld, proj, proj_ld, dt_off, dt_bias, A_log, D, state, slot_stride,
                                      seg_slot, cu_rows, y, y_ld, n_segments, H, P, N, G, st);
  return CBIS_ERR_BAD_DTYPE;
}

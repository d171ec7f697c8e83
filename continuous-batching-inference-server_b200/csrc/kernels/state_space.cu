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
                       float* state, long long slot_stride, const int* seg_slot, const int* cu_rows, TT* out,
                       int out_ld, int C, int K, int act, int update_state) {
  pdl_trigger();
  pdl_wait();
  const int c = blockIdx.x * 128 + threadIdx.x;
  const int s = blockIdx.y;
  const int row0 = cu_rows[s], n = cu_rows[s + 1] - row0;
  const int first = blockIdx.z * kConvRows;
  if (c >= C || first >= n) return;
  const int last = min(n, first + kConvRows);
  float* st = state + (long long)seg_slot[s] * slot_stride;
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
  // `update_state` (only where no segment is longer than one block's rows, so this block has seen all of them and
  // nobody else reads this channel's state): the window now ends with the segment's last row
  if (update_state) {
#pragma unroll
    for (int j = 0; j < M - 1; ++j) {
      const int place = j - (M - K);             // state place of window place j
      if (place >= 0) st[(size_t)place * C + c] = hist[j];
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

__device__ __forceinline__ void cp_async_16(void* smem, const void* gmem) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"((unsigned)__cvta_generic_to_shared(smem)), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

__device__ __forceinline__ float softplus_f32(float z) { return z > 20.f ? z : log1pf(expf(z)); }

constexpr int kScanTokens = 16;     // rows of a segment staged in shared memory at a time

// grid (ceil(P / CB), H, S), 256 threads, CB = 256 / L columns of one head's state a block: thread t owns column
// p = CB * blockIdx.x + t / L and the states n = (t % L) * NPL + i, i < NPL, of that column; the L lanes of a column add
// their shares of y by shuffles.  L is 8 where the step has blocks enough, 16 where few segments (one long prompt)
// would leave most of the machine idle: the state's values do not depend on L, y's last bit may.
// State of a slot: S[h][p][n].  xbc row: x (H*P) | B (G*N) | C (G*N); the raw step sizes are H columns of `proj`.
// The rows are walked 16 at a time: B, C and x of 16 rows wait in shared memory, with the step size dt and
// expm1(-exp(A_log) dt) of each row computed once for the block; the next 16 rows' loads are in flight meanwhile.
// In shared memory a lane's NPL values of B (and of C) are followed by four unused floats, so the lanes' 16-byte
// loads fall into different banks.
template <typename TT, int NPL, int L>
__global__ void __launch_bounds__(256)
ssm_scan_kernel(const TT* xbc, int xbc_ld, const TT* proj, int proj_ld, int dt_off, const float* __restrict__ dt_bias,
                const float* __restrict__ A_log, const float* __restrict__ Dskip, float* state, long long slot_stride,
                const int* seg_slot, const int* cu_rows, float* y, int y_ld, int H, int P, int N, int G, int use_async,
                int mode, int n_chunks, int chunk_rows, float* chunk_state, float* chunk_logdecay) {
  constexpr int NP = L * NPL;                       // the state size rounded up
  constexpr int TC = kScanTokens;
  constexpr int CB = 256 / L;                       // columns a block
  constexpr int BC_PER_THREAD = TC * 2 * NP / 256;
  constexpr int X_PER_THREAD = (TC * CB + 255) / 256;
  constexpr int LS = NPL + (NPL >= 4 ? 4 : 0);      // a lane's stretch of a row of B or C, padded
  __shared__ __align__(16) float bc[TC * 2 * L * LS];   // [row][B | C][lane][LS]
  __shared__ float xs[TC * CB];                     // [row][column of this block]
  __shared__ float dts[TC], dm1s[TC];
  // with `use_async` (every run of B, C and x starts on 16 bytes): the next rows arrive here by cp.async while this
  // block works, as they are stored; they are converted and spread into `bc` and `xs` when their turn comes
  constexpr bool kAsyncFits = NP <= 128;            // beyond that the static 48 KB of shared memory do not hold both
  __shared__ __align__(16) TT raw_bc[kAsyncFits ? TC * 2 * NP : 8];  // [row][B | C][n]
  __shared__ __align__(16) TT raw_x[TC * CB];
  if (!kAsyncFits) use_async = 0;
  pdl_trigger();
  pdl_wait();
  // mode 0: a segment's rows from and into the request's state.  A long segment may instead be cut into n_chunks
  // pieces of chunk_rows rows that run side by side: mode 1 walks every piece but the last from a zero state and
  // leaves its end state and the sum of its log-decays; scan_chain_kernel turns these into every piece's start state;
  // mode 2 walks every piece from its start state, writes y, and the last piece leaves the request's state.
  const int h = blockIdx.y, s = blockIdx.z / n_chunks, chunk = blockIdx.z % n_chunks;
  const int seg_row0 = cu_rows[s], seg_rows = cu_rows[s + 1] - seg_row0;
  const int first_row = mode == 0 ? 0 : chunk * chunk_rows;
  if (first_row >= seg_rows) return;
  const int n_rows = mode == 0 ? seg_rows : min(chunk_rows, seg_rows - first_row);
  const bool last_piece = first_row + n_rows == seg_rows;
  if (mode == 1 && last_piece) return;          // nobody comes after it
  const int row0 = seg_row0 + first_row;
  const int nl = threadIdx.x % L, pl = threadIdx.x / L;
  const int p = blockIdx.x * CB + pl;
  const bool live = p < P;
  const int g = h / (H / G);
  const int x_col0 = h * P + blockIdx.x * CB;
  const int b_col = H * P + g * N, c_col = H * P + G * N + g * N;
  float* request_state = state + (long long)seg_slot[s] * slot_stride + ((size_t)h * P + (live ? p : 0)) * N;
  float* piece_state = mode == 0 ? nullptr
                                 : chunk_state + ((size_t)(s * n_chunks + chunk) * H * P + (size_t)h * P + (live ? p : 0)) * N;
  float* sp = mode == 2 ? piece_state : request_state;      // where the walk starts from (mode 1: from zero)
  float S[NPL];
  // a lane's states lie side by side: 16-byte loads and stores where the row of states allows them
  const bool vec = NPL >= 4 && N == NP && !(((uintptr_t)request_state | (uintptr_t)piece_state) & 15);
  if (mode == 1) {
#pragma unroll
    for (int i = 0; i < NPL; ++i) S[i] = 0.f;
  } else if (vec) {
#pragma unroll
    for (int i = 0; i < NPL; i += 4) {
      const float4 v = live ? *reinterpret_cast<const float4*>(sp + nl * NPL + i) : make_float4(0.f, 0.f, 0.f, 0.f);
      S[i] = v.x;
      if (i + 1 < NPL) S[i + 1] = v.y;
      if (i + 2 < NPL) S[i + 2] = v.z;
      if (i + 3 < NPL) S[i + 3] = v.w;
    }
  } else {
#pragma unroll
    for (int i = 0; i < NPL; ++i) {
      const int n = nl * NPL + i;
      S[i] = (live && n < N) ? sp[n] : 0.f;
    }
  }
  const float neg_a = -expf(A_log[h]), bias = dt_bias[h], dskip = Dskip[h];

  // what this thread fetches of a chunk of rows: values of B | C, of x, and (the first TC threads) a step size
  constexpr int E16 = 16 / (int)sizeof(TT);         // elements of a 16-byte piece
  float r_bc[BC_PER_THREAD], r_x[X_PER_THREAD], r_dt = 0.f;
  float log_decay = 0.f;      // the first TC threads: the sum of -exp(A_log) dt over their rows of this walk
  auto fetch = [&](int first) {
    const int tc = min(TC, n_rows - first);
    if (threadIdx.x < TC)
      r_dt = threadIdx.x < tc ? to_f32(proj[(size_t)(row0 + first + threadIdx.x) * proj_ld + dt_off + h]) : 0.f;
    if (use_async) {
      for (int piece = threadIdx.x; piece < TC * 2 * NP / E16; piece += 256) {
        const int idx = piece * E16, t = idx / (2 * NP), rem = idx % (2 * NP), n = rem % NP;
        if (t < tc && n < N)
          cp_async_16(raw_bc + idx, xbc + (size_t)(row0 + first + t) * xbc_ld + (rem < NP ? b_col : c_col) + n);
      }
      for (int piece = threadIdx.x; piece < TC * CB / E16; piece += 256) {
        const int idx = piece * E16, t = idx / CB, c = idx % CB;
        if (t < tc && blockIdx.x * CB + c < P)
          cp_async_16(raw_x + idx, xbc + (size_t)(row0 + first + t) * xbc_ld + x_col0 + c);
      }
      cp_async_commit();
      return;
    }
#pragma unroll
    for (int j = 0; j < BC_PER_THREAD; ++j) {
      const int idx = threadIdx.x + 256 * j, t = idx / (2 * NP), rem = idx % (2 * NP), n = rem % NP;
      r_bc[j] = (t < tc && n < N) ? to_f32(xbc[(size_t)(row0 + first + t) * xbc_ld + (rem < NP ? b_col : c_col) + n]) : 0.f;
    }
#pragma unroll
    for (int j = 0; j < X_PER_THREAD; ++j) {
      const int idx = threadIdx.x + 256 * j, t = idx / CB, c = idx % CB;
      r_x[j] = (t < tc && blockIdx.x * CB + c < P) ? to_f32(xbc[(size_t)(row0 + first + t) * xbc_ld + x_col0 + c]) : 0.f;
    }
  };
  auto stage = [&](int first) {
    if (use_async) {
      const int tc = min(TC, n_rows - first);
      cp_async_wait_all();
      __syncthreads();               // every thread's pieces have arrived
#pragma unroll
      for (int j = 0; j < BC_PER_THREAD; ++j) {
        const int idx = threadIdx.x + 256 * j, n = idx % NP;
        r_bc[j] = (idx / (2 * NP) < tc && n < N) ? to_f32(raw_bc[idx]) : 0.f;
      }
#pragma unroll
      for (int j = 0; j < X_PER_THREAD; ++j) {
        const int idx = threadIdx.x + 256 * j;
        r_x[j] = (idx < TC * CB && idx / CB < tc && blockIdx.x * CB + idx % CB < P) ? to_f32(raw_x[idx]) : 0.f;
      }
    }
#pragma unroll
    for (int j = 0; j < BC_PER_THREAD; ++j) {
      const int idx = threadIdx.x + 256 * j, n = idx % NP;      // idx = (row * 2 + B|C) * NP + n
      bc[(idx / NP * L + n / NPL) * LS + n % NPL] = r_bc[j];
    }
#pragma unroll
    for (int j = 0; j < X_PER_THREAD; ++j)
      if (threadIdx.x + 256 * j < TC * CB) xs[threadIdx.x + 256 * j] = r_x[j];
    if (threadIdx.x < TC) {
      const float dt = softplus_f32(r_dt + bias);
      dts[threadIdx.x] = dt;
      if (first + (int)threadIdx.x < n_rows) log_decay += neg_a * dt;
      // The decay is applied as S += (decay - 1) S with decay - 1 = expm1(-exp(A_log) dt): a decay close to 1 rounded
      // to a float just below 1 loses most of the digits of 1 - decay, the same way at every step when the step size
      // barely changes, and a state that is read a thousand tokens later would carry a thousand times that error.
      dm1s[threadIdx.x] = expm1f(neg_a * dt);
    }
  };
  fetch(0);
  for (int first = 0; first < n_rows; first += TC) {
    __syncthreads();                 // the rows staged before have been used
    stage(first);
    __syncthreads();                 // (and the raw rows have been read: the next ones may overwrite them)
    if (first + TC < n_rows) fetch(first + TC);
    const int tc = min(TC, n_rows - first);
#pragma unroll 4
    for (int t = 0; t < tc; ++t) {
      const float xv = xs[t * CB + pl];
      const float dx = dts[t] * xv, decay_m1 = dm1s[t];
      const float* Bt = bc + (t * 2 * L + nl) * LS;
      const float* Ct = Bt + L * LS;
      float acc = 0.f;
      if constexpr (NPL >= 4) {
        float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;       // four short chains of sums instead of one long one
#pragma unroll
        for (int i = 0; i < NPL; i += 4) {
          const float4 b4 = *reinterpret_cast<const float4*>(Bt + i), c4 = *reinterpret_cast<const float4*>(Ct + i);
          S[i] = fmaf(decay_m1, S[i], fmaf(b4.x, dx, S[i]));
          S[i + 1] = fmaf(decay_m1, S[i + 1], fmaf(b4.y, dx, S[i + 1]));
          S[i + 2] = fmaf(decay_m1, S[i + 2], fmaf(b4.z, dx, S[i + 2]));
          S[i + 3] = fmaf(decay_m1, S[i + 3], fmaf(b4.w, dx, S[i + 3]));
          a0 = fmaf(S[i], c4.x, a0);
          a1 = fmaf(S[i + 1], c4.y, a1);
          a2 = fmaf(S[i + 2], c4.z, a2);
          a3 = fmaf(S[i + 3], c4.w, a3);
        }
        acc = (a0 + a1) + (a2 + a3);
      } else {
#pragma unroll
        for (int i = 0; i < NPL; ++i) {
          S[i] = fmaf(decay_m1, S[i], fmaf(Bt[i], dx, S[i]));
          acc = fmaf(S[i], Ct[i], acc);
        }
      }
#pragma unroll
      for (int o = 1; o < L; o <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if (live && nl == 0 && mode != 1) y[(size_t)(row0 + first + t) * y_ld + h * P + p] = fmaf(dskip, xv, acc);
    }
  }
  if (mode == 1 && blockIdx.x == 0 && threadIdx.x < 32) {      // the piece's whole decay, as its logarithm
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) log_decay += __shfl_xor_sync(0xffffffffu, log_decay, o);   // threads >= TC hold 0
    if (threadIdx.x == 0) chunk_logdecay[(size_t)(s * n_chunks + chunk) * H + h] = log_decay;
  }
  if (mode == 2 && !last_piece) return;         // only the last piece's end is the request's state
  sp = mode == 1 ? piece_state : request_state;
  if (live && vec) {
#pragma unroll
    for (int i = 0; i < NPL; i += 4)
      *reinterpret_cast<float4*>(sp + nl * NPL + i) =
          make_float4(S[i], S[i + 1 < NPL ? i + 1 : i], S[i + 2 < NPL ? i + 2 : i], S[i + 3 < NPL ? i + 3 : i]);
  } else if (live) {
#pragma unroll
    for (int i = 0; i < NPL; ++i) {
      const int n = nl * NPL + i;
      if (n < N) sp[n] = S[i];
    }
  }
}

// grid (ceil(H * P * N / 256), S): element e of segment s's state.  buf[s][c][e] holds piece c's end state from zero
// (pieces before the last) and takes piece c's START state: S_0 = the request's state, S_(c+1) = S_c + expm1(l_c) S_c + E_c
// with l_c the piece's summed log-decay of the element's head.
__global__ void scan_chain_kernel(float* buf, const float* logdecay, const float* state, long long slot_stride,
                                  const int* seg_slot, const int* cu_rows, int n_chunks, int chunk_rows, int H, int PN) {
  pdl_trigger();
  pdl_wait();
  const int s = blockIdx.y;
  const long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= (long long)H * PN) return;
  const int rows = cu_rows[s + 1] - cu_rows[s];
  const int pieces = (rows + chunk_rows - 1) / chunk_rows;
  if (pieces <= 0) return;
  const int h = (int)(e / PN);
  float S = state[(long long)seg_slot[s] * slot_stride + e];
  for (int c = 0; c < pieces; ++c) {
    float* at = buf + ((size_t)(s * n_chunks + c) * H) * PN + e;
    const float end = c + 1 < pieces ? *at : 0.f;
    *at = S;
    if (c + 1 < pieces) S = fmaf(expm1f(logdecay[(size_t)(s * n_chunks + c) * H + h]), S, S + end);
  }
}

template <typename TT>
static int launch_scan(const void* xbc, int xbc_ld, const void* proj, int proj_ld, int dt_off, const float* dt_bias,
                       const float* A_log, const float* D, float* state, long long slot_stride, const int* seg_slot,
                       const int* cu_rows, float* y, int y_ld, int S, int H, int P, int N, int G, int mode, int n_chunks,
                       int chunk_rows, float* chunk_state, float* chunk_logdecay, cudaStream_t st) {
  // lanes a column: 8, or 16 while the warps (segments x heads x columns x lanes / 32) would not give every SM its
  // sixteen.  Not 32: the blocks of one long prompt (every one walks the whole prompt) must all run at once, and 512
  // blocks of 33 KB of shared memory do not (measured: 32 lanes took twice as long as 8).
  int L = 8;
  if ((long long)S * n_chunks * H * P * L / 32 < 148 * 16 && N >= 64) L = 16;
  // rows may come by cp.async where every run of B, C and x of a row starts on 16 bytes
  const int e16 = 16 / (int)sizeof(TT);
  const int use_async = (N % e16 == 0 && P % e16 == 0 && (H * P) % e16 == 0 && xbc_ld % e16 == 0 &&
                         !((uintptr_t)xbc & 15)) ? 1 : 0;
#define CBIS_SCAN(NPL, LL)                                                                                          \
  return (int)launch_pdl(ssm_scan_kernel<TT, NPL, LL>, dim3((P + 256 / LL - 1) / (256 / LL), H, S * n_chunks), dim3(256), 0, st, \
                         (const TT*)xbc, xbc_ld, (const TT*)proj, proj_ld, dt_off, dt_bias, A_log, D, state, slot_stride, \
                         seg_slot, cu_rows, y, y_ld, H, P, N, G, use_async, mode, n_chunks, chunk_rows, chunk_state, \
                         chunk_logdecay)
  if (L == 16) {
    if (N <= 64) CBIS_SCAN(4, 16);
    if (N <= 128) CBIS_SCAN(8, 16);
    if (N <= 256) CBIS_SCAN(16, 16);
  }
  if (N <= 8) CBIS_SCAN(1, 8);
  if (N <= 16) CBIS_SCAN(2, 8);
  if (N <= 32) CBIS_SCAN(4, 8);
  if (N <= 64) CBIS_SCAN(8, 8);
  if (N <= 128) CBIS_SCAN(16, 8);
  if (N <= 256) CBIS_SCAN(32, 8);
#undef CBIS_SCAN
  return CBIS_ERR_TOO_LARGE;
}

}  // namespace cbis

using namespace cbis;

CBIS_EXPORT int cbis_conv_max_taps() { return kMaxTaps; }
CBIS_EXPORT int cbis_scan_max_state() { return 256; }

// in: [T, in_ld] of the compute type, the convolution's channels at columns c0 .. c0 + C - 1; out: [T, out_ld].
// w [C, K] and bias [C] 32-bit; state: 32-bit, (K-1) * C floats at `state + slot * slot_stride`.
CBIS_EXPORT int cbis_conv_rows_per_block() { return kConvRows; }

// `update_state` (max_seg_rows <= cbis_conv_rows_per_block() only): the kernel also leaves the state as
// cbis_conv_state_update would.
CBIS_EXPORT int cbis_causal_conv_act(const void* in, int in_ld, int c0, const float* w, const float* bias,
                                     float* state, long long slot_stride, const int* seg_slot, const int* cu_rows,
                                     void* out, int out_ld, int C, int K, int act, int n_segments, int max_seg_rows,
                                     int update_state, int dtype, void* stream) {
  if (n_segments <= 0 || max_seg_rows <= 0) return CBIS_OK;
  if (C <= 0 || K < 1 || K > kMaxTaps) return CBIS_ERR_BAD_SIZE;
  if (update_state && max_seg_rows > kConvRows) return CBIS_ERR_BAD_SIZE;
  if (n_segments > 65535) return CBIS_ERR_TOO_LARGE;
  const dim3 grid((C + 127) / 128, n_segments, (max_seg_rows + kConvRows - 1) / kConvRows);
  if (grid.z > 65535) return CBIS_ERR_TOO_LARGE;
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == CBIS_F32)
    return (int)launch_pdl(causal_conv_act_kernel<float>, grid, dim3(128), 0, st, (const float*)in, in_ld, c0, w, bias,
                           state, slot_stride, seg_slot, cu_rows, (float*)out, out_ld, C, K, act, update_state);
  if (dtype == CBIS_BF16)
    return (int)launch_pdl(causal_conv_act_kernel<__nv_bfloat16>, grid, dim3(128), 0, st, (const __nv_bfloat16*)in, in_ld,
                           c0, w, bias, state, slot_stride, seg_slot, cu_rows, (__nv_bfloat16*)out, out_ld, C, K, act,
                           update_state);
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
                              int n_segments, int H, int P, int N, int G, int dtype, int n_chunks, int chunk_rows,
                              float* chunk_state, float* chunk_logdecay, void* stream) {
  if (n_segments <= 0) return CBIS_OK;
  if (H <= 0 || P <= 0 || N <= 0 || G <= 0 || H % G) return CBIS_ERR_BAD_SIZE;
  if (n_chunks < 1 || (n_chunks > 1 && (chunk_rows < 1 || !chunk_state || !chunk_logdecay))) return CBIS_ERR_BAD_SIZE;
  if ((long long)n_segments * n_chunks > 65535 || H > 65535) return CBIS_ERR_TOO_LARGE;
  cudaStream_t st = (cudaStream_t)stream;
  auto run = [&](int mode) {
    if (dtype == CBIS_F32)
      return launch_scan<float>(xbc, xbc_ld, proj, proj_ld, dt_off, dt_bias, A_log, D, state, slot_stride, seg_slot,
                                cu_rows, y, y_ld, n_segments, H, P, N, G, mode, n_chunks, chunk_rows, chunk_state,
                                chunk_logdecay, st);
    if (dtype == CBIS_BF16)
      return launch_scan<__nv_bfloat16>(xbc, xbc_ld, proj, proj_ld, dt_off, dt_bias, A_log, D, state, slot_stride,
                                        seg_slot, cu_rows, y, y_ld, n_segments, H, P, N, G, mode, n_chunks, chunk_rows,
                                        chunk_state, chunk_logdecay, st);
    return CBIS_ERR_BAD_DTYPE;
  };
  if (n_chunks == 1) return run(0);
  // pieces side by side: end states from zero, the chain of start states, then every piece from its start state
  int err = run(1);
  if (err) return err;
  const long long elems = (long long)H * P * N;
  err = (int)launch_pdl(scan_chain_kernel, dim3((unsigned)((elems + 255) / 256), n_segments), dim3(256), 0, st, chunk_state,
                        (const float*)chunk_logdecay, (const float*)state, slot_stride, seg_slot, cu_rows, n_chunks,
                        chunk_rows, H, P * N);
  if (err) return err;
  return run(2);
}

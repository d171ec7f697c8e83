// A matrix memory with exponential gates (the mLSTM recurrence), in 32-bit arithmetic whatever the storage type.
//
// Per request and head the state is a matrix S [D x V], a vector n [D] and a running maximum m (all zero at the
// start; m = 0, not minus infinity).  For every token, with the log input gate li and the log forget gate lf
//   li = cap * tanh((i_raw + i_bias) / cap),   lf = logsigmoid(cap * tanh((f_raw + f_bias) / cap))    (cap <= 0: no cap)
//   m' = max(lf + m, li);  keep = exp(lf + m - m');  take = exp(li - m')
//   S <- keep S + take k v^T;   n <- keep n + take k
//   y = S^T q / (max(|n . q|, exp(-m')) + den_eps)            q already times q_scale
// A segment's rows are walked in order from the request's state, so a position's values are the same bits whether
// its prompt came whole, in portions or token by token.
//
// grid (column blocks, heads, segments).  A block owns CB columns of S (16, or 32 in steps of short segments); a column
// is spread over L lanes, lane l holding the rows d = l, l + L, ... in registers.  One more warp carries n the same
// way.  Rows come through shared memory TC at a time (32; 4 in steps of short segments): k and q as 32-bit, the block's slice of v, and the three gate numbers of each row (one lane
// of the first warp a row: everything transcendental side by side, the chain of maxima walked with shuffles); the
// next TC rows are on their way from memory, into registers, while these are walked.
// State of a slot: S as [H][V][D], then n as [H][units][D] and m as [H][units], a unit being 16 columns: every block
// reads the copies of n and m of its first unit and writes those of all its units (blocks of 16 or of 32 columns: all
// copies of a head always hold the same numbers), so no block can meet the state another block of its head has
// already moved on.
#include "common.cuh"

namespace cbis {

constexpr int kMemRows = 32;      // rows of a batch for long segments, one lane of the first warp each
constexpr int kMemRowsShort = 4;  // rows of a batch where no segment of the step is longer (decode steps)
constexpr int kMemUnit = 16;      // columns per copy of n and m in the state

__host__ __device__ inline int mem_lanes(int D) { return D <= 256 ? 8 : 16; }


template <typename TT, int NPL, int L, int CB, int TC>
__global__ void __launch_bounds__(CB * L + 32)
matrix_memory_kernel(const TT* qkv, int ld, int q_off, int k_off, int v_off, const float* gates, int gates_ld,
                     const float* __restrict__ i_bias, const float* __restrict__ f_bias, float cap, float q_scale,
                     float den_eps, float* state, long long slot_stride, const int* seg_slot, const int* cu_rows,
                     float* y, int y_ld, int H, int D, int V) {
  constexpr int DP = NPL * L, WORK = CB * L, THREADS = WORK + 32, UNITS = CB / kMemUnit;
  constexpr int KQ_PER = (TC * DP + THREADS - 1) / THREADS, V_PER = (TC * CB + THREADS - 1) / THREADS;
  extern __shared__ float smem[];
  float* ks = smem;                      // [TC][DP]
  float* qs = ks + TC * DP;              // [TC][DP]
  float* vs = qs + TC * DP;              // [TC][CB]
  float* nums = vs + TC * CB;            // [TC][CB]
  float* g_keep = nums + TC * CB;        // [TC]
  float* g_take = g_keep + TC;
  float* g_floor = g_take + TC;          // exp(-m')
  float* nq = g_floor + TC;              // [TC]
  __shared__ float m_run;
  pdl_trigger();
  pdl_wait();
  const int xb = blockIdx.x, h = blockIdx.y, s = blockIdx.z, XB = (V + kMemUnit - 1) / kMemUnit;
  const int row0 = cu_rows[s], n_rows = cu_rows[s + 1] - row0;
  if (n_rows <= 0) return;
  const int tid = threadIdx.x;
  const bool carrier = tid >= WORK;              // the warp that carries n
  const int l = tid % L, c = carrier ? 0 : tid / L;
  const int col = xb * CB + c;
  const bool live = carrier ? (tid - WORK) < L : col < V;
  float* slot = state + (long long)seg_slot[s] * slot_stride;
  // the copies of n and m of this block's first unit of columns are read; all the units it covers are written
  float* sp = carrier ? slot + (size_t)H * V * D + ((size_t)h * XB + xb * UNITS) * D
                      : slot + ((size_t)h * V + (live ? col : 0)) * D;
  float* mp = slot + (size_t)H * V * D + (size_t)H * XB * D + (size_t)h * XB + xb * UNITS;
  float S[NPL];
#pragma unroll
  for (int i = 0; i < NPL; ++i) {
    const int d = l + L * i;
    S[i] = (live && d < D) ? sp[d] : 0.f;
  }
  if (tid == 0) m_run = *mp;
  const TT* qrow = qkv + (size_t)row0 * ld + q_off + h * D;
  const TT* krow = qkv + (size_t)row0 * ld + k_off + h * D;
  const TT* vrow = qkv + (size_t)row0 * ld + v_off + h * V + xb * CB;
  const int vcols = min(CB, V - xb * CB);

  // what this thread fetches of a batch of rows: entries of k and q (row t = idx / DP, entry d = idx % DP), of the
  // block's slice of v, and (the first TC threads) a row's two raw gates
  float r_k[KQ_PER], r_q[KQ_PER], r_v[V_PER], r_gi = 0.f, r_gf = 0.f;
  auto fetch = [&](int first) {
    const int tc = min(TC, n_rows - first);
#pragma unroll
    for (int j = 0; j < KQ_PER; ++j) {
      const int idx = tid + THREADS * j, t = idx / DP, d = idx % DP;
      const bool ok = t < tc && d < D;
      r_k[j] = ok ? to_f32(krow[(size_t)(first + t) * ld + d]) : 0.f;
      r_q[j] = ok ? to_f32(qrow[(size_t)(first + t) * ld + d]) : 0.f;
    }
#pragma unroll
    for (int j = 0; j < V_PER; ++j) {
      const int idx = tid + THREADS * j, t = idx / CB, cc = idx % CB;
      r_v[j] = (t < tc && cc < vcols) ? to_f32(vrow[(size_t)(first + t) * ld + cc]) : 0.f;
    }
    if (tid < tc) {
      const float* g = gates + (size_t)(row0 + first + tid) * gates_ld;
      r_gi = g[h];
      r_gf = g[H + h];
    }
  };
  const float bias_i = i_bias[h], bias_f = f_bias[h];
  fetch(0);
  for (int first = 0; first < n_rows; first += TC) {
    const int tc = min(TC, n_rows - first);
    __syncthreads();                 // the rows staged before have been used
#pragma unroll
    for (int j = 0; j < KQ_PER; ++j) {
      const int idx = tid + THREADS * j;
      if (idx < TC * DP) {
        ks[idx] = r_k[j];
        qs[idx] = r_q[j] * q_scale;
      }
    }
#pragma unroll
    for (int j = 0; j < V_PER; ++j) {
      const int idx = tid + THREADS * j;
      if (idx < TC * CB) vs[idx] = r_v[j];
    }
    if (tid < 32) {                  // the gates of these rows: lane t has row t
      float li = 0.f, lf = 0.f;
      if (tid < tc) {
        float zi = r_gi + bias_i, zf = r_gf + bias_f;
        if (cap > 0.f) {
          zi = cap * tanhf(zi / cap);
          zf = cap * tanhf(zf / cap);
        }
        li = zi;
        lf = fminf(zf, 0.f) - log1pf(expf(-fabsf(zf)));       // logsigmoid
      }
      // the chain of maxima in the rows' order, every lane walking it with the gates handed round by shuffles: the
      // same sums in the same order wherever a batch starts
      float m = m_run, m_before = 0.f, m_after = 0.f;
      for (int t = 0; t < tc; ++t) {
        const float f = __shfl_sync(0xffffffffu, lf, t), i = __shfl_sync(0xffffffffu, li, t);
        const float mn = fmaxf(f + m, i);
        if (tid == t) {
          m_before = m;
          m_after = mn;
        }
        m = mn;
      }
      __syncwarp();
      if (tid == 0) m_run = m;
      if (tid < tc) {
        g_keep[tid] = expf(lf + m_before - m_after);
        g_take[tid] = expf(li - m_after);
        g_floor[tid] = expf(-m_after);
      }
    }
    __syncthreads();
    if (first + TC < n_rows) fetch(first + TC);      // in flight while these rows are walked
    if (!carrier) {
#pragma unroll 4     // rows in flight together: 2 took 860 us for 2,048 rows of 8 heads of 128 x 256, 4 takes 660, 8 takes 760
      for (int t = 0; t < tc; ++t) {
        const float keep = g_keep[t], tv = g_take[t] * vs[t * CB + c];
        const float* kt = ks + t * DP + l;
        const float* qt = qs + t * DP + l;
        float a0 = 0.f, a1 = 0.f;
#pragma unroll
        for (int i = 0; i < NPL; ++i) {
          S[i] = fmaf(keep, S[i], tv * kt[L * i]);
          if (i & 1) a1 = fmaf(S[i], qt[L * i], a1);
          else a0 = fmaf(S[i], qt[L * i], a0);
        }
        float acc = a0 + a1;
#pragma unroll
        for (int o = 1; o < L; o <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (l == 0) nums[t * CB + c] = acc;
      }
    } else {
#pragma unroll 4
      for (int t = 0; t < tc; ++t) {
        const float keep = g_keep[t], take = g_take[t];
        const float* kt = ks + t * DP + l;
        const float* qt = qs + t * DP + l;
        float acc = 0.f;
#pragma unroll
        for (int i = 0; i < NPL; ++i) {
          S[i] = fmaf(keep, S[i], take * kt[L * i]);
          acc = fmaf(S[i], qt[L * i], acc);
        }
        if (!live) acc = 0.f;
#pragma unroll
        for (int o = 1; o < L; o <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (tid == WORK) nq[t] = acc;
      }
    }
    __syncthreads();
    for (int i = tid; i < tc * CB; i += blockDim.x) {
      const int t = i / CB, cc = i % CB;
      if (cc < vcols) {
        const float den = fmaxf(fabsf(nq[t]), g_floor[t]) + den_eps;
        y[(size_t)(row0 + first + t) * y_ld + h * V + xb * CB + cc] = nums[i] / den;
      }
    }
  }
  if (live) {
    const int copies = carrier ? min(UNITS, XB - xb * UNITS) : 1;
    for (int u = 0; u < copies; ++u)
#pragma unroll
      for (int i = 0; i < NPL; ++i) {
        const int d = l + L * i;
        if (d < D) sp[(size_t)u * D + d] = S[i];
      }
  }
  __syncthreads();
  if (tid == 0)
    for (int u = 0; u < min(UNITS, XB - xb * UNITS); ++u) mp[u] = m_run;
}

template <typename TT>
static int launch_memory(const void* qkv, int ld, int q_off, int k_off, int v_off, const float* gates, int gates_ld,
                         const float* i_bias, const float* f_bias, float cap, float q_scale, float den_eps, float* state,
                         long long slot_stride, const int* seg_slot, const int* cu_rows, float* y, int y_ld, int S, int H,
                         int D, int V, int max_seg_rows, cudaStream_t st) {
  const int L = mem_lanes(D);
  const int npl = (D + L - 1) / L;
  // long segments: blocks of 16 columns (a memory of 8 heads of 256 columns gives 128 blocks to the 148 SMs where
  // blocks of 32 gave 64) walking 32 rows a batch; steps of short segments (decoding): blocks of 32 columns (half
  // as many blocks fetch k and q) and batches of 4 rows (a batch's staging is sized for its rows)
  const bool shorts = max_seg_rows > 0 && max_seg_rows <= kMemRowsShort;
#define CBIS_MEM_AS(NPL, LL, CBB, TCC)                                                                                \
  do {                                                                                                               \
    const size_t smem = ((size_t)2 * TCC * NPL * LL + 2 * TCC * CBB + 4 * TCC) * sizeof(float);                      \
    if (smem > 48 * 1024)                                                                                            \
      cudaFuncSetAttribute(matrix_memory_kernel<TT, NPL, LL, CBB, TCC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    return (int)launch_pdl(matrix_memory_kernel<TT, NPL, LL, CBB, TCC>, dim3((V + CBB - 1) / CBB, H, S), dim3(CBB * LL + 32), \
                           smem, st, (const TT*)qkv, ld, q_off, k_off, v_off, gates, gates_ld, i_bias, f_bias, cap,  \
                           q_scale, den_eps, state, slot_stride, seg_slot, cu_rows, y, y_ld, H, D, V);               \
  } while (0)
#define CBIS_MEM(NPL, LL)                                          \
  do {                                                             \
    if (shorts) CBIS_MEM_AS(NPL, LL, 32, kMemRowsShort);           \
    CBIS_MEM_AS(NPL, LL, 16, kMemRows);                            \
  } while (0)
  if (L == 8) {
    if (npl <= 2) CBIS_MEM(2, 8);
    if (npl <= 4) CBIS_MEM(4, 8);
    if (npl <= 6) CBIS_MEM(6, 8);
    if (npl <= 8) CBIS_MEM(8, 8);
    if (npl <= 12) CBIS_MEM(12, 8);
    if (npl <= 16) CBIS_MEM(16, 8);
    if (npl <= 24) CBIS_MEM(24, 8);
    CBIS_MEM(32, 8);
  }
  if (npl <= 24) CBIS_MEM(24, 16);
  CBIS_MEM(32, 16);
#undef CBIS_MEM
#undef CBIS_MEM_AS
}

}  // namespace cbis

using namespace cbis;

CBIS_EXPORT int cbis_matrix_memory_max_dim() { return 512; }

// Floats of one request's state for H heads of D x V (the kernel's own layout, see above).
CBIS_EXPORT long long cbis_matrix_memory_state_floats(int H, int D, int V) {
  if (H <= 0 || D <= 0 || V <= 0 || D > 512) return -1;
  const int XB = (V + kMemUnit - 1) / kMemUnit;
  return (long long)H * V * D + (long long)H * XB * D + (long long)H * XB;
}

// qkv [T, ld] of the compute type: q at columns q_off + h * D, k at k_off + h * D, v at v_off + h * V;
// gates [T, gates_ld] 32-bit: the raw input gate of head h at column h, the raw forget gate at column H + h;
// max_seg_rows: the longest segment of the step (0: unknown); y [T, y_ld] 32-bit, H * V columns; state: 32-bit, cbis_matrix_memory_state_floats per slot at `state + slot * slot_stride`.
CBIS_EXPORT int cbis_matrix_memory(const void* qkv, int ld, int q_off, int k_off, int v_off, const float* gates,
                                   int gates_ld, const float* i_bias, const float* f_bias, float cap, float q_scale,
                                   float den_eps, float* state, long long slot_stride, const int* seg_slot,
                                   const int* cu_rows, float* y, int y_ld, int n_segments, int H, int D, int V, int dtype,
                                   void* stream, int max_seg_rows) {
  if (n_segments <= 0) return CBIS_OK;
  if (H <= 0 || D <= 0 || V <= 0 || D > 512) return CBIS_ERR_BAD_SIZE;
  if (n_segments > 65535 || H > 65535) return CBIS_ERR_TOO_LARGE;
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == CBIS_F32)
    return launch_memory<float>(qkv, ld, q_off, k_off, v_off, gates, gates_ld, i_bias, f_bias, cap, q_scale, den_eps,
                                state, slot_stride, seg_slot, cu_rows, y, y_ld, n_segments, H, D, V, max_seg_rows, st);
  if (dtype == CBIS_BF16)
    return launch_memory<__nv_bfloat16>(qkv, ld, q_off, k_off, v_off, gates, gates_ld, i_bias, f_bias, cap, q_scale,
                                        den_eps, state, slot_stride, seg_slot, cu_rows, y, y_ld, n_segments, H, D, V, max_seg_rows, st);
  return CBIS_ERR_BAD_DTYPE;
}

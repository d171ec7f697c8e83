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
// grid (column blocks, heads, segments).  A block owns CB = 256 / L columns of S; a column is spread over L lanes,
// lane l holding the rows d = l, l + L, ... in registers.  One more warp carries n the same way.  Rows come through
// shared memory TC at a time: k and q as 32-bit, the block's slice of v, and the three gate numbers of each row (the
// chain of maxima is walked by one thread, everything transcendental around it by TC threads side by side).
// State of a slot: S as [H][V][D], then n as [H][column blocks][D] and m as [H][column blocks]: every block reads
// and writes copies of n and m of its own, so no block can meet the state another block of its head has already
// moved on.
#include "common.cuh"

namespace cbis {

constexpr int kMemRows = 16;      // TC

__host__ __device__ inline int mem_lanes(int D) { return D <= 256 ? 8 : 16; }

template <typename TT, int NPL, int L>
__global__ void __launch_bounds__(256 + 32)
matrix_memory_kernel(const TT* qkv, int ld, int q_off, int k_off, int v_off, const float* gates, int gates_ld,
                     const float* __restrict__ i_bias, const float* __restrict__ f_bias, float cap, float q_scale,
                     float den_eps, float* state, long long slot_stride, const int* seg_slot, const int* cu_rows,
                     float* y, int y_ld, int H, int D, int V) {
  constexpr int CB = 256 / L, DP = NPL * L, TC = kMemRows;
  extern __shared__ float smem[];
  float* ks = smem;                      // [TC][DP]
  float* qs = ks + TC * DP;              // [TC][DP]
  float* vs = qs + TC * DP;              // [TC][CB]
  float* nums = vs + TC * CB;            // [TC][CB]
  float* g_keep = nums + TC * CB;        // [TC]
  float* g_take = g_keep + TC;
  float* g_floor = g_take + TC;          // exp(-m')
  float* g_li = g_floor + TC;
  float* g_lf = g_li + TC;
  float* g_m0 = g_lf + TC;               // m before the row
  float* g_m1 = g_m0 + TC;               // m after the row
  float* nq = g_m1 + TC;                 // [TC]
  __shared__ float m_run;
  pdl_trigger();
  pdl_wait();
  const int xb = blockIdx.x, h = blockIdx.y, s = blockIdx.z, XB = gridDim.x;
  const int row0 = cu_rows[s], n_rows = cu_rows[s + 1] - row0;
  if (n_rows <= 0) return;
  const int tid = threadIdx.x;
  const bool carrier = tid >= 256;               // the warp that carries n
  const int l = tid % L, c = carrier ? 0 : tid / L;
  const int col = xb * CB + c;
  const bool live = carrier ? (tid - 256) < L : col < V;
  float* slot = state + (long long)seg_slot[s] * slot_stride;
  float* sp = carrier ? slot + (size_t)H * V * D + ((size_t)h * XB + xb) * D
                      : slot + ((size_t)h * V + (live ? col : 0)) * D;
  float* mp = slot + (size_t)H * V * D + (size_t)H * XB * D + (size_t)h * XB + xb;
  float S[NPL];
#pragma unroll
  for (int i = 0; i < NPL; ++i) {
    const int d = l + L * i;
    S[i] = (live && d < D) ? sp[d] : 0.f;
  }
  if (tid == 0) m_run = *mp;
  for (int i = tid; i < 2 * TC * DP; i += blockDim.x) ks[i] = 0.f;      // the padding beyond D stays zero
  const TT* qrow = qkv + (size_t)row0 * ld + q_off + h * D;
  const TT* krow = qkv + (size_t)row0 * ld + k_off + h * D;
  const TT* vrow = qkv + (size_t)row0 * ld + v_off + h * V + xb * CB;
  const int vcols = min(CB, V - xb * CB);

  for (int first = 0; first < n_rows; first += TC) {
    const int tc = min(TC, n_rows - first);
    __syncthreads();                 // the rows staged before have been used (and the zero fill is done)
    for (int i = tid; i < tc * D; i += blockDim.x) {
      const int t = i / D, d = i % D;
      ks[t * DP + d] = to_f32(krow[(size_t)(first + t) * ld + d]);
      qs[t * DP + d] = to_f32(qrow[(size_t)(first + t) * ld + d]) * q_scale;
    }
    for (int i = tid; i < tc * CB; i += blockDim.x) {
      const int t = i / CB, cc = i % CB;
      vs[i] = cc < vcols ? to_f32(vrow[(size_t)(first + t) * ld + cc]) : 0.f;
    }
    if (tid < 32) {                  // the gates of these rows
      if (tid < tc) {
        const float* g = gates + (size_t)(row0 + first + tid) * gates_ld;
        float zi = g[h] + i_bias[h], zf = g[H + h] + f_bias[h];
        if (cap > 0.f) {
          zi = cap * tanhf(zi / cap);
          zf = cap * tanhf(zf / cap);
        }
        g_li[tid] = zi;
        g_lf[tid] = fminf(zf, 0.f) - log1pf(expf(-fabsf(zf)));       // logsigmoid
      }
      __syncwarp();
      if (tid == 0) {
        float m = m_run;
        for (int t = 0; t < tc; ++t) {
          g_m0[t] = m;
          m = fmaxf(g_lf[t] + m, g_li[t]);
          g_m1[t] = m;
        }
        m_run = m;
      }
      __syncwarp();
      if (tid < tc) {
        g_keep[tid] = expf(g_lf[tid] + g_m0[tid] - g_m1[tid]);
        g_take[tid] = expf(g_li[tid] - g_m1[tid]);
        g_floor[tid] = expf(-g_m1[tid]);
      }
    }
    __syncthreads();
    if (!carrier) {
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
        if (tid == 256) nq[t] = acc;
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
#pragma unroll
    for (int i = 0; i < NPL; ++i) {
      const int d = l + L * i;
      if (d < D) sp[d] = S[i];
    }
  }
  __syncthreads();
  if (tid == 0) *mp = m_run;
}

template <typename TT>
static int launch_memory(const void* qkv, int ld, int q_off, int k_off, int v_off, const float* gates, int gates_ld,
                         const float* i_bias, const float* f_bias, float cap, float q_scale, float den_eps, float* state,
                         long long slot_stride, const int* seg_slot, const int* cu_rows, float* y, int y_ld, int S, int H,
                         int D, int V, cudaStream_t st) {
  const int L = mem_lanes(D), CB = 256 / L;
  const int npl = (D + L - 1) / L;
#define CBIS_MEM(NPL, LL)                                                                                            \
  do {                                                                                                               \
    const size_t smem = ((size_t)2 * kMemRows * NPL * LL + 2 * kMemRows * (256 / LL) + 8 * kMemRows) * sizeof(float); \
    if (smem > 48 * 1024)                                                                                            \
      cudaFuncSetAttribute(matrix_memory_kernel<TT, NPL, LL>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    return (int)launch_pdl(matrix_memory_kernel<TT, NPL, LL>, dim3((V + CB - 1) / CB, H, S), dim3(256 + 32), smem, st, \
                           (const TT*)qkv, ld, q_off, k_off, v_off, gates, gates_ld, i_bias, f_bias, cap, q_scale,   \
                           den_eps, state, slot_stride, seg_slot, cu_rows, y, y_ld, H, D, V);                        \
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
}

}  // namespace cbis

using namespace cbis;

CBIS_EXPORT int cbis_matrix_memory_max_dim() { return 512; }

// Floats of one request's state for H heads of D x V (the kernel's own layout, see above).
CBIS_EXPORT long long cbis_matrix_memory_state_floats(int H, int D, int V) {
  if (H <= 0 || D <= 0 || V <= 0 || D > 512) return -1;
  const int CB = 256 / mem_lanes(D), XB = (V + CB - 1) / CB;
  return (long long)H * V * D + (long long)H * XB * D + (long long)H * XB;
}

// qkv [T, ld] of the compute type: q at columns q_off + h * D, k at k_off + h * D, v at v_off + h * V;
// gates [T, gates_ld] 32-bit: the raw input gate of head h at column h, the raw forget gate at column H + h;
// y [T, y_ld] 32-bit, H * V columns; state: 32-bit, cbis_matrix_memory_state_floats per slot at `state + slot * slot_stride`.
CBIS_EXPORT int cbis_matrix_memory(const void* qkv, int ld, int q_off, int k_off, int v_off, const float* gates,
                                   int gates_ld, const float* i_bias, const float* f_bias, float cap, float q_scale,
                                   float den_eps, float* state, long long slot_stride, const int* seg_slot,
                                   const int* cu_rows, float* y, int y_ld, int n_segments, int H, int D, int V, int dtype,
                                   void* stream) {
  if (n_segments <= 0) return CBIS_OK;
  if (H <= 0 || D <= 0 || V <= 0 || D > 512) return CBIS_ERR_BAD_SIZE;
  if (n_segments > 65535 || H > 65535) return CBIS_ERR_TOO_LARGE;
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == CBIS_F32)
    return launch_memory<float>(qkv, ld, q_off, k_off, v_off, gates, gates_ld, i_bias, f_bias, cap, q_scale, den_eps,
                                state, slot_stride, seg_slot, cu_rows, y, y_ld, n_segments, H, D, V, st);
  if (dtype == CBIS_BF16)
    return launch_memory<__nv_bfloat16>(qkv, ld, q_off, k_off, v_off, gates, gates_ld, i_bias, f_bias, cap, q_scale,
                                        den_eps, state, slot_stride, seg_slot, cu_rows, y, y_ld, n_segments, H, D, V, st);
  return CBIS_ERR_BAD_DTYPE;
}

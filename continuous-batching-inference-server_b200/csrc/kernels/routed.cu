// A routed mixture of gated feed-forwards.
//   * route_topk: router logits in 32-bit, a score per expert (sigmoid or softmax), the `top` largest chosen
//     (ties: the lower index), their weights the scores as they are or divided by their sum;
//   * routed_gate_up / routed_down: the chosen experts of every row, one (row, choice) pair at a time, the experts'
//     matrices streamed by warps (a row's result depends on nothing but the row: no other row of the batch and no
//     position inside it changes a sum's order).  The weight of a choice multiplies the expert's input
//     (`weight_on_input`), which for the two first products is the same as multiplying their 32-bit sums, or its output.
#include "common.cuh"

namespace cbis {

constexpr int kScoreSigmoid = 0, kScoreSoftmax = 1;

// grid (rows), 128 threads; shared: E floats.  ids [rows, top] int32, weights [rows, top] float.
template <typename TT>
__global__ void __launch_bounds__(128)
route_topk_kernel(const TT* h, int h_ld, const TT* __restrict__ router, int* ids, float* weights, int W, int E, int top,
                  int score, int renormalize) {
  extern __shared__ float z[];
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const TT* hr = h + (size_t)r * h_ld;
  for (int e = warp; e < E; e += 4) {
    const TT* wr = router + (size_t)e * W;
    float acc = 0.f;
    for (int k = lane; k < W; k += 32) acc = fmaf(to_f32(hr[k]), to_f32(wr[k]), acc);
    acc = warp_sum(acc);
    if (lane == 0) z[e] = acc;
  }
  __syncthreads();
  if (warp != 0) return;
  float zmax = -INFINITY, denom = 1.f;
  if (score == kScoreSoftmax) {
    for (int e = lane; e < E; e += 32) zmax = fmaxf(zmax, z[e]);
    zmax = warp_max(zmax);
    float d = 0.f;
    for (int e = lane; e < E; e += 32) d += expf(z[e] - zmax);
    denom = warp_sum(d);
  }
  float total = 0.f;
  for (int k = 0; k < top; ++k) {
    // the largest logit not taken yet; equal logits: the lower index
    float best = -INFINITY;
    int arg = E;
    for (int e = lane; e < E; e += 32) {
      const float v = z[e];
      if (v > best) { best = v; arg = e; }      // within a lane indices rise, so the first of equals stays
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
      if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
    }
    if (arg >= E) arg = k < E ? k : 0;          // rows of not-a-numbers (padding): any valid expert
    const float sc = score == kScoreSoftmax ? expf(best - zmax) / denom : sigmoid_f32(best);
    total += sc;
    if (lane == 0) {
      ids[(size_t)r * top + k] = arg;
      weights[(size_t)r * top + k] = sc;
      z[arg] = -INFINITY;
    }
    __syncwarp();
  }
  if (renormalize && lane == 0)
    for (int k = 0; k < top; ++k) weights[(size_t)r * top + k] /= total;
}

// grid (pairs, ceil(F / 8)), 256 threads = 8 warps, a warp per hidden column f of pair (row, choice):
//   hid[pair, f] = act(s * (Wg_e[f, :] . h[row])) * (s * (Wu_e[f, :] . h[row])),  s = weight (on input) or 1.
// gate_up: [E, 2F, W] (an expert's gate rows, then its up rows).
template <typename TT>
__global__ void __launch_bounds__(256)
routed_gate_up_kernel(const TT* h, int h_ld, const TT* __restrict__ gate_up, const int* ids, const float* weights,
                      TT* hid, int W, int F, int top, int act, int weight_on_input) {
  extern __shared__ float hs[];
  pdl_trigger();
  pdl_wait();
  const int pair = blockIdx.x, row = pair / top;
  const TT* hr = h + (size_t)row * h_ld;
  for (int k = threadIdx.x; k < W; k += 256) hs[k] = to_f32(hr[k]);
  __syncthreads();
  const int lane = threadIdx.x & 31, f = blockIdx.y * 8 + (threadIdx.x >> 5);
  if (f >= F) return;
  const int e = ids[pair];
  const TT* wg = gate_up + ((size_t)e * 2 * F + f) * W;
  const TT* wu = wg + (size_t)F * W;
  float g = 0.f, u = 0.f;
  for (int k = lane; k < W; k += 32) {
    const float x = hs[k];
    g = fmaf(to_f32(wg[k]), x, g);
    u = fmaf(to_f32(wu[k]), x, u);
  }
  g = warp_sum(g);
  u = warp_sum(u);
  if (lane == 0) {
    const float s = weight_on_input ? weights[pair] : 1.f;
    from_f32(hid[(size_t)pair * F + f], activate(s * g, act) * (s * u));
  }
}

// grid (rows, ceil(W / 8)), 256 threads: out[row, n] = sum over the row's choices k of
//   (weight on output ? weight : 1) * (Wd_e[n, :] . hid[row * top + k, :]),   down: [E, W, F].  out is 32-bit.
template <typename TT>
__global__ void __launch_bounds__(256)
routed_down_kernel(const TT* hid, const TT* __restrict__ down, const int* ids, const float* weights, float* out,
                   int out_ld, int W, int F, int top, int weight_on_input) {
  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.x, lane = threadIdx.x & 31, n = blockIdx.y * 8 + (threadIdx.x >> 5);
  if (n >= W) return;
  float total = 0.f;
  for (int k = 0; k < top; ++k) {
    const int pair = row * top + k;
    const TT* wd = down + ((size_t)ids[pair] * W + n) * F;
    const TT* hp = hid + (size_t)pair * F;
    float acc = 0.f;
    for (int f = lane; f < F; f += 32) acc = fmaf(to_f32(wd[f]), to_f32(hp[f]), acc);
    acc = warp_sum(acc);
    total += weight_on_input ? acc : acc * weights[pair];
  }
  if (lane == 0) out[(size_t)row * out_ld + n] = total;
}

}  // namespace cbis

using namespace cbis;

CBIS_EXPORT int cbis_route_topk(const void* h, int h_ld, const void* router, int* ids, float* weights, int rows, int W,
                                int E, int top, int score, int renormalize, int dtype, void* stream) {
  if (rows <= 0) return CBIS_OK;
  if (W <= 0 || E <= 0 || top <= 0 || top > E || (score != kScoreSigmoid && score != kScoreSoftmax)) return CBIS_ERR_BAD_SIZE;
  if (E > 8192) return CBIS_ERR_TOO_LARGE;
  cudaStream_t st = (cudaStream_t)stream;
  const size_t smem = (size_t)E * sizeof(float);
  if (dtype == CBIS_F32)
    return (int)launch_pdl(route_topk_kernel<float>, dim3(rows), dim3(128), smem, st, (const float*)h, h_ld,
                           (const float*)router, ids, weights, W, E, top, score, renormalize);
  if (dtype == CBIS_BF16)
    return (int)launch_pdl(route_topk_kernel<__nv_bfloat16>, dim3(rows), dim3(128), smem, st, (const __nv_bfloat16*)h, h_ld,
                           (const __nv_bfloat16*)router, ids, weights, W, E, top, score, renormalize);
  return CBIS_ERR_BAD_DTYPE;
}

CBIS_EXPORT int cbis_routed_gate_up(const void* h, int h_ld, const void* gate_up, const int* ids, const float* weights,
                                    void* hid, int rows, int W, int F, int top, int act, int weight_on_input, int dtype,
                                    void* stream) {
  if (rows <= 0) return CBIS_OK;
  if (W <= 0 || F <= 0 || top <= 0) return CBIS_ERR_BAD_SIZE;
  if (W > 12288 || F > 8 * 65535) return CBIS_ERR_TOO_LARGE;
  cudaStream_t st = (cudaStream_t)stream;
  const dim3 grid(rows * top, (F + 7) / 8);
  const size_t smem = (size_t)W * sizeof(float);
  if (dtype == CBIS_F32)
    return (int)launch_pdl(routed_gate_up_kernel<float>, grid, dim3(256), smem, st, (const float*)h, h_ld,
                           (const float*)gate_up, ids, weights, (float*)hid, W, F, top, act, weight_on_input);
  if (dtype == CBIS_BF16)
    return (int)launch_pdl(routed_gate_up_kernel<__nv_bfloat16>, grid, dim3(256), smem, st, (const __nv_bfloat16*)h, h_ld,
                           (const __nv_bfloat16*)gate_up, ids, weights, (__nv_bfloat16*)hid, W, F, top, act,
                           weight_on_input);
  return CBIS_ERR_BAD_DTYPE;
}

CBIS_EXPORT int cbis_routed_down(const void* hid, const void* down, const int* ids, const float* weights, float* out,
                                 int out_ld, int rows, int W, int F, int top, int weight_on_input, int dtype,
                                 void* stream) {
  if (rows <= 0) return CBIS_OK;
  if (W <= 0 || F <= 0 || top <= 0) return CBIS_ERR_BAD_SIZE;
  if (W > 8 * 65535) return CBIS_ERR_TOO_LARGE;
  cudaStream_t st = (cudaStream_t)stream;
  const dim3 grid(rows, (W + 7) / 8);
  if (dtype == CBIS_F32)
    return (int)launch_pdl(routed_down_kernel<float>, grid, dim3(256), 0, st, (const float*)hid, (const float*)down, ids,
                           weights, out, out_ld, W, F, top, weight_on_input);
  if (dtype == CBIS_BF16)
    return (int)launch_pdl(routed_down_kernel<__nv_bfloat16>, grid, dim3(256), 0, st, (const __nv_bfloat16*)hid,
                           (const __nv_bfloat16*)down, ids, weights, out, out_ld, W, F, top, weight_on_input);
  return CBIS_ERR_BAD_DTYPE;
}

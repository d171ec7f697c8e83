// Root-mean-square norms around the residual stream, in 32-bit arithmetic whatever the storage types.
//
//   add_rmsnorm: what a part produced is (optionally) normalised itself, added to the residual stream, and the
//   stream's row is normalised for the next part, all in one pass over the row:
//     d = delta[s,:] (+ delta_bias)                                           what the part before left
//     if post_w: d = d / sqrt(mean(d^2) + post_eps) * (post_offset + post_w)   a norm AFTER the part
//     v = x[s,:] + d;  x[s,:] = v                                             the stream moves on (32-bit)
//     out[r,:] = v / sqrt(mean(v^2) + eps) * (offset + w)                      the norm BEFORE the next part
//   offset 1 is for weights stored around zero, offset 0 for weights stored as they are applied.  With `rows` only
//   those rows are produced and x is left as it is (the rows whose logits are wanted, before the head).
#include "common.cuh"

namespace cbis {

// One block per output row r; source row s = rows ? rows[r] : r.  The row and the delta wait in shared memory
// (2 d floats) between the passes, so x and delta are read once.
template <typename TD, typename TO>
__global__ void add_rmsnorm_kernel(float* x, const TD* delta, int delta_ld, const float* __restrict__ delta_bias,
                                   const float* __restrict__ post_w, float post_eps, float post_offset,
                                   const float* __restrict__ w, float eps, float offset, TO* out, const int* rows,
                                   int d) {
  extern __shared__ float smem[];
  float* row = smem;           // d floats
  float* dl = smem + d;        // d floats
  __shared__ float red[33];
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x;
  const int s = rows ? rows[r] : r;
  float* xrow = x + (size_t)s * d;
  const TD* drow = delta ? delta + (size_t)s * delta_ld : nullptr;
  float dscale = 1.f;
  if (drow) {
    float ss = 0.f;
    for (int c = threadIdx.x; c < d; c += blockDim.x) {
      float v = to_f32(drow[c]);
      if (delta_bias) v += delta_bias[c];
      dl[c] = v;
      ss += v * v;
    }
    if (post_w) dscale = 1.0f / sqrtf(block_sum(ss, red) / (float)d + post_eps);
  }
  float ss = 0.f;
  for (int c = threadIdx.x; c < d; c += blockDim.x) {
    float v = xrow[c];
    if (drow) v += post_w ? dl[c] * dscale * (post_offset + post_w[c]) : dl[c];
    row[c] = v;
    ss += v * v;
  }
  const float inv = 1.0f / sqrtf(block_sum(ss, red) / (float)d + eps);
  const bool write_x = rows == nullptr && drow != nullptr;
  TO* orow = out ? out + (size_t)r * d : nullptr;
  for (int c = threadIdx.x; c < d; c += blockDim.x) {
    const float v = row[c];
    if (write_x) xrow[c] = v;
    if (orow) from_f32(orow[c], w ? v * inv * (offset + w[c]) : v);
  }
}

}  // namespace cbis

using namespace cbis;

CBIS_EXPORT int cbis_rms_residual_max_width() { return (200 * 1024 / 4 - 64) / 2; }

// x: 32-bit [*, d]; delta (may be null): [*, delta_ld] of delta_dtype; out (may be null): [n, d] of out_dtype.
CBIS_EXPORT int cbis_add_rmsnorm(float* x, const void* delta, int delta_ld, int delta_dtype, const float* delta_bias,
                                 const float* post_w, float post_eps, float post_offset, const float* w, float eps,
                                 float offset, void* out, int out_dtype, const int* rows, int n, int d, void* stream) {
  if (n <= 0) return CBIS_OK;
  if (d <= 0 || d > cbis_rms_residual_max_width()) return CBIS_ERR_BAD_SIZE;
  const int threads = d >= 2048 ? 512 : (d >= 512 ? 256 : 128);
  const size_t smem = (size_t)2 * d * sizeof(float);
  cudaStream_t st = (cudaStream_t)stream;
#define CBIS_ARN(TD, TO)                                                                                              \
  do {                                                                                                                \
    if (smem > 48 * 1024)                                                                                             \
      cudaFuncSetAttribute(add_rmsnorm_kernel<TD, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);       \
    return (int)launch_pdl(add_rmsnorm_kernel<TD, TO>, dim3(n), dim3(threads), smem, st, x, (const TD*)delta, delta_ld, \
                           delta_bias, post_w, post_eps, post_offset, w, eps, offset, (TO*)out, rows, d);             \
  } while (0)
  const int dd = delta ? delta_dtype : CBIS_F32;
  if (dd == CBIS_F32 && out_dtype == CBIS_F32) CBIS_ARN(float, float);
  if (dd == CBIS_F32 && out_dtype == CBIS_BF16) CBIS_ARN(float, __nv_bfloat16);
  if (dd == CBIS_BF16 && out_dtype == CBIS_BF16) CBIS_ARN(__nv_bfloat16, __nv_bfloat16);
  if (dd == CBIS_BF16 && out_dtype == CBIS_F32) CBIS_ARN(__nv_bfloat16, float);
#undef CBIS_ARN
  return CBIS_ERR_BAD_DTYPE;
}

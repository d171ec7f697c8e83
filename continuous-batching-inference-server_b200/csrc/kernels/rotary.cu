// Rotary positions and a gate per head, in 32-bit arithmetic whatever the storage type.
//
//   rope_rows: in every row r (position p = positions[r]) and every head, `dims` entries starting at a column are
//   rotated in pairs: entry i with entry i + dims/2 ("rotate half"), by the angle p * base^(-2 i / dims):
//     (u, v) -> (u cos a - v sin a, v cos a + u sin a).
//   Source and destination may be different buffers with different strides between heads (a head's rotated part is
//   moved to its place among the columns the attention kernel reads); entries beyond `dims` up to `width` are copied.
//   head_gate_mul: out[r, h, :] = x[r, h, :] * sigmoid(gate[r, h]), one number per row and head.
#include "common.cuh"

namespace cbis {

// grid (rows); a thread takes pairs (head, i).  Angles in 32-bit from the integer position: a = p * f_i with the
// frequencies f_i = base^(-2 i / dims) handed in as a table (made on the host in 64-bit, rounded once); sincosf keeps
// its full range reduction (no fast-math).
template <typename TT>
__global__ void rope_rows_kernel(const TT* src, int src_ld, int src_col0, int src_head_stride, TT* dst, int dst_ld,
                                 int dst_col0, int dst_head_stride, const int* positions, int heads, int width, int dims,
                                 const float* __restrict__ freqs) {
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x;
  const float p = (float)positions[r];
  const int half = dims / 2;
  const TT* s0 = src + (size_t)r * src_ld + src_col0;
  TT* d0 = dst + (size_t)r * dst_ld + dst_col0;
  const int per_head = half + (width - dims);      // pairs, then entries that pass unchanged
  for (int u = threadIdx.x; u < heads * per_head; u += blockDim.x) {
    const int h = u / per_head, i = u % per_head;
    const TT* sh = s0 + (size_t)h * src_head_stride;
    TT* dh = d0 + (size_t)h * dst_head_stride;
    if (i < half) {
      float sn, cs;
      sincosf(p * freqs[i], &sn, &cs);
      const float a = to_f32(sh[i]), b = to_f32(sh[i + half]);
      from_f32(dh[i], a * cs - b * sn);
      from_f32(dh[i + half], b * cs + a * sn);
    } else {
      const int c = dims + (i - half);
      dh[c] = sh[c];
    }
  }
}

// grid over elements; x, out: [rows, heads * width]; gate: [rows, gate_ld] with the heads' numbers at gate_col0...
template <typename TT, typename TG>
__global__ void head_gate_mul_kernel(const TT* x, int x_ld, const TG* gate, int gate_ld, TT* out, int out_ld, int rows,
                                     int heads, int width) {
  pdl_trigger();
  pdl_wait();
  const size_t n = (size_t)heads * width, total = (size_t)rows * n;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t r = i / n;
    const int c = (int)(i % n);
    const float g = sigmoid_f32(to_f32(gate[r * gate_ld + c / width]));
    from_f32(out[r * out_ld + c], to_f32(x[r * x_ld + c]) * g);
  }
}

}  // namespace cbis

using namespace cbis;

CBIS_EXPORT int cbis_rope_rows(const void* src, int src_ld, int src_col0, int src_head_stride, void* dst, int dst_ld,
                               int dst_col0, int dst_head_stride, const int* positions, int rows, int heads, int width,
                               int dims, const float* freqs, int dtype, void* stream) {
  if (rows <= 0 || heads <= 0 || width <= 0) return CBIS_OK;
  if (dims < 0 || dims > width || dims % 2 || (dims > 0 && !freqs)) return CBIS_ERR_BAD_SIZE;
  const int units = heads * (dims / 2 + width - dims);
  const int threads = units >= 256 ? 256 : (units >= 128 ? 128 : 64);
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == CBIS_F32)
    return (int)launch_pdl(rope_rows_kernel<float>, dim3(rows), dim3(threads), 0, st, (const float*)src, src_ld, src_col0,
                           src_head_stride, (float*)dst, dst_ld, dst_col0, dst_head_stride, positions, heads, width, dims,
                           freqs);
  if (dtype == CBIS_BF16)
    return (int)launch_pdl(rope_rows_kernel<__nv_bfloat16>, dim3(rows), dim3(threads), 0, st, (const __nv_bfloat16*)src,
                           src_ld, src_col0, src_head_stride, (__nv_bfloat16*)dst, dst_ld, dst_col0, dst_head_stride,
                           positions, heads, width, dims, freqs);
  return CBIS_ERR_BAD_DTYPE;
}

// gate_dtype: the gate's numbers may be 32-bit beside values of the compute type.
CBIS_EXPORT int cbis_head_gate_mul(const void* x, int x_ld, const void* gate, int gate_ld, int gate_dtype, void* out,
                                   int out_ld, int rows, int heads, int width, int dtype, void* stream) {
  if (rows <= 0 || heads <= 0 || width <= 0) return CBIS_OK;
  const size_t total = (size_t)rows * heads * width;
  size_t blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  cudaStream_t st = (cudaStream_t)stream;
#define CBIS_HG(TT, TG)                                                                                            \
  return (int)launch_pdl(head_gate_mul_kernel<TT, TG>, dim3((int)blocks), dim3(256), 0, st, (const TT*)x, x_ld,    \
                         (const TG*)gate, gate_ld, (TT*)out, out_ld, rows, heads, width)
  if (dtype == CBIS_F32 && gate_dtype == CBIS_F32) CBIS_HG(float, float);
  if (dtype == CBIS_BF16 && gate_dtype == CBIS_BF16) CBIS_HG(__nv_bfloat16, __nv_bfloat16);
  if (dtype == CBIS_BF16 && gate_dtype == CBIS_F32) CBIS_HG(__nv_bfloat16, float);
#undef CBIS_HG
  return CBIS_ERR_BAD_DTYPE;
}

// Elementwise pieces: the Dynamic Tanh norm, rotary positions on interleaved pairs, and a
// scalar multiple of a float32 tensor.
//
//   dyt:     y = tanh(alpha * x) * w + b      (no statistic of the row enters)
//   rotary:  the pair (v[2i], v[2i+1]) of the first `dims` entries of a vector at position p
//            turns by the angle p * f_i:  (u c - v s, v c + u s),  f_i = base^(-2i/dims).
//            The table f (dims/2 floats) comes from the host, formed in double.  The angle is
//            formed in double and reduced there, so that its error does not grow with p.
#include "common.cuh"
#include "rotary.cuh"

namespace hs {

template <typename TO>
__global__ void dyt_kernel(TO* __restrict__ out, const float* __restrict__ x,
                           const float* __restrict__ w, const float* __restrict__ b,
                           const int* __restrict__ rows, int width, float alpha) {
  const int o = blockIdx.x;
  const int src = rows ? rows[o] : o;
  const float* xr = x + (size_t)src * width;
  TO* orow = out + (size_t)o * width;
  for (int e = threadIdx.x; e < width; e += blockDim.x)
    orow[e] = from_f<TO>(tanhf(alpha * xr[e]) * w[e] + b[e]);
}

__global__ void scale_kernel(float* __restrict__ t, long long n, float s) {
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long step = (long long)gridDim.x * blockDim.x;
  for (; i < n; i += step) t[i] = t[i] * s;
}

// One block per token row; `n_vec` vectors at columns offset + v * vec_stride.
__global__ void rotary_kernel(float* __restrict__ buf, const int* __restrict__ tok_pos,
                              const int* __restrict__ tok_req, const float* __restrict__ freq,
                              int row_stride, int n_vec, int vec_stride, int offset, int dims) {
  const int t = blockIdx.x;
  if (tok_req[t] < 0) return;
  const int p = tok_pos[t];
  const int half = dims / 2;
  float* row = buf + (size_t)t * row_stride + offset;
  for (int i = threadIdx.x; i < n_vec * half; i += blockDim.x) {
    const int v = i / half, j = i - v * half;
    float c, s;
    pair_angle(p, freq[j], &c, &s);
    float* e = row + (size_t)v * vec_stride + 2 * j;
    const float a = e[0], b = e[1];
    e[0] = a * c - b * s;
    e[1] = b * c + a * s;
  }
}

}  // namespace hs

HS_EXPORT int hs_dyt_norm(void* out, const float* x, const float* w, const float* b,
                          const int* rows, int n_rows, int width, float alpha, int out_dtype,
                          void* stream) {
  if (!out || !x || !w || !b) return HS_ERR_ARGUMENT;
  if (n_rows <= 0) return HS_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const int threads = width >= 1024 ? 256 : 128;
  if (out_dtype == HS_DT_F32)
    hs::dyt_kernel<float><<<n_rows, threads, 0, st>>>((float*)out, x, w, b, rows, width, alpha);
  else if (out_dtype == HS_DT_BF16)
    hs::dyt_kernel<__nv_bfloat16><<<n_rows, threads, 0, st>>>((__nv_bfloat16*)out, x, w, b, rows,
                                                             width, alpha);
  else
    return HS_ERR_UNSUPPORTED;
  HS_LAUNCH_CHECK();
  return HS_OK;
}

HS_EXPORT int hs_scale(float* t, long long n, float s, void* stream) {
  if (!t) return HS_ERR_ARGUMENT;
  if (n <= 0) return HS_OK;
  long long blocks = (n + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  hs::scale_kernel<<<(int)blocks, 256, 0, (cudaStream_t)stream>>>(t, n, s);
  HS_LAUNCH_CHECK();
  return HS_OK;
}

HS_EXPORT int hs_rotary_pairs(float* buf, const int* tok_pos, const int* tok_req,
                              const float* freq, int n_tokens, int row_stride, int n_vec,
                              int vec_stride, int offset, int dims, void* stream) {
  if (!buf || !tok_pos || !tok_req || !freq) return HS_ERR_ARGUMENT;
  if (dims < 0 || dims % 2 || n_vec < 0) return HS_ERR_UNSUPPORTED;
  if (n_tokens <= 0 || dims == 0 || n_vec == 0) return HS_OK;
  hs::rotary_kernel<<<n_tokens, 128, 0, (cudaStream_t)stream>>>(buf, tok_pos, tok_req, freq,
                                                                 row_stride, n_vec, vec_stride,
                                                                 offset, dims);
  HS_LAUNCH_CHECK();
  return HS_OK;
}

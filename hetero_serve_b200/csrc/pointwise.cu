// Elementwise pieces: the Dynamic Tanh norm, rotary positions on interleaved pairs, and a
// scalar multiple of a float32 tensor.
//
//   dyt:     y = tanh(alpha * x) * w + b      (no statistic of the row enters)
//   rotary:  the pair (v[2i], v[2i+1]) of the first `dims` entries of a vector at position p
//            turns by the angle p * f_i:  (u c - v s, v c + u s),  f_i = base^(-2i/dims).
//            The table f (dims/2 floats) comes from the host, formed in double.  The angle is
//            formed in double and reduced there, so that its error does not grow with p.
//   gated:   out[t, f] = act(gu[t, f]) * gu[t, ff + f] * s_t  with  s_t = sigmoid(h[t] . w_s)
//            (one number per token; 1 without w_s): the middle of a gated feed-forward whose
//            gate and up projections came as one product [gate | up].
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

template <typename T>
__global__ void __launch_bounds__(256)
gated_act_kernel(T* __restrict__ out, const T* __restrict__ gu, const T* __restrict__ h,
                 const T* __restrict__ w_s, const int* __restrict__ tok_req, int ff, int width,
                 int act) {
  __shared__ float s_part[8];
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  if (tok_req && tok_req[t] < 0) return;
  float scale = 1.0f;
  if (w_s) {
    float dot = 0.f;
    for (int k = threadIdx.x; k < width; k += 256)
      dot = fmaf(to_f(h[(size_t)t * width + k]), to_f(w_s[k]), dot);
    dot = warp_sum(dot);
    if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = dot;
    __syncthreads();
    float z = 0.f;
    for (int i = 0; i < 8; ++i) z += s_part[i];
    scale = 1.0f / (1.0f + expf(-z));
  }
  const T* row = gu + (size_t)t * 2 * ff;
  for (int f = threadIdx.x; f < ff; f += 256)
    out[(size_t)t * ff + f] = from_f<T>(apply_act(to_f(row[f]), act) * to_f(row[ff + f]) * scale);
}

}  // namespace hs

HS_EXPORT int hs_gated_act(void* out, const void* gu, const void* h, const void* w_s,
                           const int* tok_req, int n_tokens, int ff, int width, int act,
                           int dtype, void* stream) {
  if (!out || !gu || (w_s && !h)) return HS_ERR_ARGUMENT;
  if (ff <= 0 || act < HS_ACT_NONE || act > HS_ACT_LAST) return HS_ERR_UNSUPPORTED;
  if (n_tokens <= 0) return HS_OK;
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t e = cudaSuccess;
  if (dtype == HS_DT_F32)
    e = hs_launch(hs::gated_act_kernel<float>, dim3(n_tokens), dim3(256), 0, st, hs_pdl_enabled(),
                  (float*)out, (const float*)gu, (const float*)h, (const float*)w_s, tok_req, ff,
                  width, act);
  else if (dtype == HS_DT_BF16)
    e = hs_launch(hs::gated_act_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(256), 0, st,
                  hs_pdl_enabled(), (__nv_bfloat16*)out, (const __nv_bfloat16*)gu,
                  (const __nv_bfloat16*)h, (const __nv_bfloat16*)w_s, tok_req, ff, width, act);
  else
    return HS_ERR_UNSUPPORTED;
  return e == cudaSuccess ? HS_OK : (int)e;
}

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

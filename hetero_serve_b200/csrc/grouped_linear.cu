// Block-diagonal linear on the CUDA cores, float32 accumulation:
//
//   out[t, g * n + j] = sum_k a[t, a_off + g * a_gstride + k] * w[g][k][j]
//
// `a` is float32 with row stride a_stride, so a group's input may be a slice of a wider row
// (the unrotated part of one head's query, say); the weights are held k-major ([groups, k, n],
// transposed once at binding) so that a warp's loads of one k are contiguous.  A block covers TT
// tokens x 32 output columns; its four warps each sum a quarter of k for every column, and the
// quarters are added in a fixed order, so a row's result depends on nothing else in the batch.
#include "common.cuh"

namespace hs {

constexpr int GL_TT = 8;          // tokens a block covers
constexpr int GL_THREADS = 128;   // four warps: each takes a quarter of the summed index
constexpr int GL_COLS = 32;       // output columns a block covers (one a lane)

template <typename TW, typename TO>
__global__ void __launch_bounds__(GL_THREADS)
grouped_linear_kernel(TO* __restrict__ out, const float* __restrict__ a,
                      const TW* __restrict__ w, int n_tokens, int a_stride, int a_off,
                      int a_gstride, int groups, int n, int k) {
  extern __shared__ float s_a[];                    // [GL_TT][k]
  __shared__ float s_part[GL_THREADS / 32][GL_TT][GL_COLS];
  const int t0 = blockIdx.x * GL_TT;
  const int g = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int j = blockIdx.z * GL_COLS + lane;
  const int nt = min(GL_TT, n_tokens - t0);
  for (int i = threadIdx.x; i < GL_TT * k; i += GL_THREADS) {
    const int tt = i / k, kk = i - tt * k;
    s_a[i] = tt < nt ? a[(size_t)(t0 + tt) * a_stride + a_off + (size_t)g * a_gstride + kk] : 0.f;
  }
  __syncthreads();
  float acc[GL_TT];
#pragma unroll
  for (int tt = 0; tt < GL_TT; ++tt) acc[tt] = 0.f;
  const int per = (k + 3) / 4;
  const int k_lo = warp * per, k_hi = min(k, k_lo + per);
  if (j < n) {
    const TW* wg = w + (size_t)g * k * n + j;
#pragma unroll 8
    for (int kk = k_lo; kk < k_hi; ++kk) {
      const float wv = to_f(wg[(size_t)kk * n]);
#pragma unroll
      for (int tt = 0; tt < GL_TT; ++tt) acc[tt] = fmaf(s_a[tt * k + kk], wv, acc[tt]);
    }
  }
#pragma unroll
  for (int tt = 0; tt < GL_TT; ++tt) s_part[warp][tt][lane] = acc[tt];
  __syncthreads();
  // the four quarters are added in a fixed order: a row's sum never depends on the batch
  for (int i = threadIdx.x; i < GL_TT * GL_COLS; i += GL_THREADS) {
    const int tt = i / GL_COLS, c = i - tt * GL_COLS;
    const int col = blockIdx.z * GL_COLS + c;
    if (tt < nt && col < n) {
      const float v = ((s_part[0][tt][c] + s_part[1][tt][c]) + s_part[2][tt][c]) + s_part[3][tt][c];
      out[(size_t)(t0 + tt) * groups * n + (size_t)g * n + col] = from_f<TO>(v);
    }
  }
}

}  // namespace hs

HS_EXPORT int hs_grouped_linear(void* out, const float* a, const void* w, int n_tokens,
                                int a_stride, int a_off, int a_gstride, int groups, int n, int k,
                                int w_dtype, int out_dtype, void* stream) {
  if (!out || !a || !w) return HS_ERR_ARGUMENT;
  if (groups <= 0 || n <= 0 || k <= 0) return HS_ERR_UNSUPPORTED;
  if (n_tokens <= 0) return HS_OK;
  const size_t smem = (size_t)hs::GL_TT * k * sizeof(float);
  if (smem > 200 * 1024) return HS_ERR_UNSUPPORTED;
  dim3 grid((n_tokens + hs::GL_TT - 1) / hs::GL_TT, groups, (n + hs::GL_COLS - 1) / hs::GL_COLS);
  cudaStream_t st = (cudaStream_t)stream;
#define HS_GL(TW, TO)                                                                         \
  do {                                                                                        \
    auto kern = hs::grouped_linear_kernel<TW, TO>;                                            \
    if (smem > 48 * 1024)                                                                     \
      cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);     \
    kern<<<grid, hs::GL_THREADS, smem, st>>>((TO*)out, a, (const TW*)w, n_tokens, a_stride,  \
                                             a_off, a_gstride, groups, n, k);                 \
  } while (0)
  if (w_dtype == HS_DT_F32 && out_dtype == HS_DT_F32) HS_GL(float, float);
  else if (w_dtype == HS_DT_BF16 && out_dtype == HS_DT_F32) HS_GL(__nv_bfloat16, float);
  else if (w_dtype == HS_DT_BF16 && out_dtype == HS_DT_BF16) HS_GL(__nv_bfloat16, __nv_bfloat16);
  else return HS_ERR_UNSUPPORTED;
#undef HS_GL
  HS_LAUNCH_CHECK();
  return HS_OK;
}

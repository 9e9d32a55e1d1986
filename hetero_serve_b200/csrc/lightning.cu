// Linear attention with a constant decay per head (lightning attention), as a recurrence on a
// float32 state S [dim, vdim] per head and request:
//
//     q, k, v = act(projection columns)        act = silu, applied here in float32
//     S <- decay_h * S + k v^T ;   o = S^T q    token after token
//
// The state lives in the request's state slot ([heads, dim, vdim] floats) and is carried from
// step to step.  One block per (request, head, group of value columns): a thread keeps 16 rows
// of one column of S in registers, the P = ceil(dim / 16) (rounded up to a power of two) parts
// of a column are neighbouring lanes of one warp and fold their shares of o by a butterfly.
// The tokens' rows are staged through shared memory 16 tokens at a time.  A token's arithmetic
// is the same chain whatever the batch or the cut of the prompt: results are bit-equal across
// both.
#include "common.cuh"

namespace hs {

constexpr int LA_THREADS = 128;
constexpr int LA_ROWS = 16;          // state rows a thread keeps
constexpr int LA_TOK = 16;           // tokens staged at a time

__device__ __forceinline__ float la_act(float z, int act) {
  return act == HS_ACT_SILU ? z / (1.0f + expf(-z)) : z;
}

__global__ void __launch_bounds__(LA_THREADS)
lightning_kernel(float* __restrict__ o, float* __restrict__ state, const float* __restrict__ proj,
                 const float* __restrict__ decay, const int* __restrict__ req_start,
                 const int* __restrict__ req_len, const int* __restrict__ req_slot, int stride,
                 int q_off, int k_off, int v_off, int H, int D, int V, int P, int act) {
  extern __shared__ __align__(16) float smem[];
  const int Dp = P * LA_ROWS;                       // dim padded to whole parts
  const int cols = LA_THREADS / P;                  // value columns of this block
  float* s_q = smem;                                // [LA_TOK][Dp]
  float* s_k = s_q + LA_TOK * Dp;                   // [LA_TOK][Dp]
  float* s_v = s_k + LA_TOK * Dp;                   // [LA_TOK][cols]
  const int r = blockIdx.z, h = blockIdx.y;
  const int n = req_len[r];
  if (n <= 0) return;
  const int t0 = req_start[r];
  const int slot = req_slot[r];
  const int part = threadIdx.x % P, col = threadIdx.x / P;
  const int v = blockIdx.x * cols + col;
  const bool col_ok = v < V;
  const float dh = decay[h];
  float* S = state + ((size_t)slot * H + h) * D * V;
  float s[LA_ROWS];
#pragma unroll
  for (int i = 0; i < LA_ROWS; ++i) {
    const int d = part * LA_ROWS + i;
    s[i] = (col_ok && d < D) ? S[(size_t)d * V + v] : 0.f;
  }
  for (int base = 0; base < n; base += LA_TOK) {
    const int here = min(LA_TOK, n - base);
    __syncthreads();                                // the portion before has been walked
    for (int e = threadIdx.x; e < here * Dp; e += LA_THREADS) {
      const int tt = e / Dp, d = e - tt * Dp;
      const float* row = proj + (size_t)(t0 + base + tt) * stride + (size_t)h * D;
      s_q[e] = d < D ? la_act(row[q_off + d], act) : 0.f;
      s_k[e] = d < D ? la_act(row[k_off + d], act) : 0.f;
    }
    for (int e = threadIdx.x; e < here * cols; e += LA_THREADS) {
      const int tt = e / cols, c = e - tt * cols;
      const int vv = blockIdx.x * cols + c;
      s_v[e] = vv < V ? la_act(proj[(size_t)(t0 + base + tt) * stride + v_off + (size_t)h * V + vv], act)
                      : 0.f;
    }
    __syncthreads();
    for (int tt = 0; tt < here; ++tt) {
      const float vt = s_v[tt * cols + col];
      const float4* kq = (const float4*)(s_k + tt * Dp + part * LA_ROWS);
      const float4* qq = (const float4*)(s_q + tt * Dp + part * LA_ROWS);
      float acc = 0.f;
#pragma unroll
      for (int i4 = 0; i4 < LA_ROWS / 4; ++i4) {
        const float4 k4 = kq[i4], q4 = qq[i4];
        float* si = s + 4 * i4;
        si[0] = fmaf(k4.x, vt, dh * si[0]); acc = fmaf(si[0], q4.x, acc);
        si[1] = fmaf(k4.y, vt, dh * si[1]); acc = fmaf(si[1], q4.y, acc);
        si[2] = fmaf(k4.z, vt, dh * si[2]); acc = fmaf(si[2], q4.z, acc);
        si[3] = fmaf(k4.w, vt, dh * si[3]); acc = fmaf(si[3], q4.w, acc);
      }
      for (int off = 1; off < P; off <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
      if (part == 0 && col_ok) o[(size_t)(t0 + base + tt) * H * V + (size_t)h * V + v] = acc;
    }
  }
#pragma unroll
  for (int i = 0; i < LA_ROWS; ++i) {
    const int d = part * LA_ROWS + i;
    if (col_ok && d < D) S[(size_t)d * V + v] = s[i];
  }
}

}  // namespace hs

// proj: float32 rows of `stride` columns holding q (H*D at q_off), k (H*D at k_off) and v (H*V at
// v_off), head by head; o: float32 [tokens, H*V]; state: [slots, H*D*V] float32.
HS_EXPORT int hs_lightning_recurrence(float* o, float* state, const float* proj,
                                      const float* decay, const int* req_start,
                                      const int* req_len, const int* req_slot, int n_requests,
                                      int stride, int q_off, int k_off, int v_off, int H, int D,
                                      int V, int act, void* stream) {
  if (!o || !state || !proj || !decay || !req_start || !req_len || !req_slot)
    return HS_ERR_ARGUMENT;
  if (H <= 0 || D <= 0 || V <= 0 || D > 16 * hs::LA_ROWS || (act != HS_ACT_NONE && act != HS_ACT_SILU))
    return HS_ERR_UNSUPPORTED;
  if (n_requests <= 0) return HS_OK;
  int P = 1;
  while (P * hs::LA_ROWS < D) P *= 2;
  const int cols = hs::LA_THREADS / P;
  const size_t smem = (size_t)hs::LA_TOK * (2 * P * hs::LA_ROWS + cols) * sizeof(float);
  dim3 grid((V + cols - 1) / cols, H, n_requests);
  hs::lightning_kernel<<<grid, hs::LA_THREADS, smem, (cudaStream_t)stream>>>(
      o, state, proj, decay, req_start, req_len, req_slot, stride, q_off, k_off, v_off, H, D, V,
      P, act);
  HS_LAUNCH_CHECK();
  return HS_OK;
}

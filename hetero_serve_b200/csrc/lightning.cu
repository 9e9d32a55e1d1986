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
// The tokens' rows are staged through shared memory 16 tokens at a time, two buffers in turn:
// for steps of many tokens the activations are applied by a pass of their own into compact rows
// and the recurrence fetches the next portion by cp.async while it walks the current one.  A
// token's arithmetic is the same chain whatever the batch or the cut of the prompt: results are
// bit-equal across both.
#include "common.cuh"

namespace hs {

constexpr int LA_THREADS = 128;
constexpr int LA_ROWS = 16;          // state rows a thread keeps
constexpr int LA_TOK = 16;           // tokens staged at a time (8 when dim is above 128)

__device__ __forceinline__ float la_act(float z, int act) {
  return act == HS_ACT_SILU ? z / (1.0f + expf(-z)) : z;
}
__device__ __forceinline__ void la_cp16(void* smem_dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(src)
               : "memory");
}

// dst[t, :] = act(q | k | v columns of proj[t]) as one compact row of 2 H D + H V floats
__global__ void lightning_act_kernel(float* __restrict__ dst, const float* __restrict__ proj,
                                     int n_tokens, int stride, int q_off, int k_off, int v_off,
                                     int hd, int hv, int act) {
  const int row_len = 2 * hd + hv;
  const long long total = (long long)n_tokens * row_len;
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total;
       e += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(e / row_len), c = (int)(e - (long long)t * row_len);
    const int src = c < hd ? q_off + c : (c < 2 * hd ? k_off + c - hd : v_off + c - 2 * hd);
    dst[e] = la_act(proj[(size_t)t * stride + src], act);
  }
}

// A portion of up to ntok tokens of request rows (from token `tok` on) into one buffer (q [ntok][Dp],
// k [ntok][Dp], v [ntok][cols]).  `bulk`: the rows are activated already and 16-byte aligned,
// and go in by cp.async (the walk over the portion before runs meanwhile); otherwise plain loads
// with the activation applied on the way.
__device__ __forceinline__ void la_stage(float* s_q, const float* __restrict__ proj, int tok,
                                         int here, int stride, int q_off, int k_off, int v_off,
                                         int h, int D, int V, int Dp, int cols, int v0, int ntok,
                                         int act, int bulk) {
  float* s_k = s_q + ntok * Dp;
  float* s_v = s_k + ntok * Dp;
  if (bulk) {
    const int dq = D / 4, cq = cols / 4;
    for (int e = threadIdx.x; e < here * dq; e += LA_THREADS) {
      const int tt = e / dq, c = e - tt * dq;
      const float* row = proj + (size_t)(tok + tt) * stride + (size_t)h * D + 4 * c;
      la_cp16(s_q + tt * Dp + 4 * c, row + q_off);
      la_cp16(s_k + tt * Dp + 4 * c, row + k_off);
    }
    for (int e = threadIdx.x; e < here * cq; e += LA_THREADS) {
      const int tt = e / cq, c = e - tt * cq;
      if (v0 + 4 * c < V)
        la_cp16(s_v + tt * cols + 4 * c,
                proj + (size_t)(tok + tt) * stride + v_off + (size_t)h * V + v0 + 4 * c);
    }
  } else {
#pragma unroll 4
    for (int e = threadIdx.x; e < here * D; e += LA_THREADS) {
      const int tt = e / D, d = e - tt * D;
      const float* row = proj + (size_t)(tok + tt) * stride + (size_t)h * D;
      s_q[tt * Dp + d] = la_act(row[q_off + d], act);
      s_k[tt * Dp + d] = la_act(row[k_off + d], act);
    }
    for (int e = threadIdx.x; e < here * cols; e += LA_THREADS) {
      const int tt = e / cols, c = e - tt * cols;
      if (v0 + c < V)
        s_v[e] = la_act(proj[(size_t)(tok + tt) * stride + v_off + (size_t)h * V + v0 + c], act);
    }
  }
  asm volatile("cp.async.commit_group;" ::: "memory");
}

__global__ void __launch_bounds__(LA_THREADS)
lightning_kernel(float* __restrict__ o, float* __restrict__ state, const float* __restrict__ proj,
                 const float* __restrict__ decay, const int* __restrict__ req_start,
                 const int* __restrict__ req_len, const int* __restrict__ req_slot, int stride,
                 int q_off, int k_off, int v_off, int H, int D, int V, int P, int act, int ntok,
                 int bulk) {
  extern __shared__ __align__(16) float smem[];
  const int Dp = P * LA_ROWS;                       // dim padded to whole parts
  const int cols = LA_THREADS / P;                  // value columns of this block
  const int per_buf = ntok * (2 * Dp + cols);       // a buffer: q [ntok][Dp], k [ntok][Dp], v [ntok][cols]
  const int r = blockIdx.z, h = blockIdx.y;
  const int n = req_len[r];
  if (n <= 0) return;
  const int t0 = req_start[r];
  const int slot = req_slot[r];
  const int part = threadIdx.x % P, col = threadIdx.x / P;
  const int v0 = blockIdx.x * cols;
  const int v = v0 + col;
  const bool col_ok = v < V;
  const float dh = decay[h];
  float* S = state + ((size_t)slot * H + h) * D * V;
  float s[LA_ROWS];
#pragma unroll
  for (int i = 0; i < LA_ROWS; ++i) {
    const int d = part * LA_ROWS + i;
    s[i] = (col_ok && d < D) ? S[(size_t)d * V + v] : 0.f;
  }
  for (int e = threadIdx.x; e < 2 * per_buf; e += LA_THREADS) smem[e] = 0.f;   // the padding stays zero
  __syncthreads();
  la_stage(smem, proj, t0, min(ntok, n), stride, q_off, k_off, v_off, h, D, V, Dp, cols, v0, ntok,
           act, bulk);
  int buf = 0;
  for (int base = 0; base < n; base += ntok, buf ^= 1) {
    const int here = min(ntok, n - base);
    if (base + ntok < n) {
      la_stage(smem + (buf ^ 1) * per_buf, proj, t0 + base + ntok, min(ntok, n - base - ntok), stride,
               q_off, k_off, v_off, h, D, V, Dp, cols, v0, ntok, act, bulk);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    const float* s_q = smem + buf * per_buf;
    const float* s_k = s_q + ntok * Dp;
    const float* s_v = s_k + ntok * Dp;
    for (int tt = 0; tt < here; ++tt) {
      const float vt = s_v[tt * cols + col];
      const float4* kq = (const float4*)(s_k + tt * Dp + part * LA_ROWS);
      const float4* qq = (const float4*)(s_q + tt * Dp + part * LA_ROWS);
      float acc = 0.f;
#pragma unroll
      for (int i4 = 0; i4 < LA_ROWS / 4; ++i4) {
        const float4 k4 = kq[i4], q4 = qq[i4];
        s[4 * i4 + 0] = fmaf(k4.x, vt, dh * s[4 * i4 + 0]); acc = fmaf(s[4 * i4 + 0], q4.x, acc);
        s[4 * i4 + 1] = fmaf(k4.y, vt, dh * s[4 * i4 + 1]); acc = fmaf(s[4 * i4 + 1], q4.y, acc);
        s[4 * i4 + 2] = fmaf(k4.z, vt, dh * s[4 * i4 + 2]); acc = fmaf(s[4 * i4 + 2], q4.z, acc);
        s[4 * i4 + 3] = fmaf(k4.w, vt, dh * s[4 * i4 + 3]); acc = fmaf(s[4 * i4 + 3], q4.w, acc);
      }
      for (int off = 1; off < P; off <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
      if (part == 0 && col_ok) o[(size_t)(t0 + base + tt) * H * V + (size_t)h * V + v] = acc;
    }
    __syncthreads();                                // this buffer is staged into again next turn
  }
#pragma unroll
  for (int i = 0; i < LA_ROWS; ++i) {
    const int d = part * LA_ROWS + i;
    if (col_ok && d < D) S[(size_t)d * V + v] = s[i];
  }
}

}  // namespace hs

// proj: float32 rows of `stride` columns holding q (H*D at q_off), k (H*D at k_off) and v (H*V at
// v_off), head by head; o: float32 [tokens, H*V]; state: [slots, H*D*V] float32.  `scratch`
// (n_tokens * (2 H D + H V) floats, or null): with it the activations are applied in a pass of
// their own and the recurrence streams the activated rows; the results are the same bits.
HS_EXPORT int hs_lightning_recurrence(float* o, float* state, const float* proj,
                                      const float* decay, const int* req_start,
                                      const int* req_len, const int* req_slot, int n_requests,
                                      int n_tokens, int stride, int q_off, int k_off, int v_off,
                                      int H, int D, int V, int act, float* scratch,
                                      void* stream) {
  if (!o || !state || !proj || !decay || !req_start || !req_len || !req_slot)
    return HS_ERR_ARGUMENT;
  if (H <= 0 || D <= 0 || V <= 0 || D > 16 * hs::LA_ROWS || (act != HS_ACT_NONE && act != HS_ACT_SILU))
    return HS_ERR_UNSUPPORTED;
  if (n_requests <= 0 || n_tokens <= 0) return HS_OK;
  cudaStream_t st = (cudaStream_t)stream;
  int P = 1;
  while (P * hs::LA_ROWS < D) P *= 2;
  const int cols = hs::LA_THREADS / P;
  const int ntok = P * hs::LA_ROWS > 128 ? hs::LA_TOK / 2 : hs::LA_TOK;
  int bulk = 0;
  if (scratch && D % 4 == 0 && V % 4 == 0 && (((uintptr_t)scratch) & 15) == 0) {
    const int hd = H * D, hv = H * V;
    const long long total = (long long)n_tokens * (2 * hd + hv);
    long long blocks = (total + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    hs::lightning_act_kernel<<<(int)blocks, 256, 0, st>>>(scratch, proj, n_tokens, stride, q_off,
                                                         k_off, v_off, hd, hv, act);
    HS_LAUNCH_CHECK();
    proj = scratch;
    stride = 2 * hd + hv;
    q_off = 0; k_off = hd; v_off = 2 * hd;
    act = HS_ACT_NONE;
    bulk = 1;
  }
  const size_t smem = (size_t)2 * ntok * (2 * P * hs::LA_ROWS + cols) * sizeof(float);
  dim3 grid((V + cols - 1) / cols, H, n_requests);
  hs::lightning_kernel<<<grid, hs::LA_THREADS, smem, st>>>(
      o, state, proj, decay, req_start, req_len, req_slot, stride, q_off, k_off, v_off, H, D, V,
      P, act, ntok, bulk);
  HS_LAUNCH_CHECK();
  return HS_OK;
}

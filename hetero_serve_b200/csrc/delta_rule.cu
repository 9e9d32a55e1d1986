// Gated delta rule with one decay per head and key channel, as a recurrent mixer.
//
// A token's row of the fused input projection holds  [q | k | v | b | a | g]:
//   q, k: kv_heads x D     v: heads x V     b: heads     a: ra numbers     g: rg numbers.
// Four kernels:
//   prepare    per token: causal short convolution over time (taps weights per channel, the
//              last one on the current token; inputs before a portion's start come from the
//              request's state) and silu on q, k, v; q and k to unit length per head
//              (x / sqrt(sum x^2 + 1e-6)), q also times D^-1/2; beta = sigmoid(b);
//              decay = exp(-exp(A_log[h]) * softplus(W_a2 a + dt_bias))   [heads x D]
//   conv state per request: keeps the last taps-1 inputs of q, k, v
//   recurrence per request and head, token after token on the float32 state S [D x V]:
//                 S <- decay * S (row-wise);  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
//   finish     per token and head: o / sqrt(mean(o^2) + eps) * w * sigmoid(W_g2 g)
// Everything here is float32 whatever the model's matrix type is.  The two small matrices W_a2
// and W_g2 are held with the summed index slowest ([ra, heads x D] and [rg, heads x V]) so that
// neighbouring threads read neighbouring weights.
//
// State of a slot: [heads x D x V | (taps-1) x channels] floats.
#include "common.cuh"

namespace hs {

__device__ __forceinline__ float sigmoidf_(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplusf_(float z) { return z > 20.f ? z : log1pf(expf(z)); }

struct DeltaShape {
  int heads, kv_heads, D, V, taps, ra, rg;
  int stride;                    // floats in a projection row
  int b_off, a_off, g_off;       // columns of b, a, g (q, k, v start at 0)
  int state_stride;              // floats in a slot
};

__device__ __forceinline__ int channels(const DeltaShape& s) {
  return 2 * s.kv_heads * s.D + s.heads * s.V;
}

__global__ void __launch_bounds__(256)
delta_prepare_kernel(float* __restrict__ qn, float* __restrict__ kn, float* __restrict__ vv,
                     float* __restrict__ beta, float* __restrict__ decay,
                     const float* __restrict__ proj, const float* __restrict__ conv_w,
                     const float* __restrict__ a2, const float* __restrict__ dt_bias,
                     const float* __restrict__ A_log, const float* __restrict__ state,
                     const int* __restrict__ tok_req, const int* __restrict__ req_start,
                     const int* __restrict__ req_slot, DeltaShape s) {
  extern __shared__ float s_c[];                 // [channels] after convolution and silu
  const int t = blockIdx.x;
  const int r = tok_req[t];
  if (r < 0) return;
  const int C = channels(s);
  const int first = req_start[r];
  const int l = t - first;
  const float* cst = state + (size_t)req_slot[r] * s.state_stride + (size_t)s.heads * s.D * s.V;
  const int hist = s.taps - 1;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    float acc = 0.f;
    for (int j = 0; j < s.taps; ++j) {
      const int local = l - (hist - j);
      const float in = local >= 0 ? proj[(size_t)(first + local) * s.stride + c]
                                  : cst[(size_t)(local + hist) * C + c];
      acc = fmaf(conv_w[(size_t)c * s.taps + j], in, acc);
    }
    s_c[c] = acc * sigmoidf_(acc);
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const int QK = s.kv_heads * s.D;
  for (int vec = warp; vec < 2 * s.kv_heads; vec += nw) {       // q heads, then k heads
    const float* src = s_c + (size_t)vec * s.D;
    float ss = 0.f;
    for (int d = lane; d < s.D; d += 32) ss = fmaf(src[d], src[d], ss);
    ss = warp_sum(ss);
    float inv = 1.0f / sqrtf(ss + 1e-6f);
    const bool is_q = vec < s.kv_heads;
    if (is_q) inv *= 1.0f / sqrtf((float)s.D);
    float* dst = is_q ? qn + (size_t)t * QK + (size_t)vec * s.D
                      : kn + (size_t)t * QK + (size_t)(vec - s.kv_heads) * s.D;
    for (int d = lane; d < s.D; d += 32) dst[d] = src[d] * inv;
  }
  const int HV = s.heads * s.V;
  for (int i = threadIdx.x; i < HV; i += blockDim.x) vv[(size_t)t * HV + i] = s_c[2 * QK + i];
  const float* row = proj + (size_t)t * s.stride;
  for (int h = threadIdx.x; h < s.heads; h += blockDim.x)
    beta[(size_t)t * s.heads + h] = sigmoidf_(row[s.b_off + h]);
  const int HD = s.heads * s.D;
  for (int i = threadIdx.x; i < HD; i += blockDim.x) {
    float z = 0.f;
    for (int k = 0; k < s.ra; ++k) z = fmaf(a2[(size_t)k * HD + i], row[s.a_off + k], z);
    z += dt_bias[i];
    decay[(size_t)t * HD + i] = expf(-expf(A_log[i / s.D]) * softplusf_(z));
  }
}

__global__ void delta_conv_state_kernel(float* __restrict__ state, const float* __restrict__ proj,
                                        const int* __restrict__ req_start,
                                        const int* __restrict__ req_len,
                                        const int* __restrict__ req_slot, DeltaShape s) {
  const int r = blockIdx.y;
  const int n = req_len[r];
  if (n <= 0) return;
  const int C = channels(s);
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int hist = s.taps - 1;
  float* cst = state + (size_t)req_slot[r] * s.state_stride + (size_t)s.heads * s.D * s.V;
  const int first = req_start[r];
  // slot i receives the input at local index n - hist + i; an index below zero is an older
  // input, found at n + i of the old state, which lies ahead of every slot written so far
  for (int i = 0; i < hist; ++i) {
    const int local = n - hist + i;
    cst[(size_t)i * C + c] = local >= 0 ? proj[(size_t)(first + local) * s.stride + c]
                                        : cst[(size_t)(n + i) * C + c];
  }
}

constexpr int DR_DP = 8;          // state rows a thread keeps
constexpr int DR_THREADS = 128;

// Thread (col, part) keeps rows part*DP .. part*DP+DP-1 of column col of S; the KS parts of a
// column are neighbouring lanes and sum their shares with a butterfly.  The tokens' q, k, decay
// rows (padded with zeros to KS*DP), v columns and betas come through shared memory a chunk of
// CH tokens at a time, so that the latency of fetching them is paid once a chunk, not once a
// token.
__global__ void __launch_bounds__(DR_THREADS)
delta_recurrence_kernel(float* __restrict__ o, float* __restrict__ state,
                        const float* __restrict__ qn, const float* __restrict__ kn,
                        const float* __restrict__ vv, const float* __restrict__ beta,
                        const float* __restrict__ decay, const int* __restrict__ req_start,
                        const int* __restrict__ req_len, const int* __restrict__ req_slot,
                        DeltaShape s, int KS, int CH) {
  extern __shared__ __align__(16) float sm[];
  const int r = blockIdx.x, h = blockIdx.y;
  const int n = req_len[r];
  if (n <= 0) return;
  const int Dp = KS * DR_DP;
  const int cols = DR_THREADS / KS;
  float* s_k = sm;
  float* s_q = s_k + CH * Dp;
  float* s_g = s_q + CH * Dp;
  float* s_v = s_g + CH * Dp;
  float* s_b = s_v + CH * cols;
  const int part = threadIdx.x % KS;
  const int lc = threadIdx.x / KS;
  const int col = blockIdx.z * cols + lc;
  const bool col_ok = col < s.V;
  const int kh = h / (s.heads / s.kv_heads);
  const int d0 = part * DR_DP;
  float* S = state + (size_t)req_slot[r] * s.state_stride + (size_t)h * s.D * s.V;
  float st[DR_DP];
#pragma unroll
  for (int i = 0; i < DR_DP; ++i)
    st[i] = (col_ok && d0 + i < s.D) ? S[(size_t)(d0 + i) * s.V + col] : 0.f;
  const int QK = s.kv_heads * s.D, HV = s.heads * s.V, HD = s.heads * s.D;
  const int first = req_start[r];
  for (int c0 = 0; c0 < n; c0 += CH) {
    const int nc = min(CH, n - c0);
    __syncthreads();                               // the chunk before has been used
    for (int i = threadIdx.x; i < nc * Dp; i += DR_THREADS) {
      const int tt = i / Dp, d = i - tt * Dp;
      const size_t row = first + c0 + tt;
      const bool ok = d < s.D;
      s_k[i] = ok ? kn[row * QK + kh * s.D + d] : 0.f;
      s_q[i] = ok ? qn[row * QK + kh * s.D + d] : 0.f;
      s_g[i] = ok ? decay[row * HD + h * s.D + d] : 0.f;
    }
    for (int i = threadIdx.x; i < nc * cols; i += DR_THREADS) {
      const int tt = i / cols, cc = i - tt * cols;
      const int cg = blockIdx.z * cols + cc;
      s_v[i] = cg < s.V ? vv[(size_t)(first + c0 + tt) * HV + h * s.V + cg] : 0.f;
    }
    if (threadIdx.x < nc) s_b[threadIdx.x] = beta[(size_t)(first + c0 + threadIdx.x) * s.heads + h];
    __syncthreads();
    for (int tt = 0; tt < nc; ++tt) {
      const float4* k4 = (const float4*)(s_k + tt * Dp + d0);
      const float4* q4 = (const float4*)(s_q + tt * Dp + d0);
      const float4* g4 = (const float4*)(s_g + tt * Dp + d0);
      float kk[DR_DP], qq[DR_DP], gg[DR_DP];
#pragma unroll
      for (int j = 0; j < DR_DP / 4; ++j) {
        const float4 a = k4[j], b = q4[j], c = g4[j];
        kk[4 * j] = a.x; kk[4 * j + 1] = a.y; kk[4 * j + 2] = a.z; kk[4 * j + 3] = a.w;
        qq[4 * j] = b.x; qq[4 * j + 1] = b.y; qq[4 * j + 2] = b.z; qq[4 * j + 3] = b.w;
        gg[4 * j] = c.x; gg[4 * j + 1] = c.y; gg[4 * j + 2] = c.z; gg[4 * j + 3] = c.w;
      }
      float dot = 0.f;
#pragma unroll
      for (int j = 0; j < DR_DP; ++j) {
        st[j] *= gg[j];
        dot = fmaf(st[j], kk[j], dot);
      }
      for (int off = 1; off < KS; off <<= 1) dot += __shfl_xor_sync(0xffffffffu, dot, off);
      const float u = s_b[tt] * (s_v[tt * cols + lc] - dot);
      float out = 0.f;
#pragma unroll
      for (int j = 0; j < DR_DP; ++j) {
        st[j] = fmaf(kk[j], u, st[j]);
        out = fmaf(st[j], qq[j], out);
      }
      for (int off = 1; off < KS; off <<= 1) out += __shfl_xor_sync(0xffffffffu, out, off);
      if (part == 0 && col_ok) o[(size_t)(first + c0 + tt) * HV + h * s.V + col] = out;
    }
  }
#pragma unroll
  for (int i = 0; i < DR_DP; ++i)
    if (col_ok && d0 + i < s.D) S[(size_t)(d0 + i) * s.V + col] = st[i];
}

template <typename TO>
__global__ void __launch_bounds__(256)
delta_finish_kernel(TO* __restrict__ out, const float* __restrict__ o,
                    const float* __restrict__ proj, const float* __restrict__ g2,
                    const float* __restrict__ norm_w, const int* __restrict__ tok_req,
                    float eps, DeltaShape s) {
  const int t = blockIdx.x;
  if (tok_req[t] < 0) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const int HV = s.heads * s.V;
  const float* gin = proj + (size_t)t * s.stride + s.g_off;
  for (int h = warp; h < s.heads; h += nw) {
    const float* src = o + (size_t)t * HV + (size_t)h * s.V;
    float ss = 0.f;
    for (int e = lane; e < s.V; e += 32) ss = fmaf(src[e], src[e], ss);
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)s.V + eps);
    for (int e = lane; e < s.V; e += 32) {
      const float* gcol = g2 + (size_t)h * s.V + e;
      float z = 0.f;
      for (int k = 0; k < s.rg; ++k) z = fmaf(gcol[(size_t)k * HV], gin[k], z);
      out[(size_t)t * HV + h * s.V + e] = from_f<TO>(src[e] * inv * norm_w[e] * sigmoidf_(z));
    }
  }
}

}  // namespace hs

static int delta_shape(hs::DeltaShape* s, int heads, int kv_heads, int D, int V, int taps, int ra,
                       int rg) {
  if (heads <= 0 || kv_heads <= 0 || heads % kv_heads || D <= 0 || V <= 0 || taps < 1 ||
      ra <= 0 || rg <= 0)
    return HS_ERR_UNSUPPORTED;
  s->heads = heads; s->kv_heads = kv_heads; s->D = D; s->V = V; s->taps = taps;
  s->ra = ra; s->rg = rg;
  const int C = 2 * kv_heads * D + heads * V;
  s->b_off = C;
  s->a_off = C + heads;
  s->g_off = C + heads + ra;
  s->stride = C + heads + ra + rg;
  s->state_stride = heads * D * V + (taps - 1) * C;
  return HS_OK;
}

HS_EXPORT int hs_delta_prepare(float* qn, float* kn, float* vv, float* beta, float* decay,
                               const float* proj, const float* conv_w, const float* a2,
                               const float* dt_bias, const float* A_log, float* state,
                               const int* tok_req, const int* req_start, const int* req_len,
                               const int* req_slot, int n_tokens, int n_requests, int heads,
                               int kv_heads, int D, int V, int taps, int ra, int rg,
                               void* stream) {
  if (!qn || !kn || !vv || !beta || !decay || !proj || !conv_w || !a2 || !dt_bias || !A_log ||
      !state || !tok_req || !req_start || !req_len || !req_slot)
    return HS_ERR_ARGUMENT;
  hs::DeltaShape s;
  int rc = delta_shape(&s, heads, kv_heads, D, V, taps, ra, rg);
  if (rc) return rc;
  if (n_tokens <= 0 || n_requests <= 0) return HS_OK;
  const int C = 2 * kv_heads * D + heads * V;
  const size_t smem = (size_t)C * sizeof(float);
  if (smem > 200 * 1024) return HS_ERR_UNSUPPORTED;
  cudaStream_t st = (cudaStream_t)stream;
  if (smem > 48 * 1024)
    cudaFuncSetAttribute(hs::delta_prepare_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         (int)smem);
  hs::delta_prepare_kernel<<<n_tokens, 256, smem, st>>>(qn, kn, vv, beta, decay, proj, conv_w, a2,
                                                        dt_bias, A_log, state, tok_req, req_start,
                                                        req_slot, s);
  HS_LAUNCH_CHECK();
  if (taps > 1) {
    dim3 grid((C + 127) / 128, n_requests);
    hs::delta_conv_state_kernel<<<grid, 128, 0, st>>>(state, proj, req_start, req_len, req_slot, s);
    HS_LAUNCH_CHECK();
  }
  return HS_OK;
}

HS_EXPORT int hs_delta_recurrence(float* o, float* state, const float* qn, const float* kn,
                                  const float* vv, const float* beta, const float* decay,
                                  const int* req_start, const int* req_len, const int* req_slot,
                                  int n_requests, int heads, int kv_heads, int D, int V, int taps,
                                  int ra, int rg, void* stream) {
  if (!o || !state || !qn || !kn || !vv || !beta || !decay || !req_start || !req_len || !req_slot)
    return HS_ERR_ARGUMENT;
  hs::DeltaShape s;
  int rc = delta_shape(&s, heads, kv_heads, D, V, taps, ra, rg);
  if (rc) return rc;
  if (D > hs::DR_DP * 32) return HS_ERR_UNSUPPORTED;
  if (n_requests <= 0) return HS_OK;
  int KS = 1;
  while (KS * hs::DR_DP < D) KS <<= 1;
  const int cols = hs::DR_THREADS / KS;
  const int CH = KS * hs::DR_DP <= 128 ? 16 : 8;
  const size_t smem = (size_t)(3 * CH * KS * hs::DR_DP + CH * cols + CH) * sizeof(float);
  dim3 grid(n_requests, heads, (V + cols - 1) / cols);
  hs::delta_recurrence_kernel<<<grid, hs::DR_THREADS, smem, (cudaStream_t)stream>>>(
      o, state, qn, kn, vv, beta, decay, req_start, req_len, req_slot, s, KS, CH);
  HS_LAUNCH_CHECK();
  return HS_OK;
}

HS_EXPORT int hs_delta_finish(void* out, const float* o, const float* proj, const float* g2,
                              const float* norm_w, const int* tok_req, int n_tokens, float eps,
                              int heads, int kv_heads, int D, int V, int taps, int ra, int rg,
                              int out_dtype, void* stream) {
  if (!out || !o || !proj || !g2 || !norm_w || !tok_req) return HS_ERR_ARGUMENT;
  hs::DeltaShape s;
  int rc = delta_shape(&s, heads, kv_heads, D, V, taps, ra, rg);
  if (rc) return rc;
  if (n_tokens <= 0) return HS_OK;
  cudaStream_t st = (cudaStream_t)stream;
  if (out_dtype == HS_DT_F32)
    hs::delta_finish_kernel<float><<<n_tokens, 256, 0, st>>>((float*)out, o, proj, g2, norm_w,
                                                             tok_req, eps, s);
  else if (out_dtype == HS_DT_BF16)
    hs::delta_finish_kernel<__nv_bfloat16><<<n_tokens, 256, 0, st>>>(
        (__nv_bfloat16*)out, o, proj, g2, norm_w, tok_req, eps, s);
  else
    return HS_ERR_UNSUPPORTED;
  HS_LAUNCH_CHECK();
  return HS_OK;
}

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

// Three blocks a token (blockIdx.y): 0 convolves q and k and makes them unit vectors, 1 convolves
// v and forms beta, 2 forms the decay.  They share nothing.
__global__ void __launch_bounds__(256)
delta_prepare_kernel(float* __restrict__ qn, float* __restrict__ kn, float* __restrict__ vv,
                     float* __restrict__ beta, float* __restrict__ decay,
                     const float* __restrict__ proj, const float* __restrict__ conv_w,
                     const float* __restrict__ a2, const float* __restrict__ dt_bias,
                     const float* __restrict__ A_log, const float* __restrict__ state,
                     const int* __restrict__ tok_req, const int* __restrict__ req_start,
                     const int* __restrict__ req_slot, DeltaShape s,
                     const float* __restrict__ z_a) {
  extern __shared__ float s_c[];                 // [2 * kv_heads * D] q and k after conv and silu
  const int t = blockIdx.x;
  const int r = tok_req[t];
  if (r < 0) return;
  const int C = channels(s);
  const int QK = s.kv_heads * s.D;
  const float* row = proj + (size_t)t * s.stride;
  if (blockIdx.y == 2) {
    const int HD = s.heads * s.D;
    for (int i = threadIdx.x; i < HD; i += blockDim.x) {
      float z = 0.f;
      if (z_a) {                                   // W_a2 a was formed as a matrix product
        z = z_a[(size_t)t * HD + i];
      } else {
#pragma unroll 8
        for (int k = 0; k < s.ra; ++k) z = fmaf(a2[(size_t)k * HD + i], row[s.a_off + k], z);
      }
      z += dt_bias[i];
      decay[(size_t)t * HD + i] = expf(-expf(A_log[i / s.D]) * softplusf_(z));
    }
    return;
  }
  const int first = req_start[r];
  const int l = t - first;
  const float* cst = state + (size_t)req_slot[r] * s.state_stride + (size_t)s.heads * s.D * s.V;
  const int hist = s.taps - 1;
  auto conv = [&](int c) {
    float acc = 0.f;
#pragma unroll 4
    for (int j = 0; j < s.taps; ++j) {
      const int local = l - (hist - j);
      const float in = local >= 0 ? proj[(size_t)(first + local) * s.stride + c]
                                  : cst[(size_t)(local + hist) * C + c];
      acc = fmaf(conv_w[(size_t)c * s.taps + j], in, acc);
    }
    return acc * sigmoidf_(acc);
  };
  if (blockIdx.y == 1) {
    const int HV = s.heads * s.V;
    for (int i = threadIdx.x; i < HV; i += blockDim.x) vv[(size_t)t * HV + i] = conv(2 * QK + i);
    for (int h = threadIdx.x; h < s.heads; h += blockDim.x)
      beta[(size_t)t * s.heads + h] = sigmoidf_(row[s.b_off + h]);
    return;
  }
  for (int c = threadIdx.x; c < 2 * QK; c += blockDim.x) s_c[c] = conv(c);
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
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

constexpr int DR_DP = 16;         // state rows a thread keeps
constexpr int DR_STAGES = 3;      // chunks of tokens in shared memory
constexpr int DR_THREADS = 64;   // few warps a block: the shared-memory pipe of an SM bounds a block's step from token to token

__device__ __forceinline__ void cp_async4(float* dst, const float* src) {
  const unsigned sa = (unsigned)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(sa), "l"(src));
}
__device__ __forceinline__ void cp_async16(float* dst, const float* src) {
  const unsigned sa = (unsigned)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(sa), "l"(src));
}

// Thread (col, part) keeps DP rows of column col of S: the four rows 4*part + 4*KS*j .. + 3 for
// j = 0 .. DP/4 - 1, so that the KS neighbouring lanes of a column read neighbouring 16-byte
// pieces of a row in shared memory (no bank conflict); they sum their shares with a butterfly.
// The tokens' q, k, decay
// rows (padded with zeros to KS*DP), v columns and betas come through shared memory a chunk of
// CH tokens at a time, fetched asynchronously two chunks ahead: the latency of fetching them is
// off the token-to-token chain.
__global__ void __launch_bounds__(DR_THREADS)
delta_recurrence_kernel(float* __restrict__ o, float* __restrict__ state,
                        const float* __restrict__ qn, const float* __restrict__ kn,
                        const float* __restrict__ vv, const float* __restrict__ beta,
                        const float* __restrict__ decay, const int* __restrict__ req_start,
                        const int* __restrict__ req_len, const int* __restrict__ req_slot,
                        DeltaShape s, int KS, int CH, int vec) {
  extern __shared__ __align__(16) float sm[];
  const int r = blockIdx.x, h = blockIdx.y;
  const int n = req_len[r];
  if (n <= 0) return;
  const int Dp = KS * DR_DP;
  const int cols = DR_THREADS / KS;
  const int per_buf = (3 * CH * Dp + CH * cols + CH + 3) & ~3;      // buffers 16-byte aligned
  const int part = threadIdx.x % KS;
  const int lc = threadIdx.x / KS;
  const int col0 = blockIdx.z * cols;
  const int col = col0 + lc;
  const bool col_ok = col < s.V;
  const int kh = h / (s.heads / s.kv_heads);
  const int d0 = part * 4;                       // row of st[i]: d0 + 4*KS*(i/4) + i%4
  const int dj = 4 * KS;
  float* S = state + (size_t)req_slot[r] * s.state_stride + (size_t)h * s.D * s.V;
  float st[DR_DP];
#pragma unroll
  for (int i = 0; i < DR_DP; ++i) {
    const int d = d0 + dj * (i >> 2) + (i & 3);
    st[i] = (col_ok && d < s.D) ? S[(size_t)d * s.V + col] : 0.f;
  }
  const int QK = s.kv_heads * s.D, HV = s.heads * s.V, HD = s.heads * s.D;
  const int first = req_start[r];
  for (int i = threadIdx.x; i < DR_STAGES * per_buf; i += DR_THREADS) sm[i] = 0.f;   // padding stays 0
  __syncthreads();
  auto fetch = [&](int buf, int c0) {
    float* b_k = sm + buf * per_buf;
    float* b_q = b_k + CH * Dp;
    float* b_g = b_q + CH * Dp;
    float* b_v = b_g + CH * Dp;
    float* b_b = b_v + CH * cols;
    const int nc = min(CH, n - c0);
    if (vec) {
      const int D4 = s.D >> 2;
      for (int i = threadIdx.x; i < nc * D4; i += DR_THREADS) {
        const int tt = i / D4, d = (i - tt * D4) * 4;
        const size_t row = first + c0 + tt;
        cp_async16(b_k + tt * Dp + d, kn + row * QK + kh * s.D + d);
        cp_async16(b_q + tt * Dp + d, qn + row * QK + kh * s.D + d);
        cp_async16(b_g + tt * Dp + d, decay + row * HD + h * s.D + d);
      }
    } else {
      for (int i = threadIdx.x; i < nc * s.D; i += DR_THREADS) {
        const int tt = i / s.D, d = i - tt * s.D;
        const size_t row = first + c0 + tt;
        cp_async4(b_k + tt * Dp + d, kn + row * QK + kh * s.D + d);
        cp_async4(b_q + tt * Dp + d, qn + row * QK + kh * s.D + d);
        cp_async4(b_g + tt * Dp + d, decay + row * HD + h * s.D + d);
      }
    }
    for (int i = threadIdx.x; i < nc * cols; i += DR_THREADS) {
      const int tt = i / cols, cc = i - tt * cols;
      if (col0 + cc < s.V)
        cp_async4(b_v + i, vv + (size_t)(first + c0 + tt) * HV + h * s.V + col0 + cc);
    }
    if (threadIdx.x < nc)
      cp_async4(b_b + threadIdx.x, beta + (size_t)(first + c0 + threadIdx.x) * s.heads + h);
    asm volatile("cp.async.commit_group;");
  };
  // three buffers: while a chunk is worked on, the two behind it are on their way (a fetch
  // takes longer than a chunk of tokens does).  Every turn commits a group, an empty one at
  // the end, so that "all but the newest two have landed" always names the chunk of this turn.
  fetch(0, 0);
  if (CH < n) fetch(1, CH); else asm volatile("cp.async.commit_group;");
  int buf = 0;
  for (int c0 = 0; c0 < n; c0 += CH, buf = (buf + 1) % DR_STAGES) {
    const int nc = min(CH, n - c0);
    if (c0 + 2 * CH < n) fetch((buf + 2) % DR_STAGES, c0 + 2 * CH);
    else asm volatile("cp.async.commit_group;");
    asm volatile("cp.async.wait_group 2;");
    __syncthreads();
    const float* b_k = sm + buf * per_buf;
    const float* b_q = b_k + CH * Dp;
    const float* b_g = b_q + CH * Dp;
    const float* b_v = b_g + CH * Dp;
    const float* b_b = b_v + CH * cols;
    // Two register sets alternate: while a token is worked on, the rows of the next one are
    // already on their way from shared memory.  The sum over a column's lanes for a token's
    // output (needed only by the store) rides along with the next token's sum for its dot
    // product, stage by stage, so the chain from token to token holds one butterfly, not two.
    struct Rows { float k[DR_DP], q[DR_DP], g[DR_DP], v, b; };
    auto read = [&](int tt, Rows& r) {
      const float4* k4 = (const float4*)(b_k + tt * Dp + d0);
      const float4* q4 = (const float4*)(b_q + tt * Dp + d0);
      const float4* g4 = (const float4*)(b_g + tt * Dp + d0);
#pragma unroll
      for (int j = 0; j < DR_DP / 4; ++j) {
        const float4 a = k4[j * KS], b = q4[j * KS], c = g4[j * KS];
        r.k[4 * j] = a.x; r.k[4 * j + 1] = a.y; r.k[4 * j + 2] = a.z; r.k[4 * j + 3] = a.w;
        r.q[4 * j] = b.x; r.q[4 * j + 1] = b.y; r.q[4 * j + 2] = b.z; r.q[4 * j + 3] = b.w;
        r.g[4 * j] = c.x; r.g[4 * j + 1] = c.y; r.g[4 * j + 2] = c.z; r.g[4 * j + 3] = c.w;
      }
      r.v = b_v[tt * cols + lc];
      r.b = b_b[tt];
    };
    float pend = 0.f;               // the token before: its output, not yet summed over the lanes
    int pend_tt = -1;
    auto work = [&](int tt, const Rows& r, Rows& next) {
      if (tt + 1 < nc) read(tt + 1, next);
      float dot0 = 0.f, dot1 = 0.f;
#pragma unroll
      for (int j = 0; j < DR_DP; j += 2) {
        st[j] *= r.g[j];
        st[j + 1] *= r.g[j + 1];
        dot0 = fmaf(st[j], r.k[j], dot0);
        dot1 = fmaf(st[j + 1], r.k[j + 1], dot1);
      }
      float dot = dot0 + dot1;
      for (int off = 1; off < KS; off <<= 1) {
        const float d2 = __shfl_xor_sync(0xffffffffu, dot, off);
        const float p2 = __shfl_xor_sync(0xffffffffu, pend, off);
        dot += d2;
        pend += p2;
      }
      if (pend_tt >= 0 && part == 0 && col_ok)
        o[(size_t)(first + c0 + pend_tt) * HV + h * s.V + col] = pend;
      const float u = r.b * (r.v - dot);
      float out0 = 0.f, out1 = 0.f;
#pragma unroll
      for (int j = 0; j < DR_DP; j += 2) {
        st[j] = fmaf(r.k[j], u, st[j]);
        st[j + 1] = fmaf(r.k[j + 1], u, st[j + 1]);
        out0 = fmaf(st[j], r.q[j], out0);
        out1 = fmaf(st[j + 1], r.q[j + 1], out1);
      }
      pend = out0 + out1;
      pend_tt = tt;
    };
    Rows ra, rb;
    read(0, ra);
    for (int tt = 0; tt < nc; tt += 2) {
      work(tt, ra, rb);
      if (tt + 1 < nc) work(tt + 1, rb, ra);
    }
    for (int off = 1; off < KS; off <<= 1) pend += __shfl_xor_sync(0xffffffffu, pend, off);
    if (part == 0 && col_ok) o[(size_t)(first + c0 + pend_tt) * HV + h * s.V + col] = pend;
    __syncthreads();                              // this buffer is fetched into again next turn
  }
#pragma unroll
  for (int i = 0; i < DR_DP; ++i) {
    const int d = d0 + dj * (i >> 2) + (i & 3);
    if (col_ok && d < s.D) S[(size_t)d * s.V + col] = st[i];
  }
}

// One block per token and head: the head's root mean square by a block reduction, then one
// thread per output forms its gate (a sum over the rg inputs, several loads in flight).
template <typename TO>
__global__ void __launch_bounds__(128)
delta_finish_kernel(TO* __restrict__ out, const float* __restrict__ o,
                    const float* __restrict__ proj, const float* __restrict__ g2,
                    const float* __restrict__ norm_w, const int* __restrict__ tok_req,
                    float eps, DeltaShape s, const float* __restrict__ z_g) {
  __shared__ float red[4];
  extern __shared__ float s_gin[];                  // [rg]
  const int t = blockIdx.x, h = blockIdx.y;
  if (tok_req[t] < 0) return;
  const int HV = s.heads * s.V;
  const float* gin = proj + (size_t)t * s.stride + s.g_off;
  for (int k = threadIdx.x; k < s.rg; k += blockDim.x) s_gin[k] = gin[k];
  const float* src = o + (size_t)t * HV + (size_t)h * s.V;
  float ss = 0.f;
  for (int e = threadIdx.x; e < s.V; e += blockDim.x) ss = fmaf(src[e], src[e], ss);
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
  for (int i = 0; i < (int)(blockDim.x >> 5); ++i) tot += red[i];
  const float inv = 1.0f / sqrtf(tot / (float)s.V + eps);
  for (int e = threadIdx.x; e < s.V; e += blockDim.x) {
    const float* gcol = g2 + (size_t)h * s.V + e;
    float z = 0.f;
    if (z_g) {                                     // W_g2 g was formed as a matrix product
      z = z_g[(size_t)t * HV + h * s.V + e];
    } else {
#pragma unroll 8
      for (int k = 0; k < s.rg; ++k) z = fmaf(gcol[(size_t)k * HV], s_gin[k], z);
    }
    out[(size_t)t * HV + h * s.V + e] = from_f<TO>(src[e] * inv * norm_w[e] * sigmoidf_(z));
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
                               const float* z_a, void* stream) {
  if (!qn || !kn || !vv || !beta || !decay || !proj || !conv_w || !a2 || !dt_bias || !A_log ||
      !state || !tok_req || !req_start || !req_len || !req_slot)
    return HS_ERR_ARGUMENT;
  hs::DeltaShape s;
  int rc = delta_shape(&s, heads, kv_heads, D, V, taps, ra, rg);
  if (rc) return rc;
  if (n_tokens <= 0 || n_requests <= 0) return HS_OK;
  const int C = 2 * kv_heads * D + heads * V;
  const size_t smem = (size_t)2 * kv_heads * D * sizeof(float);
  if (smem > 200 * 1024) return HS_ERR_UNSUPPORTED;
  cudaStream_t st = (cudaStream_t)stream;
  if (smem > 48 * 1024)
    cudaFuncSetAttribute(hs::delta_prepare_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         (int)smem);
  hs::delta_prepare_kernel<<<dim3(n_tokens, 3), 256, smem, st>>>(qn, kn, vv, beta, decay, proj, conv_w, a2,
                                                        dt_bias, A_log, state, tok_req, req_start,
                                                        req_slot, s, z_a);
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
  if (D > hs::DR_DP * 32) return HS_ERR_UNSUPPORTED;   // a column's parts are lanes of one warp
  if (n_requests <= 0) return HS_OK;
  int KS = 1;
  while (KS * hs::DR_DP < D) KS <<= 1;
  const int cols = hs::DR_THREADS / KS;
  const int Dp = KS * hs::DR_DP;
  int CH = 1024 / Dp;                               // tokens a chunk: 3 * CH * Dp <= 3072 floats
  CH = CH < 2 ? 2 : (CH > 16 ? 16 : CH);
  const size_t smem = hs::DR_STAGES * (size_t)((3 * CH * Dp + CH * cols + CH + 3) & ~3) * sizeof(float);
  // 16-byte copies need rows of q, k and the decay that start on 16-byte boundaries
  const int vec = D % 4 == 0 && !((uintptr_t)qn & 15) && !((uintptr_t)kn & 15) &&
                  !((uintptr_t)decay & 15);
  dim3 grid(n_requests, heads, (V + cols - 1) / cols);
  hs::delta_recurrence_kernel<<<grid, hs::DR_THREADS, smem, (cudaStream_t)stream>>>(
      o, state, qn, kn, vv, beta, decay, req_start, req_len, req_slot, s, KS, CH, vec);
  HS_LAUNCH_CHECK();
  return HS_OK;
}

HS_EXPORT int hs_delta_finish(void* out, const float* o, const float* proj, const float* g2,
                              const float* norm_w, const int* tok_req, int n_tokens, float eps,
                              int heads, int kv_heads, int D, int V, int taps, int ra, int rg,
                              int out_dtype, const float* z_g, void* stream) {
  if (!out || !o || !proj || !g2 || !norm_w || !tok_req) return HS_ERR_ARGUMENT;
  hs::DeltaShape s;
  int rc = delta_shape(&s, heads, kv_heads, D, V, taps, ra, rg);
  if (rc) return rc;
  if (n_tokens <= 0) return HS_OK;
  cudaStream_t st = (cudaStream_t)stream;
  if (out_dtype == HS_DT_F32)
    hs::delta_finish_kernel<float><<<dim3(n_tokens, heads), 128, rg * sizeof(float), st>>>(
        (float*)out, o, proj, g2, norm_w, tok_req, eps, s, z_g);
  else if (out_dtype == HS_DT_BF16)
    hs::delta_finish_kernel<__nv_bfloat16><<<dim3(n_tokens, heads), 128, rg * sizeof(float), st>>>(
        (__nv_bfloat16*)out, o, proj, g2, norm_w, tok_req, eps, s, z_g);
  else
    return HS_ERR_UNSUPPORTED;
  HS_LAUNCH_CHECK();
  return HS_OK;
}

// Routed feed-forward (mixture of experts) on the CUDA cores.
//
// route    per token: z = W_r h in float32, s = sigmoid(z).  Experts form `n_groups` equal groups
//          of neighbours; a group's score is the sum of its two largest s; only experts of the
//          `keep` best groups are eligible; the `top` eligible experts with the largest s are
//          chosen (the lower index wins a tie) with weights s / (sum of the chosen s + 1e-20).
// gate_up  per (token, chosen expert): g = min(W_g h, limit), u = clamp(W_u h, -limit, limit),
//          y = g * sigmoid(1.702 g) * (u + 1)
// down     per token: x += sum_k weight_k * (W_d[e_k] y_k), experts in the order they were chosen
//
// Expert matrices are held k-major: gate/up [E, width, ff], down [E, ff, width], so that the
// threads of a warp (one output each) read neighbouring weights.  Sums over k are sequential per
// output in float32: a token's result does not depend on the batch around it.
#include "common.cuh"

namespace hs {

constexpr int MOE_ROUTE_WARPS = 4;

// (value, index) argmax over a warp; larger value wins, then the lower index
__device__ __forceinline__ void warp_argmax(float& v, int& i) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, i, o);
    if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
  }
}

template <typename TH>
__global__ void __launch_bounds__(MOE_ROUTE_WARPS * 32)
moe_route_kernel(int* __restrict__ sel_idx, float* __restrict__ sel_w, const TH* __restrict__ h,
                 const float* __restrict__ w_router, const int* __restrict__ tok_req,
                 int n_tokens, int width, int E, int top, int n_groups, int keep) {
  extern __shared__ float smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * MOE_ROUTE_WARPS + warp;
  if (t >= n_tokens || tok_req[t] < 0) return;        // a warp works alone: no block barrier below
  float* s_s = smem + (size_t)warp * (E + n_groups);  // [E] scores (then -1 when taken / barred)
  float* s_g = s_s + E;                               // [n_groups]
  const TH* hr = h + (size_t)t * width;
  for (int e = 0; e < E; ++e) {
    const float* wr = w_router + (size_t)e * width;
    float z = 0.f;
    for (int k = lane; k < width; k += 32) z = fmaf(wr[k], to_f(hr[k]), z);
    z = warp_sum(z);
    if (lane == 0) s_s[e] = 1.0f / (1.0f + expf(-z));
  }
  __syncwarp();
  const int per = E / n_groups;
  for (int g = lane; g < n_groups; g += 32) {
    float a = -1.f, b = -1.f;                          // the two largest of the group
    for (int j = 0; j < per; ++j) {
      const float v = s_s[g * per + j];
      if (v > a) { b = a; a = v; } else if (v > b) { b = v; }
    }
    s_g[g] = per > 1 ? a + b : a;
  }
  __syncwarp();
  // the `keep` best groups stay; the others are barred.  A kept group is marked by score -2.
  for (int round = 0; round < keep; ++round) {
    float bv = -1.f;
    int bi = 0x7fffffff;
    for (int g = lane; g < n_groups; g += 32)
      if (s_g[g] > bv) { bv = s_g[g]; bi = g; }
    warp_argmax(bv, bi);
    if (lane == 0) s_g[bi] = -2.f;
    __syncwarp();
  }
  // choose: `top` rounds of argmax over eligible experts
  float chosen_v = 0.f;                                // lane k keeps the k-th choice (top <= 32)
  int chosen_i = 0;
  float total = 0.f;
  for (int round = 0; round < top; ++round) {
    float bv = -1.f;
    int bi = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float v = s_g[e / per] == -2.f ? s_s[e] : -1.f;
      if (v > bv) { bv = v; bi = e; }
    }
    warp_argmax(bv, bi);
    if (lane == round) { chosen_v = bv; chosen_i = bi; }
    total += bv;
    if (lane == 0) s_s[bi] = -1.f;                     // taken
    __syncwarp();
  }
  if (lane < top) {
    sel_idx[(size_t)t * top + lane] = chosen_i;
    sel_w[(size_t)t * top + lane] = chosen_v / (total + 1e-20f);
  }
}

constexpr int MOE_THREADS = 128;

template <typename TW>
__global__ void __launch_bounds__(MOE_THREADS)
moe_gate_up_kernel(float* __restrict__ y, const TW* __restrict__ h, const TW* __restrict__ w_gate,
                   const TW* __restrict__ w_up, const int* __restrict__ sel_idx,
                   const int* __restrict__ tok_req, int width, int ff, int top, int E,
                   float limit) {
  extern __shared__ float s_h[];                       // [width]
  const int pair = blockIdx.x;
  const int t = pair / top;
  if (tok_req[t] < 0) return;
  const int e = sel_idx[pair];
  if (e < 0 || e >= E) return;
  for (int k = threadIdx.x; k < width; k += MOE_THREADS) s_h[k] = to_f(h[(size_t)t * width + k]);
  __syncthreads();
  const int f = blockIdx.y * MOE_THREADS + threadIdx.x;
  if (f >= ff) return;
  const TW* wg = w_gate + (size_t)e * width * ff + f;
  const TW* wu = w_up + (size_t)e * width * ff + f;
  float g = 0.f, u = 0.f;
  for (int k = 0; k < width; ++k) {
    const float hv = s_h[k];
    g = fmaf(to_f(wg[(size_t)k * ff]), hv, g);
    u = fmaf(to_f(wu[(size_t)k * ff]), hv, u);
  }
  g = fminf(g, limit);
  u = fminf(fmaxf(u, -limit), limit);
  y[(size_t)pair * ff + f] = g * (1.0f / (1.0f + expf(-1.702f * g))) * (u + 1.0f);
}

template <typename TW>
__global__ void __launch_bounds__(MOE_THREADS)
moe_down_kernel(float* __restrict__ x, const float* __restrict__ y, const TW* __restrict__ w_down,
                const int* __restrict__ sel_idx, const float* __restrict__ sel_w,
                const int* __restrict__ tok_req, int width, int ff, int top, int E) {
  extern __shared__ float s_y[];                       // [top][ff]
  const int t = blockIdx.x;
  if (tok_req[t] < 0) return;
  for (int i = threadIdx.x; i < top * ff; i += MOE_THREADS) s_y[i] = y[(size_t)t * top * ff + i];
  __syncthreads();
  const int n = blockIdx.y * MOE_THREADS + threadIdx.x;
  if (n >= width) return;
  float sum = 0.f;
  for (int k = 0; k < top; ++k) {
    const int e = sel_idx[(size_t)t * top + k];
    if (e < 0 || e >= E) continue;
    const TW* wd = w_down + (size_t)e * ff * width + n;
    const float* yk = s_y + (size_t)k * ff;
    float acc = 0.f;
    for (int f = 0; f < ff; ++f) acc = fmaf(to_f(wd[(size_t)f * width]), yk[f], acc);
    sum = fmaf(sel_w[(size_t)t * top + k], acc, sum);
  }
  x[(size_t)t * width + n] += sum;
}

}  // namespace hs

HS_EXPORT int hs_moe_route(int* sel_idx, float* sel_w, const void* h, const float* w_router,
                           const int* tok_req, int n_tokens, int width, int E, int top,
                           int n_groups, int keep, int h_dtype, void* stream) {
  if (!sel_idx || !sel_w || !h || !w_router || !tok_req) return HS_ERR_ARGUMENT;
  if (E <= 0 || top <= 0 || top > 32 || n_groups <= 0 || E % n_groups || keep <= 0 ||
      keep > n_groups || top > keep * (E / n_groups))
    return HS_ERR_UNSUPPORTED;
  if (n_tokens <= 0) return HS_OK;
  const size_t smem = (size_t)hs::MOE_ROUTE_WARPS * (E + n_groups) * sizeof(float);
  if (smem > 48 * 1024) return HS_ERR_UNSUPPORTED;
  const int grid = (n_tokens + hs::MOE_ROUTE_WARPS - 1) / hs::MOE_ROUTE_WARPS;
  cudaStream_t st = (cudaStream_t)stream;
  if (h_dtype == HS_DT_F32)
    hs::moe_route_kernel<float><<<grid, hs::MOE_ROUTE_WARPS * 32, smem, st>>>(
        sel_idx, sel_w, (const float*)h, w_router, tok_req, n_tokens, width, E, top, n_groups,
        keep);
  else if (h_dtype == HS_DT_BF16)
    hs::moe_route_kernel<__nv_bfloat16><<<grid, hs::MOE_ROUTE_WARPS * 32, smem, st>>>(
        sel_idx, sel_w, (const __nv_bfloat16*)h, w_router, tok_req, n_tokens, width, E, top,
        n_groups, keep);
  else
    return HS_ERR_UNSUPPORTED;
  HS_LAUNCH_CHECK();
  return HS_OK;
}

HS_EXPORT int hs_moe_experts(float* x, float* y, const void* h, const void* w_gate,
                             const void* w_up, const void* w_down, const int* sel_idx,
                             const float* sel_w, const int* tok_req, int n_tokens, int width,
                             int ff, int top, int E, float limit, int dtype, void* stream) {
  if (!x || !y || !h || !w_gate || !w_up || !w_down || !sel_idx || !sel_w || !tok_req)
    return HS_ERR_ARGUMENT;
  if (width <= 0 || ff <= 0 || top <= 0 || E <= 0) return HS_ERR_UNSUPPORTED;
  if (n_tokens <= 0) return HS_OK;
  const size_t smem_h = (size_t)width * sizeof(float);
  const size_t smem_y = (size_t)top * ff * sizeof(float);
  if (smem_h > 200 * 1024 || smem_y > 200 * 1024) return HS_ERR_UNSUPPORTED;
  cudaStream_t st = (cudaStream_t)stream;
  dim3 g1(n_tokens * top, (ff + hs::MOE_THREADS - 1) / hs::MOE_THREADS);
  dim3 g2(n_tokens, (width + hs::MOE_THREADS - 1) / hs::MOE_THREADS);
#define HS_MOE(TW)                                                                             \
  do {                                                                                         \
    auto k1 = hs::moe_gate_up_kernel<TW>;                                                      \
    auto k2 = hs::moe_down_kernel<TW>;                                                         \
    if (smem_h > 48 * 1024)                                                                    \
      cudaFuncSetAttribute(k1, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_h);      \
    if (smem_y > 48 * 1024)                                                                    \
      cudaFuncSetAttribute(k2, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_y);      \
    k1<<<g1, hs::MOE_THREADS, smem_h, st>>>(y, (const TW*)h, (const TW*)w_gate,                \
                                            (const TW*)w_up, sel_idx, tok_req, width, ff, top, \
                                            E, limit);                                         \
    HS_LAUNCH_CHECK();                                                                         \
    k2<<<g2, hs::MOE_THREADS, smem_y, st>>>(x, y, (const TW*)w_down, sel_idx, sel_w, tok_req,  \
                                            width, ff, top, E);                                \
  } while (0)
  if (dtype == HS_DT_F32) HS_MOE(float);
  else if (dtype == HS_DT_BF16) HS_MOE(__nv_bfloat16);
  else return HS_ERR_UNSUPPORTED;
#undef HS_MOE
  HS_LAUNCH_CHECK();
  return HS_OK;
}

// Attention over a shared latent: per token the cache holds ONE row [latent (R) | rotated key
// part (P)] for all heads.  Queries arrive absorbed: qa[h] = W_uk[h]^T q_plain[h] (R numbers)
// and the rotated part qr[h] (P numbers), so that
//
//   score(i, j) = (qa_i . c_j + qr_i . kr_j) * scale        for every j <= i (causal)
//   weights     = exp(score - m) / (sum_j exp(score_j - m) + exp(sink_h - m))
//   out_lat[h]  = sum_j weight_j * c_j                        (R numbers; W_uv[h] follows)
//
// The sink of a head is a learned logit without key or value: it only enters the denominator.
// Scores, the running maximum, the denominator and the accumulator are float32.  A step of few
// tokens splits each token's keys over several blocks whose shares (maximum, sum, weighted rows)
// a second kernel merges; the split depends on the number of tokens in the step only.
//
// `plan` (may be null): the step's attention work lists; with it `n_tokens` blocks are launched
// and block i works on the i-th single-query token of the plan, if there is one.
//
// Pool rows: [pages, page_size, R + P] in the cache type; row of position p of request r is
// table[r, p / page_size] * page_size + p % page_size.
#include "common.cuh"
#include "rotary.cuh"

namespace hs {

// -- append: RMS-norm the latent, rotate the key part (the first rot_dims entries; 0: it arrives
//    rotated), write the cache row -----------------------------------------------------------------
template <typename TC>
__global__ void latent_append_kernel(TC* __restrict__ pool, const float* __restrict__ proj,
                                     const float* __restrict__ norm_w,
                                     const int* __restrict__ table,
                                     const int* __restrict__ tok_pos,
                                     const int* __restrict__ tok_req, int proj_stride, int c_off,
                                     int R, int P, float eps, int page_size, int num_pages,
                                     int max_pages, int* status,
                                     const float* __restrict__ freq, int rot_dims) {
  __shared__ float red[4];
  __shared__ float bcast;
  const int t = blockIdx.x;
  const int r = tok_req[t];
  if (r < 0) return;
  const int p = tok_pos[t];
  const int pi = p / page_size;
  const int page = (p >= 0 && pi < max_pages) ? table[(size_t)r * max_pages + pi] : -1;
  if (page < 0 || page >= num_pages) {
    if (threadIdx.x == 0) atomicOr(status, HS_STATUS_BAD_PAGE);
    return;
  }
  const float* src = proj + (size_t)t * proj_stride + c_off;
  float ss = 0.f;
  for (int e = threadIdx.x; e < R; e += blockDim.x) ss = fmaf(src[e], src[e], ss);
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x == 0) {
    float tot = 0.f;
    for (int i = 0; i < (int)(blockDim.x >> 5); ++i) tot += red[i];
    bcast = 1.0f / sqrtf(tot / (float)R + eps);
  }
  __syncthreads();
  const float rs = bcast;
  TC* dst = pool + ((size_t)page * page_size + (p % page_size)) * (R + P);
  for (int e = threadIdx.x; e < R; e += blockDim.x) dst[e] = from_f<TC>(src[e] * rs * norm_w[e]);
  for (int e = threadIdx.x; e < P; e += blockDim.x)
    dst[R + e] = from_f<TC>(e < rot_dims ? rotate_entry(src[R + e], src[R + (e ^ 1)], e, rot_dims, p, freq)
                                         : src[R + e]);
}

// -- attention ---------------------------------------------------------------------------------
constexpr int LA_TILE = 32;     // keys per tile: one per lane when scores are formed
constexpr int LA_HB = 8;        // heads (warps) per block

// Shared rows are padded to a multiple of 4 floats (zeros), read 16 bytes at a time.  Key rows
// have a stride of 4 (mod 32) floats, so that the lanes of a quarter warp, each on a row of its
// own while scores are formed, hit distinct banks; while the weighted rows are summed, lane l
// owns the dims 4 l + 128 i .. + 3 and the lanes read neighbouring pieces of one row.
__host__ __device__ inline int la_w4(int W) { return (W + 3) & ~3; }
__host__ __device__ inline int la_stride(int W) { return ((la_w4(W) + 27) / 32) * 32 + 4; }

template <typename TC, int RC>      // RC: accumulator floats a lane keeps, a multiple of 4
__global__ void __launch_bounds__(LA_HB * 32)
latent_attention_kernel(float* __restrict__ out, const float* __restrict__ qa,
                        const float* __restrict__ qr, const TC* __restrict__ pool,
                        const int* __restrict__ table, const int* __restrict__ tok_pos,
                        const int* __restrict__ tok_req, const float* __restrict__ sink,
                        int n_heads, int R, int P, int qr_stride, int qr_hstride, int qr_off,
                        float scale, int page_size, int num_pages, int max_pages, int* status,
                        int nsplit, float* __restrict__ partial,
                        const float* __restrict__ freq, int rot_dims,
                        const int* __restrict__ plan) {
  extern __shared__ __align__(16) float smem[];
  const int W = R + P;
  const int W4 = la_w4(W), ks = la_stride(W);
  float* s_q = smem;                            // [LA_HB][W4]
  float* s_k = smem + LA_HB * W4;               // [LA_TILE][ks]
  // with a plan, only its single-query tokens are this kernel's (the tiles go elsewhere)
  if (plan && (int)blockIdx.x >= plan[0]) return;
  const int t = plan ? plan[4 + 3 * blockIdx.x] : blockIdx.x;
  const int r = tok_req[t];
  if (r < 0) return;
  const int pos = tok_pos[t];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.y * LA_HB + warp;
  const bool live = h < n_heads;
  // queries of this block's heads
  for (int i = threadIdx.x; i < LA_HB * W4; i += blockDim.x) {
    const int hh = i / W4, d = i - hh * W4;
    const int head = blockIdx.y * LA_HB + hh;
    float v = 0.f;
    if (head < n_heads && d < W) {
      if (d < R) {
        v = qa[((size_t)t * n_heads + head) * R + d];
      } else {                      // the rotated part: turned here when it arrives unrotated
        const float* src = qr + (size_t)t * qr_stride + (size_t)head * qr_hstride + qr_off;
        const int e = d - R;
        v = e < rot_dims ? rotate_entry(src[e], src[e ^ 1], e, rot_dims, pos, freq) : src[e];
      }
    }
    s_q[i] = v;
  }
  // alone, a block opens its running softmax with the sink (weight 1); as one of `nsplit`
  // blocks over the keys it starts empty and the sink joins when the shares are merged
  float m = nsplit > 1 ? -INFINITY : (live ? sink[h] : 0.f);
  float l = nsplit > 1 ? 0.f : 1.f;
  float acc[RC];
#pragma unroll
  for (int i = 0; i < RC; ++i) acc[i] = 0.f;
  const float4* q4 = (const float4*)(s_q + warp * W4);
  const int n_tiles = pos / LA_TILE + 1;
  const int per = (n_tiles + nsplit - 1) / nsplit;
  const int tile_lo = blockIdx.z * per, tile_hi = min(n_tiles, tile_lo + per);
  for (int base = tile_lo * LA_TILE; base < tile_hi * LA_TILE; base += LA_TILE) {
    __syncthreads();                            // the tile before has been used (and s_q is set)
    const int nk = min(LA_TILE, pos + 1 - base);
    for (int j = warp; j < nk; j += LA_HB) {
      const int kp = base + j;
      const int pi = kp / page_size;
      const int page = pi < max_pages ? table[(size_t)r * max_pages + pi] : -1;
      float* dst = s_k + j * ks;
      if (page < 0 || page >= num_pages) {
        if (lane == 0) atomicOr(status, HS_STATUS_BAD_PAGE);
        for (int d = lane; d < W4; d += 32) dst[d] = 0.f;
      } else {
        const TC* src = pool + ((size_t)page * page_size + (kp % page_size)) * W;
        for (int d = lane; d < W4; d += 32) dst[d] = d < W ? to_f(src[d]) : 0.f;
      }
    }
    __syncthreads();
    if (!live) continue;
    float s = -INFINITY;
    if (lane < nk) {
      const float4* k4 = (const float4*)(s_k + lane * ks);
      float d0 = 0.f, d1 = 0.f;
      for (int d = 0; d < W4 / 4; ++d) {
        const float4 a = q4[d], b = k4[d];
        d0 = fmaf(a.x, b.x, d0); d1 = fmaf(a.y, b.y, d1);
        d0 = fmaf(a.z, b.z, d0); d1 = fmaf(a.w, b.w, d1);
      }
      s = (d0 + d1) * scale;
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float corr = expf(m - m_new);
    const float pj = lane < nk ? expf(s - m_new) : 0.f;
    l = l * corr + warp_sum(pj);
    m = m_new;
#pragma unroll
    for (int i = 0; i < RC; ++i) acc[i] *= corr;
    for (int j = 0; j < nk; ++j) {
      const float w = __shfl_sync(0xffffffffu, pj, j);
      const float* kr = s_k + j * ks + 4 * lane;
#pragma unroll
      for (int i = 0; i < RC / 4; ++i) {
        if (4 * lane + 128 * i < R) {           // the piece lies within the padded row
          const float4 c = *(const float4*)(kr + 128 * i);
          acc[4 * i] = fmaf(w, c.x, acc[4 * i]);
          acc[4 * i + 1] = fmaf(w, c.y, acc[4 * i + 1]);
          acc[4 * i + 2] = fmaf(w, c.z, acc[4 * i + 2]);
          acc[4 * i + 3] = fmaf(w, c.w, acc[4 * i + 3]);
        }
      }
    }
  }
  if (!live) return;
  float* dst;
  float inv = 1.f;
  if (nsplit > 1) {                             // this block's share: maximum, sum, weighted rows
    float* ps = partial + (((size_t)t * n_heads + h) * nsplit + blockIdx.z) * (R + 2);
    if (lane == 0) { ps[0] = m; ps[1] = l; }
    dst = ps + 2;
  } else {
    inv = 1.0f / l;
    dst = out + ((size_t)t * n_heads + h) * R;
  }
#pragma unroll
  for (int i = 0; i < RC; ++i) {
    const int d = 4 * lane + 128 * (i >> 2) + (i & 3);
    if (d < R) dst[d] = acc[i] * inv;
  }
}

// Merges the shares of the blocks that split a token's keys, and lets the sink in (once).
__global__ void latent_merge_kernel(float* __restrict__ out, const float* __restrict__ partial,
                                    const float* __restrict__ sink,
                                    const int* __restrict__ tok_req, int n_heads, int R,
                                    int nsplit, const int* __restrict__ plan) {
  if (plan && (int)blockIdx.x >= plan[0]) return;
  const int t = plan ? plan[4 + 3 * blockIdx.x] : blockIdx.x;
  const int h = blockIdx.y;
  if (tok_req[t] < 0) return;
  const float* ps = partial + ((size_t)t * n_heads + h) * nsplit * (R + 2);
  float m = sink[h];
  for (int s = 0; s < nsplit; ++s) m = fmaxf(m, ps[(size_t)s * (R + 2)]);
  float l = expf(sink[h] - m);
  for (int s = 0; s < nsplit; ++s) {
    const float ms = ps[(size_t)s * (R + 2)];
    if (ms > -INFINITY) l += ps[(size_t)s * (R + 2) + 1] * expf(ms - m);
  }
  const float inv = 1.0f / l;
  for (int d = threadIdx.x; d < R; d += blockDim.x) {
    float a = 0.f;
    for (int s = 0; s < nsplit; ++s) {
      const float ms = ps[(size_t)s * (R + 2)];
      if (ms > -INFINITY) a = fmaf(ps[(size_t)s * (R + 2) + 2 + d], expf(ms - m), a);
    }
    out[((size_t)t * n_heads + h) * R + d] = a * inv;
  }
}

}  // namespace hs

HS_EXPORT int hs_latent_append(void* pool, const float* proj, const float* norm_w,
                               const int* table, const int* tok_pos, const int* tok_req,
                               int n_tokens, int proj_stride, int c_off, int R, int P, float eps,
                               int page_size, int num_pages, int max_pages, int cache_dtype,
                               int* status, const float* freq, int rot_dims, void* stream) {
  if (rot_dims < 0 || rot_dims % 2 || rot_dims > P || (rot_dims && !freq)) return HS_ERR_ARGUMENT;
  if (!pool || !proj || !norm_w || !table || !tok_pos || !tok_req || !status)
    return HS_ERR_ARGUMENT;
  if (R <= 0 || P < 0 || page_size <= 0) return HS_ERR_UNSUPPORTED;
  if (n_tokens <= 0) return HS_OK;
  cudaStream_t st = (cudaStream_t)stream;
  if (cache_dtype == HS_DT_F32)
    hs::latent_append_kernel<float><<<n_tokens, 128, 0, st>>>(
        (float*)pool, proj, norm_w, table, tok_pos, tok_req, proj_stride, c_off, R, P, eps,
        page_size, num_pages, max_pages, status, freq, rot_dims);
  else if (cache_dtype == HS_DT_BF16)
    hs::latent_append_kernel<__nv_bfloat16><<<n_tokens, 128, 0, st>>>(
        (__nv_bfloat16*)pool, proj, norm_w, table, tok_pos, tok_req, proj_stride, c_off, R, P,
        eps, page_size, num_pages, max_pages, status, freq, rot_dims);
  else
    return HS_ERR_UNSUPPORTED;
  HS_LAUNCH_CHECK();
  return HS_OK;
}

template <typename TC, int RC>
static int launch_latent_attention(float* out, const float* qa, const float* qr, const void* pool,
                                   const int* table, const int* tok_pos, const int* tok_req,
                                   const float* sink, int n_tokens, int n_heads, int R, int P,
                                   int qr_stride, int qr_hstride, int qr_off, float scale,
                                   int page_size, int num_pages, int max_pages, int* status,
                                   int nsplit, float* partial, const float* freq, int rot_dims,
                                   const int* plan, cudaStream_t st) {
  const int W = R + P;
  const size_t smem = ((size_t)hs::LA_HB * hs::la_w4(W) + (size_t)hs::LA_TILE * hs::la_stride(W)) *
                      sizeof(float);
  if (smem > 200 * 1024) return HS_ERR_UNSUPPORTED;
  auto kern = hs::latent_attention_kernel<TC, RC>;
  if (smem > 48 * 1024)
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  dim3 grid(n_tokens, (n_heads + hs::LA_HB - 1) / hs::LA_HB, nsplit);
  kern<<<grid, hs::LA_HB * 32, smem, st>>>(out, qa, qr, (const TC*)pool, table, tok_pos, tok_req,
                                           sink, n_heads, R, P, qr_stride, qr_hstride, qr_off,
                                           scale, page_size, num_pages, max_pages, status, nsplit,
                                           partial, freq, rot_dims, plan);
  HS_LAUNCH_CHECK();
  if (nsplit > 1) {
    hs::latent_merge_kernel<<<dim3(n_tokens, n_heads), 128, 0, st>>>(out, partial, sink, tok_req,
                                                                     n_heads, R, nsplit, plan);
    HS_LAUNCH_CHECK();
  }
  return HS_OK;
}

HS_EXPORT int hs_latent_attention(float* out, const float* qa, const float* qr, const void* pool,
                                  const int* table, const int* tok_pos, const int* tok_req,
                                  const float* sink, int n_tokens, int n_heads, int R, int P,
                                  int qr_stride, int qr_hstride, int qr_off, float scale,
                                  int page_size, int num_pages, int max_pages, int cache_dtype,
                                  int* status, int nsplit, float* partial, const float* freq,
                                  int rot_dims, const int* plan, void* stream) {
  if (nsplit < 1 || (nsplit > 1 && !partial)) return HS_ERR_ARGUMENT;
  if (rot_dims < 0 || rot_dims % 2 || rot_dims > P || (rot_dims && !freq)) return HS_ERR_ARGUMENT;
  if (!out || !qa || !qr || !pool || !table || !tok_pos || !tok_req || !sink || !status)
    return HS_ERR_ARGUMENT;
  if (R <= 0 || R > 512 || P < 0 || n_heads <= 0 || page_size <= 0) return HS_ERR_UNSUPPORTED;
  if (n_tokens <= 0) return HS_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const int rc = (R + 31) / 32;
#define HS_LA(TC, RC)                                                                         \
  return launch_latent_attention<TC, RC>(out, qa, qr, pool, table, tok_pos, tok_req, sink,    \
                                         n_tokens, n_heads, R, P, qr_stride, qr_hstride,      \
                                         qr_off, scale, page_size, num_pages, max_pages,      \
                                         status, nsplit, partial, freq, rot_dims, plan, st)
#define HS_LA_RC(TC)                   \
  do {                                 \
    if (rc <= 4) HS_LA(TC, 4);         \
    if (rc <= 8) HS_LA(TC, 8);         \
    HS_LA(TC, 16);                     \
  } while (0)
  if (cache_dtype == HS_DT_F32) HS_LA_RC(float);
  if (cache_dtype == HS_DT_BF16) HS_LA_RC(__nv_bfloat16);
#undef HS_LA_RC
#undef HS_LA
  return HS_ERR_UNSUPPORTED;
}

// Attention with a learned bias of the distance, a tanh cap on the scores, a chunked (or
// windowed) causal mask, keys normed over their whole projection and a sigmoid gate per head.
//
//   qk_prepare   per token, from a float32 projection row [.. q (H*D) .. k (G*D) .. (v) ..]:
//                    qn = q / rms(q) * wq      over ALL H*D entries at once (wq null: q as is)
//                    kn = k / rms(k) * wk      over all G*D entries
//                    v  = the value columns, or the keys as projected (before their norm)
//                qn goes to a [T, H*D] buffer in the compute type, kn and v into the token's
//                page (plane 0 and plane 1 of the cache entry).
//   attention    score(i, j) = cap * tanh((qn_i . kn_j) * scale / cap) + bias[h][i - j]
//                (cap 0: no cap; bias null: none), over the keys j <= i that lie in i's chunk
//                (floor(i / chunk) == floor(j / chunk), chunks counted from position 0) and
//                inside the window (i - j < window); softmax; out = sum_j p_j v_j, times
//                sigmoid(gate[t, h]) when a gate is given.
//
// Cache layout as the other attention kernels: pool[page][plane][kv_head][slot][d].
// One warp per (token, head): 32 keys a step, one per lane (the score is one chain of fused
// multiply-adds over d), an online softmax in float32, lane e accumulates output entries
// e, e + 32, ...  The first step starts at the first visible key, so the order of every sum
// depends on the positions alone, never on the batch, the cut of the prompt or the pages.
// This kernel serves float32, single tokens (decoding) and every size the tile kernel
// (attention_biased_mma.cu) does not take.
#include "common.cuh"

namespace hs {

struct BiasedGeom {
  int n_heads, n_kv_heads, head_dim, page_size, num_pages, max_pages;
  int chunk, window, n_dist;
  float scale, cap;
};

constexpr int QKP_THREADS = 256;

__device__ __forceinline__ float qkp_block_sum(float v, float* s_part) {
  v = warp_sum(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = v;
  __syncthreads();
  float total = 0.f;
  for (int i = 0; i < QKP_THREADS / 32; ++i) total += s_part[i];
  return total;
}

template <typename T>
__global__ void __launch_bounds__(QKP_THREADS)
qk_prepare_kernel(T* __restrict__ q_out, T* __restrict__ pool, const float* __restrict__ proj,
                  const float* __restrict__ wq, const float* __restrict__ wk,
                  const int* __restrict__ table, const int* __restrict__ tok_pos,
                  const int* __restrict__ tok_req, int stride, int q_off, int k_off, int v_off,
                  float eps, int writes, BiasedGeom g, int* status) {
  __shared__ float s_part[QKP_THREADS / 32];
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const int r = tok_req[t];
  if (r < 0) return;
  const int qw = g.n_heads * g.head_dim, kw = g.n_kv_heads * g.head_dim;
  const float* row = proj + (size_t)t * stride;
  float sq = 0.f, sk = 0.f;
  for (int e = threadIdx.x; e < qw; e += QKP_THREADS) sq = fmaf(row[q_off + e], row[q_off + e], sq);
  for (int e = threadIdx.x; e < kw; e += QKP_THREADS) sk = fmaf(row[k_off + e], row[k_off + e], sk);
  const float rq = wq ? 1.0f / sqrtf(qkp_block_sum(sq, s_part) / (float)qw + eps) : 1.0f;
  const float rk = wk ? 1.0f / sqrtf(qkp_block_sum(sk, s_part) / (float)kw + eps) : 1.0f;
  for (int e = threadIdx.x; e < qw; e += QKP_THREADS)
    q_out[(size_t)t * qw + e] = from_f<T>(wq ? row[q_off + e] * rq * wq[e] : row[q_off + e]);
  if (!writes) return;
  const int p = tok_pos[t];
  if (p < 0 || p / g.page_size >= g.max_pages) {
    if (threadIdx.x == 0) atomicOr(status, HS_STATUS_BAD_POSITION);
    return;
  }
  const int page = table[(size_t)r * g.max_pages + p / g.page_size];
  if (page < 0 || page >= g.num_pages) {
    if (threadIdx.x == 0) atomicOr(status, HS_STATUS_BAD_PAGE);
    return;
  }
  const size_t tile = (size_t)g.page_size * g.head_dim;
  T* pk = pool + (size_t)page * 2 * g.n_kv_heads * tile + (size_t)(p % g.page_size) * g.head_dim;
  T* pv = pk + (size_t)g.n_kv_heads * tile;
  const int vo = v_off >= 0 ? v_off : k_off;          // no value projection: the keys as projected
  for (int e = threadIdx.x; e < kw; e += QKP_THREADS) {
    const int hk = e / g.head_dim, d = e - hk * g.head_dim;
    const float k = row[k_off + e];
    pk[(size_t)hk * tile + d] = from_f<T>(wk ? k * rk * wk[e] : k);
    pv[(size_t)hk * tile + d] = from_f<T>(row[vo + e]);
  }
}

constexpr int BA_WARPS = 4;
constexpr int BA_MAX_D = 256;

// q . k over d = 0 .. D-1 as one chain of fused multiply-adds; 16-byte loads of the key row when
// the head size allows them (the order of the chain is the same either way)
__device__ __forceinline__ float ba_dot(const float* q, const float* k, int D) {
  float dot = 0.f;
  if ((D & 3) == 0) {
    for (int d = 0; d < D; d += 4) {
      const float4 v = *(const float4*)(k + d);
      dot = fmaf(q[d], v.x, dot); dot = fmaf(q[d + 1], v.y, dot);
      dot = fmaf(q[d + 2], v.z, dot); dot = fmaf(q[d + 3], v.w, dot);
    }
  } else {
    for (int d = 0; d < D; ++d) dot = fmaf(q[d], k[d], dot);
  }
  return dot;
}
__device__ __forceinline__ float ba_dot(const float* q, const __nv_bfloat16* k, int D) {
  float dot = 0.f;
  if ((D & 7) == 0) {
    for (int d = 0; d < D; d += 8) {
      const uint4 raw = *(const uint4*)(k + d);
      const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        dot = fmaf(q[d + 2 * i], __uint_as_float(w[i] << 16), dot);
        dot = fmaf(q[d + 2 * i + 1], __uint_as_float(w[i] & 0xffff0000u), dot);
      }
    }
  } else {
    for (int d = 0; d < D; ++d) dot = fmaf(q[d], __bfloat162float(k[d]), dot);
  }
  return dot;
}

template <typename T>
__global__ void __launch_bounds__(BA_WARPS * 32)
biased_attention_kernel(T* __restrict__ out, const T* __restrict__ q, const T* __restrict__ pool,
                        const int* __restrict__ table, const int* __restrict__ tok_pos,
                        const int* __restrict__ tok_req, const float* __restrict__ bias,
                        const float* __restrict__ gate, int g_off, int g_stride, int n_tokens,
                        const int* __restrict__ listed, const int* __restrict__ plan_head,
                        BiasedGeom g, int* status) {
  extern __shared__ __align__(16) unsigned char ba_smem[];
  float* s_q = (float*)ba_smem;                        // [BA_WARPS][head_dim]
  pdl_trigger();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int item = blockIdx.x * BA_WARPS + warp;       // (token, head) pairs, heads fastest
  // with a list (the step's single-query tokens: flat index, request row, position per entry)
  // only the listed tokens are served, as many as the list's head says
  const int n_here = listed ? min(n_tokens, plan_head[0]) : n_tokens;
  if (item >= n_here * g.n_heads) return;
  const int entry = item / g.n_heads, h = item - entry * g.n_heads;
  const int t = listed ? listed[3 * entry] : entry;
  const int r = tok_req[t];
  if (r < 0) return;
  const int D = g.head_dim;
  // the warp's 32 value rows of a step: staged by 16-byte cp.async copies (a lane fetches its own
  // key's row) while the scores are formed, then read with lane e on entries e, e + 32, ...
  T* s_v = (T*)(ba_smem + ((BA_WARPS * D * sizeof(float) + 15) & ~(size_t)15)) + (size_t)warp * 32 * D;
  const bool bulk = (D * sizeof(T)) % 16 == 0;
  const int i = tok_pos[t];
  const int hk = h / (g.n_heads / g.n_kv_heads);
  float* qs = s_q + warp * D;
  const T* qr = q + ((size_t)t * g.n_heads + h) * D;
  for (int d = lane; d < D; d += 32) qs[d] = to_f(qr[d]);
  __syncwarp();
  int lo = g.chunk > 0 ? i / g.chunk * g.chunk : 0;
  if (g.window > 0) lo = max(lo, i - g.window + 1);
  const size_t tile = (size_t)g.page_size * D;
  const float* brow = bias ? bias + (size_t)h * g.n_dist : nullptr;
  float m = -INFINITY, l = 0.f;
  float acc[BA_MAX_D / 32];
#pragma unroll
  for (int c = 0; c < BA_MAX_D / 32; ++c) acc[c] = 0.f;
  for (int j0 = lo; j0 <= i; j0 += 32) {
    const int j = j0 + lane;
    const bool live = j <= i;
    const T* krow = nullptr;
    if (live) {
      const int page = table[(size_t)r * g.max_pages + j / g.page_size];
      if (page < 0 || page >= g.num_pages) {
        atomicOr(status, HS_STATUS_BAD_PAGE);
      } else {
        krow = pool + ((size_t)page * 2 * g.n_kv_heads + hk) * tile + (size_t)(j % g.page_size) * D;
      }
    }
    __syncwarp();                                      // the step before has read its value rows
    if (krow) {
      const T* vrow = krow + (size_t)g.n_kv_heads * tile;                        // plane 1
      T* dst = s_v + (size_t)lane * D;
      if (bulk) {
        for (int b16 = 0; b16 < (int)(D * sizeof(T)); b16 += 16)
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(
                           (uint32_t)__cvta_generic_to_shared((char*)dst + b16)),
                       "l"((const char*)vrow + b16)
                       : "memory");
      } else {
        for (int d = 0; d < D; ++d) dst[d] = vrow[d];
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    float s = -INFINITY;
    if (krow) {
      s = ba_dot(qs, krow, D) * g.scale;
      if (g.cap > 0.f) s = g.cap * tanhf(s / g.cap);
      if (brow) s += brow[min(i - j, g.n_dist - 1)];
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float corr = m == -INFINITY ? 0.f : expf(m - m_new);
    const float pj = krow ? expf(s - m_new) : 0.f;
    l = l * corr + warp_sum(pj);
#pragma unroll
    for (int c = 0; c < BA_MAX_D / 32; ++c) acc[c] *= corr;
    const unsigned have = __ballot_sync(0xffffffffu, krow != nullptr);
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncwarp();                                      // every lane's row has landed
    const int n_keys = min(32, i - j0 + 1);
    for (int k = 0; k < n_keys; ++k) {
      const float pk = __shfl_sync(0xffffffffu, pj, k);
      if (!((have >> k) & 1u)) continue;
      const T* vrow = s_v + (size_t)k * D;
#pragma unroll
      for (int c = 0; c < BA_MAX_D / 32; ++c) {
        const int d = lane + 32 * c;
        if (d < D) acc[c] = fmaf(pk, to_f(vrow[d]), acc[c]);
      }
    }
    m = m_new;
  }
  float gv = 1.0f;
  if (gate) gv = 1.0f / (1.0f + expf(-gate[(size_t)t * g_stride + g_off + h]));
  const float inv = l > 0.f ? gv / l : 0.f;
  T* orow = out + ((size_t)t * g.n_heads + h) * D;
#pragma unroll
  for (int c = 0; c < BA_MAX_D / 32; ++c) {
    const int d = lane + 32 * c;
    if (d < D) orow[d] = from_f<T>(acc[c] * inv);
  }
}

}  // namespace hs

static int biased_geom_ok(const hs::BiasedGeom& g) {
  return g.n_heads > 0 && g.n_kv_heads > 0 && g.n_heads % g.n_kv_heads == 0 && g.head_dim > 0 &&
         g.head_dim <= hs::BA_MAX_D && g.page_size > 0 && g.num_pages > 0 && g.max_pages > 0 &&
         g.chunk >= 0 && g.window >= 0;
}

HS_EXPORT int hs_qk_prepare(void* q_out, void* pool, const float* proj, const float* wq,
                            const float* wk, const int* table, const int* tok_pos,
                            const int* tok_req, int n_tokens, int stride, int q_off, int k_off,
                            int v_off, float eps, int writes, int n_heads, int n_kv_heads,
                            int head_dim, int page_size, int num_pages, int max_pages, int dtype,
                            int* status, void* stream) {
  if (!q_out || !pool || !proj || !table || !tok_pos || !tok_req || !status)
    return HS_ERR_ARGUMENT;
  hs::BiasedGeom g = {n_heads, n_kv_heads, head_dim, page_size, num_pages, max_pages,
                      0, 0, 0, 1.f, 0.f};
  if (!biased_geom_ok(g) || q_off < 0 || k_off < 0) return HS_ERR_UNSUPPORTED;
  if (n_tokens <= 0) return HS_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const bool pdl = hs_pdl_enabled();
  cudaError_t e = cudaSuccess;
  if (dtype == HS_DT_F32)
    e = hs_launch(hs::qk_prepare_kernel<float>, dim3(n_tokens), dim3(hs::QKP_THREADS), 0, st, pdl,
        (float*)q_out, (float*)pool, proj, wq, wk, table, tok_pos, tok_req, stride, q_off, k_off,
        v_off, eps, writes, g, status);
  else if (dtype == HS_DT_BF16)
    e = hs_launch(hs::qk_prepare_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(hs::QKP_THREADS), 0,
        st, pdl, (__nv_bfloat16*)q_out, (__nv_bfloat16*)pool, proj, wq, wk, table, tok_pos, tok_req,
        stride, q_off, k_off, v_off, eps, writes, g, status);
  else
    return HS_ERR_UNSUPPORTED;
  return e == cudaSuccess ? HS_OK : (int)e;
}

HS_EXPORT int hs_biased_attention(void* out, const void* q, const void* pool, const int* table,
                                  const int* tok_pos, const int* tok_req, const float* bias,
                                  int n_dist, const float* gate, int g_off, int g_stride,
                                  int n_tokens, int n_heads, int n_kv_heads, int head_dim,
                                  int page_size, int num_pages, int max_pages, float scale,
                                  float cap, int chunk, int window, int dtype,
                                  const int* listed, const int* plan_head, int* status,
                                  void* stream) {
  if (!out || !q || !pool || !table || !tok_pos || !tok_req || !status) return HS_ERR_ARGUMENT;
  hs::BiasedGeom g = {n_heads, n_kv_heads, head_dim, page_size, num_pages, max_pages,
                      chunk, window, n_dist, scale, cap};
  if (!biased_geom_ok(g) || (bias && n_dist <= 0) || cap < 0.f || (listed && !plan_head))
    return HS_ERR_UNSUPPORTED;
  if (n_tokens <= 0) return HS_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const bool pdl = hs_pdl_enabled();
  cudaError_t e = cudaSuccess;
  const long long items = (long long)n_tokens * n_heads;
  const int blocks = (int)((items + hs::BA_WARPS - 1) / hs::BA_WARPS);
  const size_t esz = dtype == HS_DT_F32 ? 4 : 2;
  const size_t smem = (((size_t)hs::BA_WARPS * head_dim * sizeof(float) + 15) & ~(size_t)15) +
                      (size_t)hs::BA_WARPS * 32 * head_dim * esz;
  if (smem > 48 * 1024) {
    cudaError_t ea = dtype == HS_DT_F32
        ? cudaFuncSetAttribute(hs::biased_attention_kernel<float>,
                               cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)
        : cudaFuncSetAttribute(hs::biased_attention_kernel<__nv_bfloat16>,
                               cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (ea != cudaSuccess) return (int)ea;
  }
  if (dtype == HS_DT_F32)
    e = hs_launch(hs::biased_attention_kernel<float>, dim3(blocks), dim3(hs::BA_WARPS * 32), smem,
        st, pdl, (float*)out, (const float*)q, (const float*)pool, table, tok_pos, tok_req, bias, gate,
        g_off, g_stride, n_tokens, listed, plan_head, g, status);
  else if (dtype == HS_DT_BF16)
    e = hs_launch(hs::biased_attention_kernel<__nv_bfloat16>, dim3(blocks),
        dim3(hs::BA_WARPS * 32), smem, st, pdl, (__nv_bfloat16*)out, (const __nv_bfloat16*)q, (const __nv_bfloat16*)pool, table, tok_pos,
        tok_req, bias, gate, g_off, g_stride, n_tokens, listed, plan_head, g, status);
  else
    return HS_ERR_UNSUPPORTED;
  return e == cudaSuccess ? HS_OK : (int)e;
}

// Attention over a shared latent for prompt portions, on the tensor cores (mma.sync m16n8k16,
// bfloat16 operands, float32 accumulators).  Same mathematics as latent_attention.cu:
//
//   score(i, j) = (qa_i . c_j + qr_i . kr_j) * scale  (j <= i),  softmax with a sink per head,
//   out_lat     = sum_j weight_j c_j
//
// Because every head of a token reads the same cache rows, a block's 64 query rows are (token,
// head) pairs of consecutive tokens of ONE request: rows = token-major, head-minor, cut from a
// work tile of up to 128 queries (the step's attention plan lists those tiles).  Per 32 keys:
//   S = Q K^T      Q [64 x W] and K [32 x W] in shared memory as bfloat16 (W = R + P, padded)
//   running softmax on the accumulator fragments (rows g and g + 8 of a warp's 16)
//   O += P V       V is the first R columns of the same key rows, read transposed by ldmatrix
// Four warps own 16 rows each; with R > 256 eight warps run, the second four owning the upper
// half of the R output columns of the same rows (they form S a second time).
#include "common.cuh"
#include "rotary.cuh"

namespace hs {

constexpr int LM_ROWS = 64;     // query rows a block
constexpr int LM_KEYS = 32;     // keys a tile

__device__ __forceinline__ void mma16816(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *(uint32_t*)&v;
}

// plan: [0] single-query tokens, [1] tiles, ...; tile i at plan[tiles_off + 4 i]: first flat
// token, number of tokens, request row, position of the first token.
template <int NTM>              // accumulator tiles of 8 output columns a warp keeps (16 or 32)
__global__ void __launch_bounds__(256)
latent_prefill_mma_kernel(float* __restrict__ out, const float* __restrict__ qa,
                          const float* __restrict__ qr, const __nv_bfloat16* __restrict__ pool,
                          const int* __restrict__ table, const float* __restrict__ sink,
                          const int* __restrict__ plan, int tiles_off, int n_heads, int R, int P,
                          int qr_stride, int qr_hstride, int qr_off, float scale, int page_size,
                          int num_pages, int max_pages, int* status,
                          const float* __restrict__ freq, int rot_dims) {
  extern __shared__ __align__(16) __nv_bfloat16 sm_b[];
  if ((int)blockIdx.x >= plan[1]) return;
  const int* tile = plan + tiles_off + 4 * blockIdx.x;
  const int t_first = tile[0], n_q = tile[1], req = tile[2], pos_first = tile[3];
  const int row_lo = blockIdx.y * LM_ROWS;
  const int n_rows = n_q * n_heads;
  if (row_lo >= n_rows) return;
  const int W = R + P;
  const int W16 = (W + 15) & ~15;
  const int WS = W16 + 8;                         // row stride in elements: 16 bytes (mod 64)
  __nv_bfloat16* sQ = sm_b;                       // [LM_ROWS][WS]
  __nv_bfloat16* sK = sm_b + LM_ROWS * WS;        // [LM_KEYS][WS]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, tq = lane & 3;
  const int rg = warp & 3, dh = warp >> 2;        // row group, half of the output columns
  const int halves = blockDim.x >> 7;             // 1 or 2
  const int r_per = R / halves;                   // output columns of this warp
  const int nt_count = r_per >> 3;
  const int dim_lo = dh * r_per;

  // queries: float32 -> bfloat16, the rotated part turned on the way; rows beyond the tile zero
  for (int i = threadIdx.x; i < LM_ROWS * WS; i += blockDim.x) {
    const int rr = i / WS, d = i - rr * WS;
    const int row = row_lo + rr;
    float v = 0.f;
    if (row < n_rows && d < W) {
      const int tl = row / n_heads, head = row - tl * n_heads;
      const int t = t_first + tl;
      if (d < R) {
        v = qa[((size_t)t * n_heads + head) * R + d];
      } else {
        const float* src = qr + (size_t)t * qr_stride + (size_t)head * qr_hstride + qr_off;
        const int e = d - R;
        v = e < rot_dims ? rotate_entry(src[e], src[e ^ 1], e, rot_dims, pos_first + tl, freq)
                         : src[e];
      }
    }
    sQ[i] = __float2bfloat16_rn(v);
  }
  for (int i = threadIdx.x; i < LM_KEYS * WS; i += blockDim.x) sK[i] = __float2bfloat16_rn(0.f);

  // this thread's two rows: rg*16 + g and + 8
  int row_pos[2], row_head[2];
  bool row_ok[2];
  float m[2], l[2];
#pragma unroll
  for (int x = 0; x < 2; ++x) {
    const int row = row_lo + rg * 16 + g + 8 * x;
    row_ok[x] = row < n_rows;
    const int tl = row_ok[x] ? row / n_heads : 0;
    row_head[x] = row_ok[x] ? row - tl * n_heads : 0;
    row_pos[x] = pos_first + tl;
    m[x] = sink[row_head[x]];                     // the sink opens the running softmax
    l[x] = tq == 0 ? 1.f : 0.f;                   // its weight 1 is counted once a row
  }
  float acc_o[NTM][4];
#pragma unroll
  for (int i = 0; i < NTM; ++i)
#pragma unroll
    for (int c = 0; c < 4; ++c) acc_o[i][c] = 0.f;

  const int last_row = min(n_rows, row_lo + LM_ROWS) - 1;
  const int pos_max = pos_first + last_row / n_heads;        // the block's newest key
  const bool vec = (W & 7) == 0;
  for (int base = 0; base <= pos_max; base += LM_KEYS) {
    __syncthreads();                              // sQ is set / the tile before has been used
    const int nk = min(LM_KEYS, pos_max + 1 - base);
    for (int j = warp; j < LM_KEYS; j += (blockDim.x >> 5)) {
      __nv_bfloat16* dst = sK + j * WS;
      const int kp = base + j;
      const int pi = kp / page_size;
      int page = -1;
      if (j < nk) {
        page = pi < max_pages ? table[(size_t)req * max_pages + pi] : -1;
        if (page < 0 || page >= num_pages) {
          if (lane == 0) atomicOr(status, HS_STATUS_BAD_PAGE);
          page = -1;
        }
      }
      if (page < 0) {
        for (int d = lane; d < W; d += 32) dst[d] = __float2bfloat16_rn(0.f);
      } else {
        const __nv_bfloat16* src = pool + ((size_t)page * page_size + (kp % page_size)) * W;
        if (vec) {
          for (int d = lane * 8; d < W; d += 256) *(uint4*)(dst + d) = *(const uint4*)(src + d);
        } else {
          for (int d = lane; d < W; d += 32) dst[d] = src[d];
        }
      }
    }
    __syncthreads();
    // S = Q K^T for this warp's 16 rows x 32 keys
    float acc_s[4][4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc_s[j][c] = 0.f;
    const __nv_bfloat16* qrow = sQ + (rg * 16 + g) * WS + 2 * tq;
    const __nv_bfloat16* krow = sK + g * WS + 2 * tq;
    for (int kk = 0; kk < W16; kk += 16) {
      uint32_t a[4];
      a[0] = *(const uint32_t*)(qrow + kk);
      a[1] = *(const uint32_t*)(qrow + 8 * WS + kk);
      a[2] = *(const uint32_t*)(qrow + kk + 8);
      a[3] = *(const uint32_t*)(qrow + 8 * WS + kk + 8);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const __nv_bfloat16* p = krow + 8 * j * WS + kk;
        mma16816(acc_s[j], a, *(const uint32_t*)p, *(const uint32_t*)(p + 8));
      }
    }
    // mask, scale, running softmax on rows g (values 0, 1) and g + 8 (values 2, 3)
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int x = c >> 1;
        const int kp = base + 8 * j + 2 * tq + (c & 1);
        const bool ok = row_ok[x] && kp <= row_pos[x];
        acc_s[j][c] = ok ? acc_s[j][c] * scale : -INFINITY;
        mx[x] = fmaxf(mx[x], acc_s[j][c]);
      }
    float corr[2];
#pragma unroll
    for (int x = 0; x < 2; ++x) {
      mx[x] = fmaxf(mx[x], __shfl_xor_sync(0xffffffffu, mx[x], 1));
      mx[x] = fmaxf(mx[x], __shfl_xor_sync(0xffffffffu, mx[x], 2));
      const float m_new = fmaxf(m[x], mx[x]);
      corr[x] = expf(m[x] - m_new);
      m[x] = m_new;
      l[x] *= corr[x];
    }
    uint32_t pa[2][4];                            // P as the A operand of two steps of 16 keys
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float p0 = expf(acc_s[j][0] - m[0]), p1 = expf(acc_s[j][1] - m[0]);
      const float p2 = expf(acc_s[j][2] - m[1]), p3 = expf(acc_s[j][3] - m[1]);
      l[0] += p0 + p1;
      l[1] += p2 + p3;
      pa[j >> 1][(j & 1) * 2] = pack_bf16(p0, p1);
      pa[j >> 1][(j & 1) * 2 + 1] = pack_bf16(p2, p3);
    }
    // O = O * corr + P V; V = key rows' first R columns, columns dim_lo .. of this warp
    const uint32_t k_addr = (uint32_t)__cvta_generic_to_shared(sK + lane * WS + dim_lo);
#pragma unroll
    for (int nt = 0; nt < NTM; ++nt) {
      if (nt < nt_count) {
        acc_o[nt][0] *= corr[0]; acc_o[nt][1] *= corr[0];
        acc_o[nt][2] *= corr[1]; acc_o[nt][3] *= corr[1];
        uint32_t b0, b1, b2, b3;
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                     : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3)
                     : "r"(k_addr + (uint32_t)(nt * 8 * sizeof(__nv_bfloat16))));
        mma16816(acc_o[nt], pa[0], b0, b1);
        mma16816(acc_o[nt], pa[1], b2, b3);
      }
    }
  }
  // the denominators: each thread summed its own columns
#pragma unroll
  for (int x = 0; x < 2; ++x) {
    l[x] += __shfl_xor_sync(0xffffffffu, l[x], 1);
    l[x] += __shfl_xor_sync(0xffffffffu, l[x], 2);
  }
#pragma unroll
  for (int x = 0; x < 2; ++x) {
    if (!row_ok[x]) continue;
    const int row = row_lo + rg * 16 + g + 8 * x;
    const int t = t_first + row / n_heads;
    float* dst = out + ((size_t)t * n_heads + row_head[x]) * R + dim_lo + 2 * tq;
    const float inv = 1.0f / l[x];
#pragma unroll
    for (int nt = 0; nt < NTM; ++nt)
      if (nt < nt_count) {
        dst[8 * nt] = acc_o[nt][2 * x] * inv;
        dst[8 * nt + 1] = acc_o[nt][2 * x + 1] * inv;
      }
  }
}

}  // namespace hs

// Returns HS_ERR_UNSUPPORTED for sizes the kernel does not take (the caller then uses the
// CUDA-core kernel): R a multiple of 16 up to 512, the shared tiles within 200 KB.
HS_EXPORT int hs_latent_prefill_mma(float* out, const float* qa, const float* qr,
                                    const void* pool, const int* table, const float* sink,
                                    const int* plan, int tiles_off, int tile_cap, int n_heads,
                                    int R, int P, int qr_stride, int qr_hstride, int qr_off,
                                    float scale, int page_size, int num_pages, int max_pages,
                                    int* status, const float* freq, int rot_dims, void* stream) {
  if (!out || !qa || !qr || !pool || !table || !sink || !plan || !status) return HS_ERR_ARGUMENT;
  if (rot_dims < 0 || rot_dims % 2 || rot_dims > P || (rot_dims && !freq)) return HS_ERR_ARGUMENT;
  if (R <= 0 || R % 16 || R > 512 || P < 0 || n_heads <= 0 || page_size <= 0)
    return HS_ERR_UNSUPPORTED;
  const int W16 = (R + P + 15) & ~15;
  const size_t smem = (size_t)(hs::LM_ROWS + hs::LM_KEYS) * (W16 + 8) * sizeof(__nv_bfloat16);
  if (smem > 200 * 1024) return HS_ERR_UNSUPPORTED;
  if (tile_cap <= 0) return HS_OK;
  const int halves = R > 256 ? 2 : 1;
  const int per = R / halves;
  dim3 grid(tile_cap, (128 * n_heads + hs::LM_ROWS - 1) / hs::LM_ROWS);
  cudaStream_t st = (cudaStream_t)stream;
#define HS_LM(NTM)                                                                             \
  do {                                                                                         \
    auto kern = hs::latent_prefill_mma_kernel<NTM>;                                            \
    if (smem > 48 * 1024)                                                                      \
      cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);      \
    kern<<<grid, 128 * halves, smem, st>>>(out, qa, qr, (const __nv_bfloat16*)pool, table,     \
                                           sink, plan, tiles_off, n_heads, R, P, qr_stride,    \
                                           qr_hstride, qr_off, scale, page_size, num_pages,    \
                                           max_pages, status, freq, rot_dims);                 \
  } while (0)
  if (per <= 128) HS_LM(16);
  else HS_LM(32);
#undef HS_LM
  HS_LAUNCH_CHECK();
  return HS_OK;
}

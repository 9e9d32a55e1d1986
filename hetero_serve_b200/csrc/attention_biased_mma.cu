// Prompt portions of the attention with a distance bias, a score cap and a chunked (or windowed)
// causal mask, on the tensor cores (bfloat16; head sizes 16 to 128 in steps of 16).
//
// The tiling is that of the plain causal prefill kernel of this library (attention_prefill.cu): a
// work item is up to 128 consecutive queries of one request x one head, 8 warps of 16 queries,
// persistent CTAs that take items from a counter, keys and values 64 positions at a time through
// the block table into a ring of three cp.async stages, S = Q K^T and O += P V on mma.sync
// m16n8k16 with float32 accumulators, an online softmax in float32.  What differs:
//   * the queries come from a buffer of their own ([T, heads * D], already normed);
//   * a score is cap * tanh(s * scale / cap) + bias[h][i - j], formed in float32 on the
//     accumulator (tanh as 1 - 2 / (1 + e^2x), the head's bias row staged in shared memory);
//   * a row sees the keys lo(i) <= j <= i with lo(i) the start of i's chunk (chunks counted
//     from position 0) or of its window; the walk over the key tiles starts at the tile that
//     holds lo of the item's first query, and a warp skips tiles none of its rows can see;
//   * the head's output is multiplied by sigmoid(gate[t, h]) on the way out.
#include "common.cuh"

namespace hs {

constexpr int BP_BQ = 128, BP_BKV = 64, BP_WARPS = 8, BP_STAGES = 3;
constexpr int BP_MAX_BIAS = 4096;      // distances staged in shared memory

struct BiasedPrefillParams {
  const __nv_bfloat16* q;
  const __nv_bfloat16* pool;
  __nv_bfloat16* out;
  const int* table;
  const int* tile_info;    // per tile: first query's flat index, queries, request row, first position
  const int* plan_head;
  const float* bias;       // [heads, n_dist] or null
  const float* gate;       // rows of g_stride floats, head h at g_off + h; or null
  int* status;
  int* work_counter;       // next work item; zero at launch
  int n_heads, n_kv_heads, page_size, num_pages, max_pages;
  int ps_log2;             // log2(page_size) when it is a power of two, else -1
  int chunk, window, n_dist, g_off, g_stride;
  float scale, cap;
};

template <int D>
__device__ __forceinline__ int swz(int row, int chunk) {
  constexpr int CPR = D / 8;                       // 16-byte chunks per row
  constexpr int RPL = CPR >= 8 ? 1 : (8 / CPR > 0 ? 8 / CPR : 1);   // rows per 128-byte line
  // chunks are permuted inside groups of 8, or of the largest power of two that divides a row
  // (head sizes 48, 80, 96, 112: groups of 2 or 4, some bank conflicts, the same result)
  constexpr int GROUP = CPR % 8 == 0 ? 8 : (CPR % 4 == 0 ? 4 : (CPR % 2 == 0 ? 2 : 1));
  return row * CPR + (chunk ^ ((row / RPL) & (GROUP - 1)));
}

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* smem) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(s));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], const void* smem) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(s));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                         uint32_t b1) {
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


__device__ __forceinline__ int bp_first_key(int i, int chunk, int window) {
  int lo = chunk > 0 ? i / chunk * chunk : 0;
  if (window > 0) lo = max(lo, i - window + 1);
  return lo;
}

// cap * tanh(x / cap) in float32 (cap 0: x)
__device__ __forceinline__ float bp_cap(float x, float cap, float two_over_cap_l2) {
  if (cap <= 0.f) return x;
  const float e = exp2f(x * two_over_cap_l2);            // e^(2 x / cap)
  return cap * (1.0f - __fdividef(2.0f, 1.0f + e));
}

template <int D>
__global__ void __launch_bounds__(BP_WARPS * 32, (D <= 64 ? 2 : 1))
biased_prefill_kernel(const BiasedPrefillParams p) {
  constexpr int CPR = D / 8;
  constexpr int KSTEPS = D / 16;       // k-steps of Q K^T
  constexpr int DT = D / 8;            // n-tiles of the output
  extern __shared__ __align__(128) uint8_t smem_raw[];
  uint4* sQ = (uint4*)smem_raw;                          // [128][CPR]
  uint4* sK = sQ + BP_BQ * CPR;                          // [BP_STAGES][64][CPR]
  uint4* sV = sK + BP_STAGES * BP_BKV * CPR;             // [BP_STAGES][64][CPR]
  float* sB = (float*)(sV + BP_STAGES * BP_BKV * CPR);   // [min(n_dist, BP_MAX_BIAS)]

  __shared__ int s_item;
  pdl_trigger();
  pdl_wait();
  const int n_items = p.plan_head[1] * p.n_heads;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int n_bias = p.bias ? min(p.n_dist, BP_MAX_BIAS) : 0;
  const float LOG2E = 1.4426950408889634f;
  const float two_over_cap_l2 = p.cap > 0.f ? 2.0f / p.cap * LOG2E : 0.f;
  while (true) {
  __syncthreads();            // the previous item's shared memory has been consumed
  if (threadIdx.x == 0) s_item = atomicAdd(p.work_counter, 1);
  __syncthreads();
  const int item = s_item;
  if (item >= n_items) break;
  const int tile = item / p.n_heads, h = item - tile * p.n_heads;
  const int4 ti = *(const int4*)(p.tile_info + 4 * tile);
  const int tok0 = ti.x, nq = ti.y, r = ti.z, pos0 = ti.w;
  if (r < 0 || nq <= 0 || pos0 < 0) continue;
  const int pos_last = pos0 + nq - 1;
  if (pos_last / p.page_size >= p.max_pages) {
    if (threadIdx.x == 0) atomicOr(p.status, HS_STATUS_BAD_POSITION);
    continue;
  }
  const int hk = h / (p.n_heads / p.n_kv_heads);
  const int PS = p.page_size;
  const size_t ptile = (size_t)PS * D;
  const size_t page_stride = 2 * (size_t)p.n_kv_heads * ptile;
  const int* trow = p.table + (size_t)r * p.max_pages;
  const uint4 zero4 = make_uint4(0, 0, 0, 0);

  // ---- Q tile and the head's bias row -> shared memory (rows past nq are zero)
  for (int c = threadIdx.x; c < BP_BQ * CPR; c += blockDim.x) {
    const int row = c / CPR, ch = c % CPR;
    uint4 v = zero4;
    if (row < nq)
      v = *(const uint4*)(p.q + ((size_t)(tok0 + row) * p.n_heads + h) * D + ch * 8);
    sQ[swz<D>(row, ch)] = v;
  }
  for (int c = threadIdx.x; c < n_bias; c += blockDim.x) sB[c] = p.bias[(size_t)h * p.n_dist + c];
  const float* gbias = p.bias ? p.bias + (size_t)h * p.n_dist : nullptr;

  // keys before the first key the item's first query sees are never read: their pages may have
  // been given back already (the rows of such a tile's head are filled with zeros)
  const int key_lo = bp_first_key(pos0, p.chunk, p.window);
  const int kt_first = key_lo / BP_BKV;
  const int kt_end = pos_last / BP_BKV + 1;
  auto load_tile = [&](int kt, int stage) {
    uint4* dK = sK + stage * BP_BKV * CPR;
    uint4* dV = sV + stage * BP_BKV * CPR;
    for (int c = threadIdx.x; c < BP_BKV * CPR; c += blockDim.x) {
      const int row = c / CPR, ch = c % CPR;
      const int j = kt * BP_BKV + row;
      const int dst = swz<D>(row, ch);
      bool ok = j <= pos_last && j >= key_lo;
      int page = 0;
      int slot_in_page = 0;
      if (ok) {
        const int pg = p.ps_log2 >= 0 ? (j >> p.ps_log2) : (j / PS);
        slot_in_page = j - pg * PS;
        page = trow[pg];
        if (page < 0 || page >= p.num_pages) {
          atomicOr(p.status, HS_STATUS_BAD_PAGE);
          ok = false;
        }
      }
      if (ok) {
        const __nv_bfloat16* kp = p.pool + (size_t)page * page_stride + (size_t)hk * ptile +
                                  (size_t)slot_in_page * D + ch * 8;
        cp_async16(&dK[dst], kp);
        cp_async16(&dV[dst], kp + (size_t)p.n_kv_heads * ptile);
      } else {
        dK[dst] = zero4;
        dV[dst] = zero4;
      }
    }
  };

  // the first BP_STAGES-1 tiles are requested up front; one commit group per tile (empty ones too)
#pragma unroll
  for (int st = 0; st < BP_STAGES - 1; ++st) {
    if (kt_first + st < kt_end) load_tile(kt_first + st, st);
    cp_async_commit();
  }
  __syncthreads();          // Q and the bias row are in shared memory

  // ---- Q fragments stay in registers
  uint32_t qf[KSTEPS][4];
#pragma unroll
  for (int ks = 0; ks < KSTEPS; ++ks)
    ldsm_x4(qf[ks], &sQ[swz<D>(warp * 16 + (lane & 15), ks * 2 + (lane >> 4))]);

  float o[DT][4];
#pragma unroll
  for (int i = 0; i < DT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;
  const int row_a = warp * 16 + g, row_b = row_a + 8;
  const int pos_a = min(pos0 + row_a, pos_last), pos_b = min(pos0 + row_b, pos_last);
  const int lo_a = bp_first_key(pos_a, p.chunk, p.window);
  const int lo_b = bp_first_key(pos_b, p.chunk, p.window);
  // the keys any query of this warp sees: from lo of its first row to its last row's position;
  // a warp whose rows are all past nq sees nothing
  const int warp_last = (warp * 16 < nq) ? min(pos0 + warp * 16 + 15, pos_last) : -1;
  const int warp_lo = bp_first_key(min(pos0 + warp * 16, pos_last), p.chunk, p.window);

  for (int kt = kt_first; kt < kt_end; ++kt) {
    const int stage = (kt - kt_first) % BP_STAGES;
    cp_async_wait<BP_STAGES - 2>();     // tile kt has landed (for this thread's copies)
    __syncthreads();                    // ... for everyone's; and tile kt-1 has been consumed
    if (kt + BP_STAGES - 1 < kt_end)
      load_tile(kt + BP_STAGES - 1, (kt - kt_first + BP_STAGES - 1) % BP_STAGES);
    cp_async_commit();
    if (kt * BP_BKV <= warp_last && kt * BP_BKV + BP_BKV - 1 >= warp_lo) {
      const uint4* tK = sK + stage * BP_BKV * CPR;
      const uint4* tV = sV + stage * BP_BKV * CPR;
      float s[8][4];
#pragma unroll
      for (int i = 0; i < 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
      for (int ks = 0; ks < KSTEPS; ++ks) {
#pragma unroll
        for (int np = 0; np < 4; ++np) {           // pairs of 8-key tiles
          uint32_t b[4];
          const int mi = lane >> 3;
          const int key = np * 16 + (mi >> 1) * 8 + (lane & 7);
          ldsm_x4(b, &tK[swz<D>(key, ks * 2 + (mi & 1))]);
          mma_bf16(s[np * 2], qf[ks], b[0], b[1]);
          mma_bf16(s[np * 2 + 1], qf[ks], b[2], b[3]);
        }
      }
      // the score proper (scale, cap, bias), in units of log2(e); the mask; the running maximum
      float mx_a = -INFINITY, mx_b = -INFINITY;
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int j = kt * BP_BKV + nt * 8 + t * 2 + (c & 1);
          const int i = c < 2 ? pos_a : pos_b;
          const int lo = c < 2 ? lo_a : lo_b;
          float v = -INFINITY;
          if (j <= i && j >= lo) {
            v = bp_cap(s[nt][c] * p.scale, p.cap, two_over_cap_l2);
            if (gbias) {
              const int dist = min(i - j, p.n_dist - 1);
              v += dist < n_bias ? sB[dist] : gbias[dist];
            }
            v *= LOG2E;
          }
          s[nt][c] = v;
        }
        mx_a = fmaxf(mx_a, fmaxf(s[nt][0], s[nt][1]));
        mx_b = fmaxf(mx_b, fmaxf(s[nt][2], s[nt][3]));
      }
      mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
      mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
      mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
      mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
      const float mn_a = fmaxf(m_a, mx_a), mn_b = fmaxf(m_b, mx_b);
      // a row whose keys of this tile are all masked keeps its state (mn == m); a row with
      // no key at all yet (mn == -inf) contributes zeros
      const float ca = (mn_a == -INFINITY) ? 1.f : exp2f(m_a - mn_a);
      const float cb = (mn_b == -INFINITY) ? 1.f : exp2f(m_b - mn_b);
      const float base_a = (mn_a == -INFINITY) ? 0.f : mn_a;
      const float base_b = (mn_b == -INFINITY) ? 0.f : mn_b;
      float sum_a = 0.f, sum_b = 0.f;
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        s[nt][0] = exp2f(s[nt][0] - base_a);
        s[nt][1] = exp2f(s[nt][1] - base_a);
        s[nt][2] = exp2f(s[nt][2] - base_b);
        s[nt][3] = exp2f(s[nt][3] - base_b);
        sum_a += s[nt][0] + s[nt][1];
        sum_b += s[nt][2] + s[nt][3];
      }
      l_a = l_a * ca + sum_a;
      l_b = l_b * cb + sum_b;
      m_a = mn_a;
      m_b = mn_b;
#pragma unroll
      for (int i = 0; i < DT; ++i) {
        o[i][0] *= ca; o[i][1] *= ca; o[i][2] *= cb; o[i][3] *= cb;
      }
      // O += P V, 16 keys per k-step
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        uint32_t a[4];
        a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
        a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
        a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
        a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
        for (int dp = 0; dp < DT / 2; ++dp) {      // pairs of 8-wide output tiles
          uint32_t b[4];
          const int mi = lane >> 3;
          const int key = kk * 16 + (mi & 1) * 8 + (lane & 7);
          ldsm_x4_t(b, &tV[swz<D>(key, dp * 2 + (mi >> 1))]);
          mma_bf16(o[dp * 2], a, b[0], b[1]);
          mma_bf16(o[dp * 2 + 1], a, b[2], b[3]);
        }
      }
    }
  }
  cp_async_wait<0>();
  // ---- finish: the per-thread sums cover 2 of a row's 8 columns per tile; add the quad
  l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
  l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
  l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
  l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
  float ia = l_a > 0.f ? 1.f / l_a : 0.f, ib = l_b > 0.f ? 1.f / l_b : 0.f;
  if (p.gate) {
    if (row_a < nq)
      ia *= 1.0f / (1.0f + expf(-p.gate[(size_t)(tok0 + row_a) * p.g_stride + p.g_off + h]));
    if (row_b < nq)
      ib *= 1.0f / (1.0f + expf(-p.gate[(size_t)(tok0 + row_b) * p.g_stride + p.g_off + h]));
  }
  __nv_bfloat16* oa = p.out + ((size_t)(tok0 + row_a) * p.n_heads + h) * D;
  __nv_bfloat16* ob = p.out + ((size_t)(tok0 + row_b) * p.n_heads + h) * D;
#pragma unroll
  for (int i = 0; i < DT; ++i) {
    const int d = i * 8 + t * 2;
    if (row_a < nq) *(uint32_t*)(oa + d) = pack_bf16(o[i][0] * ia, o[i][1] * ia);
    if (row_b < nq) *(uint32_t*)(ob + d) = pack_bf16(o[i][2] * ib, o[i][3] * ib);
  }
  }   // next work item
}

template <int D>
static int launch_biased_prefill(const BiasedPrefillParams& p, cudaStream_t st) {
  auto kern = biased_prefill_kernel<D>;
  const int n_bias = p.bias ? (p.n_dist < BP_MAX_BIAS ? p.n_dist : BP_MAX_BIAS) : 0;
  const int smem = (BP_BQ + 2 * BP_STAGES * BP_BKV) * D * 2 + n_bias * 4;
  static int ctas = 0, smem_set = 0;   // persistent CTAs: as many as are resident at once
  if (smem > smem_set && smem > 40 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    smem_set = smem;
    ctas = 0;
  }
  if (ctas == 0) {
    int per_sm = 0;
    cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, BP_WARPS * 32,
                                                                  smem);
    if (e != cudaSuccess) return (int)e;
    if (per_sm < 1) per_sm = 1;
    if (per_sm > 2) per_sm = 2;
    ctas = per_sm * hs_sm_count();
  }
  cudaError_t e = cudaMemsetAsync(p.work_counter, 0, sizeof(int), st);
  if (e != cudaSuccess) return (int)e;
  e = hs_launch(kern, dim3(ctas), dim3(BP_WARPS * 32), (size_t)smem, st, hs_pdl_enabled(), p);
  return e == cudaSuccess ? HS_OK : (int)e;
}

}  // namespace hs

// The tiles of the step's work list (prompt portions): tile_info as the plain prefill kernel's.
HS_EXPORT int hs_biased_attention_prefill(void* out, const void* q, const void* pool,
                                          const int* table, const int* tile_info,
                                          const int* plan_head, int tile_cap, int* work_counter,
                                          const float* bias, int n_dist, const float* gate,
                                          int g_off, int g_stride, int n_heads, int n_kv_heads,
                                          int head_dim, int page_size, int num_pages,
                                          int max_pages, float scale, float cap, int chunk,
                                          int window, int* status, void* stream) {
  using namespace hs;
  if (!out || !q || !pool || !table || !tile_info || !plan_head || !status || !work_counter)
    return HS_ERR_ARGUMENT;
  if (tile_cap <= 0) return HS_OK;
  if (n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads || n_heads > 65535)
    return HS_ERR_UNSUPPORTED;
  if (page_size <= 0 || page_size % 16 || chunk < 0 || window < 0 || cap < 0.f ||
      (bias && n_dist <= 0))
    return HS_ERR_UNSUPPORTED;
  BiasedPrefillParams p;
  p.q = (const __nv_bfloat16*)q; p.pool = (const __nv_bfloat16*)pool;
  p.out = (__nv_bfloat16*)out; p.table = table; p.tile_info = tile_info; p.plan_head = plan_head;
  p.bias = bias; p.gate = gate; p.status = status; p.work_counter = work_counter;
  p.ps_log2 = (page_size & (page_size - 1)) == 0 ? __builtin_ctz(page_size) : -1;
  p.n_heads = n_heads; p.n_kv_heads = n_kv_heads; p.page_size = page_size;
  p.num_pages = num_pages; p.max_pages = max_pages;
  p.chunk = chunk; p.window = window; p.n_dist = n_dist; p.g_off = g_off; p.g_stride = g_stride;
  p.scale = scale; p.cap = cap;
  cudaStream_t st = (cudaStream_t)stream;
  switch (head_dim) {
    case 16: return launch_biased_prefill<16>(p, st);
    case 32: return launch_biased_prefill<32>(p, st);
    case 48: return launch_biased_prefill<48>(p, st);
    case 64: return launch_biased_prefill<64>(p, st);
    case 80: return launch_biased_prefill<80>(p, st);
    case 96: return launch_biased_prefill<96>(p, st);
    case 112: return launch_biased_prefill<112>(p, st);
    case 128: return launch_biased_prefill<128>(p, st);
    default: return HS_ERR_UNSUPPORTED;
  }
}

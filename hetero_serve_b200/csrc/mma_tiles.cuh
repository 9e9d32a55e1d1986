// Pieces of the mma.sync tile kernels (routed experts, block-diagonal linear): 64 x 64 output
// tiles, steps of 32 over the summed index, bfloat16 operands in shared memory with a row stride
// of 80 bytes (ldmatrix reads of eight rows then touch every bank once), float32 accumulators.
#pragma once
#include "common.cuh"

namespace hs {

constexpr int TM = 64, TN = 64, TK = 32;     // tile of pairs x outputs, step over the summed index
constexpr int TS = TK + 8;                   // shared row stride in elements (80 bytes)

__device__ __forceinline__ void mma_bf16(float* c, const uint32_t* a, const uint32_t* b) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

// Copies a [64 rows x 32] bfloat16 tile into shared memory asynchronously: thread i takes the
// 16-byte pieces i and i + 128 (piece c: row c / 4, columns 8 (c % 4) ..).  Rows at or beyond
// `rows` are filled with zeros (a copy of zero source bytes).  `row_ptr(r)` gives the start of
// row r; `any` is some valid address for the rows that are not read.
template <typename RowPtr>
__device__ __forceinline__ void tile_copy(__nv_bfloat16* s, RowPtr row_ptr, int rows, int k0,
                                          const __nv_bfloat16* any) {
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const int c = threadIdx.x + 128 * j;
    const int r = c >> 2, col = (c & 3) * 8;
    const bool ok = r < rows;
    const __nv_bfloat16* src = ok ? row_ptr(r) + k0 + col : any;
    const unsigned dst = (unsigned)__cvta_generic_to_shared(s + r * TS + col);
    const int bytes = ok ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes));
  }
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t* r, const __nv_bfloat16* p) {
  const unsigned a = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(a));
}

}  // namespace hs

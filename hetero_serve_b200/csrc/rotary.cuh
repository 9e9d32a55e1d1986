// Rotary positions on interleaved pairs: the pair (v[2i], v[2i+1]) at position p turns by the
// angle p * f_i.  The angle is formed in double and reduced to [0, 2 pi) there, so that its
// error does not grow with the position; the table f comes from the host, formed in double.
#pragma once
#include "common.cuh"

namespace hs {

__device__ __forceinline__ void pair_angle(int p, float f, float* c, float* s) {
  const double two_pi = 6.283185307179586476925286766559;
  double a = (double)p * (double)f;
  a -= two_pi * floor(a / two_pi);
  sincosf((float)a, s, c);
}

// entry d of a vector whose first `dims` entries are rotated; `partner` is entry d ^ 1
__device__ __forceinline__ float rotate_entry(float own, float partner, int d, int dims, int p,
                                              const float* __restrict__ freq) {
  if (d >= dims) return own;
  float c, s;
  pair_angle(p, freq[d >> 1], &c, &s);
  return (d & 1) ? own * c + partner * s : own * c - partner * s;
}

}  // namespace hs

// SRHT normalise-rotate of one 128-vector spread over 8 lanes (16 dimensions per lane), shared by the key
// coder, the query preparation and the fused ranking kernel.  Fixed fp32 operation order.
#pragma once
#include "common.cuh"

namespace pk {
namespace {

constexpr unsigned FULL = 0xffffffffu;

// x: 16 bf16 values (as floats) of dims [16s, 16s+16) of one vector; sg: the SRHT signs of those dims.
// On return x holds the rotated, scaled, bf16-rounded coordinates; the return value is the bf16 norm.
__device__ __forceinline__ float rotate16(float (&x)[16], const float (&sg)[16], int s) {
  float t[16];
#pragma unroll
  for (int i = 0; i < 16; i++) t[i] = __fmul_rn(x[i], x[i]);
#pragma unroll
  for (int w = 16; w > 1; w >>= 1)
#pragma unroll
    for (int i = 0; i < w / 2; i++) t[i] = __fadd_rn(t[2 * i], t[2 * i + 1]);
  float sum = t[0];
#pragma unroll
  for (int off = 1; off < 8; off <<= 1) sum = __fadd_rn(sum, __shfl_xor_sync(FULL, sum, off));
  const float n = bfround(__fsqrt_rn(sum));
  const float den = fmaxf(n, bfround(1e-8f));
#pragma unroll
  for (int i = 0; i < 16; i++) x[i] = __fmul_rn(bfround(__fdiv_rn(x[i], den)), sg[i]);
#pragma unroll
  for (int h = 1; h < 16; h <<= 1)
#pragma unroll
    for (int i = 0; i < 16; i++)
      if ((i & h) == 0) {
        float a = x[i], b = x[i + h];
        x[i] = __fadd_rn(a, b);
        x[i + h] = __fsub_rn(a, b);
      }
#pragma unroll
  for (int bit = 1; bit < 8; bit <<= 1)
#pragma unroll
    for (int i = 0; i < 16; i++) {
      float p = __shfl_xor_sync(FULL, x[i], bit);
      x[i] = (s & bit) ? __fsub_rn(p, x[i]) : __fadd_rn(x[i], p);
    }
#pragma unroll
  for (int i = 0; i < 16; i++) x[i] = bfround(__fmul_rn(x[i], 0.08838834764831845f));
  return n;
}

__device__ __forceinline__ void unpack8(uint4 v, float* out) {
  uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; i++) {
    out[2 * i] = __uint_as_float(w[i] << 16);
    out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}

}  // namespace
}  // namespace pk

// The elementwise steps of a decoder layer that sit between the projections and the cache calls of a decode step:
// q/k RMS-norm + rotate-half RoPE, residual add + RMS-norm, and the gated activation.  One launch each, rows of one
// token per sequence.  They are not retrieval operators (the reference takes them from its attention library,
// model_hub/qwen.py:381 silu_and_mul, :405 and :429 rmsnorm, :482 the rotary embedding); they are here because a
// decode step of 36 layers is launch-latency bound outside the host-link fetch, and every separate elementwise
// launch between two cache calls costs as much as the collision count itself.
#include "common.cuh"

namespace pk {
namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
  return v;
}

// One warp per (sequence, head) of the first Hq + Hk heads of a fused q/k/v row; lane L holds dims 4L .. 4L+3, whose
// rotate-half partners (d xor 64) sit in lane L xor 16.
//   y   = bf16( x * rsqrt(mean(x^2) + eps) * w[head] )
//   out = bf16( y * cos + y[d xor 64] * sin )            (the sign of rotate-half is folded into sin by the caller)
__global__ void __launch_bounds__(128) qk_norm_rope_kernel(const uint16_t* __restrict__ qkv, int64_t row_stride,
                                                           const uint16_t* __restrict__ w, const uint16_t* __restrict__ cosv,
                                                           const uint16_t* __restrict__ sinv, int64_t cs_stride,
                                                           uint16_t* __restrict__ out, int heads, int64_t n_warps, float eps) {
  pdl_wait();
  pdl_trigger();
  const int64_t wid = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (wid >= n_warps) return;
  const int lane = threadIdx.x & 31;
  const int64_t b = wid / heads;
  const int hd = (int)(wid % heads);
  const uint2 raw = *reinterpret_cast<const uint2*>(qkv + b * row_stride + (int64_t)hd * 128 + 4 * lane);
  float x[4] = {__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xffff0000u), __uint_as_float(raw.y << 16),
                __uint_as_float(raw.y & 0xffff0000u)};
  const float ss = warp_sum(x[0] * x[0] + x[1] * x[1] + x[2] * x[2] + x[3] * x[3]);
  const float rstd = rsqrtf(ss * (1.0f / 128.0f) + eps);
  const uint2 wr = *reinterpret_cast<const uint2*>(w + (int64_t)hd * 128 + 4 * lane);
  const float wf[4] = {__uint_as_float(wr.x << 16), __uint_as_float(wr.x & 0xffff0000u), __uint_as_float(wr.y << 16),
                       __uint_as_float(wr.y & 0xffff0000u)};
  float y[4], yr[4];
#pragma unroll
  for (int i = 0; i < 4; i++) y[i] = bfround(x[i] * rstd * wf[i]);
#pragma unroll
  for (int i = 0; i < 4; i++) yr[i] = __shfl_xor_sync(0xffffffffu, y[i], 16);
  const uint2 cr = *reinterpret_cast<const uint2*>(cosv + b * cs_stride + 4 * lane);
  const uint2 sr = *reinterpret_cast<const uint2*>(sinv + b * cs_stride + 4 * lane);
  const float cf[4] = {__uint_as_float(cr.x << 16), __uint_as_float(cr.x & 0xffff0000u), __uint_as_float(cr.y << 16),
                       __uint_as_float(cr.y & 0xffff0000u)};
  const float sf[4] = {__uint_as_float(sr.x << 16), __uint_as_float(sr.x & 0xffff0000u), __uint_as_float(sr.y << 16),
                       __uint_as_float(sr.y & 0xffff0000u)};
  uint16_t o[4];
#pragma unroll
  for (int i = 0; i < 4; i++) o[i] = f2bf(fmaf(y[i], cf[i], yr[i] * sf[i]));
  uint2 ov;
  ov.x = (uint32_t)o[0] | ((uint32_t)o[1] << 16);
  ov.y = (uint32_t)o[2] | ((uint32_t)o[3] << 16);
  *reinterpret_cast<uint2*>(out + wid * 128 + 4 * lane) = ov;
}

// One block per row: h = bf16(a + r) (r optional), x = bf16( h * rsqrt(mean(h^2) + eps) * w ).
__global__ void __launch_bounds__(512) add_rmsnorm_kernel(const uint16_t* __restrict__ a, const uint16_t* __restrict__ r,
                                                          const uint16_t* __restrict__ w, uint16_t* __restrict__ h_out,
                                                          uint16_t* __restrict__ x_out, int n, float eps) {
  pdl_wait();
  pdl_trigger();
  const int tid = threadIdx.x;
  const int64_t base = (int64_t)blockIdx.x * n;
  __shared__ float s_part[16];
  __shared__ float s_rstd;
  float ss = 0.0f;
  for (int i = tid * 8; i < n; i += 512 * 8) {
    const uint4 av = *reinterpret_cast<const uint4*>(a + base + i);
    const uint4 rv = r ? *reinterpret_cast<const uint4*>(r + base + i) : make_uint4(0, 0, 0, 0);
    const uint32_t aw[4] = {av.x, av.y, av.z, av.w}, rw[4] = {rv.x, rv.y, rv.z, rv.w};
    uint32_t ow[4];
#pragma unroll
    for (int k = 0; k < 4; k++) {
      const uint16_t lo = f2bf(__uint_as_float(aw[k] << 16) + __uint_as_float(rw[k] << 16));
      const uint16_t hi = f2bf(__uint_as_float(aw[k] & 0xffff0000u) + __uint_as_float(rw[k] & 0xffff0000u));
      const float fl = bf2f(lo), fh = bf2f(hi);
      ss += fl * fl + fh * fh;
      ow[k] = (uint32_t)lo | ((uint32_t)hi << 16);
    }
    *reinterpret_cast<uint4*>(h_out + base + i) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
  }
  ss = warp_sum(ss);
  if ((tid & 31) == 0) s_part[tid >> 5] = ss;
  __syncthreads();
  if (tid < 32) {
    float v = tid < 16 ? s_part[tid] : 0.0f;
    v = warp_sum(v);
    if (tid == 0) s_rstd = rsqrtf(v / (float)n + eps);
  }
  __syncthreads();
  const float rstd = s_rstd;
  for (int i = tid * 8; i < n; i += 512 * 8) {   // every thread re-reads the values it wrote itself
    const uint4 hv = *reinterpret_cast<const uint4*>(h_out + base + i);
    const uint4 wv = *reinterpret_cast<const uint4*>(w + i);
    const uint32_t hw[4] = {hv.x, hv.y, hv.z, hv.w}, ww[4] = {wv.x, wv.y, wv.z, wv.w};
    uint32_t ow[4];
#pragma unroll
    for (int k = 0; k < 4; k++) {
      const uint16_t lo = f2bf(__uint_as_float(hw[k] << 16) * rstd * __uint_as_float(ww[k] << 16));
      const uint16_t hi = f2bf(__uint_as_float(hw[k] & 0xffff0000u) * rstd * __uint_as_float(ww[k] & 0xffff0000u));
      ow[k] = (uint32_t)lo | ((uint32_t)hi << 16);
    }
    *reinterpret_cast<uint4*>(x_out + base + i) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
  }
}

// out[row][i] = bf16( bf16(silu(g[row][i])) * u[row][i] ), g = gu[row][0:F], u = gu[row][F:2F]
__global__ void __launch_bounds__(256) silu_mul_kernel(const uint16_t* __restrict__ gu, uint16_t* __restrict__ out, int F) {
  pdl_wait();
  pdl_trigger();
  const int64_t row = blockIdx.y;
  const int i = (blockIdx.x * 256 + threadIdx.x) * 8;
  if (i >= F) return;
  const uint4 gv = *reinterpret_cast<const uint4*>(gu + row * 2 * F + i);
  const uint4 uv = *reinterpret_cast<const uint4*>(gu + row * 2 * F + F + i);
  const uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w}, uw[4] = {uv.x, uv.y, uv.z, uv.w};
  uint32_t ow[4];
#pragma unroll
  for (int k = 0; k < 4; k++) {
    const float g0 = __uint_as_float(gw[k] << 16), g1 = __uint_as_float(gw[k] & 0xffff0000u);
    const float a0 = bfround(g0 / (1.0f + __expf(-g0))), a1 = bfround(g1 / (1.0f + __expf(-g1)));
    ow[k] = (uint32_t)f2bf(a0 * __uint_as_float(uw[k] << 16)) | ((uint32_t)f2bf(a1 * __uint_as_float(uw[k] & 0xffff0000u)) << 16);
  }
  *reinterpret_cast<uint4*>(out + row * F + i) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace
}  // namespace pk

using namespace pk;

extern "C" int pk_qk_norm_rope(const pk_tensor* qkv, const pk_tensor* weight, const pk_tensor* cos, const pk_tensor* sin,
                               const pk_tensor* out, double eps, void* stream) {
  PK_CHECK_TENSOR(qkv, PK_BF16, 2);
  PK_CHECK_TENSOR(weight, PK_BF16, 2);
  PK_CHECK_TENSOR(cos, PK_BF16, 2);
  PK_CHECK_TENSOR(sin, PK_BF16, 2);
  PK_CHECK_TENSOR(out, PK_BF16, 3);
  const int64_t B = qkv->shape[0], heads = weight->shape[0];
  PK_REQUIRE(weight->shape[1] == 128 && is_contig(weight), "weight must be contiguous bf16 [heads,128]");
  PK_REQUIRE(qkv->stride[1] == 1 && qkv->shape[1] >= heads * 128 && qkv->stride[0] % 8 == 0,
             "qkv must be bf16 [B, >= heads*128] with unit inner stride and a row stride that is a multiple of 8");
  PK_REQUIRE(out->shape[0] == B && out->shape[1] == heads && out->shape[2] == 128 && is_contig(out),
             "out must be contiguous bf16 [B,heads,128]");
  PK_REQUIRE((cos->shape[0] == 1 || cos->shape[0] == B) && cos->shape[1] == 128 && is_contig(cos) &&
                 sin->shape[0] == cos->shape[0] && sin->shape[1] == 128 && is_contig(sin),
             "cos / sin must be contiguous bf16 [1 or B,128]");
  PK_REQUIRE(aligned16(qkv->data) && aligned16(weight->data) && aligned16(cos->data) && aligned16(sin->data) &&
                 aligned16(out->data),
             "tensors must be 16-byte aligned");
  const int64_t n_warps = B * heads;
  if (n_warps == 0) return PK_OK;
  PK_REQUIRE(heads < (1 << 20) && n_warps < (1LL << 31), "sizes out of range");
  StageTimer timer(ST_GLUE, (cudaStream_t)stream);
  launch_chain(qk_norm_rope_kernel, dim3((unsigned)((n_warps + 3) / 4)), dim3(128), 0, (cudaStream_t)stream,
      (const uint16_t*)qkv->data, qkv->stride[0], (const uint16_t*)weight->data, (const uint16_t*)cos->data,
      (const uint16_t*)sin->data, cos->shape[0] == 1 ? 0 : 128, (uint16_t*)out->data, (int)heads, n_warps, (float)eps);
  return check_launch("qk_norm_rope");
}

extern "C" int pk_add_rmsnorm(const pk_tensor* a, const pk_tensor* residual, const pk_tensor* weight, const pk_tensor* h_out,
                              const pk_tensor* x_out, double eps, void* stream) {
  PK_CHECK_TENSOR(a, PK_BF16, 2);
  PK_CHECK_TENSOR(weight, PK_BF16, 1);
  PK_CHECK_TENSOR(h_out, PK_BF16, 2);
  PK_CHECK_TENSOR(x_out, PK_BF16, 2);
  const int64_t B = a->shape[0], n = a->shape[1];
  PK_REQUIRE(is_contig(a) && is_contig(h_out) && is_contig(x_out) && is_contig(weight), "tensors must be contiguous");
  PK_REQUIRE(h_out->shape[0] == B && h_out->shape[1] == n && x_out->shape[0] == B && x_out->shape[1] == n &&
                 weight->shape[0] == n,
             "h_out / x_out must be [B,n] like a, weight [n]");
  PK_REQUIRE(n % 8 == 0 && n < (1 << 30) && B < 65536LL * 32768, "row length must be a multiple of 8");
  const uint16_t* r = nullptr;
  if (residual) {
    PK_CHECK_TENSOR(residual, PK_BF16, 2);
    PK_REQUIRE(is_contig(residual) && residual->shape[0] == B && residual->shape[1] == n, "residual must be [B,n] like a");
    r = (const uint16_t*)residual->data;
    PK_REQUIRE(aligned16(r), "tensors must be 16-byte aligned");
  }
  PK_REQUIRE(aligned16(a->data) && aligned16(weight->data) && aligned16(h_out->data) && aligned16(x_out->data),
             "tensors must be 16-byte aligned");
  if (B * n == 0) return PK_OK;
  StageTimer timer(ST_GLUE, (cudaStream_t)stream);
  launch_chain(add_rmsnorm_kernel, dim3((unsigned)B), dim3(512), 0, (cudaStream_t)stream, (const uint16_t*)a->data, r,
               (const uint16_t*)weight->data, (uint16_t*)h_out->data, (uint16_t*)x_out->data, (int)n, (float)eps);
  return check_launch("add_rmsnorm");
}

extern "C" int pk_silu_mul(const pk_tensor* gate_up, const pk_tensor* out, void* stream) {
  PK_CHECK_TENSOR(gate_up, PK_BF16, 2);
  PK_CHECK_TENSOR(out, PK_BF16, 2);
  const int64_t B = gate_up->shape[0], F = out->shape[1];
  PK_REQUIRE(is_contig(gate_up) && is_contig(out) && out->shape[0] == B && gate_up->shape[1] == 2 * F,
             "gate_up must be contiguous bf16 [B,2F], out [B,F]");
  PK_REQUIRE(F % 8 == 0 && F < (1 << 30) && B < 65536, "F must be a multiple of 8, B < 65536");
  PK_REQUIRE(aligned16(gate_up->data) && aligned16(out->data), "tensors must be 16-byte aligned");
  if (B * F == 0) return PK_OK;
  StageTimer timer(ST_GLUE, (cudaStream_t)stream);
  launch_chain(silu_mul_kernel, dim3((unsigned)((F / 8 + 255) / 256), (unsigned)B), dim3(256), 0, (cudaStream_t)stream,
               (const uint16_t*)gate_up->data, (uint16_t*)out->data, (int)F);
  return check_launch("silu_mul");
}

// ---- matrix-vector products of a decode step (one token): y = W x, W bf16 [O, I] row-major, fp32 accumulation ------
// HBM-bound: a warp takes two rows, every lane keeps sixteen 16-byte streaming loads in flight, x sits in shared memory.
// GATED: the rows are (o, o + F) of a stacked [gate; up] matrix and the output is silu(gate) * up, rounded like the
// separate launches would (bf16 after the product, after silu, after the multiply).
namespace pk {
namespace {

__device__ __forceinline__ void unpack8(const uint4 v, float* f) {
  f[0] = __uint_as_float(v.x << 16), f[1] = __uint_as_float(v.x & 0xffff0000u);
  f[2] = __uint_as_float(v.y << 16), f[3] = __uint_as_float(v.y & 0xffff0000u);
  f[4] = __uint_as_float(v.z << 16), f[5] = __uint_as_float(v.z & 0xffff0000u);
  f[6] = __uint_as_float(v.w << 16), f[7] = __uint_as_float(v.w & 0xffff0000u);
}

constexpr int GV_THREADS = 256;
constexpr int GV_UNROLL = 8;

template <bool GATED>
__global__ void __launch_bounds__(GV_THREADS) gemv_kernel(const uint16_t* __restrict__ W, const uint16_t* __restrict__ x,
                                                          uint16_t* __restrict__ out, int O, int I, int F) {
  extern __shared__ __align__(16) unsigned char gv_smem[];
  uint4* xs = reinterpret_cast<uint4*>(gv_smem);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int nchunk = I >> 3;
  const int n_pairs = GATED ? F : (O + 1) / 2;
  const int p = blockIdx.x * (GV_THREADS / 32) + warp;
  const bool live = p < n_pairs;
  const int r0 = GATED ? p : 2 * p, r1 = GATED ? p + F : 2 * p + 1;
  const bool has1 = live && r1 < O;
  const uint4* w0 = reinterpret_cast<const uint4*>(W + (int64_t)(live ? r0 : 0) * I);
  const uint4* w1 = reinterpret_cast<const uint4*>(W + (int64_t)(has1 ? r1 : (live ? r0 : 0)) * I);
  // The weights never change: the first batch of their loads is issued before the wait for the kernel that produces
  // x, so with programmatic dependent launch the stream of weights starts under the tail of that kernel.
  uint4 a[GV_UNROLL], b[GV_UNROLL];
  auto load_batch = [&](int c0) {
#pragma unroll
    for (int u = 0; u < GV_UNROLL; u++) {
      const int c = c0 + 32 * u;
      a[u] = (live && c < nchunk) ? __ldcs(w0 + c) : make_uint4(0, 0, 0, 0);
      b[u] = (live && c < nchunk) ? __ldcs(w1 + c) : make_uint4(0, 0, 0, 0);
    }
  };
  load_batch(lane);
  pdl_wait();
  pdl_trigger();
  for (int c = tid; c < nchunk; c += GV_THREADS) xs[c] = __ldg(reinterpret_cast<const uint4*>(x) + c);
  __syncthreads();
  if (!live) return;
  float acc0 = 0.0f, acc1 = 0.0f;
  for (int base = 0; base < nchunk; base += 32 * GV_UNROLL) {   // warp-uniform trip count
    const int c0 = base + lane;
#pragma unroll
    for (int u = 0; u < GV_UNROLL; u++) {
      const int c = c0 + 32 * u;
      if (c < nchunk) {
        float xf[8], af[8], bf[8];
        unpack8(xs[c], xf);
        unpack8(a[u], af);
        unpack8(b[u], bf);
#pragma unroll
        for (int k = 0; k < 8; k++) acc0 = fmaf(af[k], xf[k], acc0), acc1 = fmaf(bf[k], xf[k], acc1);
      }
    }
    if (base + 32 * GV_UNROLL < nchunk) load_batch(c0 + 32 * GV_UNROLL);
  }
  acc0 = warp_sum(acc0);
  acc1 = warp_sum(acc1);
  if (lane == 0) {
    if (GATED) {
      const float g = bfround(acc0), uu = bfround(acc1);
      out[p] = f2bf(bfround(g / (1.0f + __expf(-g))) * uu);
    } else {
      out[r0] = f2bf(acc0);
      if (has1) out[r1] = f2bf(acc1);
    }
  }
}

}  // namespace
}  // namespace pk

extern "C" int pk_gemv(const pk_tensor* weight, const pk_tensor* x, const pk_tensor* out, int gated, void* stream) {
  PK_CHECK_TENSOR(weight, PK_BF16, 2);
  PK_CHECK_TENSOR(x, PK_BF16, 2);
  PK_CHECK_TENSOR(out, PK_BF16, 2);
  const int64_t O = weight->shape[0], I = weight->shape[1];
  PK_REQUIRE(is_contig(weight) && is_contig(x) && is_contig(out) && x->shape[0] == 1 && x->shape[1] == I && out->shape[0] == 1,
             "weight must be contiguous bf16 [O,I], x [1,I], out [1,O] (or [1,O/2] when gated)");
  PK_REQUIRE(I % 8 == 0 && I >= 8 && I <= 24576 && O >= 1 && O < (1LL << 30), "I must be a multiple of 8, at most 24576");
  PK_REQUIRE(gated ? (O % 2 == 0 && out->shape[1] == O / 2) : out->shape[1] == O,
             "out must have O columns (O/2 when gated, with O even)");
  PK_REQUIRE(aligned16(weight->data) && aligned16(x->data), "weight and x must be 16-byte aligned");
  const int64_t pairs = gated ? O / 2 : (O + 1) / 2;
  const unsigned grid = (unsigned)((pairs + GV_THREADS / 32 - 1) / (GV_THREADS / 32));
  const size_t smem = (size_t)I * 2;
  StageTimer timer(ST_GEMV, (cudaStream_t)stream);
  if (gated)
    launch_chain(gemv_kernel<true>, dim3(grid), dim3(GV_THREADS), smem, (cudaStream_t)stream, (const uint16_t*)weight->data,
                 (const uint16_t*)x->data, (uint16_t*)out->data, (int)O, (int)I, (int)(O / 2));
  else
    launch_chain(gemv_kernel<false>, dim3(grid), dim3(GV_THREADS), smem, (cudaStream_t)stream, (const uint16_t*)weight->data,
                 (const uint16_t*)x->data, (uint16_t*)out->data, (int)O, (int)I, 0);
  return check_launch("gemv");
}

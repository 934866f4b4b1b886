// Key coding (SRHT normalise-rotate, sign code, 4-bit code, rerank weight), cluster histograms and
// query preparation.  One key is handled by 8 lanes, 16 dimensions (two 8-dim subspaces) per lane:
// the norm, the first four Hadamard stages and everything per subspace stay inside a lane; the last
// three Hadamard stages and the norm tree cross lanes with xor shuffles.  Every fp32 operation is an
// explicit round-to-nearest intrinsic in a fixed order, so results do not depend on the mapping.
#include "common.cuh"
#include "rotate.cuh"

namespace pk {
namespace {

__constant__ float c_thr[7] = {0.08447265625f, 0.169921875f, 0.2578125f, 0.349609375f,
                               0.44921875f,    0.55859375f,  0.69140625f};
__constant__ float c_cen[8] = {0.0419921875f, 0.126953125f, 0.212890625f, 0.302734375f,
                               0.396484375f,  0.5f,         0.6171875f,   0.76171875f};

// One 8-dim subspace of a rotated key: y = its 8 coordinates (bf16 values as floats), n = the key's bf16 norm.
// -> 8-bit sign code, rerank weight, four bytes of (sign << 3 | level) nibbles.  The arithmetic of
// polar_cache.batch_encode (cache_hub/polar_cache.py:950-976), every fp32 operation an explicit intrinsic.
__device__ __forceinline__ void code_subspace(const float* y, float n, unsigned* code_out, uint16_t* wt_out,
                                              uint32_t* packed_out) {
  float t[8];
  unsigned code = 0;
#pragma unroll
  for (int j = 0; j < 8; j++) {
    t[j] = __fmul_rn(y[j], y[j]);
    if (y[j] >= 0.0f) code |= 1u << j;
  }
#pragma unroll
  for (int w = 8; w > 1; w >>= 1)
#pragma unroll
    for (int i = 0; i < w / 2; i++) t[i] = __fadd_rn(t[2 * i], t[2 * i + 1]);
  const float r = bfround(__fsqrt_rn(t[0]));
  const float den = fmaxf(r, bfround(1e-8f));
  unsigned nib[8];
#pragma unroll
  for (int j = 0; j < 8; j++) {
    const float au = fabsf(bfround(__fdiv_rn(y[j], den)));
    unsigned lv = 0;
#pragma unroll
    for (int i = 0; i < 7; i++) lv += (c_thr[i] < au);
    t[j] = bfround(__fmul_rn(c_cen[lv], au));
    nib[j] = (((code >> j) & 1u) << 3) | lv;
  }
#pragma unroll
  for (int w = 8; w > 1; w >>= 1)
#pragma unroll
    for (int i = 0; i < w / 2; i++) t[i] = __fadd_rn(t[2 * i], t[2 * i + 1]);
  const float alpha = fmaxf(t[0], 1e-6f);
  *code_out = code;
  *wt_out = f2bf(__fmul_rn(__fdiv_rn(r, alpha), n));
  uint32_t packed = 0;
#pragma unroll
  for (int i = 0; i < 4; i++) packed |= ((nib[2 * i + 1] << 4) | nib[2 * i]) << (8 * i);
  *packed_out = packed;
}

struct EncodeParams {
  const uint16_t* keys;
  int64_t k_b, k_h, k_l;
  const uint16_t* signs;
  uint8_t* codes;
  int64_t c_b, c_h, c_s, c_l;
  uint16_t* w;
  int64_t w_b, w_h, w_s, w_l;
  uint8_t* pk;
  int64_t p_b, p_h, p_s, p_l;
  int32_t* counts;
  int H;
  int64_t L, chunk;
};

__global__ void __launch_bounds__(128) encode_kernel(EncodeParams p) {
  __shared__ int hist[16 * 256];
  const int tid = threadIdx.x, s = tid & 7, grp = tid >> 3;
  const int bh = blockIdx.y, b = bh / p.H, h = bh % p.H;
  if (p.counts) {
    for (int i = tid; i < 16 * 256; i += 128) hist[i] = 0;
    __syncthreads();
  }
  float sg[16];
  {
    const uint4* sp = reinterpret_cast<const uint4*>(p.signs + 16 * s);
    unpack8(__ldg(sp), sg);
    unpack8(__ldg(sp + 1), sg + 8);
  }
  const int64_t begin = (int64_t)blockIdx.x * p.chunk;
  const int64_t end = min(p.L, begin + p.chunk);
  const uint16_t* kbase = p.keys + b * p.k_b + h * p.k_h;
  for (int64_t k0 = begin; k0 < end; k0 += 16) {  // uniform per block: shuffles need whole warps
    const int64_t key = k0 + grp;
    const bool valid = key < end;
    float x[16];
    if (valid) {
      const uint4* kp = reinterpret_cast<const uint4*>(kbase + key * p.k_l + 16 * s);
      unpack8(__ldg(kp), x);
      unpack8(__ldg(kp + 1), x + 8);
    } else {
#pragma unroll
      for (int i = 0; i < 16; i++) x[i] = 0.0f;
    }
    const float n = rotate16(x, sg, s);
    if (!valid) continue;
#pragma unroll
    for (int half = 0; half < 2; half++) {
      const int sub = 2 * s + half;
      unsigned code;
      uint16_t wt;
      uint32_t packed;
      code_subspace(x + 8 * half, n, &code, &wt, &packed);
      p.codes[b * p.c_b + h * p.c_h + sub * p.c_s + key * p.c_l] = (uint8_t)code;
      p.w[b * p.w_b + h * p.w_h + sub * p.w_s + key * p.w_l] = wt;
      uint8_t* pp = p.pk + b * p.p_b + h * p.p_h + sub * p.p_s + key * p.p_l;
      if ((reinterpret_cast<uintptr_t>(pp) & 3) == 0) {
        *reinterpret_cast<uint32_t*>(pp) = packed;
      } else {
#pragma unroll
        for (int i = 0; i < 4; i++) pp[i] = (uint8_t)(packed >> (8 * i));
      }
      if (p.counts) atomicAdd(&hist[sub * 256 + code], 1);
    }
  }
  if (p.counts) {
    __syncthreads();
    int32_t* dst = p.counts + (int64_t)bh * 16 * 256;
    for (int i = tid; i < 16 * 256; i += 128)
      if (hist[i]) atomicAdd(dst + i, hist[i]);
  }
}

__global__ void __launch_bounds__(256) count_kernel(const uint8_t* codes, int64_t c_b, int64_t c_h,
                                                    int64_t c_s, int64_t c_l, int H, int B, int64_t N,
                                                    int64_t chunk, int32_t* counts) {
  extern __shared__ int hist[];
  const int tid = threadIdx.x;
  const int bh = blockIdx.y, b = bh / H, h = bh % H;
  for (int i = tid; i < B * 256; i += 256) hist[i] = 0;
  __syncthreads();
  const int64_t begin = (int64_t)blockIdx.x * chunk, end = min(N, begin + chunk);
  const uint8_t* base = codes + b * c_b + h * c_h;
  for (int64_t k = begin + tid; k < end; k += 256)
    for (int s = 0; s < B; s++) atomicAdd(&hist[s * 256 + base[s * c_s + k * c_l]], 1);
  __syncthreads();
  int32_t* dst = counts + (int64_t)bh * B * 256;
  for (int i = tid; i < B * 256; i += 256)
    if (hist[i]) atomicAdd(dst + i, hist[i]);
}

__global__ void __launch_bounds__(32) query_prep_kernel(const uint16_t* queries, int Hq, int H, int G,
                                                        float inv_g, const uint16_t* signs,
                                                        uint16_t* q_blocks, uint16_t* q_norm,
                                                        uint16_t* query_avg) {
  const int lane = threadIdx.x, s = lane & 7;
  const int bh = blockIdx.x, b = bh / H, h = bh % H;
  const uint16_t* q = queries + ((int64_t)b * Hq + (int64_t)h * G) * 128 + 16 * s;
  float x[16], sg[16];
#pragma unroll
  for (int i = 0; i < 16; i++) {
    float acc = 0.0f;
    for (int g = 0; g < G; g++) acc = __fadd_rn(acc, bf2f(q[g * 128 + i]));
    x[i] = bfround(__fmul_rn(acc, inv_g));
    sg[i] = bf2f(signs[16 * s + i]);
  }
  if (query_avg && lane < 8)
#pragma unroll
    for (int i = 0; i < 16; i++) query_avg[(int64_t)bh * 128 + 16 * s + i] = f2bf(x[i]);
  const float n = rotate16(x, sg, s);
  if (lane < 8) {
#pragma unroll
    for (int i = 0; i < 16; i++) q_blocks[(int64_t)bh * 128 + 16 * s + i] = f2bf(x[i]);
    if (lane == 0) q_norm[bh] = f2bf(n);
  }
}

// ---- append one decode token: window row, key coding, and the flush of a full update buffer, one launch ----------
// Device-side state per layer (int32): [0] rows in the window, [1] arrival counter, [2] flushes done, [3] error flag,
// [4 + b] searchable keys of sample b.  One block per (batch, KV head):
//   * warp 0 writes the K and V row at window row `pos`, codes the key (the arithmetic of encode_kernel) and stores
//     the codes, the rerank weights, the 4-bit codes and ||v|| in the window-aligned staging arrays, so every key is
//     coded exactly once, when it arrives;
//   * if that row filled the window, the oldest `interval` rows behind the sink are PUBLISHED: their staged records
//     are copied to zone records [N, N + interval), their codes are added to the cluster histogram, their K/V rows go
//     to the store (device or pinned host memory), and the rest of the window slides down;
//   * the block that finishes last advances the state words.
// Everything a later kernel needs (window length, zone length) is read from the state words, so the launch arguments
// never change and one captured CUDA graph serves the whole generation, flushes included.
struct AppendParams {
  const uint16_t* k_row;
  const uint16_t* v_row;
  int64_t kr_b, kr_h, vr_b, vr_h;   // element strides of the [bs,1,H,128] rows
  const uint16_t* signs;
  uint16_t* wk;
  uint16_t* wv;
  int64_t w_b, w_h;                 // window strides (elements); rows are 128 apart
  uint8_t* win_codes;               // [bs*H][cap_w][16]
  uint16_t* win_w;                  // [bs*H][cap_w][16]
  uint8_t* win_pk;                  // [bs*H][cap_w][64]
  float* win_vnorm;                 // [bs*H][cap_w]
  uint8_t* z_codes;                 // [bs*H][cap_z][16]   key-major zone records
  uint16_t* z_w;                    // [bs*H][cap_z][16]
  uint8_t* z_pk;                    // [bs*H][cap_z][64]
  float* z_vnorm;                   // [bs*H][cap_z] or null
  int32_t* counts;                  // [bs*H][16][256]
  uint16_t* store;                  // [bs*H][cap_s][2][128]
  int32_t* state;
  int H, cap_w, sink, interval;
  int64_t cap_z, cap_s;
};

__global__ void __launch_bounds__(256) append_encode_kernel(AppendParams p) {
  const int tid = threadIdx.x, lane = tid & 31;
  const int64_t bh = blockIdx.x;
  const int b = (int)(bh / p.H), h = (int)(bh % p.H);
  __shared__ int s_last;
  pdl_wait();     // the rows to append and the state words come from the kernels before this one
  pdl_trigger();
  const int pos = p.state[0];
  const int64_t N = p.state[4 + b];
  uint16_t* wk = p.wk + b * p.w_b + h * p.w_h;
  uint16_t* wv = p.wv + b * p.w_b + h * p.w_h;
  uint8_t* wc = p.win_codes + bh * p.cap_w * 16;
  uint16_t* ww = p.win_w + bh * p.cap_w * 16;
  uint8_t* wp = p.win_pk + bh * p.cap_w * 64;
  float* wn = p.win_vnorm + bh * p.cap_w;
  const bool ok = pos >= 0 && pos < p.cap_w;
  if (tid < 32 && ok) {
    const int s = lane & 7;
    const uint4* kr = reinterpret_cast<const uint4*>(p.k_row + b * p.kr_b + h * p.kr_h);
    const uint4* vr = reinterpret_cast<const uint4*>(p.v_row + b * p.vr_b + h * p.vr_h);
    // the rows themselves: lanes 0-15 carry K, lanes 16-31 carry V
    {
      const int l = lane & 15;
      const uint4 v = __ldg((lane < 16 ? kr : vr) + l);
      reinterpret_cast<uint4*>((lane < 16 ? wk : wv) + (int64_t)pos * 128)[l] = v;
    }
    float x[16], sg[16], y[16];
    unpack8(__ldg(kr + 2 * s), x);
    unpack8(__ldg(kr + 2 * s + 1), x + 8);
    unpack8(__ldg(reinterpret_cast<const uint4*>(p.signs) + 2 * s), sg);
    unpack8(__ldg(reinterpret_cast<const uint4*>(p.signs) + 2 * s + 1), sg + 8);
    unpack8(__ldg(vr + 2 * s), y);
    unpack8(__ldg(vr + 2 * s + 1), y + 8);
    // ||v||: fp32, pairwise tree over adjacent dimensions
#pragma unroll
    for (int i = 0; i < 16; i++) y[i] = __fmul_rn(y[i], y[i]);
#pragma unroll
    for (int w = 16; w > 1; w >>= 1)
#pragma unroll
      for (int i = 0; i < w / 2; i++) y[i] = __fadd_rn(y[2 * i], y[2 * i + 1]);
    float vs = y[0];
#pragma unroll
    for (int off = 1; off < 8; off <<= 1) vs = __fadd_rn(vs, __shfl_xor_sync(FULL, vs, off));
    const float n = rotate16(x, sg, s);
    unsigned code[2];
    uint16_t wt[2];
    uint32_t packed[2];
    code_subspace(x, n, &code[0], &wt[0], &packed[0]);
    code_subspace(x + 8, n, &code[1], &wt[1], &packed[1]);
    if (lane < 8) {
      *reinterpret_cast<uint16_t*>(wc + (int64_t)pos * 16 + 2 * s) = (uint16_t)(code[0] | (code[1] << 8));
      *reinterpret_cast<uint32_t*>(ww + (int64_t)pos * 16 + 2 * s) = (uint32_t)wt[0] | ((uint32_t)wt[1] << 16);
      *reinterpret_cast<uint2*>(wp + (int64_t)pos * 64 + 8 * s) = make_uint2(packed[0], packed[1]);
      if (lane == 0) wn[pos] = __fsqrt_rn(vs);
    }
  }
  __syncthreads();
  const int I = p.interval, sink = p.sink;
  const bool flush = ok && pos + 1 == p.cap_w;
  const bool room = N >= 0 && N + I <= p.cap_z && N + I <= p.cap_s;
  if (flush && room) {
    // publish rows [sink, sink + I): staged records -> zone records [N, N + I), K/V rows -> store, histogram
    const uint4* sc = reinterpret_cast<const uint4*>(wc + (int64_t)sink * 16);
    const uint4* sp = reinterpret_cast<const uint4*>(wp + (int64_t)sink * 64);
    const uint4* sw = reinterpret_cast<const uint4*>(ww + (int64_t)sink * 16);
    uint4* zc = reinterpret_cast<uint4*>(p.z_codes + (bh * p.cap_z + N) * 16);
    uint4* zp = reinterpret_cast<uint4*>(p.z_pk + (bh * p.cap_z + N) * 64);
    uint4* zw = reinterpret_cast<uint4*>(p.z_w + (bh * p.cap_z + N) * 16);
    for (int i = tid; i < I; i += 256) zc[i] = sc[i];
    for (int i = tid; i < 4 * I; i += 256) zp[i] = sp[i];
    for (int i = tid; i < 2 * I; i += 256) zw[i] = sw[i];
    if (p.z_vnorm)
      for (int i = tid; i < I; i += 256) p.z_vnorm[bh * p.cap_z + N + i] = wn[sink + i];
    uint4* st = reinterpret_cast<uint4*>(p.store + (bh * p.cap_s + N) * 256);
    const uint4* rk = reinterpret_cast<const uint4*>(wk + (int64_t)sink * 128);
    const uint4* rv = reinterpret_cast<const uint4*>(wv + (int64_t)sink * 128);
    for (int i = tid; i < 32 * I; i += 256) {
      const int row = i >> 5, c = i & 31;
      st[i] = c < 16 ? rk[row * 16 + c] : rv[row * 16 + (c - 16)];
    }
    int32_t* cnt = p.counts + bh * 16 * 256;
    for (int i = tid; i < 16 * I; i += 256) atomicAdd(cnt + (i & 15) * 256 + wc[(int64_t)sink * 16 + i], 1);
    __syncthreads();
    // slide rows [sink + I, cap_w) down to [sink, ...): chunks of at most I rows, in order, so a chunk's destination
    // only ever overlaps the sources of chunks already moved
    const int keep = p.cap_w - sink - I;
    const int R = min(I, 32);
    for (int r0 = 0; r0 < keep; r0 += R) {
      const int rows = min(R, keep - r0);
      for (int i = tid; i < rows * 39; i += 256) {
        const int row = r0 + i / 39, c = i % 39;
        const int64_t src = sink + I + row, dst = sink + row;
        if (c < 16) reinterpret_cast<uint4*>(wk + dst * 128)[c] = reinterpret_cast<const uint4*>(wk + src * 128)[c];
        else if (c < 32) reinterpret_cast<uint4*>(wv + dst * 128)[c - 16] = reinterpret_cast<const uint4*>(wv + src * 128)[c - 16];
        else if (c < 36) reinterpret_cast<uint4*>(wp + dst * 64)[c - 32] = reinterpret_cast<const uint4*>(wp + src * 64)[c - 32];
        else if (c < 38) reinterpret_cast<uint4*>(ww + dst * 16)[c - 36] = reinterpret_cast<const uint4*>(ww + src * 16)[c - 36];
        else reinterpret_cast<uint4*>(wc + dst * 16)[0] = reinterpret_cast<const uint4*>(wc + src * 16)[0];
      }
      for (int i = tid; i < rows; i += 256) wn[sink + r0 + i] = wn[sink + I + r0 + i];
      __syncthreads();
    }
  }
  // the block that arrives last advances the state (every block has read it by then)
  __threadfence();
  __syncthreads();
  if (tid == 0) s_last = atomicAdd(reinterpret_cast<unsigned*>(p.state + 1), 1u) + 1u == gridDim.x;
  __syncthreads();
  if (s_last && tid == 0) {
    if (!ok || (flush && !room)) {
      p.state[3] = 1;   // window overrun or zone full: the host checks this word
    } else if (flush) {
      p.state[0] = p.cap_w - I;
      p.state[2] += 1;
      const int bs = (int)(gridDim.x / p.H);
      for (int i = 0; i < bs; i++) p.state[4 + i] += I;
    } else {
      p.state[0] = pos + 1;
    }
    p.state[1] = 0;
  }
}

}  // namespace

// Host launchers shared with the fused retrieval entry point.
int launch_query_prep(const uint16_t* queries, int bs, int Hq, int H, const uint16_t* signs,
                      uint16_t* q_blocks, uint16_t* q_norm, uint16_t* query_avg, cudaStream_t st) {
  const int G = Hq / H;
  StageTimer tm(ST_QUERY_PREP, st);
  query_prep_kernel<<<bs * H, 32, 0, st>>>(queries, Hq, H, G, 1.0f / (float)G, signs, q_blocks, q_norm,
                                           query_avg);
  return check_launch("query_prep");
}

}  // namespace pk

using namespace pk;

extern "C" int pk_encode_keys(const pk_tensor* keys, const pk_tensor* signs, const pk_tensor* codebook,
                              const pk_tensor* block_weight, const pk_tensor* packed_4bit,
                              const pk_tensor* cluster_counts, void* stream) {
  PK_CHECK_TENSOR(keys, PK_BF16, 4);
  PK_CHECK_TENSOR(signs, PK_BF16, 1);
  PK_CHECK_TENSOR(codebook, PK_U8, 4);
  PK_CHECK_TENSOR(block_weight, PK_BF16, 4);
  PK_CHECK_TENSOR(packed_4bit, PK_U8, 5);
  const int64_t bs = keys->shape[0], H = keys->shape[1], L = keys->shape[2];
  PK_REQUIRE(keys->shape[3] == 128 && signs->shape[0] == 128, "head_dim must be 128");
  PK_REQUIRE(keys->stride[3] == 1 && signs->stride[0] == 1, "keys/signs must have last stride 1");
  PK_REQUIRE((reinterpret_cast<uintptr_t>(keys->data) & 15) == 0 && keys->stride[0] % 8 == 0 &&
                 keys->stride[1] % 8 == 0 && keys->stride[2] % 8 == 0,
             "key rows must be 16-byte aligned");
  PK_REQUIRE((reinterpret_cast<uintptr_t>(signs->data) & 15) == 0, "signs must be 16-byte aligned");
  PK_REQUIRE(codebook->shape[0] == bs && codebook->shape[1] == H && codebook->shape[2] == 16 &&
                 codebook->shape[3] == L,
             "codebook must be [bs,H,16,L]");
  PK_REQUIRE(block_weight->shape[0] == bs && block_weight->shape[1] == H && block_weight->shape[2] == 16 &&
                 block_weight->shape[3] == L,
             "block_weight must be [bs,H,16,L]");
  PK_REQUIRE(packed_4bit->shape[0] == bs && packed_4bit->shape[1] == H && packed_4bit->shape[2] == 16 &&
                 packed_4bit->shape[3] == L && packed_4bit->shape[4] == 4 && packed_4bit->stride[4] == 1,
             "packed_4bit must be [bs,H,16,L,4] with last stride 1");
  if (cluster_counts) {
    PK_CHECK_TENSOR(cluster_counts, PK_I32, 4);
    PK_REQUIRE(is_contig(cluster_counts) && cluster_counts->shape[0] == bs && cluster_counts->shape[1] == H &&
                   cluster_counts->shape[2] == 16 && cluster_counts->shape[3] == 256,
               "cluster_counts must be contiguous [bs,H,16,256]");
  }
  if (bs * H * L == 0) return PK_OK;
  EncodeParams p;
  p.keys = (const uint16_t*)keys->data;
  p.k_b = keys->stride[0], p.k_h = keys->stride[1], p.k_l = keys->stride[2];
  p.signs = (const uint16_t*)signs->data;
  p.codes = (uint8_t*)codebook->data;
  p.c_b = codebook->stride[0], p.c_h = codebook->stride[1], p.c_s = codebook->stride[2], p.c_l = codebook->stride[3];
  p.w = (uint16_t*)block_weight->data;
  p.w_b = block_weight->stride[0], p.w_h = block_weight->stride[1], p.w_s = block_weight->stride[2],
  p.w_l = block_weight->stride[3];
  p.pk = (uint8_t*)packed_4bit->data;
  p.p_b = packed_4bit->stride[0], p.p_h = packed_4bit->stride[1], p.p_s = packed_4bit->stride[2],
  p.p_l = packed_4bit->stride[3];
  p.counts = cluster_counts ? (int32_t*)cluster_counts->data : nullptr;
  p.H = (int)H;
  p.L = L;
  // chunk of keys per block: enough blocks to fill the machine, at most 2048 keys per block so the
  // shared histogram is flushed by few blocks
  int64_t target = (int64_t)sm_count() * 8;
  int64_t chunk = (L * bs * H + target - 1) / target;
  chunk = ((chunk + 15) / 16) * 16;
  if (chunk < 16) chunk = 16;
  if (chunk > 2048) chunk = 2048;
  p.chunk = chunk;
  dim3 grid((unsigned)((L + chunk - 1) / chunk), (unsigned)(bs * H));
  StageTimer tm(ST_ENCODE, (cudaStream_t)stream);
  encode_kernel<<<grid, 128, 0, (cudaStream_t)stream>>>(p);
  return check_launch("encode_keys");
}

extern "C" int pk_count_clusters(const pk_tensor* codebook, const pk_tensor* counts, int accumulate,
                                 void* stream) {
  PK_CHECK_TENSOR(codebook, PK_U8, 4);
  PK_CHECK_TENSOR(counts, PK_I32, 4);
  const int64_t bs = codebook->shape[0], H = codebook->shape[1], B = codebook->shape[2], N = codebook->shape[3];
  PK_REQUIRE(B >= 1 && B <= 32, "subspaces must be in 1..32");
  PK_REQUIRE(is_contig(counts) && counts->shape[0] == bs && counts->shape[1] == H && counts->shape[2] == B &&
                 counts->shape[3] == 256,
             "counts must be contiguous [bs,H,B,256]");
  cudaStream_t st = (cudaStream_t)stream;
  if (!accumulate) {
    if (cudaMemsetAsync(counts->data, 0, (size_t)(bs * H * B * 256 * 4), st) != cudaSuccess)
      return check_launch("count_clusters memset", 0);
  }
  if (bs * H * N == 0) return PK_OK;
  int64_t target = (int64_t)sm_count() * 4;
  int64_t chunk = (N * bs * H + target - 1) / target;
  if (chunk < 256) chunk = 256;
  if (chunk > 8192) chunk = 8192;
  dim3 grid((unsigned)((N + chunk - 1) / chunk), (unsigned)(bs * H));
  StageTimer tm(ST_COUNT, st);
  count_kernel<<<grid, 256, (size_t)B * 256 * 4, st>>>((const uint8_t*)codebook->data, codebook->stride[0],
                                                       codebook->stride[1], codebook->stride[2],
                                                       codebook->stride[3], (int)H, (int)B, N, chunk,
                                                       (int32_t*)counts->data);
  return check_launch("count_clusters");
}

extern "C" int pk_query_prep(const pk_tensor* queries, const pk_tensor* signs, const pk_tensor* q_blocks,
                             const pk_tensor* q_norm, const pk_tensor* query_avg, void* stream) {
  PK_CHECK_TENSOR(queries, PK_BF16, 4);
  PK_CHECK_TENSOR(signs, PK_BF16, 1);
  PK_CHECK_TENSOR(q_blocks, PK_BF16, 4);
  PK_CHECK_TENSOR(q_norm, PK_BF16, 3);
  const int64_t bs = queries->shape[0], Hq = queries->shape[2], H = q_blocks->shape[1];
  PK_REQUIRE(queries->shape[1] == 1 && queries->shape[3] == 128 && is_contig(queries),
             "queries must be contiguous [bs,1,Hq,128]");
  PK_REQUIRE(H > 0 && Hq % H == 0, "query heads (%lld) must be a multiple of KV heads (%lld)", (long long)Hq,
             (long long)H);
  PK_REQUIRE(is_contig(q_blocks) && q_blocks->shape[0] == bs && q_blocks->shape[2] == 16 && q_blocks->shape[3] == 8,
             "q_blocks must be contiguous [bs,H,16,8]");
  PK_REQUIRE(is_contig(q_norm) && q_norm->shape[0] == bs && q_norm->shape[1] == H && q_norm->shape[2] == 1,
             "q_norm must be contiguous [bs,H,1]");
  PK_REQUIRE(signs->shape[0] == 128 && signs->stride[0] == 1, "signs must be [128]");
  uint16_t* qa = nullptr;
  if (query_avg) {
    PK_CHECK_TENSOR(query_avg, PK_BF16, 3);
    PK_REQUIRE(is_contig(query_avg) && query_avg->shape[0] == bs && query_avg->shape[1] == H &&
                   query_avg->shape[2] == 128,
               "query_avg must be contiguous [bs,H,128]");
    qa = (uint16_t*)query_avg->data;
  }
  if (bs * H == 0) return PK_OK;
  return launch_query_prep((const uint16_t*)queries->data, (int)bs, (int)Hq, (int)H, (const uint16_t*)signs->data,
                           (uint16_t*)q_blocks->data, (uint16_t*)q_norm->data, qa, (cudaStream_t)stream);
}

extern "C" int pk_append_encode(const pk_tensor* k_row, const pk_tensor* v_row, const pk_tensor* signs,
                                const pk_tensor* window_k, const pk_tensor* window_v, const pk_tensor* win_codes,
                                const pk_tensor* win_weight, const pk_tensor* win_4bit, const pk_tensor* win_vnorm,
                                const pk_tensor* codebook, const pk_tensor* block_weight, const pk_tensor* packed_4bit,
                                const pk_tensor* value_norm, const pk_tensor* cluster_counts, const pk_tensor* store_kv,
                                const pk_tensor* state, int64_t sink, int64_t interval, void* stream) {
  PK_CHECK_TENSOR(k_row, PK_BF16, 4);
  PK_CHECK_TENSOR(v_row, PK_BF16, 4);
  PK_CHECK_TENSOR(signs, PK_BF16, 1);
  PK_CHECK_TENSOR(window_k, PK_BF16, 4);
  PK_CHECK_TENSOR(window_v, PK_BF16, 4);
  PK_CHECK_TENSOR(win_codes, PK_U8, 4);
  PK_CHECK_TENSOR(win_weight, PK_BF16, 4);
  PK_CHECK_TENSOR(win_4bit, PK_U8, 5);
  PK_CHECK_TENSOR(win_vnorm, PK_F32, 3);
  PK_CHECK_TENSOR(codebook, PK_U8, 4);
  PK_CHECK_TENSOR(block_weight, PK_BF16, 4);
  PK_CHECK_TENSOR(packed_4bit, PK_U8, 5);
  PK_CHECK_TENSOR(cluster_counts, PK_I32, 4);
  PK_CHECK_TENSOR(store_kv, PK_BF16, 5);
  PK_CHECK_TENSOR(state, PK_I32, 1);
  const int64_t bs = window_k->shape[0], H = window_k->shape[1], cap_w = window_k->shape[2];
  PK_REQUIRE(bs >= 1 && H >= 1 && bs * H < (1ll << 31), "window_k must be [bs,H,cap,128]");
  PK_REQUIRE(k_row->shape[0] == bs && k_row->shape[1] == 1 && k_row->shape[2] == H && k_row->shape[3] == 128 &&
                 k_row->stride[3] == 1 && v_row->shape[0] == bs && v_row->shape[1] == 1 && v_row->shape[2] == H &&
                 v_row->shape[3] == 128 && v_row->stride[3] == 1,
             "k_row / v_row must be [bs,1,H,128] with last stride 1");
  for (const pk_tensor* t : {k_row, v_row})
    PK_REQUIRE((reinterpret_cast<uintptr_t>(t->data) & 15) == 0 && (t->shape[0] == 1 || t->stride[0] % 8 == 0) &&
                   (t->shape[2] == 1 || t->stride[2] % 8 == 0),
               "k_row / v_row rows must be 16-byte aligned");
  PK_REQUIRE(signs->shape[0] == 128 && signs->stride[0] == 1 && (reinterpret_cast<uintptr_t>(signs->data) & 15) == 0,
             "signs must be a 16-byte aligned [128]");
  PK_REQUIRE(window_k->shape[3] == 128 && window_k->stride[3] == 1 && window_k->stride[2] == 128 &&
                 (reinterpret_cast<uintptr_t>(window_k->data) & 15) == 0 && (reinterpret_cast<uintptr_t>(window_v->data) & 15) == 0,
             "window_k must be [bs,H,cap,128] with rows 128 elements apart, 16-byte aligned");
  for (int i = 0; i < 4; i++)
    PK_REQUIRE(window_v->shape[i] == window_k->shape[i] && (window_k->shape[i] == 1 || window_v->stride[i] == window_k->stride[i]),
               "window_k and window_v must have the same shape and strides");
  PK_REQUIRE(window_k->stride[0] % 8 == 0 && window_k->stride[1] % 8 == 0, "window strides must be multiples of 8 elements");
  PK_REQUIRE(sink >= 0 && interval >= 1 && sink + interval <= cap_w, "need sink + interval <= window capacity");
  // staging arrays: contiguous, window-aligned
  PK_REQUIRE(is_contig(win_codes) && win_codes->shape[0] == bs && win_codes->shape[1] == H && win_codes->shape[2] == cap_w &&
                 win_codes->shape[3] == 16 && is_contig(win_weight) && numel(win_weight) == bs * H * cap_w * 16 &&
                 is_contig(win_4bit) && numel(win_4bit) == bs * H * cap_w * 64 && is_contig(win_vnorm) &&
                 numel(win_vnorm) == bs * H * cap_w,
             "staging arrays must be contiguous [bs,H,cap,16] u8, [bs,H,cap,16] bf16, [bs,H,cap,16,4] u8, [bs,H,cap] f32");
  for (const pk_tensor* t : {win_codes, win_weight, win_4bit})
    PK_REQUIRE((reinterpret_cast<uintptr_t>(t->data) & 15) == 0, "staging arrays must be 16-byte aligned");
  // zone records: logical [bs,H,16,cap_z(,4)], stored key-major and contiguous
  const int64_t cap_z = codebook->shape[3];
  PK_REQUIRE(codebook->shape[0] == bs && codebook->shape[1] == H && codebook->shape[2] == 16 && codebook->stride[2] == 1 &&
                 codebook->stride[3] == 16 && codebook->stride[1] == cap_z * 16 && (bs == 1 || codebook->stride[0] == H * cap_z * 16),
             "codebook must be the key-major [bs,H,16,cap] view of a contiguous [bs,H,cap,16] buffer");
  PK_REQUIRE(block_weight->shape[3] == cap_z && block_weight->shape[2] == 16 && block_weight->stride[2] == 1 &&
                 block_weight->stride[3] == 16 && block_weight->stride[1] == cap_z * 16 &&
                 (bs == 1 || block_weight->stride[0] == H * cap_z * 16),
             "block_weight must be the key-major [bs,H,16,cap] view of a contiguous [bs,H,cap,16] buffer");
  PK_REQUIRE(packed_4bit->shape[3] == cap_z && packed_4bit->shape[2] == 16 && packed_4bit->shape[4] == 4 &&
                 packed_4bit->stride[4] == 1 && packed_4bit->stride[2] == 4 && packed_4bit->stride[3] == 64 &&
                 packed_4bit->stride[1] == cap_z * 64 && (bs == 1 || packed_4bit->stride[0] == H * cap_z * 64),
             "packed_4bit must be the key-major [bs,H,16,cap,4] view of a contiguous [bs,H,cap,16,4] buffer");
  for (const pk_tensor* t : {codebook, block_weight, packed_4bit})
    PK_REQUIRE((reinterpret_cast<uintptr_t>(t->data) & 15) == 0, "zone records must be 16-byte aligned");
  float* zv = nullptr;
  if (value_norm) {
    PK_CHECK_TENSOR(value_norm, PK_F32, 3);
    PK_REQUIRE(is_contig(value_norm) && value_norm->shape[0] == bs && value_norm->shape[1] == H && value_norm->shape[2] == cap_z,
               "value_norm must be contiguous [bs,H,cap] with the zone's capacity");
    zv = (float*)value_norm->data;
  }
  PK_REQUIRE(is_contig(cluster_counts) && cluster_counts->shape[0] == bs && cluster_counts->shape[1] == H &&
                 cluster_counts->shape[2] == 16 && cluster_counts->shape[3] == 256,
             "cluster_counts must be contiguous [bs,H,16,256]");
  PK_REQUIRE(is_contig(store_kv) && store_kv->shape[0] == bs && store_kv->shape[1] == H && store_kv->shape[3] == 2 &&
                 store_kv->shape[4] == 128 && (reinterpret_cast<uintptr_t>(store_kv->data) & 15) == 0,
             "store_kv must be contiguous, 16-byte aligned [bs,H,cap,2,128] (device or pinned host memory)");
  PK_REQUIRE(state->stride[0] == 1 && state->shape[0] >= 4 + bs, "state must hold 4 + bs int32 words");
  AppendParams p;
  p.k_row = (const uint16_t*)k_row->data, p.v_row = (const uint16_t*)v_row->data;
  p.kr_b = k_row->shape[0] == 1 ? 0 : k_row->stride[0], p.kr_h = k_row->shape[2] == 1 ? 0 : k_row->stride[2];
  p.vr_b = v_row->shape[0] == 1 ? 0 : v_row->stride[0], p.vr_h = v_row->shape[2] == 1 ? 0 : v_row->stride[2];
  p.signs = (const uint16_t*)signs->data;
  p.wk = (uint16_t*)window_k->data, p.wv = (uint16_t*)window_v->data;
  p.w_b = window_k->shape[0] == 1 ? 0 : window_k->stride[0], p.w_h = window_k->shape[1] == 1 ? 0 : window_k->stride[1];
  p.win_codes = (uint8_t*)win_codes->data, p.win_w = (uint16_t*)win_weight->data, p.win_pk = (uint8_t*)win_4bit->data;
  p.win_vnorm = (float*)win_vnorm->data;
  p.z_codes = (uint8_t*)codebook->data, p.z_w = (uint16_t*)block_weight->data, p.z_pk = (uint8_t*)packed_4bit->data;
  p.z_vnorm = zv;
  p.counts = (int32_t*)cluster_counts->data;
  p.store = (uint16_t*)store_kv->data;
  p.state = (int32_t*)state->data;
  p.H = (int)H, p.cap_w = (int)cap_w, p.sink = (int)sink, p.interval = (int)interval;
  p.cap_z = cap_z, p.cap_s = store_kv->shape[2];
  StageTimer tm(ST_APPEND, (cudaStream_t)stream);
  launch_chain(append_encode_kernel, dim3((unsigned)(bs * H)), dim3(256), 0, (cudaStream_t)stream, p);
  return check_launch("append_encode");
}

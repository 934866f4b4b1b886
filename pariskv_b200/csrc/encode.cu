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
      const float* y = x + 8 * half;
      const int sub = 2 * s + half;
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
      const uint16_t wt = f2bf(__fmul_rn(__fdiv_rn(r, alpha), n));
      p.codes[b * p.c_b + h * p.c_h + sub * p.c_s + key * p.c_l] = (uint8_t)code;
      p.w[b * p.w_b + h * p.w_h + sub * p.w_s + key * p.w_l] = wt;
      uint32_t packed = 0;
#pragma unroll
      for (int i = 0; i < 4; i++) packed |= ((nib[2 * i + 1] << 4) | nib[2 * i]) << (8 * i);
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

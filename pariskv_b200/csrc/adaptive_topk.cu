// Fused adaptive-k: joint max, exp * ||v|| benefits, exact radix select of the K_out largest, sort,
// chunked prefix sums and threshold search, index gather.  One block of 1024 threads per (batch, head);
// benefits are recomputed per pass instead of being parked in a global workspace.
// Every fp32 step follows a fixed order (stated inline) that the CPU oracle repeats.
#include "common.cuh"
#include "kernels.cuh"

namespace pk {
namespace {

constexpr int AK_THREADS = 1024;

struct AkParams {
  const float* sl_logits;
  int64_t sl_b, sl_h;
  const float* sl_vnorm;
  int64_t sv_b, sv_h;
  const void* cand;  // f32 or bf16
  int cand_bf16;
  int64_t c_b, c_h;
  float scale;
  const int64_t* cand_idx;
  int64_t ci_b, ci_h;
  const float* cand_vnorm;  // or null
  int64_t cv_b, cv_h;
  const float* value_norm;  // used when cand_vnorm is null
  int64_t vn_b, vn_h;
  int64_t sink;
  int H;
  int64_t S, C, K_out, min_k, max_k;
  int K_pad;
  int cache_c;   // benefits kept in shared memory (C when they fit, else 0: recomputed per pass)
  float threshold;
  int64_t* ak_out;
  int64_t* topk_out;
};

// adjacent pairwise tree over the 1024 per-thread partials (thread id = leaf index)
__device__ float tree_sum_1024(float v, float* s_red, int tid) {
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, off));
  __syncthreads();
  if ((tid & 31) == 0) s_red[tid >> 5] = v;
  __syncthreads();
  float w = s_red[tid & 31];
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) w = __fadd_rn(w, __shfl_xor_sync(0xffffffffu, w, off));
  return w;
}

__device__ float block_max_1024(float v, float* s_red, int tid) {
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, off));
  __syncthreads();
  if ((tid & 31) == 0) s_red[tid >> 5] = v;
  __syncthreads();
  float w = s_red[tid & 31];
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) w = fmaxf(w, __shfl_xor_sync(0xffffffffu, w, off));
  return w;
}

__global__ void __launch_bounds__(AK_THREADS) adaptive_topk_kernel(AkParams p) {
  extern __shared__ __align__(16) unsigned char dyn[];
  unsigned long long* sk = reinterpret_cast<unsigned long long*>(dyn);      // K_pad composite keys
  float* locs = reinterpret_cast<float*>(dyn + (size_t)p.K_pad * 8);        // K_pad in-chunk prefix sums
  float* bcache = reinterpret_cast<float*>(dyn + (size_t)p.K_pad * 12);     // cache_c benefits
  __shared__ float s_red[32];
  __shared__ unsigned hist[2048];
  __shared__ unsigned s_warp[32];
  __shared__ unsigned s_res[3];
  __shared__ unsigned s_ao[2];
  __shared__ unsigned s_scan[32];
  __shared__ unsigned s_counter;
  __shared__ int s_fk;
  __shared__ float chunk_base[130];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int64_t bh = blockIdx.x;
  const int b = (int)(bh / p.H), h = (int)(bh % p.H);
  const float* sll = p.sl_logits + b * p.sl_b + h * p.sl_h;
  const float* slv = p.sl_vnorm + b * p.sv_b + h * p.sv_h;
  const int64_t* ci = p.cand_idx + b * p.ci_b + h * p.ci_h;
  const float* cvn = p.cand_vnorm ? p.cand_vnorm + b * p.cv_b + h * p.cv_h : nullptr;
  const float* vn = p.value_norm ? p.value_norm + b * p.vn_b + h * p.vn_h : nullptr;
  const float* cf = p.cand_bf16 ? nullptr : (const float*)p.cand + b * p.c_b + h * p.c_h;
  const uint16_t* cb = p.cand_bf16 ? (const uint16_t*)p.cand + b * p.c_b + h * p.c_h : nullptr;
  auto logit = [&](int64_t c) -> float { return __fmul_rn(cb ? bf2f(cb[c]) : cf[c], p.scale); };
  auto vnorm = [&](int64_t c) -> float { return cvn ? cvn[c] : vn[ci[c] + p.sink]; };

  // 1. joint max
  float m = -3.402823466e+38f;
  for (int64_t s = tid; s < p.S; s += AK_THREADS) m = fmaxf(m, sll[s]);
  for (int64_t c = tid; c < p.C; c += AK_THREADS) m = fmaxf(m, logit(c));
  const float gmax = block_max_1024(m, s_red, tid);
  auto compute_benefit = [&](int64_t c) -> float {
    return __fmul_rn(pinned_expf(__fsub_rn(logit(c), gmax)), vnorm(c));
  };
  const bool cached = p.cache_c > 0;
  auto benefit = [&](int64_t c) -> float { return cached ? bcache[c] : compute_benefit(c); };

  // 2./3. benefit sums: strided sequential partials, then the pairwise tree
  float part = 0.0f;
  for (int64_t s = tid; s < p.S; s += AK_THREADS)
    part = __fadd_rn(part, __fmul_rn(pinned_expf(__fsub_rn(sll[s], gmax)), slv[s]));
  const float sl_ben = tree_sum_1024(part, s_red, tid);
  part = 0.0f;
  unsigned a_bits = 0xffffffffu, o_bits = 0u;
  for (int64_t c = tid; c < p.C; c += AK_THREADS) {
    const float bn = compute_benefit(c);
    if (cached) bcache[c] = bn;
    part = __fadd_rn(part, bn);
    a_bits &= __float_as_uint(bn), o_bits |= __float_as_uint(bn);
  }
  const float total = __fadd_rn(sl_ben, tree_sum_1024(part, s_red, tid));
  if (tid == 0) s_ao[0] = 0xffffffffu, s_ao[1] = 0u;
  __syncthreads();
  a_bits = __reduce_and_sync(0xffffffffu, a_bits);
  o_bits = __reduce_or_sync(0xffffffffu, o_bits);
  if (lane == 0) {
    atomicAnd(&s_ao[0], a_bits);
    atomicOr(&s_ao[1], o_bits);
  }
  __syncthreads();

  // 4. exact radix select of the K_out-th largest benefit (bit patterns of non-negative floats are ordered):
  //    11-bit digits from the highest bit on which the benefits differ; stops when a whole digit bin is taken
  const unsigned varying = s_ao[0] ^ s_ao[1];
  unsigned prefix = s_ao[0] & ~varying, pmask = ~varying, rem = (unsigned)p.K_out;
  for (int hi = varying ? 31 - __clz(varying) : -1; hi >= 0; hi -= 11) {
    const int lo = max(hi - 10, 0);
    const unsigned dm = ((hi == 31 ? 0u : (1u << (hi + 1))) - (1u << lo));
    hist[tid] = 0;
    hist[tid + 1024] = 0;
    __syncthreads();
    for (int64_t c = tid; c < p.C; c += AK_THREADS) {
      const unsigned u = __float_as_uint(benefit(c));
      if (((u ^ prefix) & pmask) == 0) atomicAdd(&hist[(u & dm) >> lo], 1u);
    }
    __syncthreads();
    const unsigned v0 = hist[2 * tid], v1 = hist[2 * tid + 1];  // thread t owns bins 2t, 2t+1
    unsigned incl = v0 + v1;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      unsigned o = __shfl_down_sync(0xffffffffu, incl, off);
      if (lane + off < 32) incl += o;
    }
    if (lane == 0) s_warp[warp] = incl;
    __syncthreads();
    unsigned higher = 0;
    for (int w = warp + 1; w < 32; w++) higher += s_warp[w];
    const unsigned suf0 = incl + higher, suf1 = suf0 - v0, ab1 = suf1 - v1;
    if (suf1 >= rem && ab1 < rem) {
      s_res[0] = 2 * tid + 1, s_res[1] = ab1, s_res[2] = v1;
    } else if (suf0 >= rem && suf1 < rem) {
      s_res[0] = 2 * tid, s_res[1] = suf1, s_res[2] = v0;
    }
    __syncthreads();
    prefix = (prefix & ~dm) | (s_res[0] << lo);
    pmask |= dm;
    rem -= s_res[1];
    const bool all = s_res[2] == rem;
    __syncthreads();
    if (all) break;  // undecided bits of prefix stay zero: the rest of the bin compares >= prefix
  }
  const unsigned T = prefix;  // take all benefits > T and the first `rem` (by position) equal to T

  // 5. collect: ties by ascending position need an ordered scan; slots are arbitrary, the sort fixes order
  for (int i = tid; i < p.K_pad; i += AK_THREADS) sk[i] = 0ull;
  if (tid == 0) s_counter = 0;
  const int64_t span = (p.C + AK_THREADS - 1) / AK_THREADS;
  const int64_t my_b = min(p.C, tid * span), my_e = min(p.C, my_b + span);
  unsigned n_eq = 0;
  for (int64_t c = my_b; c < my_e; c++) n_eq += (__float_as_uint(benefit(c)) == T);
  unsigned incl = n_eq;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    unsigned o = __shfl_up_sync(0xffffffffu, incl, off);
    if (lane >= off) incl += o;
  }
  if (lane == 31) s_scan[warp] = incl;
  __syncthreads();
  unsigned eq_run = incl - n_eq;
  for (int w = 0; w < warp; w++) eq_run += s_scan[w];
  for (int64_t c = my_b; c < my_e; c++) {
    const unsigned u = __float_as_uint(benefit(c));
    bool take = u > T;
    if (u == T) {
      take = eq_run < rem;
      eq_run++;
    }
    if (take) {
      const unsigned slot = atomicAdd(&s_counter, 1u);
      if (slot < (unsigned)p.K_out) sk[slot] = ((unsigned long long)u << 32) | (0xffffffffu - (unsigned)c);
    }
  }
  __syncthreads();

  // 6. bitonic sort, descending (benefit, then lower position first)
  for (int sz = 2; sz <= p.K_pad; sz <<= 1)
    for (int st = sz >> 1; st > 0; st >>= 1) {
      for (int i = tid; i < p.K_pad / 2; i += AK_THREADS) {
        const int l = 2 * i - (i & (st - 1)), r = l + st;
        const bool desc = ((l / sz) & 1) == 0;
        const unsigned long long a = sk[l], c2 = sk[r];
        if (desc ? (a < c2) : (a > c2)) {
          sk[l] = c2;
          sk[r] = a;
        }
      }
      __syncthreads();
    }

  // 7. prefix sums in chunks of 32 (sequential inside a chunk, sequential over chunk totals)
  const int n_chunks = (int)((p.K_out + 31) / 32);
  if (tid < n_chunks) {
    float loc = 0.0f;
    for (int i = tid * 32; i < tid * 32 + 32 && i < p.K_out; i++) {
      loc = __fadd_rn(loc, __uint_as_float((unsigned)(sk[i] >> 32)));
      locs[i] = loc;
    }
    chunk_base[tid + 1] = loc;
  }
  if (tid == 0) s_fk = (int)p.K_out;
  __syncthreads();
  if (tid == 0) {
    float base = 0.0f;
    for (int c = 0; c < n_chunks; c++) {
      const float t = chunk_base[c + 1];
      chunk_base[c] = base;
      base = __fadd_rn(base, t);
    }
  }
  __syncthreads();
  if (total <= 0.0f) {
    if (tid == 0) s_fk = 1;
  } else {
    const float tgt = __fmul_rn(p.threshold, total);
    for (int i = tid; i < p.K_out; i += AK_THREADS) {
      const float cs = __fadd_rn(chunk_base[i >> 5], locs[i]);
      if (__fadd_rn(sl_ben, cs) >= tgt) atomicMin(&s_fk, i + 1);
    }
  }
  __syncthreads();
  if (tid == 0) {
    int64_t fk = s_fk;
    if (p.max_k > 0) {
      fk = max(fk, p.min_k);
      fk = min(fk, p.max_k);
      fk = min(fk, p.K_out);
    }
    p.ak_out[bh] = fk;
  }
  // 8. indices of the K_out largest, benefit descending
  int64_t* out = p.topk_out + bh * p.K_out;
  for (int i = tid; i < p.K_out; i += AK_THREADS) {
    const unsigned pos = 0xffffffffu - (unsigned)(sk[i] & 0xffffffffu);
    out[i] = (pos < (unsigned)p.C) ? ci[pos] : 0;
  }
}

}  // namespace
}  // namespace pk

using namespace pk;

extern "C" int pk_adaptive_topk(const pk_tensor* sl_logits, const pk_tensor* cand_scores, float cand_scale,
                                const pk_tensor* sl_vnorm, const pk_tensor* cand_indices,
                                const pk_tensor* cand_vnorm, const pk_tensor* value_norm, int64_t sink_size,
                                float threshold, int64_t K_out, int64_t min_k, int64_t max_k,
                                const pk_tensor* adaptive_k, const pk_tensor* topk_indices, void* stream) {
  PK_CHECK_TENSOR(sl_logits, PK_F32, 3);
  PK_CHECK_TENSOR(sl_vnorm, PK_F32, 3);
  PK_CHECK_TENSOR(cand_indices, PK_I64, 3);
  PK_CHECK_TENSOR(adaptive_k, PK_I64, 2);
  PK_CHECK_TENSOR(topk_indices, PK_I64, 3);
  PK_REQUIRE(cand_scores && cand_scores->data && cand_scores->ndim == 3 &&
                 (cand_scores->dtype == PK_F32 || cand_scores->dtype == PK_BF16),
             "cand_scores must be a 3-D float32 or bfloat16 tensor");
  const int64_t bs = sl_logits->shape[0], H = sl_logits->shape[1], S = sl_logits->shape[2], C = cand_scores->shape[2];
  PK_REQUIRE(sl_logits->stride[2] == 1 && sl_vnorm->stride[2] == 1 && cand_scores->stride[2] == 1 &&
                 cand_indices->stride[2] == 1,
             "inputs must have last stride 1");
  PK_REQUIRE(sl_vnorm->shape[0] == bs && sl_vnorm->shape[1] == H && sl_vnorm->shape[2] == S, "sl_vnorm must be [bs,H,S]");
  PK_REQUIRE(cand_scores->shape[0] == bs && cand_scores->shape[1] == H && cand_indices->shape[0] == bs &&
                 cand_indices->shape[1] == H && cand_indices->shape[2] == C,
             "cand_scores / cand_indices must be [bs,H,C]");
  PK_REQUIRE(K_out >= 1 && K_out <= C && K_out <= 4096, "K_out must be in 1..min(C,4096), got %lld", (long long)K_out);
  PK_REQUIRE(threshold > 0.0f && threshold <= 1.0f, "threshold must be in (0,1]");
  PK_REQUIRE(is_contig(adaptive_k) && adaptive_k->shape[0] == bs && adaptive_k->shape[1] == H,
             "adaptive_k must be contiguous [bs,H]");
  PK_REQUIRE(is_contig(topk_indices) && topk_indices->shape[0] == bs && topk_indices->shape[1] == H &&
                 topk_indices->shape[2] == K_out,
             "topk_indices must be contiguous [bs,H,K_out]");
  AkParams p = {};
  if (cand_vnorm) {
    PK_CHECK_TENSOR(cand_vnorm, PK_F32, 3);
    PK_REQUIRE(cand_vnorm->shape[0] == bs && cand_vnorm->shape[1] == H && cand_vnorm->shape[2] == C &&
                   cand_vnorm->stride[2] == 1,
               "cand_vnorm must be [bs,H,C] with last stride 1");
    p.cand_vnorm = (const float*)cand_vnorm->data;
    p.cv_b = cand_vnorm->stride[0], p.cv_h = cand_vnorm->stride[1];
  } else {
    PK_CHECK_TENSOR(value_norm, PK_F32, 3);
    PK_REQUIRE(value_norm->shape[0] == bs && value_norm->shape[1] == H && value_norm->stride[2] == 1,
               "value_norm must be [bs,H,cap] with last stride 1");
    p.value_norm = (const float*)value_norm->data;
    p.vn_b = value_norm->stride[0], p.vn_h = value_norm->stride[1];
    p.sink = sink_size;
  }
  if (bs * H == 0) return PK_OK;
  p.sl_logits = (const float*)sl_logits->data, p.sl_b = sl_logits->stride[0], p.sl_h = sl_logits->stride[1];
  p.sl_vnorm = (const float*)sl_vnorm->data, p.sv_b = sl_vnorm->stride[0], p.sv_h = sl_vnorm->stride[1];
  p.cand = cand_scores->data, p.cand_bf16 = cand_scores->dtype == PK_BF16;
  p.c_b = cand_scores->stride[0], p.c_h = cand_scores->stride[1];
  p.scale = cand_scale;
  p.cand_idx = (const int64_t*)cand_indices->data, p.ci_b = cand_indices->stride[0], p.ci_h = cand_indices->stride[1];
  p.H = (int)H, p.S = S, p.C = C, p.K_out = K_out, p.min_k = min_k, p.max_k = max_k;
  int kp = 2;
  while (kp < K_out) kp <<= 1;
  p.K_pad = kp;
  p.threshold = threshold;
  p.ak_out = (int64_t*)adaptive_k->data;
  p.topk_out = (int64_t*)topk_indices->data;
  p.cache_c = C <= 36 * 1024 ? (int)C : 0;   // up to 144 KB of benefits in shared memory
  const size_t smem = (size_t)kp * 12 + (size_t)p.cache_c * 4;
  if (smem > 30 * 1024) {
    if (cudaFuncSetAttribute(adaptive_topk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return check_launch("adaptive_topk smem");
  }
  StageTimer timer(ST_ADAPTIVE, (cudaStream_t)stream);
  adaptive_topk_kernel<<<(unsigned)(bs * H), AK_THREADS, smem, (cudaStream_t)stream>>>(p);
  return check_launch("adaptive_topk");
}

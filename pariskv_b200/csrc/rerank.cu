// 4-bit RaBitQ rerank, stand-alone and fused with candidate selection.
//
// One thread per candidate.  With key-major storage a candidate is one 64-byte record of nibbles
// plus one 32-byte record of bf16 weights (three DRAM sectors); with the reference's plane-major
// storage it is 16 + 16 scattered words (correct, but 32 sectors).  The 16 signed magnitude levels sit
// in shared memory replicated once per lane (bank = lane), the query blocks are read as broadcasts.
// fp32 order (shared with the CPU oracle): per subspace dot = fma chain over j ascending,
// acc = fma(dot, w_b, acc) over b ascending, score = acc * ||q||.
#include "common.cuh"
#include "kernels.cuh"

namespace pk {
namespace {

constexpr int RR_THREADS = 128;

struct RerankSmem {
  float lev[16][32];  // lev[nibble][lane]
  float q[128];
};

__device__ __forceinline__ void rerank_setup(RerankSmem& sm, const RerankArgs& a, int64_t bh, int tid, int nthreads) {
  for (int i = tid; i < 16 * 32; i += nthreads) {
    const int nib = i >> 5;
    const float c = bf2f(a.centers[nib & 7]);
    sm.lev[nib][i & 31] = (nib & 8) ? c : -c;
  }
  for (int i = tid; i < 128; i += nthreads) sm.q[i] = bf2f(a.q_blocks[bh * 128 + i]);
}

// FAST: key-major, 16-byte aligned records.  Returns the fp32 score of key `key`.
template <bool FAST>
__device__ __forceinline__ float rerank_one(const RerankSmem& sm, const RerankArgs& a, const uint8_t* k4,
                                            const uint16_t* w, int64_t key, float qn, int lane, uint16_t* v4b_row,
                                            int64_t v4b_sub_stride) {
  uint32_t code[16];
  uint32_t wt[8];
  if (FAST) {
    const uint4* cp = reinterpret_cast<const uint4*>(k4 + key * 64);
    const uint4* wp = reinterpret_cast<const uint4*>(w + key * 16);
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const uint4 v = __ldg(cp + i);
      code[4 * i] = v.x, code[4 * i + 1] = v.y, code[4 * i + 2] = v.z, code[4 * i + 3] = v.w;
    }
#pragma unroll
    for (int i = 0; i < 2; i++) {
      const uint4 v = __ldg(wp + i);
      wt[4 * i] = v.x, wt[4 * i + 1] = v.y, wt[4 * i + 2] = v.z, wt[4 * i + 3] = v.w;
    }
  } else {
#pragma unroll
    for (int s = 0; s < 16; s++) {
      const uint8_t* cp = k4 + s * a.k4_s + key * a.k4_l;
      code[s] = (uint32_t)cp[0] | ((uint32_t)cp[1] << 8) | ((uint32_t)cp[2] << 16) | ((uint32_t)cp[3] << 24);
    }
#pragma unroll
    for (int s = 0; s < 8; s++)
      wt[s] = (uint32_t)w[(2 * s) * a.w_s + key * a.w_l] | ((uint32_t)w[(2 * s + 1) * a.w_s + key * a.w_l] << 16);
  }
  float acc = 0.0f;
#pragma unroll
  for (int s = 0; s < 16; s++) {
    const float4 q0 = *reinterpret_cast<const float4*>(&sm.q[8 * s]);
    const float4 q1 = *reinterpret_cast<const float4*>(&sm.q[8 * s + 4]);
    const float qv[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
    float dot = 0.0f;
    float lv[8];
#pragma unroll
    for (int j = 0; j < 8; j++) {
      lv[j] = sm.lev[(code[s] >> (4 * j)) & 0xFu][lane];
      dot = __fmaf_rn(lv[j], qv[j], dot);
    }
    if (v4b_row) {
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; j++) o[j] = (uint32_t)f2bf(lv[2 * j]) | ((uint32_t)f2bf(lv[2 * j + 1]) << 16);
      *reinterpret_cast<uint4*>(v4b_row + s * v4b_sub_stride) = make_uint4(o[0], o[1], o[2], o[3]);
    }
    const float wf = __uint_as_float((s & 1) ? (wt[s >> 1] & 0xffff0000u) : (wt[s >> 1] << 16));
    acc = __fmaf_rn(dot, wf, acc);
  }
  return __fmul_rn(acc, qn);
}

template <bool FAST>
__global__ void __launch_bounds__(RR_THREADS) rerank_kernel(RerankArgs a, uint16_t* scores_bf16, float* scores_f32,
                                                            uint16_t* v4b) {
  __shared__ RerankSmem sm;
  const int tid = threadIdx.x, lane = tid & 31;
  const int64_t bh = blockIdx.y;
  const int b = (int)(bh / a.H), h = (int)(bh % a.H);
  rerank_setup(sm, a, bh, tid, RR_THREADS);
  __syncthreads();
  const float qn = bf2f(a.q_norm[bh]);
  const uint8_t* k4 = a.k4 + b * a.k4_b + h * a.k4_h;
  const uint16_t* w = a.w + b * a.w_b + h * a.w_h;
  for (int64_t c = (int64_t)blockIdx.x * RR_THREADS + tid; c < a.C; c += (int64_t)gridDim.x * RR_THREADS) {
    const int64_t key = a.cand[bh * a.C + c];
    uint16_t* vrow = v4b ? v4b + (bh * 16 * a.C + c) * 8 : nullptr;  // [bh][16][C][8]
    const float s = rerank_one<FAST>(sm, a, k4, w, key, qn, lane, vrow, a.C * 8);
    if (scores_bf16) scores_bf16[bh * a.C + c] = f2bf(s);
    if (scores_f32) scores_f32[bh * a.C + c] = s;
  }
}

// ---- candidate selection from u8 counts fused with the rerank of the selected keys -----------------
// One block per (chunk of keys, batch*head).  The per-chunk histograms written by the collision kernel
// give every block the global threshold bin, the tie quota and its own output offset, so the candidate
// list comes out in ascending key order with no atomics and no second pass.
constexpr int SEL_THREADS = 512;  // the first 256 threads own the 256 count bins

struct SelParams {
  const uint8_t* counts;  // [bs*H][u8_stride], virtual keys
  int64_t u8_stride;
  const uint32_t* chunk_hist;  // [bs*H][n_chunks][256]
  int64_t n_chunks, chunk_keys, N, C;
  int mis;
  int64_t* cand_out;   // [bs*H][C]
  float* scores_f32;   // [bs*H][C]
};

template <bool FAST>
__global__ void __launch_bounds__(SEL_THREADS) select_rerank_kernel(RerankArgs a, SelParams p) {
  extern __shared__ __align__(16) unsigned char dyn[];
  RerankSmem& sm = *reinterpret_cast<RerankSmem*>(dyn);
  int* list = reinterpret_cast<int*>(dyn + sizeof(RerankSmem));  // selected keys of this chunk, in order
  __shared__ unsigned tot[256], pre[256];
  __shared__ unsigned s_warp[8];
  __shared__ unsigned s_misc[4];  // t, quota, gt_before, eq_before
  __shared__ unsigned long long s_scan[SEL_THREADS / 32];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int64_t bh = blockIdx.y, chunk = blockIdx.x;
  const int b = (int)(bh / a.H), h = (int)(bh % a.H);
  rerank_setup(sm, a, bh, tid, SEL_THREADS);  // query blocks: written two kernels back, complete by now
  pdl_wait();                                   // counts and block histograms come from the collision kernel
  pdl_trigger();
  if (tid < 256) {
    const uint32_t* hp = p.chunk_hist + bh * p.n_chunks * 256 + tid;
    unsigned t = 0, pr = 0;
    int64_t c = 0;
    for (; c + 8 <= p.n_chunks; c += 8) {  // eight independent loads in flight
      unsigned v[8];
#pragma unroll
      for (int i = 0; i < 8; i++) v[i] = __ldg(hp + (c + i) * 256);
#pragma unroll
      for (int i = 0; i < 8; i++) {
        t += v[i];
        if (c + i < chunk) pr += v[i];
      }
    }
    for (; c < p.n_chunks; c++) {
      const unsigned v = __ldg(hp + c * 256);
      t += v;
      if (c < chunk) pr += v;
    }
    tot[tid] = t;
    pre[tid] = pr;
  }
  if (tid < 4) s_misc[tid] = 0;
  __syncthreads();
  // threshold bin: suffix sums over 256 bins (8 warps x 32 bins)
  unsigned v = tid < 256 ? tot[tid] : 0u, incl = v;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    unsigned o = __shfl_down_sync(0xffffffffu, incl, off);
    if (lane + off < 32) incl += o;
  }
  if (lane == 0 && warp < 8) s_warp[warp] = incl;
  __syncthreads();
  if (tid < 256) {
    unsigned higher = 0;
    for (int w = warp + 1; w < 8; w++) higher += s_warp[w];
    const unsigned suf = incl + higher, above = suf - v;
    if (suf >= (unsigned)p.C && above < (unsigned)p.C) {
      s_misc[0] = (unsigned)tid;
      s_misc[1] = (unsigned)p.C - above;
    }
  }
  __syncthreads();
  const unsigned T = s_misc[0], quota = s_misc[1];
  if (tid < 256 && (unsigned)tid > T && pre[tid]) atomicAdd(&s_misc[2], pre[tid]);
  if ((unsigned)tid == T) s_misc[3] = pre[tid];
  __syncthreads();
  const unsigned gt_base = s_misc[2], eq_base = s_misc[3];

  const int64_t Nv = p.N + p.mis;
  const int64_t v_begin = chunk * p.chunk_keys, v_end = min(Nv, v_begin + p.chunk_keys);
  const uint8_t* cnt = p.counts + bh * p.u8_stride;
  unsigned gt_run = 0, eq_run = 0;  // running counts over this chunk (all threads hold the same values)
  unsigned n_list = 0;
  for (int64_t t0 = v_begin; t0 < v_end; t0 += 16 * SEL_THREADS) {
    const int64_t v0 = t0 + 16 * (int64_t)tid;
    uint32_t w4[4] = {0, 0, 0, 0};
    if (v0 < v_end) {
      const uint4 r = *reinterpret_cast<const uint4*>(cnt + v0);
      w4[0] = r.x, w4[1] = r.y, w4[2] = r.z, w4[3] = r.w;
    }
    unsigned gt_mask = 0, eq_mask = 0;
#pragma unroll
    for (int k = 0; k < 16; k++) {
      const unsigned c = (w4[k >> 2] >> (8 * (k & 3))) & 0xFFu;
      const int64_t key = v0 + k - p.mis;
      const bool ok = (v0 + k < v_end) && key >= 0;
      gt_mask |= (unsigned)(ok && c > T) << k;
      eq_mask |= (unsigned)(ok && c == T) << k;
    }
    unsigned long long mine = ((unsigned long long)__popc(gt_mask) << 32) | (unsigned)__popc(eq_mask), sc = mine;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      unsigned long long o = __shfl_up_sync(0xffffffffu, sc, off);
      if (lane >= off) sc += o;
    }
    if (lane == 31) s_scan[warp] = sc;
    __syncthreads();
    unsigned long long base = 0, total = 0;
#pragma unroll
    for (int w = 0; w < SEL_THREADS / 32; w++) {
      if (w < warp) base += s_scan[w];
      total += s_scan[w];
    }
    const unsigned long long excl = base + sc - mine;
    unsigned g = gt_run + (unsigned)(excl >> 32), e = eq_run + (unsigned)excl;
    // position inside this chunk's list = (#gt before in chunk) + (#eq selected before in chunk)
    const unsigned eq_sel_before_chunk = min(eq_base, quota);
#pragma unroll
    for (int k = 0; k < 16; k++) {
      const bool is_gt = (gt_mask >> k) & 1u, is_eq = (eq_mask >> k) & 1u;
      if (is_gt || (is_eq && eq_base + e < quota)) {
        const unsigned sel_eq_before = min(eq_base + e, quota) - eq_sel_before_chunk;
        list[g + sel_eq_before] = (int)(v0 + k - p.mis);
      }
      g += is_gt;
      e += is_eq;
    }
    gt_run += (unsigned)(total >> 32);
    eq_run += (unsigned)total;
    __syncthreads();
  }
  n_list = gt_run + (min(eq_base + eq_run, quota) - min(eq_base, quota));
  const int64_t out_base = bh * p.C + gt_base + min(eq_base, quota);
  const float qn = bf2f(a.q_norm[bh]);
  const uint8_t* k4 = a.k4 + b * a.k4_b + h * a.k4_h;
  const uint16_t* w = a.w + b * a.w_b + h * a.w_h;
  for (unsigned i = tid; i < n_list; i += SEL_THREADS) {
    const int64_t key = list[i];
    const float s = rerank_one<FAST>(sm, a, k4, w, key, qn, lane, nullptr, 0);
    p.scores_f32[out_base + i] = s;
    if (p.cand_out) p.cand_out[out_base + i] = key;
  }
}

bool rerank_fast_layout(const RerankArgs& a) {
  return a.k4_s == 4 && a.k4_l == 64 && a.w_s == 1 && a.w_l == 16 && (reinterpret_cast<uintptr_t>(a.k4) & 15) == 0 &&
         (reinterpret_cast<uintptr_t>(a.w) & 15) == 0 && a.k4_b % 16 == 0 && a.k4_h % 16 == 0 && a.w_b % 8 == 0 &&
         a.w_h % 8 == 0;
}

}  // namespace

int fill_rerank_args(RerankArgs* a, const pk_tensor* key_4bit, const pk_tensor* key_block_weight) {
  PK_CHECK_TENSOR(key_4bit, PK_U8, 5);
  PK_CHECK_TENSOR(key_block_weight, PK_BF16, 4);
  PK_REQUIRE(key_4bit->shape[2] == 16 && key_4bit->shape[4] == 4 && key_4bit->stride[4] == 1,
             "key_4bit must be [bs,H,16,N,4] with last stride 1");
  PK_REQUIRE(key_block_weight->shape[2] == 16 && key_block_weight->shape[0] == key_4bit->shape[0] &&
                 key_block_weight->shape[1] == key_4bit->shape[1] && key_block_weight->shape[3] == key_4bit->shape[3],
             "key_block_weight must be [bs,H,16,N]");
  a->k4 = (const uint8_t*)key_4bit->data;
  a->k4_b = key_4bit->stride[0], a->k4_h = key_4bit->stride[1], a->k4_s = key_4bit->stride[2], a->k4_l = key_4bit->stride[3];
  a->w = (const uint16_t*)key_block_weight->data;
  a->w_b = key_block_weight->stride[0], a->w_h = key_block_weight->stride[1], a->w_s = key_block_weight->stride[2],
  a->w_l = key_block_weight->stride[3];
  a->H = (int)key_4bit->shape[1];
  return PK_OK;
}

int launch_rerank(const RerankArgs& a, int64_t bs_h, uint16_t* scores_bf16, float* scores_f32, uint16_t* v4b,
                  cudaStream_t st) {
  int64_t gx = (a.C + RR_THREADS - 1) / RR_THREADS;
  dim3 grid((unsigned)gx, (unsigned)bs_h);
  StageTimer tm(ST_RERANK, st);
  if (rerank_fast_layout(a))
    rerank_kernel<true><<<grid, RR_THREADS, 0, st>>>(a, scores_bf16, scores_f32, v4b);
  else
    rerank_kernel<false><<<grid, RR_THREADS, 0, st>>>(a, scores_bf16, scores_f32, v4b);
  return check_launch("rerank");
}

int launch_select_rerank(const RerankArgs& a, int64_t bs_h, const uint8_t* counts_u8, int64_t u8_stride,
                         const uint32_t* chunk_hist, int64_t n_chunks, int64_t chunk_keys, int mis, int64_t N,
                         int64_t* cand_out, float* scores_f32, cudaStream_t st) {
  SelParams p;
  p.counts = counts_u8, p.u8_stride = u8_stride, p.chunk_hist = chunk_hist;
  p.n_chunks = n_chunks, p.chunk_keys = chunk_keys, p.N = N, p.C = a.C, p.mis = mis;
  p.cand_out = cand_out, p.scores_f32 = scores_f32;
  const size_t smem = sizeof(RerankSmem) + (size_t)chunk_keys * sizeof(int);
  dim3 grid((unsigned)n_chunks, (unsigned)bs_h);
  const bool fast = rerank_fast_layout(a);
  auto kern = fast ? select_rerank_kernel<true> : select_rerank_kernel<false>;
  if (smem > 48 * 1024) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return check_launch("select_rerank smem");
  }
  StageTimer tm(ST_SELECT_RERANK, st);
  launch_chain(kern, grid, dim3(SEL_THREADS), smem, st, a, p);
  return check_launch("select_rerank");
}

}  // namespace pk

using namespace pk;

extern "C" int pk_rerank(const pk_tensor* coarse_indices, const pk_tensor* key_4bit,
                         const pk_tensor* key_block_weight, const pk_tensor* q_blocks, const pk_tensor* q_norm,
                         const pk_tensor* mag_centers, const pk_tensor* approx_scores, const pk_tensor* scores_f32,
                         const pk_tensor* v4b, void* stream) {
  PK_CHECK_TENSOR(coarse_indices, PK_I64, 3);
  PK_CHECK_TENSOR(q_blocks, PK_BF16, 4);
  PK_CHECK_TENSOR(q_norm, PK_BF16, 3);
  PK_CHECK_TENSOR(mag_centers, PK_BF16, 1);
  RerankArgs a;
  int rc = fill_rerank_args(&a, key_4bit, key_block_weight);
  if (rc) return rc;
  const int64_t bs = key_4bit->shape[0], H = key_4bit->shape[1], C = coarse_indices->shape[2];
  PK_REQUIRE(is_contig(coarse_indices) && coarse_indices->shape[0] == bs && coarse_indices->shape[1] == H,
             "coarse_indices must be contiguous [bs,H,C]");
  PK_REQUIRE(is_contig(q_blocks) && q_blocks->shape[0] == bs && q_blocks->shape[1] == H && q_blocks->shape[2] == 16 &&
                 q_blocks->shape[3] == 8,
             "q_blocks must be contiguous [bs,H,16,8] (only B == 16, m == 8 is supported)");
  PK_REQUIRE(is_contig(q_norm) && numel(q_norm) == bs * H, "q_norm must be contiguous [bs,H,1]");
  PK_REQUIRE(mag_centers->shape[0] == 8 && mag_centers->stride[0] == 1, "mag_centers must be [8]");
  uint16_t* sbf = nullptr;
  float* s32 = nullptr;
  uint16_t* v = nullptr;
  if (approx_scores) {
    PK_CHECK_TENSOR(approx_scores, PK_BF16, 3);
    PK_REQUIRE(is_contig(approx_scores) && approx_scores->shape[0] == bs && approx_scores->shape[1] == H &&
                   approx_scores->shape[2] == C,
               "approx_scores must be contiguous [bs,H,C]");
    sbf = (uint16_t*)approx_scores->data;
  }
  if (scores_f32) {
    PK_CHECK_TENSOR(scores_f32, PK_F32, 3);
    PK_REQUIRE(is_contig(scores_f32) && scores_f32->shape[0] == bs && scores_f32->shape[1] == H &&
                   scores_f32->shape[2] == C,
               "scores_f32 must be contiguous [bs,H,C]");
    s32 = (float*)scores_f32->data;
  }
  if (v4b) {
    PK_CHECK_TENSOR(v4b, PK_BF16, 5);
    PK_REQUIRE(is_contig(v4b) && v4b->shape[0] == bs && v4b->shape[1] == H && v4b->shape[2] == 16 &&
                   v4b->shape[3] == C && v4b->shape[4] == 8 && (reinterpret_cast<uintptr_t>(v4b->data) & 15) == 0,
               "v4b must be contiguous [bs,H,16,C,8]");
    v = (uint16_t*)v4b->data;
  }
  PK_REQUIRE(sbf || s32, "at least one of approx_scores / scores_f32 is required");
  if (bs * H * C == 0) return PK_OK;
  a.cand = (const int64_t*)coarse_indices->data;
  a.q_blocks = (const uint16_t*)q_blocks->data;
  a.q_norm = (const uint16_t*)q_norm->data;
  a.centers = (const uint16_t*)mag_centers->data;
  a.C = C;
  return launch_rerank(a, bs * H, sbf, s32, v, (cudaStream_t)stream);
}

// Exact, deterministic top-k of rows of 32-bit values (int32 counts or fp32 scores).
//
// One thread-block cluster per row: the row is cut into contiguous slices, one per CTA; digit
// histograms live in each CTA's shared memory and are summed across the cluster through distributed
// shared memory, so the whole selection (varying-bit probe, up to four 8-bit radix passes, tie quota,
// ordered emission) is ONE launch with no global scratch.  Digits are cut from the highest bit on which
// the elements of the row differ, so collision counts (0..96) need a single histogram pass and fp32 scores
// spread over the first histogram instead of piling into two exponent bins.  Rows of up to 16384
// elements take a single-block variant that keeps the keys in registers.
// Selected set: first k of (value descending, index ascending); emitted in ascending index.
#include <cooperative_groups.h>

#include "common.cuh"
#include "kernels.cuh"

namespace cg = cooperative_groups;

namespace pk {
namespace {

constexpr int TK_THREADS = 512;

struct TopkParams {
  const uint32_t* in;
  int is_float;
  int64_t row_stride, L, k;
  int64_t* out;
  const int64_t* map;
  int64_t map_stride;
};

__device__ __forceinline__ uint32_t load_key(const uint32_t* row, int64_t i, int is_float) {
  const uint32_t u = __ldg(row + i);
  return is_float ? ord_key(__uint_as_float(u)) : ord_key((int32_t)u);
}

// Among 256 bins (tot[b] valid for tid < 256, in shared memory), find the bin where the suffix sum
// first reaches `rem`: returns bin and the number of elements in higher bins.
__device__ void suffix_select(const unsigned* tot, unsigned rem, unsigned* s_tmp, unsigned* s_res, int tid) {
  // s_tmp[0..7]: per-warp totals; warps 0..7 cover bins 32w..32w+31
  const int lane = tid & 31, warp = tid >> 5;
  unsigned v = 0, incl = 0;
  if (warp < 8) {
    v = tot[tid];
    incl = v;  // inclusive suffix within the warp: sum of lanes >= lane
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      unsigned o = __shfl_down_sync(0xffffffffu, incl, off);
      if (lane + off < 32) incl += o;
    }
    if (lane == 0) s_tmp[warp] = incl;
  }
  __syncthreads();
  if (warp < 8) {
    unsigned higher = 0;
    for (int w = warp + 1; w < 8; w++) higher += s_tmp[w];
    const unsigned suf = incl + higher;        // elements in bins >= tid
    const unsigned above = suf - v;            // elements in bins > tid
    if (suf >= rem && above < rem) {
      s_res[0] = (unsigned)tid;
      s_res[1] = above;
    }
  }
  __syncthreads();
}

__global__ void __launch_bounds__(TK_THREADS) topk_cluster_kernel(TopkParams p) {
  cg::cluster_group cluster = cg::this_cluster();
  __shared__ unsigned hist[256];
  __shared__ unsigned tot[256];
  __shared__ unsigned red[4];     // and, or, n_gt, n_eq of this CTA
  __shared__ unsigned s_tmp[16];
  __shared__ unsigned s_res[2];
  __shared__ unsigned long long s_scan[TK_THREADS / 32];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const unsigned rank = cluster.block_rank(), ncta = cluster.num_blocks();
  const int64_t row_id = blockIdx.y;
  const uint32_t* row = p.in + row_id * p.row_stride;
  const int64_t per = (p.L + ncta - 1) / ncta;
  const int64_t begin = min(p.L, (int64_t)rank * per), end = min(p.L, begin + per);
  const int64_t span = (per + TK_THREADS - 1) / TK_THREADS;
  const int64_t my_begin = min(end, begin + tid * span), my_end = min(end, my_begin + span);

  // ---- which bits vary over the row ----
  if (tid == 0) {
    red[0] = 0xffffffffu;
    red[1] = 0u;
  }
  __syncthreads();
  {
    unsigned a = 0xffffffffu, o = 0u;
    for (int64_t i = my_begin; i < my_end; i++) {
      const uint32_t k = load_key(row, i, p.is_float);
      a &= k;
      o |= k;
    }
    a = __reduce_and_sync(0xffffffffu, a);
    o = __reduce_or_sync(0xffffffffu, o);
    if (lane == 0) {
      atomicAnd(&red[0], a);
      atomicOr(&red[1], o);
    }
  }
  cluster.sync();
  unsigned A = 0xffffffffu, O = 0u;
  for (unsigned r = 0; r < ncta; r++) {
    const unsigned* rr = cluster.map_shared_rank(red, r);
    A &= rr[0];
    O |= rr[1];
  }
  const unsigned varying = A ^ O;

  // ---- radix passes from the highest varying bit down, 8 bits at a time ----
  unsigned prefix = A, pmask = ~varying, rem = (unsigned)p.k;  // bits that never vary are already decided
  for (int hi = 31 - __clz(varying | 0u); varying != 0 && hi >= 0; hi -= 8) {
    const int lo = max(hi - 7, 0);
    const unsigned dm = ((hi == 31 ? 0u : (1u << (hi + 1))) - (1u << lo));  // bits lo..hi
    const unsigned above = hi == 31 ? 0u : ~((1u << (hi + 1)) - 1u);        // bits above hi
    const unsigned fixed = pmask | above;
    if (tid < 256) hist[tid] = 0;
    __syncthreads();
    for (int64_t i = my_begin; i < my_end; i++) {
      const uint32_t k = load_key(row, i, p.is_float);
      if (((k ^ prefix) & fixed) == 0) atomicAdd(&hist[(k & dm) >> lo], 1u);
    }
    cluster.sync();
    if (tid < 256) {
      unsigned t = 0;
      for (unsigned r = 0; r < ncta; r++) t += cluster.map_shared_rank(hist, r)[tid];
      tot[tid] = t;
    }
    __syncthreads();
    suffix_select(tot, rem, s_tmp, s_res, tid);
    prefix = (prefix & ~dm) | (s_res[0] << lo);
    pmask |= dm;
    rem -= s_res[1];
    const bool whole_bin = tot[s_res[0]] == rem;  // every element of the threshold bin is selected
    cluster.sync();  // every CTA has read the remote histograms before they are cleared again
    if (whole_bin) {
      prefix &= pmask;  // undecided bits zero: the rest of the bin compares >= this key
      break;
    }
  }
  const unsigned T = prefix;  // key of the k-th element; take `rem` of the elements equal to it

  // ---- count, scan, emit in index order ----
  unsigned n_gt = 0, n_eq = 0;
  for (int64_t i = my_begin; i < my_end; i++) {
    const uint32_t k = load_key(row, i, p.is_float);
    n_gt += (k > T);
    n_eq += (k == T);
  }
  unsigned long long mine = ((unsigned long long)n_gt << 32) | n_eq, incl = mine;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    unsigned long long o = __shfl_up_sync(0xffffffffu, incl, off);
    if (lane >= off) incl += o;
  }
  if (lane == 31) s_scan[warp] = incl;
  __syncthreads();
  unsigned long long base = 0, total = 0;
  for (int w = 0; w < TK_THREADS / 32; w++) {
    if (w < warp) base += s_scan[w];
    total += s_scan[w];
  }
  if (tid == 0) {
    red[2] = (unsigned)(total >> 32);
    red[3] = (unsigned)total;
  }
  cluster.sync();
  unsigned gt_run = (unsigned)((base + incl - mine) >> 32), eq_run = (unsigned)(base + incl - mine);
  for (unsigned r = 0; r < rank; r++) {
    const unsigned* rr = cluster.map_shared_rank(red, r);
    gt_run += rr[2];
    eq_run += rr[3];
  }
  int64_t* out = p.out + row_id * p.k;
  const int64_t* map = p.map ? p.map + row_id * p.map_stride : nullptr;
  for (int64_t i = my_begin; i < my_end; i++) {
    const uint32_t k = load_key(row, i, p.is_float);
    if (k > T) {
      out[gt_run + min(eq_run, rem)] = map ? map[i] : i;
      gt_run++;
    } else if (k == T) {
      if (eq_run < rem) out[gt_run + eq_run] = map ? map[i] : i;
      eq_run++;
    }
  }
  cluster.sync();  // shared memory must outlive the remote reads above
}

// Single-block variant for rows of at most 1024 * SPAN elements: every thread keeps SPAN consecutive
// elements in registers, so the row is read once.  Stage A buckets the VALUES linearly between the row's
// minimum and maximum into 2048 bins (a monotone map, so bins above the threshold bin are selected outright
// and the histogram is spread even when fp32 bit patterns share their high bits); stage B runs the exact radix
// select only over the few elements of the threshold bin.
template <int SPAN>
__global__ void __launch_bounds__(1024) topk_block_kernel(TopkParams p) {
  __shared__ unsigned hist[2048];
  __shared__ float s_mn[32], s_mx[32];
  __shared__ unsigned s_tmp[32];
  __shared__ unsigned s_res[3];
  __shared__ unsigned long long s_scan[32];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int64_t row_id = blockIdx.x;
  const uint32_t* row = p.in + row_id * p.row_stride;
  const int64_t my_begin = (int64_t)tid * SPAN;
  const int nv = (int)max((int64_t)0, min((int64_t)SPAN, p.L - my_begin));
  uint32_t key[SPAN];
  float val[SPAN];
  float mn = INFINITY, mx = -INFINITY;
#pragma unroll
  for (int j = 0; j < SPAN; j++) {
    const uint32_t u = j < nv ? __ldg(row + my_begin + j) : 0u;
    val[j] = p.is_float ? __uint_as_float(u) : (float)(int32_t)u;
    key[j] = p.is_float ? ord_key(__uint_as_float(u)) : ord_key((int32_t)u);
    if (j < nv) {
      mn = fminf(mn, val[j]);
      mx = fmaxf(mx, val[j]);
    }
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, off));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
  }
  if (lane == 0) s_mn[warp] = mn, s_mx[warp] = mx;
  hist[tid] = 0;
  hist[tid + 1024] = 0;
  __syncthreads();
  mn = s_mn[lane], mx = s_mx[lane];
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, off));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
  }
  float scale = 2047.0f / (mx - mn);
  if (!(scale > 0.0f) || !(scale < INFINITY)) scale = 0.0f;  // flat or non-finite range: one bin, stage B decides
  unsigned bin[SPAN];
#pragma unroll
  for (int j = 0; j < SPAN; j++) {
    bin[j] = min(2047u, (unsigned)((val[j] - mn) * scale));
    if (j < nv) atomicAdd(&hist[bin[j]], 1u);
  }
  __syncthreads();
  // threshold bin over 2048 bins: thread t owns bins 2t, 2t+1
  unsigned rem = (unsigned)p.k;
  auto select_bin = [&]() {
    const unsigned v0 = hist[2 * tid], v1 = hist[2 * tid + 1];
    unsigned incl = v0 + v1;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      unsigned o = __shfl_down_sync(0xffffffffu, incl, off);
      if (lane + off < 32) incl += o;
    }
    if (lane == 0) s_tmp[warp] = incl;
    __syncthreads();
    unsigned higher = 0;
    for (int w = warp + 1; w < 32; w++) higher += s_tmp[w];
    const unsigned suf0 = incl + higher, suf1 = suf0 - v0, ab1 = suf1 - v1;
    if (suf1 >= rem && ab1 < rem) {
      s_res[0] = 2 * tid + 1, s_res[1] = ab1, s_res[2] = v1;
    } else if (suf0 >= rem && suf1 < rem) {
      s_res[0] = 2 * tid, s_res[1] = suf1, s_res[2] = v0;
    }
    __syncthreads();
  };
  select_bin();
  const unsigned tbin = s_res[0];
  rem -= s_res[1];
  const bool whole = s_res[2] == rem;  // every element of the threshold bin is selected
  __syncthreads();
  unsigned prefix = 0, pmask = 0;
  if (!whole) {
    // stage B: exact radix select of the rem-th largest key among the elements of the threshold bin
    for (int hi = 31; hi >= 0; hi -= 11) {
      const int lo = max(hi - 10, 0);
      const unsigned dm = ((hi == 31 ? 0u : (1u << (hi + 1))) - (1u << lo));
      hist[tid] = 0;
      hist[tid + 1024] = 0;
      __syncthreads();
#pragma unroll
      for (int j = 0; j < SPAN; j++)
        if (j < nv && bin[j] == tbin && ((key[j] ^ prefix) & pmask) == 0) atomicAdd(&hist[(key[j] & dm) >> lo], 1u);
      __syncthreads();
      select_bin();
      prefix = (prefix & ~dm) | (s_res[0] << lo);
      pmask |= dm;
      rem -= s_res[1];
      const bool all = s_res[2] == rem;
      __syncthreads();
      if (all) break;  // undecided bits of prefix are zero: the rest of the bin compares >= prefix
    }
  }
  const unsigned T = prefix;  // with `whole`, T = 0: every key of the threshold bin is >= T
  unsigned n_gt = 0, n_eq = 0;
#pragma unroll
  for (int j = 0; j < SPAN; j++)
    if (j < nv) {
      const bool in = bin[j] == tbin;
      n_gt += bin[j] > tbin || (in && key[j] > T);
      n_eq += in && key[j] == T;
    }
  unsigned long long mine = ((unsigned long long)n_gt << 32) | n_eq, incl = mine;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    unsigned long long o = __shfl_up_sync(0xffffffffu, incl, off);
    if (lane >= off) incl += o;
  }
  if (lane == 31) s_scan[warp] = incl;
  __syncthreads();
  unsigned long long base = 0;
  for (int w = 0; w < warp; w++) base += s_scan[w];
  unsigned gt_run = (unsigned)((base + incl - mine) >> 32), eq_run = (unsigned)(base + incl - mine);
  int64_t* out = p.out + row_id * p.k;
  const int64_t* map = p.map ? p.map + row_id * p.map_stride : nullptr;
#pragma unroll
  for (int j = 0; j < SPAN; j++)
    if (j < nv) {
      const int64_t i = my_begin + j;
      const bool in = bin[j] == tbin;
      if (bin[j] > tbin || (in && key[j] > T)) {
        out[gt_run + min(eq_run, rem)] = map ? map[i] : i;
        gt_run++;
      } else if (in && key[j] == T) {
        if (eq_run < rem) out[gt_run + eq_run] = map ? map[i] : i;
        eq_run++;
      }
    }
}

// Reorders an emitted top-k list by (value descending, index ascending): one block per row, k <= 4096.
__global__ void __launch_bounds__(1024) sort_by_value_kernel(const uint32_t* in, int is_float, int64_t row_stride,
                                                             int64_t k, int kp, int64_t* out) {
  extern __shared__ unsigned long long sk[];  // (key << 32) | ~idx  sorted descending
  const int tid = threadIdx.x;
  const int64_t row_id = blockIdx.x;
  const uint32_t* row = in + row_id * row_stride;
  int64_t* o = out + row_id * k;
  for (int i = tid; i < kp; i += 1024) {
    unsigned long long v = 0;
    if (i < k) {
      const int64_t idx = o[i];
      v = ((unsigned long long)load_key(row, idx, is_float) << 32) | (0xffffffffu - (unsigned)idx);
    }
    sk[i] = v;
  }
  __syncthreads();
  for (int sz = 2; sz <= kp; sz <<= 1)
    for (int st = sz >> 1; st > 0; st >>= 1) {
      for (int i = tid; i < kp / 2; i += 1024) {
        const int l = 2 * i - (i & (st - 1)), r = l + st;
        const bool desc = ((l / sz) & 1) == 0;
        const unsigned long long a = sk[l], b = sk[r];
        if (desc ? (a < b) : (a > b)) {
          sk[l] = b;
          sk[r] = a;
        }
      }
      __syncthreads();
    }
  for (int i = tid; i < k; i += 1024) o[i] = (int64_t)(0xffffffffu - (unsigned)(sk[i] & 0xffffffffu));
}

}  // namespace

int launch_topk(const void* in, bool is_float, int64_t rows, int64_t row_stride, int64_t L, int64_t k,
                int64_t* out, const int64_t* map, int64_t map_stride, int order, cudaStream_t st, int stage) {
  StageTimer tm(stage, st);
  TopkParams p;
  p.in = (const uint32_t*)in;
  p.is_float = is_float ? 1 : 0;
  p.row_stride = row_stride, p.L = L, p.k = k;
  p.out = out, p.map = map, p.map_stride = map_stride;
  if (L <= 16384) {
    if (L <= 4096)
      topk_block_kernel<4><<<(unsigned)rows, 1024, 0, st>>>(p);
    else if (L <= 8192)
      topk_block_kernel<8><<<(unsigned)rows, 1024, 0, st>>>(p);
    else
      topk_block_kernel<16><<<(unsigned)rows, 1024, 0, st>>>(p);
    int rc0 = check_launch("topk");
    if (rc0 || order == 0) return rc0;
    int kp0 = 1;
    while (kp0 < k) kp0 <<= 1;
    sort_by_value_kernel<<<(unsigned)rows, 1024, (size_t)kp0 * 8, st>>>(p.in, p.is_float, row_stride, k, kp0, out);
    return check_launch("topk sort");
  }
  unsigned ncta = 1;
  while (ncta < 8 && (int64_t)ncta * 4096 < L) ncta <<= 1;
  if (L > (1 << 18)) ncta = 16;
  static bool attr_set = false;
  if (ncta > 8 && !attr_set) {
    if (cudaFuncSetAttribute(topk_cluster_kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) != cudaSuccess) {
      cudaGetLastError();
      ncta = 8;
    } else {
      attr_set = true;
    }
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(ncta, (unsigned)rows);
  cfg.blockDim = dim3(TK_THREADS);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = ncta;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, topk_cluster_kernel, p);
  if (e != cudaSuccess) return fail(PK_ERR_CUDA, "topk launch: %s", cudaGetErrorString(e));
  int rc = check_launch("topk");
  if (rc || order == 0) return rc;
  int kp = 1;
  while (kp < k) kp <<= 1;
  sort_by_value_kernel<<<(unsigned)rows, 1024, (size_t)kp * 8, st>>>(p.in, p.is_float, row_stride, k, kp, out);
  return check_launch("topk sort");
}

}  // namespace pk

using namespace pk;

extern "C" int pk_topk(const pk_tensor* input, int64_t k, const pk_tensor* out, int order, void* stream) {
  PK_REQUIRE(input && input->data, "input is null");
  PK_REQUIRE(input->dtype == PK_I32 || input->dtype == PK_F32, "input must be int32 or float32");
  PK_REQUIRE(input->ndim == 2, "input must be [rows, L]");
  PK_CHECK_TENSOR(out, PK_I64, 2);
  const int64_t rows = input->shape[0], L = input->shape[1];
  PK_REQUIRE(input->stride[1] == 1, "input must have last stride 1");
  PK_REQUIRE(k > 0 && k <= L, "k must be in 1..L (k=%lld, L=%lld)", (long long)k, (long long)L);
  PK_REQUIRE(L < (1ll << 31), "row too long");
  PK_REQUIRE(is_contig(out) && out->shape[0] == rows && out->shape[1] == k, "out must be contiguous [rows,k]");
  PK_REQUIRE(order == 0 || (order == 1 && k <= 4096), "order 1 (sorted by value) needs k <= 4096");
  if (rows == 0) return PK_OK;
  return launch_topk(input->data, input->dtype == PK_F32, rows, input->stride[0], L, k, (int64_t*)out->data, nullptr,
                     0, order, (cudaStream_t)stream, ST_TOPK);
}

extern "C" int pk_final_topk(const pk_tensor* scores, const pk_tensor* cand, int64_t K, const pk_tensor* out,
                             void* stream) {
  PK_CHECK_TENSOR(scores, PK_F32, 3);
  PK_CHECK_TENSOR(cand, PK_I64, 3);
  PK_CHECK_TENSOR(out, PK_I64, 3);
  const int64_t bs = scores->shape[0], H = scores->shape[1], C = scores->shape[2];
  PK_REQUIRE(is_contig(scores) && is_contig(cand) && is_contig(out), "scores, cand and out must be contiguous");
  PK_REQUIRE(cand->shape[0] == bs && cand->shape[1] == H && cand->shape[2] == C, "cand must be [bs,H,C]");
  PK_REQUIRE(K > 0 && K <= C, "K must be in 1..C");
  PK_REQUIRE(out->shape[0] == bs && out->shape[1] == H && out->shape[2] == K, "out must be [bs,H,K]");
  if (bs * H == 0) return PK_OK;
  return launch_topk(scores->data, true, bs * H, C, C, K, (int64_t*)out->data, (const int64_t*)cand->data, C, 0,
                     (cudaStream_t)stream, ST_FINAL_TOPK);
}

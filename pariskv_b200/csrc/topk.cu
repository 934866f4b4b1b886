// Exact, deterministic top-k of rows of 32-bit values (int32 counts or fp32 scores).
//
// One thread-block cluster per row: the row is cut into contiguous slices, one per CTA, and all exchange
// between the CTAs goes through distributed shared memory, so the whole selection is ONE launch with no
// global scratch.  Stage A buckets the VALUES linearly between the row's minimum and maximum into 2048 bins
// (a monotone map: bins above the threshold bin are selected outright, and the histogram is spread even when
// fp32 bit patterns share their high bits); stage B runs an exact 11-bit radix select over the few elements
// of the threshold bin.  Histograms are reduced by segments: CTA r sums bins [r*2048/n, (r+1)*2048/n) over the
// cluster, the CTA whose segment holds the threshold finds it and publishes it.
// Selected set: first k of (value descending, index ascending); emitted in ascending index.
#include <cooperative_groups.h>

#include "common.cuh"
#include "kernels.cuh"

namespace cg = cooperative_groups;

namespace pk {
namespace {

constexpr int TK_THREADS = 256;
constexpr int TK_BINS = 2048;

struct TopkParams {
  const uint32_t* in;
  int is_float;
  int64_t row_stride, L, k;
  int64_t* out;
  const int64_t* map;
  int64_t map_stride;
  // one-CTA kernel only: a launch row is segment (row % nseg) of input row (row / nseg), `seg` elements long (the last
  // one shorter); out_val, when set, receives the raw 32-bit values of the selected elements next to `out`
  int64_t nseg, seg;
  uint32_t* out_val;
};

constexpr int TK_CACHE = 16384;  // elements of a CTA's slice kept in (dynamic) shared memory; the rest is re-read from L2

__device__ __forceinline__ uint32_t load_key(const uint32_t* row, int64_t i, int is_float) {
  const uint32_t u = __ldg(row + i);
  return is_float ? ord_key(__uint_as_float(u)) : ord_key((int32_t)u);
}
__device__ __forceinline__ uint32_t key_of(uint32_t u, int is_float) {
  return is_float ? ord_key(__uint_as_float(u)) : ord_key((int32_t)u);
}
__device__ __forceinline__ float val_of(uint32_t u, int is_float) {
  return is_float ? __uint_as_float(u) : (float)(int32_t)u;
}

// Threshold bin of a[0..n) (shared memory, n a multiple of 256 or n < 256 a power of two): the bin where the
// suffix sum first reaches rem.  Result (bin, elements in higher bins, elements in the bin) in res[0..2].
__device__ void block_select(const unsigned* a, int n, unsigned rem, unsigned* s_warp, unsigned* res, int tid) {
  const int lane = tid & 31, warp = tid >> 5;
  const int per = max(1, n / TK_THREADS);
  const int b0 = tid * per;
  unsigned mine = 0;
  if (b0 < n)
    for (int i = 0; i < per; i++) mine += a[b0 + i];
  unsigned incl = mine;  // inclusive suffix over threads
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    unsigned o = __shfl_down_sync(0xffffffffu, incl, off);
    if (lane + off < 32) incl += o;
  }
  if (lane == 0) s_warp[warp] = incl;
  __syncthreads();
  unsigned higher = 0;
  for (int w = warp + 1; w < TK_THREADS / 32; w++) higher += s_warp[w];
  const unsigned suf = incl + higher;  // elements in bins >= b0
  unsigned above = suf - mine;         // elements in bins >= b0 + per
  if (b0 < n && suf >= rem && above < rem) {
    for (int i = per - 1; i >= 0; i--) {  // walk my bins from the top
      const unsigned v = a[b0 + i];
      if (above + v >= rem) {
        res[0] = (unsigned)(b0 + i), res[1] = above, res[2] = v;
        break;
      }
      above += v;
    }
  }
  __syncthreads();
}

// NCTA (cluster size) is a template parameter so that every loop over the ranks is unrolled and its remote
// shared-memory loads are issued together instead of one round trip after the other.
template <int NCTA>
__global__ void __launch_bounds__(TK_THREADS) topk_cluster_kernel(TopkParams p) {
  cg::cluster_group cluster = cg::this_cluster();
  __shared__ unsigned hist[TK_BINS];
  __shared__ unsigned seg[TK_BINS];        // my segment of the cluster-wide histogram (seg_bins entries used)
  __shared__ float cl_mm[2];               // min, max of my slice
  __shared__ unsigned cl_segtot;           // elements in my segment
  __shared__ unsigned cl_res[3];           // published by the CTA that owns the threshold bin
  __shared__ unsigned cl_cnt[2];           // n_gt, n_eq of my slice
  __shared__ unsigned cl_ao[2];            // AND, OR of the keys of the threshold bin in my slice
  __shared__ unsigned s_warp[TK_THREADS / 32];
  __shared__ float s_f[2 * TK_THREADS / 32];
  __shared__ unsigned long long s_scan[TK_THREADS / 32];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const unsigned rank = cluster.block_rank();
  constexpr unsigned ncta = NCTA;
  const int64_t row_id = blockIdx.y;
  const uint32_t* row = p.in + row_id * p.row_stride;
  const int64_t per_cta = (p.L + ncta - 1) / ncta;
  const int64_t begin = min(p.L, (int64_t)rank * per_cta), end = min(p.L, begin + per_cta);
  const int64_t span = (per_cta + TK_THREADS - 1) / TK_THREADS;
  const int64_t my_begin = min(end, begin + tid * span), my_end = min(end, my_begin + span);
  constexpr int seg_bins = TK_BINS / NCTA;

  // ---- the slice is read once, coalesced, into shared memory; every pass below works from there ----
  extern __shared__ uint32_t cache[];  // min(slice, TK_CACHE) words, sized by the launcher
  const int cache_n = (int)min((int64_t)TK_CACHE, end - begin);
  pdl_wait();
  pdl_trigger();
#pragma unroll 4
  for (int j = tid; j < cache_n; j += TK_THREADS) cache[j] = __ldg(row + begin + j);
  __syncthreads();
  auto raw = [&](int64_t i) -> uint32_t { return i - begin < cache_n ? cache[i - begin] : __ldg(row + i); };

  // ---- range of the row ----
  float mn = INFINITY, mx = -INFINITY;
  for (int64_t i = my_begin; i < my_end; i++) {
    const float v = val_of(raw(i), p.is_float);
    mn = fminf(mn, v);
    mx = fmaxf(mx, v);
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, off));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
  }
  if (lane == 0) s_f[warp] = mn, s_f[TK_THREADS / 32 + warp] = mx;
  for (int i = tid; i < TK_BINS; i += TK_THREADS) hist[i] = 0;
  __syncthreads();
  if (tid == 0) {
    for (int w = 1; w < TK_THREADS / 32; w++) {
      mn = fminf(mn, s_f[w]);
      mx = fmaxf(mx, s_f[TK_THREADS / 32 + w]);
    }
    cl_mm[0] = mn, cl_mm[1] = mx;
  }
  cluster.sync();
  {
    float a[NCTA], b[NCTA];
#pragma unroll
    for (int r = 0; r < NCTA; r++) {
      const float* mm = cluster.map_shared_rank(cl_mm, r);
      a[r] = mm[0], b[r] = mm[1];
    }
    mn = a[0], mx = b[0];
#pragma unroll
    for (int r = 1; r < NCTA; r++) mn = fminf(mn, a[r]), mx = fmaxf(mx, b[r]);
  }
  float scale = (float)(TK_BINS - 1) / (mx - mn);
  if (!(scale > 0.0f) || !(scale < INFINITY)) scale = 0.0f;  // flat or non-finite range: one bin, stage B decides
  auto bin_of = [&](float v) -> unsigned { return min((unsigned)(TK_BINS - 1), (unsigned)((v - mn) * scale)); };

  // Cluster-wide threshold bin of the local histograms `hist`: every CTA returns the same (bin, above, count).
  auto cluster_select = [&](unsigned rem, unsigned& bin, unsigned& above, unsigned& count) {
    cluster.sync();  // all local histograms are complete
    unsigned part = 0;
    for (int i = tid; i < seg_bins; i += TK_THREADS) {
      unsigned v[NCTA];
#pragma unroll
      for (int r = 0; r < NCTA; r++) v[r] = cluster.map_shared_rank(hist, r)[rank * seg_bins + i];
      unsigned t = 0;
#pragma unroll
      for (int r = 0; r < NCTA; r++) t += v[r];
      seg[i] = t;
      part += t;
    }
    part = __reduce_add_sync(0xffffffffu, part);
    if (lane == 0) s_warp[warp] = part;
    __syncthreads();
    if (tid == 0) {
      unsigned t = 0;
      for (int w = 0; w < TK_THREADS / 32; w++) t += s_warp[w];
      cl_segtot = t;
    }
    cluster.sync();  // segment totals are published; nobody reads remote histograms any more
    unsigned st[NCTA];
#pragma unroll
    for (int r = 0; r < NCTA; r++) st[r] = *cluster.map_shared_rank(&cl_segtot, r);
    unsigned higher = 0;
    int owner = 0;
    bool found = false;
#pragma unroll
    for (int r = NCTA - 1; r >= 0; r--) {
      if (!found) {
        if (higher + st[r] >= rem) {
          owner = r;
          found = true;
        } else {
          higher += st[r];
        }
      }
    }
    if ((int)rank == owner) {
      block_select(seg, seg_bins, rem - higher, s_warp, cl_res, tid);
      if (tid == 0) {
        cl_res[0] += owner * seg_bins;
        cl_res[1] += higher;
      }
    }
    cluster.sync();
    const unsigned* res = cluster.map_shared_rank(cl_res, owner);
    bin = res[0], above = res[1], count = res[2];
  };

  // ---- stage A: value buckets ----
  for (int64_t i = my_begin; i < my_end; i++) atomicAdd(&hist[bin_of(val_of(raw(i), p.is_float))], 1u);
  unsigned rem = (unsigned)p.k, tbin, ab, cb;
  cluster_select(rem, tbin, ab, cb);
  rem -= ab;
  unsigned prefix = 0, pmask = 0;
  if (cb != rem) {
    // Do the keys of the threshold bin differ at all?  (Integer counts never do: distinct counts fall into
    // distinct bins.)  AND / OR over the bin, reduced through the cluster.
    unsigned a = 0xffffffffu, o = 0u;
    for (int64_t i = my_begin; i < my_end; i++) {
      const uint32_t u = raw(i);
      if (bin_of(val_of(u, p.is_float)) != tbin) continue;
      const uint32_t k = key_of(u, p.is_float);
      a &= k, o |= k;
    }
    a = __reduce_and_sync(0xffffffffu, a);
    o = __reduce_or_sync(0xffffffffu, o);
    if (tid == 0) cl_ao[0] = 0xffffffffu, cl_ao[1] = 0u;
    __syncthreads();
    if (lane == 0) {
      atomicAnd(&cl_ao[0], a);
      atomicOr(&cl_ao[1], o);
    }
    cluster.sync();
    {
      unsigned aa[NCTA], oo[NCTA];
#pragma unroll
      for (int r = 0; r < NCTA; r++) {
        const unsigned* q = cluster.map_shared_rank(cl_ao, r);
        aa[r] = q[0], oo[r] = q[1];
      }
      a = aa[0], o = oo[0];
#pragma unroll
      for (int r = 1; r < NCTA; r++) a &= aa[r], o |= oo[r];
    }
    const unsigned varying = a ^ o;
    prefix = a & ~varying;
    pmask = ~varying;
    // ---- stage B: exact radix select of the rem-th largest key among the elements of the threshold bin ----
    for (int hi = varying ? 31 - __clz(varying) : -1; hi >= 0; hi -= 11) {
      const int lo = max(hi - 10, 0);
      const unsigned dm = ((hi == 31 ? 0u : (1u << (hi + 1))) - (1u << lo));
      // remote reads of `hist` ended before the second barrier of the previous cluster_select
      for (int i = tid; i < TK_BINS; i += TK_THREADS) hist[i] = 0;
      __syncthreads();
      for (int64_t i = my_begin; i < my_end; i++) {
        const uint32_t u = raw(i);
        if (bin_of(val_of(u, p.is_float)) != tbin) continue;
        const uint32_t k = key_of(u, p.is_float);
        if (((k ^ prefix) & pmask) == 0) atomicAdd(&hist[(k & dm) >> lo], 1u);
      }
      unsigned dbin;
      cluster_select(rem, dbin, ab, cb);
      prefix = (prefix & ~dm) | (dbin << lo);
      pmask |= dm;
      rem -= ab;
      if (cb == rem) break;  // the whole digit bin is taken; undecided bits of prefix stay zero
    }
  }
  const unsigned T = prefix;  // with the whole threshold bin taken T = 0 and every key of the bin is >= T

  // ---- count, scan, emit in index order ----
  unsigned n_gt = 0, n_eq = 0;
  for (int64_t i = my_begin; i < my_end; i++) {
    const uint32_t u = raw(i);
    const unsigned b = bin_of(val_of(u, p.is_float));
    const uint32_t k = key_of(u, p.is_float);
    n_gt += b > tbin || (b == tbin && k > T);
    n_eq += b == tbin && k == T;
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
    cl_cnt[0] = (unsigned)(total >> 32);
    cl_cnt[1] = (unsigned)total;
  }
  cluster.sync();
  unsigned gt_run = (unsigned)((base + incl - mine) >> 32), eq_run = (unsigned)(base + incl - mine);
  {
    unsigned g[NCTA], e[NCTA];
#pragma unroll
    for (int r = 0; r < NCTA; r++) {
      const unsigned* c2 = cluster.map_shared_rank(cl_cnt, r);
      g[r] = c2[0], e[r] = c2[1];
    }
#pragma unroll
    for (int r = 0; r < NCTA; r++)
      if ((unsigned)r < rank) gt_run += g[r], eq_run += e[r];
  }
  int64_t* out = p.out + row_id * p.k;
  const int64_t* map = p.map ? p.map + row_id * p.map_stride : nullptr;
  for (int64_t i = my_begin; i < my_end; i++) {
    const uint32_t u = raw(i);
    const unsigned b = bin_of(val_of(u, p.is_float));
    const uint32_t k = key_of(u, p.is_float);
    if (b > tbin || (b == tbin && k > T)) {
      out[gt_run + min(eq_run, rem)] = map ? map[i] : i;
      gt_run++;
    } else if (b == tbin && k == T) {
      if (eq_run < rem) out[gt_run + eq_run] = map ? map[i] : i;
      eq_run++;
    }
  }
  cluster.sync();  // shared memory must outlive the remote reads above
}

// ---- rows of up to 16384 elements: one 1024-thread CTA per row, everything in shared memory ----------------------
// Every element carries a state: 0 = out, 1 = selected, 2 = undecided.  A level histograms a monotone digit of the
// undecided elements, finds the digit T where the count from above reaches what is still needed, and decides every
// element whose digit differs from T.  Level 1 uses 4096 equal-width value buckets between the row's minimum and
// maximum (spread-out bins, so shared-memory atomics rarely collide); if the undecided set is still larger than
// TS_TIE_CAP — a flat row, or many equal values — radix levels on the key bits (12, 12, 8) follow.  As soon as at
// most TS_TIE_CAP elements are undecided they are ranked among themselves by (key descending, index ascending); if
// the last bit is reached with more equal keys than that, the lowest indices win through an ordered count.  The
// emission is an ordered compaction, so the result comes out in ascending index order like the cluster kernel's.
constexpr int TS_THREADS = 1024;
constexpr int TS_MAX = 16384;
constexpr int TS_TIE_CAP = 1024;
constexpr int TS_BINS = 4096;
constexpr size_t TS_SMEM = (size_t)TS_MAX * 4 + TS_BINS * 4 + TS_MAX + (size_t)TS_TIE_CAP * 8;

__global__ void __launch_bounds__(TS_THREADS) topk_small_kernel(TopkParams p) {
  extern __shared__ __align__(16) unsigned char ts_dyn[];
  uint32_t* raw = reinterpret_cast<uint32_t*>(ts_dyn);
  unsigned* hist = reinterpret_cast<unsigned*>(raw + TS_MAX);
  uint8_t* flag = reinterpret_cast<uint8_t*>(hist + TS_BINS);
  uint2* tie = reinterpret_cast<uint2*>(flag + TS_MAX);
  __shared__ unsigned s_wsum[32];
  __shared__ unsigned long long s_wsum64[32];
  __shared__ float s_f[64];
  __shared__ unsigned s_res[3];
  __shared__ unsigned s_ntie;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int64_t row = blockIdx.x;
  const int64_t in_row = row / p.nseg, seg_id = row % p.nseg;
  const int L = (int)min(p.seg, p.L - seg_id * p.seg);
  const uint32_t* in = p.in + in_row * p.row_stride + seg_id * p.seg;
  pdl_wait();
  pdl_trigger();
  float mn = INFINITY, mx = -INFINITY;
  for (int base = tid; base < L; base += 8 * TS_THREADS) {  // eight independent loads in flight per thread
    uint32_t u[8];
#pragma unroll
    for (int j = 0; j < 8; j++) {
      const int i = base + j * TS_THREADS;
      u[j] = i < L ? __ldg(in + i) : 0u;
    }
#pragma unroll
    for (int j = 0; j < 8; j++) {
      const int i = base + j * TS_THREADS;
      if (i < L) {
        raw[i] = u[j];
        flag[i] = 2;
        const float v = val_of(u[j], p.is_float);
        mn = fminf(mn, v), mx = fmaxf(mx, v);
      }
    }
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, off));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
  }
  if (lane == 0) s_f[warp] = mn, s_f[32 + warp] = mx;
  __syncthreads();
  mn = s_f[lane], mx = s_f[32 + lane];
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, off));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
  }
  float scale = (float)(TS_BINS - 1) / (mx - mn);
  if (!(scale > 0.0f) || !(scale < INFINITY)) scale = 0.0f;  // flat or non-finite range: the radix levels decide

  unsigned rem = (unsigned)p.k, undecided = (unsigned)L;
  // level 0: value buckets; levels 1..3: key bits [31:20], [19:8], [7:0]
  for (int lv = (scale > 0.0f ? 0 : 1); lv < 4 && undecided > (unsigned)TS_TIE_CAP; lv++) {
    const int nb = lv == 3 ? 256 : TS_BINS;
    const int sh = lv == 1 ? 20 : (lv == 2 ? 8 : 0);
    auto digit = [&](uint32_t u) -> unsigned {
      if (lv == 0) return min((unsigned)(TS_BINS - 1), (unsigned)((val_of(u, p.is_float) - mn) * scale));
      return (key_of(u, p.is_float) >> sh) & (unsigned)(nb - 1);
    };
    for (int i = tid; i < nb; i += TS_THREADS) hist[i] = 0;
    __syncthreads();
    for (int i = tid; i < L; i += TS_THREADS)
      if (flag[i] == 2) atomicAdd(&hist[digit(raw[i])], 1u);
    __syncthreads();
    // threshold digit: highest T with (undecided elements of digit >= T) >= rem
    const int per = nb >= TS_THREADS ? nb / TS_THREADS : 1;
    unsigned mine = 0;
    if (tid * per < nb)
      for (int j = 0; j < per; j++) mine += hist[tid * per + j];
    unsigned suf = mine;  // inclusive suffix sum over threads (higher thread = higher digits)
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const unsigned o = __shfl_down_sync(0xffffffffu, suf, off);
      if (lane + off < 32) suf += o;
    }
    if (lane == 0) s_wsum[warp] = suf;
    __syncthreads();
    unsigned higher_w = 0;
    for (int w = warp + 1; w < 32; w++) higher_w += s_wsum[w];
    const unsigned incl = suf + higher_w, higher = incl - mine;
    if (mine && higher < rem && incl >= rem) {  // the crossing lies inside this thread's digits
      unsigned acc = higher;
      for (int j = per - 1; j >= 0; j--) {
        const unsigned h = hist[tid * per + j];
        if (acc + h >= rem) {
          s_res[0] = (unsigned)(tid * per + j), s_res[1] = acc, s_res[2] = h;
          break;
        }
        acc += h;
      }
    }
    __syncthreads();
    const unsigned T = s_res[0];
    rem -= s_res[1];
    undecided = s_res[2];
    for (int i = tid; i < L; i += TS_THREADS)
      if (flag[i] == 2) {
        const unsigned d = digit(raw[i]);
        if (d != T) flag[i] = d > T ? 1 : 0;
      }
    __syncthreads();
  }

  if (undecided <= (unsigned)TS_TIE_CAP) {  // rank the undecided elements among themselves
    if (tid == 0) s_ntie = 0;
    __syncthreads();
    for (int i = tid; i < L; i += TS_THREADS)
      if (flag[i] == 2) tie[atomicAdd(&s_ntie, 1u)] = make_uint2(key_of(raw[i], p.is_float), (unsigned)i);
    __syncthreads();
    const int n = (int)s_ntie;
    for (int t = tid; t < n; t += TS_THREADS) {
      const uint2 me = tie[t];
      unsigned r = 0;
      for (int j = 0; j < n; j++) {
        const uint2 o = tie[j];
        r += (o.x > me.x || (o.x == me.x && o.y < me.y)) ? 1u : 0u;
      }
      flag[me.y] = r < rem ? 1 : 0;
    }
    __syncthreads();
  }
  // ordered compaction; elements still undecided here have equal keys and are taken in index order up to rem
  const int per = (L + TS_THREADS - 1) / TS_THREADS;
  const int i0 = min(L, tid * per), i1 = min(L, i0 + per);
  unsigned n_sel = 0, n_tie = 0;
  for (int i = i0; i < i1; i++) {
    const uint8_t f = flag[i];
    n_sel += f == 1, n_tie += f == 2;
  }
  const unsigned long long mine64 = ((unsigned long long)n_sel << 32) | n_tie;
  unsigned long long sc = mine64;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const unsigned long long o = __shfl_up_sync(0xffffffffu, sc, off);
    if (lane >= off) sc += o;
  }
  if (lane == 31) s_wsum64[warp] = sc;
  __syncthreads();
  unsigned long long base = 0;
  for (int w = 0; w < warp; w++) base += s_wsum64[w];
  const unsigned long long excl = base + sc - mine64;
  unsigned sel_before = (unsigned)(excl >> 32), tie_before = (unsigned)excl;
  int64_t* out = p.out + row * p.k;
  uint32_t* out_val = p.out_val ? p.out_val + row * p.k : nullptr;
  const int64_t* map = p.map ? p.map + in_row * p.map_stride + seg_id * p.seg : nullptr;
  int64_t mv[TS_MAX / TS_THREADS];  // the chunk's output values, fetched with independent loads (per <= 16)
#pragma unroll
  for (int j = 0; j < TS_MAX / TS_THREADS; j++) {
    const int i = i0 + j;
    mv[j] = (i < i1) ? (map ? __ldg(map + i) : seg_id * p.seg + (int64_t)i) : 0;
  }
#pragma unroll
  for (int j = 0; j < TS_MAX / TS_THREADS; j++) {
    const int i = i0 + j;
    if (i < i1) {
      const uint8_t f = flag[i];
      if (f == 1 || (f == 2 && tie_before < rem)) {
        const unsigned o = sel_before + min(tie_before, rem);
        out[o] = mv[j];
        if (out_val) out_val[o] = raw[i];
      }
      sel_before += f == 1;
      tie_before += f == 2;
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

int64_t topk_scratch_bytes(int64_t rows, int64_t L, int64_t k) {
  if (L <= TS_MAX || k < 1 || k > TS_MAX / 2) return 0;
  return rows * (int64_t)TS_MAX * 12;   // (value u32, index i64) of up to TS_MAX segment winners per row
}

int launch_topk(const void* in, bool is_float, int64_t rows, int64_t row_stride, int64_t L, int64_t k,
                int64_t* out, const int64_t* map, int64_t map_stride, int order, cudaStream_t st, int stage,
                void* scratch, int64_t scratch_bytes) {
  StageTimer tm(stage, st);
  TopkParams p;
  p.in = (const uint32_t*)in;
  p.is_float = is_float ? 1 : 0;
  p.row_stride = row_stride, p.L = L, p.k = k;
  p.out = out, p.map = map, p.map_stride = map_stride;
  p.nseg = 1, p.seg = L, p.out_val = nullptr;
  // dynamic shared memory above 48 KB is an opt-in per kernel AND per device
  static PerDevice small_attr;
  bool use_small = true;
  if (const unsigned long long bit = first_on_device(small_attr)) {
    if (cudaFuncSetAttribute(topk_small_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TS_SMEM) == cudaSuccess) {
      mark_on_device(small_attr, bit);
    } else {
      cudaGetLastError();
      use_small = false;  // this device refuses the opt-in: the cluster kernel below handles every row length
    }
  }
  if (use_small && L <= TS_MAX) {  // short rows: one CTA per row, no cluster barriers
    launch_chain(topk_small_kernel, dim3((unsigned)rows), dim3(TS_THREADS), TS_SMEM, st, p);
    int rc = check_launch("topk small");
    if (rc || order == 0) return rc;
    int kp = 1;
    while (kp < k) kp <<= 1;
    sort_by_value_kernel<<<(unsigned)rows, 1024, (size_t)kp * 8, st>>>(p.in, p.is_float, row_stride, k, kp, out);
    return check_launch("topk sort");
  }
  // Long rows with scratch from the caller: cut the row into nseg segments, take the top k of every segment with the
  // one-CTA kernel (nseg CTAs per row), then the top k of the nseg*k winners.  Exact: the k best of the row are among
  // the k best of their own segments, and the winners are listed segment by segment in ascending position, so the
  // tie rule (value descending, position ascending) is the same in both passes.
  if (use_small && order == 0 && L > TS_MAX && scratch && k >= 1) {
    int64_t nseg = TS_MAX / k;
    if (nseg > 16) nseg = 16;
    if (nseg >= 2 && (L + nseg - 1) / nseg > TS_MAX) nseg = 0;   // segments must fit the one-CTA kernel
    const int64_t seg = nseg >= 2 ? (L + nseg - 1) / nseg : 0;
    const bool fits = nseg >= 2 && L - (nseg - 1) * seg >= k && scratch_bytes >= rows * (int64_t)TS_MAX * 12 &&
                      rows * nseg < (1LL << 31);
    if (fits) {
      uint32_t* win_val = (uint32_t*)scratch;                                  // [rows][nseg*k]
      int64_t* win_idx = (int64_t*)((char*)scratch + rows * (int64_t)TS_MAX * 4);  // [rows][nseg*k], 8-byte aligned
      TopkParams a = p;
      a.nseg = nseg, a.seg = seg;
      a.out = win_idx, a.out_val = win_val;
      launch_chain(topk_small_kernel, dim3((unsigned)(rows * nseg)), dim3(TS_THREADS), TS_SMEM, st, a);
      int rc = check_launch("topk segments");
      if (rc) return rc;
      TopkParams b = p;
      b.in = win_val, b.row_stride = nseg * k, b.L = nseg * k, b.seg = nseg * k, b.nseg = 1;
      b.map = win_idx, b.map_stride = nseg * k;
      launch_chain(topk_small_kernel, dim3((unsigned)rows), dim3(TS_THREADS), TS_SMEM, st, b);
      return check_launch("topk merge");
    }
  }
  // about 1024 elements per CTA, at most 8 CTAs per row (the portable cluster size)
  unsigned ncta = 1;
  while (ncta < 8 && (int64_t)ncta * 1024 < L) ncta <<= 1;  // measured on B200: 8 CTAs per row is the fastest for rows of ~13 K
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(ncta, (unsigned)rows);
  cfg.blockDim = dim3(TK_THREADS);
  const int64_t slice = (L + ncta - 1) / ncta;
  cfg.dynamicSmemBytes = (size_t)(slice < TK_CACHE ? slice : TK_CACHE) * 4;
  static PerDevice cluster_attr;
  if (const unsigned long long bit = first_on_device(cluster_attr)) {
    cudaFuncSetAttribute(topk_cluster_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, TK_CACHE * 4);
    cudaFuncSetAttribute(topk_cluster_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, TK_CACHE * 4);
    cudaFuncSetAttribute(topk_cluster_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, TK_CACHE * 4);
    cudaFuncSetAttribute(topk_cluster_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, TK_CACHE * 4);
    if (cudaGetLastError() == cudaSuccess) mark_on_device(cluster_attr, bit);
  }
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = ncta;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
  cudaError_t e;
  switch (ncta) {
    case 1: e = cudaLaunchKernelEx(&cfg, topk_cluster_kernel<1>, p); break;
    case 2: e = cudaLaunchKernelEx(&cfg, topk_cluster_kernel<2>, p); break;
    case 4: e = cudaLaunchKernelEx(&cfg, topk_cluster_kernel<4>, p); break;
    default: e = cudaLaunchKernelEx(&cfg, topk_cluster_kernel<8>, p); break;
  }
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

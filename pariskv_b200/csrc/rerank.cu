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

// ---- candidate selection from u8 counts, rerank of the selected keys and the final top-K, one launch -----------
// One block per (chunk of keys, batch*head).  The per-chunk histograms written by the collision kernel
// give every block the global threshold count, the tie quota and its own output offset, so the candidate
// list comes out in ascending key order with no atomics and no second pass.  The block that finishes last for a
// (batch, head) then selects the final top-K of that head's fp32 scores (an arrival counter per head; the scores
// of the other blocks are read back from L2), so the chain needs no further launch.
constexpr int SEL_THREADS = 512;  // the first 256 threads own the 256 count bins
constexpr int FT_BINS = 4096;     // histogram bins of one radix pass of the final selection
constexpr int FT_KEYS_MAX = 16384;  // scores kept in shared memory by the final selection (the rest is re-read from L2)

struct SelParams {
  SelectArgs s;
  int small_cap;  // longest row that the all-in-shared-memory final selection takes (a multiple of 16)
  int key_cache;  // words of the shared-memory key cache of the general final selection
  int bitmap_words;  // words of the position bitmap of the histogram-based final selection (tie list behind it)
};

// ---- final top-K of one (batch, head) by one block ------------------------------------------------------------------
// Selected set = first K of (score descending, position ascending), emitted as cand[position] in ascending position
// (positions are ascending key indices).  Two forms: rows that fit the shared-memory cache, and longer ones.

// Block-wide exclusive scan of a packed pair of counters; returns (exclusive prefix, block total).
template <int NT>
__device__ __forceinline__ unsigned long long block_scan_excl(unsigned long long mine, unsigned long long* s_scan,
                                                              unsigned long long* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  unsigned long long sc = mine;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const unsigned long long o = __shfl_up_sync(0xffffffffu, sc, off);
    if (lane >= off) sc += o;
  }
  if (lane == 31) s_scan[warp] = sc;
  __syncthreads();
  unsigned long long before = 0, tot = 0;
#pragma unroll
  for (int w = 0; w < NT / 32; w++) {
    const unsigned long long v = s_scan[w];
    if (w < warp) before += v;
    tot += v;
  }
  *total = tot;
  return before + sc - mine;
}

// Threshold bin of hist[0..nb): the highest bin d with (elements in bins >= d) >= rem.  Result in res[0..2] =
// (d, elements in higher bins, elements in d); every thread returns after the result is visible.
template <int NT>
__device__ __forceinline__ void block_threshold_bin(const unsigned* hist, int nb, unsigned rem, unsigned* s_w, unsigned* res) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int per = nb >= NT ? nb / NT : 1;
  unsigned mine = 0;
  if (tid * per < nb)
    for (int j = 0; j < per; j++) mine += hist[tid * per + j];
  unsigned suf = mine;  // inclusive suffix sum over threads (higher thread = higher bins)
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const unsigned o = __shfl_down_sync(0xffffffffu, suf, off);
    if (lane + off < 32) suf += o;
  }
  if (lane == 0) s_w[warp] = suf;
  __syncthreads();
  unsigned higher_w = 0;
  for (int w = warp + 1; w < NT / 32; w++) higher_w += s_w[w];
  const unsigned incl = suf + higher_w, higher = incl - mine;
  if (mine && higher < rem && incl >= rem) {  // the crossing lies inside this thread's bins
    unsigned acc = higher;
    for (int j = per - 1; j >= 0; j--) {
      const unsigned hv = hist[tid * per + j];
      if (acc + hv >= rem) {
        res[0] = (unsigned)(tid * per + j), res[1] = acc, res[2] = hv;
        break;
      }
      acc += hv;
    }
  }
  __syncthreads();
}

constexpr int FT_TIES = 1024;  // elements of the threshold bin that are ranked among themselves

// Rows of at most `cap` scores, everything in shared memory: one histogram over FT_BINS equal-width VALUE bins between
// the row's minimum and maximum (a monotone map, and spread out, so shared-memory atomics rarely collide), the
// threshold bin, then the few elements of that bin ranked among themselves by (key descending, position ascending).
// Returns false (nothing written) when the threshold bin holds more than FT_TIES elements - a flat row; the caller
// then uses the general form.  raw: n words, hist: FT_BINS words, flag: n bytes, tie: FT_TIES uint2.
template <int NT>
__device__ bool final_select_cached(const float* __restrict__ scores, const int64_t* __restrict__ cand, int n, int K,
                                    int64_t* __restrict__ out, uint32_t* raw, unsigned* hist, uint8_t* flag, uint2* tie,
                                    unsigned* s_w, unsigned long long* s_scan) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  constexpr int NW = NT / 32;
  float mn = INFINITY, mx = -INFINITY;
  // The row starts anywhere (its stride may be odd): a few scalar loads up to the first 16-byte boundary, then
  // 16-byte loads, eight in flight per thread, so a row of 13 K scores is one round trip to L2.
  const int head = min(n, (int)((4 - ((reinterpret_cast<uintptr_t>(scores) >> 2) & 3)) & 3));
  if (tid < head) {
    const float v = __ldcg(scores + tid);
    raw[tid] = __float_as_uint(v);
    mn = fminf(mn, v), mx = fmaxf(mx, v);
  }
  const float4* s4 = reinterpret_cast<const float4*>(scores + head);
  const int n4 = (n - head) >> 2;
  for (int base = tid; base < n4; base += NT * 8) {
    float4 v[8];
#pragma unroll
    for (int j = 0; j < 8; j++) {
      const int i = base + j * NT;
      v[j] = i < n4 ? __ldcg(s4 + i) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    }
#pragma unroll
    for (int j = 0; j < 8; j++) {
      const int i = base + j * NT;
      if (i < n4) {
        uint32_t* r4 = raw + head + 4 * i;
        r4[0] = __float_as_uint(v[j].x), r4[1] = __float_as_uint(v[j].y);
        r4[2] = __float_as_uint(v[j].z), r4[3] = __float_as_uint(v[j].w);
        mn = fminf(fminf(mn, v[j].x), fminf(fminf(v[j].y, v[j].z), v[j].w));
        mx = fmaxf(fmaxf(mx, v[j].x), fmaxf(fmaxf(v[j].y, v[j].z), v[j].w));
      }
    }
  }
  for (int i = head + 4 * n4 + tid; i < n; i += NT) {
    const float v = __ldcg(scores + i);
    raw[i] = __float_as_uint(v);
    mn = fminf(mn, v), mx = fmaxf(mx, v);
  }
  for (int i = tid; i < FT_BINS; i += NT) hist[i] = 0;
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, off));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
  }
  if (lane == 0) s_w[warp] = __float_as_uint(mn), s_w[NW + warp] = __float_as_uint(mx);
  if (tid == 0) s_w[2 * NW + 3] = 0;  // tie counter
  __syncthreads();
  mn = __uint_as_float(s_w[lane < NW ? lane : 0]), mx = __uint_as_float(s_w[NW + (lane < NW ? lane : 0)]);
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, off));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
  }
  float scale = (float)(FT_BINS - 1) / (mx - mn);
  if (!(scale > 0.0f) || !(scale < INFINITY)) return false;  // flat or non-finite range (the same for every thread)
  auto bin_of = [&](uint32_t u) -> unsigned {
    return min((unsigned)(FT_BINS - 1), (unsigned)((__uint_as_float(u) - mn) * scale));
  };
  for (int i = tid; i < n; i += NT) atomicAdd(&hist[bin_of(raw[i])], 1u);
  __syncthreads();
  block_threshold_bin<NT>(hist, FT_BINS, (unsigned)K, s_w, s_w + 2 * NW);
  const unsigned T = s_w[2 * NW], above = s_w[2 * NW + 1], in_bin = s_w[2 * NW + 2];
  if (in_bin > (unsigned)FT_TIES) return false;
  const unsigned rem = (unsigned)K - above;  // taken from the threshold bin
  for (int i = tid; i < n; i += NT) {
    const uint32_t u = raw[i];
    const unsigned bn = bin_of(u);
    uint8_t f = bn > T ? 1 : 0;
    if (bn == T) {
      f = 2;
      tie[atomicAdd(&s_w[2 * NW + 3], 1u)] = make_uint2(ord_key(__uint_as_float(u)), (unsigned)i);
    }
    flag[i] = f;
  }
  __syncthreads();
  const int n_tie = (int)s_w[2 * NW + 3];
  for (int t = tid; t < n_tie; t += NT) {
    const uint2 me = tie[t];
    unsigned rk = 0;
    for (int j = 0; j < n_tie; j++) {
      const uint2 o = tie[j];
      rk += (o.x > me.x || (o.x == me.x && o.y < me.y)) ? 1u : 0u;
    }
    flag[me.y] = rk < rem ? 1 : 0;
  }
  __syncthreads();
  // ordered compaction: a contiguous span of positions per thread, one scan; the selected positions go to a list in
  // shared memory (over the histogram, K <= FT_BINS), so that the candidate ids are then fetched in one batch
  const int per = (n + NT - 1) / NT;
  const int i0 = min(n, tid * per), i1 = min(n, i0 + per);
  unsigned cnt = 0;
  for (int i = i0; i < i1; i++) cnt += flag[i];
  unsigned long long total;
  unsigned pos = (unsigned)block_scan_excl<NT>((unsigned long long)cnt, s_scan, &total);
  if (K <= FT_BINS) {
    unsigned* sel = hist;
    for (int i = i0; i < i1; i++)
      if (flag[i]) sel[pos++] = (unsigned)i;
    __syncthreads();
    for (int base = tid; base < K; base += NT * 8) {
      int64_t cv[8];
#pragma unroll
      for (int j = 0; j < 8; j++) cv[j] = base + j * NT < K ? __ldcg(cand + sel[base + j * NT]) : 0;
#pragma unroll
      for (int j = 0; j < 8; j++)
        if (base + j * NT < K) out[base + j * NT] = cv[j];
    }
  } else {
    for (int i = i0; i < i1; i += 8) {  // the candidate ids of up to eight selected positions are fetched together
      int64_t cv[8];
#pragma unroll
      for (int j = 0; j < 8; j++) cv[j] = (i + j < i1 && flag[i + j]) ? __ldcg(cand + i + j) : 0;
#pragma unroll
      for (int j = 0; j < 8; j++)
        if (i + j < i1 && flag[i + j]) out[pos++] = cv[j];
    }
  }
  return true;
}

// Long rows.  While the scores were computed, every block added them to a histogram over the top VH_BITS bits of the
// ordered key (sign, exponent, five mantissa bits) in global memory, so the block that finishes last starts with the
// threshold bin in hand: it reads the histogram once (32 bins per thread, highest bins first), then walks the row
// twice with coalesced loads, sixteen in flight per thread: once to collect the threshold bin's elements, which are
// ranked among themselves (value descending, position ascending) and marked in a position bitmap, once to emit the
// selected positions in order.  A warp covers 1024 consecutive positions per round; lane g receives, by ballot, the
// mask of positions [32 g, 32 g + 32) and owns them in the block-wide scan.
// Returns false (nothing written) when the threshold bin holds more than FT_TIES elements.
constexpr int VH_BITS = 14;
constexpr int VH_BINS = 1 << VH_BITS;
constexpr int VH_SHIFT = 32 - VH_BITS;

template <int NT>
__device__ bool final_select_hist(const float* __restrict__ scores, const int64_t* __restrict__ cand, int n, int K,
                                  int64_t* __restrict__ out, const unsigned* __restrict__ vhist, unsigned* bitmap,
                                  uint2* tie, unsigned* sel /*K words or null*/, unsigned* s_w,
                                  unsigned long long* s_scan) {
  static_assert(VH_BINS == NT * 32, "32 histogram bins per thread");
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // ---- threshold bin: thread 0 holds the highest 32 bins ----
  const int top = VH_BINS - 32 * (tid + 1);
  unsigned sum = 0;
#pragma unroll
  for (int j = 0; j < 8; j++) {
    const uint4 v = __ldcg(reinterpret_cast<const uint4*>(vhist + top) + j);
    sum += v.x + v.y + v.z + v.w;
  }
  unsigned long long total;
  const unsigned before = (unsigned)block_scan_excl<NT>((unsigned long long)sum, s_scan, &total);
  if (tid == 0) s_w[3] = 0;  // tie counter
  {  // the K-th largest lies in the 32 bins of exactly one thread; its warp looks at them together, lane l at bin 31 - l
    const bool has = before < (unsigned)K && (unsigned)K <= before + sum;
    const unsigned who = __ballot_sync(0xffffffffu, has);
    if (who) {
      const int f = __ffs(who) - 1;
      const int ftop = __shfl_sync(0xffffffffu, top, f);
      const unsigned fbefore = __shfl_sync(0xffffffffu, before, f);
      const unsigned cj = __ldcg(vhist + ftop + 31 - lane);
      unsigned incl = cj;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const unsigned o = __shfl_up_sync(0xffffffffu, incl, off);
        if (lane >= off) incl += o;
      }
      const unsigned hit = __ballot_sync(0xffffffffu, fbefore + incl >= (unsigned)K);
      if (hit && lane == __ffs(hit) - 1) s_w[0] = (unsigned)(ftop + 31 - lane), s_w[1] = fbefore + incl - cj, s_w[2] = cj;
    }
  }
  const int n_words = (n + 31) >> 5;
  for (int i = tid; i < n_words; i += NT) bitmap[i] = 0;
  __syncthreads();
  const unsigned T = s_w[0], above = s_w[1], in_bin = s_w[2];
  if ((unsigned)total < (unsigned)K || in_bin > (unsigned)FT_TIES) return false;  // (an inconsistent histogram too)
  const unsigned rem = (unsigned)K - above;
  // ---- the threshold bin's elements ----
  for (int base = tid; base < n; base += NT * 16) {
    float v[16];
#pragma unroll
    for (int j = 0; j < 16; j++) v[j] = base + j * NT < n ? __ldcg(scores + base + j * NT) : 0.0f;
#pragma unroll
    for (int j = 0; j < 16; j++) {
      const int i = base + j * NT;
      const unsigned k = ord_key(v[j]);
      if (i < n && (k >> VH_SHIFT) == T) {
        const unsigned at = atomicAdd(&s_w[3], 1u);
        if (at < (unsigned)FT_TIES) tie[at] = make_uint2(k, (unsigned)i);
      }
    }
  }
  __syncthreads();
  const int n_tie = (int)min(s_w[3], (unsigned)FT_TIES);
  for (int t = tid; t < n_tie; t += NT) {
    const uint2 me = tie[t];
    unsigned rk = 0;
    for (int j = 0; j < n_tie; j++) {
      const uint2 o = tie[j];
      rk += (o.x > me.x || (o.x == me.x && o.y < me.y)) ? 1u : 0u;
    }
    if (rk < rem) atomicOr(&bitmap[me.y >> 5], 1u << (me.y & 31));
  }
  __syncthreads();
  // ---- ordered emission ----
  unsigned long long run = 0;
  for (int rb = 0; rb < n; rb += NT * 32) {
    const int wb = rb + warp * 1024;
    unsigned mine = 0;
#pragma unroll
    for (int half = 0; half < 2; half++) {
      float v[16];
#pragma unroll
      for (int g = 0; g < 16; g++) {
        const int pos = wb + (half * 16 + g) * 32 + lane;
        v[g] = pos < n ? __ldcg(scores + pos) : 0.0f;
      }
#pragma unroll
      for (int g = 0; g < 16; g++) {
        const int pos = wb + (half * 16 + g) * 32 + lane;
        const bool gt = pos < n && (ord_key(v[g]) >> VH_SHIFT) > T;
        const unsigned m = __ballot_sync(0xffffffffu, gt);
        if (lane == half * 16 + g) mine = m;
      }
    }
    const int gbase = wb + lane * 32;  // this lane's 32 positions
    unsigned take = mine | (gbase < n ? bitmap[gbase >> 5] : 0u);
    unsigned long long tot_round;
    unsigned o = (unsigned)(run + block_scan_excl<NT>((unsigned long long)__popc(take), s_scan, &tot_round));
    while (take) {  // positions first (shared memory); the candidate ids are fetched afterwards, many loads in flight
      const int j = __ffs(take) - 1;
      take &= take - 1;
      if (o < (unsigned)K) {
        if (sel) sel[o] = (unsigned)(gbase + j);
        else out[o] = __ldcg(cand + gbase + j);
      }
      o++;
    }
    run += tot_round;
    __syncthreads();
  }
  if (sel) {
    for (int base = tid; base < K; base += NT * 8) {
      int64_t cv[8];
#pragma unroll
      for (int j = 0; j < 8; j++) cv[j] = base + j * NT < K ? __ldcg(cand + sel[base + j * NT]) : 0;
#pragma unroll
      for (int j = 0; j < 8; j++)
        if (base + j * NT < K) out[base + j * NT] = cv[j];
    }
  }
  return true;
}

// Any row length: scores are mapped to order-preserving 32-bit keys; radix passes of up to 12 bits, starting at the
// highest bit in which the keys differ at all, narrow the threshold key down; ties of the full key go to the lowest
// positions.  keys: shared-memory cache of the first `cap` keys (the rest is re-read from L2); hist: FT_BINS words.
template <int NT>
__device__ void final_select_general(const float* __restrict__ scores, const int64_t* __restrict__ cand, int n, int K,
                                     int64_t* __restrict__ out, uint32_t* keys, int cap, unsigned* hist,
                                     unsigned* s_w /*[NT/32 * 2 + 4]*/, unsigned long long* s_scan /*[NT/32]*/) {
  constexpr int NW = NT / 32;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // pass 0: keys into shared memory, range of the keys
  unsigned kmin = 0xffffffffu, kmax = 0u;
  for (int base = tid; base < n; base += NT * 8) {
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; j++) {
      const int i = base + j * NT;
      v[j] = i < n ? __ldcg(scores + i) : 0.0f;
    }
#pragma unroll
    for (int j = 0; j < 8; j++) {
      const int i = base + j * NT;
      if (i < n) {
        const unsigned k = ord_key(v[j]);
        if (i < cap) keys[i] = k;
        kmin = min(kmin, k), kmax = max(kmax, k);
      }
    }
  }
  kmin = __reduce_min_sync(0xffffffffu, kmin);
  kmax = __reduce_max_sync(0xffffffffu, kmax);
  if (lane == 0) s_w[warp] = kmin, s_w[NW + warp] = kmax;
  __syncthreads();
  kmin = s_w[lane < NW ? lane : 0], kmax = s_w[NW + (lane < NW ? lane : 0)];
  kmin = __reduce_min_sync(0xffffffffu, kmin);
  kmax = __reduce_max_sync(0xffffffffu, kmax);
  __syncthreads();  // s_w is reused below
  auto key_at = [&](int i) -> unsigned { return i < cap ? keys[i] : ord_key(__ldcg(scores + i)); };

  // bits above the highest differing bit are common to all keys: decided from the start
  int top = (kmin == kmax) ? -1 : 31 - __clz(kmin ^ kmax);
  unsigned dm = top >= 31 ? 0u : (top < 0 ? 0xffffffffu : ~((2u << top) - 1u));  // mask of decided bits
  unsigned prefix = kmax & dm;
  unsigned rem = (unsigned)K;
  while (top >= 0) {
    const int lo = max(top - 11, 0);
    const int nb = 1 << (top - lo + 1);
    for (int i = tid; i < nb; i += NT) hist[i] = 0;
    __syncthreads();
    for (int i = tid; i < n; i += NT) {
      const unsigned k = key_at(i);
      if ((k & dm) == prefix) atomicAdd(&hist[(k >> lo) & (unsigned)(nb - 1)], 1u);
    }
    __syncthreads();
    block_threshold_bin<NT>(hist, nb, rem, s_w, s_w + 2 * NW);
    const unsigned d = s_w[2 * NW], above = s_w[2 * NW + 1], cnt = s_w[2 * NW + 2];
    __syncthreads();
    rem -= above;
    prefix |= d << lo;
    dm |= (unsigned)(nb - 1) << lo;
    top = lo - 1;
    if (cnt == rem) break;  // the whole digit bin is taken
  }
  const unsigned quota = rem;  // elements with (key & dm) == prefix that are taken, lowest positions first

  // ordered emission: 16 consecutive positions per thread and round
  unsigned long long run = 0;  // (selected outright << 32 | ties) before this round
  for (int base = 0; base < n; base += NT * 16) {
    const int i0 = base + tid * 16;
    unsigned gt_mask = 0, eq_mask = 0;
#pragma unroll
    for (int q4 = 0; q4 < 4; q4++) {
      const int i = i0 + 4 * q4;
      unsigned k4[4];
      if (i + 4 <= n && i + 4 <= cap) {
        const uint4 a = *reinterpret_cast<const uint4*>(keys + i);
        k4[0] = a.x, k4[1] = a.y, k4[2] = a.z, k4[3] = a.w;
      } else {
#pragma unroll
        for (int j = 0; j < 4; j++) k4[j] = i + j < n ? key_at(i + j) : 0u;
      }
#pragma unroll
      for (int j = 0; j < 4; j++) {
        const bool ok = i + j < n;
        const unsigned kh = k4[j] & dm;
        gt_mask |= (unsigned)(ok && kh > prefix) << (4 * q4 + j);
        eq_mask |= (unsigned)(ok && kh == prefix) << (4 * q4 + j);
      }
    }
    const unsigned long long mine = ((unsigned long long)__popc(gt_mask) << 32) | (unsigned)__popc(eq_mask);
    unsigned long long total;
    const unsigned long long before = run + block_scan_excl<NT>(mine, s_scan, &total);
    unsigned g = (unsigned)(before >> 32), e = (unsigned)before;
    // which of my sixteen are taken: everything above the threshold, ties while the quota lasts
    unsigned take = gt_mask;
    {
      unsigned em = eq_mask, ee = e;
      while (em && ee < quota) {
        const int j = __ffs(em) - 1;
        take |= 1u << j;
        em &= em - 1;
        ee++;
      }
    }
    unsigned o = g + min(e, quota);
#pragma unroll
    for (int h8 = 0; h8 < 2; h8++) {
      int64_t cv[8];
#pragma unroll
      for (int j = 0; j < 8; j++) cv[j] = ((take >> (8 * h8 + j)) & 1u) ? __ldcg(cand + i0 + 8 * h8 + j) : 0;
#pragma unroll
      for (int j = 0; j < 8; j++)
        if ((take >> (8 * h8 + j)) & 1u) out[o++] = cv[j];
    }
    run += total;
    __syncthreads();
  }
}

template <bool FAST>
__global__ void __launch_bounds__(SEL_THREADS, FAST ? 2 : 1) select_rerank_kernel(RerankArgs a, SelParams pp) {
  extern __shared__ __align__(16) unsigned char dyn[];
  const SelectArgs& p = pp.s;
  RerankSmem& sm = *reinterpret_cast<RerankSmem*>(dyn);
  int* list = reinterpret_cast<int*>(dyn + sizeof(RerankSmem));  // selected keys of this chunk, in order
  __shared__ unsigned tot[256], pre[256];
  __shared__ unsigned s_warp[2 * (SEL_THREADS / 32) + 4];
  __shared__ unsigned s_misc[8];  // t, quota, gt_base, eq_base, gt_total, last-block flag
  __shared__ unsigned long long s_scan[SEL_THREADS / 32];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int64_t bh = blockIdx.y, chunk = blockIdx.x;
  const int b = (int)(bh / a.H), h = (int)(bh % a.H);
  pdl_wait();  // counts, block histograms, query blocks and the zeroed arrival counters come from the collision kernel
  pdl_trigger();
  const int64_t N = p.n_dev ? min(max((int64_t)p.n_dev[b], (int64_t)1), p.N) : p.N;
  const int64_t Nv = N + p.mis;
  const int64_t v_begin = chunk * p.chunk_keys;
  if (v_begin >= Nv) return;  // beyond this sample's zone (whole block, before any barrier)
  const int64_t v_end = min(Nv, v_begin + p.chunk_keys);
  const int64_t live_chunks = (Nv + p.chunk_keys - 1) / p.chunk_keys;
  // candidates wanted over the whole zone (all shards together)
  const int64_t C_want = p.n_dev ? min((int64_t)zone_candidates(p.sched, N), p.C) : p.C_want;
  // this block's counts (one 16-byte load per thread and round of the scan below): issued first, needed last
  const uint8_t* cnt = p.counts_u8 + bh * p.u8_stride;
  uint4 cnt0 = make_uint4(0, 0, 0, 0);
  if (v_begin + 16 * (int64_t)tid < v_end) cnt0 = __ldcg(reinterpret_cast<const uint4*>(cnt + v_begin + 16 * (int64_t)tid));
  rerank_setup(sm, a, bh, tid, SEL_THREADS);
  // Bin `tid & 255` of the histogram rows: the two halves of the block take alternate rows, sixteen loads in flight
  // per thread, so a few dozen rows cost one round trip to L2.
  unsigned g_tot = 0, g_before = 0;  // sharded: bin totals over all shards / over the shards before this one
  {
    const int bin = tid & 255, par = tid >> 8;
    const uint32_t* hp = p.chunk_hist + bh * p.n_chunks * 256 + bin;
    unsigned t = 0, pr = 0;
    for (int64_t c0 = par; c0 < live_chunks; c0 += 32) {
      unsigned v[16];
#pragma unroll
      for (int i = 0; i < 16; i++) v[i] = (c0 + 2 * i < live_chunks) ? __ldcg(hp + (c0 + 2 * i) * 256) : 0u;
#pragma unroll
      for (int i = 0; i < 16; i++) {
        t += v[i];
        if (c0 + 2 * i < chunk) pr += v[i];
      }
    }
    if (par) tot[bin] = t, pre[bin] = pr;
    __syncthreads();
    if (!par) {
      t += tot[bin], pr += pre[bin];
      tot[bin] = t, pre[bin] = pr;
      g_tot = t;
      if (p.shard_hist) {
        g_tot = 0;
        const int64_t rows = (int64_t)gridDim.y;  // bs*H
        for (int r = 0; r < p.world; r++) {
          const unsigned v = __ldg(p.shard_hist + ((int64_t)r * rows + bh) * 256 + bin);
          g_tot += v;
          if (r < p.rank) g_before += v;
        }
      }
    }
  }
  if (tid < 8) s_misc[tid] = 0;
  __syncthreads();
  // threshold bin: suffix sums over 256 bins (8 warps x 32 bins)
  unsigned v = tid < 256 ? g_tot : 0u, incl = v;
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
    if (suf >= (unsigned)C_want && above < (unsigned)C_want) {
      s_misc[0] = (unsigned)tid;
      // ties of the threshold count taken over the whole zone; a shard takes what the shards before it left
      const unsigned q_all = (unsigned)C_want - above;
      const unsigned left = q_all > g_before ? q_all - g_before : 0u;
      s_misc[1] = p.shard_hist ? min(left, tot[tid]) : q_all;
    }
  }
  __syncthreads();
  const unsigned T = s_misc[0], quota = s_misc[1];
  if (tid < 256 && (unsigned)tid > T) {
    if (pre[tid]) atomicAdd(&s_misc[2], pre[tid]);
    if (tot[tid]) atomicAdd(&s_misc[4], tot[tid]);
  }
  if ((unsigned)tid == T) s_misc[3] = pre[tid];
  __syncthreads();
  const unsigned gt_base = s_misc[2], eq_base = s_misc[3];
  // candidates of this (batch, head) held by this shard
  const int64_t C_here = min((int64_t)s_misc[4] + (int64_t)min(tot[T], quota), p.C);

  unsigned gt_run = 0, eq_run = 0;  // running counts over this chunk (all threads hold the same values)
  unsigned n_list = 0;
  for (int64_t t0 = v_begin; t0 < v_end; t0 += 16 * SEL_THREADS) {
    const int64_t v0 = t0 + 16 * (int64_t)tid;
    uint32_t w4[4] = {cnt0.x, cnt0.y, cnt0.z, cnt0.w};  // first round: loaded at the top of the kernel
    if (t0 != v_begin) {
      w4[0] = w4[1] = w4[2] = w4[3] = 0;
      if (v0 < v_end) {
        const uint4 r = __ldcg(reinterpret_cast<const uint4*>(cnt + v0));
        w4[0] = r.x, w4[1] = r.y, w4[2] = r.z, w4[3] = r.w;
      }
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
  const int64_t row_base = bh * p.C;
  const int64_t out_pos = (int64_t)gt_base + min(eq_base, quota);
  const float qn = bf2f(a.q_norm[bh]);
  const uint8_t* k4 = a.k4 + b * a.k4_b + h * a.k4_h;
  const uint16_t* w = a.w + b * a.w_b + h * a.w_h;
  for (unsigned i = tid; i < n_list; i += SEL_THREADS) {
    if (out_pos + i >= p.C) break;  // cannot happen with consistent histograms; keeps a bad input inside the row
    const int64_t key = list[i];
    const float s = rerank_one<FAST>(sm, a, k4, w, key, qn, lane, nullptr, 0);
    p.scores_f32[row_base + out_pos + i] = s;
    p.cand_out[row_base + out_pos + i] = key;
    if (p.val_hist) atomicAdd(p.val_hist + bh * VH_BINS + (ord_key(s) >> VH_SHIFT), 1u);
  }
  if (chunk == 0) {
    if (tid == 0 && p.n_cand_out) p.n_cand_out[bh] = (int32_t)C_here;
    // per-sample lengths or shards: rows are longer than this candidate list; the tail gets (score -inf, key 0), so
    // a consumer that walks whole rows (the adaptive selection, a separate top-K launch) gives those entries no weight
    if (p.fill_tail)
      for (int64_t i = C_here + tid; i < p.C; i += SEL_THREADS) {
        p.scores_f32[row_base + i] = -INFINITY;
        p.cand_out[row_base + i] = 0;
      }
  }
  if (p.K <= 0) return;

  // ---- the block that arrives last for this (batch, head) selects the final top-K ----
  __threadfence();
  __syncthreads();
  if (tid == 0) s_misc[5] = atomicAdd(p.counters + bh, 1u) + 1u == (unsigned)live_chunks;
  __syncthreads();
  if (!s_misc[5]) return;
  __threadfence();
  const int K_here = (int)min(p.K, C_here);
  if (K_here > 0) {
    // shared memory of the final stage (over the candidate list, no longer needed):
    // [histogram FT_BINS words | scores / keys | flags | tie list]
    unsigned* hist = reinterpret_cast<unsigned*>(list);
    uint32_t* keys = reinterpret_cast<uint32_t*>(list) + FT_BINS;
    bool done = false;
    if (C_here <= pp.small_cap) {
      uint8_t* flag = reinterpret_cast<uint8_t*>(keys + pp.small_cap);
      uint2* tie = reinterpret_cast<uint2*>(flag + pp.small_cap);
      done = final_select_cached<SEL_THREADS>(p.scores_f32 + row_base, p.cand_out + row_base, (int)C_here, K_here,
                                              p.final_out + bh * p.K, keys, hist, flag, tie, s_warp, s_scan);
      __syncthreads();
    }
    if (!done && p.val_hist && (C_here + 31) / 32 <= pp.bitmap_words) {
      unsigned* bitmap = reinterpret_cast<unsigned*>(list);
      uint2* tie = reinterpret_cast<uint2*>(bitmap + pp.bitmap_words);
      // the position list sits in the unused upper part of the bitmap area when there is room for it
      const int n_words = (int)((C_here + 31) / 32);
      unsigned* sel = n_words + K_here <= pp.bitmap_words ? bitmap + n_words : nullptr;
      done = final_select_hist<SEL_THREADS>(p.scores_f32 + row_base, p.cand_out + row_base, (int)C_here, K_here,
                                            p.final_out + bh * p.K, p.val_hist + bh * VH_BINS, bitmap, tie, sel, s_warp,
                                            s_scan);
      __syncthreads();
    }
    if (!done)
      final_select_general<SEL_THREADS>(p.scores_f32 + row_base, p.cand_out + row_base, (int)C_here, K_here,
                                        p.final_out + bh * p.K, keys, pp.key_cache, hist, s_warp, s_scan);
  }
  if (tid == 0) {
    if (p.n_sel_out) p.n_sel_out[bh] = K_here;
    p.counters[bh] = 0;
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

namespace {
inline int64_t final_small_cap(int64_t C) { return (C < FT_KEYS_MAX ? (C + 15) / 16 * 16 : (int64_t)FT_KEYS_MAX); }
}  // namespace

int64_t select_final_max_row() { return FT_KEYS_MAX; }
int64_t select_value_bins() { return VH_BINS; }

int64_t select_smem_bytes(int64_t chunk_keys, int64_t C, int64_t K) {
  int64_t body = chunk_keys * (int64_t)sizeof(int);  // the chunk's candidate list
  if (K > 0) {
    const int64_t cap = final_small_cap(C);
    const int64_t ft = ((int64_t)FT_BINS + cap) * 4 + cap + (int64_t)FT_TIES * 8;
    if (ft > body) body = ft;
  }
  return (int64_t)sizeof(RerankSmem) + body;
}

int launch_select_rerank(const RerankArgs& a, int64_t bs_h, const SelectArgs& sa, cudaStream_t st) {
  SelParams p;
  p.s = sa;
  const int64_t smem = select_smem_bytes(sa.chunk_keys, sa.C, sa.K);
  p.small_cap = sa.K > 0 ? (int)final_small_cap(sa.C) : 0;
  p.key_cache = sa.K > 0 ? (int)((smem - (int64_t)sizeof(RerankSmem)) / 4 - FT_BINS) : 0;
  p.bitmap_words = sa.K > 0 ? (int)((smem - (int64_t)sizeof(RerankSmem) - (int64_t)FT_TIES * 8) / 4) : 0;
  if (sa.C >= (1ll << 31) || sa.N >= (1ll << 31)) return fail(PK_ERR_ARG, "zone too long for the selection kernel");
  dim3 grid((unsigned)sa.n_chunks, (unsigned)bs_h);
  const bool fast = rerank_fast_layout(a);
  auto kern = fast ? select_rerank_kernel<true> : select_rerank_kernel<false>;
  // dynamic + static shared memory above 48 KB is an opt-in per device: set on every launch that may need it (the
  // kernel's static part is a few KB, so the margin is taken generously)
  if (smem > 40 * 1024) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return check_launch("select_rerank smem");
  }
  StageTimer tm(ST_SELECT_RERANK, st);
  launch_chain(kern, grid, dim3(SEL_THREADS), (size_t)smem, st, a, p);
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


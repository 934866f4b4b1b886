// Cluster ranking, tier look-up tables and the weighted multi-tier collision count.
//
// The six cumulative tier bitsets of a subspace collapse into one 256-entry byte table (number of tiers a
// cluster belongs to), 4 KB per (batch, head) in shared memory at a link-time address, so one look-up is a
// byte extract, a byte load with an immediate offset and an add.  Codes are streamed with 128-bit loads,
// every thread keeps 256 bytes in flight before it starts counting.
#include <mutex>

#include "common.cuh"
#include "kernels.cuh"
#include "rotate.cuh"

namespace pk {
namespace {

struct Tiers {
  long long t[8];
  int n;
};

// ---- table builders -----------------------------------------------------------------------------

// From a given cluster order (the collision_fused op): one block per (batch, head, subspace).
template <typename IdT>
__global__ void __launch_bounds__(256) lut_from_sorted_kernel(const IdT* __restrict__ ids,
                                                              const int32_t* __restrict__ counts, int NC,
                                                              Tiers tiers, uint32_t* __restrict__ lut) {
  __shared__ long long warp_tot[8];
  __shared__ unsigned mask[256];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int64_t blk = blockIdx.x;
  mask[tid] = 0;
  long long id = -1;
  long long cnt = 0;
  if (tid < NC) {
    id = (long long)ids[blk * NC + tid];
    if (id >= 0 && id < NC) cnt = counts[blk * NC + id];
  }
  long long incl = cnt;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    long long v = __shfl_up_sync(0xffffffffu, incl, off);
    if (lane >= off) incl += v;
  }
  if (lane == 31) warp_tot[warp] = incl;
  __syncthreads();
  long long base = 0;
  for (int w = 0; w < warp; w++) base += warp_tot[w];
  const long long excl = base + incl - cnt;
  unsigned bits = 0;
  for (int t = 0; t < tiers.n; t++)
    if (excl < tiers.t[t]) bits |= 1u << t;
  if (id >= 0 && id < NC && bits) atomicOr(&mask[id], bits);
  __syncthreads();
  if (tid < 64) {
    uint32_t w = 0;
#pragma unroll
    for (int i = 0; i < 4; i++) w |= (uint32_t)__popc(mask[tid * 4 + i]) << (8 * i);
    lut[blk * 64 + tid] = w;
  }
}

// From the query (the fused chain) and/or to produce the explicit order (rank_clusters op):
// one block per (batch, head, subspace), thread c owns cluster c.
// score_c = bf16(sum_j +-q_j), fp32 sum j ascending; order: score descending, id ascending.
// With `queries` set, warp 0 first does the query preparation itself (group mean, normalise, rotate),
// so the fused chain needs no separate query kernel; the block of subspace 0 publishes q_blocks / q_norm
// / query_avg for the later stages.
struct RankParams {
  const uint16_t* queries;   // [bs][Hq][128] or null
  const uint16_t* signs;
  int Hq, H, G;
  float inv_g;
  uint16_t* q_blocks;        // [bs*H][128]: input when queries == null, output otherwise
  uint16_t* q_norm;          // [bs*H] output (queries != null)
  uint16_t* query_avg;       // [bs*H][128] optional output
  const int32_t* counts;     // [bs*H][16][256] or null
  Tiers tiers;
  uint32_t* lut;             // [bs*H][16][64] or null
  int64_t* sorted_ids;       // [bs*H][16][256] or null
};

__global__ void __launch_bounds__(256) rank_kernel(RankParams p) {
  // entry o: x = sortable key ((ordered bf16 score) << 8 | (255 - o)), y = keys in cluster o
  __shared__ __align__(16) uint2 ent[256];
  __shared__ unsigned nib[256];
  __shared__ float s_q[8];
  const int c = threadIdx.x;
  const int64_t blk = blockIdx.x;  // (b*H + h)*16 + subspace
  const int64_t bh = blk >> 4;
  const int sub = (int)(blk & 15);
  pdl_wait();     // first kernel of the chain: its inputs come from kernels outside the chain
  pdl_trigger();
  const unsigned my_cnt = p.counts ? (unsigned)__ldg(p.counts + blk * 256 + c) : 0u;
  if (p.queries) {
    if (c < 32) {
      const int s = c & 7;
      const int b = (int)(bh / p.H), h = (int)(bh % p.H);
      const uint16_t* q = p.queries + ((int64_t)b * p.Hq + (int64_t)h * p.G) * 128 + 16 * s;
      float x[16], sg[16], acc[16];
      unpack8(__ldg(reinterpret_cast<const uint4*>(p.signs + 16 * s)), sg);
      unpack8(__ldg(reinterpret_cast<const uint4*>(p.signs + 16 * s) + 1), sg + 8);
#pragma unroll
      for (int i = 0; i < 16; i++) acc[i] = 0.0f;
      for (int g = 0; g < p.G; g++) {  // fp32 sum over the group, g ascending
        float v[16];
        unpack8(__ldg(reinterpret_cast<const uint4*>(q + g * 128)), v);
        unpack8(__ldg(reinterpret_cast<const uint4*>(q + g * 128) + 1), v + 8);
#pragma unroll
        for (int i = 0; i < 16; i++) acc[i] = __fadd_rn(acc[i], v[i]);
      }
#pragma unroll
      for (int i = 0; i < 16; i++) x[i] = bfround(__fmul_rn(acc[i], p.inv_g));
      if (sub == 0 && p.query_avg && c < 8)
#pragma unroll
        for (int i = 0; i < 16; i++) p.query_avg[bh * 128 + 16 * s + i] = f2bf(x[i]);
      const float n = rotate16(x, sg, s);
      if (c < 8) {
        if (sub == 0) {
#pragma unroll
          for (int i = 0; i < 16; i++) p.q_blocks[bh * 128 + 16 * s + i] = f2bf(x[i]);
          if (c == 0) p.q_norm[bh] = f2bf(n);
        }
        if (s == (sub >> 1))
#pragma unroll
          for (int j = 0; j < 8; j++) s_q[j] = x[8 * (sub & 1) + j];
      }
    }
  } else if (c < 8) {
    s_q[c] = bf2f(p.q_blocks[blk * 8 + c]);
  }
  __syncthreads();
  float s = 0.0f;
#pragma unroll
  for (int j = 0; j < 8; j++) {
    const float qv = s_q[j];
    s = __fadd_rn(s, ((c >> j) & 1) ? qv : -qv);
  }
  // order of (score descending, id ascending) as one unsigned compare; -0 counts as +0 like a float compare
  unsigned bits = f2bf(s);
  if (bits == 0x8000u) bits = 0u;
  const unsigned ord = (bits & 0x8000u) ? (~bits & 0xFFFFu) : (bits | 0x8000u);
  const unsigned my_key = (ord << 8) | (unsigned)(255 - c);
  ent[c] = make_uint2(my_key, my_cnt);
  __syncthreads();
  unsigned excl = 0, rank = 0;
  const uint4* e4 = reinterpret_cast<const uint4*>(ent);
#pragma unroll 16
  for (int o = 0; o < 128; o++) {
    const uint4 e = e4[o];  // two entries per 128-bit read (a broadcast: every thread reads the same word)
    const bool b0 = e.x > my_key, b1 = e.z > my_key;
    rank += (unsigned)b0 + (unsigned)b1;
    excl += (b0 ? e.y : 0u) + (b1 ? e.w : 0u);
  }
  if (p.sorted_ids) p.sorted_ids[blk * 256 + rank] = c;
  if (p.lut) {
    unsigned wgt = 0;
    for (int t = 0; t < p.tiers.n; t++) wgt += ((long long)excl < p.tiers.t[t]);
    nib[c] = wgt;
    __syncthreads();
    if (c < 64) {
      uint32_t w = 0;
#pragma unroll
      for (int i = 0; i < 4; i++) w |= nib[c * 4 + i] << (8 * i);
      p.lut[blk * 64 + c] = w;
    }
  }
}

// ---- the streaming count --------------------------------------------------------------------------

struct CollParams {
  const uint8_t* codes;          // element (b,h,s,k) at codes[b*c_b + h*c_h + s*c_s + k*c_l]
  int64_t c_b, c_h, c_s, c_l;
  const uint32_t* lut;           // [bs*H][B][64] words = 256 byte entries per subspace (FUSED == false)
  int32_t* out_i32;              // [bs*H][N]            (OUT_U8 == false)
  uint8_t* out_u8;               // [bs*H][u8_stride], indexed by virtual key (OUT_U8 == true)
  uint32_t* chunk_hist;          // [bs*H][n_chunks][256] (OUT_U8 == true)
  int64_t u8_stride;
  int H, B;
  int64_t N;                     // keys per head
  int mis;                       // virtual key v = key + mis; loads are 16-byte aligned in v
  int64_t chunk_keys;            // virtual keys per block
  int64_t n_hist;                // histogram rows per (batch, head) of chunk_hist (chain kernel)
  ChainQuery q;                  // FUSED == true: the table is built in the block from the query
  int G;
  float inv_g;
};

// byte k (0..3) of w, zero-extended: one PRMT
__device__ __forceinline__ unsigned byte_of(uint32_t w, int k) { return __byte_perm(w, 0, 0x4440 | k); }

// Sorts the 256 keys of a warp (8 per lane, element index e = 8 * lane + r) into DESCENDING order of e with a
// bitonic network: exchanges at distance < 8 stay inside a lane, the others are xor shuffles.  Keys are distinct.
__device__ __forceinline__ void warp_sort_desc_256(unsigned (&v)[8], int lane) {
#pragma unroll
  for (int k = 2; k <= 256; k <<= 1) {
#pragma unroll
    for (int j = k >> 1; j > 0; j >>= 1) {
      if (j >= 8) {
        const int lj = j >> 3;
        // block direction: "up" blocks end descending; the lower element of a pair keeps the maximum there
        const bool up = ((lane << 3) & k) == 0;
        const bool lower = (lane & lj) == 0;
        const bool take_max = up == lower;
#pragma unroll
        for (int r = 0; r < 8; r++) {
          const unsigned o = __shfl_xor_sync(0xffffffffu, v[r], lj);
          v[r] = take_max ? max(v[r], o) : min(v[r], o);
        }
      } else {
#pragma unroll
        for (int r = 0; r < 8; r++) {
          const int l = r ^ j;
          if (l > r) {
            const bool up = ((((lane << 3) | r) & k) == 0);
            const unsigned a = v[r], b = v[l];
            const unsigned mx = max(a, b), mn = min(a, b);
            v[r] = up ? mx : mn;
            v[l] = up ? mn : mx;
          }
        }
      }
    }
  }
}

// The stand-alone op (tier table from global memory, int32 counts out), 256 threads.
// LAYOUT 0: plane-major ([.., 16, N], key stride 1): a thread owns 16 consecutive keys.
// LAYOUT 1: key-major ([.., N, 16], subspace stride 1): a warp owns 512 consecutive keys, lane-strided.
// LAYOUT 2: any strides, any B <= 32: a thread owns one key at a time.
template <int LAYOUT, bool OUT_U8>
__global__ void __launch_bounds__(256, 2) collision_kernel(CollParams p) {
  __shared__ __align__(16) uint8_t s_lut[32 * 256];
  __shared__ __align__(16) unsigned hist[8 * 256];  // eight replicas (lane & 7) cut same-bin collisions inside a warp
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int bh = blockIdx.y, b = bh / p.H, h = bh % p.H;
  unsigned* my_hist = hist + ((lane & 7) << 8);
  const int64_t N = p.N;
  const int64_t Nv = N + p.mis;
  const int64_t v_begin = (int64_t)blockIdx.x * p.chunk_keys;
  const int64_t v_end = min(Nv, v_begin + p.chunk_keys);
  const uint8_t* base = p.codes + b * p.c_b + h * p.c_h - p.mis * p.c_l;
  int32_t* out32 = OUT_U8 ? nullptr : p.out_i32 + (int64_t)bh * p.N;
  uint8_t* out8 = OUT_U8 ? p.out_u8 + (int64_t)bh * p.u8_stride : nullptr;

  // the first batch of code loads is issued before the table is staged, so both latencies overlap
  uint4 r[16];
  if (LAYOUT == 1) {
    const int64_t w0 = v_begin + 512 * (int64_t)warp;
#pragma unroll
    for (int j = 0; j < 16; j++) {
      const int64_t v = w0 + 32 * j + lane;
      r[j] = (v < v_end) ? __ldg(reinterpret_cast<const uint4*>(base + v * 16)) : make_uint4(0, 0, 0, 0);
    }
  } else if (LAYOUT == 0) {
    const int64_t v0 = v_begin + 16 * (int64_t)tid;
#pragma unroll
    for (int s = 0; s < 16; s++)
      r[s] = (v0 < v_end) ? __ldg(reinterpret_cast<const uint4*>(base + s * p.c_s + v0)) : make_uint4(0, 0, 0, 0);
  }
  if (OUT_U8)
    for (int i = tid; i < 8 * 256; i += 256) hist[i] = 0;
  {
    const uint4* src = reinterpret_cast<const uint4*>(p.lut + (int64_t)bh * p.B * 64);
    uint4* dst = reinterpret_cast<uint4*>(s_lut);
    for (int i = tid; i < p.B * 16; i += 256) dst[i] = __ldg(src + i);
  }
  __syncthreads();

  if (LAYOUT == 0) {
    for (int64_t t0 = v_begin; t0 < v_end; t0 += 16 * 256) {  // block-uniform trip count (the warp votes below)
      const int64_t v0 = t0 + 16 * (int64_t)tid;
      const bool live = v0 < v_end;
      int cnt[16];
#pragma unroll
      for (int k = 0; k < 16; k++) cnt[k] = 0;
#pragma unroll
      for (int s = 0; s < 16; s++) {
        const uint32_t w4[4] = {r[s].x, r[s].y, r[s].z, r[s].w};
#pragma unroll
        for (int k = 0; k < 16; k++) cnt[k] += s_lut[s * 256 + byte_of(w4[k >> 2], k & 3)];
      }
      const int64_t vn = v0 + 16 * 256;
      if (vn < v_end) {
#pragma unroll
        for (int s = 0; s < 16; s++) r[s] = __ldg(reinterpret_cast<const uint4*>(base + s * p.c_s + vn));
      }
      const int64_t key0 = v0 - p.mis;
      if (OUT_U8) {
        uint32_t pk4[4] = {0, 0, 0, 0};
#pragma unroll
        for (int k = 0; k < 16; k++) {
          pk4[k >> 2] |= (uint32_t)cnt[k] << (8 * (k & 3));
          if (live && key0 + k >= 0 && key0 + k < N) atomicAdd(&my_hist[cnt[k]], 1u);
        }
        if (live) *reinterpret_cast<uint4*>(out8 + v0) = make_uint4(pk4[0], pk4[1], pk4[2], pk4[3]);
      } else if (live) {
        if (key0 >= 0 && key0 + 16 <= N && ((reinterpret_cast<uintptr_t>(out32 + key0) & 15) == 0)) {
#pragma unroll
          for (int q = 0; q < 4; q++)
            *reinterpret_cast<int4*>(out32 + key0 + 4 * q) =
                make_int4(cnt[4 * q], cnt[4 * q + 1], cnt[4 * q + 2], cnt[4 * q + 3]);
        } else {
#pragma unroll
          for (int k = 0; k < 16; k++)
            if (key0 + k >= 0 && key0 + k < N) out32[key0 + k] = cnt[k];
        }
      }
    }
  } else if (LAYOUT == 1) {
    for (int64_t w0 = v_begin + 512 * (int64_t)warp; w0 < v_end; w0 += 512 * 8) {
      int cnt[16];
#pragma unroll
      for (int j = 0; j < 16; j++) {
        const uint32_t w4[4] = {r[j].x, r[j].y, r[j].z, r[j].w};
        int c = 0;
#pragma unroll
        for (int s = 0; s < 16; s++) c += s_lut[s * 256 + byte_of(w4[s >> 2], s & 3)];
        cnt[j] = c;
      }
      const int64_t wn = w0 + 512 * 8;
      if (wn < v_end) {
#pragma unroll
        for (int j = 0; j < 16; j++) {
          const int64_t v = wn + 32 * j + lane;
          r[j] = (v < v_end) ? __ldg(reinterpret_cast<const uint4*>(base + v * 16)) : make_uint4(0, 0, 0, 0);
        }
      }
#pragma unroll
      for (int j = 0; j < 16; j++) {
        const int64_t v = w0 + 32 * j + lane;
        if (v < v_end) {
          if (OUT_U8) {
            out8[v] = (uint8_t)cnt[j];
            atomicAdd(&my_hist[cnt[j]], 1u);
          } else {
            out32[v] = cnt[j];
          }
        }
      }
    }
  } else {
    for (int64_t v = v_begin + tid; v < v_end; v += 256) {
      const int64_t key = v - p.mis;
      if (key < 0) continue;
      int cnt = 0;
      for (int s = 0; s < p.B; s++) cnt += s_lut[s * 256 + base[s * p.c_s + v * p.c_l]];
      if (OUT_U8) {
        out8[v] = (uint8_t)cnt;
        atomicAdd(&my_hist[cnt], 1u);
      } else {
        out32[key] = cnt;
      }
    }
  }
  if (OUT_U8) {
    __syncthreads();
    unsigned t = 0;
#pragma unroll
    for (int r = 0; r < 8; r++) t += hist[r * 256 + tid];
    p.chunk_hist[((int64_t)bh * gridDim.x + blockIdx.x) * 256 + tid] = t;
  }
}

// ---- the collision kernel of the decode chain -------------------------------------------------------------------
// 512 threads, one block per SM.  While its first code loads are in flight every block builds the tier table itself:
// warp 0 prepares the query (group mean, normalise, rotate: 4 dimensions per lane, the arithmetic and the fixed
// operation order of rotate16 / query_prep_kernel), then warp w ranks the 256 clusters of subspace w by (score
// descending, id ascending) with a register bitonic sort, takes the exclusive prefix sum of the cluster sizes in
// that order and writes, per cluster, the number of tiers whose threshold the prefix is below.  Output: one u8 count
// per virtual key and 256-bin histograms of the counts, one per `hist_keys` keys (two per block when the block covers
// its chunk in one pass), from which the selection kernel derives thresholds and output offsets.
constexpr int CC_THREADS = 512;
constexpr int CC_PASS = 8192;  // keys a block covers per pass: 16 warps x 512

// x: dims [4*lane, 4*lane+4) of the group-mean query (bf16 values as floats); sg: their SRHT signs.
// Same pairwise trees and butterflies as rotate16, spread over 32 lanes.  Returns the bf16 norm.
__device__ __forceinline__ float rotate4(float (&x)[4], const float (&sg)[4], int lane) {
  float t0 = __fadd_rn(__fmul_rn(x[0], x[0]), __fmul_rn(x[1], x[1]));
  float t1 = __fadd_rn(__fmul_rn(x[2], x[2]), __fmul_rn(x[3], x[3]));
  float sum = __fadd_rn(t0, t1);
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) sum = __fadd_rn(sum, __shfl_xor_sync(0xffffffffu, sum, off));
  const float n = bfround(__fsqrt_rn(sum));
  const float den = fmaxf(n, bfround(1e-8f));
#pragma unroll
  for (int i = 0; i < 4; i++) x[i] = __fmul_rn(bfround(__fdiv_rn(x[i], den)), sg[i]);
  {  // h = 1, 2 inside the lane
    float a = x[0], b = x[1], c = x[2], d = x[3];
    x[0] = __fadd_rn(a, b), x[1] = __fsub_rn(a, b), x[2] = __fadd_rn(c, d), x[3] = __fsub_rn(c, d);
    a = x[0], b = x[1], c = x[2], d = x[3];
    x[0] = __fadd_rn(a, c), x[2] = __fsub_rn(a, c), x[1] = __fadd_rn(b, d), x[3] = __fsub_rn(b, d);
  }
#pragma unroll
  for (int bit = 1; bit < 32; bit <<= 1)  // h = 4 .. 64 across lanes
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const float pv = __shfl_xor_sync(0xffffffffu, x[i], bit);
      x[i] = (lane & bit) ? __fsub_rn(pv, x[i]) : __fadd_rn(x[i], pv);
    }
#pragma unroll
  for (int i = 0; i < 4; i++) x[i] = bfround(__fmul_rn(x[i], 0.08838834764831845f));
  return n;
}

__device__ __forceinline__ void unpack4(uint2 v, float* out) {
  out[0] = __uint_as_float(v.x << 16), out[1] = __uint_as_float(v.x & 0xffff0000u);
  out[2] = __uint_as_float(v.y << 16), out[3] = __uint_as_float(v.y & 0xffff0000u);
}

template <int LAYOUT>
__global__ void __launch_bounds__(CC_THREADS, 1) chain_collision_kernel(CollParams p) {
  __shared__ __align__(16) uint8_t s_lut[16 * 256];
  // prologue: cluster sizes, 256 words per warp; afterwards: two histograms (one per half of a single-pass chunk) of
  // eight replicas each (lane & 7 picks the replica, which cuts same-bin collisions inside a warp)
  __shared__ __align__(16) unsigned hist[16 * 256];
  __shared__ float s_q[128];
  __shared__ unsigned s_tiers[9];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int bh = blockIdx.y, b = bh / p.H, h = bh % p.H;
  const ChainQuery& cq = p.q;
  // ---- query part of the prologue: warp 0 averages, normalises and rotates the query; then every warp scores the 256
  // clusters of its subspace and sorts them (registers only).  It reads nothing but the queries and the signs, so where
  // the caller vouches that those were complete before the PREVIOUS kernel on the stream started (cq.early_query: e.g.
  // the append launch sits in between), it runs before the wait for that kernel, under its tail.
  float qx[4] = {0.0f, 0.0f, 0.0f, 0.0f}, qavg[4] = {0.0f, 0.0f, 0.0f, 0.0f}, qn = 0.0f;
  unsigned key[8];
  auto prepare_query = [&]() {
    if (warp == 0) {
      const uint16_t* q = cq.queries + ((int64_t)b * cq.Hq + (int64_t)h * p.G) * 128 + 4 * lane;
      float sg[4], acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
      unpack4(__ldg(reinterpret_cast<const uint2*>(cq.signs + 4 * lane)), sg);
      for (int g = 0; g < p.G; g++) {  // fp32 sum over the group, g ascending
        float v[4];
        unpack4(__ldg(reinterpret_cast<const uint2*>(q + g * 128)), v);
#pragma unroll
        for (int i = 0; i < 4; i++) acc[i] = __fadd_rn(acc[i], v[i]);
      }
#pragma unroll
      for (int i = 0; i < 4; i++) qx[i] = qavg[i] = bfround(__fmul_rn(acc[i], p.inv_g));
      qn = rotate4(qx, sg, lane);
#pragma unroll
      for (int i = 0; i < 4; i++) s_q[4 * lane + i] = qx[i];
    }
  };
  auto rank_clusters = [&]() {   // after a barrier behind prepare_query()
    // register r of a lane starts with cluster c = 32 * r + lane: the first five terms of the score (bits 0..4 of c)
    // are the lane's, the last three (bits 5..7) the register's; the sum is taken in the order j = 0..7
    float qv[8];
#pragma unroll
    for (int j = 0; j < 8; j++) qv[j] = s_q[warp * 8 + j];
    float s5 = 0.0f;
#pragma unroll
    for (int j = 0; j < 5; j++) s5 = __fadd_rn(s5, ((lane >> j) & 1) ? qv[j] : -qv[j]);
#pragma unroll
    for (int rr = 0; rr < 8; rr++) {
      float sc = s5;
#pragma unroll
      for (int j = 5; j < 8; j++) sc = __fadd_rn(sc, ((rr >> (j - 5)) & 1) ? qv[j] : -qv[j]);
      // order of (score descending, id ascending) as one unsigned compare; -0 counts as +0 like a float compare
      unsigned bits = f2bf(sc);
      if (bits == 0x8000u) bits = 0u;
      const unsigned ord = (bits & 0x8000u) ? (~bits & 0xFFFFu) : (bits | 0x8000u);
      key[rr] = (ord << 8) | (unsigned)(255 - (32 * rr + lane));
    }
    warp_sort_desc_256(key, lane);
  };
  const bool early = cq.early_query != 0;
  if (early) {
    prepare_query();
    __syncthreads();
    rank_clusters();
  }
  if (cq.n_dev) pdl_wait();  // the zone length may have been written by the kernel just before this one
  const int64_t N = cq.n_dev ? min(max((int64_t)cq.n_dev[b], (int64_t)1), p.N) : p.N;
  const int64_t Nv = N + p.mis;
  const int64_t v_begin = (int64_t)blockIdx.x * p.chunk_keys;
  // every block clears its slice of the next kernel's value histogram, also a block beyond a short zone; a write, so
  // it comes after the wait for the kernels before this one
  auto clear_slice = [&]() {
    if (!cq.zero_area) return;
    const int per = (cq.zero_area_words + (int)gridDim.x - 1) / (int)gridDim.x;
    const int lo = (int)blockIdx.x * per, hi = min(cq.zero_area_words, lo + per);
    for (int i = lo + tid; i < hi; i += CC_THREADS) cq.zero_area[(int64_t)bh * cq.zero_area_words + i] = 0u;
  };
  if (v_begin >= Nv) {  // beyond this sample's zone (whole block, before any barrier)
    pdl_wait();
    pdl_trigger();
    clear_slice();
    return;
  }
  const int64_t v_end = min(Nv, v_begin + p.chunk_keys);
  const uint8_t* base = p.codes + b * p.c_b + h * p.c_h - p.mis * p.c_l;
  uint8_t* out8 = p.out_u8 + (int64_t)bh * p.u8_stride;
  const int pass_keys = (int)min(p.chunk_keys, (int64_t)CC_PASS);
  const int tile = pass_keys >> 4;  // keys per warp and pass (LAYOUT 1), a multiple of 32
  const int kpl = tile >> 5;        // keys per lane and pass, 1..16
  const bool publish = blockIdx.x == 0;

  // the first batch of code loads is issued before anything else, so their latency overlaps the prologue
  uint4 r[16];
  if (LAYOUT == 1) {
    const int64_t w0 = v_begin + (int64_t)tile * warp;
#pragma unroll
    for (int j = 0; j < 16; j++) {
      const int64_t v = w0 + 32 * j + lane;
      r[j] = (j < kpl && v < v_end) ? __ldg(reinterpret_cast<const uint4*>(base + v * 16)) : make_uint4(0, 0, 0, 0);
    }
  } else if (LAYOUT == 0) {
    const int64_t v0 = v_begin + 16 * (int64_t)tid;
#pragma unroll
    for (int s = 0; s < 16; s++)
      r[s] = (16 * tid < pass_keys && v0 < v_end) ? __ldg(reinterpret_cast<const uint4*>(base + s * p.c_s + v0))
                                                   : make_uint4(0, 0, 0, 0);
  }
  pdl_wait();     // the code loads above do not depend on the kernel before this one; the query below does
  pdl_trigger();
  clear_slice();

  // ---- prologue: query, cluster ranking, tier table ----
  {
    const int sub = warp;
    unsigned* my = hist + warp * 256;
    // cluster sizes of this warp's subspace: 8 consecutive clusters per lane
    const int4* cp = reinterpret_cast<const int4*>(cq.counts + ((int64_t)bh * 16 + sub) * 256 + lane * 8);
    const int4 c0 = __ldg(cp), c1 = __ldg(cp + 1);
    if (!early) prepare_query();
    if (warp == 0 && publish) {
      if (cq.query_avg)
        *reinterpret_cast<uint2*>(cq.query_avg + (int64_t)bh * 128 + 4 * lane) =
            make_uint2((uint32_t)f2bf(qavg[0]) | ((uint32_t)f2bf(qavg[1]) << 16),
                       (uint32_t)f2bf(qavg[2]) | ((uint32_t)f2bf(qavg[3]) << 16));
      *reinterpret_cast<uint2*>(cq.q_blocks + (int64_t)bh * 128 + 4 * lane) =
          make_uint2((uint32_t)f2bf(qx[0]) | ((uint32_t)f2bf(qx[1]) << 16), (uint32_t)f2bf(qx[2]) | ((uint32_t)f2bf(qx[3]) << 16));
      if (lane == 0) cq.q_norm[bh] = f2bf(qn);
    }
    if (tid == 32) {  // thresholds of this sample
      if (cq.n_dev || cq.n_plan > 0) {
        unsigned t[8];
        zone_tiers(cq.sched, cq.n_dev ? (long long)N : cq.n_plan, t);
        for (int i = 0; i < cq.sched.n_tiers; i++) s_tiers[i] = t[i];
        s_tiers[8] = (unsigned)cq.sched.n_tiers;
      } else {
        for (int i = 0; i < cq.n_tiers; i++) s_tiers[i] = cq.tiers[i];
        s_tiers[8] = (unsigned)cq.n_tiers;
      }
      if (publish && cq.zero_words) cq.zero_words[bh] = 0u;
    }
    *reinterpret_cast<int4*>(my + lane * 8) = c0;
    *reinterpret_cast<int4*>(my + lane * 8 + 4) = c1;
    __syncthreads();
    if (!early) rank_clusters();
    const int n_tiers = (int)s_tiers[8];
    unsigned tier[8];
#pragma unroll
    for (int t = 0; t < 8; t++) tier[t] = t < n_tiers ? s_tiers[t] : 0u;
    unsigned cnt[8], run = 0;
#pragma unroll
    for (int rr = 0; rr < 8; rr++) {
      cnt[rr] = my[255u - (key[rr] & 255u)];
      run += cnt[rr];
    }
    unsigned incl = run;  // inclusive prefix over lanes
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const unsigned o = __shfl_up_sync(0xffffffffu, incl, off);
      if (lane >= off) incl += o;
    }
    unsigned excl = incl - run;
#pragma unroll
    for (int rr = 0; rr < 8; rr++) {
      unsigned wgt = 0;
#pragma unroll
      for (int t = 0; t < 8; t++) wgt += (t < n_tiers && excl < tier[t]) ? 1u : 0u;
      s_lut[sub * 256 + (255u - (key[rr] & 255u))] = (uint8_t)wgt;
      excl += cnt[rr];
    }
    __syncthreads();  // the table is complete and the staging area is free again
    for (int i = tid; i < 16 * 256; i += CC_THREADS) hist[i] = 0;
    __syncthreads();
  }

  // a chunk covered in one pass gets two histograms (its halves), so the selection kernel can run two blocks on it
  const bool split = p.chunk_keys <= CC_PASS;
  const int64_t hist_keys = split ? (p.chunk_keys >> 1) : p.chunk_keys;
  unsigned* hist_rep = hist + ((lane & 7) << 8);
  if (LAYOUT == 0) {
    for (int64_t t0 = v_begin; t0 < v_end; t0 += CC_PASS) {  // block-uniform trip count
      const int64_t v0 = t0 + 16 * (int64_t)tid;
      const bool live = 16 * tid < pass_keys && v0 < v_end;
      int cnt[16];
#pragma unroll
      for (int k = 0; k < 16; k++) cnt[k] = 0;
#pragma unroll
      for (int s = 0; s < 16; s++) {
        const uint32_t w4[4] = {r[s].x, r[s].y, r[s].z, r[s].w};
#pragma unroll
        for (int k = 0; k < 16; k++) cnt[k] += s_lut[s * 256 + byte_of(w4[k >> 2], k & 3)];
      }
      const int64_t vn = v0 + CC_PASS;
      if (16 * tid < pass_keys && vn < v_end) {
#pragma unroll
        for (int s = 0; s < 16; s++) r[s] = __ldg(reinterpret_cast<const uint4*>(base + s * p.c_s + vn));
      }
      if (live) {
        const int64_t key0 = v0 - p.mis;
        unsigned* hh = hist_rep + ((split && v0 - v_begin >= hist_keys) ? 8 * 256 : 0);
        uint32_t pk4[4] = {0, 0, 0, 0};
#pragma unroll
        for (int k = 0; k < 16; k++) {
          pk4[k >> 2] |= (uint32_t)cnt[k] << (8 * (k & 3));
          if (key0 + k >= 0 && key0 + k < N) atomicAdd(&hh[cnt[k]], 1u);
        }
        *reinterpret_cast<uint4*>(out8 + v0) = make_uint4(pk4[0], pk4[1], pk4[2], pk4[3]);
      }
    }
  } else if (LAYOUT == 1) {
    for (int64_t t0 = v_begin; t0 < v_end; t0 += CC_PASS) {
      const int64_t w0 = t0 + (int64_t)tile * warp;
      int cnt[16];
#pragma unroll
      for (int j = 0; j < 16; j++) {
        int c = 0;
        if (j < kpl) {
          const uint32_t w4[4] = {r[j].x, r[j].y, r[j].z, r[j].w};
#pragma unroll
          for (int s = 0; s < 16; s++) c += s_lut[s * 256 + byte_of(w4[s >> 2], s & 3)];
        }
        cnt[j] = c;
      }
      const int64_t wn = w0 + CC_PASS;
      if (wn < v_end) {
#pragma unroll
        for (int j = 0; j < 16; j++) {
          const int64_t v = wn + 32 * j + lane;
          r[j] = (j < kpl && v < v_end) ? __ldg(reinterpret_cast<const uint4*>(base + v * 16)) : make_uint4(0, 0, 0, 0);
        }
      }
      unsigned* hh = hist_rep + ((split && w0 - v_begin >= hist_keys) ? 8 * 256 : 0);
#pragma unroll
      for (int j = 0; j < 16; j++) {
        const int64_t v = w0 + 32 * j + lane;
        if (j < kpl && v < v_end) {
          out8[v] = (uint8_t)cnt[j];
          atomicAdd(&hh[cnt[j]], 1u);
        }
      }
    }
  } else {
    for (int64_t v = v_begin + tid; v < v_end; v += CC_THREADS) {
      const int64_t key = v - p.mis;
      if (key < 0) continue;
      int cnt = 0;
      for (int s = 0; s < 16; s++) cnt += s_lut[s * 256 + base[s * p.c_s + v * p.c_l]];
      out8[v] = (uint8_t)cnt;
      atomicAdd(&hist_rep[((split && v - v_begin >= hist_keys) ? 8 * 256 : 0) + cnt], 1u);
    }
  }
  __syncthreads();
  {
    const int half = tid >> 8, bin = tid & 255;
    if (half == 0 || split) {
      unsigned t = 0;
#pragma unroll
      for (int rep = 0; rep < 8; rep++) t += hist[(half * 8 + rep) * 256 + bin];
      const int64_t row = split ? 2 * (int64_t)blockIdx.x + half : (int64_t)blockIdx.x;
      if (row < p.n_hist)  // the second half of the last block may lie beyond the zone: it has no row
        p.chunk_hist[((int64_t)bh * p.n_hist + row) * 256 + bin] = t;
    }
  }
}

// Unfused single-tier op: codes are int32 [bs,H,N,B] contiguous; one thread per key.
__global__ void __launch_bounds__(256) collision_i32_kernel(const int32_t* __restrict__ codes,
                                                            const uint32_t* __restrict__ lut_g, int B, int NC,
                                                            int64_t N, int32_t* __restrict__ out) {
  extern __shared__ uint32_t lut_w[];
  const uint8_t* lut = reinterpret_cast<const uint8_t*>(lut_w);
  const int bh = blockIdx.y;
  for (int i = threadIdx.x; i < B * 64; i += 256) lut_w[i] = lut_g[(int64_t)bh * B * 64 + i];
  __syncthreads();
  for (int64_t k = (int64_t)blockIdx.x * 256 + threadIdx.x; k < N; k += (int64_t)gridDim.x * 256) {
    const int32_t* row = codes + ((int64_t)bh * N + k) * B;
    int cnt = 0;
    for (int s = 0; s < B; s++) {
      const int32_t c = row[s];
      if (c >= 0 && c < NC) cnt += lut[s * 256 + c];
    }
    out[(int64_t)bh * N + k] = cnt;
  }
}

// single-tier table from (sorted ids, how many leading clusters are selected)
__global__ void __launch_bounds__(256) lut_single_kernel(const int32_t* __restrict__ ids,
                                                         const int32_t* __restrict__ topk_cnt, int NC,
                                                         uint32_t* __restrict__ lut) {
  __shared__ unsigned sel[256];
  const int tid = threadIdx.x;
  const int64_t blk = blockIdx.x;
  sel[tid] = 0;
  __syncthreads();
  if (tid < NC && tid < topk_cnt[blk]) {
    const int id = ids[blk * NC + tid];
    if (id >= 0 && id < NC) sel[id] = 1;
  }
  __syncthreads();
  if (tid < 64) {
    uint32_t w = 0;
#pragma unroll
    for (int i = 0; i < 4; i++) w |= sel[tid * 4 + i] << (8 * i);
    lut[blk * 64 + tid] = w;
  }
}

Tiers make_tiers(const int64_t* tier_counts, int n) {
  Tiers t;
  t.n = n;
  for (int i = 0; i < 8; i++) t.t[i] = i < n ? (long long)tier_counts[i] : 0;
  return t;
}

}  // namespace

int64_t collision_chunk_keys(int64_t bs_h, int64_t Nv) {
  // one block = 8 warps x 512 keys per pass; about two blocks per SM over the whole grid
  int64_t n_chunks = (2 * (int64_t)sm_count()) / (bs_h > 0 ? bs_h : 1);
  if (n_chunks < 1) n_chunks = 1;
  int64_t chunk = (Nv + n_chunks - 1) / n_chunks;
  chunk = ((chunk + 4095) / 4096) * 4096;
  if (chunk > 32768) chunk = 32768;  // the selection kernel keeps one int per key of a chunk in shared memory
  return chunk;
}

int launch_rank(const uint16_t* queries, const uint16_t* signs, int Hq, int H, uint16_t* q_blocks, uint16_t* q_norm,
                uint16_t* query_avg, const int32_t* counts, const int64_t* tier_counts, int n_tiers, int64_t bs_h,
                uint32_t* lut, int64_t* sorted_ids, cudaStream_t st) {
  RankParams p;
  p.queries = queries, p.signs = signs, p.Hq = Hq, p.H = H, p.G = H > 0 ? Hq / H : 1;
  p.inv_g = 1.0f / (float)p.G;
  p.q_blocks = q_blocks, p.q_norm = q_norm, p.query_avg = query_avg, p.counts = counts;
  p.tiers = make_tiers(tier_counts, n_tiers);
  p.lut = lut, p.sorted_ids = sorted_ids;
  StageTimer tm(ST_RANK, st);
  if (launch_chain(rank_kernel, dim3((unsigned)(bs_h * 16)), dim3(256), 0, st, p) != cudaSuccess)
    return check_launch("rank_clusters");
  return check_launch("rank_clusters");
}

// Launch geometry of the chain's collision kernel: about one block per SM over the whole grid.  A block covers
// chunk_keys virtual keys: a multiple of 512 up to 8192 (one pass), else a multiple of 8192 up to 32768 (the selection
// kernel keeps one int per key of a histogram row in shared memory).
void chain_geometry(int64_t bs_h, int64_t Nv, int64_t* chunk_keys, int64_t* hist_keys, int64_t* n_hist) {
  int64_t target = (int64_t)sm_count() / (bs_h > 0 ? bs_h : 1);
  if (target < 1) target = 1;
  int64_t chunk = (Nv + target - 1) / target;
  if (chunk < 2048) chunk = 2048;  // every block of the selection kernel reads all histogram rows: keep them few
  if (chunk <= CC_PASS) {
    chunk = (chunk + 511) / 512 * 512;
  } else {
    chunk = (chunk + CC_PASS - 1) / CC_PASS * CC_PASS;
    if (chunk > 32768) chunk = 32768;
  }
  *chunk_keys = chunk;
  *hist_keys = chunk <= CC_PASS ? chunk / 2 : chunk;
  *n_hist = (Nv + *hist_keys - 1) / *hist_keys;
}

// The stand-alone op: streams the codes of N keys per (batch, head) and writes int32 counts; table from `lut`.
int launch_collision(const pk_tensor* codebook, const uint32_t* lut, int32_t* out_i32, cudaStream_t st) {
  const int64_t bs = codebook->shape[0], H = codebook->shape[1], B = codebook->shape[2], N = codebook->shape[3];
  CollParams p = {};
  p.codes = (const uint8_t*)codebook->data;
  p.c_b = codebook->stride[0], p.c_h = codebook->stride[1], p.c_s = codebook->stride[2], p.c_l = codebook->stride[3];
  p.lut = lut;
  p.out_i32 = out_i32;
  p.H = (int)H, p.B = (int)B, p.N = N;
  const uintptr_t addr = reinterpret_cast<uintptr_t>(p.codes);
  int layout = 2, mis = 0;
  if (B == 16 && p.c_l == 1 && p.c_s % 16 == 0 && p.c_h % 16 == 0 && p.c_b % 16 == 0) {
    layout = 0;
    mis = (int)(addr & 15);
  } else if (B == 16 && p.c_s == 1 && p.c_l == 16 && (addr & 15) == 0 && p.c_h % 16 == 0 && p.c_b % 16 == 0) {
    layout = 1;
  }
  p.mis = mis;
  const int64_t Nv = N + mis;
  p.chunk_keys = collision_chunk_keys(bs * H, Nv);
  const int64_t n_chunks = (Nv + p.chunk_keys - 1) / p.chunk_keys;
  dim3 grid((unsigned)n_chunks, (unsigned)(bs * H));
  StageTimer tm(ST_COLLISION, st);
  if (layout == 0) collision_kernel<0, false><<<grid, 256, 0, st>>>(p);
  else if (layout == 1) collision_kernel<1, false><<<grid, 256, 0, st>>>(p);
  else collision_kernel<2, false><<<grid, 256, 0, st>>>(p);
  return check_launch("collision");
}

// The decode chain: query preparation, cluster ranking, tier table and the count in one kernel; compact output
// (u8 per virtual key + 256-bin histograms, one per hist_keys keys).
int launch_chain_collision(const pk_tensor* codebook, const ChainQuery& cq, uint8_t* counts_u8, int64_t u8_stride,
                           uint32_t* chunk_hist, int* mis_out, int64_t* hist_keys_out, int64_t* n_hist_out,
                           cudaStream_t st) {
  const int64_t bs = codebook->shape[0], H = codebook->shape[1], B = codebook->shape[2], N = codebook->shape[3];
  if (B != 16) return fail(PK_ERR_ARG, "the fused chain supports 16 subspaces");
  CollParams p = {};
  p.codes = (const uint8_t*)codebook->data;
  p.c_b = codebook->stride[0], p.c_h = codebook->stride[1], p.c_s = codebook->stride[2], p.c_l = codebook->stride[3];
  p.out_u8 = counts_u8;
  p.chunk_hist = chunk_hist;
  p.u8_stride = u8_stride;
  p.H = (int)H, p.B = 16, p.N = N;
  p.q = cq;
  p.G = H > 0 ? cq.Hq / (int)H : 1;
  p.inv_g = 1.0f / (float)p.G;
  int layout = 2;
  p.mis = chain_layout(codebook, &layout);
  int64_t hist_keys = 0;
  chain_geometry(bs * H, N + p.mis, &p.chunk_keys, &hist_keys, &p.n_hist);
  const int64_t n_blocks = (N + p.mis + p.chunk_keys - 1) / p.chunk_keys;
  if (mis_out) *mis_out = p.mis;
  if (hist_keys_out) *hist_keys_out = hist_keys;
  if (n_hist_out) *n_hist_out = p.n_hist;
  dim3 grid((unsigned)n_blocks, (unsigned)(bs * H));
  StageTimer tm(ST_COLLISION, st);
  if (layout == 0) launch_chain(chain_collision_kernel<0>, grid, dim3(CC_THREADS), 0, st, p);
  else if (layout == 1) launch_chain(chain_collision_kernel<1>, grid, dim3(CC_THREADS), 0, st, p);
  else launch_chain(chain_collision_kernel<2>, grid, dim3(CC_THREADS), 0, st, p);
  return check_launch("chain collision");
}

// Which code path a codebook view takes in the chain kernel (0 plane-major, 1 key-major, 2 generic) and, for the
// plane-major one, how many bytes its first key lies past a 16-byte boundary.
int chain_layout(const pk_tensor* codebook, int* layout) {
  const int64_t c_b = codebook->stride[0], c_h = codebook->stride[1], c_s = codebook->stride[2], c_l = codebook->stride[3];
  const uintptr_t addr = reinterpret_cast<uintptr_t>(codebook->data);
  *layout = 2;
  if (c_l == 1 && c_s % 16 == 0 && c_h % 16 == 0 && c_b % 16 == 0) {
    *layout = 0;
    return (int)(addr & 15);
  }
  if (c_s == 1 && c_l == 16 && (addr & 15) == 0 && c_h % 16 == 0 && c_b % 16 == 0) *layout = 1;
  return 0;
}

namespace {
// One block per (batch, head): bin `tid` summed over the chunks that hold keys of this sample.
__global__ void __launch_bounds__(256) hist_reduce_kernel(const uint32_t* __restrict__ chunk_hist, int64_t n_chunks,
                                                          int64_t chunk_keys, int mis, int H, int64_t N,
                                                          const int32_t* __restrict__ n_dev,
                                                          uint32_t* __restrict__ local_hist) {
  const int64_t bh = blockIdx.x;
  const int tid = threadIdx.x;
  pdl_wait();
  pdl_trigger();
  const int64_t n = n_dev ? min(max((int64_t)n_dev[bh / H], (int64_t)1), N) : N;
  const int64_t live = min(n_chunks, (n + mis + chunk_keys - 1) / chunk_keys);
  const uint32_t* hp = chunk_hist + bh * n_chunks * 256 + tid;
  unsigned t = 0;
  int64_t c = 0;
  for (; c + 8 <= live; c += 8) {
    unsigned v[8];
#pragma unroll
    for (int i = 0; i < 8; i++) v[i] = __ldg(hp + (c + i) * 256);
#pragma unroll
    for (int i = 0; i < 8; i++) t += v[i];
  }
  for (; c < live; c++) t += __ldg(hp + c * 256);
  local_hist[bh * 256 + tid] = t;
}
}  // namespace

int launch_hist_reduce(const uint32_t* chunk_hist, int64_t bs_h, int64_t n_chunks, int64_t chunk_keys, int mis, int H,
                       int64_t N, const int32_t* n_dev, uint32_t* local_hist, cudaStream_t st) {
  StageTimer tm(ST_HIST_REDUCE, st);
  launch_chain(hist_reduce_kernel, dim3((unsigned)bs_h), dim3(256), 0, st, chunk_hist, n_chunks, chunk_keys, mis, H, N,
               n_dev, local_hist);
  return check_launch("shard histogram");
}

}  // namespace pk

using namespace pk;

extern "C" int64_t pk_collision_workspace_bytes(int64_t bs, int64_t H, int64_t B, int64_t NC) {
  (void)NC;
  return bs * H * B * 64 * 4;
}

extern "C" int pk_rank_clusters(const pk_tensor* q_blocks, const pk_tensor* sorted_ids, void* stream) {
  PK_CHECK_TENSOR(q_blocks, PK_BF16, 4);
  PK_CHECK_TENSOR(sorted_ids, PK_I64, 4);
  const int64_t bs = q_blocks->shape[0], H = q_blocks->shape[1];
  PK_REQUIRE(is_contig(q_blocks) && q_blocks->shape[2] == 16 && q_blocks->shape[3] == 8,
             "q_blocks must be contiguous [bs,H,16,8]");
  PK_REQUIRE(is_contig(sorted_ids) && sorted_ids->shape[0] == bs && sorted_ids->shape[1] == H &&
                 sorted_ids->shape[2] == 16 && sorted_ids->shape[3] == 256,
             "sorted_ids must be contiguous [bs,H,16,256]");
  if (bs * H == 0) return PK_OK;
  return launch_rank(nullptr, nullptr, 0, (int)H, (uint16_t*)q_blocks->data, nullptr, nullptr, nullptr, nullptr, 0, bs * H,
                     nullptr, (int64_t*)sorted_ids->data, (cudaStream_t)stream);
}

extern "C" int pk_collision_fused(const pk_tensor* sorted_cluster_ids, const pk_tensor* cluster_key_counts,
                                  const pk_tensor* codebook, const int64_t* tier_counts, int n_tiers,
                                  const pk_tensor* cache_cnt, void* workspace, int64_t workspace_bytes,
                                  void* stream) {
  PK_REQUIRE(sorted_cluster_ids && sorted_cluster_ids->data, "sorted_cluster_ids is null");
  PK_REQUIRE(sorted_cluster_ids->dtype == PK_I64 || sorted_cluster_ids->dtype == PK_I32,
             "sorted_cluster_ids must be int64 or int32");
  PK_REQUIRE(sorted_cluster_ids->ndim == 4, "sorted_cluster_ids must be 4-D");
  PK_CHECK_TENSOR(cluster_key_counts, PK_I32, 4);
  PK_CHECK_TENSOR(codebook, PK_U8, 4);
  PK_CHECK_TENSOR(cache_cnt, PK_I32, 3);
  const int64_t bs = codebook->shape[0], H = codebook->shape[1], B = codebook->shape[2], N = codebook->shape[3];
  const int64_t NC = sorted_cluster_ids->shape[3];
  PK_REQUIRE(n_tiers >= 1 && n_tiers <= 8 && tier_counts, "n_tiers must be in 1..8");
  PK_REQUIRE(B >= 1 && B <= 32, "subspaces must be in 1..32, got %lld", (long long)B);
  PK_REQUIRE(NC >= 1 && NC <= 256, "clusters per subspace must be in 1..256, got %lld", (long long)NC);
  PK_REQUIRE(B * n_tiers <= 255, "subspaces x tiers must not exceed 255");
  PK_REQUIRE(is_contig(sorted_cluster_ids) && sorted_cluster_ids->shape[0] == bs && sorted_cluster_ids->shape[1] == H &&
                 sorted_cluster_ids->shape[2] == B,
             "sorted_cluster_ids must be contiguous [bs,H,B,NC]");
  PK_REQUIRE(is_contig(cluster_key_counts) && cluster_key_counts->shape[0] == bs && cluster_key_counts->shape[1] == H &&
                 cluster_key_counts->shape[2] == B && cluster_key_counts->shape[3] == NC,
             "cluster_key_counts must be contiguous [bs,H,B,NC]");
  PK_REQUIRE(is_contig(cache_cnt) && cache_cnt->shape[0] == bs && cache_cnt->shape[1] == H && cache_cnt->shape[2] == N,
             "cache_cnt must be contiguous [bs,H,N]");
  if (bs * H * N == 0) return PK_OK;
  if (!workspace || workspace_bytes < pk_collision_workspace_bytes(bs, H, B, NC))
    return fail(PK_ERR_WORKSPACE, "collision workspace too small: %lld < %lld", (long long)workspace_bytes,
                (long long)pk_collision_workspace_bytes(bs, H, B, NC));
  cudaStream_t st = (cudaStream_t)stream;
  uint32_t* lut = (uint32_t*)workspace;
  Tiers tiers = make_tiers(tier_counts, n_tiers);
  const unsigned nblk = (unsigned)(bs * H * B);
  int rc;
  {
    StageTimer tm(ST_RANK, st);
    if (sorted_cluster_ids->dtype == PK_I64)
      lut_from_sorted_kernel<int64_t><<<nblk, 256, 0, st>>>((const int64_t*)sorted_cluster_ids->data,
                                                            (const int32_t*)cluster_key_counts->data, (int)NC, tiers, lut);
    else
      lut_from_sorted_kernel<int32_t><<<nblk, 256, 0, st>>>((const int32_t*)sorted_cluster_ids->data,
                                                            (const int32_t*)cluster_key_counts->data, (int)NC, tiers, lut);
    rc = check_launch("collision table");
  }
  if (rc) return rc;
  return launch_collision(codebook, lut, (int32_t*)cache_cnt->data, st);
}

extern "C" int pk_collision(const pk_tensor* sorted_cluster_ids, const pk_tensor* topk_cluster_cnt,
                            const pk_tensor* code_book, const pk_tensor* cache_cnt, void* workspace,
                            int64_t workspace_bytes, void* stream) {
  PK_CHECK_TENSOR(sorted_cluster_ids, PK_I32, 4);
  PK_CHECK_TENSOR(topk_cluster_cnt, PK_I32, 3);
  PK_CHECK_TENSOR(code_book, PK_I32, 4);
  PK_CHECK_TENSOR(cache_cnt, PK_I32, 3);
  const int64_t bs = code_book->shape[0], H = code_book->shape[1], N = code_book->shape[2], B = code_book->shape[3];
  const int64_t NC = sorted_cluster_ids->shape[3];
  PK_REQUIRE(B >= 1 && B <= 32 && NC >= 1 && NC <= 256, "need B <= 32 and NC <= 256");
  PK_REQUIRE(is_contig(sorted_cluster_ids) && is_contig(topk_cluster_cnt) && is_contig(code_book) && is_contig(cache_cnt),
             "all tensors must be contiguous");
  PK_REQUIRE(sorted_cluster_ids->shape[0] == bs && sorted_cluster_ids->shape[1] == H && sorted_cluster_ids->shape[2] == B &&
                 topk_cluster_cnt->shape[0] == bs && topk_cluster_cnt->shape[1] == H && topk_cluster_cnt->shape[2] == B &&
                 cache_cnt->shape[0] == bs && cache_cnt->shape[1] == H && cache_cnt->shape[2] == N,
             "shape mismatch: ids [bs,H,B,NC], cnt [bs,H,B], code_book [bs,H,N,B], cache_cnt [bs,H,N]");
  if (bs * H * N == 0) return PK_OK;
  if (!workspace || workspace_bytes < pk_collision_workspace_bytes(bs, H, B, NC))
    return fail(PK_ERR_WORKSPACE, "collision workspace too small");
  cudaStream_t st = (cudaStream_t)stream;
  uint32_t* lut = (uint32_t*)workspace;
  lut_single_kernel<<<(unsigned)(bs * H * B), 256, 0, st>>>((const int32_t*)sorted_cluster_ids->data,
                                                            (const int32_t*)topk_cluster_cnt->data, (int)NC, lut);
  int rc = check_launch("collision table");
  if (rc) return rc;
  int64_t gx = (N + 255) / 256;
  int64_t cap = (int64_t)sm_count() * 8 / (bs * H) + 1;
  if (gx > cap) gx = cap;
  collision_i32_kernel<<<dim3((unsigned)gx, (unsigned)(bs * H)), 256, (size_t)B * 64 * 4, st>>>(
      (const int32_t*)code_book->data, lut, (int)B, (int)NC, N, (int32_t*)cache_cnt->data);
  return check_launch("collision");
}

// ---------------------------------------------------------------------------------------------------------
// Collision count for callers that may not allocate.
//
// pk_collision_fused needs a scratch table from its caller.  Some callers have nowhere to get one: a plugin
// loaded into a serving process whose runtime has already claimed nearly all of HBM for its own pool (a
// cudaMalloc from the plugin then fails or fragments the pool), a real-time decode thread that is forbidden to
// touch the device allocator because an allocation can stall the whole device, or code that was handed raw
// input / output pointers and nothing else.  For them the table lives in the array below, which is part of
// the library image: every GPU that loads the library holds these 256 KB until the process exits.
// ---------------------------------------------------------------------------------------------------------
namespace {
constexpr int64_t kStaticTableBytes = 256 * 1024;  // tables for up to 1024 (batch x head x subspace) triples
static __device__ __align__(256) unsigned char g_static_tier_table[kStaticTableBytes];

// Device address of the array, looked up once per device.  The array's name is only a host-side handle here;
// a kernel must be given the address that cudaGetSymbolAddress returns for the device that is current.
static std::mutex g_static_mu;
static void* g_static_ptr[64] = {nullptr};

int static_table_address(void** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64)
    return fail(PK_ERR_CUDA, "cannot identify the current device");
  std::lock_guard<std::mutex> lk(g_static_mu);
  if (!g_static_ptr[dev]) {
    void* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, g_static_tier_table);
    if (e != cudaSuccess || p == nullptr) {
      cudaGetLastError();
      return fail(PK_ERR_CUDA, "cudaGetSymbolAddress(static tier table): %s", cudaGetErrorString(e));
    }
    g_static_ptr[dev] = p;
  }
  *out = g_static_ptr[dev];
  return PK_OK;
}
}  // namespace

extern "C" int64_t pk_collision_fused_static_max_triples(void) { return kStaticTableBytes / 256; }

extern "C" int pk_collision_fused_static(const pk_tensor* sorted_cluster_ids, const pk_tensor* cluster_key_counts,
                                         const pk_tensor* codebook, const int64_t* tier_counts, int n_tiers,
                                         const pk_tensor* cache_cnt, void* stream) {
  PK_CHECK_TENSOR(codebook, PK_U8, 4);
  PK_CHECK_TENSOR(cluster_key_counts, PK_I32, 4);
  PK_CHECK_TENSOR(cache_cnt, PK_I32, 3);
  PK_REQUIRE(sorted_cluster_ids && sorted_cluster_ids->data && sorted_cluster_ids->ndim == 4,
             "sorted_cluster_ids must be a 4-D tensor");
  const int64_t triples = codebook->shape[0] * codebook->shape[1] * codebook->shape[2];
  if (triples * 256 > kStaticTableBytes)
    return fail(PK_ERR_WORKSPACE,
                "pk_collision_fused_static handles at most %lld (batch x head x subspace) triples, got %lld; use "
                "pk_collision_fused with caller-provided scratch for larger problems",
                (long long)(kStaticTableBytes / 256), (long long)triples);
  void* table = nullptr;
  const int rc = static_table_address(&table);
  if (rc) return rc;
  // The table kernel rewrites every word that the counting kernel reads (64 words per triple), so nothing left
  // over from an earlier call can leak into this one and nothing has to be cleared.
  return pk_collision_fused(sorted_cluster_ids, cluster_key_counts, codebook, tier_counts, n_tiers, cache_cnt, table,
                            kStaticTableBytes, stream);
}


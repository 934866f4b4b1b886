// Split-K sparse decode attention with the UVA fetch of the selected rows fused in.
//
// Per (batch, KV head) the attended rows are the first n_window rows of the GPU window
// ([sink | local | update buffer]) followed by the K selected rows of the big K/V store, which may
// live in pinned host memory.  The rows are cut into tiles of 64; a block takes one tile, or several consecutive
// ones that it streams through two staging buffers, and stages a tile with TMA bulk copies (cp.async.bulk, one
// 512-byte copy per selected key where its K and V rows are adjacent, completion counted on an mbarrier), so a whole
// grid keeps megabytes outstanding on the host link.  16 groups of 8 lanes then run an online softmax over the staged
// rows for the query heads that share the KV head (four at a time), and the block writes one partial (m, l, o) record.
// The block that finishes last for a (batch, KV head) merges the partials and writes the output: one launch, no
// second kernel, no waiting on other blocks.  Scores are kept in the log2 domain.
#include "common.cuh"
#include "kernels.cuh"

namespace pk {
namespace {

constexpr int ATT_THREADS = 128;
constexpr int ATT_TILE = 64;
constexpr int ATT_GQ = 4;       // query heads per pass
constexpr int ATT_REC = 132;    // floats per partial: o[128], m, l, pad, pad
constexpr int ATT_WAIT_LIMIT = 4000000;  // polls of the copy barrier before giving up
// Elements (bf16) between two staged rows [K 128 | V 128 | pad].  The tensor-core form pads a row by 16 bytes, so that
// the eight rows of an 8x8 fragment fall into eight different groups of four banks.
template <bool MMA> struct AttRow { static constexpr int stride = MMA ? 264 : 256; };

struct AttParams {
  const uint16_t* q;  // [bs][Hq][128]
  const uint16_t* wk;
  const uint16_t* wv;
  int64_t w_b, w_h, w_l;  // window strides (elements)
  int64_t n_window;       // host value; an upper bound when n_window_dev is set
  const int32_t* n_window_dev;  // optional: actual window rows = n_window_dev[0] + n_window_add (device memory)
  int64_t n_window_add;
  const uint16_t* sk;
  const uint16_t* sv;
  int64_t cap_s;          // rows per (b,h) of the store
  int64_t s_b, s_h, s_l;  // store strides in elements (batch, head, row); K and V share them
  int kv_pair;            // the V row of a store key directly follows its K row: one 512-byte copy fetches both
  const int64_t* sel;     // [bs*H][K]
  const int32_t* n_sel;   // [bs*H] or null
  int64_t K, index_offset;
  int H, Hq, G, n_qgroups;
  int tiles_per_block;    // consecutive tiles of a (batch, KV head) that one block streams; the grid has ceil(tiles / it) groups
  float scale_log2;
  unsigned* counters;     // [bs*H] arrival counters, zero between calls
  int* status;            // set to 1 if a copy barrier was never completed
  float* ws;              // [bs*Hq][groups][ATT_REC]
  uint16_t* out;          // [bs][Hq][128]
  float* lse;             // optional [bs][Hq]: log2 of the softmax denominator (scaled scores, log2 domain)
};

__device__ __forceinline__ void unpack8f(uint4 v, float* out) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; i++) {
    out[2 * i] = __uint_as_float(w[i] << 16);
    out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}

__device__ __forceinline__ bool mbar_wait(unsigned mb, unsigned parity, int limit) {
  unsigned done = 0;
  for (int it = 0; it < limit && !done; it++)
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(mb), "r"(parity)
        : "memory");
  return done != 0;
}

__device__ __forceinline__ void mbar_arrive(unsigned mb) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(mb) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect(unsigned mb, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(mb), "r"(bytes) : "memory");
}

// One block takes `tiles_per_block` consecutive tiles of a (batch, KV head) and streams them through two staging
// buffers: while the online softmax runs over tile j, the copies of tile j + 1 are in flight.  With few tiles in the
// whole launch (one sequence) every block has one tile and all copies of the launch are outstanding at once, which is
// what the host link wants; with many (a batch of sequences, rows in HBM) a block amortises its fixed costs - index
// loads, the partial record, the fence and the arrival - over its tiles and the grid is a single wave.
//
// MMA: the scores and the weighted sum of a tile run on the tensor cores (mma.sync m16n8k16, bf16 in, fp32 out) in the
// arrangement of a flash-attention step with the query heads of the KV head as the 16 rows of the A operand (at most
// eight are real): a warp takes 16 rows of the tile, S[head][row] = Q K^T is two n-tiles of eight k-steps, its C
// fragments ARE the A fragments of P for O[head][dim] += P V (sixteen n-tiles over the 128 dims), V^T comes from
// ldmatrix.trans.  The probabilities are rounded to bf16 for the second product, as the reference's attention
// library does.
template <bool MMA>
__global__ void __launch_bounds__(ATT_THREADS, 3) sparse_attention_kernel(AttParams p) {
  constexpr int RS = AttRow<MMA>::stride;  // elements per staged row
  extern __shared__ __align__(128) unsigned char dyn[];
  uint16_t* KVs = reinterpret_cast<uint16_t*>(dyn);                          // [2 buffers][64][RS]: K row, V row of a key
  float* obuf = reinterpret_cast<float*>(dyn + 2 * ATT_TILE * RS);           // [16][4][128], over the SECOND buffer:
                                                                             // used when that buffer is idle
  __shared__ __align__(8) unsigned long long mbar[2];
  __shared__ float s_m[16][ATT_GQ], s_l[16][ATT_GQ];
  __shared__ unsigned char s_valid[2][ATT_TILE];
  __shared__ int s_last;
  const int tid = threadIdx.x;
  const int h = blockIdx.y, b = blockIdx.z;
  const int64_t bh = (int64_t)b * p.H + h;
  const int n_groups = (int)gridDim.x, tpb = p.tiles_per_block;
  const int t_first = (int)blockIdx.x * tpb;
  const unsigned mb0 = (unsigned)__cvta_generic_to_shared(&mbar[0]);
  pdl_wait();  // the selected indices and the per-head row counts come from the kernels before this one
  const int64_t n_sel = p.n_sel ? min((int64_t)p.n_sel[bh], p.K) : p.K;
  const int64_t n_window =
      p.n_window_dev ? min(p.n_window, max((int64_t)0, (int64_t)p.n_window_dev[0] + p.n_window_add)) : p.n_window;
  const int64_t n_rows = n_window + n_sel;
  if (tid == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(mb0), "r"(ATT_THREADS) : "memory");
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(mb0 + 8), "r"(ATT_THREADS) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  // ---- stage a tile: thread t copies row t/2, K for even t and V for odd t; where the store keeps the V row of a
  // key right behind its K row, the even thread fetches both with one 512-byte copy (half as many requests on the
  // host link).  Every thread arrives on the tile's barrier exactly once, the copying ones with their byte count ----
  auto tile_rows = [&](int t) -> int {
    return (int)max((int64_t)0, min((int64_t)ATT_TILE, n_rows - (int64_t)t * ATT_TILE));
  };
  auto issue = [&](int t, int buf) {
    const int i = tid >> 1;
    const bool is_v = tid & 1;
    const uint16_t* src = nullptr;
    bool ok = i < tile_rows(t), paired = false;
    if (ok) {
      const int64_t r = (int64_t)t * ATT_TILE + i;
      if (r < n_window) {
        src = (is_v ? p.wv : p.wk) + b * p.w_b + h * p.w_h + r * p.w_l;
      } else {
        const int64_t row = p.sel[bh * p.K + (r - n_window)] + p.index_offset;
        ok = row >= 0 && row < p.cap_s;
        paired = p.kv_pair != 0;
        src = ((is_v && !paired) ? p.sv : p.sk) + b * p.s_b + h * p.s_h + (ok ? row : 0) * p.s_l;
      }
    }
    if (!is_v) s_valid[buf][i] = ok;
    const unsigned mb = mb0 + 8 * buf;
    if (ok && !(paired && is_v)) {
      const unsigned dst =
          (unsigned)__cvta_generic_to_shared(KVs + buf * (ATT_TILE * RS) + i * RS + ((is_v && !paired) ? 128 : 0));
      mbar_arrive_expect(mb, paired ? 512u : 256u);
      if (paired)
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], 512, [%2];" ::"r"(dst),
                     "l"(src), "r"(mb)
                     : "memory");
      else
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], 256, [%2];" ::"r"(dst),
                     "l"(src), "r"(mb)
                     : "memory");
    } else {
      if (MMA && !ok) {  // a row without a copy is an operand of the matrix products all the same: make it zero
        uint4* z = reinterpret_cast<uint4*>(KVs + buf * (ATT_TILE * RS) + i * RS + (is_v ? 128 : 0));
#pragma unroll
        for (int k = 0; k < 16; k++) z[k] = make_uint4(0, 0, 0, 0);
      }
      mbar_arrive(mb);
    }
  };
  issue(t_first, 0);

  bool dead = false;  // a copy barrier never completed: reported, the remaining tiles count as empty
  // Called by every thread once per tile j of the block: starts the copies of tile j + 1 (its buffer was released by
  // the barrier that ends tile j - 1), waits for tile j, returns its live rows.
  // The copies never completed: report it, give them (and those of the tile just issued) one more bounded chance to
  // land, and go on with EMPTY tiles (partials m = -inf, l = 0), so that this block still arrives on the counter of
  // its (batch, KV head), the merge runs and the counter returns to zero.  The host must treat a raised status word
  // as fatal.
  auto acquire = [&](int j) -> int {
    const int buf = j & 1;
    if (j + 1 < tpb && !dead) issue(t_first + j + 1, buf ^ 1);
    if (!dead && !__syncthreads_and(mbar_wait(mb0 + 8 * buf, (unsigned)((j >> 1) & 1), ATT_WAIT_LIMIT))) {
      if (tid == 0) atomicExch(p.status, 1);
      mbar_wait(mb0 + 8 * buf, (unsigned)((j >> 1) & 1), ATT_WAIT_LIMIT);
      if (j + 1 < tpb) mbar_wait(mb0 + 8 * (buf ^ 1), (unsigned)(((j + 1) >> 1) & 1), ATT_WAIT_LIMIT);
      dead = true;
    }
    return dead ? 0 : tile_rows(t_first + j);
  };
  // Partial record of this block for up to ATT_GQ query heads from the groups' (m, l, o) in shared memory.
  auto block_partial = [&](int qg, int n_heads, int n_grp) {
    for (int g = 0; g < n_heads; g++) {
      float M = -INFINITY;
      for (int t = 0; t < n_grp; t++) M = fmaxf(M, s_m[t][g]);
      float L = 0.0f, O = 0.0f;
      for (int t = 0; t < n_grp; t++) {
        const float f = (s_m[t][g] == -INFINITY) ? 0.0f : exp2f(s_m[t][g] - M);
        L += s_l[t][g] * f;
        O += obuf[(t * ATT_GQ + g) * 128 + tid] * f;
      }
      float* rec = p.ws + (((int64_t)b * p.Hq + h * p.G + qg * ATT_GQ + g) * n_groups + blockIdx.x) * ATT_REC;
      __stcg(rec + tid, O);
      if (tid == 0) {
        __stcg(rec + 128, M);
        __stcg(rec + 129, L);
      }
    }
  };

  if constexpr (MMA) {
    // ---- tensor-core form: one pass, at most ATT_GQ query heads per KV head ----
    const int lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
    const bool head_ok = g < p.G;
    uint32_t qa[8][2];  // A fragments of Q for the eight k-steps: rows g (a0, a2); rows g + 8 are zero (a1, a3)
    {
      const uint32_t* qrow = reinterpret_cast<const uint32_t*>(p.q + ((int64_t)b * p.Hq + h * p.G + (head_ok ? g : 0)) * 128);
#pragma unroll
      for (int k = 0; k < 8; k++) {
        qa[k][0] = head_ok ? __ldg(qrow + 8 * k + t) : 0u;
        qa[k][1] = head_ok ? __ldg(qrow + 8 * k + 4 + t) : 0u;
      }
    }
    float oacc[16][4];
#pragma unroll
    for (int n = 0; n < 16; n++) oacc[n][0] = oacc[n][1] = oacc[n][2] = oacc[n][3] = 0.0f;
    float m_run = -INFINITY, l_run = 0.0f;  // head g; l is this lane's share, summed over the four lanes at the end
    const int r0 = warp * 16;               // this warp's rows of every tile
    for (int j = 0; j < tpb; j++) {
      const int buf = j & 1;
      const int n_live = acquire(j);
      const uint16_t* tile = KVs + buf * (ATT_TILE * RS);
      if (r0 < n_live) {  // warp-uniform
        // S[head][row] = Q K^T over the warp's 16 rows: two n-tiles of eight rows
        float sc[2][4];
#pragma unroll
        for (int nt = 0; nt < 2; nt++) {
          sc[nt][0] = sc[nt][1] = sc[nt][2] = sc[nt][3] = 0.0f;
          const uint32_t* krow = reinterpret_cast<const uint32_t*>(tile + (r0 + nt * 8 + g) * RS);
#pragma unroll
          for (int k = 0; k < 8; k++) {
            const uint32_t b0 = krow[8 * k + t], b1 = krow[8 * k + 4 + t];
            asm volatile(
                "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                : "+f"(sc[nt][0]), "+f"(sc[nt][1]), "+f"(sc[nt][2]), "+f"(sc[nt][3])
                : "r"(qa[k][0]), "r"(0u), "r"(qa[k][1]), "r"(0u), "r"(b0), "r"(b1));
          }
        }
        // online softmax of head g over the rows this lane holds: n-tile nt, columns 2t and 2t + 1
        float v[2][2], mx = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < 2; nt++)
#pragma unroll
          for (int e = 0; e < 2; e++) {
            const int row = r0 + nt * 8 + 2 * t + e;
            const bool live = row < n_live && s_valid[buf][row];
            v[nt][e] = live ? sc[nt][e] * p.scale_log2 : -INFINITY;
            mx = fmaxf(mx, v[nt][e]);
          }
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m_run, mx);
        const bool none = m_new == -INFINITY;  // no live row so far
        const float corr = none ? 1.0f : exp2f(m_run - m_new);
        float pr[2][2];
#pragma unroll
        for (int nt = 0; nt < 2; nt++)
#pragma unroll
          for (int e = 0; e < 2; e++) pr[nt][e] = none ? 0.0f : exp2f(v[nt][e] - m_new);
        l_run = l_run * corr + (pr[0][0] + pr[0][1]) + (pr[1][0] + pr[1][1]);
        m_run = m_new;
#pragma unroll
        for (int n = 0; n < 16; n++) oacc[n][0] *= corr, oacc[n][1] *= corr;
        // P as the A operand of the second product (bf16): rows g hold the probabilities, rows g + 8 are zero
        uint32_t pa0, pa2;
        {
          const __nv_bfloat162 x0 = __floats2bfloat162_rn(pr[0][0], pr[0][1]), x1 = __floats2bfloat162_rn(pr[1][0], pr[1][1]);
          pa0 = *reinterpret_cast<const uint32_t*>(&x0), pa2 = *reinterpret_cast<const uint32_t*>(&x1);
        }
        // O[head][dim] += P V: sixteen n-tiles of eight dims, two per ldmatrix (V^T fragments)
        const int mi = lane >> 3;
        const uint16_t* vrow = tile + (r0 + (mi & 1) * 8 + (lane & 7)) * RS + 128 + (mi >> 1) * 8;
#pragma unroll
        for (int np = 0; np < 8; np++) {
          uint32_t b0, b1, b2, b3;
          const unsigned addr = (unsigned)__cvta_generic_to_shared(vrow + np * 16);
          asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                       : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3)
                       : "r"(addr));
          asm volatile(
              "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
              : "+f"(oacc[2 * np][0]), "+f"(oacc[2 * np][1]), "+f"(oacc[2 * np][2]), "+f"(oacc[2 * np][3])
              : "r"(pa0), "r"(0u), "r"(pa2), "r"(0u), "r"(b0), "r"(b1));
          asm volatile(
              "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
              : "+f"(oacc[2 * np + 1][0]), "+f"(oacc[2 * np + 1][1]), "+f"(oacc[2 * np + 1][2]), "+f"(oacc[2 * np + 1][3])
              : "r"(pa0), "r"(0u), "r"(pa2), "r"(0u), "r"(b2), "r"(b3));
        }
      }
      __syncthreads();  // the tile has been consumed: its buffer may be refilled (after the last tile obuf is free)
    }
    // the four warps are the groups of the block-level merge
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
    if (g < ATT_GQ) {
#pragma unroll
      for (int n = 0; n < 16; n++) {
        obuf[(warp * ATT_GQ + g) * 128 + 8 * n + 2 * t] = oacc[n][0];
        obuf[(warp * ATT_GQ + g) * 128 + 8 * n + 2 * t + 1] = oacc[n][1];
      }
      if (t == 0) {
        s_m[warp][g] = head_ok ? m_run : -INFINITY;
        s_l[warp][g] = head_ok ? l_run : 0.0f;
      }
    }
    __syncthreads();
    block_partial(0, min(ATT_GQ, p.G), ATT_THREADS / 32);
  } else {
    const int s = tid & 7, grp = tid >> 3;
    for (int qg = 0; qg < p.n_qgroups; qg++) {  // more than one pass only for more than four query heads per KV head,
                                                // and then a block has a single tile, which stays staged
      const int n_heads = min(ATT_GQ, p.G - qg * ATT_GQ);
      float qf[ATT_GQ][16];
#pragma unroll
      for (int g = 0; g < ATT_GQ; g++) {
        if (g < n_heads) {
          const uint4* qp =
              reinterpret_cast<const uint4*>(p.q + ((int64_t)b * p.Hq + h * p.G + qg * ATT_GQ + g) * 128 + 16 * s);
          unpack8f(__ldg(qp), qf[g]);
          unpack8f(__ldg(qp + 1), qf[g] + 8);
        } else {
#pragma unroll
          for (int i = 0; i < 16; i++) qf[g][i] = 0.0f;
        }
      }
      float m[ATT_GQ], lsum[ATT_GQ], o[ATT_GQ][16];
#pragma unroll
      for (int g = 0; g < ATT_GQ; g++) {
        m[g] = -INFINITY;
        lsum[g] = 0.0f;
#pragma unroll
        for (int i = 0; i < 16; i++) o[g][i] = 0.0f;
      }
      for (int j = 0; j < tpb; j++) {
        const int buf = j & 1;
        const int n_live = qg == 0 ? acquire(j) : (dead ? 0 : tile_rows(t_first + j));
        const uint16_t* tile = KVs + buf * (ATT_TILE * RS);
        for (int i = grp; i < ATT_TILE; i += 16) {  // uniform trip count per warp: shuffles need all lanes
          const bool live = i < n_live && s_valid[buf][i];
          float kf[16], vf[16];
          if (live) {
            const uint4* kp = reinterpret_cast<const uint4*>(tile + i * RS + 16 * s);
            const uint4* vp = reinterpret_cast<const uint4*>(tile + i * RS + 128 + 16 * s);
            unpack8f(kp[0], kf);
            unpack8f(kp[1], kf + 8);
            unpack8f(vp[0], vf);
            unpack8f(vp[1], vf + 8);
          } else {
#pragma unroll
            for (int jj = 0; jj < 16; jj++) kf[jj] = 0.0f, vf[jj] = 0.0f;
          }
#pragma unroll
          for (int g = 0; g < ATT_GQ; g++) {
            float d = 0.0f;
#pragma unroll
            for (int jj = 0; jj < 16; jj++) d = fmaf(kf[jj], qf[g][jj], d);
            d += __shfl_xor_sync(0xffffffffu, d, 1);
            d += __shfl_xor_sync(0xffffffffu, d, 2);
            d += __shfl_xor_sync(0xffffffffu, d, 4);
            if (live) {
              const float sc = d * p.scale_log2;
              const float mn = fmaxf(m[g], sc);
              const float corr = exp2f(m[g] - mn);  // m = -inf on the first row gives 0
              const float pr = exp2f(sc - mn);
              lsum[g] = lsum[g] * corr + pr;
#pragma unroll
              for (int jj = 0; jj < 16; jj++) o[g][jj] = o[g][jj] * corr + pr * vf[jj];
              m[g] = mn;
            }
          }
        }
        __syncthreads();  // the tile has been consumed: its buffer may be refilled (and, after the last tile or
                          // between passes, obuf / s_m / s_l are free)
      }
#pragma unroll
      for (int g = 0; g < ATT_GQ; g++) {
#pragma unroll
        for (int jj = 0; jj < 16; jj++) obuf[(grp * ATT_GQ + g) * 128 + 16 * s + jj] = o[g][jj];
        if (s == 0) {
          s_m[grp][g] = m[g];
          s_l[grp][g] = lsum[g];
        }
      }
      __syncthreads();
      block_partial(qg, n_heads, 16);
      __syncthreads();  // obuf / s_m / s_l have been consumed before the next pass writes them
    }
  }

  // ---- the block that arrives last for this (batch, KV head) merges all tiles ----
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const unsigned prev = atomicAdd(p.counters + bh, 1u);
    s_last = prev + 1 == (unsigned)n_groups;
    if (s_last) p.counters[bh] = 0;  // ready for the next call on this stream
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  // Up to ATT_GQ query heads are merged at a time.  Warp g takes head g: it reads the tiles' (m, l), reduces the
  // maximum and the denominator with shuffles and leaves one scale factor per tile in shared memory; after ONE
  // block barrier every thread sums its output dimension over the tiles for all of these heads, the loads of
  // several tiles and heads in flight together (no serial chain of L2 round trips, no barrier per head).
  float* s_f = obuf;                    // [ATT_GQ][1024] scale factor per tile (reuses the merge buffer)
  __shared__ float s_L[ATT_GQ], s_M[ATT_GQ];
  static_assert(ATT_THREADS == 32 * ATT_GQ, "one warp per query head of a group");
  const int warp = tid >> 5, lane = tid & 31;
  for (int qg = 0; qg < p.n_qgroups; qg++) {
    const int n_heads = min(ATT_GQ, p.G - qg * ATT_GQ);
    const int64_t bq0 = (int64_t)b * p.Hq + h * p.G + qg * ATT_GQ;
    if (qg) __syncthreads();            // the scale factors of the previous group have been consumed
    if (warp < n_heads) {
      const float* rec = p.ws + (bq0 + warp) * n_groups * ATT_REC;
      float mloc = -INFINITY;
      for (int64_t t = lane; t < n_groups; t += 32) {
        const float mt = __ldcg(rec + t * ATT_REC + 128);
        s_f[warp * 1024 + t] = mt;
        mloc = fmaxf(mloc, mt);
      }
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) mloc = fmaxf(mloc, __shfl_xor_sync(0xffffffffu, mloc, off));
      float L = 0.0f;
      for (int64_t t = lane; t < n_groups; t += 32) {
        const float mt = s_f[warp * 1024 + t];
        const float f = (mt == -INFINITY) ? 0.0f : exp2f(mt - mloc);
        s_f[warp * 1024 + t] = f;
        L += __ldcg(rec + t * ATT_REC + 129) * f;
      }
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) L += __shfl_xor_sync(0xffffffffu, L, off);
      if (lane == 0) s_L[warp] = L, s_M[warp] = mloc;
    }
    __syncthreads();
    float O[ATT_GQ];
#pragma unroll
    for (int g = 0; g < ATT_GQ; g++) O[g] = 0.0f;
    const float* rec0 = p.ws + bq0 * n_groups * ATT_REC + tid;
    int64_t t = 0;
    for (; t + 4 <= n_groups; t += 4) {
      float v[ATT_GQ][4];
#pragma unroll
      for (int g = 0; g < ATT_GQ; g++)
#pragma unroll
        for (int i = 0; i < 4; i++) v[g][i] = g < n_heads ? __ldcg(rec0 + (g * n_groups + t + i) * ATT_REC) : 0.0f;
#pragma unroll
      for (int g = 0; g < ATT_GQ; g++)
#pragma unroll
        for (int i = 0; i < 4; i++) O[g] += v[g][i] * s_f[g * 1024 + t + i];
    }
    for (; t < n_groups; t++)
#pragma unroll
      for (int g = 0; g < ATT_GQ; g++)
        if (g < n_heads) O[g] += __ldcg(rec0 + (g * n_groups + t) * ATT_REC) * s_f[g * 1024 + t];
#pragma unroll
    for (int g = 0; g < ATT_GQ; g++) {
      if (g >= n_heads) continue;
      const float L = s_L[g];
      p.out[(bq0 + g) * 128 + tid] = f2bf(L > 0.0f ? O[g] / L : 0.0f);
      if (p.lse && tid == 0) p.lse[bq0 + g] = L > 0.0f ? s_M[g] + log2f(L) : -INFINITY;
    }
  }
}

}  // namespace
}  // namespace pk

using namespace pk;

namespace {
inline int64_t att_header_bytes(int64_t bs, int64_t H) { return (bs * H * 4 + 4 + 255) / 256 * 256; }
}  // namespace

extern "C" int64_t pk_attention_workspace_bytes(int64_t bs, int64_t Hq, int64_t max_rows) {
  // header (arrival counters + status word, sized for one KV head per query head) followed by the partials
  const int64_t tiles = (max_rows + ATT_TILE - 1) / ATT_TILE;
  return att_header_bytes(bs, Hq) + bs * Hq * (tiles > 0 ? tiles : 1) * ATT_REC * 4;
}

extern "C" int pk_sparse_attention(const pk_tensor* queries, const pk_tensor* window_k, const pk_tensor* window_v,
                                   int64_t n_window, const pk_tensor* n_window_dev, int64_t n_window_add,
                                   const pk_tensor* store_k, const pk_tensor* store_v,
                                   const pk_tensor* selected, const pk_tensor* n_sel, int64_t index_offset,
                                   float scale, const pk_tensor* out, const pk_tensor* lse, void* workspace,
                                   int64_t workspace_bytes, void* stream) {
  PK_CHECK_TENSOR(queries, PK_BF16, 4);
  PK_CHECK_TENSOR(out, PK_BF16, 4);
  const int64_t bs = queries->shape[0], Hq = queries->shape[2];
  PK_REQUIRE(queries->shape[1] == 1 && queries->shape[3] == 128 && is_contig(queries) &&
                 (reinterpret_cast<uintptr_t>(queries->data) & 15) == 0,
             "queries must be contiguous, 16-byte aligned [bs,1,Hq,128]");
  PK_REQUIRE(is_contig(out) && out->shape[0] == bs && out->shape[1] == 1 && out->shape[2] == Hq && out->shape[3] == 128,
             "out must be contiguous [bs,1,Hq,128]");
  AttParams p = {};
  int64_t H = 0;
  if (n_window > 0) {
    PK_CHECK_TENSOR(window_k, PK_BF16, 4);
    PK_CHECK_TENSOR(window_v, PK_BF16, 4);
    H = window_k->shape[1];
    PK_REQUIRE(window_k->shape[0] == bs && window_k->shape[3] == 128 && window_k->stride[3] == 1 &&
                   window_k->shape[2] >= n_window,
               "window_k must be [bs,H,cap>=n_window,128] with last stride 1");
    for (int i = 0; i < 4; i++)
      PK_REQUIRE(window_k->shape[i] == window_v->shape[i] &&
                     (window_k->shape[i] == 1 || window_k->stride[i] == window_v->stride[i]),
                 "window_k and window_v must have the same shape and strides");
    PK_REQUIRE((reinterpret_cast<uintptr_t>(window_k->data) & 15) == 0 && (reinterpret_cast<uintptr_t>(window_v->data) & 15) == 0 &&
                   window_k->stride[0] % 8 == 0 && window_k->stride[1] % 8 == 0 && window_k->stride[2] % 8 == 0,
               "window rows must be 16-byte aligned");
    p.wk = (const uint16_t*)window_k->data, p.wv = (const uint16_t*)window_v->data;
    p.w_b = window_k->stride[0], p.w_h = window_k->stride[1], p.w_l = window_k->stride[2];
  }
  int64_t K = 0;
  if (selected) {
    PK_CHECK_TENSOR(selected, PK_I64, 3);
    PK_CHECK_TENSOR(store_k, PK_BF16, 4);
    PK_CHECK_TENSOR(store_v, PK_BF16, 4);
    K = selected->shape[2];
    PK_REQUIRE(H == 0 || store_k->shape[1] == H, "window and store disagree on the number of KV heads");
    H = store_k->shape[1];
    PK_REQUIRE(store_k->shape[0] == bs && store_k->shape[3] == 128 && store_v->shape[0] == bs && store_v->shape[1] == H &&
                   store_v->shape[2] == store_k->shape[2] && store_v->shape[3] == 128 && store_k->stride[3] == 1 &&
                   store_v->stride[3] == 1,
               "store_k / store_v must be [bs,H,cap,128] with last stride 1");
    for (int i = 0; i < 3; i++) {
      PK_REQUIRE(store_k->shape[i] == 1 || store_k->stride[i] == store_v->stride[i], "store_k and store_v must have the same strides");
      PK_REQUIRE(store_k->shape[i] == 1 || store_k->stride[i] % 8 == 0, "store rows must be 16-byte aligned");
    }
    PK_REQUIRE((reinterpret_cast<uintptr_t>(store_k->data) & 15) == 0 && (reinterpret_cast<uintptr_t>(store_v->data) & 15) == 0,
               "store rows must be 16-byte aligned");
    p.s_b = store_k->shape[0] == 1 ? 0 : store_k->stride[0];
    p.s_h = store_k->shape[1] == 1 ? 0 : store_k->stride[1];
    p.s_l = store_k->shape[2] == 1 ? 128 : store_k->stride[2];
    PK_REQUIRE(is_contig(selected) && selected->shape[0] == bs && selected->shape[1] == H,
               "selected must be contiguous [bs,H,K]");
    p.sk = (const uint16_t*)store_k->data, p.sv = (const uint16_t*)store_v->data;
    p.kv_pair = (p.sv == p.sk + 128 && p.s_l >= 256) ? 1 : 0;
    p.cap_s = store_k->shape[2];
    p.sel = (const int64_t*)selected->data;
    if (n_sel) {
      PK_CHECK_TENSOR(n_sel, PK_I32, 2);
      PK_REQUIRE(is_contig(n_sel) && n_sel->shape[0] == bs && n_sel->shape[1] == H, "n_sel must be contiguous [bs,H]");
      p.n_sel = (const int32_t*)n_sel->data;
    }
  }
  PK_REQUIRE(H > 0 && Hq % H == 0, "need at least one of window / selected rows, and Hq a multiple of H");
  PK_REQUIRE(n_window >= 0, "n_window must be non-negative");
  if (bs == 0) return PK_OK;
  const int64_t max_rows = n_window + K;
  const int64_t n_tiles = max_rows > 0 ? (max_rows + ATT_TILE - 1) / ATT_TILE : 1;
  PK_REQUIRE(n_tiles <= 1024, "too many rows for one call: %lld (limit 65536)", (long long)max_rows);
  if (!workspace || workspace_bytes < pk_attention_workspace_bytes(bs, Hq, max_rows))
    return fail(PK_ERR_WORKSPACE, "attention workspace too small: %lld < %lld", (long long)workspace_bytes,
                (long long)pk_attention_workspace_bytes(bs, Hq, max_rows));
  p.q = (const uint16_t*)queries->data;
  p.n_window = n_window;
  if (n_window_dev) {
    PK_CHECK_TENSOR(n_window_dev, PK_I32, 1);
    PK_REQUIRE(n_window_dev->shape[0] >= 1, "n_window_dev must hold one int32");
    p.n_window_dev = (const int32_t*)n_window_dev->data;
    p.n_window_add = n_window_add;
  }
  p.K = K, p.index_offset = index_offset;
  p.H = (int)H, p.Hq = (int)Hq, p.G = (int)(Hq / H);
  p.n_qgroups = (p.G + ATT_GQ - 1) / ATT_GQ;
  // Blocks per (batch, KV head): all the tiles when the launch is small (every copy of the launch outstanding at once),
  // otherwise as many as give ONE wave of three blocks per SM, each streaming several tiles.  More than four query
  // heads per KV head need the staged tile for several passes: one tile per block then.
  int64_t groups = n_tiles;
  if (p.n_qgroups == 1) {
    const int64_t fit = (int64_t)sm_count() * 3 / (H * bs);
    groups = fit < 1 ? 1 : (fit < n_tiles ? fit : n_tiles);
  }
  p.tiles_per_block = (int)((n_tiles + groups - 1) / groups);
  groups = (n_tiles + p.tiles_per_block - 1) / p.tiles_per_block;
  p.scale_log2 = scale * 1.4426950408889634f;
  PK_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 15) == 0, "workspace must be 16-byte aligned");
  p.counters = (unsigned*)workspace;
  p.status = (int*)workspace + bs * Hq;
  p.ws = (float*)((char*)workspace + att_header_bytes(bs, Hq));
  p.out = (uint16_t*)out->data;
  if (lse) {
    PK_CHECK_TENSOR(lse, PK_F32, 2);
    PK_REQUIRE(is_contig(lse) && lse->shape[0] == bs && lse->shape[1] == Hq, "lse must be contiguous [bs,Hq]");
    p.lse = (float*)lse->data;
  }
  cudaStream_t st = (cudaStream_t)stream;
  // at most ATT_GQ query heads per KV head: scores and weighted sum on the tensor cores; more: the scalar form in passes
  const bool mma = p.G <= ATT_GQ;
  const int smem = 2 * ATT_TILE * (mma ? AttRow<true>::stride : AttRow<false>::stride) * 2;   // two staging buffers
  static PerDevice smem_attr[2];  // the opt-in to more than 48 KB of dynamic shared memory is per kernel and device
  if (const unsigned long long bit = first_on_device(smem_attr[mma])) {
    const cudaError_t e = mma ? cudaFuncSetAttribute(sparse_attention_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)
                              : cudaFuncSetAttribute(sparse_attention_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return check_launch("sparse_attention smem");
    mark_on_device(smem_attr[mma], bit);
  }
  dim3 grid((unsigned)groups, (unsigned)H, (unsigned)bs);
  StageTimer tm(ST_ATTENTION, st);
  if (mma) launch_chain(sparse_attention_kernel<true>, grid, dim3(ATT_THREADS), (size_t)smem, st, p);
  else launch_chain(sparse_attention_kernel<false>, grid, dim3(ATT_THREADS), (size_t)smem, st, p);
  return check_launch("sparse_attention");
}

// Exchange glue of the sequence-sharded form: every rank retrieves over its contiguous chunk of the zone, the local
// top lists are all-gathered, the global top-K is selected from them, each rank attends the rows it owns and the
// partial results are merged through their softmax denominators.  The collectives themselves are issued by the
// host (NCCL all-gather of one packed buffer each); these kernels are the packing, unpacking and merging on either
// side of them, one launch each.
#include "common.cuh"

namespace pk {

// Position of `key` in the ascending row a[0..n): first element >= key.
__device__ __forceinline__ int lower_bound_i64(const int64_t* __restrict__ a, int n, int64_t key) {
  int lo = 0, hi = n;
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if (__ldg(a + mid) < key) lo = mid + 1; else hi = mid;
  }
  return lo;
}

// One entry of a rank's local top list: (fp32 score bits, global key index), or (-inf, -1) past the row's valid
// entries.  cand / scores rows have stride C and n_cand[row] (default C) valid entries; local_final rows have n_sel[row]
// (default Kl) valid entries.
__device__ __forceinline__ longlong2 shard_entry(const int64_t* __restrict__ cand, const float* __restrict__ scores,
                                                 const int64_t* __restrict__ local_final, const int32_t* __restrict__ n_sel,
                                                 const int32_t* __restrict__ n_cand, int row, int j, int C, int Kl, int64_t start) {
  longlong2 v;
  v.x = (int64_t)__float_as_int(-INFINITY);
  v.y = -1;
  const int valid = n_sel ? min(max(n_sel[row], 0), Kl) : Kl;
  const int nc = n_cand ? min(max(n_cand[row], 0), C) : C;
  if (j < valid && nc > 0) {
    const int64_t idx = local_final[(int64_t)row * Kl + j];
    int p = lower_bound_i64(cand + (int64_t)row * C, nc, idx);
    if (p >= nc) p = nc - 1;
    v.x = (int64_t)__float_as_int(scores[(int64_t)row * C + p]);
    v.y = idx + start;
  }
  return v;
}

// packed[row][j] = (score bits of local_final[row][j] as int64, local_final[row][j] + start)
__global__ void __launch_bounds__(256) shard_pack_kernel(const int64_t* __restrict__ cand, const float* __restrict__ scores,
                                                         const int64_t* __restrict__ local_final, int64_t* __restrict__ packed,
                                                         int C, int Kl, int64_t start, const int32_t* __restrict__ n_sel,
                                                         const int32_t* __restrict__ n_cand) {
  const int row = blockIdx.y;
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= Kl) return;
  *reinterpret_cast<longlong2*>(packed + ((int64_t)row * Kl + j) * 2) =
      shard_entry(cand, scores, local_final, n_sel, n_cand, row, j, C, Kl, start);
}

// gathered [world][rows][Kl][2] -> scores [rows][world*Kl], indices [rows][world*Kl] (rank-major within a row)
__global__ void __launch_bounds__(256) shard_unpack_kernel(const int64_t* __restrict__ gathered, float* __restrict__ scores,
                                                           int64_t* __restrict__ indices, int world, int rows, int Kl) {
  const int row = blockIdx.y;
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= world * Kl) return;
  const int w = t / Kl, j = t - w * Kl;
  const longlong2 v = *reinterpret_cast<const longlong2*>(gathered + (((int64_t)w * rows + row) * Kl + j) * 2);
  scores[(int64_t)row * world * Kl + t] = __int_as_float((int)v.x);
  indices[(int64_t)row * world * Kl + t] = v.y;
}

// final [rows][K] ascending global indices -> local [rows][K] (the rows inside [start,end) first, minus start, the
// rest 0) and n_owned [rows]
__global__ void __launch_bounds__(256) shard_owned_kernel(const int64_t* __restrict__ final_idx, int64_t* __restrict__ local,
                                                          int32_t* __restrict__ n_owned, int K, int64_t start, int64_t end) {
  const int row = blockIdx.x;
  const int64_t* f = final_idx + (int64_t)row * K;
  __shared__ int s_lo, s_n;
  if (threadIdx.x == 0) {
    const int lo = lower_bound_i64(f, K, start);
    const int hi = lower_bound_i64(f, K, end);
    s_lo = lo;
    s_n = hi - lo;
    n_owned[row] = hi - lo;
  }
  __syncthreads();
  const int lo = s_lo, n = s_n;
  for (int j = threadIdx.x; j < K; j += blockDim.x)
    local[(int64_t)row * K + j] = j < n ? f[lo + j] - start : 0;
}

// packed [rows][129] fp32 = (attention output over the local rows, log2 of the local softmax denominator)
__global__ void __launch_bounds__(128) shard_pack_partial_kernel(const __nv_bfloat16* __restrict__ out, const float* __restrict__ lse,
                                                                 float* __restrict__ packed) {
  const int row = blockIdx.x, d = threadIdx.x;
  packed[(int64_t)row * 129 + d] = __bfloat162float(out[(int64_t)row * 128 + d]);
  if (d == 0) packed[(int64_t)row * 129 + 128] = lse[row];
}

// gathered [world][rows][129] -> out [rows][128]: exact softmax over the union of the ranks' row sets
__global__ void __launch_bounds__(128) shard_merge_partial_kernel(const float* __restrict__ gathered, __nv_bfloat16* __restrict__ out,
                                                                  int world, int rows) {
  const int row = blockIdx.x, d = threadIdx.x;
  float m = -INFINITY;
  for (int w = 0; w < world; w++) m = fmaxf(m, gathered[((int64_t)w * rows + row) * 129 + 128]);
  float acc = 0.f, den = 0.f;
  for (int w = 0; w < world; w++) {
    const float* g = gathered + ((int64_t)w * rows + row) * 129;
    const float l = g[128];
    const float wt = (l == -INFINITY) ? 0.f : exp2f(l - m);   // a rank without rows contributes nothing
    if (wt != 0.f) acc = fmaf(wt, g[d], acc);
    den += wt;
  }
  out[(int64_t)row * 128 + d] = __float2bfloat16(den > 0.f ? acc / den : 0.f);
}


// ---- the same exchanges over peer memory ----------------------------------------------------------------------
// Every rank owns one symmetric buffer (same layout on every GPU, mapped into every peer's address space):
//   gather 1  [world][rows][Kl][2] i64, gather 2 [world][rows_q][129] f32, flags 1 u32[world], flags 2 u32[world].
// The packing kernel stores its rows straight into slot `rank` of EVERY peer's gather area (16-byte stores over
// NVLink), and after its last block has finished it publishes the exchange number into word `rank` of every peer's
// flag array (release, system scope).  The consuming kernel on each GPU polls its OWN flag words (acquire, system
// scope) until all `world` of them carry the current exchange number, then reads its own gather area with L1
// bypassed.  Exchange numbers come from a word in local memory that the packing kernel advances, so a replayed
// CUDA graph needs no host-side argument.  One gather area per exchange is enough: a rank can only overwrite a
// peer's slot after it has passed the other exchange of the same layer, which the peer feeds only after it has
// consumed this one.  The poll is bounded (about a second): on expiry the kernel raises the status word in the
// local control block and carries on with whatever is in the buffer; the host checks the word.
struct PeerSet { char* base[16]; };
struct PeerCtl { unsigned epoch, arrivals, status, pad; };   // one per exchange, local memory

constexpr long long SHARD_WAIT_POLLS = 1500000;   // x (200 ns back-off + one load): about a second

__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Called by every thread of every block after its remote stores; the last block to arrive publishes the flags.
__device__ __forceinline__ void peer_publish(PeerCtl* ctl, const PeerSet& peers, int64_t flags_off, int rank, int world,
                                             unsigned total_blocks) {
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned prev = atomicAdd(&ctl->arrivals, 1u);
    if (prev == total_blocks - 1) {
      __threadfence_system();
      const unsigned epoch = ctl->epoch + 1;
      for (int p = 0; p < world; p++)
        st_release_sys(reinterpret_cast<unsigned*>(peers.base[p] + flags_off) + rank, epoch);
      ctl->arrivals = 0;
      ctl->epoch = epoch;     // read by the consuming kernel, which is ordered after this one on the stream
    }
  }
}

// Thread 0 of the block polls the local flag words; returns after a block barrier.
__device__ __forceinline__ void peer_wait(PeerCtl* ctl, const unsigned* flags, int world) {
  if (threadIdx.x == 0) {
    const unsigned want = *reinterpret_cast<volatile unsigned*>(&ctl->epoch);
    for (int r = 0; r < world; r++) {
      long long polls = 0;
      while ((int)(ld_acquire_sys(flags + r) - want) < 0) {
        if (++polls > SHARD_WAIT_POLLS) {
          atomicExch(&ctl->status, 1u);
          break;
        }
        __nanosleep(200);
      }
    }
  }
  __syncthreads();
}

__global__ void __launch_bounds__(256) shard_pack_peer_kernel(const int64_t* __restrict__ cand, const float* __restrict__ scores,
                                                              const int64_t* __restrict__ local_final, int C, int Kl,
                                                              int64_t start, PeerSet peers, int64_t gather_off,
                                                              int64_t flags_off, int rank, int world, int rows, PeerCtl* ctl,
                                                              const int32_t* __restrict__ n_sel,
                                                              const int32_t* __restrict__ n_cand) {
  const int row = blockIdx.y;
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j < Kl) {
    const longlong2 v = shard_entry(cand, scores, local_final, n_sel, n_cand, row, j, C, Kl, start);
    const int64_t slot = (((int64_t)rank * rows + row) * Kl + j) * 16;
    for (int q = 0; q < world; q++) *reinterpret_cast<longlong2*>(peers.base[q] + gather_off + slot) = v;
  }
  peer_publish(ctl, peers, flags_off, rank, world, gridDim.x * gridDim.y);
}

__global__ void __launch_bounds__(256) shard_unpack_peer_kernel(const int64_t* gathered, const unsigned* flags, PeerCtl* ctl,
                                                                float* __restrict__ scores, int64_t* __restrict__ indices,
                                                                int world, int rows, int Kl) {
  peer_wait(ctl, flags, world);
  const int row = blockIdx.y;
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= world * Kl) return;
  const int w = t / Kl, j = t - w * Kl;
  const longlong2 v = __ldcg(reinterpret_cast<const longlong2*>(gathered + (((int64_t)w * rows + row) * Kl + j) * 2));
  scores[(int64_t)row * world * Kl + t] = __int_as_float((int)v.x);
  indices[(int64_t)row * world * Kl + t] = v.y;
}

__global__ void __launch_bounds__(128) shard_pack_partial_peer_kernel(const __nv_bfloat16* __restrict__ out, const float* __restrict__ lse,
                                                                      PeerSet peers, int64_t gather_off, int64_t flags_off,
                                                                      int rank, int world, int rows, PeerCtl* ctl) {
  const int row = blockIdx.x, d = threadIdx.x;
  const float v = __bfloat162float(out[(int64_t)row * 128 + d]);
  const float l = lse[row];
  const int64_t slot = ((int64_t)rank * rows + row) * 129;
  for (int q = 0; q < world; q++) {
    float* g = reinterpret_cast<float*>(peers.base[q] + gather_off) + slot;
    g[d] = v;
    if (d == 0) g[128] = l;
  }
  peer_publish(ctl, peers, flags_off, rank, world, gridDim.x);
}

__global__ void __launch_bounds__(128) shard_merge_partial_peer_kernel(const float* gathered, const unsigned* flags, PeerCtl* ctl,
                                                                       __nv_bfloat16* __restrict__ out, int world, int rows) {
  peer_wait(ctl, flags, world);
  const int row = blockIdx.x, d = threadIdx.x;
  float m = -INFINITY;
  for (int w = 0; w < world; w++) m = fmaxf(m, __ldcg(gathered + ((int64_t)w * rows + row) * 129 + 128));
  float acc = 0.f, den = 0.f;
  for (int w = 0; w < world; w++) {
    const float* g = gathered + ((int64_t)w * rows + row) * 129;
    const float l = __ldcg(g + 128);
    const float wt = (l == -INFINITY) ? 0.f : exp2f(l - m);
    if (wt != 0.f) acc = fmaf(wt, __ldcg(g + d), acc);
    den += wt;
  }
  out[(int64_t)row * 128 + d] = __float2bfloat16(den > 0.f ? acc / den : 0.f);
}

// ---- tensor-parallel reduction / all-gather of one short row over peer memory, one launch ------------------------
// Every 32-bit data word (two bf16) travels with the exchange number in ONE 8-byte store {data, number} into the
// receiver's gather area, slot [source rank][word].  An aligned 8-byte store is single-copy atomic, so a receiver that
// reads the number it expects in a slot has that slot's data with it: no separate flag words, no fence between data
// and flag, and the exchange costs one NVLink store latency plus the polling.  Each thread owns words t, t + 512, ...:
// it stores them into every peer's area, then polls its own words of every source (bounded), sums the `world`
// contributions in rank order in fp32 (bit-identical results on every rank), and optionally the block takes the
// RMS-norm of the reduced row.  Consecutive exchanges alternate between two gather areas (exchange number parity): a
// rank can send exchange k + 2 only after it completed k + 1, for which every peer had to send k + 1, i.e. had finished
// reading k; so a slot of area (k & 1) is never overwritten before its reader is done with it.
__device__ __forceinline__ void st_slot(unsigned long long* p, unsigned data, unsigned tag) {
  asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(data), "r"(tag) : "memory");
}
__device__ __forceinline__ uint2 ld_slot(const unsigned long long* p) {
  uint2 v;
  asm volatile("ld.relaxed.sys.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
  return v;
}

constexpr int TP_THREADS = 512;
constexpr int TP_WORDS_MAX = 8;   // words per thread: rows of up to 8192 bf16
constexpr int TP_WORLD_MAX = 16;

__global__ void __launch_bounds__(TP_THREADS) tp_allreduce_kernel(const unsigned* __restrict__ partial,
                                                                  const unsigned* __restrict__ residual,
                                                                  unsigned* __restrict__ out, int n32, PeerSet peers,
                                                                  int64_t gather_off, int64_t area_bytes, int rank, int world,
                                                                  PeerCtl* ctl, const unsigned* __restrict__ norm_w,
                                                                  unsigned* __restrict__ normed, float eps, int gather_only) {
  const int tid = threadIdx.x;
  __shared__ unsigned s_epoch;
  __shared__ float s_part[TP_THREADS / 32];
  pdl_wait();     // the partial row comes from the kernel before this one
  pdl_trigger();
  if (tid == 0) s_epoch = ctl->epoch + 1;
  __syncthreads();
  const unsigned epoch = s_epoch;
  if (tid == 0) ctl->epoch = epoch;
  const int64_t area = gather_off + (int64_t)(epoch & 1u) * area_bytes;
  // ---- send ----
#pragma unroll
  for (int k = 0; k < TP_WORDS_MAX; k++) {
    const int w = tid + k * TP_THREADS;
    if (w < n32) {
      const unsigned v = partial[w];
      for (int q = 0; q < world; q++)
        st_slot(reinterpret_cast<unsigned long long*>(peers.base[q] + area) + (int64_t)rank * n32 + w, v, epoch);
    }
  }
  // ---- receive: my words of every source, in rank order ----
  const unsigned long long* mine = reinterpret_cast<const unsigned long long*>(peers.base[rank] + area);
  float ss = 0.0f;
  bool late = false;
#pragma unroll
  for (int k = 0; k < TP_WORDS_MAX; k++) {
    const int w = tid + k * TP_THREADS;
    if (w >= n32) continue;
    float lo = 0.0f, hi = 0.0f;
    if (!gather_only && residual) {
      const unsigned r = residual[w];
      lo = __uint_as_float(r << 16), hi = __uint_as_float(r & 0xffff0000u);
    }
    // one sweep loads this word's slot of every source back to back (all loads in flight), then looks at the numbers;
    // sweeps repeat (bounded) until every source's store has landed
    uint2 v[TP_WORLD_MAX];
    long long polls = 0;
    for (;;) {
#pragma unroll
      for (int r = 0; r < TP_WORLD_MAX; r++)
        if (r < world) v[r] = ld_slot(mine + (int64_t)r * n32 + w);
      bool all = true;
#pragma unroll
      for (int r = 0; r < TP_WORLD_MAX; r++)
        if (r < world) all = all && v[r].y == epoch;
      if (all) break;
      // one full budget per thread and launch: after a first expiry the remaining words get a token budget, so a
      // launch whose peer never arrives still ends after about a second
      if (++polls > (late ? 1000 : SHARD_WAIT_POLLS)) {
        late = true;
        break;
      }
      __nanosleep(20);
    }
#pragma unroll
    for (int r = 0; r < TP_WORLD_MAX; r++) {
      if (r >= world) continue;
      if (gather_only) {
        out[(int64_t)r * n32 + w] = v[r].x;
      } else {
        lo = __fadd_rn(lo, __uint_as_float(v[r].x << 16));
        hi = __fadd_rn(hi, __uint_as_float(v[r].x & 0xffff0000u));
      }
    }
    if (!gather_only) {
      const unsigned o = (unsigned)f2bf(lo) | ((unsigned)f2bf(hi) << 16);
      out[w] = o;
      const float a = __uint_as_float(o << 16), b = __uint_as_float(o & 0xffff0000u);
      ss = fmaf(a, a, fmaf(b, b, ss));
    }
  }
  if (late) atomicExch(&ctl->status, 1u);
  if (gather_only || !normed) return;
  // the RMS-norm of the reduced row, for the projection that follows: x = bf16(out * rsqrt(mean(out^2) + eps) * w)
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
  if ((tid & 31) == 0) s_part[tid >> 5] = ss;
  __syncthreads();
  float tot = 0.0f;
#pragma unroll
  for (int k = 0; k < TP_THREADS / 32; k++) tot += s_part[k];
  const float rstd = rsqrtf(tot / (float)(n32 * 2) + eps);
#pragma unroll
  for (int k = 0; k < TP_WORDS_MAX; k++) {   // every thread re-reads what it wrote itself
    const int w = tid + k * TP_THREADS;
    if (w < n32) {
      const unsigned h = out[w], g = norm_w[w];
      normed[w] = (unsigned)f2bf(__uint_as_float(h << 16) * rstd * __uint_as_float(g << 16)) |
                  ((unsigned)f2bf(__uint_as_float(h & 0xffff0000u) * rstd * __uint_as_float(g & 0xffff0000u)) << 16);
    }
  }
}

}  // namespace pk

using namespace pk;

static int counts_arg(const pk_tensor* t, int64_t bs, int64_t H, const char* name, const int32_t** out) {
  *out = nullptr;
  if (!t) return PK_OK;
  PK_REQUIRE(t->data && t->dtype == PK_I32 && t->ndim == 2 && is_contig(t) && t->shape[0] == bs && t->shape[1] == H,
             "%s must be contiguous i32 [bs,H]", name);
  *out = (const int32_t*)t->data;
  return PK_OK;
}

extern "C" int pk_shard_pack_topk(const pk_tensor* cand, const pk_tensor* scores, const pk_tensor* local_final,
                                  int64_t start, const pk_tensor* n_sel, const pk_tensor* n_cand,
                                  const pk_tensor* packed, void* stream) {
  PK_CHECK_TENSOR(cand, PK_I64, 3);
  PK_CHECK_TENSOR(scores, PK_F32, 3);
  PK_CHECK_TENSOR(local_final, PK_I64, 3);
  PK_CHECK_TENSOR(packed, PK_I64, 4);
  const int64_t bs = cand->shape[0], H = cand->shape[1], C = cand->shape[2], Kl = local_final->shape[2];
  PK_REQUIRE(is_contig(cand) && is_contig(scores) && is_contig(local_final) && is_contig(packed), "tensors must be contiguous");
  PK_REQUIRE(scores->shape[0] == bs && scores->shape[1] == H && scores->shape[2] == C, "scores must be [bs,H,C] like cand");
  PK_REQUIRE(local_final->shape[0] == bs && local_final->shape[1] == H, "local_final must be [bs,H,Kl]");
  PK_REQUIRE(packed->shape[0] == bs && packed->shape[1] == H && packed->shape[2] == Kl && packed->shape[3] == 2,
             "packed must be [bs,H,Kl,2]");
  PK_REQUIRE(C >= 1 && C < (1LL << 31) && Kl < (1LL << 31) && bs * H < 65536, "sizes out of range");
  PK_REQUIRE((reinterpret_cast<uintptr_t>(packed->data) & 15) == 0, "packed must be 16-byte aligned");
  if (bs * H * Kl == 0) return PK_OK;
  const int32_t *ns = nullptr, *nc = nullptr;
  int rc;
  if ((rc = counts_arg(n_sel, bs, H, "n_sel", &ns)) || (rc = counts_arg(n_cand, bs, H, "n_cand", &nc))) return rc;
  StageTimer timer(ST_SHARD_SEND, (cudaStream_t)stream);
  shard_pack_kernel<<<dim3((unsigned)((Kl + 255) / 256), (unsigned)(bs * H)), 256, 0, (cudaStream_t)stream>>>(
      (const int64_t*)cand->data, (const float*)scores->data, (const int64_t*)local_final->data, (int64_t*)packed->data,
      (int)C, (int)Kl, start, ns, nc);
  return check_launch("shard_pack_topk");
}

extern "C" int pk_shard_unpack_topk(const pk_tensor* gathered, const pk_tensor* scores, const pk_tensor* indices,
                                    void* stream) {
  PK_CHECK_TENSOR(gathered, PK_I64, 5);
  PK_CHECK_TENSOR(scores, PK_F32, 3);
  PK_CHECK_TENSOR(indices, PK_I64, 3);
  const int64_t world = gathered->shape[0], bs = gathered->shape[1], H = gathered->shape[2], Kl = gathered->shape[3];
  PK_REQUIRE(gathered->shape[4] == 2 && is_contig(gathered) && is_contig(scores) && is_contig(indices),
             "gathered must be contiguous [world,bs,H,Kl,2], outputs contiguous");
  PK_REQUIRE(scores->shape[0] == bs && scores->shape[1] == H && scores->shape[2] == world * Kl &&
                 indices->shape[0] == bs && indices->shape[1] == H && indices->shape[2] == world * Kl,
             "scores / indices must be [bs,H,world*Kl]");
  PK_REQUIRE(world * Kl < (1LL << 31) && bs * H < 65536, "sizes out of range");
  PK_REQUIRE((reinterpret_cast<uintptr_t>(gathered->data) & 15) == 0, "gathered must be 16-byte aligned");
  if (numel(gathered) == 0) return PK_OK;
  StageTimer timer(ST_SHARD_RECV, (cudaStream_t)stream);
  shard_unpack_kernel<<<dim3((unsigned)((world * Kl + 255) / 256), (unsigned)(bs * H)), 256, 0, (cudaStream_t)stream>>>(
      (const int64_t*)gathered->data, (float*)scores->data, (int64_t*)indices->data, (int)world, (int)(bs * H), (int)Kl);
  return check_launch("shard_unpack_topk");
}

extern "C" int pk_shard_owned_rows(const pk_tensor* final_indices, int64_t start, int64_t end, const pk_tensor* local,
                                   const pk_tensor* n_owned, void* stream) {
  PK_CHECK_TENSOR(final_indices, PK_I64, 3);
  PK_CHECK_TENSOR(local, PK_I64, 3);
  PK_CHECK_TENSOR(n_owned, PK_I32, 2);
  const int64_t bs = final_indices->shape[0], H = final_indices->shape[1], K = final_indices->shape[2];
  PK_REQUIRE(is_contig(final_indices) && is_contig(local) && is_contig(n_owned), "tensors must be contiguous");
  PK_REQUIRE(local->shape[0] == bs && local->shape[1] == H && local->shape[2] == K && n_owned->shape[0] == bs &&
                 n_owned->shape[1] == H,
             "local must be [bs,H,K] and n_owned [bs,H]");
  PK_REQUIRE(start <= end && K < (1LL << 31), "bad shard range");
  if (bs * H == 0) return PK_OK;
  StageTimer timer(ST_SHARD_OWNED, (cudaStream_t)stream);
  shard_owned_kernel<<<(unsigned)(bs * H), 256, 0, (cudaStream_t)stream>>>(
      (const int64_t*)final_indices->data, (int64_t*)local->data, (int32_t*)n_owned->data, (int)K, start, end);
  return check_launch("shard_owned_rows");
}

extern "C" int pk_shard_pack_partial(const pk_tensor* out, const pk_tensor* lse, const pk_tensor* packed, void* stream) {
  PK_CHECK_TENSOR(out, PK_BF16, 4);
  PK_CHECK_TENSOR(lse, PK_F32, 2);
  PK_CHECK_TENSOR(packed, PK_F32, 3);
  const int64_t bs = out->shape[0], Hq = out->shape[2];
  PK_REQUIRE(out->shape[1] == 1 && out->shape[3] == 128 && is_contig(out), "out must be contiguous [bs,1,Hq,128]");
  PK_REQUIRE(lse->shape[0] == bs && lse->shape[1] == Hq && is_contig(lse), "lse must be contiguous [bs,Hq]");
  PK_REQUIRE(packed->shape[0] == bs && packed->shape[1] == Hq && packed->shape[2] == 129 && is_contig(packed),
             "packed must be contiguous [bs,Hq,129]");
  if (bs * Hq == 0) return PK_OK;
  StageTimer timer(ST_SHARD_SEND, (cudaStream_t)stream);
  shard_pack_partial_kernel<<<(unsigned)(bs * Hq), 128, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)out->data, (const float*)lse->data, (float*)packed->data);
  return check_launch("shard_pack_partial");
}

extern "C" int pk_shard_merge_partial(const pk_tensor* gathered, const pk_tensor* out, void* stream) {
  PK_CHECK_TENSOR(gathered, PK_F32, 4);
  PK_CHECK_TENSOR(out, PK_BF16, 4);
  const int64_t world = gathered->shape[0], bs = gathered->shape[1], Hq = gathered->shape[2];
  PK_REQUIRE(gathered->shape[3] == 129 && is_contig(gathered), "gathered must be contiguous [world,bs,Hq,129]");
  PK_REQUIRE(out->shape[0] == bs && out->shape[1] == 1 && out->shape[2] == Hq && out->shape[3] == 128 && is_contig(out),
             "out must be contiguous [bs,1,Hq,128]");
  PK_REQUIRE(world >= 1 && world <= 1024, "world size out of range");
  if (bs * Hq == 0) return PK_OK;
  StageTimer timer(ST_SHARD_RECV, (cudaStream_t)stream);
  shard_merge_partial_kernel<<<(unsigned)(bs * Hq), 128, 0, (cudaStream_t)stream>>>(
      (const float*)gathered->data, (__nv_bfloat16*)out->data, (int)world, (int)(bs * Hq));
  return check_launch("shard_merge_partial");
}

// ---- peer-memory forms ------------------------------------------------------------------------------------------
static int fill_peers(PeerSet* ps, const uint64_t* peer_bases, int world, int rank) {
  PK_REQUIRE(peer_bases != nullptr, "peer_bases is null");
  PK_REQUIRE(world >= 1 && world <= 16 && rank >= 0 && rank < world, "world must be 1..16 and rank inside it");
  for (int i = 0; i < 16; i++) ps->base[i] = nullptr;
  for (int i = 0; i < world; i++) {
    PK_REQUIRE(peer_bases[i] != 0 && (peer_bases[i] & 15) == 0, "peer buffer %d is null or not 16-byte aligned", i);
    ps->base[i] = reinterpret_cast<char*>(peer_bases[i]);
  }
  return PK_OK;
}

extern "C" int pk_shard_exchange_topk(const pk_tensor* cand, const pk_tensor* scores, const pk_tensor* local_final,
                                      int64_t start, const pk_tensor* n_sel, const pk_tensor* n_cand,
                                      const uint64_t* peer_bases, int world, int rank,
                                      int64_t gather_offset, int64_t flags_offset, void* control, void* stream) {
  PK_CHECK_TENSOR(cand, PK_I64, 3);
  PK_CHECK_TENSOR(scores, PK_F32, 3);
  PK_CHECK_TENSOR(local_final, PK_I64, 3);
  const int64_t bs = cand->shape[0], H = cand->shape[1], C = cand->shape[2], Kl = local_final->shape[2];
  PK_REQUIRE(is_contig(cand) && is_contig(scores) && is_contig(local_final), "tensors must be contiguous");
  PK_REQUIRE(scores->shape[0] == bs && scores->shape[1] == H && scores->shape[2] == C, "scores must be [bs,H,C] like cand");
  PK_REQUIRE(local_final->shape[0] == bs && local_final->shape[1] == H, "local_final must be [bs,H,Kl]");
  PK_REQUIRE(C >= 1 && C < (1LL << 31) && Kl >= 1 && Kl < (1LL << 31) && bs * H >= 1 && bs * H < 65536, "sizes out of range");
  PK_REQUIRE(control != nullptr && gather_offset >= 0 && flags_offset >= 0 && gather_offset % 16 == 0 && flags_offset % 4 == 0,
             "control block or offsets invalid");
  PeerSet ps;
  int rc;
  if ((rc = fill_peers(&ps, peer_bases, world, rank))) return rc;
  const int32_t *ns = nullptr, *nc = nullptr;
  if ((rc = counts_arg(n_sel, bs, H, "n_sel", &ns)) || (rc = counts_arg(n_cand, bs, H, "n_cand", &nc))) return rc;
  StageTimer timer(ST_SHARD_SEND, (cudaStream_t)stream);
  shard_pack_peer_kernel<<<dim3((unsigned)((Kl + 255) / 256), (unsigned)(bs * H)), 256, 0, (cudaStream_t)stream>>>(
      (const int64_t*)cand->data, (const float*)scores->data, (const int64_t*)local_final->data, (int)C, (int)Kl, start, ps,
      gather_offset, flags_offset, rank, world, (int)(bs * H), (PeerCtl*)control, ns, nc);
  return check_launch("shard_exchange_topk");
}

extern "C" int pk_shard_collect_topk(uint64_t local_base, int64_t gather_offset, int64_t flags_offset, void* control,
                                     int world, int64_t Kl, const pk_tensor* scores, const pk_tensor* indices, void* stream) {
  PK_CHECK_TENSOR(scores, PK_F32, 3);
  PK_CHECK_TENSOR(indices, PK_I64, 3);
  const int64_t bs = scores->shape[0], H = scores->shape[1];
  PK_REQUIRE(world >= 1 && world <= 16 && Kl >= 1 && world * Kl < (1LL << 31) && bs * H >= 1 && bs * H < 65536, "sizes out of range");
  PK_REQUIRE(is_contig(scores) && is_contig(indices) && scores->shape[2] == world * Kl && indices->shape[0] == bs &&
                 indices->shape[1] == H && indices->shape[2] == world * Kl,
             "scores / indices must be contiguous [bs,H,world*Kl]");
  PK_REQUIRE(local_base != 0 && control != nullptr && gather_offset % 16 == 0 && flags_offset % 4 == 0, "buffer or offsets invalid");
  char* base = reinterpret_cast<char*>(local_base);
  StageTimer timer(ST_SHARD_RECV, (cudaStream_t)stream);
  shard_unpack_peer_kernel<<<dim3((unsigned)((world * Kl + 255) / 256), (unsigned)(bs * H)), 256, 0, (cudaStream_t)stream>>>(
      (const int64_t*)(base + gather_offset), (const unsigned*)(base + flags_offset), (PeerCtl*)control, (float*)scores->data,
      (int64_t*)indices->data, world, (int)(bs * H), (int)Kl);
  return check_launch("shard_collect_topk");
}

extern "C" int pk_shard_exchange_partial(const pk_tensor* out, const pk_tensor* lse, const uint64_t* peer_bases, int world,
                                         int rank, int64_t gather_offset, int64_t flags_offset, void* control, void* stream) {
  PK_CHECK_TENSOR(out, PK_BF16, 4);
  PK_CHECK_TENSOR(lse, PK_F32, 2);
  const int64_t bs = out->shape[0], Hq = out->shape[2];
  PK_REQUIRE(out->shape[1] == 1 && out->shape[3] == 128 && is_contig(out), "out must be contiguous [bs,1,Hq,128]");
  PK_REQUIRE(lse->shape[0] == bs && lse->shape[1] == Hq && is_contig(lse), "lse must be contiguous [bs,Hq]");
  PK_REQUIRE(bs * Hq >= 1 && control != nullptr && gather_offset % 16 == 0 && flags_offset % 4 == 0, "control block or offsets invalid");
  PeerSet ps;
  int rc;
  if ((rc = fill_peers(&ps, peer_bases, world, rank))) return rc;
  StageTimer timer(ST_SHARD_SEND, (cudaStream_t)stream);
  shard_pack_partial_peer_kernel<<<(unsigned)(bs * Hq), 128, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)out->data, (const float*)lse->data, ps, gather_offset, flags_offset, rank, world, (int)(bs * Hq),
      (PeerCtl*)control);
  return check_launch("shard_exchange_partial");
}

extern "C" int pk_shard_collect_partial(uint64_t local_base, int64_t gather_offset, int64_t flags_offset, void* control,
                                        int world, const pk_tensor* out, void* stream) {
  PK_CHECK_TENSOR(out, PK_BF16, 4);
  const int64_t bs = out->shape[0], Hq = out->shape[2];
  PK_REQUIRE(out->shape[1] == 1 && out->shape[3] == 128 && is_contig(out) && bs * Hq >= 1, "out must be contiguous [bs,1,Hq,128]");
  PK_REQUIRE(world >= 1 && world <= 16 && local_base != 0 && control != nullptr && gather_offset % 16 == 0 && flags_offset % 4 == 0,
             "buffer or offsets invalid");
  char* base = reinterpret_cast<char*>(local_base);
  StageTimer timer(ST_SHARD_RECV, (cudaStream_t)stream);
  shard_merge_partial_peer_kernel<<<(unsigned)(bs * Hq), 128, 0, (cudaStream_t)stream>>>(
      (const float*)(base + gather_offset), (const unsigned*)(base + flags_offset), (PeerCtl*)control,
      (__nv_bfloat16*)out->data, world, (int)(bs * Hq));
  return check_launch("shard_collect_partial");
}

extern "C" int pk_tp_allreduce(const pk_tensor* partial, const pk_tensor* residual, const pk_tensor* out,
                               const uint64_t* peer_bases, int world, int rank, int64_t gather_offset, int64_t area_bytes,
                               int64_t flags_offset, void* control, const pk_tensor* norm_weight,
                               const pk_tensor* normed_out, double eps, void* stream) {
  PK_CHECK_TENSOR(partial, PK_BF16, 2);
  PK_CHECK_TENSOR(out, PK_BF16, 2);
  const int64_t n = numel(partial);
  const uint4* nw = nullptr;
  uint4* nout = nullptr;
  if (normed_out) {
    PK_CHECK_TENSOR(normed_out, PK_BF16, 2);
    PK_CHECK_TENSOR(norm_weight, PK_BF16, 1);
    PK_REQUIRE(partial->shape[0] == 1, "the fused RMS-norm takes one row (partial must be [1,n])");
    PK_REQUIRE(is_contig(normed_out) && numel(normed_out) == n && is_contig(norm_weight) && numel(norm_weight) == n &&
                   (reinterpret_cast<uintptr_t>(normed_out->data) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(norm_weight->data) & 15) == 0,
               "normed_out / norm_weight must be contiguous bf16 of n elements, 16-byte aligned");
    nw = (const uint4*)norm_weight->data;
    nout = (uint4*)normed_out->data;
  }
  PK_REQUIRE(is_contig(partial) && is_contig(out) && numel(out) == n && n >= 8 && n % 8 == 0 &&
                 n <= 2 * TP_THREADS * TP_WORDS_MAX,
             "partial / out must be contiguous bf16 with the same number of elements, a multiple of 8, at most 8192");
  PK_REQUIRE((reinterpret_cast<uintptr_t>(partial->data) & 15) == 0 && (reinterpret_cast<uintptr_t>(out->data) & 15) == 0,
             "partial / out must be 16-byte aligned");
  const uint4* res = nullptr;
  if (residual) {
    PK_CHECK_TENSOR(residual, PK_BF16, 2);
    PK_REQUIRE(is_contig(residual) && numel(residual) == n && (reinterpret_cast<uintptr_t>(residual->data) & 15) == 0,
               "residual must match partial and be 16-byte aligned");
    res = (const uint4*)residual->data;
  }
  PK_REQUIRE(control != nullptr && gather_offset >= 0 && gather_offset % 16 == 0 && flags_offset >= 0 && flags_offset % 4 == 0 &&
                 area_bytes >= (int64_t)world * n * 4 && area_bytes % 16 == 0,
             "control block, offsets or area size invalid (one area holds world x n/2 eight-byte slots; two areas follow "
             "each other)");
  PeerSet ps;
  int rc;
  if ((rc = fill_peers(&ps, peer_bases, world, rank))) return rc;
  StageTimer timer(ST_REDUCE, (cudaStream_t)stream);
  launch_chain(tp_allreduce_kernel, dim3(1), dim3(TP_THREADS), 0, (cudaStream_t)stream, (const unsigned*)partial->data,
               (const unsigned*)res, (unsigned*)out->data, (int)(n / 2), ps, gather_offset, area_bytes, rank, world,
               (PeerCtl*)control, (const unsigned*)nw, (unsigned*)nout, (float)eps, 0);
  return check_launch("tp_allreduce");
}

extern "C" int pk_tp_allgather(const pk_tensor* part, const pk_tensor* out, const uint64_t* peer_bases, int world, int rank,
                               int64_t gather_offset, int64_t area_bytes, int64_t flags_offset, void* control,
                               void* stream) {
  PK_CHECK_TENSOR(part, PK_BF16, 2);
  PK_CHECK_TENSOR(out, PK_BF16, 2);
  const int64_t n = numel(part);
  PK_REQUIRE(is_contig(part) && is_contig(out) && numel(out) == n * world && n >= 8 && n % 8 == 0 &&
                 n <= 2 * TP_THREADS * TP_WORDS_MAX,
             "part must be contiguous bf16 of n elements (a multiple of 8, at most 8192), out of world x n");
  PK_REQUIRE((reinterpret_cast<uintptr_t>(part->data) & 15) == 0 && (reinterpret_cast<uintptr_t>(out->data) & 15) == 0,
             "part / out must be 16-byte aligned");
  PK_REQUIRE(control != nullptr && gather_offset >= 0 && gather_offset % 16 == 0 && flags_offset >= 0 && flags_offset % 4 == 0 &&
                 area_bytes >= (int64_t)world * n * 4 && area_bytes % 16 == 0,
             "control block, offsets or area size invalid (one area holds world x n/2 eight-byte slots; two areas follow "
             "each other)");
  PeerSet ps;
  int rc;
  if ((rc = fill_peers(&ps, peer_bases, world, rank))) return rc;
  StageTimer timer(ST_REDUCE, (cudaStream_t)stream);
  launch_chain(tp_allreduce_kernel, dim3(1), dim3(TP_THREADS), 0, (cudaStream_t)stream, (const unsigned*)part->data,
               (const unsigned*)nullptr, (unsigned*)out->data, (int)(n / 2), ps, gather_offset, area_bytes, rank, world,
               (PeerCtl*)control, (const unsigned*)nullptr, (unsigned*)nullptr, 0.0f, 1);
  return check_launch("tp_allgather");
}

/*
 * pariskv_b200 -- C ABI of the B200 (sm_100a) ParisKV retrieval engine.
 *
 * Every entry point takes plain tensor descriptors (pointer, shape, strides, dtype tag) and a
 * CUDA stream handle, launches asynchronously on that stream, allocates nothing on the device
 * (scratch is passed in by the caller, see pk_*_workspace_bytes) and returns a status code:
 * 0 on success, non-zero on a rejected argument or a CUDA launch error; pk_last_error() then
 * holds a message (thread local).  The caller makes the device of the tensors current.
 *
 * Each declaration names the reference interface it replaces (path inside the reference
 * project : line).  Logical tensor shapes are the reference's; strides are free unless stated,
 * so the reference's plane-major tensors ([bs,H,16,N]) and this library's preferred key-major
 * storage ([bs,H,N,16] exposed as a permuted view) both work; the key-major form is the fast one.
 *
 * Deterministic selection everywhere: ties are broken by the lowest index and outputs have a
 * fixed order (stated per function); the reference's own kernels leave both to atomics order.
 */
#ifndef PARISKV_B200_H
#define PARISKV_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PK_MAX_DIMS 6

enum pk_dtype { PK_U8 = 0, PK_I32 = 1, PK_I64 = 2, PK_F32 = 3, PK_BF16 = 4 };

enum pk_status {
  PK_OK = 0,
  PK_ERR_ARG = 1,       /* bad shape / dtype / stride / null pointer */
  PK_ERR_CUDA = 2,      /* a CUDA runtime call or launch failed */
  PK_ERR_UNSUPPORTED = 3,
  PK_ERR_WORKSPACE = 4  /* workspace missing or too small */
};

/* A strided view.  stride[] is in ELEMENTS of dtype.  data may be a device pointer or, where
 * a function says "host", a pinned host pointer that the device can read (UVA). */
typedef struct pk_tensor {
  void* data;
  int32_t dtype; /* enum pk_dtype */
  int32_t ndim;
  int64_t shape[PK_MAX_DIMS];
  int64_t stride[PK_MAX_DIMS];
} pk_tensor;

int pk_version(void);
const char* pk_last_error(void);
/* Number of kernels launched by this library in this process (all threads). */
int64_t pk_launch_count(void);

/* Optional instrumentation, no counterpart in the reference: when enabled, every kernel launch of the
 * decode path is bracketed by CUDA events on its own stream.  pk_timing_read waits for the recorded
 * events, sums elapsed milliseconds and launch counts per stage (stage ids: 0 query prep, 1 cluster
 * ranking/table, 2 collision, 3 select+rerank, 4 final top-k, 5 attention tiles, 6 attention merge,
 * 7 encode, 8 stand-alone top-k, 9 stand-alone rerank, 10 UVA gather, 11 cluster histogram, 12 row append,
 * 13 decode glue, 14 tensor-parallel reduce, 15 shard pack / send, 16 shard receive / merge, 17 shard owned rows,
 * 18 shard count-histogram reduce, 19 matrix-vector product, 20 adaptive-k selection) and clears the record. */
int pk_timing_enable(int on);
int pk_timing_read(double* ms_per_stage, int64_t* spans_per_stage, int n_stages);
/* Launches issued INTO A STREAM CAPTURE while timing is enabled are bracketed by external event-record nodes, which
 * every replay of the captured graph stamps again: pk_timing_read_graph waits for them and sums, per stage, what the
 * LAST replay measured (all graphs captured with timing on; it clears nothing).  pk_timing_clear_graph destroys those
 * events: call it only after the graphs that record them are gone. */
int pk_timing_read_graph(double* ms_per_stage, int64_t* spans_per_stage, int n_stages);
int pk_timing_clear_graph(void);

/* Process-wide option, no counterpart in the reference: launch the kernels of this library with programmatic
 * dependent launch.  A kernel may then be scheduled while its predecessor on the stream still runs; it does only
 * what does not depend on earlier kernels (the collision kernel its first code loads, a projection its first weight
 * loads) and then waits for the predecessor to complete, and every kernel releases its successor only after its own
 * wait, so completion is transitive along the stream.  Off by default; with the decode step replayed as a CUDA graph
 * it measured +1.9 % tokens/s at the 128K configuration on B200. */
int pk_set_pdl(int on);

/* ---- (a) key coding ---------------------------------------------------------------------- */

/* SRHT normalise-rotate + 8-bit sign code + 4-bit (sign | 3-bit level) code + fused rerank weight
 * for L keys per (batch, head); optionally adds the per-subspace code histogram of those keys.
 * Replaces polar_cache.batch_encode + _pack_4bit_codes + _count_cluster_keys
 * (cache_hub/polar_cache.py:924-978, :887-893, :980-996).
 *   keys          bf16 [bs,H,L,128]   last stride 1
 *   signs         bf16 [128]          SRHT diagonal (+1/-1)
 *   codebook      u8   [bs,H,16,L]
 *   block_weight  bf16 [bs,H,16,L]
 *   packed_4bit   u8   [bs,H,16,L,4]  last stride 1
 *   cluster_counts i32 [bs,H,16,256] contiguous, ADDED to; may be NULL */
int pk_encode_keys(const pk_tensor* keys, const pk_tensor* signs, const pk_tensor* codebook,
                   const pk_tensor* block_weight, const pk_tensor* packed_4bit,
                   const pk_tensor* cluster_counts, void* stream);

/* Histogram of codes per (batch, head, subspace): polar_cache._count_cluster_keys
 * (cache_hub/polar_cache.py:980-996).  counts i32 [bs,H,16,256] contiguous; accumulate != 0 adds
 * to the existing contents (as :774-775), 0 overwrites (as :600-601). */
int pk_count_clusters(const pk_tensor* codebook, const pk_tensor* counts, int accumulate, void* stream);

/* ---- query side -------------------------------------------------------------------------- */

/* GQA group mean + normalise + SRHT of the decode query: polar_cache.compute :1027-1031 and
 * _encode_query_blocks (cache_hub/polar_cache.py:905-922).
 *   queries  bf16 [bs,1,Hq,128] contiguous;  q_blocks bf16 [bs,H,16,8];  q_norm bf16 [bs,H,1]
 *   query_avg bf16 [bs,H,128] or NULL (the group mean, needed by the adaptive-k variants) */
int pk_query_prep(const pk_tensor* queries, const pk_tensor* signs, const pk_tensor* q_blocks,
                  const pk_tensor* q_norm, const pk_tensor* query_avg, void* stream);

/* Cluster ranking: scores = q_blocks @ sign_table^T, argsort descending
 * (cache_hub/polar_cache.py:1216-1217).  Ties go to the lower cluster id.
 *   q_blocks bf16 [bs,H,16,8] contiguous;  sorted_ids i64 [bs,H,16,256] contiguous */
int pk_rank_clusters(const pk_tensor* q_blocks, const pk_tensor* sorted_ids, void* stream);

/* ---- (b) collision counting --------------------------------------------------------------- */

/* Weighted multi-tier collision count: module update_cache_cnt.update_cache_cnt of
 * cache_hub/collision_fused/collision.cu:395-416 (Python: collison_interface.py:60-86).
 *   sorted_cluster_ids i64|i32 [bs,H,B,NC] contiguous, NC <= 256, B <= 32
 *   cluster_key_counts i32 [bs,H,B,NC] contiguous
 *   codebook           u8  [bs,H,B,N]  any strides
 *   tier_counts        host array of n_tiers (1..8) thresholds
 *   cache_cnt          i32 [bs,H,N] contiguous (output)
 *   workspace          >= pk_collision_workspace_bytes(bs,H,B,NC) bytes, device */
int64_t pk_collision_workspace_bytes(int64_t bs, int64_t H, int64_t B, int64_t NC);
int pk_collision_fused(const pk_tensor* sorted_cluster_ids, const pk_tensor* cluster_key_counts,
                       const pk_tensor* codebook, const int64_t* tier_counts, int n_tiers,
                       const pk_tensor* cache_cnt, void* workspace, int64_t workspace_bytes,
                       void* stream);

/* The same count for callers that cannot allocate device memory and have no scratch buffer to pass: code
 * running inside a serving runtime that owns the whole HBM pool, a latency-critical thread that must stay off
 * the device allocator, a caller that only holds input and output pointers.  It has no counterpart in the
 * reference.  The tier table lives in a 256 KB array inside the library image (held on every GPU that loads
 * the library, until exit), so the problem is limited to pk_collision_fused_static_max_triples() = 1024
 * (batch x head x subspace) triples, e.g. batch 8 x 8 heads x 16 subspaces; larger calls are rejected with
 * PK_ERR_WORKSPACE.  No cudaMalloc / cudaFree or allocating library call is made.  The first call on a device
 * looks up the array's device address (cudaGetSymbolAddress with that device current); make that first call
 * before any stream capture begins.  All calls share the one array and it keeps the last call's table:
 * nothing needs clearing (each call rewrites every word it reads), but two calls whose kernels may overlap on
 * the GPU (different streams, or different host threads on different streams) race on it - serialise them.
 * Arguments and results are those of pk_collision_fused. */
int64_t pk_collision_fused_static_max_triples(void);
int pk_collision_fused_static(const pk_tensor* sorted_cluster_ids, const pk_tensor* cluster_key_counts,
                              const pk_tensor* codebook, const int64_t* tier_counts, int n_tiers,
                              const pk_tensor* cache_cnt, void* stream);

/* Single-tier unfused collision count: module update_cache_cnt.update_cache_cnt of
 * cache_hub/collision/collision.cu:161-281 (Python: collision.py:87-98).
 *   sorted_cluster_ids i32 [bs,H,B,NC]; topk_cluster_cnt i32 [bs,H,B];
 *   code_book i32 [bs,H,N,B] contiguous; cache_cnt i32 [bs,H,N]; workspace as above */
int pk_collision(const pk_tensor* sorted_cluster_ids, const pk_tensor* topk_cluster_cnt,
                 const pk_tensor* code_book, const pk_tensor* cache_cnt, void* workspace,
                 int64_t workspace_bytes, void* stream);

/* ---- (c) top-k ------------------------------------------------------------------------------ */

/* Exact top-k of every row of input [rows, L] (i32 or f32, row stride free, last stride 1):
 * radix_topk_ext.{bucket_topk,radix_topk}[_3d] of cache_hub/topk/radix_topk.cu:258-401.
 * The selected set is the first k of (value descending, index ascending).
 *   out    i64 [rows, k] contiguous
 *   order  0: ascending index;  1: value descending (index ascending among equals), k <= 4096 */
int pk_topk(const pk_tensor* input, int64_t k, const pk_tensor* out, int order, void* stream);

/* Final select of the retrieval chain: torch.topk + gather of cache_hub/polar_cache.py:1300-1302,
 * on fp32 scores.  out[i] = cand[position], positions chosen as in pk_topk order 0.
 *   scores f32 [bs,H,C]; cand i64 [bs,H,C]; out i64 [bs,H,K] */
int pk_final_topk(const pk_tensor* scores, const pk_tensor* cand, int64_t K, const pk_tensor* out,
                  void* stream);

/* Fused adaptive-k: module adaptive_topk.adaptive_topk of
 * cache_hub/adaptive_k_fused/adaptive_topk.cu:272-314, and the varlen call contract of
 * cache_hub/polar_cache_adaptivek_varlen.py:1741-1753.
 *   sl_logits   f32 [bs,H,S]   already scaled, last stride 1
 *   cand_scores f32|bf16 [bs,H,C]; logit = float(score) * cand_scale
 *   sl_vnorm    f32 [bs,H,S]   last stride 1
 *   cand_indices i64 [bs,H,C]
 *   cand_vnorm  f32 [bs,H,C], or NULL with value_norm f32 [bs,H,cap] and sink_size:
 *               norm of candidate i = value_norm[b,h, cand_indices[i] + sink_size]
 *   adaptive_k  i64 [bs,H]; topk_indices i64 [bs,H,K_out], benefit descending;
 *   min_k/max_k clamp the result when max_k > 0 (polar_cache_adaptivek_varlen.py:1759) */
int pk_adaptive_topk(const pk_tensor* sl_logits, const pk_tensor* cand_scores, float cand_scale,
                     const pk_tensor* sl_vnorm, const pk_tensor* cand_indices,
                     const pk_tensor* cand_vnorm, const pk_tensor* value_norm, int64_t sink_size,
                     float threshold, int64_t K_out, int64_t min_k, int64_t max_k,
                     const pk_tensor* adaptive_k, const pk_tensor* topk_indices, void* stream);

/* ---- (d) rerank ------------------------------------------------------------------------------ */

/* 4-bit RaBitQ rerank: module rerank.partial_rerank of cache_hub/rerank/rerank.cu:141-224
 * (Python: rerank.py:214-263).  fp32 accumulation; correct for any batch size.
 *   coarse_indices i64 [bs,H,C] contiguous
 *   key_4bit  u8 [bs,H,16,N,4] last stride 1;  key_block_weight bf16 [bs,H,16,N] any strides
 *   q_blocks bf16 [bs,H,16,8] contiguous; q_norm bf16 [bs,H,1]; mag_centers bf16 [8]
 *   approx_scores bf16 [bs,H,C]; scores_f32 f32 [bs,H,C] or NULL; v4b bf16 [bs,H,16,C,8] or NULL */
int pk_rerank(const pk_tensor* coarse_indices, const pk_tensor* key_4bit,
              const pk_tensor* key_block_weight, const pk_tensor* q_blocks, const pk_tensor* q_norm,
              const pk_tensor* mag_centers, const pk_tensor* approx_scores,
              const pk_tensor* scores_f32, const pk_tensor* v4b, void* stream);

/* ---- (e) gather and sparse decode attention ----------------------------------------------------- */

/* UVA gather of selected K/V rows from pinned host memory: module h2d_gather_kv.h2d_gather_kv of
 * cache_hub/gather_trans/trans_h2d.cu:79-126 (Python: trans_h2d.py:65-105).
 *   src_k/src_v bf16 [bs,H,N,128] contiguous, pinned HOST (or device) memory
 *   selected_indices i64 [bs,H,K] contiguous (device); dst_k/dst_v bf16 [bs,H,cap>=K,128] device */
int pk_h2d_gather_kv(const pk_tensor* src_k, const pk_tensor* src_v, const pk_tensor* selected_indices,
                     const pk_tensor* dst_k, const pk_tensor* dst_v, void* stream);

/* Packed (varlen) UVA gather: call contract of cache_hub/polar_cache_adaptivek_varlen.py:1634-1644.
 * For virtual head vh = b*H + h and j < cu_seqlens_topk[vh+1]-cu_seqlens_topk[vh]:
 *   k_packed[cu_seqlens_k[vh] + sink_local_end + j] = src_k[b,h, indices_packed[cu_seqlens_topk[vh]+j]]
 *   k_packed/v_packed bf16 [total_k,128]; indices_packed i64 [total_topk]; cu_* i32 [bs*H+1] */
int pk_h2d_gather_kv_packed(const pk_tensor* src_k, const pk_tensor* src_v, const pk_tensor* k_packed,
                            const pk_tensor* v_packed, const pk_tensor* indices_packed,
                            const pk_tensor* cu_seqlens_topk, const pk_tensor* cu_seqlens_k,
                            int64_t sink_local_end, int64_t global_k, void* stream);

/* Host-side row gather out[b,h,k,:] = src[b,h,index[b,h,k],:] on CPU threads: module
 * polar_gather_ext.gather_kv_out_cpu of cache_hub/gather/gather_cpu.cpp:116-174.  All host memory;
 * returns PK_ERR_ARG on an out-of-range index.  n_threads <= 0 uses the hardware concurrency. */
int pk_gather_kv_out_cpu(const pk_tensor* src, const pk_tensor* index, const pk_tensor* out,
                         int n_threads);

/* Split-K sparse decode attention with the UVA fetch fused in: replaces h2d_gather_kv + torch.cat +
 * flash_attn_with_kvcache of cache_hub/polar_cache.py:1075-1105 (and the gather-on-GPU branch
 * :1090-1095).  Per (batch, KV head) attends, non-causally, the first n_window rows of the GPU
 * window plus K selected rows of the big store:
 *   queries   bf16 [bs,1,Hq,128] contiguous
 *   window_k/window_v bf16 [bs,H,cap_w,128] device, last stride 1, row stride 128
 *   store_k/store_v   bf16 [bs,H,cap_s,128], last stride 1, other strides equal for both and multiples of 8
 *                     elements (e.g. the two halves of one [bs,H,cap_s,2,128] buffer, which puts the K and V row
 *                     of a key in the same page); pinned HOST (UVA) or device
 *   selected  i64 [bs,H,K] (device) or NULL with K = 0;  row = selected + index_offset
 *   n_window_dev i32 [1] device, or NULL.  When given, the number of window rows is read on the device as
 *             min(n_window, n_window_dev[0] + n_window_add) and n_window only sizes the grid, so a captured
 *             CUDA graph can be replayed while the window fills.
 *   n_sel     i32 [bs,H] per-head count of valid entries of selected, or NULL (all K)
 *   out       bf16 [bs,1,Hq,128]
 *   lse       f32 [bs,Hq] or NULL: log2 of the softmax denominator of every query head (scores scaled and in
 *             the log2 domain, -inf for an empty row set); lets partial results over disjoint row sets be
 *             merged exactly: out = sum_r out_r * 2^(lse_r - LSE), LSE = log2 sum_r 2^lse_r
 *   workspace >= pk_attention_workspace_bytes(bs,Hq,n_window+K) bytes, device, 16-byte aligned.  Its first
 *             256-byte-rounded header (arrival counters and a status word) must be ZERO before the first
 *             call; every call leaves it zero again.  The status word (int at index bs*Hq) becomes 1 if a
 *             block gave up waiting for its copies (the output of that head is then not written). */
int64_t pk_attention_workspace_bytes(int64_t bs, int64_t Hq, int64_t max_rows);
int pk_sparse_attention(const pk_tensor* queries, const pk_tensor* window_k, const pk_tensor* window_v,
                        int64_t n_window, const pk_tensor* n_window_dev, int64_t n_window_add,
                        const pk_tensor* store_k, const pk_tensor* store_v,
                        const pk_tensor* selected, const pk_tensor* n_sel, int64_t index_offset,
                        float scale, const pk_tensor* out, const pk_tensor* lse, void* workspace,
                        int64_t workspace_bytes, void* stream);

/* Append one decode step's K/V row to the GPU window: the row writes of polar_cache.decode_update_kv_cache
 * (cache_hub/polar_cache.py:849-850) as one launch.
 *   k_row/v_row bf16 [bs,1,H,128]; window_k/window_v bf16 [bs,H,cap,128] (same strides)
 *   the row index is pos, or pos_dev[0] + pos_add when pos_dev (i32 [1], device) is given; a row index
 *   outside [0, cap) read from the device is ignored. */
int pk_append_kv(const pk_tensor* k_row, const pk_tensor* v_row, const pk_tensor* window_k,
                 const pk_tensor* window_v, int64_t pos, const pk_tensor* pos_dev, int64_t pos_add, void* stream);

/* One decode token into the cache, with the key coded once, when it is appended, and the flush of a full update
 * buffer inside the same launch: the row writes of polar_cache.decode_update_kv_cache (cache_hub/polar_cache.py:827-881)
 * and the index update of _update_polar_index (:743-821, which codes a whole buffer at flush time, for all layers,
 * and then blocks on the copy stream).  All positions live in `state` (int32, device):
 *   state[0] rows in the window   state[1] arrival counter (zero)   state[2] flushes so far   state[3] error flag
 *   state[4 + b] searchable keys of sample b
 * so the launch arguments never change and a captured CUDA graph stays valid across flushes.
 *   k_row/v_row    bf16 [bs,1,H,128]
 *   window_k/_v    bf16 [bs,H,cap_w,128], cap_w = sink + local + interval; the row goes to window row state[0]
 *   win_codes u8 [bs,H,cap_w,16], win_weight bf16 [bs,H,cap_w,16], win_4bit u8 [bs,H,cap_w,16,4], win_vnorm f32
 *                  [bs,H,cap_w]: contiguous staging records of the window rows (codes, rerank weights, 4-bit codes, ||v||)
 *   codebook / block_weight / packed_4bit: the zone records in the reference's logical shapes, stored key-major
 *                  (as pk_encode_keys prefers); value_norm f32 [bs,H,cap_z] or NULL
 *   store_kv       bf16 [bs,H,cap_s,2,128]: K row and V row of a zone key next to each other, device or pinned host
 * When the appended row fills the window, rows [sink, sink + interval) are published: records -> zone records
 * [n, n + interval), codes -> cluster_counts, K/V rows -> store rows, remaining rows slide down, state[0] =
 * cap_w - interval, state[4 + b] += interval.  state[3] becomes 1 (and nothing is published) if the zone or the
 * store has no room, or if state[0] is outside the window. */
int pk_append_encode(const pk_tensor* k_row, const pk_tensor* v_row, const pk_tensor* signs,
                     const pk_tensor* window_k, const pk_tensor* window_v, const pk_tensor* win_codes,
                     const pk_tensor* win_weight, const pk_tensor* win_4bit, const pk_tensor* win_vnorm,
                     const pk_tensor* codebook, const pk_tensor* block_weight, const pk_tensor* packed_4bit,
                     const pk_tensor* value_norm, const pk_tensor* cluster_counts, const pk_tensor* store_kv,
                     const pk_tensor* state, int64_t sink, int64_t interval, void* stream);

/* ---- the whole retrieval chain in one call ------------------------------------------------------- */

/* queries -> final top-K key indices for one layer and one decode step: the body of
 * polar_cache.collision_based_topk_batch (cache_hub/polar_cache.py:1126-1162, :1207-1304), as TWO launches:
 * (1) query preparation + cluster ranking + tier table + collision count, (2) candidate selection + 4-bit rerank +
 * final top-K.
 *   codebook / key_block_weight / key_4bit: views of the N searchable keys (as pk_collision_fused /
 *   pk_rerank); cluster_key_counts i32 [bs,H,16,256]; tier_counts host array (1..8 thresholds);
 *   C candidates, K final; final_indices i64 [bs,H,K] ascending key index.  K = 0 stops after the rerank
 *   (final_indices may be NULL): the adaptive-k variants rank the C candidates themselves.
 *   Optional outputs (NULL to skip): cand i64 [bs,H,C], scores_f32 f32 [bs,H,C],
 *   q_blocks bf16 [bs,H,16,8], q_norm bf16 [bs,H,1], query_avg bf16 [bs,H,128].
 *   workspace: pk_retrieve_workspace_bytes(bs,H,N,C) bytes, device, 256-byte aligned; nothing in it has to be
 *   cleared by the caller and nothing in it carries over between calls. */
int64_t pk_retrieve_workspace_bytes(int64_t bs, int64_t H, int64_t N, int64_t C);
int pk_retrieve(const pk_tensor* queries, const pk_tensor* signs, const pk_tensor* mag_centers,
                const pk_tensor* codebook, const pk_tensor* key_block_weight, const pk_tensor* key_4bit,
                const pk_tensor* cluster_key_counts, const int64_t* tier_counts, int n_tiers, int64_t C,
                int64_t K, const pk_tensor* final_indices, const pk_tensor* cand,
                const pk_tensor* scores_f32, const pk_tensor* q_blocks, const pk_tensor* q_norm,
                const pk_tensor* query_avg, void* workspace, int64_t workspace_bytes, void* stream);

/* How the tier thresholds and the candidate count follow from the zone length N: the ratio schedule of
 * polar_cache._get_adaptive_ratios (cache_hub/polar_cache.py:1113-1124) with the arithmetic of :1221-1222 and
 * :1239-1240.  Row i applies when N < bound[i] (bounds ascending), the last row otherwise:
 *   tier t  = ceil(N * collision_ratio[row] * tier_ratio[t])     (IEEE double, left to right, as Python computes it)
 *   C       = max(1, ceil(N * candidate_ratio[row])) */
typedef struct pk_zone_schedule {
  int32_t n_rows;   /* 1..4 */
  int32_t n_tiers;  /* 1..8 */
  int64_t bound[3];
  double candidate_ratio[4];
  double collision_ratio[4];
  double tier_ratio[8];
} pk_zone_schedule;

/* The same chain with the options that the reference, a single-sequence single-GPU cache, does not have.  Fields
 * left zero / NULL give exactly pk_retrieve.
 *   kv_len + schedule   per-sample zone lengths read ON THE DEVICE: sample b searches the first kv_len[b] keys of
 *                       the views (1 <= kv_len[b] <= N; values outside are clamped) with thresholds and candidate
 *                       count from `schedule`; tier_counts is ignored, C is the row stride of cand / scores_f32
 *                       and must be >= pk_zone_max_candidates(schedule, N), K an upper bound: sample b gets
 *                       min(K, its candidates) final indices, reported in n_sel.  One captured launch sequence
 *                       then serves a zone that grows, and a batch of sequences of different lengths
 *                       (the reference asserts equal lengths: cache_hub/polar_cache.py:396-403).
 *   phase / shard_hist  exact selection when the zone is cut into contiguous shards, one per rank: phase 1 runs
 *                       launch (1) and writes local_hist u32 [bs,H,256] (how many local keys have each count);
 *                       the caller all-gathers these rank-major into shard_hist [world,bs,H,256]; phase 2 runs
 *                       launch (2): the threshold count and the tie quota are taken from the SUM of the shards'
 *                       histograms, ties go to the shards in rank order, so the union of the shards' candidate
 *                       lists is exactly the single-GPU candidate set.  C is then the GLOBAL candidate count
 *                       and the row stride; n_cand reports the local count.  tier_counts must come from the
 *                       global zone length.  phase 0 = both launches, no sharding.
 *   n_sel  i32 [bs,H]   valid entries of final_indices;  n_cand i32 [bs,H]  valid entries of cand / scores_f32 */
typedef struct pk_retrieve_args {
  const pk_tensor* queries;
  const pk_tensor* signs;
  const pk_tensor* mag_centers;
  const pk_tensor* codebook;
  const pk_tensor* key_block_weight;
  const pk_tensor* key_4bit;
  const pk_tensor* cluster_key_counts;
  const int64_t* tier_counts;
  int32_t n_tiers;
  int32_t phase;
  int64_t C;
  int64_t K;
  const pk_tensor* kv_len;
  const pk_zone_schedule* schedule;
  const pk_tensor* local_hist;
  const pk_tensor* shard_hist;
  int32_t world;
  int32_t rank;
  const pk_tensor* final_indices;
  const pk_tensor* n_sel;
  const pk_tensor* cand;
  const pk_tensor* n_cand;
  const pk_tensor* scores_f32;
  const pk_tensor* q_blocks;
  const pk_tensor* q_norm;
  const pk_tensor* query_avg;
  void* workspace;
  int64_t workspace_bytes;
  int32_t queries_settled; /* nonzero: `queries` were complete before the kernel launched just before this call STARTED
                              (another launch, e.g. pk_append_encode, sits between their producer and this call).  With
                              pk_set_pdl(1) the collision kernel then prepares the query and ranks the clusters before it
                              waits for that kernel.  Zero is always safe. */
  int32_t reserved;
} pk_retrieve_args;
int pk_retrieve_ex(const pk_retrieve_args* args, void* stream);
/* Largest candidate count the schedule gives for any zone length in 1..N. */
int64_t pk_zone_max_candidates(const pk_zone_schedule* schedule, int64_t N);

/* ---- sequence-sharded form: the glue on either side of the two all-gathers ------------------------- */

/* The reference has no multi-GPU retrieval; its single-GPU selection (cache_hub/polar_cache.py:1207-1304) and
 * attention (attn_hub/polar_attn.py:17-113) are what the sharded form must reproduce.  Every rank holds one
 * contiguous chunk [start, end) of the zone, runs pk_retrieve over it (local indices), and then:
 *   pk_shard_pack_topk     cand i64 [bs,H,C] ascending, scores f32 [bs,H,C], local_final i64 [bs,H,Kl] (a subset
 *                          of cand) -> packed i64 [bs,H,Kl,2] = (fp32 score bits, global index = local + start);
 *                          n_cand / n_sel (i32 [bs,H], or NULL = all) give the valid entries of the cand / local_final
 *                          rows (the outputs of pk_retrieve_ex phase 2); entries past n_sel become (-inf, -1) and
 *                          never win the merge; the host all-gathers `packed` rank-major into [world,bs,H,Kl,2];
 *   pk_shard_unpack_topk   gathered -> scores f32 / indices i64 [bs,H,world*Kl], rank-major per row (ascending
 *                          global index, because the chunks are ascending), ready for pk_final_topk;
 *   pk_shard_owned_rows    final i64 [bs,H,K] ascending global -> local i64 [bs,H,K] (the rows inside
 *                          [start,end) first, minus start; the rest 0) and n_owned i32 [bs,H] (pk_sparse_attention's
 *                          selected / n_sel);
 *   pk_shard_pack_partial  out bf16 [bs,1,Hq,128], lse f32 [bs,Hq] -> packed f32 [bs,Hq,129]; all-gathered into
 *                          [world,bs,Hq,129];
 *   pk_shard_merge_partial gathered -> out bf16 [bs,1,Hq,128]: sum_r 2^(lse_r - max) out_r / sum_r 2^(lse_r - max),
 *                          ranks with lse = -inf (no rows) skipped. */
int pk_shard_pack_topk(const pk_tensor* cand, const pk_tensor* scores, const pk_tensor* local_final, int64_t start,
                       const pk_tensor* n_sel, const pk_tensor* n_cand, const pk_tensor* packed, void* stream);
int pk_shard_unpack_topk(const pk_tensor* gathered, const pk_tensor* scores, const pk_tensor* indices, void* stream);
int pk_shard_owned_rows(const pk_tensor* final_indices, int64_t start, int64_t end, const pk_tensor* local,
                        const pk_tensor* n_owned, void* stream);
int pk_shard_pack_partial(const pk_tensor* out, const pk_tensor* lse, const pk_tensor* packed, void* stream);
int pk_shard_merge_partial(const pk_tensor* gathered, const pk_tensor* out, void* stream);

/* The same two exchanges over peer memory instead of a collective.  Every rank owns one buffer with the same layout,
 * mapped into every peer's address space (peer_bases[r] = address of rank r's buffer as seen from THIS process):
 * at gather_offset the gather area of the exchange ([world][bs*H][Kl][2] i64, or [world][bs*Hq][129] f32), at
 * flags_offset `world` u32 flag words, zero before the first use.  `control` points to 16 bytes of LOCAL device
 * memory per exchange (exchange number, arrival counter, status, pad), zero before the first use.
 *   pk_shard_exchange_*  computes this rank's rows (as pk_shard_pack_*), stores them into slot `rank` of every
 *                        peer's gather area and then publishes the exchange number in word `rank` of every
 *                        peer's flags;
 *   pk_shard_collect_*   (launched after the matching exchange on the same stream) waits until all `world` local
 *                        flag words carry the current exchange number and then does the work of
 *                        pk_shard_unpack_topk / pk_shard_merge_partial on the local gather area.
 * The wait is bounded (about a second); on expiry control[2] is set to 1, the kernel continues on whatever the
 * buffer holds, and the caller must treat the results as invalid.  Ranks must issue the exchanges in the same
 * order; the two exchanges of a layer use different areas, flags and control blocks.  At most 16 ranks.
 * No counterpart in the reference. */
int pk_shard_exchange_topk(const pk_tensor* cand, const pk_tensor* scores, const pk_tensor* local_final, int64_t start,
                           const pk_tensor* n_sel, const pk_tensor* n_cand,
                           const uint64_t* peer_bases, int world, int rank, int64_t gather_offset,
                           int64_t flags_offset, void* control, void* stream);
int pk_shard_collect_topk(uint64_t local_base, int64_t gather_offset, int64_t flags_offset, void* control, int world,
                          int64_t Kl, const pk_tensor* scores, const pk_tensor* indices, void* stream);
int pk_shard_exchange_partial(const pk_tensor* out, const pk_tensor* lse, const uint64_t* peer_bases, int world,
                              int rank, int64_t gather_offset, int64_t flags_offset, void* control, void* stream);
int pk_shard_collect_partial(uint64_t local_base, int64_t gather_offset, int64_t flags_offset, void* control, int world,
                             const pk_tensor* out, void* stream);

/* ---- KV-head-sharded (tensor-parallel) form ------------------------------------------------------------ */

/* With the KV heads split over ranks every stage of the retrieval path is independent per rank: a rank builds its
 * cache with H / world heads (the reference puts the whole cache on one device, cache_hub/polar_cache.py:171) and no
 * collective touches the path.  What a tensor-parallel model adds around it is the reduction of its row-parallel
 * projections; at decode time that is one short vector, and this entry point does it in ONE launch over peer memory:
 *   out = residual + sum over ranks of partial          (bf16 [1,n] each, fp32 accumulation in rank order, so the
 *                                                        result is bit-identical on every rank)
 * Every 32-bit data word travels with the exchange number in one 8-byte store into the receiver's gather area, so a
 * slot that shows the expected number carries its data: no separate flag words, one NVLink store latency per exchange.
 * Layout of every rank's symmetric buffer (peer_bases[r] as seen from this process): two gather areas of area_bytes
 * (>= world * n * 4: world x n/2 eight-byte slots) each, one after the other from gather_offset, used alternately,
 * ZERO before the first use (flags_offset is kept in the signature and ignored); `control` = 16 bytes of LOCAL device
 * memory (exchange number, unused, status, pad), zero before the first use.  n <= 8192.  All ranks must issue the same
 * sequence of exchanges.  The wait is bounded (about a second); on expiry control[2] becomes 1 and the result is
 * invalid.  One rank per GPU.
 * No counterpart in the reference. */
int pk_tp_allreduce(const pk_tensor* partial, const pk_tensor* residual, const pk_tensor* out,
                    const uint64_t* peer_bases, int world, int rank, int64_t gather_offset, int64_t area_bytes,
                    int64_t flags_offset, void* control, const pk_tensor* norm_weight, const pk_tensor* normed_out,
                    double eps, void* stream);

/* The all-gather on the same buffers, flags and control block (it counts as one exchange in the common sequence):
 * out bf16 [1, world*n] = the ranks' part bf16 [1,n] in rank order.  A model whose dense layers are tensor-parallel
 * while its cache is sharded along the sequence gathers the q/k/v rows of all heads with it. */
int pk_tp_allgather(const pk_tensor* part, const pk_tensor* out, const uint64_t* peer_bases, int world, int rank,
                    int64_t gather_offset, int64_t area_bytes, int64_t flags_offset, void* control, void* stream);

/* ---- decode glue: the elementwise steps of a decoder layer around the cache calls ----------------------- */

/* One launch each, bf16, one token per sequence.  The reference takes these from its attention library
 * (model_hub/qwen.py:381 silu_and_mul, :405 / :429 rmsnorm, :482 rotary embedding); they are part of this library
 * because a decode step is launch-latency bound outside the host-link fetch.
 *
 * pk_qk_norm_rope: per-head RMS-norm (weight bf16 [heads,128], heads = q heads followed by KV heads) of the first
 *   heads*128 columns of the fused q/k/v row qkv bf16 [B, >= heads*128] (unit inner stride), then rotate-half RoPE
 *   with cos / sin bf16 [1 or B,128] (sin carries the sign: [-sin, sin]):  y = bf16(x * rstd * w),
 *   out[b,h,d] = bf16(y[d] * cos[d] + y[d xor 64] * sin[d]);  out bf16 [B,heads,128].
 * pk_add_rmsnorm: h_out = bf16(a + residual) (residual may be NULL), x_out = bf16(h_out * rstd(h_out) * weight);
 *   a, residual, h_out, x_out bf16 [B,n], weight bf16 [n], n a multiple of 8.  h_out may alias residual or a.
 * pk_silu_mul: out[b,i] = bf16( bf16(silu(gate_up[b,i])) * gate_up[b,F+i] );  gate_up bf16 [B,2F], out bf16 [B,F].
 * pk_tp_allreduce with normed_out != NULL additionally writes normed_out = RMS-norm(out) * norm_weight (bf16 [n];
 *   one row), so that a tensor-parallel layer needs no separate norm launch after a reduction. */
int pk_qk_norm_rope(const pk_tensor* qkv, const pk_tensor* weight, const pk_tensor* cos, const pk_tensor* sin,
                    const pk_tensor* out, double eps, void* stream);
int pk_add_rmsnorm(const pk_tensor* a, const pk_tensor* residual, const pk_tensor* weight, const pk_tensor* h_out,
                   const pk_tensor* x_out, double eps, void* stream);
int pk_silu_mul(const pk_tensor* gate_up, const pk_tensor* out, void* stream);
/* pk_gemv: out[1,O] = x[1,I] * weight[O,I]^T (bf16, fp32 accumulation), one token; HBM-bound streaming kernel, two rows
 *   per warp.  gated != 0: weight is a stacked [gate; up] matrix of O = 2F rows and out[1,F] = silu(gate x) * (up x),
 *   rounded like pk_silu_mul after a separate product.  I a multiple of 8, at most 24576. */
int pk_gemv(const pk_tensor* weight, const pk_tensor* x, const pk_tensor* out, int gated, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* PARISKV_B200_H */

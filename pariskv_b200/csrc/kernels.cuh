// Launchers shared between translation units of the pariskv_b200 library (host side only).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/pariskv_b200.h"

namespace pk {

// encode.cu
int launch_query_prep(const uint16_t* queries, int bs, int Hq, int H, const uint16_t* signs,
                      uint16_t* q_blocks, uint16_t* q_norm, uint16_t* query_avg, cudaStream_t st);

// ---- zone plan: tier thresholds and candidate count as functions of the zone length ------------------------------
// Same arithmetic on the host and on the device (IEEE double products, left to right, then ceil), which is what the
// reference's Python computes: int(math.ceil(N * collision_ratio * r)) and max(1, ceil(N * candidate_ratio))
// (cache_hub/polar_cache.py:1221-1222, :1239-1240) with the ratios picked by zone length (:1113-1124).
__host__ __device__ inline int zone_row(const pk_zone_schedule& s, long long N) {
  int row = s.n_rows - 1;
  for (int i = s.n_rows - 2; i >= 0; i--)
    if (N < s.bound[i]) row = i;
  return row;
}
__host__ __device__ inline void zone_tiers(const pk_zone_schedule& s, long long N, unsigned* tiers) {
  const double base = (double)N * s.collision_ratio[zone_row(s, N)];
  for (int t = 0; t < s.n_tiers; t++) {
    double x = ceil(base * s.tier_ratio[t]);
    if (!(x > 0.0)) x = 0.0;
    if (x > 4294967295.0) x = 4294967295.0;
    tiers[t] = (unsigned)x;
  }
}
__host__ __device__ inline long long zone_candidates(const pk_zone_schedule& s, long long N) {
  const double x = ceil((double)N * s.candidate_ratio[zone_row(s, N)]);
  const long long c = (long long)x;
  return c < 1 ? 1 : (c > N ? N : c);
}

// collision.cu
int64_t collision_chunk_keys(int64_t bs_h, int64_t Nv);
// queries != null: query preparation is done inside (q_blocks / q_norm / query_avg become outputs)
int launch_rank(const uint16_t* queries, const uint16_t* signs, int Hq, int H, uint16_t* q_blocks, uint16_t* q_norm,
                uint16_t* query_avg, const int32_t* counts, const int64_t* tier_counts, int n_tiers, int64_t bs_h,
                uint32_t* lut, int64_t* sorted_ids, cudaStream_t st);

// The query side of the fused chain: the collision kernel prepares the query, ranks the clusters of every subspace
// and builds the tier table itself, in every block, while its first code loads are in flight.
struct ChainQuery {
  const uint16_t* queries;    // [bs][Hq][128]
  const uint16_t* signs;      // [128]
  int Hq;
  uint16_t* q_blocks;         // [bs*H][128]  written by the first block of every (batch, head)
  uint16_t* q_norm;           // [bs*H]
  uint16_t* query_avg;        // [bs*H][128] or null
  const int32_t* counts;      // [bs*H][16][256] cluster histogram
  unsigned tiers[8];          // thresholds when n_dev == null
  int n_tiers;
  const int32_t* n_dev;       // [bs] searchable keys per sample (device), or null: all N keys of the view
  pk_zone_schedule sched;     // thresholds = zone_tiers(sched, n_dev[b]) when n_dev is set
  long long n_plan;           // > 0: thresholds from this zone length instead (a shard of a longer zone)
  unsigned* zero_words;       // [bs*H] words set to zero here (arrival counters of the selection kernel), or null
  int early_query;            // the queries were complete before the previous kernel on the stream started
  unsigned* zero_area;        // [bs*H][zero_area_words] set to zero here (the selection kernel's value histogram), or null
  int zero_area_words;
};
int launch_collision(const pk_tensor* codebook, const uint32_t* lut, int32_t* out_i32, cudaStream_t st);
int chain_layout(const pk_tensor* codebook, int* layout);
void chain_geometry(int64_t bs_h, int64_t Nv, int64_t* chunk_keys, int64_t* hist_keys, int64_t* n_hist);
int launch_chain_collision(const pk_tensor* codebook, const ChainQuery& cq, uint8_t* counts_u8, int64_t u8_stride,
                           uint32_t* chunk_hist, int* mis_out, int64_t* hist_keys_out, int64_t* n_hist_out,
                           cudaStream_t st);
// local_hist[bh][bin] = sum over chunks of chunk_hist[bh][chunk][bin]
int launch_hist_reduce(const uint32_t* chunk_hist, int64_t bs_h, int64_t n_chunks, int64_t chunk_keys, int mis, int H,
                       int64_t N, const int32_t* n_dev, uint32_t* local_hist, cudaStream_t st);

// topk.cu: exact top-k of rows of 32-bit values; out[row][i] = map ? map[row*map_stride + pos] : pos
// With `scratch` (topk_scratch_bytes(rows, L, k) bytes, 256-byte aligned; 0 = not needed) rows longer than 16384
// elements are selected in two passes of the one-CTA kernel instead of the cluster kernel.
int64_t topk_scratch_bytes(int64_t rows, int64_t L, int64_t k);
int launch_topk(const void* in, bool is_float, int64_t rows, int64_t row_stride, int64_t L, int64_t k,
                int64_t* out, const int64_t* map, int64_t map_stride, int order, cudaStream_t st, int stage,
                void* scratch = nullptr, int64_t scratch_bytes = 0);

// rerank.cu
struct RerankArgs {
  const int64_t* cand;   // [bs*H][C] or nullptr when candidates come from a per-block list
  const uint8_t* k4;     // element (b,h,s,k,i) at k4[b*k4_b + h*k4_h + s*k4_s + k*k4_l + i]
  int64_t k4_b, k4_h, k4_s, k4_l;
  const uint16_t* w;     // element (b,h,s,k) at w[b*w_b + h*w_h + s*w_s + k*w_l]
  int64_t w_b, w_h, w_s, w_l;
  const uint16_t* q_blocks;  // [bs*H][128]
  const uint16_t* q_norm;    // [bs*H]
  const uint16_t* centers;   // [8]
  int H;
  int64_t C;
};
int fill_rerank_args(RerankArgs* a, const pk_tensor* key_4bit, const pk_tensor* key_block_weight);
int launch_rerank(const RerankArgs& a, int64_t bs_h, uint16_t* scores_bf16, float* scores_f32, uint16_t* v4b,
                  cudaStream_t st);

// Candidate selection from u8 counts + per-block histograms, the rerank of the selected keys and the final top-K
// (by the block that finishes last for a (batch, head)) in one kernel.
struct SelectArgs {
  const uint8_t* counts_u8;      // [bs*H][u8_stride] virtual keys
  int64_t u8_stride;
  const uint32_t* chunk_hist;    // [bs*H][n_chunks][256]
  int64_t n_chunks, chunk_keys;
  int mis;
  int64_t N;                     // keys per head of the view (upper bound when n_dev is set)
  int64_t C;                     // row stride (and capacity) of cand_out / scores_f32
  int64_t C_want;                // candidates wanted per head over the whole zone, all shards together (n_dev == null)
  int64_t K;                     // final top-K; 0 = stop after the rerank
  int fill_tail;                 // rows may be longer than the candidate list: the tail gets (score -inf, key 0)
  unsigned* val_hist;            // [bs*H][select_value_bins()] zero at launch, or null: histogram of the scores' top
                                 // key bits, filled while the scores are computed; long rows select their top-K from it
  const int32_t* n_dev;          // [bs] searchable keys per sample, or null
  pk_zone_schedule sched;        // candidates = zone_candidates(sched, n_dev[b]) when n_dev is set
  const uint32_t* shard_hist;    // [world][bs*H][256] histograms of every shard (exact sequence-sharded selection)
  int world, rank;
  int64_t* cand_out;             // [bs*H][C]
  float* scores_f32;             // [bs*H][C]
  int64_t* final_out;            // [bs*H][K] ascending key index (K > 0)
  int32_t* n_sel_out;            // [bs*H] or null: entries of final_out that are valid = min(K, candidates)
  int32_t* n_cand_out;           // [bs*H] or null: candidates of this (batch, head)
  unsigned* counters;            // [bs*H] arrival counters, zero at launch (K > 0)
};
int64_t select_smem_bytes(int64_t chunk_keys, int64_t C, int64_t K);
int64_t select_value_bins();     // words per (batch, head) of SelectArgs::val_hist
int64_t select_final_max_row();  // longest score row whose final top-K the selection kernel finishes entirely in shared memory
int launch_select_rerank(const RerankArgs& a, int64_t bs_h, const SelectArgs& s, cudaStream_t st);

}  // namespace pk

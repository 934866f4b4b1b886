// Launchers shared between translation units of the pariskv_b200 library (host side only).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/pariskv_b200.h"

namespace pk {

// encode.cu
int launch_query_prep(const uint16_t* queries, int bs, int Hq, int H, const uint16_t* signs,
                      uint16_t* q_blocks, uint16_t* q_norm, uint16_t* query_avg, cudaStream_t st);

// collision.cu
int64_t collision_chunk_keys(int64_t bs_h, int64_t Nv);
// queries != null: query preparation is done inside (q_blocks / q_norm / query_avg become outputs)
int launch_rank(const uint16_t* queries, const uint16_t* signs, int Hq, int H, uint16_t* q_blocks, uint16_t* q_norm,
                uint16_t* query_avg, const int32_t* counts, const int64_t* tier_counts, int n_tiers, int64_t bs_h,
                uint32_t* lut, int64_t* sorted_ids, cudaStream_t st);
int launch_collision(const pk_tensor* codebook, const uint32_t* lut, int32_t* out_i32, uint8_t* counts_u8,
                     int64_t u8_stride, uint32_t* chunk_hist, int* mis_out, int64_t* chunk_keys_out,
                     int64_t* n_chunks_out, cudaStream_t st);

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
// select candidates from u8 counts + per-block histograms and rerank them in the same kernel
int launch_select_rerank(const RerankArgs& a, int64_t bs_h, const uint8_t* counts_u8, int64_t u8_stride,
                         const uint32_t* chunk_hist, int64_t n_chunks, int64_t chunk_keys, int mis, int64_t N,
                         int64_t* cand_out, float* scores_f32, cudaStream_t st);

}  // namespace pk

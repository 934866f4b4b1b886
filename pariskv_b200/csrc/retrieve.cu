// The whole retrieval chain of one decode step as one host call and four launches:
// query prep + cluster ranking + tier table (one kernel) -> collision count (u8 + per-block histograms) ->
// candidate selection fused with the 4-bit rerank -> final top-K.  All scratch comes from the caller.
#include "common.cuh"
#include "kernels.cuh"

using namespace pk;

namespace {
inline int64_t align256(int64_t x) { return (x + 255) / 256 * 256; }

struct RetrieveLayout {
  int64_t q_blocks, q_norm, lut, counts, hist, scores, cand, topk, topk_bytes, total;
  int64_t u8_stride, n_chunks_max;
};

RetrieveLayout make_layout(int64_t bs, int64_t H, int64_t N, int64_t C) {
  RetrieveLayout l;
  const int64_t bh = bs * H;
  l.u8_stride = (N + 15 + 15) / 16 * 16 + 16;
  const int64_t chunk = collision_chunk_keys(bh, N + 15);
  l.n_chunks_max = (N + 15 + chunk - 1) / chunk + 1;
  int64_t off = 0;
  l.q_blocks = off, off += align256(bh * 128 * 2);
  l.q_norm = off, off += align256(bh * 2);
  l.lut = off, off += align256(bh * 16 * 64 * 4);
  l.counts = off, off += align256(bh * l.u8_stride);
  l.hist = off, off += align256(bh * l.n_chunks_max * 256 * 4);
  l.scores = off, off += align256(bh * C * 4);
  l.cand = off, off += align256(bh * C * 8);
  l.topk_bytes = topk_scratch_bytes(bh, C, 2048);   // sized for any K up to 8192 (the size does not depend on K)
  l.topk = off, off += align256(l.topk_bytes);
  l.total = off;
  return l;
}
}  // namespace

extern "C" int64_t pk_retrieve_workspace_bytes(int64_t bs, int64_t H, int64_t N, int64_t C) {
  return make_layout(bs, H, N, C).total;
}

extern "C" int pk_retrieve(const pk_tensor* queries, const pk_tensor* signs, const pk_tensor* mag_centers,
                           const pk_tensor* codebook, const pk_tensor* key_block_weight, const pk_tensor* key_4bit,
                           const pk_tensor* cluster_key_counts, const int64_t* tier_counts, int n_tiers, int64_t C,
                           int64_t K, const pk_tensor* final_indices, const pk_tensor* cand,
                           const pk_tensor* scores_f32, const pk_tensor* q_blocks, const pk_tensor* q_norm,
                           const pk_tensor* query_avg, void* workspace, int64_t workspace_bytes, void* stream) {
  PK_CHECK_TENSOR(queries, PK_BF16, 4);
  PK_CHECK_TENSOR(signs, PK_BF16, 1);
  PK_CHECK_TENSOR(mag_centers, PK_BF16, 1);
  PK_CHECK_TENSOR(codebook, PK_U8, 4);
  PK_CHECK_TENSOR(cluster_key_counts, PK_I32, 4);
  if (K > 0) PK_CHECK_TENSOR(final_indices, PK_I64, 3);
  const int64_t bs = codebook->shape[0], H = codebook->shape[1], N = codebook->shape[3], Hq = queries->shape[2];
  const int64_t bh = bs * H;
  PK_REQUIRE(codebook->shape[2] == 16, "the fused chain supports 16 subspaces of 8 dims");
  PK_REQUIRE(queries->shape[0] == bs && queries->shape[1] == 1 && queries->shape[3] == 128 && is_contig(queries) &&
                 Hq % H == 0,
             "queries must be contiguous [bs,1,Hq,128] with Hq a multiple of H");
  PK_REQUIRE(signs->shape[0] == 128 && signs->stride[0] == 1 && mag_centers->shape[0] == 8 && mag_centers->stride[0] == 1,
             "signs must be [128], mag_centers [8]");
  PK_REQUIRE((reinterpret_cast<uintptr_t>(queries->data) & 15) == 0 && (reinterpret_cast<uintptr_t>(signs->data) & 15) == 0,
             "queries and signs must be 16-byte aligned");
  PK_REQUIRE(is_contig(cluster_key_counts) && cluster_key_counts->shape[0] == bs && cluster_key_counts->shape[1] == H &&
                 cluster_key_counts->shape[2] == 16 && cluster_key_counts->shape[3] == 256,
             "cluster_key_counts must be contiguous [bs,H,16,256]");
  PK_REQUIRE(n_tiers >= 1 && n_tiers <= 8 && tier_counts, "n_tiers must be in 1..8");
  PK_REQUIRE(N >= 1 && N < (1ll << 31), "N out of range");
  PK_REQUIRE(C >= 1 && C <= N && K >= 0 && K <= C, "need 0 <= K <= C <= N (K=%lld C=%lld N=%lld)", (long long)K,
             (long long)C, (long long)N);
  if (K > 0)
    PK_REQUIRE(is_contig(final_indices) && final_indices->shape[0] == bs && final_indices->shape[1] == H &&
                   final_indices->shape[2] == K,
               "final_indices must be contiguous [bs,H,K]");
  RerankArgs ra;
  int rc = fill_rerank_args(&ra, key_4bit, key_block_weight);
  if (rc) return rc;
  PK_REQUIRE(key_4bit->shape[0] == bs && key_4bit->shape[1] == H && key_4bit->shape[3] == N,
             "key_4bit must cover the same N keys as codebook");
  const RetrieveLayout lay = make_layout(bs, H, N, C);
  if (!workspace || workspace_bytes < lay.total)
    return fail(PK_ERR_WORKSPACE, "retrieve workspace too small: %lld < %lld", (long long)workspace_bytes,
                (long long)lay.total);
  PK_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 255) == 0, "workspace must be 256-byte aligned");
  char* ws = (char*)workspace;
  uint16_t* qb = (uint16_t*)(ws + lay.q_blocks);
  uint16_t* qn = (uint16_t*)(ws + lay.q_norm);
  uint16_t* qa = nullptr;
  float* sc = (float*)(ws + lay.scores);
  int64_t* cd = (int64_t*)(ws + lay.cand);
  if (q_blocks) {
    PK_CHECK_TENSOR(q_blocks, PK_BF16, 4);
    PK_REQUIRE(is_contig(q_blocks) && numel(q_blocks) == bh * 128, "q_blocks must be contiguous [bs,H,16,8]");
    qb = (uint16_t*)q_blocks->data;
  }
  if (q_norm) {
    PK_CHECK_TENSOR(q_norm, PK_BF16, 3);
    PK_REQUIRE(is_contig(q_norm) && numel(q_norm) == bh, "q_norm must be contiguous [bs,H,1]");
    qn = (uint16_t*)q_norm->data;
  }
  if (query_avg) {
    PK_CHECK_TENSOR(query_avg, PK_BF16, 3);
    PK_REQUIRE(is_contig(query_avg) && numel(query_avg) == bh * 128, "query_avg must be contiguous [bs,H,128]");
    qa = (uint16_t*)query_avg->data;
  }
  if (scores_f32) {
    PK_CHECK_TENSOR(scores_f32, PK_F32, 3);
    PK_REQUIRE(is_contig(scores_f32) && numel(scores_f32) == bh * C, "scores_f32 must be contiguous [bs,H,C]");
    sc = (float*)scores_f32->data;
  }
  if (cand) {
    PK_CHECK_TENSOR(cand, PK_I64, 3);
    PK_REQUIRE(is_contig(cand) && numel(cand) == bh * C, "cand must be contiguous [bs,H,C]");
    cd = (int64_t*)cand->data;
  }
  cudaStream_t st = (cudaStream_t)stream;
  uint32_t* lut = (uint32_t*)(ws + lay.lut);
  if ((rc = launch_rank((const uint16_t*)queries->data, (const uint16_t*)signs->data, (int)Hq, (int)H, qb, qn, qa,
                        (const int32_t*)cluster_key_counts->data, tier_counts, n_tiers, bh, lut, nullptr, st)))
    return rc;
  int mis = 0;
  int64_t chunk_keys = 0, n_chunks = 0;
  uint8_t* counts = (uint8_t*)(ws + lay.counts);
  uint32_t* hist = (uint32_t*)(ws + lay.hist);
  if ((rc = launch_collision(codebook, lut, nullptr, counts, lay.u8_stride, hist, &mis, &chunk_keys, &n_chunks, st)))
    return rc;
  if (n_chunks > lay.n_chunks_max) return fail(PK_ERR_WORKSPACE, "internal: histogram workspace undersized");
  ra.cand = nullptr;
  ra.q_blocks = qb, ra.q_norm = qn, ra.centers = (const uint16_t*)mag_centers->data;
  ra.C = C;
  if ((rc = launch_select_rerank(ra, bh, counts, lay.u8_stride, hist, n_chunks, chunk_keys, mis, N, cd, sc, st)))
    return rc;
  if (K == 0) return PK_OK;  // the caller ranks the candidates itself (adaptive-k)
  return launch_topk(sc, true, bh, C, C, K, (int64_t*)final_indices->data, cd, C, 0, st, ST_FINAL_TOPK,
                     lay.topk_bytes ? ws + lay.topk : nullptr, lay.topk_bytes);
}

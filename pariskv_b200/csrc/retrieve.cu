// The whole retrieval chain of one decode step as one host call and two launches:
// (1) query preparation + cluster ranking + tier table + collision count (u8 counts + per-block histograms),
// (2) candidate selection + 4-bit rerank + final top-K by the last block of every (batch, head).
// All scratch comes from the caller.
#include "common.cuh"
#include "kernels.cuh"

using namespace pk;

namespace {
inline int64_t align256(int64_t x) { return (x + 255) / 256 * 256; }

struct RetrieveLayout {
  int64_t q_blocks, q_norm, counters, counts, hist, scores, cand, vhist, topk, topk_bytes, total;
  int64_t u8_stride, n_chunks_max;
};

RetrieveLayout make_layout(int64_t bs, int64_t H, int64_t N, int64_t C) {
  RetrieveLayout l;
  const int64_t bh = bs * H;
  l.u8_stride = (N + 15 + 15) / 16 * 16 + 16;
  // an upper bound on the blocks per (batch, head) that grows with N, so that scratch sized for a zone's capacity
  // serves every shorter zone: the launcher aims at one block per SM (two histogram rows each) and caps a block at
  // 32768 keys
  int64_t target = (int64_t)sm_count() / (bh > 0 ? bh : 1);
  if (target < 1) target = 1;
  const int64_t by_cap = (N + 15 + 32767) / 32768;
  l.n_chunks_max = (2 * target > by_cap ? 2 * target : by_cap) + 2;
  int64_t off = 0;
  l.q_blocks = off, off += align256(bh * 128 * 2);
  l.q_norm = off, off += align256(bh * 2);
  l.counters = off, off += align256(bh * 4);
  l.counts = off, off += align256(bh * l.u8_stride);
  l.hist = off, off += align256(bh * l.n_chunks_max * 256 * 4);
  l.scores = off, off += align256(bh * C * 4);
  l.cand = off, off += align256(bh * C * 8);
  // value histogram of the final selection: long rows only
  l.vhist = off, off += C > select_final_max_row() ? align256(bh * select_value_bins() * 4) : 0;
  l.topk_bytes = topk_scratch_bytes(bh, C, 2048);   // long rows only; the size does not depend on K
  l.topk = off, off += align256(l.topk_bytes);
  l.total = off;
  return l;
}

int check_schedule(const pk_zone_schedule* s) {
  PK_REQUIRE(s != nullptr, "kv_len needs a schedule");
  PK_REQUIRE(s->n_rows >= 1 && s->n_rows <= 4 && s->n_tiers >= 1 && s->n_tiers <= 8,
             "schedule: n_rows must be in 1..4 and n_tiers in 1..8");
  for (int i = 0; i + 2 < s->n_rows; i++) PK_REQUIRE(s->bound[i] < s->bound[i + 1], "schedule: bounds must ascend");
  for (int i = 0; i < s->n_rows; i++)
    PK_REQUIRE(s->candidate_ratio[i] > 0.0 && s->candidate_ratio[i] <= 1.0 && s->collision_ratio[i] >= 0.0,
               "schedule: candidate_ratio must be in (0,1], collision_ratio non-negative");
  return PK_OK;
}

int retrieve_impl(const pk_retrieve_args& a, cudaStream_t st) {
  PK_CHECK_TENSOR(a.queries, PK_BF16, 4);
  PK_CHECK_TENSOR(a.signs, PK_BF16, 1);
  PK_CHECK_TENSOR(a.mag_centers, PK_BF16, 1);
  PK_CHECK_TENSOR(a.codebook, PK_U8, 4);
  PK_CHECK_TENSOR(a.cluster_key_counts, PK_I32, 4);
  const int64_t K = a.K, C = a.C;
  PK_REQUIRE(a.phase >= 0 && a.phase <= 2, "phase must be 0, 1 or 2");
  if (K > 0 && a.phase != 1) PK_CHECK_TENSOR(a.final_indices, PK_I64, 3);
  const pk_tensor *queries = a.queries, *codebook = a.codebook, *counts_t = a.cluster_key_counts;
  const int64_t bs = codebook->shape[0], H = codebook->shape[1], N = codebook->shape[3], Hq = queries->shape[2];
  const int64_t bh = bs * H;
  PK_REQUIRE(codebook->shape[2] == 16, "the fused chain supports 16 subspaces of 8 dims");
  PK_REQUIRE(queries->shape[0] == bs && queries->shape[1] == 1 && queries->shape[3] == 128 && is_contig(queries) &&
                 H > 0 && Hq % H == 0,
             "queries must be contiguous [bs,1,Hq,128] with Hq a multiple of H");
  PK_REQUIRE(a.signs->shape[0] == 128 && a.signs->stride[0] == 1 && a.mag_centers->shape[0] == 8 &&
                 a.mag_centers->stride[0] == 1,
             "signs must be [128], mag_centers [8]");
  PK_REQUIRE((reinterpret_cast<uintptr_t>(queries->data) & 15) == 0 && (reinterpret_cast<uintptr_t>(a.signs->data) & 15) == 0,
             "queries and signs must be 16-byte aligned");
  PK_REQUIRE(is_contig(counts_t) && counts_t->shape[0] == bs && counts_t->shape[1] == H && counts_t->shape[2] == 16 &&
                 counts_t->shape[3] == 256 && (reinterpret_cast<uintptr_t>(counts_t->data) & 15) == 0,
             "cluster_key_counts must be contiguous, 16-byte aligned [bs,H,16,256]");
  PK_REQUIRE(N >= 1 && N < (1ll << 31), "N out of range");
  PK_REQUIRE(K >= 0 && C >= 1, "need K >= 0 and C >= 1");
  const bool sharded = a.phase != 0;
  const bool varlen = a.kv_len != nullptr;
  PK_REQUIRE(!(sharded && varlen), "per-sample zone lengths and sharded selection cannot be combined");
  if (!sharded && !varlen) PK_REQUIRE(C <= N && K <= C, "need K <= C <= N (K=%lld C=%lld N=%lld)", (long long)K, (long long)C, (long long)N);
  if (varlen) PK_REQUIRE(C <= N, "need C <= N (C=%lld N=%lld)", (long long)C, (long long)N);
  ChainQuery cq = {};
  SelectArgs sa = {};
  if (varlen) {
    PK_CHECK_TENSOR(a.kv_len, PK_I32, 1);
    PK_REQUIRE(a.kv_len->shape[0] == bs && a.kv_len->stride[0] == 1, "kv_len must be contiguous i32 [bs]");
    int rc = check_schedule(a.schedule);
    if (rc) return rc;
    PK_REQUIRE(C >= pk_zone_max_candidates(a.schedule, N) || C >= N,
               "C (%lld) is the row stride of the candidate lists and must cover the largest candidate count of the "
               "schedule (%lld)", (long long)C, (long long)pk_zone_max_candidates(a.schedule, N));
    cq.n_dev = sa.n_dev = (const int32_t*)a.kv_len->data;
    cq.sched = sa.sched = *a.schedule;
  } else {
    PK_REQUIRE(a.n_tiers >= 1 && a.n_tiers <= 8 && a.tier_counts, "n_tiers must be in 1..8");
    cq.n_tiers = a.n_tiers;
    for (int i = 0; i < a.n_tiers; i++) {
      const int64_t t = a.tier_counts[i];
      cq.tiers[i] = t < 0 ? 0u : (t > 0xffffffffll ? 0xffffffffu : (unsigned)t);
    }
  }
  if (K > 0 && a.phase != 1)
    PK_REQUIRE(is_contig(a.final_indices) && a.final_indices->shape[0] == bs && a.final_indices->shape[1] == H &&
                   a.final_indices->shape[2] == K,
               "final_indices must be contiguous [bs,H,K]");
  RerankArgs ra;
  int rc = fill_rerank_args(&ra, a.key_4bit, a.key_block_weight);
  if (rc) return rc;
  PK_REQUIRE(a.key_4bit->shape[0] == bs && a.key_4bit->shape[1] == H && a.key_4bit->shape[3] == N,
             "key_4bit must cover the same N keys as codebook");
  const int64_t Cw = C < N ? C : N;   // candidates of one shard never exceed its keys
  const RetrieveLayout lay = make_layout(bs, H, N, sharded ? Cw : C);
  if (!a.workspace || a.workspace_bytes < lay.total)
    return fail(PK_ERR_WORKSPACE, "retrieve workspace too small: %lld < %lld", (long long)a.workspace_bytes,
                (long long)lay.total);
  PK_REQUIRE((reinterpret_cast<uintptr_t>(a.workspace) & 255) == 0, "workspace must be 256-byte aligned");
  char* ws = (char*)a.workspace;
  uint16_t* qb = (uint16_t*)(ws + lay.q_blocks);
  uint16_t* qn = (uint16_t*)(ws + lay.q_norm);
  uint16_t* qa = nullptr;
  float* sc = (float*)(ws + lay.scores);
  int64_t* cd = (int64_t*)(ws + lay.cand);
  const int64_t row = sharded ? Cw : C;  // row stride of cand / scores
  if (a.q_blocks) {
    PK_CHECK_TENSOR(a.q_blocks, PK_BF16, 4);
    PK_REQUIRE(is_contig(a.q_blocks) && numel(a.q_blocks) == bh * 128 && (reinterpret_cast<uintptr_t>(a.q_blocks->data) & 7) == 0,
               "q_blocks must be contiguous, 8-byte aligned [bs,H,16,8]");
    qb = (uint16_t*)a.q_blocks->data;
  }
  if (a.q_norm) {
    PK_CHECK_TENSOR(a.q_norm, PK_BF16, 3);
    PK_REQUIRE(is_contig(a.q_norm) && numel(a.q_norm) == bh, "q_norm must be contiguous [bs,H,1]");
    qn = (uint16_t*)a.q_norm->data;
  }
  if (a.query_avg) {
    PK_CHECK_TENSOR(a.query_avg, PK_BF16, 3);
    PK_REQUIRE(is_contig(a.query_avg) && numel(a.query_avg) == bh * 128 && (reinterpret_cast<uintptr_t>(a.query_avg->data) & 7) == 0,
               "query_avg must be contiguous, 8-byte aligned [bs,H,128]");
    qa = (uint16_t*)a.query_avg->data;
  }
  if (a.scores_f32) {
    PK_CHECK_TENSOR(a.scores_f32, PK_F32, 3);
    PK_REQUIRE(is_contig(a.scores_f32) && numel(a.scores_f32) == bh * row, "scores_f32 must be contiguous [bs,H,%lld]",
               (long long)row);
    sc = (float*)a.scores_f32->data;
  }
  if (a.cand) {
    PK_CHECK_TENSOR(a.cand, PK_I64, 3);
    PK_REQUIRE(is_contig(a.cand) && numel(a.cand) == bh * row, "cand must be contiguous [bs,H,%lld]", (long long)row);
    cd = (int64_t*)a.cand->data;
  }
  int32_t *n_sel = nullptr, *n_cand = nullptr;
  if (a.n_sel) {
    PK_CHECK_TENSOR(a.n_sel, PK_I32, 2);
    PK_REQUIRE(is_contig(a.n_sel) && numel(a.n_sel) == bh, "n_sel must be contiguous i32 [bs,H]");
    n_sel = (int32_t*)a.n_sel->data;
  }
  if (a.n_cand) {
    PK_CHECK_TENSOR(a.n_cand, PK_I32, 2);
    PK_REQUIRE(is_contig(a.n_cand) && numel(a.n_cand) == bh, "n_cand must be contiguous i32 [bs,H]");
    n_cand = (int32_t*)a.n_cand->data;
  }
  uint8_t* counts = (uint8_t*)(ws + lay.counts);
  uint32_t* hist = (uint32_t*)(ws + lay.hist);
  unsigned* counters = (unsigned*)(ws + lay.counters);
  // the launch geometry is a function of the view alone, so phase 2 finds what phase 1 left in the workspace;
  // chunk_keys / n_chunks: keys per histogram row and rows per (batch, head), the selection kernel's grid
  int mis = 0;
  int64_t chunk_keys = 0, n_chunks = 0;
  if (a.phase != 2) {
    cq.queries = (const uint16_t*)queries->data, cq.signs = (const uint16_t*)a.signs->data, cq.Hq = (int)Hq;
    cq.q_blocks = qb, cq.q_norm = qn, cq.query_avg = qa;
    cq.counts = (const int32_t*)counts_t->data;
    cq.zero_words = counters;
    cq.early_query = a.queries_settled != 0;
    if (K > 0 && row > select_final_max_row() && (varlen || sharded || n_sel))
      cq.zero_area = (unsigned*)(ws + lay.vhist), cq.zero_area_words = (int)select_value_bins();
    if ((rc = launch_chain_collision(codebook, cq, counts, lay.u8_stride, hist, &mis, &chunk_keys, &n_chunks, st)))
      return rc;
    if (n_chunks > lay.n_chunks_max) return fail(PK_ERR_WORKSPACE, "internal: histogram workspace undersized");
    if (a.phase == 1) {
      PK_CHECK_TENSOR(a.local_hist, PK_I32, 3);
      PK_REQUIRE(is_contig(a.local_hist) && a.local_hist->shape[0] == bs && a.local_hist->shape[1] == H &&
                     a.local_hist->shape[2] == 256,
                 "local_hist must be contiguous i32 [bs,H,256]");
      return launch_hist_reduce(hist, bh, n_chunks, chunk_keys, mis, (int)H, N, nullptr, (uint32_t*)a.local_hist->data, st);
    }
  } else {
    int layout = 0;
    mis = chain_layout(codebook, &layout);
    int64_t block_keys = 0;
    chain_geometry(bh, N + mis, &block_keys, &chunk_keys, &n_chunks);
  }
  sa.counts_u8 = counts, sa.u8_stride = lay.u8_stride, sa.chunk_hist = hist;
  sa.n_chunks = n_chunks, sa.chunk_keys = chunk_keys, sa.mis = mis, sa.N = N;
  sa.C = row, sa.C_want = C, sa.K = K;
  if (a.phase == 2) {
    PK_CHECK_TENSOR(a.shard_hist, PK_I32, 4);
    PK_REQUIRE(a.world >= 1 && a.world <= 64 && a.rank >= 0 && a.rank < a.world, "rank / world out of range");
    PK_REQUIRE(is_contig(a.shard_hist) && a.shard_hist->shape[0] == a.world && a.shard_hist->shape[1] == bs &&
                   a.shard_hist->shape[2] == H && a.shard_hist->shape[3] == 256,
               "shard_hist must be contiguous i32 [world,bs,H,256]");
    sa.shard_hist = (const uint32_t*)a.shard_hist->data, sa.world = a.world, sa.rank = a.rank;
  }
  sa.cand_out = cd, sa.scores_f32 = sc;
  // Long score rows.  Full rows of a fixed length (no per-sample lengths, no shards): the final top-K runs as the
  // two-pass selection over many blocks after the selection kernel (measured faster at 100 K scores per row than one
  // block per head).  Rows whose length is only known on the device: every block of the selection kernel adds its
  // scores to a histogram of their top key bits, which the collision kernel cleared (phase 2 finds it cleared by
  // phase 1), and the last block of a (batch, head) selects from it - still one launch.
  sa.fill_tail = varlen;
  const bool long_rows = K > 0 && row > select_final_max_row();
  const bool separate_final = long_rows && !varlen && !sharded && !n_sel;
  sa.val_hist = long_rows && !separate_final ? (unsigned*)(ws + lay.vhist) : nullptr;
  if (separate_final) sa.K = 0;
  sa.final_out = K > 0 ? (int64_t*)a.final_indices->data : nullptr;
  sa.n_sel_out = n_sel, sa.n_cand_out = n_cand, sa.counters = counters;
  ra.cand = nullptr;
  ra.q_blocks = qb, ra.q_norm = qn, ra.centers = (const uint16_t*)a.mag_centers->data;
  ra.C = row;
  if ((rc = launch_select_rerank(ra, bh, sa, st)) || !separate_final) return rc;
  return launch_topk(sc, true, bh, row, row, K, (int64_t*)a.final_indices->data, cd, row, 0, st, ST_FINAL_TOPK,
                     lay.topk_bytes ? ws + lay.topk : nullptr, lay.topk_bytes);
}
}  // namespace

extern "C" int64_t pk_retrieve_workspace_bytes(int64_t bs, int64_t H, int64_t N, int64_t C) {
  return make_layout(bs, H, N, C < N ? C : N).total;
}

extern "C" int64_t pk_zone_max_candidates(const pk_zone_schedule* s, int64_t N) {
  if (!s || N < 1 || s->n_rows < 1 || s->n_rows > 4) return 0;
  // within a row the count grows with N: the maximum lies at the top end of a row
  int64_t best = zone_candidates(*s, N);
  for (int i = 0; i + 1 < s->n_rows; i++) {
    const int64_t n = s->bound[i] - 1;
    if (n >= 1 && n <= N) {
      const int64_t c = zone_candidates(*s, n);
      if (c > best) best = c;
    }
  }
  return best;
}

extern "C" int pk_retrieve(const pk_tensor* queries, const pk_tensor* signs, const pk_tensor* mag_centers,
                           const pk_tensor* codebook, const pk_tensor* key_block_weight, const pk_tensor* key_4bit,
                           const pk_tensor* cluster_key_counts, const int64_t* tier_counts, int n_tiers, int64_t C,
                           int64_t K, const pk_tensor* final_indices, const pk_tensor* cand,
                           const pk_tensor* scores_f32, const pk_tensor* q_blocks, const pk_tensor* q_norm,
                           const pk_tensor* query_avg, void* workspace, int64_t workspace_bytes, void* stream) {
  pk_retrieve_args a = {};
  a.queries = queries, a.signs = signs, a.mag_centers = mag_centers, a.codebook = codebook;
  a.key_block_weight = key_block_weight, a.key_4bit = key_4bit, a.cluster_key_counts = cluster_key_counts;
  a.tier_counts = tier_counts, a.n_tiers = n_tiers, a.C = C, a.K = K;
  a.final_indices = final_indices, a.cand = cand, a.scores_f32 = scores_f32;
  a.q_blocks = q_blocks, a.q_norm = q_norm, a.query_avg = query_avg;
  a.workspace = workspace, a.workspace_bytes = workspace_bytes;
  return retrieve_impl(a, (cudaStream_t)stream);
}

extern "C" int pk_retrieve_ex(const pk_retrieve_args* args, void* stream) {
  PK_REQUIRE(args != nullptr, "args is null");
  return retrieve_impl(*args, (cudaStream_t)stream);
}

/*
 * CPU oracle for the ParisKV retrieval path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C, the arithmetic of the reference's decode-time
 * retrieval path so that the CUDA kernels can be checked against it bit for bit.
 * It is never linked into, imported by, or called from the product path; only the
 * tests, the smoke check and the CPU-baseline leg of the benchmark load it.
 *
 * Each function cites the reference lines it follows (paths are relative to the
 * reference project root).  Where the reference leaves an order of floating-point
 * operations open (reduction order inside torch / cuBLAS / the Hadamard wheel,
 * unstable sorts, atomics-ordered outputs) this file PINS one order, stated beside
 * the code; the CUDA kernels implement the same order.
 *
 * Parity status.  Collision counts, candidate sets, rerank scores and adaptive-k are
 * pinned against the reference's own torch reference functions (golden fixtures are
 * generated from them).  The SRHT encode and the query preparation have no test in
 * the reference and call a third-party Hadamard wheel that is not available:
 * PARITY UNPINNED for those two steps beyond the literal torch restatement of the
 * same lines that the fixtures hold.
 *
 * All per-head arrays are KEY-MAJOR unless a stride is passed: codes[L][16],
 * weights[L][16] (bf16 bits), packed[L][16][4].
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define PK_D 128
#define PK_B 16
#define PK_M 8

/* ---- bf16 helpers (round to nearest even, as torch's float->bfloat16 cast) ---- */
static inline float bf2f(uint16_t h) {
  uint32_t u = ((uint32_t)h) << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}
static inline uint16_t f2bf(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40); /* NaN */
  uint32_t lsb = (u >> 16) & 1u;
  u += 0x7fffu + lsb;
  return (uint16_t)(u >> 16);
}
static inline float bfround(float f) { return bf2f(f2bf(f)); }

/* Magnitude thresholds / centers: the bf16 roundings of the literals at
 * cache_hub/polar_cache.py:188-193. */
static const float PK_THR[7] = {0.08447265625f, 0.169921875f, 0.2578125f, 0.349609375f,
                                0.44921875f,    0.55859375f,  0.69140625f};
static const float PK_CEN[8] = {0.0419921875f, 0.126953125f, 0.212890625f, 0.302734375f,
                                0.396484375f,  0.5f,         0.6171875f,   0.76171875f};

void pko_constants(float* thr7, float* cen8) {
  memcpy(thr7, PK_THR, sizeof(PK_THR));
  memcpy(cen8, PK_CEN, sizeof(PK_CEN));
}

/* Pinned reduction: adjacent pairwise tree over n (power of two) fp32 values. */
static float tree_sum(float* v, int n) {
  for (int w = n; w > 1; w >>= 1)
    for (int i = 0; i < w / 2; i++) v[i] = v[2 * i] + v[2 * i + 1];
  return v[0];
}

/* Pinned Walsh-Hadamard transform (Sylvester order): in-place butterflies for
 * h = 1, 2, 4, ..., 64; each output is one fp32 add or subtract. */
static void wht128(float* x) {
  for (int h = 1; h < PK_D; h <<= 1)
    for (int i = 0; i < PK_D; i++)
      if ((i & h) == 0) {
        float a = x[i], b = x[i + h];
        x[i] = a + b;
        x[i + h] = a - b;
      }
}

/* Normalise + sign flip + Hadamard + scale of one 128-vector given as bf16 bits.
 * Follows cache_hub/polar_cache.py:938-945 (keys) and :915-920 (queries):
 *   n  = bf16(sqrt(sum x^2))                 (fp32 pairwise tree, bf16 result)
 *   xn = bf16(x / max(n, bf16(1e-8)))        (fp32 divide, bf16 result)
 *   y  = bf16(WHT(xn * s) * 1/sqrt(128))     (fp32 butterflies, one bf16 rounding)
 * Returns n (as float holding a bf16 value); y holds bf16 values as floats. */
static float srht_rotate(const uint16_t* x, const uint16_t* signs, float* y) {
  float sq[PK_D], xv[PK_D];
  for (int i = 0; i < PK_D; i++) {
    xv[i] = bf2f(x[i]);
    sq[i] = xv[i] * xv[i];
  }
  float n = bfround(sqrtf(tree_sum(sq, PK_D)));
  float den = fmaxf(n, bfround(1e-8f));
  for (int i = 0; i < PK_D; i++) y[i] = bfround(xv[i] / den) * bf2f(signs[i]);
  wht128(y);
  for (int i = 0; i < PK_D; i++) y[i] = bfround(y[i] * 0.08838834764831845f);
  return n;
}

/* Key encode: cache_hub/polar_cache.py:924-978 and :887-893.
 * keys[L][128] bf16 bits -> codes[L][16] u8, weights[L][16] bf16 bits, packed[L][16][4]. */
void pko_encode(const uint16_t* keys, int64_t L, const uint16_t* signs, uint8_t* codes,
                uint16_t* weights, uint8_t* packed) {
#pragma omp parallel for schedule(static)
  for (int64_t k = 0; k < L; k++) {
    float y[PK_D];
    float n = srht_rotate(keys + k * PK_D, signs, y);
    for (int b = 0; b < PK_B; b++) {
      const float* yb = y + b * PK_M;
      float sq[PK_M];
      unsigned code = 0;
      for (int j = 0; j < PK_M; j++) {
        sq[j] = yb[j] * yb[j];
        if (yb[j] >= 0.0f) code |= 1u << j; /* :950-951, zero counts as positive */
      }
      float r = bfround(sqrtf(tree_sum(sq, PK_M))); /* :958 */
      float den = fmaxf(r, bfround(1e-8f));         /* :959 */
      float prod[PK_M];
      unsigned nib[PK_M];
      for (int j = 0; j < PK_M; j++) {
        float au = fabsf(bfround(yb[j] / den)); /* :960, :963 */
        unsigned t = 0;                          /* :965 bucketize, right=False */
        for (int i = 0; i < 7; i++) t += (PK_THR[i] < au);
        prod[j] = bfround(PK_CEN[t] * au); /* :967, :972 bf16 product */
        nib[j] = (((code >> j) & 1u) << 3) | t;
      }
      float alpha = fmaxf(tree_sum(prod, PK_M), 1e-6f);          /* :972-973 */
      weights[k * PK_B + b] = f2bf((r / alpha) * n);             /* :975-976 */
      codes[k * PK_B + b] = (uint8_t)code;
      for (int i = 0; i < 4; i++) /* :889-892: low nibble = even dim */
        packed[(k * PK_B + b) * 4 + i] = (uint8_t)((nib[2 * i + 1] << 4) | nib[2 * i]);
    }
  }
}

/* Per-subspace histogram of codes, added into counts[16][256]:
 * cache_hub/polar_cache.py:980-996, accumulated as at :600-601 and :774-775. */
void pko_cluster_counts(const uint8_t* codes, int64_t L, int32_t* counts) {
  for (int64_t k = 0; k < L; k++)
    for (int b = 0; b < PK_B; b++) counts[b * 256 + codes[k * PK_B + b]] += 1;
}

/* Query preparation: mean over the G query heads of a KV group
 * (cache_hub/polar_cache.py:1027-1031; fp32 sequential sum times 1/G, bf16 result),
 * then the same normalise-rotate as keys (:905-922).
 * q[G][128] -> q_blocks[128] (bf16 bits), q_norm (bf16 bits). */
void pko_query_prep(const uint16_t* q, int G, const uint16_t* signs, uint16_t* q_blocks,
                    uint16_t* q_norm) {
  uint16_t avg[PK_D];
  float inv = 1.0f / (float)G;
  for (int i = 0; i < PK_D; i++) {
    float s = 0.0f;
    for (int g = 0; g < G; g++) s += bf2f(q[g * PK_D + i]);
    avg[i] = f2bf(s * inv);
  }
  float y[PK_D];
  float n = srht_rotate(avg, signs, y);
  for (int i = 0; i < PK_D; i++) q_blocks[i] = f2bf(y[i]);
  *q_norm = f2bf(n);
}

/* Cluster ranking: cache_hub/polar_cache.py:1216-1217.  score_c = bf16(sum_j +-q_j)
 * with the sign pattern of cluster c (bit j set -> +), fp32 sum j ascending;
 * order = score descending, cluster id ascending on ties (the stable order). */
void pko_cluster_rank(const uint16_t* q_blocks, int64_t* sorted_ids) {
  for (int b = 0; b < PK_B; b++) {
    float sc[256];
    for (int c = 0; c < 256; c++) {
      float s = 0.0f;
      for (int j = 0; j < PK_M; j++) {
        float qv = bf2f(q_blocks[b * PK_M + j]);
        s += ((c >> j) & 1) ? qv : -qv;
      }
      sc[c] = bfround(s);
    }
    for (int c = 0; c < 256; c++) {
      int rank = 0;
      for (int o = 0; o < 256; o++) rank += (sc[o] > sc[c]) || (sc[o] == sc[c] && o < c);
      sorted_ids[b * 256 + rank] = c;
    }
  }
}

/* Weighted multi-tier collision count for one (batch, head):
 * cache_hub/collision_fused/collision_test.py:56-98 (== collision.cu:92-139, :204-228).
 * A cluster belongs to tier i when the number of keys in clusters ranked before it is
 * < tier_counts[i]; a key's count is the number of (subspace, tier) memberships.
 * codes are read at codes[k*key_stride + b*sub_stride]. */
void pko_collision(const int64_t* sorted_ids, const int32_t* cluster_counts, const uint8_t* codes,
                   int64_t key_stride, int64_t sub_stride, int64_t N, int B, int NC,
                   const int64_t* tier_counts, int n_tiers, int32_t* out) {
  uint8_t* lut = (uint8_t*)calloc((size_t)B * NC, 1);
  for (int b = 0; b < B; b++) {
    uint8_t* mask = (uint8_t*)calloc((size_t)NC, 1);
    int64_t excl = 0;
    for (int p = 0; p < NC; p++) {
      int64_t id = sorted_ids[b * NC + p];
      for (int t = 0; t < n_tiers; t++)
        if (excl < tier_counts[t]) mask[id] |= (uint8_t)(1u << t);
      excl += cluster_counts[b * NC + id];
    }
    for (int c = 0; c < NC; c++) lut[b * NC + c] = (uint8_t)__builtin_popcount(mask[c]);
    free(mask);
  }
#pragma omp parallel for schedule(static)
  for (int64_t k = 0; k < N; k++) {
    int cnt = 0;
    for (int b = 0; b < B; b++) cnt += lut[b * NC + codes[k * key_stride + b * sub_stride]];
    out[k] = cnt;
  }
  free(lut);
}

/* Single-tier, unfused collision count: cache_hub/collision/collision.py:29-45.
 * codes are int32 [N][B] (the kernel-side layout, collision.cu:18-29). */
void pko_collision_single(const int32_t* sorted_ids, const int32_t* topk_cluster_cnt,
                          const int32_t* codes, int64_t N, int B, int NC, int32_t* out) {
  uint8_t* sel = (uint8_t*)calloc((size_t)B * NC, 1);
  for (int b = 0; b < B; b++)
    for (int p = 0; p < NC && p < topk_cluster_cnt[b]; p++) sel[b * NC + sorted_ids[b * NC + p]] = 1;
  for (int64_t k = 0; k < N; k++) {
    int cnt = 0;
    for (int b = 0; b < B; b++) {
      int32_t c = codes[k * B + b];
      if (c >= 0 && c < NC) cnt += sel[b * NC + c];
    }
    out[k] = cnt;
  }
  free(sel);
}

/* ---- deterministic top-k ------------------------------------------------------
 * The reference kernels (cache_hub/topk/radix_topk.cu:39-120, :161-239) keep an
 * arbitrary subset of the elements tied at the threshold and emit in atomics order.
 * Pinned contract: the selected SET is the first k elements in (value descending,
 * index ascending) order; the output lists that set in ASCENDING INDEX order. */
typedef struct {
  uint32_t key;
  int64_t idx;
} pk_kv;
static int cmp_desc(const void* a, const void* b) {
  const pk_kv *x = (const pk_kv*)a, *y = (const pk_kv*)b;
  if (x->key != y->key) return x->key > y->key ? -1 : 1;
  return x->idx < y->idx ? -1 : (x->idx > y->idx);
}
static int cmp_i64(const void* a, const void* b) {
  int64_t x = *(const int64_t*)a, y = *(const int64_t*)b;
  return x < y ? -1 : (x > y);
}
static uint32_t ord_f32(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
static void topk_keys(pk_kv* kv, int64_t n, int64_t k, int64_t* out, int sorted_by_value) {
  qsort(kv, (size_t)n, sizeof(pk_kv), cmp_desc);
  for (int64_t i = 0; i < k; i++) out[i] = kv[i].idx;
  if (!sorted_by_value) qsort(out, (size_t)k, sizeof(int64_t), cmp_i64);
}
void pko_topk_i32(const int32_t* v, int64_t n, int64_t k, int64_t* out, int sorted_by_value) {
  pk_kv* kv = (pk_kv*)malloc(sizeof(pk_kv) * (size_t)n);
  for (int64_t i = 0; i < n; i++) {
    kv[i].key = (uint32_t)v[i] ^ 0x80000000u;
    kv[i].idx = i;
  }
  topk_keys(kv, n, k, out, sorted_by_value);
  free(kv);
}
void pko_topk_f32(const float* v, int64_t n, int64_t k, int64_t* out, int sorted_by_value) {
  pk_kv* kv = (pk_kv*)malloc(sizeof(pk_kv) * (size_t)n);
  for (int64_t i = 0; i < n; i++) {
    kv[i].key = ord_f32(v[i]);
    kv[i].idx = i;
  }
  topk_keys(kv, n, k, out, sorted_by_value);
  free(kv);
}

/* 4-bit RaBitQ rerank: cache_hub/rerank/rerank.py:146-165 (== polar_cache.py:1281-1298).
 * Pinned fp32 order: per subspace dot = fma chain over j ascending (each product of
 * two bf16 values is exact in fp32), acc = fma(dot, w_b, acc) over b ascending,
 * score = acc * ||q||.  packed at packed[k*pk_key + b*pk_sub + i], weights at
 * w[k*w_key + b*w_sub].  Writes fp32 scores and their bf16 roundings. */
void pko_rerank(const int64_t* cand, int64_t C, const uint8_t* packed, int64_t pk_key,
                int64_t pk_sub, const uint16_t* w, int64_t w_key, int64_t w_sub,
                const uint16_t* q_blocks, uint16_t q_norm, const uint16_t* centers, float* score32,
                uint16_t* score_bf) {
  float lev[16];
  for (int t = 0; t < 8; t++) {
    lev[t] = -bf2f(centers[t]);
    lev[8 + t] = bf2f(centers[t]);
  }
  float qn = bf2f(q_norm);
#pragma omp parallel for schedule(static)
  for (int64_t c = 0; c < C; c++) {
    int64_t k = cand[c];
    float acc = 0.0f;
    for (int b = 0; b < PK_B; b++) {
      float dot = 0.0f;
      for (int j = 0; j < PK_M; j++) {
        uint8_t byte = packed[k * pk_key + b * pk_sub + (j >> 1)];
        unsigned nib = (j & 1) ? (byte >> 4) : (byte & 0x0F);
        dot = fmaf(lev[nib], bf2f(q_blocks[b * PK_M + j]), dot);
      }
      acc = fmaf(dot, bf2f(w[k * w_key + b * w_sub]), acc);
    }
    float s = acc * qn;
    score32[c] = s;
    if (score_bf) score_bf[c] = f2bf(s);
  }
}

/* Final select: cache_hub/polar_cache.py:1300-1302.  Pinned: top-K by the fp32 score
 * (a refinement of the bf16 order the reference sorts by), candidate key index
 * ascending on ties; output = key indices, ascending.  cand must be ascending. */
void pko_final_topk(const float* score32, const int64_t* cand, int64_t C, int64_t K, int64_t* out) {
  int64_t* pos = (int64_t*)malloc(sizeof(int64_t) * (size_t)K);
  pko_topk_f32(score32, C, K, pos, 0);
  for (int64_t i = 0; i < K; i++) out[i] = cand[pos[i]];
  free(pos);
}

/* ---- adaptive-k ---------------------------------------------------------------
 * cache_hub/adaptive_k_fused/adaptive_topk.py:275-313 (== adaptive_topk.cu:141-265).
 * Pinned arithmetic shared with the CUDA kernel:
 *  - exp by pk_expf below (range reduction + degree-6 polynomial, all fmaf);
 *  - sums over S / C elements: 1024 strided partials (partial t adds elements
 *    t, t+1024, ... in order), then an adjacent pairwise tree over the partials;
 *  - prefix sums over the sorted top-K_out in chunks of 32: sequential inside a
 *    chunk, chunk offsets by a sequential sum of chunk totals;
 *  - order: benefit descending, candidate position ascending on ties. */
static float pk_expf(float x) {
  if (x < -87.0f) return 0.0f;
  float n = rintf(x * 1.44269504088896341f);
  float r = fmaf(n, -0.693145751953125f, x);
  r = fmaf(n, -1.428606765330187045e-06f, r);
  float p = 1.3888889225e-3f;
  p = fmaf(p, r, 8.3333337680e-3f);
  p = fmaf(p, r, 4.1666667908e-2f);
  p = fmaf(p, r, 1.6666667163e-1f);
  p = fmaf(p, r, 0.5f);
  p = fmaf(p, r, 1.0f);
  p = fmaf(p, r, 1.0f);
  uint32_t e = (uint32_t)((int)n + 127) << 23;
  float sc;
  memcpy(&sc, &e, 4);
  return p * sc;
}
float pko_expf(float x) { return pk_expf(x); }

#define PK_RT 1024
static float strided_tree_sum(const float* v, int64_t n) {
  float part[PK_RT];
  for (int t = 0; t < PK_RT; t++) {
    float p = 0.0f;
    for (int64_t i = t; i < n; i += PK_RT) p += v[i];
    part[t] = p;
  }
  return tree_sum(part, PK_RT);
}

typedef struct {
  uint32_t key;
  int64_t pos;
} pk_bp;
static int cmp_bp(const void* a, const void* b) {
  const pk_bp *x = (const pk_bp*)a, *y = (const pk_bp*)b;
  if (x->key != y->key) return x->key > y->key ? -1 : 1;
  return x->pos < y->pos ? -1 : (x->pos > y->pos);
}

/* One (batch, head).  sl_logits/cand_logits are fp32 and already scaled.
 * Returns adaptive_k; topk_out[K_out] = cand_indices of the K_out largest benefits,
 * benefit descending. */
int64_t pko_adaptive_topk(const float* sl_logits, const float* sl_vnorm, int64_t S,
                          const float* cand_logits, const float* cand_vnorm,
                          const int64_t* cand_indices, int64_t C, float threshold, int64_t K_out,
                          int64_t* topk_out) {
  float gmax = -3.402823466e+38f;
  for (int64_t i = 0; i < S; i++) gmax = fmaxf(gmax, sl_logits[i]);
  for (int64_t i = 0; i < C; i++) gmax = fmaxf(gmax, cand_logits[i]);
  float* tmp = (float*)malloc(sizeof(float) * (size_t)(S > C ? S : C) + 4);
  for (int64_t i = 0; i < S; i++) tmp[i] = pk_expf(sl_logits[i] - gmax) * sl_vnorm[i];
  float sl_ben = strided_tree_sum(tmp, S);
  pk_bp* bp = (pk_bp*)malloc(sizeof(pk_bp) * (size_t)C);
  for (int64_t i = 0; i < C; i++) {
    tmp[i] = pk_expf(cand_logits[i] - gmax) * cand_vnorm[i];
    memcpy(&bp[i].key, &tmp[i], 4);
    bp[i].pos = i;
  }
  float total = sl_ben + strided_tree_sum(tmp, C);
  qsort(bp, (size_t)C, sizeof(pk_bp), cmp_bp);
  int64_t fk = K_out;
  if (total <= 0.0f) {
    fk = 1;
  } else {
    float tgt = threshold * total, base = 0.0f;
    int found = 0;
    for (int64_t c0 = 0; c0 < K_out && !found; c0 += 32) {
      float loc = 0.0f;
      for (int64_t i = c0; i < c0 + 32 && i < K_out; i++) {
        float b;
        memcpy(&b, &bp[i].key, 4);
        loc += b;
        if (sl_ben + (base + loc) >= tgt) {
          fk = i + 1;
          found = 1;
          break;
        }
      }
      base += loc;
    }
  }
  for (int64_t i = 0; i < K_out; i++) topk_out[i] = cand_indices[bp[i].pos];
  free(bp);
  free(tmp);
  return fk;
}

/* Row gather out[k] = src[idx[k]] (row_bytes each):
 * cache_hub/gather_trans/trans_h2d.py:129-139, cache_hub/gather/gather_cpu.cpp:21-114. */
void pko_gather_rows(const uint8_t* src, const int64_t* idx, int64_t K, int64_t row_bytes,
                     uint8_t* out) {
  for (int64_t k = 0; k < K; k++) memcpy(out + k * row_bytes, src + idx[k] * row_bytes, (size_t)row_bytes);
}

/* Decode attention for one KV head: softmax(q K^T * scale) V over n rows, G query heads,
 * non-causal (cache_hub/polar_cache.py:1084-1105).  Double accumulation; out fp32 [G][128].
 * K/V rows are given as arrays of row pointers so window rows and gathered rows mix. */
void pko_attention(const uint16_t* q, int G, const uint16_t* const* krows,
                   const uint16_t* const* vrows, int64_t n, float scale, float* out) {
  double* logit = (double*)malloc(sizeof(double) * (size_t)(n > 0 ? n : 1));
  for (int g = 0; g < G; g++) {
    double m = -1e300;
    for (int64_t r = 0; r < n; r++) {
      double s = 0.0;
      for (int d = 0; d < PK_D; d++) s += (double)bf2f(q[g * PK_D + d]) * (double)bf2f(krows[r][d]);
      logit[r] = s * (double)scale;
      if (logit[r] > m) m = logit[r];
    }
    double acc[PK_D] = {0}, den = 0.0;
    for (int64_t r = 0; r < n; r++) {
      double p = exp(logit[r] - m);
      den += p;
      for (int d = 0; d < PK_D; d++) acc[d] += p * (double)bf2f(vrows[r][d]);
    }
    for (int d = 0; d < PK_D; d++) out[g * PK_D + d] = (float)(n > 0 ? acc[d] / den : 0.0);
  }
  free(logit);
}

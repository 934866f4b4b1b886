// Host-side row gather out[b,h,k,:] = src[b,h,index[b,h,k],:] on CPU threads.  Work is split over
// (batch, head) pairs; rows are copied with memcpy and the next rows are prefetched.
#include <algorithm>
#include <atomic>
#include <cstring>
#include <thread>
#include <vector>

#include "common.cuh"

using namespace pk;

extern "C" int pk_gather_kv_out_cpu(const pk_tensor* src, const pk_tensor* index, const pk_tensor* out,
                                    int n_threads) {
  PK_REQUIRE(src && src->data && out && out->data && index && index->data, "null tensor");
  PK_REQUIRE(src->ndim == 4 && out->ndim == 4 && index->ndim == 3, "src/out must be 4-D, index 3-D");
  PK_REQUIRE(index->dtype == PK_I64, "index must be int64");
  PK_REQUIRE(src->dtype == out->dtype, "src and out dtypes differ");
  const int64_t B = src->shape[0], H = src->shape[1], N = src->shape[2], D = src->shape[3], K = index->shape[2];
  PK_REQUIRE(index->shape[0] == B && index->shape[1] == H, "index must be [B,H,K]");
  PK_REQUIRE(out->shape[0] == B && out->shape[1] == H && out->shape[2] == K && out->shape[3] == D,
             "out must be [B,H,K,D]");
  const int es = elem_size(src->dtype);
  PK_REQUIRE(es > 0, "unsupported dtype");
  const int64_t* idx = (const int64_t*)index->data;
  for (int64_t b = 0; b < B; b++)
    for (int64_t h = 0; h < H; h++)
      for (int64_t k = 0; k < K; k++) {
        const int64_t v = idx[b * index->stride[0] + h * index->stride[1] + k * index->stride[2]];
        PK_REQUIRE(v >= 0 && v < N, "index %lld is out of bounds for dimension 2 with size %lld", (long long)v,
                   (long long)N);
      }
  const bool rows_contig = src->stride[3] == 1 && out->stride[3] == 1;
  const char* sp = (const char*)src->data;
  char* op = (char*)out->data;
  int nt = n_threads > 0 ? n_threads : (int)std::thread::hardware_concurrency();
  nt = (int)std::max<int64_t>(1, std::min<int64_t>(nt, B * H));
  std::atomic<int64_t> next{0};
  auto work = [&]() {
    for (;;) {
      const int64_t bh = next.fetch_add(1);
      if (bh >= B * H) return;
      const int64_t b = bh / H, h = bh % H;
      const int64_t* ib = idx + b * index->stride[0] + h * index->stride[1];
      const char* sb = sp + (b * src->stride[0] + h * src->stride[1]) * es;
      char* ob = op + (b * out->stride[0] + h * out->stride[1]) * es;
      for (int64_t k = 0; k < K; k++) {
        if (k + 4 < K) __builtin_prefetch(sb + ib[(k + 4) * index->stride[2]] * src->stride[2] * es, 0, 0);
        const char* srow = sb + ib[k * index->stride[2]] * src->stride[2] * es;
        char* orow = ob + k * out->stride[2] * es;
        if (rows_contig) {
          std::memcpy(orow, srow, (size_t)(D * es));
        } else {
          for (int64_t d = 0; d < D; d++) std::memcpy(orow + d * out->stride[3] * es, srow + d * src->stride[3] * es, es);
        }
      }
    }
  };
  if (nt == 1) {
    work();
  } else {
    std::vector<std::thread> th;
    for (int i = 0; i < nt; i++) th.emplace_back(work);
    for (auto& t : th) t.join();
  }
  return PK_OK;
}

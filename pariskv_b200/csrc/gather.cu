// UVA gathers of selected K/V rows (256 bytes each) from pinned host memory into device buffers.
// One warp moves one (K row, V row) pair per step: lanes 0-15 carry the K row, lanes 16-31 the V row,
// 16 bytes per lane; warps stride over the rows so thousands of 512-byte requests are in flight on
// the host link at once.
#include "common.cuh"
#include "kernels.cuh"

namespace pk {
namespace {

__device__ __forceinline__ uint4 ld_stream(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

__global__ void __launch_bounds__(256) h2d_gather_kernel(const uint4* __restrict__ src_k, const uint4* __restrict__ src_v,
                                                         const int64_t* __restrict__ idx, uint4* __restrict__ dst_k,
                                                         uint4* __restrict__ dst_v, int64_t n_bh, int64_t src_len,
                                                         int64_t dst_len, int64_t K) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t n_warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  const int64_t total = n_bh * K;
  const uint4* src = lane < 16 ? src_k : src_v;
  uint4* dst = lane < 16 ? dst_k : dst_v;
  const int l = lane & 15;
  for (int64_t r = warp; r < total; r += n_warps) {
    const int64_t bh = r / K, j = r - bh * K;
    const int64_t row = __ldg(idx + r);
    if (row < 0 || row >= src_len) continue;  // out-of-range index: row left untouched
    dst[(bh * dst_len + j) * 16 + l] = ld_stream(src + (bh * src_len + row) * 16 + l);
  }
}

__global__ void __launch_bounds__(256) h2d_gather_packed_kernel(
    const uint4* __restrict__ src_k, const uint4* __restrict__ src_v, uint4* __restrict__ k_packed,
    uint4* __restrict__ v_packed, const int64_t* __restrict__ indices, const int32_t* __restrict__ cu_topk,
    const int32_t* __restrict__ cu_k, int64_t src_len, int64_t sink_local_end, int64_t global_k) {
  const int lane = threadIdx.x & 31;
  const int64_t vh = blockIdx.y;
  const int64_t n = min((int64_t)(cu_topk[vh + 1] - cu_topk[vh]), global_k);
  const int64_t in_base = cu_topk[vh], out_base = (int64_t)cu_k[vh] + sink_local_end;
  const uint4* src = lane < 16 ? src_k : src_v;
  uint4* dst = lane < 16 ? k_packed : v_packed;
  const int l = lane & 15;
  const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t n_warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t j = warp; j < n; j += n_warps) {
    const int64_t row = __ldg(indices + in_base + j);
    if (row < 0 || row >= src_len) continue;
    dst[(out_base + j) * 16 + l] = ld_stream(src + (vh * src_len + row) * 16 + l);
  }
}

// One block per (batch, head): lanes 0-15 copy the K row, lanes 16-31 the V row, to window row pos.
__global__ void __launch_bounds__(32) append_kv_kernel(const uint4* __restrict__ k_row, const uint4* __restrict__ v_row,
                                                       int64_t k_b, int64_t k_h, int64_t v_b, int64_t v_h,
                                                       uint4* __restrict__ wk,
                                                       uint4* __restrict__ wv, int64_t w_b, int64_t w_h, int64_t w_l,
                                                       int H, int64_t cap, int64_t pos, const int32_t* __restrict__ pos_dev,
                                                       int64_t pos_add) {
  const int lane = threadIdx.x, l = lane & 15;
  const int b = blockIdx.x / H, h = blockIdx.x % H;
  const int64_t row = pos_dev ? (int64_t)pos_dev[0] + pos_add : pos;
  if (row < 0 || row >= cap) return;
  const uint4* src = lane < 16 ? k_row + b * k_b + h * k_h : v_row + b * v_b + h * v_h;
  uint4* dst = (lane < 16 ? wk : wv) + b * w_b + h * w_h + row * w_l;
  dst[l] = __ldg(src + l);
}

}  // namespace
}  // namespace pk

using namespace pk;

static int check_store(const pk_tensor* t, const char* name) {
  PK_REQUIRE(t && t->data, "%s is null", name);
  PK_REQUIRE(t->dtype == PK_BF16 && t->ndim == 4 && t->shape[3] == 128 && is_contig(t),
             "%s must be a contiguous bf16 [bs,H,N,128] tensor", name);
  PK_REQUIRE((reinterpret_cast<uintptr_t>(t->data) & 15) == 0, "%s must be 16-byte aligned", name);
  return PK_OK;
}

extern "C" int pk_h2d_gather_kv(const pk_tensor* src_k, const pk_tensor* src_v, const pk_tensor* selected_indices,
                                const pk_tensor* dst_k, const pk_tensor* dst_v, void* stream) {
  int rc;
  if ((rc = check_store(src_k, "src_k")) || (rc = check_store(src_v, "src_v")) || (rc = check_store(dst_k, "dst_k")) ||
      (rc = check_store(dst_v, "dst_v")))
    return rc;
  PK_CHECK_TENSOR(selected_indices, PK_I64, 3);
  const int64_t bs = src_k->shape[0], H = src_k->shape[1], N = src_k->shape[2], K = selected_indices->shape[2];
  PK_REQUIRE(src_v->shape[0] == bs && src_v->shape[1] == H && src_v->shape[2] == N, "src_k and src_v shapes differ");
  PK_REQUIRE(dst_k->shape[0] == bs && dst_k->shape[1] == H && dst_v->shape[0] == bs && dst_v->shape[1] == H &&
                 dst_k->shape[2] == dst_v->shape[2] && dst_k->shape[2] >= K,
             "dst must be [bs,H,cap>=K,128]");
  PK_REQUIRE(is_contig(selected_indices) && selected_indices->shape[0] == bs && selected_indices->shape[1] == H,
             "selected_indices must be contiguous [bs,H,K]");
  if (bs * H * K == 0) return PK_OK;
  const int64_t rows = bs * H * K;
  int64_t blocks = (rows + 7) / 8;
  const int64_t cap = (int64_t)sm_count() * 8;
  if (blocks > cap) blocks = cap;
  StageTimer tm(ST_GATHER, (cudaStream_t)stream);
  h2d_gather_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(
      (const uint4*)src_k->data, (const uint4*)src_v->data, (const int64_t*)selected_indices->data, (uint4*)dst_k->data,
      (uint4*)dst_v->data, bs * H, N, dst_k->shape[2], K);
  return check_launch("h2d_gather_kv");
}

extern "C" int pk_h2d_gather_kv_packed(const pk_tensor* src_k, const pk_tensor* src_v, const pk_tensor* k_packed,
                                       const pk_tensor* v_packed, const pk_tensor* indices_packed,
                                       const pk_tensor* cu_seqlens_topk, const pk_tensor* cu_seqlens_k,
                                       int64_t sink_local_end, int64_t global_k, void* stream) {
  int rc;
  if ((rc = check_store(src_k, "src_k")) || (rc = check_store(src_v, "src_v"))) return rc;
  PK_CHECK_TENSOR(k_packed, PK_BF16, 2);
  PK_CHECK_TENSOR(v_packed, PK_BF16, 2);
  PK_CHECK_TENSOR(indices_packed, PK_I64, 1);
  PK_CHECK_TENSOR(cu_seqlens_topk, PK_I32, 1);
  PK_CHECK_TENSOR(cu_seqlens_k, PK_I32, 1);
  const int64_t V = src_k->shape[0] * src_k->shape[1];
  PK_REQUIRE(is_contig(k_packed) && is_contig(v_packed) && k_packed->shape[1] == 128 && v_packed->shape[1] == 128 &&
                 k_packed->shape[0] == v_packed->shape[0],
             "k_packed / v_packed must be contiguous [total_k,128]");
  PK_REQUIRE((reinterpret_cast<uintptr_t>(k_packed->data) & 15) == 0 && (reinterpret_cast<uintptr_t>(v_packed->data) & 15) == 0,
             "packed buffers must be 16-byte aligned");
  PK_REQUIRE(cu_seqlens_topk->shape[0] == V + 1 && cu_seqlens_k->shape[0] == V + 1 && is_contig(cu_seqlens_topk) &&
                 is_contig(cu_seqlens_k) && is_contig(indices_packed),
             "cu_seqlens_* must be contiguous [bs*H+1]");
  PK_REQUIRE(global_k >= 0 && sink_local_end >= 0, "global_k and sink_local_end must be non-negative");
  if (V == 0 || global_k == 0) return PK_OK;
  int64_t bx = (global_k + 7) / 8;
  int64_t cap = (int64_t)sm_count() * 8 / V + 1;
  if (bx > cap) bx = cap;
  h2d_gather_packed_kernel<<<dim3((unsigned)bx, (unsigned)V), 256, 0, (cudaStream_t)stream>>>(
      (const uint4*)src_k->data, (const uint4*)src_v->data, (uint4*)k_packed->data, (uint4*)v_packed->data,
      (const int64_t*)indices_packed->data, (const int32_t*)cu_seqlens_topk->data, (const int32_t*)cu_seqlens_k->data,
      src_k->shape[2], sink_local_end, global_k);
  return check_launch("h2d_gather_kv_packed");
}

extern "C" int pk_append_kv(const pk_tensor* k_row, const pk_tensor* v_row, const pk_tensor* window_k,
                            const pk_tensor* window_v, int64_t pos, const pk_tensor* pos_dev, int64_t pos_add,
                            void* stream) {
  PK_CHECK_TENSOR(k_row, PK_BF16, 4);
  PK_CHECK_TENSOR(v_row, PK_BF16, 4);
  PK_CHECK_TENSOR(window_k, PK_BF16, 4);
  PK_CHECK_TENSOR(window_v, PK_BF16, 4);
  const int64_t bs = window_k->shape[0], H = window_k->shape[1], cap = window_k->shape[2];
  PK_REQUIRE(k_row->shape[0] == bs && k_row->shape[1] == 1 && k_row->shape[2] == H && k_row->shape[3] == 128 &&
                 k_row->stride[3] == 1,
             "k_row must be [bs,1,H,128] with last stride 1");
  for (int i = 0; i < 4; i++) {
    PK_REQUIRE(k_row->shape[i] == v_row->shape[i], "k_row and v_row must have the same shape");
    PK_REQUIRE(window_k->shape[i] == window_v->shape[i] &&
                   (window_k->shape[i] == 1 || window_k->stride[i] == window_v->stride[i]),
               "window_k and window_v must have the same shape and strides");
  }
  PK_REQUIRE(v_row->stride[3] == 1, "v_row must have last stride 1");
  PK_REQUIRE(window_k->shape[3] == 128 && window_k->stride[3] == 1, "window must be [bs,H,cap,128] with last stride 1");
  const pk_tensor* ts[4] = {k_row, v_row, window_k, window_v};
  for (const pk_tensor* t : ts) {
    PK_REQUIRE((reinterpret_cast<uintptr_t>(t->data) & 15) == 0, "rows must be 16-byte aligned");
    for (int i = 0; i < 3; i++) PK_REQUIRE(t->stride[i] % 8 == 0, "rows must be 16-byte aligned");
  }
  const int32_t* pd = nullptr;
  if (pos_dev) {
    PK_CHECK_TENSOR(pos_dev, PK_I32, 1);
    pd = (const int32_t*)pos_dev->data;
  } else {
    PK_REQUIRE(pos >= 0 && pos < cap, "append position %lld outside the window (capacity %lld)", (long long)pos,
               (long long)cap);
  }
  if (bs * H == 0) return PK_OK;
  StageTimer tm(ST_APPEND, (cudaStream_t)stream);
  append_kv_kernel<<<(unsigned)(bs * H), 32, 0, (cudaStream_t)stream>>>(
      (const uint4*)k_row->data, (const uint4*)v_row->data, k_row->stride[0] / 8, k_row->stride[2] / 8,
      v_row->stride[0] / 8, v_row->stride[2] / 8, (uint4*)window_k->data, (uint4*)window_v->data, window_k->stride[0] / 8, window_k->stride[1] / 8,
      window_k->stride[2] / 8, (int)H, cap, pos, pd, pos_add);
  return check_launch("append_kv");
}

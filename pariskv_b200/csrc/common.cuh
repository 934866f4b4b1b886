// Shared host/device helpers of the pariskv_b200 CUDA library (sm_100a).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/pariskv_b200.h"

namespace pk {

// ---- host side: status, argument checks, launch accounting (defined in common.cu) ----
int fail(int code, const char* fmt, ...);
int check_launch(const char* what, int n_kernels = 1);
int sm_count();

// Stages of the decode path, for the optional event timing (pk_timing_enable / pk_timing_read).
enum Stage { ST_QUERY_PREP = 0, ST_RANK = 1, ST_COLLISION = 2, ST_SELECT_RERANK = 3, ST_FINAL_TOPK = 4,
             ST_ATTENTION = 5, ST_ATTENTION_MERGE = 6, ST_ENCODE = 7, ST_TOPK = 8, ST_RERANK = 9, ST_GATHER = 10,
             ST_COUNT = 11, ST_APPEND = 12, ST_GLUE = 13, ST_REDUCE = 14, ST_SHARD_SEND = 15, ST_SHARD_RECV = 16,
             ST_SHARD_OWNED = 17, ST_HIST_REDUCE = 18, ST_GEMV = 19, ST_ADAPTIVE = 20 };
// Records one event before and one after the launches issued during its lifetime, on the launch stream.
class StageTimer {
 public:
  StageTimer(int stage, cudaStream_t st);
  ~StageTimer();
 private:
  int stage_;
  cudaStream_t st_;
  cudaEvent_t a_;
  bool on_, cap_;
};

#define PK_REQUIRE(cond, ...)                               \
  do {                                                      \
    if (!(cond)) return pk::fail(PK_ERR_ARG, __VA_ARGS__);  \
  } while (0)

inline bool is_contig(const pk_tensor* t) {
  int64_t s = 1;
  for (int i = t->ndim - 1; i >= 0; --i) {
    if (t->shape[i] != 1 && t->stride[i] != s) return false;
    s *= t->shape[i];
  }
  return true;
}
inline int64_t numel(const pk_tensor* t) {
  int64_t n = 1;
  for (int i = 0; i < t->ndim; ++i) n *= t->shape[i];
  return n;
}
inline int elem_size(int dtype) {
  switch (dtype) {
    case PK_U8: return 1;
    case PK_I32: return 4;
    case PK_I64: return 8;
    case PK_F32: return 4;
    case PK_BF16: return 2;
  }
  return 0;
}
#define PK_CHECK_TENSOR(t, dt, nd)                                                        \
  do {                                                                                    \
    PK_REQUIRE((t) != nullptr && (t)->data != nullptr, #t " is null");                    \
    PK_REQUIRE((t)->dtype == (dt), #t " has dtype tag %d, expected %d", (t)->dtype, (dt)); \
    PK_REQUIRE((t)->ndim == (nd), #t " has %d dims, expected %d", (t)->ndim, (nd));       \
  } while (0)

// ---- programmatic dependent launch --------------------------------------------------------------------
// The kernels of the decode chain are launched with the programmatic-stream-serialization attribute: a kernel
// may be scheduled while its predecessor is still running, does the part of its prologue that does not read the
// predecessor's output, and then blocks in pdl_wait() until the predecessor has completed and flushed.  Every
// kernel signals pdl_trigger() only AFTER its own pdl_wait(), so completion is transitive along the chain.
// Without the launch attribute both instructions do nothing.  The attribute is set only after pk_set_pdl(1).
// EVERY kernel launched through launch_chain() must call pdl_wait() before it reads or writes anything an earlier
// kernel may touch: a kernel that skipped the wait would break the chain for its successors.
bool pdl_enabled();

// Per-device "done once" flags for settings that belong to a device (cudaFuncSetAttribute opt-ins): bit d is set
// once the setting has been applied with device d current.  first_on_device() returns the bit to set, or 0 when
// the current device already has it.
struct PerDevice {
  unsigned long long done = 0;  // guarded by per_device_mutex()
};
unsigned long long first_on_device(PerDevice& p);
void mark_on_device(PerDevice& p, unsigned long long bit);

#ifdef __CUDACC__
template <typename... KArgs, typename... Args>
inline cudaError_t launch_chain(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, args...);
}
#endif

// ---- device side ----
#ifdef __CUDACC__
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ float bf2f(uint16_t b) { return __uint_as_float(((uint32_t)b) << 16); }
__device__ __forceinline__ uint16_t f2bf(float f) {
  return __bfloat16_as_ushort(__float2bfloat16_rn(f));
}
__device__ __forceinline__ float bfround(float f) { return bf2f(f2bf(f)); }

// Order-preserving map of fp32 / int32 to uint32 (larger value -> larger key).
__device__ __forceinline__ uint32_t ord_key(float f) {
  uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ uint32_t ord_key(int32_t v) { return (uint32_t)v ^ 0x80000000u; }

// exp for non-positive arguments with a fixed operation sequence (the CPU oracle runs the same
// sequence, so both sides produce identical bits).
__device__ __forceinline__ float pinned_expf(float x) {
  if (x < -87.0f) return 0.0f;
  float n = rintf(__fmul_rn(x, 1.44269504088896341f));
  float r = __fmaf_rn(n, -0.693145751953125f, x);
  r = __fmaf_rn(n, -1.428606765330187045e-06f, r);
  float p = 1.3888889225e-3f;
  p = __fmaf_rn(p, r, 8.3333337680e-3f);
  p = __fmaf_rn(p, r, 4.1666667908e-2f);
  p = __fmaf_rn(p, r, 1.6666667163e-1f);
  p = __fmaf_rn(p, r, 0.5f);
  p = __fmaf_rn(p, r, 1.0f);
  p = __fmaf_rn(p, r, 1.0f);
  float sc = __uint_as_float((uint32_t)((int)n + 127) << 23);
  return __fmul_rn(p, sc);
}
#endif

}  // namespace pk

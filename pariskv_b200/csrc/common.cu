// Status reporting, launch accounting and small host utilities of the pariskv_b200 library.
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <mutex>
#include <vector>

#include "common.cuh"

namespace pk {
static thread_local char g_err[512] = "";
static std::atomic<int64_t> g_launches{0};

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

int check_launch(const char* what, int n_kernels) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(PK_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
  g_launches.fetch_add(n_kernels, std::memory_order_relaxed);
  return PK_OK;
}

// ---- optional per-stage timing with CUDA events (off by default) ----
namespace {
struct Span { int stage; cudaEvent_t a, b; };
constexpr int kMaxSpans = 1 << 16;
std::mutex g_tmu;
bool g_timing = false;
std::vector<Span> g_spans;       // recorded since the last read
std::vector<Span> g_graph_spans; // recorded into a stream capture: re-recorded by every replay of that graph
std::vector<cudaEvent_t> g_pool; // reusable events
cudaEvent_t take_event() {
  if (!g_pool.empty()) { cudaEvent_t e = g_pool.back(); g_pool.pop_back(); return e; }
  cudaEvent_t e = nullptr;
  cudaEventCreate(&e);
  return e;
}
}  // namespace

// Inside a stream capture the events are recorded as EXTERNAL event nodes (cudaEventRecordExternal): they become
// part of the graph and every replay stamps them, so a stage can be timed where it actually runs, between its
// neighbours inside the replayed step.
StageTimer::StageTimer(int stage, cudaStream_t st) : stage_(stage), st_(st), a_(nullptr), on_(false), cap_(false) {
  if (!g_timing) return;
  std::lock_guard<std::mutex> lk(g_tmu);
  cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(st_, &cs) != cudaSuccess) return;
  cap_ = cs == cudaStreamCaptureStatusActive;
  if ((int)(cap_ ? g_graph_spans.size() : g_spans.size()) >= kMaxSpans) return;
  if (cap_) {
    if (cudaEventCreate(&a_) != cudaSuccess) return;   // owned by the graph's span list, not by the pool
  } else {
    a_ = take_event();
  }
  if (a_ && cudaEventRecordWithFlags(a_, st_, cap_ ? cudaEventRecordExternal : cudaEventRecordDefault) == cudaSuccess)
    on_ = true;
}
StageTimer::~StageTimer() {
  if (!on_) return;
  std::lock_guard<std::mutex> lk(g_tmu);
  cudaEvent_t b = nullptr;
  if (cap_) {
    if (cudaEventCreate(&b) != cudaSuccess) return;
  } else {
    b = take_event();
  }
  if (b && cudaEventRecordWithFlags(b, st_, cap_ ? cudaEventRecordExternal : cudaEventRecordDefault) == cudaSuccess)
    (cap_ ? g_graph_spans : g_spans).push_back({stage_, a_, b});
}

static std::atomic<int> g_pdl{0};  // off unless asked for: measured neutral when the step is replayed as a graph
bool pdl_enabled() { return g_pdl.load(std::memory_order_relaxed) != 0; }

static std::mutex g_dev_mu;
unsigned long long first_on_device(PerDevice& p) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
  std::lock_guard<std::mutex> lk(g_dev_mu);
  const unsigned long long bit = 1ull << dev;
  return (p.done & bit) ? 0ull : bit;
}
void mark_on_device(PerDevice& p, unsigned long long bit) {
  std::lock_guard<std::mutex> lk(g_dev_mu);
  p.done |= bit;
}

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}
}  // namespace pk

extern "C" {
int pk_version(void) { return 1; }
const char* pk_last_error(void) { return pk::g_err; }
int64_t pk_launch_count(void) { return pk::g_launches.load(std::memory_order_relaxed); }

int pk_set_pdl(int on) {
  pk::g_pdl.store(on ? 1 : 0, std::memory_order_relaxed);
  return PK_OK;
}

int pk_timing_enable(int on) {
  std::lock_guard<std::mutex> lk(pk::g_tmu);
  pk::g_timing = on != 0;
  return PK_OK;
}

int pk_timing_read(double* ms_per_stage, int64_t* spans_per_stage, int n_stages) {
  std::lock_guard<std::mutex> lk(pk::g_tmu);
  for (int i = 0; i < n_stages; i++) ms_per_stage[i] = 0.0, spans_per_stage[i] = 0;
  for (auto& s : pk::g_spans) {
    float ms = 0.0f;
    if (cudaEventSynchronize(s.b) == cudaSuccess && cudaEventElapsedTime(&ms, s.a, s.b) == cudaSuccess &&
        s.stage >= 0 && s.stage < n_stages) {
      ms_per_stage[s.stage] += ms;
      spans_per_stage[s.stage] += 1;
    }
    pk::g_pool.push_back(s.a);
    pk::g_pool.push_back(s.b);
  }
  pk::g_spans.clear();
  return PK_OK;
}

int pk_timing_read_graph(double* ms_per_stage, int64_t* spans_per_stage, int n_stages) {
  std::lock_guard<std::mutex> lk(pk::g_tmu);
  for (int i = 0; i < n_stages; i++) ms_per_stage[i] = 0.0, spans_per_stage[i] = 0;
  for (auto& s : pk::g_graph_spans) {
    float ms = 0.0f;
    if (cudaEventSynchronize(s.b) == cudaSuccess && cudaEventElapsedTime(&ms, s.a, s.b) == cudaSuccess &&
        s.stage >= 0 && s.stage < n_stages) {
      ms_per_stage[s.stage] += ms;
      spans_per_stage[s.stage] += 1;
    }
  }
  return PK_OK;
}

int pk_timing_clear_graph(void) {
  std::lock_guard<std::mutex> lk(pk::g_tmu);
  for (auto& s : pk::g_graph_spans) {
    cudaEventDestroy(s.a);
    cudaEventDestroy(s.b);
  }
  pk::g_graph_spans.clear();
  return PK_OK;
}
}

// Error side channel, per-thread stream, per-device status word, launch counting and
// per-launch event timing.  The reference has none of this: it aborts the process on any
// CUDA error (include/NVGPUKernels/Utils.h:45-52) and always uses the null stream.
#include <atomic>
#include <cstdlib>
#include <map>
#include <mutex>
#include <string>
#include <utility>
#include <vector>

#include "hom_common.cuh"

#ifdef HOM_NVTX
#include <nvtx3/nvToolsExt.h>
#endif

namespace hom {

namespace {

thread_local int tl_error_code = HOM_OK;
thread_local char tl_error_text[512] = "";
thread_local cudaStream_t tl_stream = nullptr;

constexpr int kMaxDevices = 64;

struct DeviceState {
  std::once_flag once;
  int *status_host = nullptr;  // pinned, mapped
  int *status_dev = nullptr;   // device alias of status_host
  int sm_count = 0;
};
DeviceState g_devices[kMaxDevices];

std::atomic<int64_t> g_launch_count{0};

struct TimingRecord {
  int32_t kind;
  double flops;
  double bytes;
  cudaEvent_t start;
  cudaEvent_t stop;
};
std::mutex g_timing_mutex;
std::vector<TimingRecord> g_timing_log;
std::atomic<bool> g_timing_enabled{false};

// Device address ranges that hold constants (weights): begin -> end.  A GEMM whose B operand
// lies inside one may request its first B tiles before the previous kernel of the stream has
// finished, because no kernel writes a constant.
std::mutex g_const_mutex;
std::map<uintptr_t, uintptr_t> g_const_ranges;

DeviceState &device_state() {
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= kMaxDevices) dev = 0;
  DeviceState &st = g_devices[dev];
  std::call_once(st.once, [&st, dev]() {
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, dev) == cudaSuccess) st.sm_count = prop.multiProcessorCount;
    void *host = nullptr;
    if (cudaHostAlloc(&host, sizeof(int) * 16, cudaHostAllocMapped) == cudaSuccess) {
      st.status_host = static_cast<int *>(host);
      for (int i = 0; i < 16; ++i) st.status_host[i] = 0;
      void *devp = nullptr;
      if (cudaHostGetDevicePointer(&devp, host, 0) == cudaSuccess)
        st.status_dev = static_cast<int *>(devp);
    }
  });
  return st;
}

}  // namespace

void set_error(int code, const char *fmt, ...) {
  tl_error_code = code;
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(tl_error_text, sizeof(tl_error_text), fmt, ap);
  va_end(ap);
  // The slot keeps the latest error only; HOM_TRACE_ERRORS=1 prints every one as it is set.
  static const bool trace = std::getenv("HOM_TRACE_ERRORS") != nullptr;
  if (trace) std::fprintf(stderr, "[hom error %d] %s\n", code, tl_error_text);
}

bool check_cuda(cudaError_t e, const char *what) {
  if (e == cudaSuccess) return true;
  set_error(HOM_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
  return false;
}

cudaStream_t current_stream() { return tl_stream; }

namespace {
struct SplitBuffers {
  float *slots = nullptr;
  size_t slot_floats = 0;
  int *counters = nullptr;
  size_t counter_ints = 0;
  uint64_t clean_epoch = 0;
};
thread_local std::map<std::pair<int, cudaStream_t>, SplitBuffers> tl_split;
std::atomic<uint64_t> g_split_dirty_epoch{0};
}  // namespace

void split_workspace_mark_dirty() { g_split_dirty_epoch.fetch_add(1); }

bool split_workspace(size_t slot_floats, size_t blocks, cudaStream_t stream, SplitWorkspace *out) {
  int dev = 0;
  cudaGetDevice(&dev);
  SplitBuffers &b = tl_split[{dev, stream}];
  if (b.slot_floats < slot_floats) {
    // Round up generously: the typical caller alternates between a few shapes.
    size_t want = slot_floats < (size_t{8} << 20) ? (size_t{8} << 20) : slot_floats + slot_floats / 2;
    // The outgrown buffer is kept, not freed: a captured graph may still hold its address.
    b.slots = nullptr;
    b.slot_floats = 0;
    void *ptr = nullptr;
    if (!check_cuda(cudaMalloc(&ptr, want * sizeof(float)), "cudaMalloc(split-K partials)")) return false;
    b.slots = static_cast<float *>(ptr);
    b.slot_floats = want;
  }
  const uint64_t epoch = g_split_dirty_epoch.load();
  const size_t ints = blocks;
  if (b.counter_ints < ints) {
    size_t want = ints < (size_t{1} << 16) ? (size_t{1} << 16) : 2 * ints;
    b.counters = nullptr;  // kept, like the slots
    b.counter_ints = 0;
    void *ptr = nullptr;
    if (!check_cuda(cudaMalloc(&ptr, want * sizeof(int)), "cudaMalloc(split-K counters)")) return false;
    if (!check_cuda(cudaMemset(ptr, 0, want * sizeof(int)), "cudaMemset(split-K counters)")) {
      cudaFree(ptr);
      return false;
    }
    b.counters = static_cast<int *>(ptr);
    b.counter_ints = want;
    b.clean_epoch = epoch;
  } else if (b.counters && b.clean_epoch != epoch) {
    // A kernel gave up a wait since these counters were last known clean.
    if (!check_cuda(cudaDeviceSynchronize(), "cudaDeviceSynchronize(split-K counters)")) return false;
    if (!check_cuda(cudaMemset(b.counters, 0, b.counter_ints * sizeof(int)), "cudaMemset(split-K counters)"))
      return false;
    b.clean_epoch = epoch;
  }
  out->slots = b.slots;
  out->counters = b.counters;
  return true;
}

namespace {
struct PaddedKey {
  uintptr_t ptr;
  int64_t k, n;  // n < 0: the entry holds the column sums of the [k, -n] weight
  bool operator<(const PaddedKey &o) const {
    return ptr != o.ptr ? ptr < o.ptr : k != o.k ? k < o.k : n < o.n;
  }
};
std::map<PaddedKey, void *> g_padded_weights;  // guarded by g_const_mutex
}  // namespace

namespace {
void *derived_lookup(const void *ptr, int64_t k, int64_t n) {
  std::lock_guard<std::mutex> lock(g_const_mutex);
  auto it = g_padded_weights.find(PaddedKey{reinterpret_cast<uintptr_t>(ptr), k, n});
  return it == g_padded_weights.end() ? nullptr : it->second;
}
void derived_insert(const void *ptr, int64_t k, int64_t n, void *data) {
  std::lock_guard<std::mutex> lock(g_const_mutex);
  void *&slot = g_padded_weights[PaddedKey{reinterpret_cast<uintptr_t>(ptr), k, n}];
  if (slot) cudaFree(slot);
  slot = data;
}
}  // namespace

const __half *padded_weight_lookup(const void *ptr, int64_t k, int64_t n) {
  return static_cast<const __half *>(derived_lookup(ptr, k, n));
}
void padded_weight_insert(const void *ptr, int64_t k, int64_t n, __half *copy) { derived_insert(ptr, k, n, copy); }
const float *weight_colsum_lookup(const void *ptr, int64_t k, int64_t n) {
  return static_cast<const float *>(derived_lookup(ptr, k, -n));
}
void weight_colsum_insert(const void *ptr, int64_t k, int64_t n, float *sums) { derived_insert(ptr, k, -n, sums); }

void declare_constant_range(const void *ptr, size_t bytes) {
  if (!ptr || bytes == 0) return;
  const uintptr_t b = reinterpret_cast<uintptr_t>(ptr);
  std::lock_guard<std::mutex> lock(g_const_mutex);
  // A (re)declaration says "constant from now on": whatever was derived from an earlier content
  // of these addresses (re-pitched copies, column sums) is stale.
  for (auto it = g_padded_weights.lower_bound(PaddedKey{b, INT64_MIN, INT64_MIN});
       it != g_padded_weights.end() && it->first.ptr < b + bytes;) {
    cudaFree(it->second);
    it = g_padded_weights.erase(it);
  }
  g_const_ranges[b] = b + bytes;
}

void forget_constant_range(const void *ptr) {
  std::lock_guard<std::mutex> lock(g_const_mutex);
  const uintptr_t b = reinterpret_cast<uintptr_t>(ptr);
  auto range = g_const_ranges.find(b);
  const uintptr_t e = range == g_const_ranges.end() ? b + 1 : range->second;
  if (range != g_const_ranges.end()) g_const_ranges.erase(range);
  // re-pitched copies of weights inside the withdrawn range go with it
  for (auto it = g_padded_weights.lower_bound(PaddedKey{b, INT64_MIN, INT64_MIN});
       it != g_padded_weights.end() && it->first.ptr < e;) {
    cudaFree(it->second);
    it = g_padded_weights.erase(it);
  }
}

bool is_constant_range(const void *ptr, size_t bytes) {
  const uintptr_t b = reinterpret_cast<uintptr_t>(ptr);
  std::lock_guard<std::mutex> lock(g_const_mutex);
  auto it = g_const_ranges.upper_bound(b);
  if (it == g_const_ranges.begin()) return false;
  --it;
  return b >= it->first && b + bytes <= it->second;
}

bool pdl_enabled() {
  static const bool on = std::getenv("HOM_DISABLE_PDL") == nullptr;
  return on;
}

int *device_status_word() { return device_state().status_dev; }

int *device_status_word_if_ready() {
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= kMaxDevices) dev = 0;
  return g_devices[dev].status_dev;  // null until some earlier call initialised this device
}

int sm_count() {
  int n = device_state().sm_count;
  return n > 0 ? n : 148;
}

namespace {
// Inside stream capture a plain cudaEventRecord only expresses a dependency; the external flag
// turns it into an event-record node that is re-recorded by every replay and can be timed.
void record_event(cudaEvent_t ev, cudaStream_t stream) {
  cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(stream, &st) == cudaSuccess && st == cudaStreamCaptureStatusActive)
    cudaEventRecordWithFlags(ev, stream, cudaEventRecordExternal);
  else
    cudaEventRecord(ev, stream);
}
}  // namespace

#ifdef HOM_NVTX
namespace {
const char *op_kind_name(OpKind kind) {
  switch (kind) {
    case kOpGemm: return "hom.gemm";
    case kOpLayernorm: return "hom.layernorm";
    case kOpAttention: return "hom.attention";
    case kOpElementwise: return "hom.elementwise";
    case kOpGather: return "hom.gather";
    case kOpCuSeqLen: return "hom.cu_seqlen";
  }
  return "hom.op";
}
}  // namespace
#endif

LaunchScope::LaunchScope(OpKind kind, double flops, double bytes, bool may_allocate) {
  g_launch_count.fetch_add(1, std::memory_order_relaxed);
#ifdef HOM_NVTX
  nvtxRangePushA(op_kind_name(kind));  // one range per entry-point launch (compile-time switch)
#endif
  if (!may_allocate || !g_timing_enabled.load(std::memory_order_relaxed)) return;
  TimingRecord rec{kind, flops, bytes, nullptr, nullptr};
  if (cudaEventCreate(&rec.start) != cudaSuccess) return;
  if (cudaEventCreate(&rec.stop) != cudaSuccess) {
    cudaEventDestroy(rec.start);
    return;
  }
  record_event(rec.start, current_stream());
  std::lock_guard<std::mutex> lock(g_timing_mutex);
  g_timing_log.push_back(rec);
  slot_ = static_cast<int>(g_timing_log.size()) - 1;
}

LaunchScope::~LaunchScope() {
#ifdef HOM_NVTX
  nvtxRangePop();
#endif
  if (slot_ < 0) return;
  std::lock_guard<std::mutex> lock(g_timing_mutex);
  if (slot_ < static_cast<int>(g_timing_log.size()))
    record_event(g_timing_log[slot_].stop, current_stream());
}

}  // namespace hom

extern "C" {

int homGetLastError(void) { return hom::tl_error_code; }

const char *homGetLastErrorString(void) { return hom::tl_error_text; }

void homClearLastError(void) {
  hom::tl_error_code = HOM_OK;
  hom::tl_error_text[0] = '\0';
  auto &st = hom::device_state();
  if (st.status_host) st.status_host[0] = 0;
}

void homDeclareWeights(const void *ptr, int64_t bytes) {
  if (bytes > 0) hom::declare_constant_range(ptr, static_cast<size_t>(bytes));
}

void homForgetWeights(const void *ptr) { hom::forget_constant_range(ptr); }

void homSetStream(void *stream) { hom::tl_stream = static_cast<cudaStream_t>(stream); }

void *homGetStream(void) { return hom::tl_stream; }

int homSynchronize(void) {
  cudaError_t e = cudaStreamSynchronize(hom::tl_stream);
  if (e != cudaSuccess) {
    hom::set_error(HOM_ERR_CUDA, "cudaStreamSynchronize: %s", cudaGetErrorString(e));
    return hom::tl_error_code;
  }
  auto &st = hom::device_state();
  if (st.status_host && st.status_host[0] != 0) {
    hom::split_workspace_mark_dirty();
    hom::set_error(HOM_ERR_DEVICE_TIMEOUT, "a device-side wait expired (kernel status %d)",
                   st.status_host[0]);
  }
  return hom::tl_error_code;
}

int64_t homKernelLaunchCount(void) { return hom::g_launch_count.load(); }

void homOpTimingEnable(int enable) { hom::g_timing_enabled.store(enable != 0); }

int64_t homOpTimingPeek(HomOpTiming *out, int64_t capacity) {
  cudaDeviceSynchronize();
  std::lock_guard<std::mutex> lock(hom::g_timing_mutex);
  const int64_t n = static_cast<int64_t>(hom::g_timing_log.size());
  for (int64_t i = 0; i < n && i < capacity && out; ++i) {
    auto &rec = hom::g_timing_log[i];
    float ms = 0.f;
    if (cudaEventElapsedTime(&ms, rec.start, rec.stop) != cudaSuccess) ms = -1.f;
    out[i].kind = rec.kind;
    out[i].ms = ms;
    out[i].flops = rec.flops;
    out[i].bytes = rec.bytes;
  }
  return n;
}

int64_t homOpTimingCollect(HomOpTiming *out, int64_t capacity) {
  cudaDeviceSynchronize();
  std::lock_guard<std::mutex> lock(hom::g_timing_mutex);
  const int64_t n = static_cast<int64_t>(hom::g_timing_log.size());
  for (int64_t i = 0; i < n; ++i) {
    auto &rec = hom::g_timing_log[i];
    float ms = 0.f;
    if (cudaEventElapsedTime(&ms, rec.start, rec.stop) != cudaSuccess) ms = -1.f;
    if (out && i < capacity) {
      out[i].kind = rec.kind;
      out[i].ms = ms;
      out[i].flops = rec.flops;
      out[i].bytes = rec.bytes;
    }
    cudaEventDestroy(rec.start);
    cudaEventDestroy(rec.stop);
  }
  hom::g_timing_log.clear();
  return n;
}

}  // extern "C"

// Internals shared by the runner-utils translation units: memref views, the error
// side channel, the per-thread launch context and per-launch timing.
#pragma once

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "hom_nvgpu_runner_utils.h"

namespace hom {

// ------------------------------------------------------------------ memref view

// Host-side view of an unranked memref argument.  The descriptor record is
// {basePtr, data, offset, sizes[rank], strides[rank]}; `ptr` already includes the offset.
struct MemRefView {
  int64_t rank = 0;
  char *ptr = nullptr;
  int64_t sizes[HOM_MAX_RANK] = {};
  int64_t strides[HOM_MAX_RANK] = {};
  bool valid = false;

  int64_t numel() const {
    int64_t n = 1;
    for (int64_t i = 0; i < rank; ++i) n *= sizes[i];
    return n;
  }
  // Row-major contiguous (size-1 dimensions may carry any stride).
  bool contiguous() const {
    int64_t expect = 1;
    for (int64_t i = rank - 1; i >= 0; --i) {
      if (sizes[i] != 1 && strides[i] != expect) return false;
      expect *= sizes[i];
    }
    return true;
  }
};

inline MemRefView view_memref(int64_t rank, void *descriptor, size_t elem_size) {
  MemRefView v;
  if (descriptor == nullptr || rank < 0 || rank > HOM_MAX_RANK) return v;
  auto *words = static_cast<int64_t *>(descriptor);
  char *data = reinterpret_cast<char *>(static_cast<void **>(descriptor)[1]);
  const int64_t offset = words[2];
  v.rank = rank;
  for (int64_t i = 0; i < rank; ++i) {
    v.sizes[i] = words[3 + i];
    v.strides[i] = words[3 + rank + i];
    if (v.sizes[i] < 0) return v;
  }
  v.ptr = data + offset * static_cast<int64_t>(elem_size);
  v.valid = data != nullptr;
  return v;
}

// ---------------------------------------------------------------- error channel

void set_error(int code, const char *fmt, ...);
bool check_cuda(cudaError_t e, const char *what);  // true when e == cudaSuccess

// ------------------------------------------------------------------ launch context

enum OpKind : int32_t {
  kOpGemm = 1,
  kOpLayernorm = 2,
  kOpAttention = 3,
  kOpElementwise = 4,
  kOpGather = 5,
  kOpCuSeqLen = 6,
};

cudaStream_t current_stream();
// Registry of device ranges that no kernel writes (allocConstantNVGPU* buffers and ranges
// named through homDeclareWeights).
void declare_constant_range(const void *ptr, size_t bytes);
void forget_constant_range(const void *ptr);
bool is_constant_range(const void *ptr, size_t bytes);
// Library-owned copies of declared-constant [K, N] weights whose N is not a multiple of 8,
// re-laid-out with an 8-element-aligned row pitch so that TMA can fetch them; keyed on the
// original pointer and shape, dropped when the declaration is withdrawn.  lookup returns null
// when there is none yet; insert takes ownership of a cudaMalloc'ed copy.
const __half *padded_weight_lookup(const void *ptr, int64_t k, int64_t n);
void padded_weight_insert(const void *ptr, int64_t k, int64_t n, __half *copy);
// The same store for the fp32 column sums of a declared weight (N floats; the LayerNorm-on-A
// forms of the GEMM epilogue need them): computed once, dropped with the declaration.
const float *weight_colsum_lookup(const void *ptr, int64_t k, int64_t n);
void weight_colsum_insert(const void *ptr, int64_t k, int64_t n, float *sums);
// Programmatic dependent launch is on unless HOM_DISABLE_PDL is set (diagnostics).
bool pdl_enabled();
// Host-mapped status word that device code writes on a bounded-wait expiry (device pointer).
int *device_status_word();
// The same pointer if an earlier call on this device already created it, else null; never
// allocates.
int *device_status_word_if_ready();
int sm_count();

// Library-owned split-K scratch of the calling host thread for (current device, `stream`):
// `slot_floats` fp32 values of partial accumulators and `blocks` int counters that are zero
// whenever no GEMM is in flight.  Grow-only, allocated on first use (the reference keeps
// grow-only static device scratch for its split-K semaphores too,
// include/NVGPUKernels/Utils.h:179-224); growing it, or re-zeroing the counters after a kernel
// reported an expired wait, synchronises the device.  Returns false (error recorded) on failure.
struct SplitWorkspace {
  float *slots = nullptr;
  int *counters = nullptr;
};
bool split_workspace(size_t slot_floats, size_t blocks, cudaStream_t stream, SplitWorkspace *out);
// Called when a kernel reported an expired wait: counters may have been left non-zero.
void split_workspace_mark_dirty();

// Launches `kernel` with programmatic stream serialization allowed (and, when cluster_x > 1,
// as clusters of that many CTAs along x).  Every kernel of this library calls
// griddepcontrol.wait before its first dependent global-memory access, which is what makes the
// relaxed launch order safe.
template <typename... KernelArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KernelArgs...), dim3 grid, dim3 block, size_t smem,
                              cudaStream_t stream, unsigned cluster_x, Args &&...args) {
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attrs[2];
  unsigned n = 0;
  attrs[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attrs[n].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
  ++n;
  if (cluster_x > 1) {
    attrs[n].id = cudaLaunchAttributeClusterDimension;
    attrs[n].val.clusterDim.x = cluster_x;
    attrs[n].val.clusterDim.y = 1;
    attrs[n].val.clusterDim.z = 1;
    ++n;
  }
  cfg.attrs = attrs;
  cfg.numAttrs = n;
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KernelArgs>(args)...);
}

// RAII bracket around one kernel launch: counts it and, when timing is enabled,
// records events on the current stream.
class LaunchScope {
 public:
  // `may_allocate` false: only count the launch, even while per-launch timing is enabled
  // (timing creates events and grows a host vector).
  LaunchScope(OpKind kind, double flops, double bytes, bool may_allocate = true);
  ~LaunchScope();

 private:
  int slot_ = -1;
};

}  // namespace hom

// homLayernormGemmF16NoAlloc: cutlassLayernormGemmF16 for callers that must not allocate.
//
// Who needs it: code that runs where device allocation is off the table - a serving process
// whose memory budget was fixed at start-up and whose allocator is locked afterwards, a
// callback running inside somebody else's framework where cudaMalloc would synchronise the
// whole device and stall other streams, or a real-time loop that cannot afford the latency
// and failure modes of an allocator.  The ordinary entry point keeps its column-sum vector
// in a buffer it cudaMallocs on first use; this one keeps it in a fixed array that is part of
// the loaded library image, so the only memory it ever touches is the caller's tensors and
// that array.
#include <atomic>

#include "bandwidth_kernels.cuh"
#include "gemm_sm100.cuh"
#include "hom_common.cuh"
#include "ptx_sm100.cuh"

namespace {

// Largest N (columns of B and D) the entry point accepts.  64 KB of device memory per GPU
// that loads this library, held until the process exits.
constexpr int kNoAllocMaxN = 16384;

// The scratch itself.  In host code this name is only a handle for the runtime's symbol
// table, not a device address: the address is looked up with cudaGetSymbolAddress below.
static __device__ __align__(256) float g_col_sum_scratch[kNoAllocMaxN];

// out[n] = sum over k of b[k, n]; `out` is the scratch array's device address.
__global__ void __launch_bounds__(256)
col_sum_into_scratch_kernel(const __half *b, float *out, int k_dim, int n_dim) {
  hom::ptx::pdl_launch_dependents();
  hom::ptx::pdl_wait();
  const int n = blockIdx.x * blockDim.x + threadIdx.x;
  if (n >= n_dim) return;
  float s = 0.f;
  for (int k = 0; k < k_dim; ++k) s += __half2float(b[static_cast<long long>(k) * n_dim + n]);
  out[n] = s;
}

// Device address of the scratch array on the current device, looked up once per device.
float *scratch_address() {
  static std::atomic<float *> addr[64] = {};
  int dev = 0;
  if (!hom::check_cuda(cudaGetDevice(&dev), "cudaGetDevice")) return nullptr;
  if (dev < 0 || dev >= 64) {
    hom::set_error(HOM_ERR_UNSUPPORTED, "homLayernormGemmF16NoAlloc: device index %d out of range", dev);
    return nullptr;
  }
  float *cached = addr[dev].load(std::memory_order_acquire);
  if (!cached) {
    // Host threads that race here all look up the same address; the last store wins harmlessly.
    void *ptr = nullptr;
    if (!hom::check_cuda(cudaGetSymbolAddress(&ptr, g_col_sum_scratch),
                         "cudaGetSymbolAddress(column-sum scratch)"))
      return nullptr;
    cached = static_cast<float *>(ptr);
    addr[dev].store(cached, std::memory_order_release);
  }
  return cached;
}

bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace

extern "C" __attribute__((visibility("default"))) void homLayernormGemmF16NoAlloc(
    int64_t rankA, void *dstA, int64_t rankB, void *dstB, int64_t rankC, void *dstC, int64_t rankD,
    void *dstD, int64_t rankVar, void *dstVar, int64_t rankMean, void *dstMean, float alpha,
    float beta) {
  using hom::MemRefView;
  using hom::set_error;
  const char *name = "homLayernormGemmF16NoAlloc";
  MemRefView A = hom::view_memref(rankA, dstA, 2), B = hom::view_memref(rankB, dstB, 2);
  MemRefView C = hom::view_memref(rankC, dstC, 2), D = hom::view_memref(rankD, dstD, 2);
  MemRefView V = hom::view_memref(rankVar, dstVar, 2), Mn = hom::view_memref(rankMean, dstMean, 2);
  if (!A.valid || !B.valid || !D.valid || !V.valid || !Mn.valid) {
    set_error(HOM_ERR_INVALID, "%s: null or malformed descriptor", name);
    return;
  }
  if (A.rank != 3 || B.rank != 3 || D.rank != 3 || B.sizes[0] != 1 || V.rank != 1 || Mn.rank != 1 ||
      !A.contiguous() || !B.contiguous() || !D.contiguous() || !V.contiguous() || !Mn.contiguous()) {
    set_error(HOM_ERR_INVALID, "%s: expects contiguous A [Bs,M,K], B [1,K,N], D [Bs,M,N], Var/Mean [Bs*M]",
              name);
    return;
  }
  const int64_t K = A.sizes[2], M = A.sizes[0] * A.sizes[1], N = B.sizes[2];
  if (B.sizes[1] != K || D.sizes[0] != A.sizes[0] || D.sizes[1] != A.sizes[1] || D.sizes[2] != N ||
      V.sizes[0] < M || Mn.sizes[0] < M) {
    set_error(HOM_ERR_INVALID, "%s: operand shapes do not agree", name);
    return;
  }
  if (N > kNoAllocMaxN) {
    set_error(HOM_ERR_UNSUPPORTED,
              "%s: N = %lld exceeds the built-in scratch of %d columns; use cutlassLayernormGemmF16", name,
              static_cast<long long>(N), kNoAllocMaxN);
    return;
  }
  if (M == 0 || N == 0) return;
  if (K == 0 || K % 8 != 0 || N % 8 != 0 || M > INT32_MAX || K > INT32_MAX) {
    set_error(HOM_ERR_UNSUPPORTED, "%s: K and N must be positive multiples of 8 (got K=%lld N=%lld)", name,
              static_cast<long long>(K), static_cast<long long>(N));
    return;
  }
  hom::gemm::Problem pb;
  pb.M = M;
  pb.N = N;
  pb.K = K;
  pb.A = reinterpret_cast<const __half *>(A.ptr);
  pb.B = reinterpret_cast<const __half *>(B.ptr);
  pb.D = reinterpret_cast<__half *>(D.ptr);
  pb.alpha = alpha;
  pb.beta = beta;
  if (beta != 0.f) {
    if (!C.valid || !C.contiguous() || C.rank < 1 || C.sizes[C.rank - 1] != N ||
        !(C.numel() == M * N || C.numel() == N)) {
      set_error(HOM_ERR_INVALID, "%s: beta != 0 needs C of shape [Bs,M,N] or [1,1,N]", name);
      return;
    }
    pb.C = reinterpret_cast<const __half *>(C.ptr);
    pb.c_mode = C.numel() == M * N ? 1 : 2;
  }
  if (!aligned16(pb.A) || !aligned16(pb.B) || !aligned16(pb.D) || (pb.C && !aligned16(pb.C))) {
    set_error(HOM_ERR_INVALID, "%s: A, B, C and D must be 16-byte aligned", name);
    return;
  }
  float *scratch = scratch_address();
  if (!scratch) return;
  cudaStream_t stream = hom::current_stream();
  {
    hom::LaunchScope scope(hom::kOpElementwise, 0.0, 2.0 * K * N + 4.0 * N, /*may_allocate=*/false);
    // Entries [0, N) are rewritten here on every call before the GEMM reads them, so nothing
    // left over from an earlier call (or from a larger N) is ever consumed.
    if (!hom::check_cuda(hom::launch_pdl(col_sum_into_scratch_kernel, dim3(static_cast<unsigned>((N + 255) / 256)),
                                         dim3(256), 0, stream, 1, pb.B, scratch, static_cast<int>(K),
                                         static_cast<int>(N)),
                         "column sum kernel launch"))
      return;
  }
  pb.row_scale = reinterpret_cast<const __half *>(V.ptr);
  pb.row_shift = reinterpret_cast<const __half *>(Mn.ptr);
  pb.col_sum = scratch;
  hom::gemm::run_fixed_no_alloc(pb, stream);
}

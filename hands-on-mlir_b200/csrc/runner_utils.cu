// extern "C" entry points of libhands_on_mlir_nvgpu_runner_utils.so: argument validation and
// dispatch to the sm_100a kernels.  Names and argument lists are those of the reference's
// lib/ExecutionEngine/HandsOnNVGPURunnerUtils.cu; where the reference asserts or exits, these
// record an error (homGetLastError) and launch nothing.
#include <cerrno>
#include <cstdlib>
#include <unistd.h>
#include <sys/stat.h>
#include <atomic>
#include <cstring>
#include <functional>
#include <iostream>
#include <mutex>
#include <string>
#include <vector>

#include "attention_sm100.cuh"
#include "bandwidth_kernels.cuh"
#include "gemm_sm100.cuh"
#include "hom_common.cuh"

// Allocation hook that harnesses written against the reference use directly
// (include/ExecutionEngine/HandsOnNVGPURunnerUtils.h:7, examples/torch/bert/bert.cu:28-30).
__attribute__((visibility("default"))) std::function<void(void **, size_t)> nvgpuAllocer =
    [](void **ptr, size_t size) {
      *ptr = nullptr;
      hom::check_cuda(cudaMalloc(ptr, size ? size : 1), "cudaMalloc");
    };

namespace {

using hom::MemRefView;
using hom::set_error;
using hom::view_memref;

std::mutex g_dir_mutex;
std::string g_constant_dir;

bool is_aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// {rank, malloc'ed descriptor} for a fresh row-major device buffer (allocHelper,
// include/ExecutionEngine/HandsOnRunnerUtils.h:46-73).
HomUnrankedMemRef alloc_memref(const std::vector<int64_t> &sizes, size_t elem_size) {
  HomUnrankedMemRef res{static_cast<int64_t>(sizes.size()), nullptr};
  const size_t rank = sizes.size();
  int64_t total = 1;
  for (int64_t s : sizes) {
    if (s < 0) {
      set_error(HOM_ERR_INVALID, "alloc: negative dimension %lld", static_cast<long long>(s));
      return res;
    }
    total *= s;
  }
  auto *words = static_cast<int64_t *>(std::malloc(sizeof(int64_t) * (3 + 2 * rank)));
  if (!words) {
    set_error(HOM_ERR_INVALID, "alloc: out of host memory for the descriptor");
    return res;
  }
  void *data = nullptr;
  nvgpuAllocer(&data, static_cast<size_t>(total) * elem_size);
  reinterpret_cast<void **>(words)[0] = data;
  reinterpret_cast<void **>(words)[1] = data;
  words[2] = 0;
  int64_t stride = 1;
  for (size_t i = 0; i < rank; ++i) {
    words[3 + i] = sizes[i];
    words[3 + rank + (rank - 1 - i)] = stride;
    stride *= sizes[rank - 1 - i];
  }
  res.descriptor = words;
  return res;
}

std::string constant_path(int32_t idx) {
  std::lock_guard<std::mutex> lock(g_dir_mutex);
  std::string dir = g_constant_dir;
  if (dir.empty()) {
    const char *env = std::getenv("HOM_CONSTANT_DIR");
    dir = env ? env : ".";
  }
  return dir + "/" + std::to_string(idx) + ".txt";
}

// Text weight file: first line = dimensions, then the values
// (writer: lib/WeightsEngine/WeightsEngine.cpp:22-39; reader being replaced:
// lib/ExecutionEngine/HandsOnNVGPURunnerUtils.cu:224-298).
bool read_constant_file(int32_t idx, std::vector<int64_t> *dims, std::vector<float> *values) {
  const std::string path = constant_path(idx);
  FILE *f = std::fopen(path.c_str(), "rb");
  if (!f) {
    set_error(HOM_ERR_IO, "cannot open constant file %s", path.c_str());
    return false;
  }
  std::string text;
  char buf[1 << 16];
  size_t got;
  while ((got = std::fread(buf, 1, sizeof(buf), f)) > 0) text.append(buf, got);
  std::fclose(f);
  const size_t eol = text.find('\n');
  const std::string head = text.substr(0, eol);
  const char *p = head.c_str();
  char *end = nullptr;
  for (;;) {
    errno = 0;
    const long long v = std::strtoll(p, &end, 10);
    if (end == p) break;
    dims->push_back(v);
    p = end;
  }
  if (dims->size() != 3) {
    set_error(HOM_ERR_IO, "%s: expected 3 dimensions on the first line, found %zu", path.c_str(),
              dims->size());
    return false;
  }
  int64_t total = 1;
  for (int64_t d : *dims) total *= d;
  values->reserve(static_cast<size_t>(total));
  p = eol == std::string::npos ? "" : text.c_str() + eol + 1;
  for (int64_t i = 0; i < total; ++i) {
    const float v = std::strtof(p, &end);
    if (end == p) {
      set_error(HOM_ERR_IO, "%s: expected %lld values, found %lld", path.c_str(),
                static_cast<long long>(total), static_cast<long long>(i));
      return false;
    }
    values->push_back(v);
    p = end;
  }
  return true;
}

// ---- binary cache of parsed constants (opt-in: homSetConstantCache(1) or HOM_CONSTANT_CACHE=1).
// Parsing the text of a BERT-sized weight set takes minutes; `<idx>.txt.homcache` beside the
// text file holds the parsed fp32 values and is used while the text file's size and
// modification time still match what the cache recorded.
struct CacheHeader {
  char magic[8];  // "HOMWGT1\0"
  int64_t dims[3];
  int64_t text_size;
  int64_t text_mtime_ns;
};
std::atomic<int> g_constant_cache{-1};  // -1: consult the environment

bool constant_cache_enabled() {
  int v = g_constant_cache.load();
  if (v < 0) {
    const char *env = std::getenv("HOM_CONSTANT_CACHE");
    v = (env && env[0] && env[0] != '0') ? 1 : 0;
    g_constant_cache.store(v);
  }
  return v == 1;
}

bool stat_text(const std::string &path, int64_t *size, int64_t *mtime_ns) {
  struct stat st;
  if (::stat(path.c_str(), &st) != 0) return false;
  *size = static_cast<int64_t>(st.st_size);
  *mtime_ns = static_cast<int64_t>(st.st_mtim.tv_sec) * 1000000000LL + st.st_mtim.tv_nsec;
  return true;
}

bool read_constant_cache(const std::string &text_path, std::vector<int64_t> *dims,
                         std::vector<float> *values) {
  int64_t size = 0, mtime = 0;
  if (!stat_text(text_path, &size, &mtime)) return false;
  FILE *f = std::fopen((text_path + ".homcache").c_str(), "rb");
  if (!f) return false;
  CacheHeader h;
  bool ok = std::fread(&h, sizeof(h), 1, f) == 1 && std::memcmp(h.magic, "HOMWGT1", 8) == 0 &&
            h.text_size == size && h.text_mtime_ns == mtime;
  int64_t total = 1;
  if (ok) {
    for (int64_t d : h.dims) {
      if (d < 0 || (d > 0 && total > (int64_t{1} << 40) / d)) ok = false;
      else total *= d;
    }
  }
  if (ok) {
    values->resize(static_cast<size_t>(total));
    ok = std::fread(values->data(), sizeof(float), values->size(), f) == values->size();
  }
  std::fclose(f);
  if (ok) dims->assign(h.dims, h.dims + 3);
  else values->clear();
  return ok;
}

void write_constant_cache(const std::string &text_path, const std::vector<int64_t> &dims,
                          const std::vector<float> &values) {
  CacheHeader h{};
  std::memcpy(h.magic, "HOMWGT1", 8);
  for (int i = 0; i < 3; ++i) h.dims[i] = dims[i];
  if (!stat_text(text_path, &h.text_size, &h.text_mtime_ns)) return;
  const std::string final_path = text_path + ".homcache";
  const std::string tmp_path = final_path + ".tmp" + std::to_string(static_cast<long long>(::getpid()));
  FILE *f = std::fopen(tmp_path.c_str(), "wb");
  if (!f) return;  // read-only weight directory: run without a cache
  const bool ok = std::fwrite(&h, sizeof(h), 1, f) == 1 &&
                  std::fwrite(values.data(), sizeof(float), values.size(), f) == values.size();
  if (std::fclose(f) != 0 || !ok || std::rename(tmp_path.c_str(), final_path.c_str()) != 0)
    std::remove(tmp_path.c_str());
}

template <typename T>
HomUnrankedMemRef alloc_constant(int32_t idx) {
  std::vector<int64_t> dims;
  std::vector<float> values;
  const bool cache = constant_cache_enabled();
  if (!(cache && read_constant_cache(constant_path(idx), &dims, &values))) {
    dims.clear();
    if (!read_constant_file(idx, &dims, &values)) return HomUnrankedMemRef{0, nullptr};
    if (cache) write_constant_cache(constant_path(idx), dims, values);
  }
  HomUnrankedMemRef res = alloc_memref(dims, sizeof(T));
  if (!res.descriptor) return res;
  void *data = static_cast<void **>(res.descriptor)[1];
  if (!data) return res;
  hom::declare_constant_range(data, values.size() * sizeof(T));
  if (sizeof(T) == 2) {
    std::vector<__half> h(values.size());
    for (size_t i = 0; i < values.size(); ++i) h[i] = __float2half_rn(values[i]);
    hom::check_cuda(cudaMemcpy(data, h.data(), h.size() * 2, cudaMemcpyHostToDevice),
                    "cudaMemcpy(constant)");
  } else {
    hom::check_cuda(cudaMemcpy(data, values.data(), values.size() * 4, cudaMemcpyHostToDevice),
                    "cudaMemcpy(constant)");
  }
  return res;
}

void dealloc_memref(int64_t rank, void *dst) {
  if (!dst) return;
  void *data = static_cast<void **>(dst)[1];
  (void)rank;
  hom::forget_constant_range(data);
  if (data) hom::check_cuda(cudaFree(data), "cudaFree");
}

// Validates the operands of a GEMM entry point and fills `out`; returns false when the call
// is rejected (error recorded) or there is nothing to do (M or N is 0: *empty set).
bool gemm_prepare(const char *name, bool b_is_nk, int64_t rankA, void *dstA, int64_t rankB,
                  void *dstB, int64_t rankC, void *dstC, int64_t rankD, void *dstD,
                  int64_t activation, float alpha, float beta, hom::gemm::Problem *out, bool *empty,
                  bool allow_unaligned_kn = false) {
  *empty = false;
  MemRefView A = view_memref(rankA, dstA, 2), B = view_memref(rankB, dstB, 2);
  MemRefView C = view_memref(rankC, dstC, 2), D = view_memref(rankD, dstD, 2);
  if (!A.valid || !B.valid || !D.valid) {
    set_error(HOM_ERR_INVALID, "%s: null or malformed A/B/D descriptor", name);
    return false;
  }
  if ((A.rank != 2 && A.rank != 3) || (B.rank != 2 && B.rank != 3) || D.rank != A.rank) {
    set_error(HOM_ERR_INVALID, "%s: A, D must be rank 2 or 3 and B rank 2 or 3", name);
    return false;
  }
  if (!A.contiguous() || !B.contiguous() || !D.contiguous()) {
    set_error(HOM_ERR_INVALID, "%s: operands must be row-major contiguous", name);
    return false;
  }
  if (activation != 0 && activation != 1) {
    set_error(HOM_ERR_UNSUPPORTED, "%s: activation %lld (0 = none, 1 = erf GELU)", name,
              static_cast<long long>(activation));
    return false;
  }
  const int64_t K = A.sizes[A.rank - 1];
  const int64_t M = A.numel() / (K ? K : 1);
  if (B.rank == 3 && B.sizes[0] != 1) {
    set_error(HOM_ERR_UNSUPPORTED, "%s: B must have batch 1 (weights are shared by the batch)", name);
    return false;
  }
  const int64_t b0 = B.sizes[B.rank - 2], b1 = B.sizes[B.rank - 1];
  const int64_t Kb = b_is_nk ? b1 : b0, N = b_is_nk ? b0 : b1;
  if (Kb != K) {
    set_error(HOM_ERR_INVALID, "%s: inner dimensions differ (A has K=%lld, B has K=%lld)", name,
              static_cast<long long>(K), static_cast<long long>(Kb));
    return false;
  }
  if (D.sizes[D.rank - 1] != N || D.numel() != M * N) {
    set_error(HOM_ERR_INVALID, "%s: D must be [%lld x %lld]", name, static_cast<long long>(M),
              static_cast<long long>(N));
    return false;
  }
  for (int64_t i = 0; i + 1 < A.rank; ++i) {
    if (A.sizes[i] != D.sizes[i]) {
      set_error(HOM_ERR_INVALID, "%s: leading dimensions of A and D differ", name);
      return false;
    }
  }
  if (M == 0 || N == 0) {
    *empty = true;
    return false;
  }
  if (K == 0) {
    set_error(HOM_ERR_UNSUPPORTED, "%s: K == 0", name);
    return false;
  }
  // TMA needs 16-byte rows: K % 8 == 0 for A (and for B stored [N,K]); N % 8 == 0 for B
  // stored [K,N].  With B as [N,K] any N works: C / D are then handled without TMA.
  if (K % 8 != 0 || (!b_is_nk && N % 8 != 0 && !allow_unaligned_kn)) {
    set_error(HOM_ERR_UNSUPPORTED,
              "%s: K%s must be a multiple of 8 (16-byte rows for TMA); got K=%lld N=%lld", name,
              b_is_nk ? "" : " and N", static_cast<long long>(K), static_cast<long long>(N));
    return false;
  }
  const bool unaligned_n = N % 8 != 0;
  if (M > INT32_MAX || N > INT32_MAX || K > INT32_MAX) {
    set_error(HOM_ERR_UNSUPPORTED, "%s: dimension exceeds 2^31-1", name);
    return false;
  }
  hom::gemm::Problem pb;
  pb.M = M;
  pb.N = N;
  pb.K = K;
  pb.A = reinterpret_cast<const __half *>(A.ptr);
  pb.B = reinterpret_cast<const __half *>(B.ptr);
  pb.b_is_nk = b_is_nk;
  pb.b_const = hom::is_constant_range(B.ptr, static_cast<size_t>(K) * N * 2);
  pb.D = reinterpret_cast<__half *>(D.ptr);
  pb.alpha = alpha;
  pb.beta = beta;
  pb.act = static_cast<int>(activation);
  pb.c_mode = 0;
  if (beta != 0.f) {
    if (!C.valid || !C.contiguous()) {
      set_error(HOM_ERR_INVALID, "%s: beta != 0 needs a contiguous C", name);
      return false;
    }
    if (C.numel() == M * N && C.sizes[C.rank - 1] == N) {
      pb.c_mode = 1;
    } else if (C.numel() == N && C.rank >= 1 && C.sizes[C.rank - 1] == N) {
      pb.c_mode = 2;
    } else {
      set_error(HOM_ERR_INVALID, "%s: C must be [%lld x %lld] or a length-%lld row", name,
                static_cast<long long>(M), static_cast<long long>(N), static_cast<long long>(N));
      return false;
    }
    pb.C = reinterpret_cast<const __half *>(C.ptr);
    if (!unaligned_n && !is_aligned16(pb.C)) {
      set_error(HOM_ERR_INVALID, "%s: C is not 16-byte aligned", name);
      return false;
    }
  }
  if (!is_aligned16(pb.A) || (!(unaligned_n && !b_is_nk) && !is_aligned16(pb.B)) ||
      (!unaligned_n && !is_aligned16(pb.D))) {
    set_error(HOM_ERR_INVALID, "%s: A, B and D must be 16-byte aligned", name);
    return false;
  }
  *out = pb;
  return true;
}

// B stored [K, N] with N % 8 != 0 (the vocabulary projection, N = 30522, which the reference
// serves with alignment-2 kernels, python/gemm_generator.py:232): its rows are not 16-byte
// aligned, so TMA cannot fetch it in place.  The GEMM runs on a copy whose row pitch is rounded
// up to 8 elements: made once and kept for a declared constant (model weights), re-made on every
// call into a grow-only scratch of the calling thread for any other B.
bool repitch_unaligned_b(const char *name, hom::gemm::Problem *pb) {
  const int64_t pitch = (pb->N + 7) / 8 * 8;
  cudaStream_t stream = hom::current_stream();
  const __half *copy = pb->b_const ? hom::padded_weight_lookup(pb->B, pb->K, pb->N) : nullptr;
  if (!copy) {
    __half *fresh = nullptr;
    if (pb->b_const) {
      void *ptr = nullptr;
      if (!hom::check_cuda(cudaMalloc(&ptr, static_cast<size_t>(pb->K) * pitch * 2), "cudaMalloc(re-pitched weights)"))
        return false;
      fresh = static_cast<__half *>(ptr);
    } else {
      thread_local __half *scratch = nullptr;
      thread_local size_t scratch_elems = 0;
      const size_t need = static_cast<size_t>(pb->K) * pitch;
      if (scratch_elems < need) {
        if (scratch) cudaFree(scratch);  // waits for the kernels that may still read it
        scratch = nullptr;
        scratch_elems = 0;
        void *ptr = nullptr;
        if (!hom::check_cuda(cudaMalloc(&ptr, need * 2), "cudaMalloc(re-pitched B)")) return false;
        scratch = static_cast<__half *>(ptr);
        scratch_elems = need;
      }
      fresh = scratch;
    }
    if (!hom::bw::repitch_rows_f16(pb->B, fresh, pb->K, pb->N, pitch, stream)) {
      if (pb->b_const) cudaFree(fresh);
      return false;
    }
    if (pb->b_const) {
      // other streams may use the cached copy next: make it complete before it becomes visible
      if (!hom::check_cuda(cudaStreamSynchronize(stream), "cudaStreamSynchronize(re-pitched weights)")) {
        cudaFree(fresh);
        return false;
      }
      hom::padded_weight_insert(pb->B, pb->K, pb->N, fresh);
    }
    copy = fresh;
  }
  (void)name;
  pb->B = copy;
  pb->ldb = pitch;
  return true;
}

// Shared front end of cutlassGemmF16 / nvteGemmF16.
void gemm_entry(const char *name, bool b_is_nk, int64_t rankA, void *dstA, int64_t rankB,
                void *dstB, int64_t rankC, void *dstC, int64_t rankD, void *dstD,
                int64_t activation, float alpha, float beta, int32_t tile_row, int32_t split_k) {
  hom::gemm::Problem pb;
  bool empty = false;
  if (!gemm_prepare(name, b_is_nk, rankA, dstA, rankB, dstB, rankC, dstC, rankD, dstD, activation,
                    alpha, beta, &pb, &empty, /*allow_unaligned_kn=*/true))
    return;
  if (!b_is_nk && pb.N % 8 != 0 && !repitch_unaligned_b(name, &pb)) return;
  pb.split_k = split_k;
  hom::gemm::run(pb, tile_row, hom::current_stream());
}

// Library-owned scratch for the column sums of B that the LayerNorm-on-A GEMM needs: one
// fixed buffer per device, allocated on first use (the reference keeps grow-only static device
// scratch for the same kind of purpose, include/NVGPUKernels/Utils.h:179-224).
constexpr int64_t kColSumCapacity = 65536;
float *col_sum_scratch() {
  static float *bufs[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (!bufs[dev]) {
    void *ptr = nullptr;
    if (!hom::check_cuda(cudaMalloc(&ptr, kColSumCapacity * sizeof(float)), "cudaMalloc(column sums)"))
      return nullptr;
    bufs[dev] = static_cast<float *>(ptr);
  }
  return bufs[dev];
}

// Var / Mean operands of the fused forms: rank-1 fp16 with at least `rows` entries.
bool stats_operand(const char *name, const char *what, int64_t rank, void *dst, int64_t rows,
                   __half **out) {
  MemRefView v = view_memref(rank, dst, 2);
  if (!v.valid || v.rank != 1 || v.sizes[0] < rows || !v.contiguous()) {
    set_error(HOM_ERR_INVALID, "%s: %s must be a rank-1 fp16 memref with at least %lld entries", name,
              what, static_cast<long long>(rows));
    return false;
  }
  *out = reinterpret_cast<__half *>(v.ptr);
  return true;
}


void elementwise_entry(const char *name, int op, bool is_f16, int64_t rankA, void *dstA,
                       int64_t rankB, void *dstB, int64_t rankOut, void *dstOut) {
  const size_t es = is_f16 ? 2 : 4;
  MemRefView A = view_memref(rankA, dstA, es), B = view_memref(rankB, dstB, es);
  MemRefView O = view_memref(rankOut, dstOut, es);
  if (!A.valid || !B.valid || !O.valid) {
    set_error(HOM_ERR_INVALID, "%s: null or malformed descriptor", name);
    return;
  }
  if (A.rank != B.rank || A.rank != O.rank) {
    set_error(HOM_ERR_INVALID, "%s: ranks differ (%lld, %lld, %lld)", name,
              static_cast<long long>(A.rank), static_cast<long long>(B.rank),
              static_cast<long long>(O.rank));
    return;
  }
  for (int64_t i = 0; i < A.rank; ++i) {
    if (A.sizes[i] != O.sizes[i] || (B.sizes[i] != A.sizes[i] && B.sizes[i] != 1)) {
      set_error(HOM_ERR_INVALID, "%s: shapes do not match (only B may broadcast) at dim %lld", name,
                static_cast<long long>(i));
      return;
    }
  }
  if (!A.contiguous() || !O.contiguous() || !B.contiguous()) {
    set_error(HOM_ERR_INVALID, "%s: operands must be row-major contiguous", name);
    return;
  }
  const int64_t n = A.numel();
  if (n == 0) return;
  // B repeats with period numel(B) when it broadcasts only over a leading run of dimensions.
  int64_t first_full = 0;
  while (first_full < A.rank && B.sizes[first_full] == 1) ++first_full;
  bool periodic = true;
  for (int64_t i = first_full; i < A.rank; ++i)
    if (B.sizes[i] != A.sizes[i]) periodic = false;
  hom::bw::BroadcastShape sh;
  sh.rank = static_cast<int>(A.rank);
  int64_t os = 1, bs = 1;
  for (int64_t i = A.rank - 1; i >= 0; --i) {
    sh.out_stride[i] = os;
    sh.b_size[i] = B.sizes[i];
    sh.b_stride[i] = bs;
    os *= A.sizes[i];
    bs *= B.sizes[i];
  }
  hom::bw::elementwise(op, is_f16, A.ptr, B.ptr, O.ptr, n, B.numel(), periodic ? B.numel() : 0, sh,
                       hom::current_stream());
}

void gather_entry(const char *name, bool is_f16, int64_t rankI, void *desI, int64_t rankV,
                  void *desV, int64_t rankO, void *desO) {
  const size_t es = is_f16 ? 2 : 4;
  MemRefView I = view_memref(rankI, desI, 8), V = view_memref(rankV, desV, es);
  MemRefView O = view_memref(rankO, desO, es);
  if (!I.valid || !V.valid || !O.valid) {
    set_error(HOM_ERR_INVALID, "%s: null or malformed descriptor", name);
    return;
  }
  if (V.rank != 3 || V.sizes[0] != 1 || I.rank != 2 || O.rank != 3) {
    set_error(HOM_ERR_INVALID, "%s: expects indices [bs,seq], table [1,V,H], out [bs,seq,H]", name);
    return;
  }
  if (O.sizes[2] != V.sizes[2] || O.sizes[0] != I.sizes[0] || O.sizes[1] != I.sizes[1]) {
    set_error(HOM_ERR_INVALID, "%s: output shape does not match indices/table", name);
    return;
  }
  if (!I.contiguous() || !V.contiguous() || !O.contiguous()) {
    set_error(HOM_ERR_INVALID, "%s: operands must be row-major contiguous", name);
    return;
  }
  hom::bw::gather_rows(is_f16, reinterpret_cast<const int64_t *>(I.ptr), V.ptr, O.ptr, I.numel(),
                       V.sizes[1], V.sizes[2], hom::current_stream());
}

void cu_seqlen_entry(const char *name, bool is_i64, int64_t rankIn, void *desIn, int64_t rankOut,
                     void *desOut) {
  MemRefView In = view_memref(rankIn, desIn, is_i64 ? 8 : 4), Out = view_memref(rankOut, desOut, 4);
  if (!In.valid || !Out.valid) {
    set_error(HOM_ERR_INVALID, "%s: null or malformed descriptor", name);
    return;
  }
  if (In.rank != 2 || Out.rank != 1 || Out.sizes[0] != In.sizes[0] + 1) {
    set_error(HOM_ERR_INVALID, "%s: expects mask [bs,seq] and out [bs+1]", name);
    return;
  }
  if (!In.contiguous() || !Out.contiguous() || In.sizes[0] > INT32_MAX || In.sizes[1] > INT32_MAX) {
    set_error(HOM_ERR_INVALID, "%s: operands must be contiguous and below 2^31 per dimension", name);
    return;
  }
  hom::bw::cu_seqlen(is_i64, In.ptr, reinterpret_cast<int *>(Out.ptr), In.sizes[0], In.sizes[1],
                     hom::current_stream());
}

void print_sizes(int64_t rank, void *descriptor) {
  std::cerr << "Print inside: ";
  if (descriptor) {
    auto *words = static_cast<int64_t *>(descriptor);
    for (int64_t i = 0; i < rank; ++i) std::cerr << words[3 + i] << " ";
  }
  std::cerr << std::endl;
}

bool layernorm_rows(const MemRefView &A, int64_t *rows, int64_t *hidden) {
  if (A.rank != 2 && A.rank != 3) return false;
  *hidden = A.sizes[A.rank - 1];
  *rows = *hidden ? A.numel() / *hidden : 0;
  return true;
}

}  // namespace

extern "C" {

void cutlassGemmF16(int64_t rankA, void *dstA, bool transa, int64_t rankB, void *dstB, bool transb,
                    int64_t rankC, void *dstC, int64_t rankD, void *dstD, int64_t activation,
                    float alpha, float beta, int32_t gemmNum, int32_t splitKFactor) {
  // Like the reference entry point, the transpose flags are not consulted: A is [.,M,K] and
  // B is [1,K,N].  splitKFactor >= 2 cuts every output tile's K range into that many work
  // units (include/NVGPUKernels/GemmRunner.h:279-284 hands the factor to the kernel the same
  // way); the default 1 that un-tuned models pass leaves the choice to the tile table.
  (void)transa;
  (void)transb;
  gemm_entry("cutlassGemmF16", false, rankA, dstA, rankB, dstB, rankC, dstC, rankD, dstD,
             activation, alpha, beta, gemmNum, splitKFactor);
}

void cutlassGemmF32(int64_t, void *, bool, int64_t, void *, bool, int64_t, void *, int64_t, void *,
                    int64_t, float, float) {
  set_error(HOM_ERR_UNSUPPORTED, "cutlassGemmF32: the fp32 GEMM is an empty stub in the reference");
}

void nvteGemmF16(int64_t rankA, void *dstA, bool transa, int64_t rankB, void *dstB, bool transb,
                 int64_t rankC, void *dstC, int64_t rankD, void *dstD, int64_t activation,
                 float alpha, float beta, int32_t gemmNum, int32_t) {
  // The reference ignores the two trailing integers on this path; here the first one is
  // honoured as a tile-table row like cutlassGemmF16's gemmNum (0 = automatic).
  if (transa || !transb) {
    set_error(HOM_ERR_UNSUPPORTED, "nvteGemmF16: only transa=false, transb=true (B as [1,N,K])");
    return;
  }
  if (alpha != 1.f || (beta != 0.f && beta != 1.f)) {
    set_error(HOM_ERR_UNSUPPORTED, "nvteGemmF16: needs alpha == 1 and beta in {0, 1}");
    return;
  }
  gemm_entry("nvteGemmF16", true, rankA, dstA, rankB, dstB, rankC, dstC, rankD, dstD, activation,
             alpha, beta, gemmNum, 0);
}

void cutlassGemmWithVarMeanF16(int64_t rankA, void *dstA, int64_t rankB, void *dstB, int64_t rankC,
                               void *dstC, int64_t rankD, void *dstD, int64_t rankVar, void *dstVar,
                               int64_t rankMean, void *dstMean, float alpha, float beta,
                               int64_t activation, float eps) {
  // D = alpha * A.B + beta * C, and per row of D: Var <- 1/sqrt(E[x^2] - mean^2 + eps) and
  // Mean <- -mean * Var (what the reference leaves in its first Bs*M entries after
  // ApplyFinalReduction).  Like the reference's epilogue visitor, the GEMM epilogue itself emits
  // the per-row partial sums (fp32, one pair per 64-column group) while it still holds the tile;
  // a small finaliser reduces them.  D is never read back.  `activation` is ignored, as in the
  // reference.
  (void)activation;
  hom::gemm::Problem pb;
  bool empty = false;
  if (!gemm_prepare("cutlassGemmWithVarMeanF16", false, rankA, dstA, rankB, dstB, rankC, dstC, rankD,
                    dstD, 0, alpha, beta, &pb, &empty))
    return;
  __half *var = nullptr, *mean = nullptr;
  if (!stats_operand("cutlassGemmWithVarMeanF16", "Var", rankVar, dstVar, pb.M, &var) ||
      !stats_operand("cutlassGemmWithVarMeanF16", "Mean", rankMean, dstMean, pb.M, &mean))
    return;
  const int groups = static_cast<int>((pb.N + 63) / 64);
  hom::SplitWorkspace ws;  // library-owned scratch of this thread and stream
  if (!hom::split_workspace(2 * static_cast<size_t>(groups) * pb.M, 0, hom::current_stream(), &ws)) return;
  pb.row_partials = reinterpret_cast<float2 *>(ws.slots);
  if (!hom::gemm::run(pb, 0, hom::current_stream())) return;
  hom::bw::row_stats_finalize(pb.row_partials, groups, pb.M, pb.N, eps, var, mean, hom::current_stream());
}

void cutlassLayernormGemmF32(int64_t, void *, int64_t, void *, int64_t, void *, int64_t, void *,
                             int64_t, void *, int64_t, void *, float, float, int64_t) {
  set_error(HOM_ERR_UNSUPPORTED, "cutlassLayernormGemmF32: empty stub in the reference");
}

void cutlassLayernormGemmF16(int64_t rankA, void *dstA, int64_t rankB, void *dstB, int64_t rankC,
                             void *dstC, int64_t rankD, void *dstD, int64_t rankVar, void *dstVar,
                             int64_t rankMean, void *dstMean, float alpha, float beta,
                             int64_t activation) {
  // D = alpha * (A * Var[r] + Mean[r]).B + beta * C with the row statistics a preceding
  // cutlassGemmWithVarMeanF16 produced (LayerNorm of A with scale 1, shift 0).  The GEMM runs
  // on the raw A; the epilogue applies Var[r] * acc + Mean[r] * colsum(B)[n].
  (void)activation;
  hom::gemm::Problem pb;
  bool empty = false;
  if (!gemm_prepare("cutlassLayernormGemmF16", false, rankA, dstA, rankB, dstB, rankC, dstC, rankD,
                    dstD, 0, alpha, beta, &pb, &empty))
    return;
  __half *var = nullptr, *mean = nullptr;
  if (!stats_operand("cutlassLayernormGemmF16", "Var", rankVar, dstVar, pb.M, &var) ||
      !stats_operand("cutlassLayernormGemmF16", "Mean", rankMean, dstMean, pb.M, &mean))
    return;
  if (pb.N > kColSumCapacity) {
    set_error(HOM_ERR_UNSUPPORTED, "cutlassLayernormGemmF16: N = %lld exceeds the %lld-column scratch",
              static_cast<long long>(pb.N), static_cast<long long>(kColSumCapacity));
    return;
  }
  float *col_sum = col_sum_scratch();
  if (!col_sum) return;
  if (!hom::bw::col_sum_f16(pb.B, col_sum, pb.K, pb.N, false, hom::current_stream())) return;
  pb.row_scale = var;
  pb.row_shift = mean;
  pb.col_sum = col_sum;
  hom::gemm::run(pb, 0, hom::current_stream());
}

void nvteLayernormF16(int64_t rankA, void *dstA, float eps) {
  MemRefView A = view_memref(rankA, dstA, 2);
  int64_t rows = 0, hidden = 0;
  if (!A.valid || !layernorm_rows(A, &rows, &hidden) || !A.contiguous()) {
    set_error(HOM_ERR_INVALID, "nvteLayernormF16: expects a contiguous rank-2 or rank-3 tensor");
    return;
  }
  if (hidden > INT32_MAX) {
    set_error(HOM_ERR_UNSUPPORTED, "nvteLayernormF16: hidden size too large");
    return;
  }
  auto *x = reinterpret_cast<__half *>(A.ptr);
  hom::bw::layernorm_f16(x, nullptr, nullptr, nullptr, x, rows, hidden, eps, hom::current_stream());
}

void nvteLayernormF32(int64_t rankA, void *dstA, float eps) {
  MemRefView A = view_memref(rankA, dstA, 4);
  int64_t rows = 0, hidden = 0;
  if (!A.valid || !layernorm_rows(A, &rows, &hidden) || !A.contiguous()) {
    set_error(HOM_ERR_INVALID, "nvteLayernormF32: expects a contiguous rank-2 or rank-3 tensor");
    return;
  }
  if (hidden > INT32_MAX) {
    set_error(HOM_ERR_UNSUPPORTED, "nvteLayernormF32: hidden size too large");
    return;
  }
  auto *x = reinterpret_cast<float *>(A.ptr);
  hom::bw::layernorm_f32(x, x, rows, hidden, eps, hom::current_stream());
}

void homResidualLayernormF16(int64_t rankX, void *dstX, int64_t rankR, void *dstR,
                             int64_t rankGamma, void *dstGamma, int64_t rankBeta, void *dstBeta,
                             int64_t rankOut, void *dstOut, float eps) {
  MemRefView X = view_memref(rankX, dstX, 2), O = view_memref(rankOut, dstOut, 2);
  int64_t rows = 0, hidden = 0;
  if (!X.valid || !O.valid || !layernorm_rows(X, &rows, &hidden) || !X.contiguous() ||
      !O.contiguous() || O.numel() != X.numel() || O.sizes[O.rank - 1] != hidden) {
    set_error(HOM_ERR_INVALID,
              "homResidualLayernormF16: X and Out must be contiguous rank-2/3 tensors of equal shape");
    return;
  }
  const __half *r = nullptr, *g = nullptr, *b = nullptr;
  if (dstR && rankR > 0) {
    MemRefView R = view_memref(rankR, dstR, 2);
    if (!R.valid || !R.contiguous() || R.numel() != X.numel()) {
      set_error(HOM_ERR_INVALID, "homResidualLayernormF16: residual must match X");
      return;
    }
    r = reinterpret_cast<const __half *>(R.ptr);
  }
  if (dstGamma && rankGamma > 0) {
    MemRefView G = view_memref(rankGamma, dstGamma, 2);
    if (!G.valid || !G.contiguous() || G.numel() != hidden) {
      set_error(HOM_ERR_INVALID, "homResidualLayernormF16: gamma must have H elements");
      return;
    }
    g = reinterpret_cast<const __half *>(G.ptr);
  }
  if (dstBeta && rankBeta > 0) {
    MemRefView Bt = view_memref(rankBeta, dstBeta, 2);
    if (!Bt.valid || !Bt.contiguous() || Bt.numel() != hidden) {
      set_error(HOM_ERR_INVALID, "homResidualLayernormF16: beta must have H elements");
      return;
    }
    b = reinterpret_cast<const __half *>(Bt.ptr);
  }
  if (hidden > INT32_MAX) {
    set_error(HOM_ERR_UNSUPPORTED, "homResidualLayernormF16: hidden size too large");
    return;
  }
  hom::bw::layernorm_f16(reinterpret_cast<const __half *>(X.ptr), r, g, b,
                         reinterpret_cast<__half *>(O.ptr), rows, hidden, eps,
                         hom::current_stream());
}

void homGemmResidualLayernormF16(int64_t rankA, void *dstA, int64_t rankB, void *dstB, bool weightsNK,
                                 int64_t rankR, void *dstR, int64_t rankD, void *dstD, float eps) {
  const char *name = "homGemmResidualLayernormF16";
  hom::gemm::Problem pb;
  bool empty = false;
  const bool has_r = dstR != nullptr && rankR > 0;
  if (!gemm_prepare(name, weightsNK, rankA, dstA, rankB, dstB, rankR, dstR, rankD, dstD, 0, 1.f,
                    has_r ? 1.f : 0.f, &pb, &empty))
    return;
  if (pb.c_mode == 2) {
    set_error(HOM_ERR_UNSUPPORTED, "%s: the residual must have the shape of the output", name);
    return;
  }
  if (!hom::gemm::layernorm_fusion_shape(pb.N, nullptr, nullptr)) {
    set_error(HOM_ERR_UNSUPPORTED,
              "%s: N = %lld does not factor as c x {64,128,192,256} with c in {1,2,4,8}", name,
              static_cast<long long>(pb.N));
    return;
  }
  hom::gemm::run_layernorm_fused(pb, eps, hom::current_stream());
}

// fp32 partial row sums [groups, rows, 2]; absent (rank 0 / null) gives *out = null.
bool partials_operand(const char *name, const char *what, int64_t rank, void *dst, int64_t groups,
                      int64_t rows, float2 **out) {
  *out = nullptr;
  if (dst == nullptr || rank == 0) return true;
  MemRefView v = view_memref(rank, dst, 4);
  if (!v.valid || v.rank != 3 || v.sizes[0] != groups || v.sizes[1] != rows || v.sizes[2] != 2 ||
      !v.contiguous() || (reinterpret_cast<uintptr_t>(v.ptr) & 7u) != 0) {
    set_error(HOM_ERR_INVALID, "%s: %s must be a contiguous fp32 memref of shape [%lld, %lld, 2]", name, what,
              static_cast<long long>(groups), static_cast<long long>(rows));
    return false;
  }
  *out = reinterpret_cast<float2 *>(v.ptr);
  return true;
}

void homGemmDeferredLayernormF16(int64_t rankA, void *dstA, int64_t rankStatsA, void *dstStatsA,
                                 int64_t rankB, void *dstB, bool weightsNK, int64_t rankR, void *dstR,
                                 int64_t rankStatsR, void *dstStatsR, int64_t rankD, void *dstD,
                                 int64_t rankStatsD, void *dstStatsD, int64_t activation, float eps) {
  const char *name = "homGemmDeferredLayernormF16";
  hom::gemm::Problem pb;
  bool empty = false;
  const bool has_r = dstR != nullptr && rankR > 0;
  if (!gemm_prepare(name, weightsNK, rankA, dstA, rankB, dstB, rankR, dstR, rankD, dstD, activation, 1.f,
                    has_r ? 1.f : 0.f, &pb, &empty))
    return;
  if (pb.c_mode == 2 || pb.N % 8 != 0) {
    set_error(HOM_ERR_UNSUPPORTED, "%s: the residual must have the shape of the output and N % 8 == 0", name);
    return;
  }
  float2 *stats_a = nullptr, *stats_r = nullptr, *stats_d = nullptr;
  const int64_t ga = (pb.K + 63) / 64, gd = (pb.N + 63) / 64;
  if (!partials_operand(name, "the statistics of A", rankStatsA, dstStatsA, ga, pb.M, &stats_a) ||
      !partials_operand(name, "the statistics of R", rankStatsR, dstStatsR, gd, pb.M, &stats_r) ||
      !partials_operand(name, "the statistics of D", rankStatsD, dstStatsD, gd, pb.M, &stats_d))
    return;
  if (stats_r && !has_r) {
    set_error(HOM_ERR_INVALID, "%s: statistics of R given without R", name);
    return;
  }
  if (stats_d && (stats_d == stats_r || stats_d == stats_a)) {
    set_error(HOM_ERR_INVALID,
              "%s: the statistics of D must not overwrite those of A or R (other tiles still read them)", name);
    return;
  }
  cudaStream_t stream = hom::current_stream();
  if (stats_a) {
    // LayerNorm(A).B = rstd * (A.B) - mean * rstd * colsum(B): the column sums of a declared
    // weight are computed once and kept, those of any other B on every call.
    const float *sums = pb.b_const ? hom::weight_colsum_lookup(pb.B, pb.K, pb.N) : nullptr;
    if (!sums) {
      float *fresh = nullptr;
      if (pb.b_const) {
        void *ptr = nullptr;
        if (!hom::check_cuda(cudaMalloc(&ptr, static_cast<size_t>(pb.N) * sizeof(float)), "cudaMalloc(column sums)"))
          return;
        fresh = static_cast<float *>(ptr);
      } else {
        if (pb.N > kColSumCapacity) {
          set_error(HOM_ERR_UNSUPPORTED, "%s: N = %lld exceeds the %lld-column scratch", name,
                    static_cast<long long>(pb.N), static_cast<long long>(kColSumCapacity));
          return;
        }
        fresh = col_sum_scratch();
        if (!fresh) return;
      }
      if (!hom::bw::col_sum_f16(pb.B, fresh, pb.K, pb.N, weightsNK, stream)) {
        if (pb.b_const) cudaFree(fresh);
        return;
      }
      if (pb.b_const) {
        if (!hom::check_cuda(cudaStreamSynchronize(stream), "cudaStreamSynchronize(column sums)")) {
          cudaFree(fresh);
          return;
        }
        hom::weight_colsum_insert(pb.B, pb.K, pb.N, fresh);
      }
      sums = fresh;
    }
    pb.col_sum = sums;
    pb.a_partials = stats_a;
    pb.a_groups = static_cast<int>(ga);
  }
  if (stats_r) {
    pb.r_partials = stats_r;
    pb.r_groups = static_cast<int>(gd);
  }
  pb.row_partials = stats_d;
  pb.ln_eps = eps;
  hom::gemm::run(pb, 0, stream);
}

void homBertEmbeddingF16(int64_t rankIds, void *dstIds, int64_t rankTypes, void *dstTypes,
                         int64_t rankWord, void *dstWord, int64_t rankPos, void *dstPos,
                         int64_t rankTypeEmb, void *dstTypeEmb, int64_t rankOut, void *dstOut,
                         float eps) {
  const char *name = "homBertEmbeddingF16";
  MemRefView I = view_memref(rankIds, dstIds, 8), T = view_memref(rankTypes, dstTypes, 8);
  MemRefView W = view_memref(rankWord, dstWord, 2), P = view_memref(rankPos, dstPos, 2);
  MemRefView E = view_memref(rankTypeEmb, dstTypeEmb, 2), O = view_memref(rankOut, dstOut, 2);
  if (!I.valid || !T.valid || !W.valid || !P.valid || !E.valid || !O.valid) {
    set_error(HOM_ERR_INVALID, "%s: null or malformed descriptor", name);
    return;
  }
  if (I.rank != 2 || T.rank != 2 || W.rank != 3 || P.rank != 3 || E.rank != 3 || O.rank != 3 ||
      W.sizes[0] != 1 || P.sizes[0] != 1 || E.sizes[0] != 1) {
    set_error(HOM_ERR_INVALID,
              "%s: expects ids, types [bs,seq]; word [1,V,H], pos [1,seq,H], type [1,T,H]; out [bs,seq,H]",
              name);
    return;
  }
  const int64_t bs = I.sizes[0], seq = I.sizes[1], hidden = O.sizes[2];
  if (T.sizes[0] != bs || T.sizes[1] != seq || O.sizes[0] != bs || O.sizes[1] != seq ||
      W.sizes[2] != hidden || E.sizes[2] != hidden || P.sizes[2] != hidden || P.sizes[1] != seq) {
    set_error(HOM_ERR_INVALID, "%s: shapes of the indices, tables and output do not agree", name);
    return;
  }
  if (!I.contiguous() || !T.contiguous() || !W.contiguous() || !P.contiguous() || !E.contiguous() ||
      !O.contiguous()) {
    set_error(HOM_ERR_INVALID, "%s: operands must be row-major contiguous", name);
    return;
  }
  auto aligned = [](const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
  if (hidden % 8 != 0 || hidden > 4096 || !aligned(W.ptr) || !aligned(P.ptr) || !aligned(E.ptr) ||
      !aligned(O.ptr)) {
    set_error(HOM_ERR_UNSUPPORTED,
              "%s: hidden must be a multiple of 8, at most 4096, and the tables 16-byte aligned", name);
    return;
  }
  hom::bw::embedding_layernorm_f16(
      reinterpret_cast<const int64_t *>(I.ptr), reinterpret_cast<const int64_t *>(T.ptr),
      reinterpret_cast<const __half *>(W.ptr), reinterpret_cast<const __half *>(P.ptr),
      reinterpret_cast<const __half *>(E.ptr), reinterpret_cast<__half *>(O.ptr), bs * seq, seq, hidden,
      W.sizes[1], E.sizes[1], eps, hom::current_stream());
}

void nvteBertAttentionF16(int64_t rankA, void *dstA, int64_t rankSeqlen, void *dstSeqlen,
                          int64_t rankOut, void *dstOut, float scale, int64_t headNum) {
  MemRefView A = view_memref(rankA, dstA, 2), S = view_memref(rankSeqlen, dstSeqlen, 4);
  MemRefView O = view_memref(rankOut, dstOut, 2);
  if (!A.valid || !S.valid || !O.valid) {
    set_error(HOM_ERR_INVALID, "nvteBertAttentionF16: null or malformed descriptor");
    return;
  }
  if (A.rank != 3 || O.rank != 3 || S.rank != 1 || headNum <= 0 ||
      A.sizes[2] % (headNum * 3) != 0 || O.sizes[0] != A.sizes[0] || O.sizes[1] != A.sizes[1] ||
      O.sizes[2] * 3 != A.sizes[2] || S.sizes[0] != A.sizes[0] + 1) {
    set_error(HOM_ERR_INVALID,
              "nvteBertAttentionF16: expects qkv [bs,seq,3*heads*d], cu_seqlens [bs+1], out "
              "[bs,seq,heads*d]");
    return;
  }
  if (!A.contiguous() || !O.contiguous() || !S.contiguous()) {
    set_error(HOM_ERR_INVALID, "nvteBertAttentionF16: operands must be row-major contiguous");
    return;
  }
  const int64_t head_dim = A.sizes[2] / headNum / 3;
  if (head_dim != 64) {
    set_error(HOM_ERR_UNSUPPORTED, "nvteBertAttentionF16: head_dim %lld (only 64 is built)",
              static_cast<long long>(head_dim));
    return;
  }
  if (!(scale > 0.f)) {
    set_error(HOM_ERR_INVALID, "nvteBertAttentionF16: scale must be positive");
    return;
  }
  if (!is_aligned16(A.ptr) || !is_aligned16(O.ptr) || A.sizes[0] > 65535 || headNum > 65535 ||
      A.sizes[0] * A.sizes[1] > INT32_MAX) {
    set_error(HOM_ERR_UNSUPPORTED, "nvteBertAttentionF16: alignment or size limits exceeded");
    return;
  }
  hom::attention::Problem pb;
  pb.bs = A.sizes[0];
  pb.seq = A.sizes[1];
  pb.heads = headNum;
  pb.qkv = reinterpret_cast<const __half *>(A.ptr);
  pb.cu_seqlens = reinterpret_cast<const int *>(S.ptr);
  pb.out = reinterpret_cast<__half *>(O.ptr);
  pb.scale = scale;
  hom::attention::run(pb, hom::current_stream());
}

void nvteBertAttentionF32(int64_t, void *, int64_t, void *, int64_t, void *, float, int64_t) {
  set_error(HOM_ERR_UNSUPPORTED,
            "nvteBertAttentionF32: the lowered pipeline is fp16 only; no fp32 attention is built");
}

HomUnrankedMemRef allocConstantNVGPUF32(int32_t idx) { return alloc_constant<float>(idx); }
HomUnrankedMemRef allocConstantNVGPUF16(int32_t idx) { return alloc_constant<__half>(idx); }

HomUnrankedMemRef alloc3DMemRefNVGPUF32(int32_t a, int32_t b, int32_t c) {
  return alloc_memref({a, b, c}, 4);
}
HomUnrankedMemRef alloc3DMemRefNVGPUF16(int32_t a, int32_t b, int32_t c) {
  return alloc_memref({a, b, c}, 2);
}
HomUnrankedMemRef alloc1DMemRefNVGPUI32(int32_t n) { return alloc_memref({n}, 4); }

void deallocNVGPUF32(int64_t rank, void *dst) { dealloc_memref(rank, dst); }
void deallocNVGPUF16(int64_t rank, void *dst) { dealloc_memref(rank, dst); }
void deallocNVGPUI32(int64_t rank, void *dst) { dealloc_memref(rank, dst); }

#define HOM_ELEMENTWISE_DEF(OPNAME, OPID)                                                         \
  void thrustElementwise##OPNAME##F32(int64_t ra, void *a, int64_t rb, void *b, int64_t ro,       \
                                      void *o) {                                                  \
    elementwise_entry("thrustElementwise" #OPNAME "F32", OPID, false, ra, a, rb, b, ro, o);       \
  }                                                                                               \
  void thrustElementwise##OPNAME##F16(int64_t ra, void *a, int64_t rb, void *b, int64_t ro,       \
                                      void *o) {                                                  \
    elementwise_entry("thrustElementwise" #OPNAME "F16", OPID, true, ra, a, rb, b, ro, o);        \
  }
HOM_ELEMENTWISE_DEF(Add, 0)
HOM_ELEMENTWISE_DEF(Sub, 1)
HOM_ELEMENTWISE_DEF(Mul, 2)
HOM_ELEMENTWISE_DEF(Div, 3)
#undef HOM_ELEMENTWISE_DEF

void thrustGatherF32(int64_t ri, void *i, int64_t rv, void *v, int64_t ro, void *o) {
  gather_entry("thrustGatherF32", false, ri, i, rv, v, ro, o);
}
void thrustGatherF16(int64_t ri, void *i, int64_t rv, void *v, int64_t ro, void *o) {
  gather_entry("thrustGatherF16", true, ri, i, rv, v, ro, o);
}

void thrustCuSeqLenI32(int64_t ri, void *i, int64_t ro, void *o) {
  cu_seqlen_entry("thrustCuSeqLenI32", false, ri, i, ro, o);
}
void thrustCuSeqLenI64(int64_t ri, void *i, int64_t ro, void *o) {
  cu_seqlen_entry("thrustCuSeqLenI64", true, ri, i, ro, o);
}

void printMemrefSizeF32(int64_t rank, void *d) { print_sizes(rank, d); }
void printMemrefSizeF16(int64_t rank, void *d) { print_sizes(rank, d); }
void printMemrefSizeI64(int64_t rank, void *d) { print_sizes(rank, d); }
void printMemrefSizeI32(int64_t rank, void *d) { print_sizes(rank, d); }

#if HOM_DIAG_ENABLED
// Diagnostics only (HOM_GEMM_PROFILE=1 HOM_GEMM_TIMELINE=1): copies the 64-word profile buffer.
__attribute__((visibility("default"))) void homDebugReadGemmProfile(long long *out) {
  long long *buf = hom::gemm::profile_buffer();
  cudaDeviceSynchronize();
  if (buf) cudaMemcpy(out, buf, 64 * sizeof(long long), cudaMemcpyDeviceToHost);
}

__attribute__((visibility("default"))) void homDebugReadProfile(long long *out, int count) {
  long long *buf = hom::gemm::profile_buffer_raw();
  cudaDeviceSynchronize();
  if (buf && count > 0 && count <= 4096) cudaMemcpy(out, buf, count * sizeof(long long), cudaMemcpyDeviceToHost);
}
#endif  // HOM_DIAG_ENABLED

void homSetConstantCache(int enable) { g_constant_cache.store(enable ? 1 : 0); }

void homSetConstantDir(const char *dir) {
  std::lock_guard<std::mutex> lock(g_dir_mutex);
  g_constant_dir = dir ? dir : "";
}

int32_t homGemmQueryTile(int64_t m, int64_t n, int64_t k, int64_t activation, int32_t *bn,
                         int32_t *stages, int32_t *splitK) {
  int b = 0, s = 0, sk = 1;
  const int row = hom::gemm::query_tile(m, n, k, static_cast<int>(activation), &b, &s, &sk);
  if (bn) *bn = b;
  if (stages) *stages = s;
  if (splitK) *splitK = sk;
  return row;
}

int32_t homGemmTune(int64_t m, int64_t n, int64_t k, int64_t activation, float alpha, float beta,
                    int32_t weights_nk, int32_t iterations, int32_t *tile_row, int32_t *split_k,
                    float *best_us, float *row_us) {
  if (activation != 0 && activation != 1) {
    hom::set_error(HOM_ERR_UNSUPPORTED, "homGemmTune: activation %lld is not supported",
                   static_cast<long long>(activation));
    return HOM_ERR_UNSUPPORTED;
  }
  int row = 0, split = 1;
  float us = 0.f;
  if (!hom::gemm::tune(m, n, k, static_cast<int>(activation), alpha, beta, weights_nk != 0, iterations,
                       &row, &split, &us, row_us, hom::current_stream()))
    return homGetLastError() ? homGetLastError() : HOM_ERR_CUDA;
  if (tile_row) *tile_row = row;
  if (split_k) *split_k = split;
  if (best_us) *best_us = us;
  return 0;
}

int32_t homGemmTuneSave(const char *path) { return hom::gemm::tune_cache_save(path); }
int32_t homGemmTuneLoad(const char *path) { return hom::gemm::tune_cache_load(path); }

}  // extern "C"

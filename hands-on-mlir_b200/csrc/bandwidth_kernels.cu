// HBM-bound kernels of the runner-utils layer: LayerNorm (plain in-place and
// residual + affine), elementwise binary ops with B-side broadcast, embedding gather and
// the cu_seqlens prefix sum.  All use 128-bit coalesced accesses where the shape allows
// and warp-shuffle reductions; none uses scratch memory.
//
// They replace TransformerEngine's LayerNorm (include/NVGPUKernels/Layernorm.h:584-694) and
// the Thrust pipelines of include/NVGPUKernels/{ElementwiseRunner,GatherRunner,CuSeqLen}.h.
#include <cstdlib>

#include "bandwidth_kernels.cuh"
#include "hom_diag.cuh"
#include "ptx_sm100.cuh"

namespace hom {
namespace bw {

namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// ---------------------------------------------------------------- LayerNorm

// One warp per row; the row lives in registers as VPT 16-byte vectors per lane.
// y = (x [+ r] - mean) * rsqrt(var + eps) [* gamma] [+ beta]; statistics in fp32 with the
// variance taken around the mean (two passes over registers).
// With EMBED the row is not read from `x` but assembled from three embedding tables:
// word[ids[row]] + type[types[row]], rounded to fp16, + pos[row % seq], rounded to fp16 - the
// values the separate gather / add / add calls would have left in memory - and then normalised
// by the same code, so the fused kernel reproduces the five-call sequence bit for bit.
struct EmbedArgs {
  const long long *ids = nullptr, *types = nullptr;
  const __half *type_emb = nullptr, *pos_emb = nullptr;
  long long vocab = 0, type_vocab = 0;
  int seq = 1;
};

template <int VPT, bool EMBED>
__global__ void __launch_bounds__(512)
layernorm_f16_warp_kernel(const __half *x, const __half *res,
                          const __half *gamma, const __half *beta,
                          __half *out, long long rows, int hidden, float eps, const EmbedArgs emb) {
  hom::ptx::pdl_launch_dependents();
  hom::ptx::pdl_wait();
  const int lane = threadIdx.x & 31;
  const long long row = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int nvec = hidden >> 3;
  const uint4 *xr = reinterpret_cast<const uint4 *>(x + row * hidden);
  const uint4 *rr = res ? reinterpret_cast<const uint4 *>(res + row * hidden) : nullptr;
  const uint4 *tr = nullptr, *pr = nullptr;
  bool word_ok = true, type_ok = true;
  if (EMBED) {
    const long long id = emb.ids[row], ty = emb.types[row];
    word_ok = id >= 0 && id < emb.vocab;  // out-of-range indices read as zero rows, like the gather
    type_ok = ty >= 0 && ty < emb.type_vocab;
    xr = reinterpret_cast<const uint4 *>(x + (word_ok ? id : 0) * hidden);
    tr = reinterpret_cast<const uint4 *>(emb.type_emb + (type_ok ? ty : 0) * hidden);
    pr = reinterpret_cast<const uint4 *>(emb.pos_emb + (row % emb.seq) * hidden);
  }

  float v[VPT][8];
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int vi = lane + 32 * i;
    if (vi < nvec) {
      uint4 raw = xr[vi];
      if (EMBED) {
        const uint4 zero = make_uint4(0, 0, 0, 0);
        if (!word_ok) raw = zero;
        uint4 raw_t = tr[vi];
        if (!type_ok) raw_t = zero;
        const uint4 raw_p = pr[vi];
        __half2 *w2 = reinterpret_cast<__half2 *>(&raw);
        const __half2 *t2 = reinterpret_cast<const __half2 *>(&raw_t);
        const __half2 *p2 = reinterpret_cast<const __half2 *>(&raw_p);
#pragma unroll
        for (int j = 0; j < 4; ++j) w2[j] = __hadd2(__hadd2(w2[j], t2[j]), p2[j]);
      }
      const __half2 *h2 = reinterpret_cast<const __half2 *>(&raw);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __half22float2(h2[j]);
        v[i][2 * j] = f.x;
        v[i][2 * j + 1] = f.y;
      }
      if (rr) {
        const uint4 raw_r = rr[vi];
        const __half2 *r2 = reinterpret_cast<const __half2 *>(&raw_r);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __half22float2(r2[j]);
          v[i][2 * j] += f.x;
          v[i][2 * j + 1] += f.y;
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) sum += v[i][j];
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) v[i][j] = 0.f;
    }
  }
  const float inv_n = 1.f / static_cast<float>(hidden);
  const float mean = warp_sum(sum) * inv_n;
  float sq = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    if (lane + 32 * i < nvec) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float d = v[i][j] - mean;
        sq = fmaf(d, d, sq);
      }
    }
  }
  const float rstd = rsqrtf(warp_sum(sq) * inv_n + eps);

  uint4 *orow = reinterpret_cast<uint4 *>(out + row * hidden);
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int vi = lane + 32 * i;
    if (vi < nvec) {
      float y[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) y[j] = (v[i][j] - mean) * rstd;
      if (gamma) {
        const uint4 raw = reinterpret_cast<const uint4 *>(gamma)[vi];
        const __half2 *g2 = reinterpret_cast<const __half2 *>(&raw);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __half22float2(g2[j]);
          y[2 * j] *= f.x;
          y[2 * j + 1] *= f.y;
        }
      }
      if (beta) {
        const uint4 raw = reinterpret_cast<const uint4 *>(beta)[vi];
        const __half2 *b2 = reinterpret_cast<const __half2 *>(&raw);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __half22float2(b2[j]);
          y[2 * j] += f.x;
          y[2 * j + 1] += f.y;
        }
      }
      uint4 o;
      __half2 *o2 = reinterpret_cast<__half2 *>(&o);
#pragma unroll
      for (int j = 0; j < 4; ++j) o2[j] = __floats2half2_rn(y[2 * j], y[2 * j + 1]);
      orow[vi] = o;
    }
  }
}

// Any hidden size / alignment and fp32 data: one warp per row, scalar strided accesses,
// the row is re-read for each pass.
template <typename T>
__global__ void __launch_bounds__(128)
layernorm_generic_kernel(const T *x, const T *res,
                         const T *gamma, const T *beta,
                         T *out, long long rows, int hidden, float eps) {
  hom::ptx::pdl_launch_dependents();
  hom::ptx::pdl_wait();
  const int lane = threadIdx.x & 31;
  const long long row = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const T *xr = x + row * hidden;
  const T *rr = res ? res + row * hidden : nullptr;
  auto load = [&](int i) {
    float f = static_cast<float>(xr[i]);
    if (rr) f += static_cast<float>(rr[i]);
    return f;
  };
  float sum = 0.f;
  for (int i = lane; i < hidden; i += 32) sum += load(i);
  const float inv_n = 1.f / static_cast<float>(hidden);
  const float mean = warp_sum(sum) * inv_n;
  float sq = 0.f;
  for (int i = lane; i < hidden; i += 32) {
    const float d = load(i) - mean;
    sq = fmaf(d, d, sq);
  }
  const float rstd = rsqrtf(warp_sum(sq) * inv_n + eps);
  // Every lane must have finished reading the row before it is overwritten in place.
  __syncwarp();
  T *orow = out + row * hidden;
  for (int i = lane; i < hidden; i += 32) {
    float y = (load(i) - mean) * rstd;
    if (gamma) y *= static_cast<float>(gamma[i]);
    if (beta) y += static_cast<float>(beta[i]);
    orow[i] = static_cast<T>(y);
  }
}

// ------------------------------------------------ LayerNorm statistics for the fused forms

// One warp per row of x [rows, n]: rstd = 1 / sqrt(E[x^2] - mean^2 + eps) and
// shift = -mean * rstd, stored as fp16 like the reference's finaliser
// (include/NVGPUKernels/Layernorm.h:107-194).
__global__ void __launch_bounds__(128)
row_stats_f16_kernel(const __half *x, __half *rstd_out, __half *shift_out, long long rows, int n,
                     float eps) {
  hom::ptx::pdl_launch_dependents();
  hom::ptx::pdl_wait();
  const int lane = threadIdx.x & 31;
  const long long row = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const __half *xr = x + row * n;
  float sum = 0.f, sq = 0.f;
  if ((n & 7) == 0 && (reinterpret_cast<uintptr_t>(xr) & 15u) == 0) {
    const uint4 *xv = reinterpret_cast<const uint4 *>(xr);
    for (int i = lane; i < (n >> 3); i += 32) {
      const uint4 raw = xv[i];
      const __half2 *h2 = reinterpret_cast<const __half2 *>(&raw);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __half22float2(h2[j]);
        sum += f.x + f.y;
        sq = fmaf(f.x, f.x, fmaf(f.y, f.y, sq));
      }
    }
  } else {
    for (int i = lane; i < n; i += 32) {
      const float f = __half2float(xr[i]);
      sum += f;
      sq = fmaf(f, f, sq);
    }
  }
  sum = warp_sum(sum);
  sq = warp_sum(sq);
  if (lane == 0) {
    const float inv_n = 1.f / static_cast<float>(n);
    const float mean = sum * inv_n;
    const float rstd = rsqrtf(sq * inv_n - mean * mean + eps);
    rstd_out[row] = __float2half_rn(rstd);
    shift_out[row] = __float2half_rn(-mean * rstd);
  }
}

// Finaliser of the row statistics a GEMM epilogue left as per-column-group partial sums
// (partials[g * rows + r] = {sum, sum of squares} of row r over columns [64 g, 64 g + 64)):
// rstd = 1 / sqrt(E[x^2] - mean^2 + eps) and shift = -mean * rstd, stored as fp16 like the
// reference's ApplyFinalReduction (include/NVGPUKernels/Layernorm.h:107-194).
__global__ void __launch_bounds__(256)
row_stats_finalize_kernel(const float2 *partials, int groups, long long rows, int n, float eps,
                          __half *rstd_out, __half *shift_out) {
  hom::ptx::pdl_launch_dependents();
  hom::ptx::pdl_wait();
  const long long r = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (r >= rows) return;
  float sum = 0.f, sq = 0.f;
  for (int g = 0; g < groups; ++g) {
    const float2 v = partials[static_cast<long long>(g) * rows + r];
    sum += v.x;
    sq += v.y;
  }
  const float inv_n = 1.f / static_cast<float>(n);
  const float mean = sum * inv_n;
  const float rstd = rsqrtf(fmaxf(sq * inv_n - mean * mean, 0.f) + eps);
  rstd_out[r] = __float2half_rn(rstd);
  shift_out[r] = __float2half_rn(-mean * rstd);
}

// dst[r, c] = src[r, c] for c < cols, 0 for cols <= c < dst_pitch: a row-major matrix copied to a
// larger row pitch (2-byte accesses: neither side's rows need any alignment).
__global__ void __launch_bounds__(256)
repitch_rows_f16_kernel(const __half *src, __half *dst, long long rows, int cols, int dst_pitch) {
  hom::ptx::pdl_launch_dependents();
  hom::ptx::pdl_wait();
  const long long total = rows * dst_pitch;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / dst_pitch;
    const int c = static_cast<int>(i - r * dst_pitch);
    dst[i] = c < cols ? src[r * cols + c] : __float2half(0.f);
  }
}

// out[n] = sum_k b[k, n] (b is [K, N]) or sum_k b[n, k] (b is [N, K]), fp32.
__global__ void __launch_bounds__(256)
col_sum_f16_kernel(const __half *b, float *out, int k_dim, int n_dim, int b_is_nk) {
  hom::ptx::pdl_launch_dependents();
  hom::ptx::pdl_wait();
  if (b_is_nk) {
    const int lane = threadIdx.x & 31;
    const int n = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (n >= n_dim) return;
    float s = 0.f;
    for (int k = lane; k < k_dim; k += 32) s += __half2float(b[static_cast<long long>(n) * k_dim + k]);
    s = warp_sum(s);
    if (lane == 0) out[n] = s;
  } else {
    const int n = blockIdx.x * blockDim.x + threadIdx.x;
    if (n >= n_dim) return;
    float s = 0.f;
    for (int k = 0; k < k_dim; ++k) s += __half2float(b[static_cast<long long>(k) * n_dim + n]);
    out[n] = s;
  }
}

// -------------------------------------------------------------- elementwise

template <int OP>
__device__ __forceinline__ __half2 apply_h2(__half2 a, __half2 b) {
  if (OP == 0) return __hadd2(a, b);
  if (OP == 1) return __hsub2(a, b);
  if (OP == 2) return __hmul2(a, b);
  return __h2div(a, b);
}
template <int OP>
__device__ __forceinline__ __half apply_h(__half a, __half b) {
  if (OP == 0) return __hadd(a, b);
  if (OP == 1) return __hsub(a, b);
  if (OP == 2) return __hmul(a, b);
  return __hdiv(a, b);
}
template <int OP>
__device__ __forceinline__ float apply_f(float a, float b) {
  if (OP == 0) return a + b;
  if (OP == 1) return a - b;
  if (OP == 2) return a * b;
  return a / b;
}

// out[i] = a[i] op b[i % period] on 16-byte vectors (period counted in vectors).
template <int OP>
__global__ void __launch_bounds__(256)
elementwise_f16_vec_kernel(const uint4 *a, const uint4 *b,
                           uint4 *out, long long nvec, long long period) {
  hom::ptx::pdl_launch_dependents();
  hom::ptx::pdl_wait();
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec;
       i += stride) {
    const uint4 ra = a[i];
    const uint4 rb = b[period == nvec ? i : i % period];
    uint4 ro;
    const __half2 *a2 = reinterpret_cast<const __half2 *>(&ra);
    const __half2 *b2 = reinterpret_cast<const __half2 *>(&rb);
    __half2 *o2 = reinterpret_cast<__half2 *>(&ro);
#pragma unroll
    for (int j = 0; j < 4; ++j) o2[j] = apply_h2<OP>(a2[j], b2[j]);
    out[i] = ro;
  }
}

template <int OP>
__global__ void __launch_bounds__(256)
elementwise_f32_vec_kernel(const float4 *a, const float4 *b,
                           float4 *out, long long nvec, long long period) {
  hom::ptx::pdl_launch_dependents();
  hom::ptx::pdl_wait();
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec;
       i += stride) {
    const float4 ra = a[i];
    const float4 rb = b[period == nvec ? i : i % period];
    float4 ro;
    ro.x = apply_f<OP>(ra.x, rb.x);
    ro.y = apply_f<OP>(ra.y, rb.y);
    ro.z = apply_f<OP>(ra.z, rb.z);
    ro.w = apply_f<OP>(ra.w, rb.w);
    out[i] = ro;
  }
}

// Any broadcast pattern: the flat output index is decomposed over A's row-major strides
// and each coordinate is clamped to B's extent (size 1 => 0), as the reference does
// (ElementwiseRunner.h:101-113).
template <typename T, int OP>
__global__ void __launch_bounds__(256)
elementwise_generic_kernel(const T *a, const T *b, T *out,
                           long long n, BroadcastShape sh) {
  hom::ptx::pdl_launch_dependents();
  hom::ptx::pdl_wait();
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += stride) {
    long long rem = i, bi = 0;
    for (int d = 0; d < sh.rank; ++d) {
      const long long coord = rem / sh.out_stride[d];
      rem -= coord * sh.out_stride[d];
      bi += (coord < sh.b_size[d] ? coord : sh.b_size[d] - 1) * sh.b_stride[d];
    }
    if constexpr (sizeof(T) == 2) {
      out[i] = apply_h<OP>(a[i], b[bi]);
    } else {
      out[i] = apply_f<OP>(a[i], b[bi]);
    }
  }
}

// ------------------------------------------------------------------- gather

// One warp per output row; rows are copied as 16-byte vectors when `vec_per_row` > 0,
// otherwise element by element.  An index outside [0, vocab) yields a zero row.
template <typename T>
__global__ void __launch_bounds__(256)
gather_rows_kernel(const long long *__restrict__ idx, const T *__restrict__ table,
                   T *__restrict__ out, long long rows, long long vocab, int hidden,
                   int vec_per_row) {
  hom::ptx::pdl_launch_dependents();
  hom::ptx::pdl_wait();
  const int lane = threadIdx.x & 31;
  const long long row = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const long long src = idx[row];
  const bool in_range = src >= 0 && src < vocab;
  if (vec_per_row > 0) {
    const uint4 *s = reinterpret_cast<const uint4 *>(table + src * hidden);
    uint4 *d = reinterpret_cast<uint4 *>(out + row * hidden);
    for (int i = lane; i < vec_per_row; i += 32) d[i] = in_range ? s[i] : make_uint4(0, 0, 0, 0);
  } else {
    const T *s = table + src * hidden;
    T *d = out + row * hidden;
    for (int i = lane; i < hidden; i += 32) d[i] = in_range ? s[i] : static_cast<T>(0.f);
  }
}

// --------------------------------------------------------------- cu_seqlens

// Single CTA: warp-per-row sums into out[1..bs], then an in-place inclusive scan.
template <typename T>
__global__ void __launch_bounds__(1024)
cu_seqlen_kernel(const T *__restrict__ mask, int *__restrict__ out, int bs, int seq) {
  hom::ptx::pdl_launch_dependents();
  hom::ptx::pdl_wait();
  __shared__ int warp_tot[32];
  __shared__ int carry_s;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  for (int b = warp; b < bs; b += nwarps) {
    int s = 0;
    const T *row = mask + static_cast<long long>(b) * seq;
    for (int j = lane; j < seq; j += 32) s += static_cast<int>(row[j]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) out[b + 1] = s;
  }
  if (threadIdx.x == 0) {
    out[0] = 0;
    carry_s = 0;
  }
  __syncthreads();
  for (int base = 0; base < bs; base += blockDim.x) {
    const int i = base + threadIdx.x;
    int v = i < bs ? out[i + 1] : 0;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, v, o);
      if (lane >= o) v += t;
    }
    if (lane == 31) warp_tot[warp] = v;
    __syncthreads();
    if (warp == 0) {
      int w = lane < nwarps ? warp_tot[lane] : 0;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, w, o);
        if (lane >= o) w += t;
      }
      warp_tot[lane] = w;  // inclusive totals of warps 0..lane
    }
    __syncthreads();
    const int prefix = carry_s + (warp > 0 ? warp_tot[warp - 1] : 0);
    if (i < bs) out[i + 1] = v + prefix;
    __syncthreads();
    if (threadIdx.x == 0) carry_s += warp_tot[nwarps - 1];
    __syncthreads();
  }
}

inline int grid_for(long long work_items, int per_block) {
  long long blocks = (work_items + per_block - 1) / per_block;
  const long long cap = static_cast<long long>(sm_count()) * 16;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return static_cast<int>(blocks);
}

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace

// ------------------------------------------------------------------ launchers

bool layernorm_f16(const __half *x, const __half *res, const __half *gamma, const __half *beta,
                   __half *out, int64_t rows, int64_t hidden, float eps, cudaStream_t stream) {
  if (rows == 0 || hidden == 0) return true;
  const double bytes = 2.0 * rows * hidden * (2 + (res ? 1 : 0)) +
                       2.0 * hidden * ((gamma ? 1 : 0) + (beta ? 1 : 0));
  LaunchScope scope(kOpLayernorm, 0.0, bytes);
  // One launch wave of few, large blocks starts sooner (measured 4.4 vs 4.8 us at 4096 x 768);
  // with many waves, small blocks retire and refill more evenly (5.27 vs 4.64 TB/s at 131072 rows).
  int warps_per_block = rows <= 8192 ? 16 : 4;
  HOM_DIAG(if (const char *env = std::getenv("HOM_LN_WARPS")) {  // experiment knob
    const int v = std::atoi(env);
    if (v == 4 || v == 8 || v == 16) warps_per_block = v;
  })
  const unsigned blocks = static_cast<unsigned>((rows + warps_per_block - 1) / warps_per_block);
  const unsigned threads = 32u * warps_per_block;
  const bool vec_ok = hidden % 8 == 0 && hidden <= 32 * 8 * 16 && aligned16(x) && aligned16(out) &&
                      (!res || aligned16(res)) && (!gamma || aligned16(gamma)) &&
                      (!beta || aligned16(beta));
  cudaError_t err = cudaSuccess;
  if (vec_ok) {
    const int nvec = static_cast<int>(hidden / 8);
    const int vpt = (nvec + 31) / 32;
#define HOM_LN_CASE(V)                                                                            \
  err = launch_pdl(layernorm_f16_warp_kernel<V, false>, dim3(blocks), dim3(threads), 0, stream, 1, x, \
                   res, gamma, beta, out, static_cast<long long>(rows), static_cast<int>(hidden),  \
                   eps, EmbedArgs{})
    if (vpt <= 1) HOM_LN_CASE(1);
    else if (vpt == 2) HOM_LN_CASE(2);
    else if (vpt == 3) HOM_LN_CASE(3);
    else if (vpt == 4) HOM_LN_CASE(4);
    else if (vpt <= 8) HOM_LN_CASE(8);
    else HOM_LN_CASE(16);
#undef HOM_LN_CASE
  } else {
    err = launch_pdl(layernorm_generic_kernel<__half>, dim3((rows + 3) / 4), dim3(128), 0, stream, 1, x, res,
                     gamma, beta, out, static_cast<long long>(rows), static_cast<int>(hidden), eps);
  }
  return check_cuda(err, "layernorm kernel launch") &&
         check_cuda(cudaGetLastError(), "layernorm kernel launch");
}

bool embedding_layernorm_f16(const int64_t *ids, const int64_t *types, const __half *word_emb,
                             const __half *pos_emb, const __half *type_emb, __half *out, int64_t rows,
                             int64_t seq, int64_t hidden, int64_t vocab, int64_t type_vocab, float eps,
                             cudaStream_t stream) {
  if (rows == 0 || hidden == 0) return true;
  // per row: two indices, three table rows read, one row written
  LaunchScope scope(kOpLayernorm, 0.0, rows * (16.0 + 2.0 * hidden * 4));
  const int warps_per_block = rows <= 8192 ? 16 : 4;
  const unsigned blocks = static_cast<unsigned>((rows + warps_per_block - 1) / warps_per_block);
  const unsigned threads = 32u * warps_per_block;
  EmbedArgs emb;
  emb.ids = reinterpret_cast<const long long *>(ids);
  emb.types = reinterpret_cast<const long long *>(types);
  emb.type_emb = type_emb;
  emb.pos_emb = pos_emb;
  emb.vocab = vocab;
  emb.type_vocab = type_vocab;
  emb.seq = static_cast<int>(seq);
  const __half *none = nullptr;
  const int vpt = (static_cast<int>(hidden / 8) + 31) / 32;
  cudaError_t err = cudaSuccess;
#define HOM_EMB_CASE(V)                                                                           \
  err = launch_pdl(layernorm_f16_warp_kernel<V, true>, dim3(blocks), dim3(threads), 0, stream, 1,  \
                   word_emb, none, none, none, out, static_cast<long long>(rows),                  \
                   static_cast<int>(hidden), eps, emb)
  if (vpt <= 1) HOM_EMB_CASE(1);
  else if (vpt == 2) HOM_EMB_CASE(2);
  else if (vpt == 3) HOM_EMB_CASE(3);
  else if (vpt == 4) HOM_EMB_CASE(4);
  else if (vpt <= 8) HOM_EMB_CASE(8);
  else HOM_EMB_CASE(16);
#undef HOM_EMB_CASE
  return check_cuda(err, "embedding kernel launch");
}

bool layernorm_f32(const float *x, float *out, int64_t rows, int64_t hidden, float eps,
                   cudaStream_t stream) {
  if (rows == 0 || hidden == 0) return true;
  LaunchScope scope(kOpLayernorm, 0.0, 8.0 * rows * hidden);
  const unsigned blocks = static_cast<unsigned>((rows + 3) / 4);
  const float *none = nullptr;
  return check_cuda(launch_pdl(layernorm_generic_kernel<float>, dim3(blocks), dim3(128), 0, stream, 1,
                               x, none, none, none, out, static_cast<long long>(rows),
                               static_cast<int>(hidden), eps),
                    "layernorm kernel launch");
}

template <int OP>
static bool elementwise_dispatch(bool is_f16, const void *a, const void *b, void *out, int64_t n,
                                 int64_t b_period, const BroadcastShape &sh, cudaStream_t stream) {
  const int esize = is_f16 ? 2 : 4;
  const int vec_elems = 16 / esize;
  const bool periodic = b_period > 0;
  const bool vec_ok = periodic && n % vec_elems == 0 && b_period % vec_elems == 0 && aligned16(a) &&
                      aligned16(b) && aligned16(out);
  cudaError_t err = cudaSuccess;
  if (vec_ok) {
    const long long nvec = n / vec_elems, pvec = b_period / vec_elems;
    const int grid = grid_for(nvec, 256);
    if (is_f16)
      err = launch_pdl(elementwise_f16_vec_kernel<OP>, dim3(grid), dim3(256), 0, stream, 1,
                       static_cast<const uint4 *>(a), static_cast<const uint4 *>(b),
                       static_cast<uint4 *>(out), nvec, pvec);
    else
      err = launch_pdl(elementwise_f32_vec_kernel<OP>, dim3(grid), dim3(256), 0, stream, 1,
                       static_cast<const float4 *>(a), static_cast<const float4 *>(b),
                       static_cast<float4 *>(out), nvec, pvec);
  } else {
    const int grid = grid_for(n, 256);
    if (is_f16)
      err = launch_pdl(elementwise_generic_kernel<__half, OP>, dim3(grid), dim3(256), 0, stream, 1,
                       static_cast<const __half *>(a), static_cast<const __half *>(b),
                       static_cast<__half *>(out), static_cast<long long>(n), sh);
    else
      err = launch_pdl(elementwise_generic_kernel<float, OP>, dim3(grid), dim3(256), 0, stream, 1,
                       static_cast<const float *>(a), static_cast<const float *>(b),
                       static_cast<float *>(out), static_cast<long long>(n), sh);
  }
  return check_cuda(err, "elementwise kernel launch");
}

bool elementwise(int op, bool is_f16, const void *a, const void *b, void *out, int64_t n,
                 int64_t b_numel, int64_t b_period, const BroadcastShape &sh,
                 cudaStream_t stream) {
  if (n == 0) return true;
  const double esize = is_f16 ? 2.0 : 4.0;
  LaunchScope scope(kOpElementwise, 0.0, esize * (2.0 * n + b_numel));
  switch (op) {
    case 0: return elementwise_dispatch<0>(is_f16, a, b, out, n, b_period, sh, stream);
    case 1: return elementwise_dispatch<1>(is_f16, a, b, out, n, b_period, sh, stream);
    case 2: return elementwise_dispatch<2>(is_f16, a, b, out, n, b_period, sh, stream);
    default: return elementwise_dispatch<3>(is_f16, a, b, out, n, b_period, sh, stream);
  }
}

bool repitch_rows_f16(const __half *src, __half *dst, int64_t rows, int64_t cols, int64_t dst_pitch,
                      cudaStream_t stream) {
  if (rows == 0 || dst_pitch == 0) return true;
  LaunchScope scope(kOpElementwise, 0.0, 2.0 * rows * (cols + dst_pitch));
  const long long total = rows * dst_pitch;
  const unsigned blocks = static_cast<unsigned>(std::min<long long>((total + 255) / 256, 148 * 16));
  return check_cuda(launch_pdl(repitch_rows_f16_kernel, dim3(blocks), dim3(256), 0, stream, 1, src, dst,
                               static_cast<long long>(rows), static_cast<int>(cols), static_cast<int>(dst_pitch)),
                    "row re-pitch kernel launch");
}

bool row_stats_finalize(const float2 *partials, int groups, int64_t rows, int64_t n, float eps, __half *rstd_out,
                        __half *shift_out, cudaStream_t stream) {
  if (rows == 0) return true;
  LaunchScope scope(kOpLayernorm, 0.0, 8.0 * groups * rows + 4.0 * rows);
  const unsigned blocks = static_cast<unsigned>((rows + 255) / 256);
  return check_cuda(launch_pdl(row_stats_finalize_kernel, dim3(blocks), dim3(256), 0, stream, 1, partials, groups,
                               static_cast<long long>(rows), static_cast<int>(n), eps, rstd_out, shift_out),
                    "row statistics finaliser launch");
}

bool row_stats_f16(const __half *x, __half *rstd_out, __half *shift_out, int64_t rows, int64_t n,
                   float eps, cudaStream_t stream) {
  if (rows == 0 || n == 0) return true;
  LaunchScope scope(kOpLayernorm, 0.0, 2.0 * rows * n + 4.0 * rows);
  const unsigned blocks = static_cast<unsigned>((rows + 3) / 4);
  return check_cuda(launch_pdl(row_stats_f16_kernel, dim3(blocks), dim3(128), 0, stream, 1, x, rstd_out,
                               shift_out, static_cast<long long>(rows), static_cast<int>(n), eps),
                    "row statistics kernel launch");
}

bool col_sum_f16(const __half *b, float *out, int64_t k_dim, int64_t n_dim, bool b_is_nk,
                 cudaStream_t stream) {
  if (n_dim == 0) return true;
  LaunchScope scope(kOpElementwise, 0.0, 2.0 * k_dim * n_dim + 4.0 * n_dim);
  const unsigned blocks = b_is_nk ? static_cast<unsigned>((n_dim + 7) / 8)
                                  : static_cast<unsigned>((n_dim + 255) / 256);
  return check_cuda(launch_pdl(col_sum_f16_kernel, dim3(blocks), dim3(256), 0, stream, 1, b, out,
                               static_cast<int>(k_dim), static_cast<int>(n_dim), b_is_nk ? 1 : 0),
                    "column sum kernel launch");
}

bool gather_rows(bool is_f16, const int64_t *idx, const void *table, void *out, int64_t rows,
                 int64_t vocab, int64_t hidden, cudaStream_t stream) {
  if (rows == 0 || hidden == 0) return true;
  const int esize = is_f16 ? 2 : 4;
  LaunchScope scope(kOpGather, 0.0, 2.0 * esize * rows * hidden + 8.0 * rows);
  const int64_t row_bytes = hidden * esize;
  const int vec = (row_bytes % 16 == 0 && aligned16(table) && aligned16(out))
                      ? static_cast<int>(row_bytes / 16)
                      : 0;
  const unsigned blocks = static_cast<unsigned>((rows + 7) / 8);
  const long long *idx_ll = reinterpret_cast<const long long *>(idx);
  cudaError_t err;
  if (is_f16)
    err = launch_pdl(gather_rows_kernel<__half>, dim3(blocks), dim3(256), 0, stream, 1, idx_ll,
                     static_cast<const __half *>(table), static_cast<__half *>(out),
                     static_cast<long long>(rows), static_cast<long long>(vocab),
                     static_cast<int>(hidden), vec);
  else
    err = launch_pdl(gather_rows_kernel<float>, dim3(blocks), dim3(256), 0, stream, 1, idx_ll,
                     static_cast<const float *>(table), static_cast<float *>(out),
                     static_cast<long long>(rows), static_cast<long long>(vocab),
                     static_cast<int>(hidden), vec);
  return check_cuda(err, "gather kernel launch");
}

bool cu_seqlen(bool is_i64, const void *mask, int *out, int64_t bs, int64_t seq,
               cudaStream_t stream) {
  LaunchScope scope(kOpCuSeqLen, 0.0, (is_i64 ? 8.0 : 4.0) * bs * seq + 4.0 * (bs + 1));
  cudaError_t err;
  if (is_i64)
    err = launch_pdl(cu_seqlen_kernel<long long>, dim3(1), dim3(1024), 0, stream, 1,
                     static_cast<const long long *>(mask), out, static_cast<int>(bs),
                     static_cast<int>(seq));
  else
    err = launch_pdl(cu_seqlen_kernel<int>, dim3(1), dim3(1024), 0, stream, 1,
                     static_cast<const int *>(mask), out, static_cast<int>(bs), static_cast<int>(seq));
  return check_cuda(err, "cu_seqlen kernel launch");
}

}  // namespace bw
}  // namespace hom

// Epilogue arithmetic shared by the GEMM kernels: v = alpha * acc + beta * C, optional erf
// GELU, one rounding to fp16, 128-bit stores.  Everything is evaluated in fp32, like the
// reference's CUTLASS LinearCombination[GELU] epilogue with a float compute type
// (python/hom_manifest.py:43-47).
#pragma once

#include <cuda_fp16.h>
#include <cstdint>

#include "hom_diag.cuh"
#include "ptx_sm100.cuh"

namespace hom {
namespace gemm {

struct EpilogueParams {
  const __half *C;
  long long ldc;
  int c_mode;  // 0: no C, 1: C is [M, N] (may alias D), 2: C is a length-N row broadcast
  __half *D;
  long long ldd;
  float alpha, beta;
  int act;  // 1: erf GELU
  int M, N;
  // Optional LayerNorm-on-A form: the accumulator holds A.B for the raw A and the epilogue
  // applies acc <- row_scale[r] * acc + row_shift[r] * col_sum[n], which equals
  // (A * row_scale + row_shift).B.  All three null when unused.
  const __half *row_scale;
  const __half *row_shift;
  const float *col_sum;
  // Deferred LayerNorm (both null when unused).  `a_partials` / `r_partials` hold, per row, the
  // sums and sums of squares of the raw A rows / raw residual rows per 64-column group
  // ([groups][M] float2, what an earlier GEMM's `row_partials` wrote).  With a_partials the
  // accumulator of the raw A is turned into LayerNorm(A).B (rstd * acc - mean * rstd * col_sum);
  // with r_partials the residual added is LayerNorm(R) = rstd * R - mean * rstd instead of R.
  const float2 *a_partials;
  const float2 *r_partials;
  int a_groups, r_groups;
  float a_inv_n, r_inv_n, ln_eps;
  // 1 when N is not a multiple of 8: rows of C / D are then not 16-byte aligned, so C is read
  // element by element and D is written by the warp from its staging tile with 4- or 2-byte
  // stores instead of a TMA store.
  int unaligned_n;
  // Optional row statistics of D for a following LayerNorm (null when unused): every epilogue
  // warp writes, per output row, the sum and the sum of squares of the fp16-rounded values of
  // its 64-column group to row_partials[group * M + row] (group = column / 64); a small
  // finalising kernel turns them into 1/sqrt(var + eps) and -mean/sqrt(var + eps).  This is what
  // the reference's epilogue visitor does per N-tile (include/NVGPUKernels/Layernorm.h:409-479).
  float2 *row_partials;
  // Diagnostics builds: bit mask that removes parts of the epilogue (1 accumulator read,
  // 2 arithmetic, 4 staging stores, 8 global store, 16 C read, 32 everything but the release).
  HOM_DIAG(int dbg;)
};

// GELU on two values at once for the tile epilogues, built so that the special-function unit
// (16 results per clock per SM) is used once per element instead of twice: with a = min(|x|, 6),
//   GELU(x) = max(x, 0) - a * T(a),   T(a) = erfc(a / sqrt2) / 2 = 2^Q(a),
// where Q is a degree-7 polynomial fitted (Chebyshev nodes on [0, 6], least squares) to
// log2(erfc(a / sqrt2) / 2), evaluated with the packed fp32 FMA of sm_100 (fma.rn.f32x2).
// Beyond |x| = 6 the true tail term is below 6e-9 and the clamped one stays there too.
// Against the exact erf GELU on fp32 inputs over [-12, 12]: max abs error 6.2e-7, max relative
// error 4e-6 where |GELU| > 1e-4; 7 instructions per element.
__device__ __forceinline__ float2 gelu_erf_fast2(float2 x) {
  const float2 a = make_float2(fminf(fabsf(x.x), 6.0f), fminf(fabsf(x.y), 6.0f));
  float2 q = make_float2(-1.889626219e-06f, -1.889626219e-06f);
  q = __ffma2_rn(q, a, make_float2(6.268139987e-05f, 6.268139987e-05f));
  q = __ffma2_rn(q, a, make_float2(-9.388679173e-04f, -9.388679173e-04f));
  q = __ffma2_rn(q, a, make_float2(8.539461531e-03f, 8.539461531e-03f));
  q = __ffma2_rn(q, a, make_float2(-5.402068794e-02f, -5.402068794e-02f));
  q = __ffma2_rn(q, a, make_float2(-4.584097862e-01f, -4.584097862e-01f));
  q = __ffma2_rn(q, a, make_float2(-1.151269197e+00f, -1.151269197e+00f));
  q = __ffma2_rn(q, a, make_float2(-9.999943376e-01f, -9.999943376e-01f));
  float2 t;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(t.x) : "f"(q.x));
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(t.y) : "f"(q.y));
  const float2 relu = make_float2(fmaxf(x.x, 0.f), fmaxf(x.y, 0.f));
  return __ffma2_rn(make_float2(-a.x, -a.y), t, relu);
}

// ---------------------------------------------------------------------------- split-K
// A tile whose K range is cut into `parts` work units is reduced serially, in part order, by
// the epilogue warps that own the same [32 rows x 64 columns] block of the tile in each unit
// (the scheme of a serial split-K semaphore).  The block has one fp32 slot in the workspace and
// one counter that holds the number of parts already folded into the slot:
//   part 0            writes its accumulator block to the slot and sets the counter to 1;
//   part q (0<q<last) waits for counter == q, adds its block to the slot, sets counter = q + 1;
//   the last part     waits for counter == parts - 1, adds the slot to its accumulator (taken
//                     straight from tensor memory), applies the epilogue, resets the counter.
// The sum is therefore always ((p0 + p1) + p2) + ...: bit-identical from run to run.  A part
// only ever waits for parts with a lower unit number; units are handed out in increasing order
// to CTAs that are all resident, so those parts are running or finished: every wait ends (and
// is bounded anyway).  Slot layout is private to the block: chunk j of lane l at float offset
// j * 128 + l * 4, so every load and store instruction moves 512 contiguous bytes.
// The counters are zero whenever no GEMM is in flight (zeroed at allocation, reset after use).
struct SplitK {
  int parts = 1;   // K parts per tile (1: no split)
  int part = 0;    // this unit's part index
  float *slot = nullptr;   // this block's kSplitSlotFloats floats of workspace
  int *counter = nullptr;  // this block's counter
};
constexpr int kSplitSlotFloats = 32 * 64;

// Epilogue warps per CTA and the shared-memory staging each of them owns.  Sixteen warps -
// four per tensor-memory lane quarter, each draining one 64-column group of the tile - put
// four epilogue warps on every scheduler: the epilogue arithmetic (dependent FMA / SFU chains)
// is latency-bound with fewer, and the last tile's drain, which nothing overlaps, is one
// 64-column block per warp instead of two.  Each warp stages its [32 rows x 64 fp16 columns]
// block in one 128-byte-swizzled tile that a TMA store then writes out.
constexpr int kEpilogueWarps = 16;
// Warp 0 is the TMA producer, warp 1 issues the MMAs, the epilogue warps follow.
constexpr int kControlWarps = 2;
constexpr uint32_t kEpilogueTileBytes = 32 * 128;
constexpr uint32_t kEpilogueStageBytes = kEpilogueTileBytes;
constexpr uint32_t kEpilogueStagingBytes = kEpilogueWarps * kEpilogueStageBytes;

// Bits of the FORMS mask of the GEMM kernels and of epilogue_warp_block.
constexpr int kFormLnA = 1, kFormLnR = 2, kFormStats = 4;

// EPI: which of alpha, the C operand and the activation the instantiation handles.  The epilogue
// is bound by instruction issue (every instruction per output element costs a tile about
// elements / 128 cycles), so the three combinations a transformer layer is made of get
// instantiations without the switches of the others; everything else takes the generic one.
//   kEpiPlain  D = A.B                 (alpha 1, no C, no activation)
//   kEpiGelu   D = gelu(A.B)           (alpha 1, no C)
//   kEpiAddC   D = A.B + C             (alpha 1, beta 1, C a matrix or a row vector, no activation)
constexpr int kEpiGeneric = 0, kEpiPlain = 1, kEpiGelu = 2, kEpiAddC = 3;

// Per-row scalars of the LayerNorm forms of the epilogue: acc <- rs * acc + sh * col_sum[n]
// (LayerNorm on A) and c <- rr * c + rt (LayerNorm on the residual); identity when unused.
struct RowAffine {
  float rs = 1.f, sh = 0.f, rr = 1.f, rt = 0.f;
};

__device__ __forceinline__ void row_stats_from_partials(const float2 *partials, int groups, int M, int row,
                                                        float inv_n, float eps, float *rstd, float *shift) {
  // Sixteen independent loads in flight at a time: the partial sums sit in L2 (the previous
  // kernel wrote them), an L2 round trip under the operand stream takes a microsecond or more,
  // and a dependent chain of them would outlast a short main loop.
  float sum = 0.f, sq = 0.f;
  const float2 *src = partials + row;
  for (int g0 = 0; g0 < groups; g0 += 16) {
    float2 v[16];
#pragma unroll
    for (int j = 0; j < 16; ++j)
      v[j] = g0 + j < groups ? __ldcg(src + static_cast<long long>(g0 + j) * M) : make_float2(0.f, 0.f);
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      sum += v[j].x;
      sq += v[j].y;
    }
  }
  const float mean = sum * inv_n;
  const float r = rsqrtf(fmaxf(fmaf(sq, inv_n, -mean * mean), 0.f) + eps);
  *rstd = r;
  *shift = -mean * r;
}

// Called before the accumulator wait so that the loads hide behind the main loop.
__device__ __forceinline__ RowAffine epilogue_row_affine(const EpilogueParams &ep, int row) {
  RowAffine ra;
  if (row >= ep.M HOM_DIAG(|| (ep.dbg & 2048))) return ra;
  if (ep.row_scale != nullptr) {
    ra.rs = __half2float(ep.row_scale[row]);
    ra.sh = __half2float(ep.row_shift[row]);
  } else if (ep.a_partials != nullptr) {
    row_stats_from_partials(ep.a_partials, ep.a_groups, ep.M, row, ep.a_inv_n, ep.ln_eps, &ra.rs, &ra.sh);
  }
  if (ep.r_partials != nullptr)
    row_stats_from_partials(ep.r_partials, ep.r_groups, ep.M, row, ep.r_inv_n, ep.ln_eps, &ra.rr, &ra.rt);
  return ra;
}

// The column sums of B for the 64 columns of a block, spread over the warp: lane l holds those
// of columns c0 + l (x) and c0 + 32 + l (y), zeros beyond N.  The epilogue hands them round with
// shuffles.  A CTA that works through several tiles requests the next tile's pair before it
// starts on the current tile's epilogue: by then the next main loop is usually over, and the
// round trip would be in the open.
__device__ __forceinline__ float2 epilogue_load_col_sums(const EpilogueParams &ep, int c0, int lane) {
  float2 cs = make_float2(0.f, 0.f);
  if (ep.col_sum == nullptr HOM_DIAG(|| (ep.dbg & 4096))) return cs;
  // (L2 loads: both these sums, when B is not a declared weight, and the row statistics above
  // were written by the kernel just before this one)
  if (c0 + lane < ep.N) cs.x = __ldcg(ep.col_sum + c0 + lane);
  if (c0 + 32 + lane < ep.N) cs.y = __ldcg(ep.col_sum + c0 + 32 + lane);
  return cs;
}

// Requests the residual / bias values of one 64-column row segment (row `row`, columns
// [c0, c0 + 64)), or of its 8-column groups [G0, G1) only; out-of-range groups come back as zeros.
template <int G0 = 0, int G1 = 8, bool ALIGNED_ONLY = false>
__device__ __forceinline__ void epilogue_load_c(const EpilogueParams &ep, int row, int c0, uint4 (&cval)[8]) {
  if (ep.c_mode == 0) return;
  HOM_DIAG(if (ep.dbg & 48) {
    for (int g = G0; g < G1; ++g) cval[g] = make_uint4(0, 0, 0, 0);
    return;
  })
  const __half *cp = ep.c_mode == 1 ? ep.C + static_cast<long long>(row) * ep.ldc + c0 : ep.C + c0;
  const bool row_ok = ep.c_mode == 2 || row < ep.M;
  if (!ALIGNED_ONLY && ep.unaligned_n) {
    // element-wise reads, packed in registers (no addressable array: keeps cval out of local memory)
    const unsigned short *cu = reinterpret_cast<const unsigned short *>(cp);
#pragma unroll
    for (int g = G0; g < G1; ++g) {
      uint32_t w[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int i = g * 8 + 2 * j;
        const uint32_t lo = (row_ok && c0 + i < ep.N) ? cu[i] : 0u;
        const uint32_t hi = (row_ok && c0 + i + 1 < ep.N) ? cu[i + 1] : 0u;
        w[j] = lo | (hi << 16);
      }
      cval[g] = make_uint4(w[0], w[1], w[2], w[3]);
    }
    return;
  }
#pragma unroll
  for (int g = G0; g < G1; ++g) {
    const bool ok = row_ok && c0 + g * 8 < ep.N;
    cval[g] = ok ? *reinterpret_cast<const uint4 *>(cp + g * 8) : make_uint4(0, 0, 0, 0);
  }
}

// One warp drains a [32 rows x 64 columns] block of an accumulator: thread `lane` owns output
// row `row0 + lane`.  The block is read from tensor memory in two 32-column halves (keeps the
// live registers below the 112 a 576-thread CTA allows), the epilogue is applied in fp32, the
// fp16 results go into the warp's 128-byte-swizzled staging tile and one lane hands the tile to
// TMA, which writes full 128-byte rows to global memory and clips rows >= M and columns >= N.
// `tmem_addr` already selects the warp's lane quarter and the block's first column.  `cval`
// holds the residual / bias values of the block, requested by the caller (epilogue_load_c)
// before it waited for the accumulator so that their latency hides behind the main loop.
// After the last accumulator read the function calls `release()` (the accumulator may be
// overwritten) while the store drains.  A warp whose column group lies outside the tile
// (`active` false) only releases.
// Returns false only when a split-K wait expired (the CTA's abort flag is then set).
template <bool SPLIT = false, int FORMS = 0, int EPI = 0, typename Release>
__device__ __forceinline__ bool epilogue_warp_block(const EpilogueParams &ep, const CUtensorMap *tmD,
                                                    uint32_t tmem_addr, int row0, int c0, bool active,
                                                    uint32_t stage_smem, int lane, uint4 (&cval)[8],
                                                    Release release, const SplitK sk = SplitK(),
                                                    volatile int *abort_flag = nullptr, int *status = nullptr,
                                                    const RowAffine ra = RowAffine(),
                                                    const float2 col_sums = float2{0.f, 0.f}) {
  using namespace hom::ptx;
  if (!active HOM_DIAG(|| (ep.dbg & 32))) {
    tc_fence_before_sync();
    __syncwarp();
    release();
    return true;
  }
  if constexpr (SPLIT) {
    const bool last = sk.part == sk.parts - 1;
    if (sk.part > 0) {
      // Wait until the parts before this one are in the slot.  One lane polls (with an acquire
      // load); the warp barrier that follows orders the other lanes' slot reads after it.
      bool ok = true;
      if (lane == 0 HOM_DIAG(&& !(ep.dbg & 64))) {
        const long long t0 = clock64();
        for (uint32_t it = 0;; ++it) {
          int have;
          asm volatile("ld.acquire.gpu.global.b32 %0, [%1];" : "=r"(have) : "l"(sk.counter) : "memory");
          if (have >= sk.part) break;
          if ((it & 15u) == 15u && ((abort_flag && *abort_flag) || clock64() - t0 > kWaitLimitCycles)) {
            ok = false;
            break;
          }
          __nanosleep(100);
        }
      }
      __syncwarp();
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        if (lane == 0) {
          if (abort_flag) *abort_flag = 1;
          if (status) {
            atomicCAS(status, 0, static_cast<int>(kDevWaitTimeoutEpilogue));
            __threadfence_system();
          }
        }
        tc_fence_before_sync();
        __syncwarp();
        release();
        return false;
      }
    }
    if (!last) {
      float *slot = sk.slot + lane * 4;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t acc[32];
        tmem_ld_32x32(tmem_addr + half * 32, acc);
        tmem_ld_wait();
        if (half == 1) {
          tc_fence_before_sync();
          __syncwarp();
          release();
        }
        if (sk.part > 0) {
          float4 v[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) v[j] = __ldcg(reinterpret_cast<const float4 *>(slot + (half * 8 + j) * 128));
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            acc[4 * j] = __float_as_uint(v[j].x + __uint_as_float(acc[4 * j]));
            acc[4 * j + 1] = __float_as_uint(v[j].y + __uint_as_float(acc[4 * j + 1]));
            acc[4 * j + 2] = __float_as_uint(v[j].z + __uint_as_float(acc[4 * j + 2]));
            acc[4 * j + 3] = __float_as_uint(v[j].w + __uint_as_float(acc[4 * j + 3]));
          }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j)
          __stcg(reinterpret_cast<uint4 *>(slot + (half * 8 + j) * 128),
                 make_uint4(acc[4 * j], acc[4 * j + 1], acc[4 * j + 2], acc[4 * j + 3]));
      }
      HOM_DIAG(if (!(ep.dbg & 128)))
      __threadfence();
      __syncwarp();
      if (lane == 0) asm volatile("st.release.gpu.global.b32 [%0], %1;" ::"l"(sk.counter), "r"(sk.part + 1) : "memory");
      return true;
    }
    // Last part: every lane has seen the counter; nobody else will touch it before the next launch.
    __syncwarp();
    if (lane == 0) *sk.counter = 0;
  }
  const int row = row0 + lane;
  const uint32_t my_row = stage_smem + lane * 128;
  // The LayerNorm forms exist only in the instantiations whose FORMS mask names them (kFormLnA:
  // LayerNorm on A, kFormLnR: on the residual, kFormStats: statistics of D); inside such an
  // instantiation each is still switched by its pointer.  The plain epilogue (FORMS 0) carries
  // none of their code: the epilogue's instruction footprint is paid at every launch.
  constexpr bool kLnA = (FORMS & kFormLnA) != 0, kLnR = (FORMS & kFormLnR) != 0, kStats = (FORMS & kFormStats) != 0;
  const bool ln_on_a = kLnA && (ep.row_scale != nullptr || ep.a_partials != nullptr);
  const bool ln_on_r = kLnR && ep.r_partials != nullptr;
  const int valid_cols = ep.N - c0;  // columns of this block inside the matrix
  const float2 rs2 = make_float2(ra.rs, ra.rs), sh2 = make_float2(ra.sh, ra.sh);
  const float2 rr2 = make_float2(ra.rr, ra.rr);
  float s1 = 0.f, s2 = 0.f;  // sum and sum of squares of this thread's 64 rounded outputs
  const float2 alpha2 = make_float2(ep.alpha, ep.alpha), beta2 = make_float2(ep.beta, ep.beta);
  const bool unit_alpha = ep.alpha == 1.0f;
  // One 32-column half of the block (both halves unrolled: the second half's accumulator read
  // overlaps the first half's arithmetic).
  auto do_half = [&](const int half) {
    uint32_t acc[32];
#if HOM_DIAG_ENABLED
    if (ep.dbg & 1) {
#pragma unroll
      for (int i = 0; i < 32; ++i) acc[i] = 0x3f000000u + lane;
    } else
#endif
    {
      tmem_ld_32x32(tmem_addr + half * 32, acc);
      tmem_ld_wait();
    }
    if constexpr (SPLIT) {
      // acc <- (p0 + ... + p_{last-1}) + p_last, the left operand being what the slot holds.
      // The residual / bias values of this half are requested together with the slot (the
      // caller fetches nothing ahead of time for a split tile: registers).
      const float *slot = sk.slot + lane * 4 + half * 8 * 128;
      float4 v[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = __ldcg(reinterpret_cast<const float4 *>(slot + j * 128));
      if (half == 0) epilogue_load_c<0, 4>(ep, row, c0, cval);
      else epilogue_load_c<4, 8>(ep, row, c0, cval);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        acc[4 * j] = __float_as_uint(v[j].x + __uint_as_float(acc[4 * j]));
        acc[4 * j + 1] = __float_as_uint(v[j].y + __uint_as_float(acc[4 * j + 1]));
        acc[4 * j + 2] = __float_as_uint(v[j].z + __uint_as_float(acc[4 * j + 2]));
        acc[4 * j + 3] = __float_as_uint(v[j].w + __uint_as_float(acc[4 * j + 3]));
      }
    }
    if (half == 1) {
      tc_fence_before_sync();
      __syncwarp();
      release();
    } else {
      // The staging tile was handed to TMA by this warp's previous block: that read must be over.
      if (lane == 0) bulk_wait_group_read_0();
      __syncwarp();
    }
    if constexpr (kLnA) {
      if (ln_on_a HOM_DIAG(&& !(ep.dbg & 1024))) {
        // acc <- rstd * acc - mean * rstd * col_sum[column]; the shuffles are warp-uniform
        const float mine = half == 0 ? col_sums.x : col_sums.y;
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float2 cs = make_float2(__shfl_sync(0xffffffffu, mine, i), __shfl_sync(0xffffffffu, mine, i + 1));
          const float2 a2 = make_float2(__uint_as_float(acc[i]), __uint_as_float(acc[i + 1]));
          const float2 r = __ffma2_rn(rs2, a2, __fmul2_rn(sh2, cs));
          acc[i] = __float_as_uint(r.x);
          acc[i + 1] = __float_as_uint(r.y);
        }
      }
    }
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      const __half2 *h2 = reinterpret_cast<const __half2 *>(&cval[half * 4 + g]);
      uint32_t w[4];
      // LayerNorm on the residual adds -mean * rstd: not beyond column N, where D stays zero
      const float rt_1 = kLnR && half * 32 + g * 8 < valid_cols ? ra.rt : 0.f;
      const float2 rt_g = make_float2(rt_1, rt_1);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int i0 = g * 8 + 2 * j;
        float2 v = make_float2(__uint_as_float(acc[i0]), __uint_as_float(acc[i0 + 1]));
        HOM_DIAG(if (!(ep.dbg & 2))) {
          if constexpr (EPI == kEpiGeneric) {
            if (!unit_alpha) v = __fmul2_rn(alpha2, v);  // alpha * x is exact for alpha == 1: skip it
          }
          if (EPI == kEpiAddC || (EPI == kEpiGeneric && ep.c_mode != 0)) {
            float2 c = __half22float2(h2[j]);
            if constexpr (kLnR) {
              if (ln_on_r) c = __ffma2_rn(rr2, c, rt_g);
            }
            v = EPI == kEpiAddC ? __fadd2_rn(c, v) : __ffma2_rn(beta2, c, v);
          }
          if (EPI == kEpiGelu || (EPI == kEpiGeneric && ep.act == 1)) v = gelu_erf_fast2(v);
        }
        const __half2 h = __floats2half2_rn(v.x, v.y);
        w[j] = *reinterpret_cast<const uint32_t *>(&h);
        if constexpr (kStats) {
          HOM_DIAG(if (ep.dbg & 256) continue;)
          // statistics of what is stored: the rounded values (columns beyond N hold zeros)
          const float2 q = __half22float2(h);
          s1 += q.x + q.y;
          s2 = fmaf(q.x, q.x, fmaf(q.y, q.y, s2));
        }
      }
      const uint32_t addr = my_row + ((static_cast<uint32_t>(half * 4 + g) ^ (lane & 7u)) << 4);
#if HOM_DIAG_ENABLED
      if (ep.dbg & 4) {
        asm volatile("" ::"r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]));
        continue;
      }
#endif
      asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(w[0]), "r"(w[1]),
                   "r"(w[2]), "r"(w[3])
                   : "memory");
    }
    };
  do_half(0);
  do_half(1);
  if constexpr (kStats) {
    if (ep.row_partials != nullptr && row < ep.M HOM_DIAG(&& !(ep.dbg & 512)))
      ep.row_partials[static_cast<long long>(c0 >> 6) * ep.M + row] = make_float2(s1, s2);
  }
  // (the specialised epilogues and the LayerNorm forms are only chosen when N % 8 == 0)
  if ((EPI != kEpiGeneric || FORMS != 0) || !ep.unaligned_n) {
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) {
      if (c0 < ep.N && row0 < ep.M HOM_DIAG(&& !(ep.dbg & 8))) tma_store_2d(tmD, stage_smem, c0, row0);
      bulk_commit_group();
    }
  } else {
    // Rows of D are not 16-byte aligned: the warp copies its staging tile out row by row,
    // lane l writing columns c0 + 2l, c0 + 2l + 1 (one 128-byte row segment per instruction).
    __syncwarp();
    const int col = c0 + 2 * lane;
    const uint32_t chunk = static_cast<uint32_t>(lane) >> 2, within = (static_cast<uint32_t>(lane) & 3u) << 2;
    for (int r = 0; r < 32; ++r) {
      const int grow = row0 + r;
      if (grow >= ep.M) break;
      uint32_t word;
      asm volatile("ld.shared.b32 %0, [%1];"
                   : "=r"(word)
                   : "r"(stage_smem + r * 128 + ((chunk ^ (static_cast<uint32_t>(r) & 7u)) << 4) + within)
                   : "memory");
      __half *dp = ep.D + static_cast<long long>(grow) * ep.ldd + col;
      if (col + 1 < ep.N && (reinterpret_cast<uintptr_t>(dp) & 3u) == 0) {
        *reinterpret_cast<uint32_t *>(dp) = word;
      } else {
        const __half2 h = *reinterpret_cast<const __half2 *>(&word);
        if (col < ep.N) dp[0] = __low2half(h);
        if (col + 1 < ep.N) dp[1] = __high2half(h);
      }
    }
    __syncwarp();
  }
  return true;
}

// Epilogue of the fused GEMM + residual + LayerNorm kernel.  The CTAs of one cluster hold the
// N / BN column tiles of the same 128 rows, so together they hold whole output rows.
//   pass 1: x = fp16(acc + R) - the value the unfused GEMM would have written - goes into the
//           warp's staging tile, and the thread's sum and sum of squares of its row over the
//           warp's 64 columns go to `stats` (shared memory, [4 column groups][128 rows] float2);
//   cluster barrier; every thread adds up the partials of its row from all column groups of
//           all CTAs of the cluster (distributed shared memory) -> mean and 1/sqrt(var + eps);
//   pass 2: the staged values are normalised in place and the tile is handed to TMA.
// Every thread of the CTA must reach the two cluster barriers: a warp whose column group lies
// outside the tile (`active` false) publishes zeros and only takes part in the barriers; the
// second barrier (keeps `stats` alive while peers read it) is the caller's.
struct LayernormFusion {
  uint32_t stats_smem;  // shared-memory address of this CTA's float2 stats[4][128] + totals[128]
  int cluster_n;        // CTAs per cluster = column tiles per row
  int row_in_tile;      // 32 * lane quarter + lane
  int group;            // this warp's column group
  float eps, inv_n;
};

__device__ __forceinline__ void epilogue_warp_block_ln(const EpilogueParams &ep, const CUtensorMap *tmD,
                                                       uint32_t tmem_addr, int row0, int c0, bool active,
                                                       uint32_t stage_smem, int lane, uint4 (&cval)[8],
                                                       const LayernormFusion &ln) {
  using namespace hom::ptx;
  const uint32_t my_row = stage_smem + lane * 128;
  float s1 = 0.f, s2 = 0.f;
  if (active) {
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      uint32_t acc[32];
      tmem_ld_32x32(tmem_addr + half * 32, acc);
      tmem_ld_wait();
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        const __half2 *h2 = reinterpret_cast<const __half2 *>(&cval[half * 4 + g]);
        uint32_t w[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int i0 = g * 8 + 2 * j;
          float2 v = make_float2(__uint_as_float(acc[i0]), __uint_as_float(acc[i0 + 1]));
          if (ep.c_mode != 0) {
            const float2 r = __half22float2(h2[j]);
            v.x += r.x;
            v.y += r.y;
          }
          const __half2 h = __floats2half2_rn(v.x, v.y);
          const float2 q = __half22float2(h);  // statistics of the rounded values, like the LN kernel sees
          const bool in0 = c0 + half * 32 + i0 < ep.N, in1 = c0 + half * 32 + i0 + 1 < ep.N;
          s1 += (in0 ? q.x : 0.f) + (in1 ? q.y : 0.f);
          s2 = fmaf(in0 ? q.x : 0.f, q.x, s2);
          s2 = fmaf(in1 ? q.y : 0.f, q.y, s2);
          w[j] = *reinterpret_cast<const uint32_t *>(&h);
        }
        const uint32_t addr = my_row + ((static_cast<uint32_t>(half * 4 + g) ^ (lane & 7u)) << 4);
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(w[0]), "r"(w[1]),
                     "r"(w[2]), "r"(w[3])
                     : "memory");
      }
    }
  }
  const uint32_t my_stat = ln.stats_smem + static_cast<uint32_t>(ln.group * 128 + ln.row_in_tile) * 8u;
  asm volatile("st.shared.v2.f32 [%0], {%1, %2};" ::"r"(my_stat), "f"(s1), "f"(s2) : "memory");
  // The sixteen epilogue warps of this CTA meet (named barrier 1), then the warps of column
  // group 0 add up the four partials of their rows: one float2 per row and CTA crosses the
  // cluster instead of four.
  asm volatile("bar.sync 1, 512;" ::: "memory");
  if (ln.group == 0) {
    float c1 = 0.f, c2 = 0.f;
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      float a, b;
      asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];"
                   : "=f"(a), "=f"(b)
                   : "r"(ln.stats_smem + static_cast<uint32_t>(g * 128 + ln.row_in_tile) * 8u)
                   : "memory");
      c1 += a;
      c2 += b;
    }
    asm volatile("st.shared.v2.f32 [%0], {%1, %2};" ::"r"(ln.stats_smem + 4096u + static_cast<uint32_t>(ln.row_in_tile) * 8u),
                 "f"(c1), "f"(c2)
                 : "memory");
  }
  cluster_sync_all();  // the row totals of every CTA of the cluster are published

  float ra[8], rb[8];
#pragma unroll
  for (int cta = 0; cta < 8; ++cta) {
    ra[cta] = 0.f;
    rb[cta] = 0.f;
    if (cta < ln.cluster_n) {
      const uint32_t remote = map_to_cta(ln.stats_smem + 4096u + static_cast<uint32_t>(ln.row_in_tile) * 8u,
                                         static_cast<uint32_t>(cta));
      asm volatile("ld.shared::cluster.v2.f32 {%0, %1}, [%2];" : "=f"(ra[cta]), "=f"(rb[cta]) : "r"(remote) : "memory");
    }
  }
  float t1 = 0.f, t2 = 0.f;
#pragma unroll
  for (int cta = 0; cta < 8; ++cta) {
    t1 += ra[cta];
    t2 += rb[cta];
  }
  const float mean = t1 * ln.inv_n;
  const float var = fmaxf(fmaf(t2, ln.inv_n, -mean * mean), 0.f);
  const float rstd = rsqrtf(var + ln.eps);
  if (!active) return;

#pragma unroll
  for (int chunk = 0; chunk < 8; ++chunk) {
    const uint32_t addr = my_row + ((static_cast<uint32_t>(chunk) ^ (lane & 7u)) << 4);
    uint32_t w[4];
    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3])
                 : "r"(addr)
                 : "memory");
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 q = __half22float2(*reinterpret_cast<const __half2 *>(&w[j]));
      const __half2 h = __floats2half2_rn((q.x - mean) * rstd, (q.y - mean) * rstd);
      w[j] = *reinterpret_cast<const uint32_t *>(&h);
    }
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(w[0]), "r"(w[1]), "r"(w[2]),
                 "r"(w[3])
                 : "memory");
  }
  fence_proxy_async_smem();
  __syncwarp();
  if (lane == 0) {
    if (c0 < ep.N && row0 < ep.M) tma_store_2d(tmD, stage_smem, c0, row0);
    bulk_commit_group();
  }
}

}  // namespace gemm
}  // namespace hom

// Host interface of the sm_100a fp16 GEMM family (gemm_sm100.cu).
#pragma once

#include <cuda.h>

#include "hom_common.cuh"
#include "hom_diag.cuh"

namespace hom {
namespace gemm {

struct Problem {
  int64_t M = 0, N = 0, K = 0;  // M already includes the flattened batch
  const __half *A = nullptr;    // [M, K]
  const __half *B = nullptr;    // [K, N], or [N, K] when b_is_nk
  bool b_is_nk = false;
  // Row pitch of B stored [K, N], in elements (0 = N).  A pitch that is a multiple of 8 lets TMA
  // fetch a B whose N is not (the vocabulary projection, N = 30522).
  int64_t ldb = 0;
  // B lies in a declared constant range: its first tiles may be requested before the previous
  // kernel of the stream has finished.
  bool b_const = false;
  const __half *C = nullptr;
  int c_mode = 0;  // 0 none, 1 full [M, N] (may alias D), 2 length-N row broadcast
  __half *D = nullptr;
  float alpha = 1.f, beta = 0.f;
  int act = 0;  // 1 = erf GELU
  // K parts per output tile: >= 2 as given (clamped to the number of 64-wide K blocks and 16),
  // anything else lets the tile table / tuner / heuristic decide.
  int split_k = 0;
  // LayerNorm-on-A form (all null when unused): D = epilogue(alpha * (A * row_scale + row_shift).B ...)
  // evaluated as row_scale[r] * (A.B)[r,n] + row_shift[r] * col_sum[n] with col_sum = column sums of B.
  const __half *row_scale = nullptr;
  const __half *row_shift = nullptr;
  const float *col_sum = nullptr;
  // Deferred LayerNorm (see EpilogueParams): fp32 per-row partial sums of the raw A ([a_groups][M]
  // float2, needs col_sum) and / or of the raw residual ([r_groups][M] float2).
  const float2 *a_partials = nullptr;
  const float2 *r_partials = nullptr;
  int a_groups = 0, r_groups = 0;
  float ln_eps = 0.f;
  // When set: the epilogue also leaves per-row, per-64-column-group sums and sums of squares of
  // D here ([ceil(N / 64)][M] float2), see EpilogueParams::row_partials.  Forces split_k = 1.
  float2 *row_partials = nullptr;
};

// Which LayerNorm forms the epilogue applies (bits: 1 LayerNorm on A, 2 LayerNorm on the
// residual, 4 statistics of D; the kForm* constants of gemm_epilogue.cuh).  Those forms live in
// their own kernel instantiations and need whole-K tiles (no split-K).
inline int layernorm_forms(const Problem &pb) {
  return ((pb.row_scale != nullptr || pb.a_partials != nullptr) ? 1 : 0) | (pb.r_partials != nullptr ? 2 : 0) |
         (pb.row_partials != nullptr ? 4 : 0);
}
inline bool has_layernorm_form(const Problem &pb) { return layernorm_forms(pb) != 0; }

// Which specialised epilogue fits `pb` (the kEpi* constants of gemm_epilogue.cuh): 1 D = A.B,
// 2 D = gelu(A.B), 3 D = A.B + C, each with alpha = 1 (and beta = 1); 0 the generic one.
inline int epilogue_kind(const Problem &pb) {
  if (pb.alpha != 1.0f || pb.N % 8 != 0) return 0;
  if (pb.c_mode == 0) return pb.act == 0 ? 1 : pb.act == 1 ? 2 : 0;
  return pb.beta == 1.0f && pb.act == 0 ? 3 : 0;
}

// Enqueues the GEMM; tile_row 1..4 forces one CTA per 128 x {64,128,192,256} tile, 5..6 one
// CTA pair per 256 x {128,256} tile; anything else lets the tile table / heuristic decide.
// Returns false (error recorded) on failure.
bool run(const Problem &pb, int tile_row, cudaStream_t stream);
// D = LayerNorm(fp16(A.B + C)) over the last dimension, no affine (C: c_mode 0 or 1; alpha, beta,
// act of `pb` are ignored): the GEMM kernel with one cluster of N-tile CTAs per 128 rows that
// exchange row statistics through distributed shared memory.  N must factor as c x
// {64,128,192,256} with c in {1,2,4,8} (layernorm_fusion_shape).
bool run_layernorm_fused(const Problem &pb, float eps, cudaStream_t stream);
bool layernorm_fusion_shape(int64_t n, int *cluster_n, int *bn);
// The CTA-pair kernels (gemm_pair_sm100.cu); bn2 is 128 or 256.
bool run_pair(const Problem &pb, int bn2, int split_k, cudaStream_t stream);

// The 128 x 128 single-CTA kernel for `pb` (B as [K, N]) launched without any allocation (no
// tensor-map cache insert, no status-word creation).
bool run_fixed_no_alloc(const Problem &pb, cudaStream_t stream);

// Tile-table row and K split for a shape (tuned entry, else table, else cost heuristic).
int select_tile_row(int64_t m, int64_t n, int64_t k, int act, int *split_k = nullptr);
// Split the heuristic would use for a given row.
int select_split(int row, int64_t m, int64_t n, int64_t k, int act);
int query_tile(int64_t m, int64_t n, int64_t k, int act, int *bn, int *stages, int *split_k);

// Run-time tuner (GemmProfiler's contract): times the tile-table rows for one shape, remembers
// the winner for later automatic selections, and can persist the table as text.
bool tune(int64_t m, int64_t n, int64_t k, int act, float alpha, float beta, bool b_is_nk, int iters,
          int *best_row, int *best_split, float *best_us, float *row_us, cudaStream_t stream);
int tuned_row(int64_t m, int64_t n, int64_t k, int act);
bool tuned_choice(int64_t m, int64_t n, int64_t k, int act, int *row, int *split);
int tune_cache_load(const char *path);  // entries read, or -1
int tune_cache_save(const char *path);  // entries written, or -1

#if HOM_DIAG_ENABLED
// Diagnostics builds only (HOM_GEMM_PROFILE=1): per-role cycle counters of CTA 0 and launch
// timelines in a small device buffer.
long long *profile_buffer();
long long *profile_buffer_raw();  // the buffer if it exists; touches nothing
long long *launch_timeline_slot();  // where this launch stamps its CTA entry/exit times
void profile_report(const char *what, int tiles, int grid, int num_kb, cudaStream_t stream);
#endif

// Cached cuTensorMapEncodeTiled for a 2-D fp16 tensor [outer, inner], 128-byte swizzle.
bool make_tensor_map_2d(const void *ptr, uint64_t inner, uint64_t outer, uint32_t box_inner,
                        uint32_t box_outer, CUtensorMap *out, uint64_t pitch = 0);

// Row-major [rows, cols] fp16 matrix, cols % 64 == 0, as (64, rows, cols/64): one box of
// (64, box_rows, groups) becomes `groups` consecutive swizzled [box_rows x 64] sub-tiles.
bool make_tensor_map_grouped(const void *ptr, uint64_t cols, uint64_t rows, uint32_t box_rows,
                             uint32_t groups, CUtensorMap *out);

}  // namespace gemm
}  // namespace hom

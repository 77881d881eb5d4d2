// Host interface of the sm_100a fp16 GEMM family (gemm_sm100.cu).
#pragma once

#include <cuda.h>

#include "hom_common.cuh"

namespace hom {
namespace gemm {

struct Problem {
  int64_t M = 0, N = 0, K = 0;  // M already includes the flattened batch
  const __half *A = nullptr;    // [M, K]
  const __half *B = nullptr;    // [K, N], or [N, K] when b_is_nk
  bool b_is_nk = false;
  const __half *C = nullptr;
  int c_mode = 0;  // 0 none, 1 full [M, N] (may alias D), 2 length-N row broadcast
  __half *D = nullptr;
  float alpha = 1.f, beta = 0.f;
  int act = 0;  // 1 = erf GELU
};

// Enqueues the GEMM; tile_row 1..4 forces the 128 x {64,128,192,256} tile, anything else
// lets the tile table / heuristic decide.  Returns false (error recorded) on failure.
bool run(const Problem &pb, int tile_row, cudaStream_t stream);

int select_bn(int64_t m, int64_t n, int64_t k, int act);
int query_tile(int64_t m, int64_t n, int64_t k, int act, int *bn, int *stages, int *split_k);

// Cached cuTensorMapEncodeTiled for a 2-D fp16 tensor [outer, inner], 128-byte swizzle.
bool make_tensor_map_2d(const void *ptr, uint64_t inner, uint64_t outer, uint32_t box_inner,
                        uint32_t box_outer, CUtensorMap *out);

}  // namespace gemm
}  // namespace hom

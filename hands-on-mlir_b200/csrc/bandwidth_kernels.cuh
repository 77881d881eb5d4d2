// Host interface of the HBM-bound kernels (bandwidth_kernels.cu).
#pragma once

#include "hom_common.cuh"

namespace hom {
namespace bw {

// Shapes for the general broadcast path, passed to the kernel by value.
struct BroadcastShape {
  int rank = 0;
  long long out_stride[HOM_MAX_RANK] = {};  // row-major strides of A / Out
  long long b_size[HOM_MAX_RANK] = {};
  long long b_stride[HOM_MAX_RANK] = {};
};

// out = LayerNorm(x [+ res]) [* gamma] [+ beta]; res/gamma/beta may be null; out may alias x.
bool layernorm_f16(const __half *x, const __half *res, const __half *gamma, const __half *beta,
                   __half *out, int64_t rows, int64_t hidden, float eps, cudaStream_t stream);
// out[row] = LayerNorm(fp16(fp16(word[ids[row]] + type[types[row]]) + pos[row % seq])), no affine:
// the embedding stage of the encoder in one pass.  hidden must be a multiple of 8 and at most
// 4096, all tables 16-byte aligned.
bool embedding_layernorm_f16(const int64_t *ids, const int64_t *types, const __half *word_emb,
                             const __half *pos_emb, const __half *type_emb, __half *out, int64_t rows,
                             int64_t seq, int64_t hidden, int64_t vocab, int64_t type_vocab, float eps,
                             cudaStream_t stream);
bool layernorm_f32(const float *x, float *out, int64_t rows, int64_t hidden, float eps,
                   cudaStream_t stream);

// rstd_out[r] = 1 / sqrt(E[x^2] - mean^2 + eps), shift_out[r] = -mean * rstd over each row of x.
// dst [rows, dst_pitch] <- src [rows, cols] (row-major, zero padding), for any cols.
bool repitch_rows_f16(const __half *src, __half *dst, int64_t rows, int64_t cols, int64_t dst_pitch,
                      cudaStream_t stream);
// Turns the per-64-column-group partial sums a GEMM epilogue left ([groups][rows] float2) into
// rstd / -mean * rstd per row (fp16).
bool row_stats_finalize(const float2 *partials, int groups, int64_t rows, int64_t n, float eps, __half *rstd_out,
                        __half *shift_out, cudaStream_t stream);
bool row_stats_f16(const __half *x, __half *rstd_out, __half *shift_out, int64_t rows, int64_t n,
                   float eps, cudaStream_t stream);
// out[n] = sum over k of B[k, n] (or B[n, k] when b_is_nk), fp32.
bool col_sum_f16(const __half *b, float *out, int64_t k_dim, int64_t n_dim, bool b_is_nk,
                 cudaStream_t stream);

// op: 0 add, 1 sub, 2 mul, 3 div.  b_period > 0 means B repeats every b_period elements of
// the flat output (leading-dimension broadcast or no broadcast); otherwise `sh` is used.
bool elementwise(int op, bool is_f16, const void *a, const void *b, void *out, int64_t n,
                 int64_t b_numel, int64_t b_period, const BroadcastShape &sh, cudaStream_t stream);

bool gather_rows(bool is_f16, const int64_t *idx, const void *table, void *out, int64_t rows,
                 int64_t vocab, int64_t hidden, cudaStream_t stream);

bool cu_seqlen(bool is_i64, const void *mask, int *out, int64_t bs, int64_t seq,
               cudaStream_t stream);

}  // namespace bw
}  // namespace hom

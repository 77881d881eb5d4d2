// Host interface of the sm_100a packed-QKV attention kernel (attention_sm100.cu).
#pragma once

#include "hom_common.cuh"

namespace hom {
namespace attention {

struct Problem {
  int64_t bs = 0, seq = 0, heads = 0;  // head_dim is fixed at 64
  const __half *qkv = nullptr;         // [bs*seq, 3*heads*64], innermost order [3][heads][64]
  const int *cu_seqlens = nullptr;     // [bs + 1] prefix sums of valid lengths
  __half *out = nullptr;               // [bs*seq, heads*64]
  float scale = 0.125f;
};

bool run(const Problem &pb, cudaStream_t stream);
// seq > 128: the persistent kernel that owns two query tiles per CTA (attention_pingpong_sm100.cu).
bool run_pingpong(const Problem &pb, cudaStream_t stream);

}  // namespace attention
}  // namespace hom

// BERT call-sequence replay: the host program a model lowered by Hands-on-MLIR amounts to,
// written by hand because the MLIR toolchain is not available.  It touches tensors only
// through the runner-utils C ABI (hom_nvgpu_runner_utils.h); the CUDA runtime is used for
// stream capture / graph replay and for the host<->device copies of the end-to-end step.
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <vector>

#include <cuda_runtime.h>

#include "hom_bert_replay.h"

namespace {

struct Tensor {
  int64_t rank = 0;
  void *desc = nullptr;  // {basePtr, data, offset, sizes[rank], strides[rank]}
  bool owned_buffer = false;
  bool owned_desc = false;
  const void *declared = nullptr;  // start of the constant range this program declared for it

  void *data() const { return desc ? static_cast<void **>(desc)[1] : nullptr; }
};

Tensor from_alloc(HomUnrankedMemRef m) {
  Tensor t;
  t.rank = m.rank;
  t.desc = m.descriptor;
  t.owned_buffer = t.owned_desc = true;
  return t;
}

// A descriptor over caller-owned or program-owned device memory.
Tensor make_view(void *data, std::initializer_list<int64_t> sizes) {
  Tensor t;
  t.rank = static_cast<int64_t>(sizes.size());
  auto *w = static_cast<int64_t *>(std::malloc(sizeof(int64_t) * (3 + 2 * t.rank)));
  reinterpret_cast<void **>(w)[0] = data;
  reinterpret_cast<void **>(w)[1] = data;
  w[2] = 0;
  int64_t i = 0;
  for (int64_t s : sizes) w[3 + i++] = s;
  int64_t stride = 1;
  for (int64_t d = t.rank - 1; d >= 0; --d) {
    w[3 + t.rank + d] = stride;
    stride *= w[3 + d];
  }
  t.desc = w;
  t.owned_desc = true;
  return t;
}

struct Program {
  HomBertConfig cfg{};
  std::vector<Tensor> weights;
  Tensor x, type_rows, qkv, ctx, ffn, cu;  // activations (hoisted allocations)
  Tensor stats[2];  // fused_layernorm == 2: fp32 row partial sums of the raw hidden states (ping-pong)
  Tensor ids_dev, mask_dev, types_dev;     // staging for the host entry point
  cudaStream_t own_stream = nullptr;
  cudaGraphExec_t graph_exec = nullptr;
  // pipelined host entry point: two device result slots, a copy stream and hand-off events
  Tensor result_slot[2];
  cudaStream_t copy_stream = nullptr;
  cudaEvent_t slot_ready[2] = {nullptr, nullptr};  // result copied into the slot (compute stream)
  cudaEvent_t slot_done[2] = {nullptr, nullptr};   // slot delivered to the host (copy stream)
  bool slot_busy[2] = {false, false};
  unsigned long long host_steps = 0;
  // one graph per slot holding the whole host step: three input copies, the call sequence and
  // the copy of the result into the slot (valid for the host input buffers it was captured on)
  cudaGraphExec_t host_graph[2] = {nullptr, nullptr};
  const void *host_graph_in[2][3] = {{nullptr, nullptr, nullptr}, {nullptr, nullptr, nullptr}};
  void *graph_ids = nullptr, *graph_mask = nullptr, *graph_types = nullptr;
  bool warmed_up = false;
  cudaStream_t warm_stream = nullptr;  // the stream of the latest eager forward
  bool warm_stream_valid = false;
};

void release(Tensor &t, bool f16) {
  if (t.desc) {
    // A caller-owned weight stops being a declared constant with the program: the caller may
    // free or rewrite it afterwards.
    if (t.declared) homForgetWeights(t.declared);
    if (t.owned_buffer) {
      if (f16) deallocNVGPUF16(t.rank, t.desc);
      else deallocNVGPUI32(t.rank, t.desc);
    }
    if (t.owned_desc) std::free(t.desc);
  }
  t = Tensor{};
}

int status() { return homGetLastError(); }

// Staging kernels of the host entry point.  Copy-engine nodes between kernel nodes cost a
// hand-over of tens of microseconds each inside a graph; plain kernels do not.
// Reads the three int64 [batch, seq] planes straight from pinned (device-accessible) host
// memory.
__global__ void stage_inputs_kernel(const long long *ids, const long long *mask, const long long *types,
                                    long long *d_ids, long long *d_mask, long long *d_types, int n) {
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    d_ids[i] = ids[i];
    d_mask[i] = mask[i];
    d_types[i] = types[i];
  }
}

__global__ void copy_u4_kernel(const uint4 *__restrict__ src, uint4 *__restrict__ dst, long long n) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    dst[i] = src[i];
}

// The device-side alias of a pinned host buffer, or null for pageable memory.
const long long *device_alias(const void *host_ptr) {
  cudaPointerAttributes attr;
  if (cudaPointerGetAttributes(&attr, host_ptr) != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  if (attr.type != cudaMemoryTypeHost || !attr.devicePointer) return nullptr;
  return static_cast<const long long *>(attr.devicePointer);
}

// The straight-line call sequence of `_hom_forward`.
int issue_forward(Program &p, int64_t rankIds, void *ids, int64_t rankMask, void *mask,
                  int64_t rankTypes, void *types) {
  const HomBertConfig &c = p.cfg;
  const float scale = 1.0f / std::sqrt(static_cast<float>(c.hidden / c.heads));
  auto gemm = [&](Tensor &a, Tensor &w, Tensor &cmat, Tensor &d, int64_t act, float beta) {
    if (c.weights_nk)
      nvteGemmF16(a.rank, a.desc, false, w.rank, w.desc, true, cmat.rank, cmat.desc, d.rank, d.desc,
                  act, 1.0f, beta, 0, 0);
    else
      cutlassGemmF16(a.rank, a.desc, false, w.rank, w.desc, false, cmat.rank, cmat.desc, d.rank,
                     d.desc, act, 1.0f, beta, 0, 1);
  };
  thrustCuSeqLenI64(rankMask, mask, p.cu.rank, p.cu.desc);
  if (c.fused_embedding) {
    homBertEmbeddingF16(rankIds, ids, rankTypes, types, p.weights[0].rank, p.weights[0].desc,
                        p.weights[1].rank, p.weights[1].desc, p.weights[2].rank, p.weights[2].desc,
                        p.x.rank, p.x.desc, c.eps);
  } else {
    thrustGatherF16(rankIds, ids, p.weights[0].rank, p.weights[0].desc, p.x.rank, p.x.desc);
    thrustGatherF16(rankTypes, types, p.weights[2].rank, p.weights[2].desc, p.type_rows.rank,
                    p.type_rows.desc);
    thrustElementwiseAddF16(p.x.rank, p.x.desc, p.type_rows.rank, p.type_rows.desc, p.x.rank, p.x.desc);
    thrustElementwiseAddF16(p.x.rank, p.x.desc, p.weights[1].rank, p.weights[1].desc, p.x.rank,
                            p.x.desc);
    nvteLayernormF16(p.x.rank, p.x.desc, c.eps);
  }
  if (c.fused_layernorm == 2) {
    // Deferred LayerNorm (homGemmDeferredLayernormF16): from the first output projection on the
    // residual stream `x` stays raw (un-normalised) and travels with the fp32 partial sums of
    // its rows; every consumer applies the LayerNorm in its epilogue - the QKV and FFN1 GEMMs
    // on their A operand, the output projection and FFN2 on their residual - and the two
    // GEMMs that write `x` emit the partial sums of what they write.  No LayerNorm launch
    // inside the layers; one at the very end normalises the last raw `x`.
    Tensor none{};
    int cur = -1;  // which stats buffer describes x (-1: x is normalised, no statistics)
    auto deferred = [&](Tensor &a, Tensor &sa, Tensor &w, Tensor &r, Tensor &sr, Tensor &d, Tensor &sd,
                        int64_t act) {
      homGemmDeferredLayernormF16(a.rank, a.desc, sa.rank, sa.desc, w.rank, w.desc, c.weights_nk != 0, r.rank,
                                  r.desc, sr.rank, sr.desc, d.rank, d.desc, sd.rank, sd.desc, act, c.eps);
    };
    for (int l = 0; l < c.layers; ++l) {
      Tensor &wqkv = p.weights[3 + 4 * l], &wo = p.weights[4 + 4 * l];
      Tensor &w1 = p.weights[5 + 4 * l], &w2 = p.weights[6 + 4 * l];
      Tensor &s_in = cur < 0 ? none : p.stats[cur];
      deferred(p.x, s_in, wqkv, none, none, p.qkv, none, 0);
      nvteBertAttentionF16(p.qkv.rank, p.qkv.desc, p.cu.rank, p.cu.desc, p.ctx.rank, p.ctx.desc, scale,
                           c.heads);
      const int mid = cur < 0 ? 0 : cur ^ 1;
      deferred(p.ctx, none, wo, p.x, s_in, p.x, p.stats[mid], 0);        // x <- ctx.Wo + LN(x), raw
      deferred(p.x, p.stats[mid], w1, none, none, p.ffn, none, 1);       // GELU(LN(x).W1)
      deferred(p.ffn, none, w2, p.x, p.stats[mid], p.x, p.stats[mid ^ 1], 0);  // x <- ffn.W2 + LN(x), raw
      cur = mid ^ 1;
    }
    if (c.layers > 0) nvteLayernormF16(p.x.rank, p.x.desc, c.eps);
    return status();
  }
  for (int l = 0; l < c.layers; ++l) {
    Tensor &wqkv = p.weights[3 + 4 * l], &wo = p.weights[4 + 4 * l];
    Tensor &w1 = p.weights[5 + 4 * l], &w2 = p.weights[6 + 4 * l];
    gemm(p.x, wqkv, p.qkv, p.qkv, 0, 0.0f);
    nvteBertAttentionF16(p.qkv.rank, p.qkv.desc, p.cu.rank, p.cu.desc, p.ctx.rank, p.ctx.desc, scale,
                         c.heads);
    if (c.fused_layernorm) {
      homGemmResidualLayernormF16(p.ctx.rank, p.ctx.desc, wo.rank, wo.desc, c.weights_nk != 0, p.x.rank,
                                  p.x.desc, p.x.rank, p.x.desc, c.eps);
      gemm(p.x, w1, p.ffn, p.ffn, 1, 0.0f);  // erf GELU
      homGemmResidualLayernormF16(p.ffn.rank, p.ffn.desc, w2.rank, w2.desc, c.weights_nk != 0, p.x.rank,
                                  p.x.desc, p.x.rank, p.x.desc, c.eps);
    } else {
      gemm(p.ctx, wo, p.x, p.x, 0, 1.0f);  // residual: C aliases D
      nvteLayernormF16(p.x.rank, p.x.desc, c.eps);
      gemm(p.x, w1, p.ffn, p.ffn, 1, 0.0f);  // erf GELU
      gemm(p.ffn, w2, p.x, p.x, 0, 1.0f);
      nvteLayernormF16(p.x.rank, p.x.desc, c.eps);
    }
  }
  return status();
}

int forward_impl(Program &p, int64_t rankIds, void *ids, int64_t rankMask, void *mask,
                 int64_t rankTypes, void *types, int use_graph) {
  for (const Tensor &w : p.weights)
    if (!w.desc) return HOM_ERR_INVALID;
  if (!use_graph || !p.warmed_up) {
    // The first call always runs eagerly: it performs the library's one-time set-up
    // (kernel attributes, tensor-map cache), which must not happen during capture.
    p.warmed_up = true;
    p.warm_stream = static_cast<cudaStream_t>(homGetStream());
    p.warm_stream_valid = true;
    return issue_forward(p, rankIds, ids, rankMask, mask, rankTypes, types);
  }
  cudaStream_t stream = static_cast<cudaStream_t>(homGetStream());
  void *ids_data = static_cast<void **>(ids)[1], *mask_data = static_cast<void **>(mask)[1];
  void *types_data = static_cast<void **>(types)[1];
  if (p.graph_exec && (ids_data != p.graph_ids || mask_data != p.graph_mask ||
                       types_data != p.graph_types)) {
    cudaGraphExecDestroy(p.graph_exec);
    p.graph_exec = nullptr;
  }
  if (!p.graph_exec) {
    cudaStream_t user_stream = stream;
    if (stream == nullptr) {  // the legacy default stream cannot be captured
      if (!p.own_stream && cudaStreamCreateWithFlags(&p.own_stream, cudaStreamNonBlocking) != cudaSuccess)
        return HOM_ERR_CUDA;
      stream = p.own_stream;
      homSetStream(stream);
    }
    if (p.warm_stream != stream || !p.warm_stream_valid) {
      // Per-stream scratch of the library (the split-K workspace) is allocated on a stream's
      // first use, which must not happen during capture: run once eagerly on this stream.
      const int wrc = issue_forward(p, rankIds, ids, rankMask, mask, rankTypes, types);
      if (wrc != 0) {
        homSetStream(user_stream);
        return wrc;
      }
      p.warm_stream = stream;
      p.warm_stream_valid = true;
    }
    cudaGraph_t graph = nullptr;
    if (cudaStreamBeginCapture(stream, cudaStreamCaptureModeThreadLocal) != cudaSuccess) {
      homSetStream(user_stream);
      return HOM_ERR_CUDA;
    }
    const int rc = issue_forward(p, rankIds, ids, rankMask, mask, rankTypes, types);
    const cudaError_t ce = cudaStreamEndCapture(stream, &graph);
    homSetStream(user_stream);
    if (rc != 0 || ce != cudaSuccess || !graph) {
      if (graph) cudaGraphDestroy(graph);
      return rc ? rc : HOM_ERR_CUDA;
    }
    const cudaError_t ie = cudaGraphInstantiate(&p.graph_exec, graph, 0);
    cudaGraphDestroy(graph);
    if (ie != cudaSuccess) {
      p.graph_exec = nullptr;
      return HOM_ERR_CUDA;
    }
    p.graph_ids = ids_data;
    p.graph_mask = mask_data;
    p.graph_types = types_data;
  }
  return cudaGraphLaunch(p.graph_exec, static_cast<cudaStream_t>(homGetStream())) == cudaSuccess
             ? status()
             : HOM_ERR_CUDA;
}

}  // namespace

extern "C" {

int32_t homBertWeightCount(const HomBertConfig *cfg) { return cfg ? 3 + 4 * cfg->layers : 0; }

void *homBertCreate(const HomBertConfig *cfg) {
  if (!cfg || cfg->layers <= 0 || cfg->hidden <= 0 || cfg->heads <= 0 || cfg->ffn <= 0 ||
      cfg->batch <= 0 || cfg->seq <= 0 || cfg->hidden % cfg->heads != 0)
    return nullptr;
  auto *p = new Program();
  p->cfg = *cfg;
  p->weights.resize(static_cast<size_t>(homBertWeightCount(cfg)));
  const int32_t b = cfg->batch, s = cfg->seq, h = cfg->hidden;
  p->x = from_alloc(alloc3DMemRefNVGPUF16(b, s, h));
  p->type_rows = from_alloc(alloc3DMemRefNVGPUF16(b, s, h));
  p->qkv = from_alloc(alloc3DMemRefNVGPUF16(b, s, 3 * h));
  p->ctx = from_alloc(alloc3DMemRefNVGPUF16(b, s, h));
  p->ffn = from_alloc(alloc3DMemRefNVGPUF16(b, s, cfg->ffn));
  p->cu = from_alloc(alloc1DMemRefNVGPUI32(b + 1));
  if (cfg->fused_layernorm == 2) {
    for (int i = 0; i < 2; ++i) p->stats[i] = from_alloc(alloc3DMemRefNVGPUF32((h + 63) / 64, b * s, 2));
  }
  // int64 staging for the host entry point: 3 x [b, s] carved from one I32 allocation.
  Tensor staging = from_alloc(alloc1DMemRefNVGPUI32(3 * 2 * b * s));
  if (status() != 0 || !p->x.data() || !p->type_rows.data() || !p->qkv.data() || !p->ctx.data() ||
      !p->ffn.data() || !p->cu.data() || !staging.data()) {
    homBertDestroy(p);
    release(staging, false);
    return nullptr;
  }
  char *base = static_cast<char *>(staging.data());
  const int64_t plane = static_cast<int64_t>(b) * s * 8;
  p->ids_dev = make_view(base, {b, s});
  p->mask_dev = make_view(base + plane, {b, s});
  p->types_dev = make_view(base + 2 * plane, {b, s});
  // ids_dev keeps the staging allocation alive and frees it.
  p->ids_dev.owned_buffer = true;
  std::free(staging.desc);
  return p;
}

void homBertDestroy(void *program) {
  auto *p = static_cast<Program *>(program);
  if (!p) return;
  if (p->graph_exec) cudaGraphExecDestroy(p->graph_exec);
  for (int i = 0; i < 2; ++i)
    if (p->host_graph[i]) cudaGraphExecDestroy(p->host_graph[i]);
  if (p->own_stream) cudaStreamDestroy(p->own_stream);
  if (p->copy_stream) {
    cudaStreamSynchronize(p->copy_stream);
    cudaStreamDestroy(p->copy_stream);
  }
  for (int i = 0; i < 2; ++i) {
    if (p->slot_ready[i]) cudaEventDestroy(p->slot_ready[i]);
    if (p->slot_done[i]) cudaEventDestroy(p->slot_done[i]);
    release(p->result_slot[i], true);
  }
  for (Tensor &w : p->weights) release(w, true);
  release(p->x, true);
  release(p->type_rows, true);
  release(p->qkv, true);
  release(p->ctx, true);
  release(p->ffn, true);
  release(p->cu, false);
  for (int i = 0; i < 2; ++i) release(p->stats[i], false);  // fp32: the untyped device free
  release(p->mask_dev, false);
  release(p->types_dev, false);
  release(p->ids_dev, false);
  delete p;
}

int homBertSetWeight(void *program, int32_t index, int64_t rank, void *descriptor) {
  auto *p = static_cast<Program *>(program);
  if (!p || index < 0 || index >= static_cast<int32_t>(p->weights.size()) || !descriptor ||
      rank != 3)
    return HOM_ERR_INVALID;
  release(p->weights[index], true);
  // Copy the descriptor record so the caller's may go away; the buffer stays the caller's.
  const size_t bytes = sizeof(int64_t) * (3 + 2 * rank);
  void *copy = std::malloc(bytes);
  std::memcpy(copy, descriptor, bytes);
  Tensor t;
  t.rank = rank;
  t.desc = copy;
  t.owned_desc = true;
  p->weights[index] = t;
  {
    // The program never writes its weights: let the GEMMs prefetch them early.
    const int64_t *w = static_cast<const int64_t *>(copy);
    int64_t n = 1;
    for (int64_t i = 0; i < rank; ++i) n *= w[3 + i];
    const char *first = reinterpret_cast<const char *>(static_cast<void *const *>(copy)[1]) + 2 * w[2];
    homDeclareWeights(first, 2 * n);
    p->weights[index].declared = first;
  }
  if (p->graph_exec) {
    cudaGraphExecDestroy(p->graph_exec);
    p->graph_exec = nullptr;
  }
  return 0;
}

int homBertLoadConstants(void *program, int32_t first_idx) {
  auto *p = static_cast<Program *>(program);
  if (!p) return HOM_ERR_INVALID;
  for (size_t i = 0; i < p->weights.size(); ++i) {
    release(p->weights[i], true);
    HomUnrankedMemRef m = allocConstantNVGPUF16(first_idx + static_cast<int32_t>(i));
    if (status() != 0 || !m.descriptor) return status() ? status() : HOM_ERR_IO;
    p->weights[i] = from_alloc(m);
  }
  return 0;
}

int homBertForward(void *program, int64_t rankIds, void *ids, int64_t rankMask, void *mask,
                   int64_t rankTypes, void *types, HomUnrankedMemRef *result, int use_graph) {
  auto *p = static_cast<Program *>(program);
  if (!p || !ids || !mask || !types) return HOM_ERR_INVALID;
  const int rc = forward_impl(*p, rankIds, ids, rankMask, mask, rankTypes, types, use_graph);
  if (result) {
    result->rank = p->x.rank;
    result->descriptor = p->x.desc;
  }
  return rc;
}

int homBertForwardHost(void *program, const int64_t *ids_host, const int64_t *mask_host,
                       const int64_t *types_host, void *out_host, int use_graph) {
  auto *p = static_cast<Program *>(program);
  if (!p || !ids_host || !mask_host || !types_host || !out_host) return HOM_ERR_INVALID;
  cudaStream_t stream = static_cast<cudaStream_t>(homGetStream());
  const size_t plane = static_cast<size_t>(p->cfg.batch) * p->cfg.seq * 8;
  if (cudaMemcpyAsync(p->ids_dev.data(), ids_host, plane, cudaMemcpyHostToDevice, stream) != cudaSuccess ||
      cudaMemcpyAsync(p->mask_dev.data(), mask_host, plane, cudaMemcpyHostToDevice, stream) != cudaSuccess ||
      cudaMemcpyAsync(p->types_dev.data(), types_host, plane, cudaMemcpyHostToDevice, stream) != cudaSuccess)
    return HOM_ERR_CUDA;
  const int rc = forward_impl(*p, 2, p->ids_dev.desc, 2, p->mask_dev.desc, 2, p->types_dev.desc,
                              use_graph);
  if (rc != 0) return rc;
  const size_t out_bytes = static_cast<size_t>(p->cfg.batch) * p->cfg.seq * p->cfg.hidden * 2;
  if (cudaMemcpyAsync(out_host, p->x.data(), out_bytes, cudaMemcpyDeviceToHost, stream) != cudaSuccess)
    return HOM_ERR_CUDA;
  return homSynchronize();
}

int homBertForwardHostAsync(void *program, const int64_t *ids_host, const int64_t *mask_host,
                            const int64_t *types_host, void *out_host, int use_graph) {
  auto *p = static_cast<Program *>(program);
  if (!p || !ids_host || !mask_host || !types_host || !out_host) return HOM_ERR_INVALID;
  const HomBertConfig &c = p->cfg;
  if (!p->copy_stream) {
    if (cudaStreamCreateWithFlags(&p->copy_stream, cudaStreamNonBlocking) != cudaSuccess) return HOM_ERR_CUDA;
    for (int i = 0; i < 2; ++i) {
      p->result_slot[i] = from_alloc(alloc3DMemRefNVGPUF16(c.batch, c.seq, c.hidden));
      if (!p->result_slot[i].data() ||
          cudaEventCreateWithFlags(&p->slot_ready[i], cudaEventDisableTiming) != cudaSuccess ||
          cudaEventCreateWithFlags(&p->slot_done[i], cudaEventDisableTiming) != cudaSuccess)
        return HOM_ERR_CUDA;
    }
  }
  cudaStream_t stream = static_cast<cudaStream_t>(homGetStream());
  const int slot = static_cast<int>(p->host_steps & 1);
  // The slot's previous delivery must be over before its device buffer is overwritten.
  if (p->slot_busy[slot] && cudaStreamWaitEvent(stream, p->slot_done[slot], 0) != cudaSuccess)
    return HOM_ERR_CUDA;
  const size_t plane = static_cast<size_t>(c.batch) * c.seq * 8;
  const size_t out_bytes = static_cast<size_t>(c.batch) * c.seq * c.hidden * 2;
  // Input copies, the call sequence and the copy that parks the result in the slot (the
  // hidden-state buffer is reused by the next forward).
  const long long *ids_alias = device_alias(ids_host), *mask_alias = device_alias(mask_host);
  const long long *types_alias = device_alias(types_host);
  const bool pinned_inputs = ids_alias && mask_alias && types_alias;
  auto issue_step = [&]() -> int {
    if (pinned_inputs) {
      const int n = c.batch * c.seq;
      stage_inputs_kernel<<<(n + 255) / 256 < 64 ? (n + 255) / 256 : 64, 256, 0, stream>>>(
          ids_alias, mask_alias, types_alias, static_cast<long long *>(p->ids_dev.data()),
          static_cast<long long *>(p->mask_dev.data()), static_cast<long long *>(p->types_dev.data()), n);
      if (cudaGetLastError() != cudaSuccess) return HOM_ERR_CUDA;
    } else {
      return HOM_ERR_INVALID;
    }
    const int rc = issue_forward(*p, 2, p->ids_dev.desc, 2, p->mask_dev.desc, 2, p->types_dev.desc);
    if (rc != 0) return rc;
    copy_u4_kernel<<<592, 256, 0, stream>>>(static_cast<const uint4 *>(p->x.data()),
                                           static_cast<uint4 *>(p->result_slot[slot].data()),
                                           static_cast<long long>(out_bytes / 16));
    return cudaGetLastError() == cudaSuccess ? 0 : HOM_ERR_CUDA;
  };
  for (const Tensor &w : p->weights)
    if (!w.desc) return HOM_ERR_INVALID;
  if (!pinned_inputs) {
    // Pageable host memory cannot be read by a kernel, and copies from it cannot be captured:
    // copy eagerly, then the (possibly graph-replayed) call sequence and the slot copy.
    if (cudaMemcpyAsync(p->ids_dev.data(), ids_host, plane, cudaMemcpyHostToDevice, stream) != cudaSuccess ||
        cudaMemcpyAsync(p->mask_dev.data(), mask_host, plane, cudaMemcpyHostToDevice, stream) != cudaSuccess ||
        cudaMemcpyAsync(p->types_dev.data(), types_host, plane, cudaMemcpyHostToDevice, stream) != cudaSuccess)
      return HOM_ERR_CUDA;
    const int rc = forward_impl(*p, 2, p->ids_dev.desc, 2, p->mask_dev.desc, 2, p->types_dev.desc, use_graph);
    if (rc != 0) return rc;
    copy_u4_kernel<<<592, 256, 0, static_cast<cudaStream_t>(homGetStream())>>>(
        static_cast<const uint4 *>(p->x.data()), static_cast<uint4 *>(p->result_slot[slot].data()),
        static_cast<long long>(out_bytes / 16));
    if (cudaGetLastError() != cudaSuccess) return HOM_ERR_CUDA;
  } else if (!use_graph || !p->warmed_up || !p->warm_stream_valid || p->warm_stream != stream ||
             stream == nullptr) {
    // eager: also the first call of a program on this stream (one-time and per-stream set-up
    // must not happen during capture) and the legacy default stream, which cannot be captured
    p->warmed_up = true;
    p->warm_stream = stream;
    p->warm_stream_valid = true;
    const int rc = issue_step();
    if (rc != 0) return rc;
  } else {
    const void *in[3] = {ids_host, mask_host, types_host};
    if (p->host_graph[slot] && (in[0] != p->host_graph_in[slot][0] || in[1] != p->host_graph_in[slot][1] ||
                                in[2] != p->host_graph_in[slot][2])) {
      cudaGraphExecDestroy(p->host_graph[slot]);
      p->host_graph[slot] = nullptr;
    }
    if (!p->host_graph[slot]) {
      cudaGraph_t graph = nullptr;
      if (cudaStreamBeginCapture(stream, cudaStreamCaptureModeThreadLocal) != cudaSuccess) return HOM_ERR_CUDA;
      const int rc = issue_step();
      const cudaError_t ce = cudaStreamEndCapture(stream, &graph);
      if (rc != 0 || ce != cudaSuccess || !graph) {
        if (graph) cudaGraphDestroy(graph);
        return rc ? rc : HOM_ERR_CUDA;
      }
      const cudaError_t ie = cudaGraphInstantiate(&p->host_graph[slot], graph, 0);
      cudaGraphDestroy(graph);
      if (ie != cudaSuccess) {
        p->host_graph[slot] = nullptr;
        return HOM_ERR_CUDA;
      }
      for (int i = 0; i < 3; ++i) p->host_graph_in[slot][i] = in[i];
    }
    if (cudaGraphLaunch(p->host_graph[slot], stream) != cudaSuccess) return HOM_ERR_CUDA;
    if (const int rc = status()) return rc;
  }
  // Let the copy stream deliver the slot while the next forward runs.
  if (cudaEventRecord(p->slot_ready[slot], stream) != cudaSuccess ||
      cudaStreamWaitEvent(p->copy_stream, p->slot_ready[slot], 0) != cudaSuccess ||
      cudaMemcpyAsync(out_host, p->result_slot[slot].data(), out_bytes, cudaMemcpyDeviceToHost,
                      p->copy_stream) != cudaSuccess ||
      cudaEventRecord(p->slot_done[slot], p->copy_stream) != cudaSuccess)
    return HOM_ERR_CUDA;
  p->slot_busy[slot] = true;
  ++p->host_steps;
  return 0;
}

int homBertWaitHost(void *program) {
  auto *p = static_cast<Program *>(program);
  if (!p) return HOM_ERR_INVALID;
  if (p->copy_stream && cudaStreamSynchronize(p->copy_stream) != cudaSuccess) return HOM_ERR_CUDA;
  p->slot_busy[0] = p->slot_busy[1] = false;
  return homSynchronize();
}

void homBertHostTraffic(void *program, int64_t *h2d_bytes, int64_t *d2h_bytes) {
  auto *p = static_cast<Program *>(program);
  if (!p) return;
  if (h2d_bytes) *h2d_bytes = 3ll * p->cfg.batch * p->cfg.seq * 8;
  if (d2h_bytes) *d2h_bytes = 2ll * p->cfg.batch * p->cfg.seq * p->cfg.hidden;
}

int32_t homBertLaunchesPerForward(void *program) {
  auto *p = static_cast<Program *>(program);
  if (!p) return 0;
  const int per_layer = p->cfg.fused_layernorm ? 5 : 7;
  const int tail = p->cfg.fused_layernorm == 2 && p->cfg.layers > 0 ? 1 : 0;  // the final LayerNorm
  return (p->cfg.fused_embedding ? 2 : 6) + per_layer * p->cfg.layers + tail;
}

}  // extern "C"

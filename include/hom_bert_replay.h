/* libhom_bert_replay.so: a C++ stand-in for the model library that Hands-on-MLIR compiles
 * from BERT (`_hom_forward`, reached through `_hom_ciface_forward(void**)`,
 * lib/Conversions/Function/UnifyLLVMFuncInterface.cpp:60-128, and driven by
 * examples/torch/bert/bert.cu:81-125).  The MLIR toolchain that would produce the real model
 * library is not available, so this program issues the same straight-line sequence of
 * runner-utils calls that the lowering emits (lib/Conversions/Function/HOMNVGPUToFunc.cpp)
 * and nothing else: every tensor operation goes through the C ABI of
 * hom_nvgpu_runner_utils.h, buffers come from alloc3DMemRefNVGPUF16 / alloc1DMemRefNVGPUI32
 * exactly as the hoisted init function allocates them
 * (lib/Conversions/Function/ExtractInitFunc.cpp:94-186).
 *
 * Per forward: thrustCuSeqLenI64; thrustGatherF16 x2, thrustElementwiseAddF16 x2,
 * nvteLayernormF16 (embeddings); then per encoder layer GEMM(QKV), nvteBertAttentionF16,
 * GEMM(out, C = D = residual, beta 1), nvteLayernormF16, GEMM(FFN1, GELU),
 * GEMM(FFN2, C = D = residual, beta 1), nvteLayernormF16.
 *
 * All functions return 0 on success, otherwise the runner-utils error code
 * (homGetLastErrorString() has the text).  Nothing here has a counterpart symbol in the
 * reference; it replaces a generated artefact.
 */
#ifndef HOM_BERT_REPLAY_H
#define HOM_BERT_REPLAY_H

#include <stdint.h>

#include "hom_nvgpu_runner_utils.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct HomBertConfig {
  int32_t layers;      /* 12 (base) / 24 (large) */
  int32_t hidden;      /* 768 / 1024 */
  int32_t heads;       /* 12 / 16 */
  int32_t ffn;         /* 3072 / 4096 */
  int32_t vocab;       /* 30522 */
  int32_t type_vocab;  /* 2 */
  int32_t batch;       /* sequences per forward on this GPU */
  int32_t seq;
  float eps;           /* 1e-12 */
  int32_t weights_nk;  /* 0: weights [1,K,N] via cutlassGemmF16; 1: [1,N,K] via nvteGemmF16 */
  int32_t fused_embedding; /* 1: homBertEmbeddingF16 in place of the five embedding calls
                              (same bits; not what the reference's lowering emits) */
  int32_t fused_layernorm; /* 0: the reference's call sequence (GEMM, then nvteLayernormF16);
                              1: homGemmResidualLayernormF16 in place of the GEMM + LayerNorm call
                              pairs (out-projection, FFN2); same values within the op tolerance;
                              2: deferred LayerNorm (homGemmDeferredLayernormF16): the residual
                              stream stays raw with fp32 row statistics and every GEMM applies
                              the LayerNorm of its operands in its epilogue - no LayerNorm launch
                              inside the layers, one after the last */
} HomBertConfig;

/* Number of weight tensors a program with this config takes: 3 embeddings + 4 per layer.
 * Order: 0 word_emb [1,vocab,H]; 1 pos_emb [1,seq,H] (the constant-folded position slice);
 * 2 type_emb [1,type_vocab,H]; then per layer wqkv [1,H,3H], wo [1,H,H], w1 [1,H,F],
 * w2 [1,F,H] (each [1,N,K] instead when weights_nk). */
HOM_EXPORT int32_t homBertWeightCount(const HomBertConfig *cfg);

/* Creates the program on the current device and allocates its activation buffers. */
HOM_EXPORT void *homBertCreate(const HomBertConfig *cfg);
HOM_EXPORT void homBertDestroy(void *program);

/* Binds weight `index` to a caller-owned device memref (kept by reference). */
HOM_EXPORT int homBertSetWeight(void *program, int32_t index, int64_t rank, void *descriptor);
/* Loads every weight with allocConstantNVGPUF16(first_idx + index), as the compiled model's
 * init function does; the program owns (and frees) those buffers. */
HOM_EXPORT int homBertLoadConstants(void *program, int32_t first_idx);

/* Enqueues one forward on the library's current stream.  ids / mask / token types are
 * int64 [batch, seq] device memrefs; *result receives the descriptor of the program-owned
 * final hidden states, fp16 [batch, seq, hidden].  use_graph != 0 captures the call sequence
 * into a CUDA graph on first use (for the given input buffers) and replays it afterwards. */
HOM_EXPORT int homBertForward(void *program, int64_t rankIds, void *ids, int64_t rankMask,
                              void *mask, int64_t rankTypes, void *types,
                              HomUnrankedMemRef *result, int use_graph);

/* End-to-end step with HOST buffers: copies ids / mask / token types (int64 [batch, seq],
 * ideally pinned) to the device, runs the forward, copies the fp16 [batch, seq, hidden]
 * result to out_host and waits for it. */
HOM_EXPORT int homBertForwardHost(void *program, const int64_t *ids_host, const int64_t *mask_host,
                                  const int64_t *types_host, void *out_host, int use_graph);

/* The same step without the final wait: the result is parked in one of two device slots and
 * delivered to out_host by a copy stream while the caller already issues the next step.
 * At most two steps are in flight; out_host buffers of consecutive calls must differ.
 * With use_graph != 0 (and a stream set with homSetStream: the default stream cannot be
 * captured) the whole step - input copies, call sequence, copy into the slot - is one CUDA
 * graph per slot, re-captured when the host input pointers change.
 * homBertWaitHost() waits until every issued step has been delivered. */
HOM_EXPORT int homBertForwardHostAsync(void *program, const int64_t *ids_host,
                                       const int64_t *mask_host, const int64_t *types_host,
                                       void *out_host, int use_graph);
HOM_EXPORT int homBertWaitHost(void *program);

/* Bytes moved per homBertForwardHost call (host->device, device->host). */
HOM_EXPORT void homBertHostTraffic(void *program, int64_t *h2d_bytes, int64_t *d2h_bytes);
/* Runner-utils calls (= kernel launches) one forward issues. */
HOM_EXPORT int32_t homBertLaunchesPerForward(void *program);

/* ---- LLVM-free loader for model libraries compiled by Hands-on-MLIR --------------------
 * The calling protocol of the reference's ExecutionEngine
 * (include/ExecutionEngine/ExecutionEngine.h:114-166, lib/ExecutionEngine/ExecutionEngine.cpp:44-97)
 * with dlopen/dlsym only: `_hom_ciface_<fn>_argNum`, `_hom_ciface_<fn>_initFn` (run once, their
 * tensors cached) and `_hom_ciface_<fn>` with the `void **` packing of
 * lib/Conversions/Function/UnifyLLVMFuncInterface.cpp:74-122.
 * `user_slots[i]` points at the i-th scalar argument of <fn> (an unranked memref contributes
 * two slots, &rank and &descriptor); `result_storage` points at storage for the result (a
 * HomUnrankedMemRef for a model returning one tensor).  homModelInvoke returns the runner-utils
 * error code after the call (0 = ok). */
HOM_EXPORT void *homModelOpen(const char *so_path);
HOM_EXPORT int homModelInvoke(void *model, const char *fn, int32_t n_user_slots, void **user_slots,
                              void *result_storage);
/* With enable != 0, homModelInvoke waits for the library's stream after the model function
 * returns and reports what homSynchronize() reports, so that a device-side wait that expired
 * (error 4) reaches the loader's caller; the default (0) returns as soon as the calls are
 * enqueued, like the reference's loader. */
HOM_EXPORT void homModelSetSynchronous(void *model, int enable);
HOM_EXPORT int32_t homModelInitTensorCount(void *model, const char *fn);
HOM_EXPORT const char *homModelLastError(void *model);
HOM_EXPORT void homModelClose(void *model);

#ifdef __cplusplus
}
#endif

#endif /* HOM_BERT_REPLAY_H */

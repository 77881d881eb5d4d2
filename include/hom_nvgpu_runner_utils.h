/* C ABI of libhands_on_mlir_nvgpu_runner_utils.so, the runtime kernel layer that a
 * BERT model lowered by Hands-on-MLIR calls into.
 *
 * Part 1 declares, with identical names and argument lists, every entry point of
 * the reference's include/ExecutionEngine/HandsOnNVGPURunnerUtils.h:70-164 (the
 * symbol names the lowering emits are listed in
 * include/Conversions/Function/FunctionUtils.h:12-49).  A model .so produced by
 * the reference's compiler links against this library unchanged.
 *
 * Part 2 declares additions (prefix `hom`) that have no counterpart in the
 * reference: an error side channel (the reference aborts the process instead),
 * stream selection (the reference always uses the null stream), the
 * residual+affine LayerNorm of the op-level benchmark configuration, and
 * measurement hooks.
 *
 * Conventions shared by all compute entry points:
 *  - tensors are `(int64_t rank, void *descriptor)` pairs, see hom_memref.h;
 *    data must be row-major contiguous; `offset` is honoured.
 *  - work is enqueued on the library's current stream (null stream unless
 *    homSetStream() was called) of the current CUDA device and is not awaited.
 *  - nothing is returned; a rejected call launches nothing and records an error
 *    that homGetLastError() reports.  The process is never aborted.
 */
#ifndef HOM_NVGPU_RUNNER_UTILS_H
#define HOM_NVGPU_RUNNER_UTILS_H

#include <stdbool.h>
#include <stdint.h>

#include "hom_memref.h"

#if defined(__GNUC__)
#define HOM_EXPORT __attribute__((visibility("default")))
#else
#define HOM_EXPORT
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* ===================================================================== Part 1 */

/* D = epilogue(alpha * A.B + beta * C); A [Bs,M,K], B [1,K,N], C/D [Bs,M,N], fp16 in and
 * out, fp32 accumulate and epilogue.  `activation` 1 = erf GELU, 0 = identity.  D may alias C.
 * C may also be [1,1,N] (bias broadcast over rows, as the reference's CPU matmulAddF32 does,
 * lib/ExecutionEngine/HandsOnRunnerUtils.cpp:258-266).  `gemmNum` 1..6 selects a row of the
 * sm_100a tile table (1-4: one CTA per 128 x {64,128,192,256} tile; 5-6: one CTA pair per
 * 256 x {128,256} tile; 0 or any other number = automatic); `splitKFactor` is a hint.
 * Replaces lib/ExecutionEngine/HandsOnNVGPURunnerUtils.cu:104-116 and
 * include/NVGPUKernels/GemmRunner.h:244-310. */
HOM_EXPORT void cutlassGemmF16(int64_t rankA, void *dstA, bool transa, int64_t rankB, void *dstB,
                               bool transb, int64_t rankC, void *dstC, int64_t rankD, void *dstD,
                               int64_t activation, float alpha, float beta, int32_t gemmNum,
                               int32_t splitKFactor);

/* Empty stub in the reference (HandsOnNVGPURunnerUtils.cu:80-102); records "unsupported". */
HOM_EXPORT void cutlassGemmF32(int64_t rankA, void *dstA, bool transa, int64_t rankB, void *dstB,
                               bool transb, int64_t rankC, void *dstC, int64_t rankD, void *dstD,
                               int64_t activation, float alpha, float beta);

/* D = act(A.B^T) (+ D when beta == 1 and C aliases D); A [Bs,M,K], B [1,N,K] with
 * transb == true, transa == false, alpha == 1, beta in {0,1}.  The reference ignores the two
 * trailing integers; here the first is a tile-table row hint like cutlassGemmF16's gemmNum.
 * Replaces HandsOnNVGPURunnerUtils.cu:172-183 and GemmRunner.h:322-426. */
HOM_EXPORT void nvteGemmF16(int64_t rankA, void *dstA, bool transa, int64_t rankB, void *dstB,
                            bool transb, int64_t rankC, void *dstC, int64_t rankD, void *dstD,
                            int64_t activation, float alpha, float beta, int32_t gemmNum,
                            int32_t unused);

/* The GEMM <-> LayerNorm-statistics pair (HandsOnNVGPURunnerUtils.cu:118-170, :191-222;
 * include/NVGPUKernels/LayernormGemmRunner.h, Layernorm.h:107-194).
 * cutlassGemmWithVarMeanF16: D = alpha * A.B + beta * C, then for every row r of D
 *   Var[r] = 1 / sqrt(E[x^2] - mean^2 + eps), Mean[r] = -mean * Var[r]   (fp16, rank 1,
 *   at least Bs*M entries; `activation` is ignored as in the reference).
 * cutlassLayernormGemmF16: D = alpha * (A * Var[r] + Mean[r]).B + beta * C, i.e. the GEMM of
 *   the LayerNorm of A (scale 1, shift 0) with those statistics.
 * Neither is emitted by the compiler for BERT.  cutlassLayernormGemmF32 is an empty stub in
 * the reference and records "unsupported". */
HOM_EXPORT void cutlassGemmWithVarMeanF16(int64_t rankA, void *dstA, int64_t rankB, void *dstB,
                                          int64_t rankC, void *dstC, int64_t rankD, void *dstD,
                                          int64_t rankVar, void *dstVar, int64_t rankMean,
                                          void *dstMean, float alpha, float beta,
                                          int64_t activation, float eps);
HOM_EXPORT void cutlassLayernormGemmF32(int64_t rankA, void *dstA, int64_t rankB, void *dstB,
                                        int64_t rankC, void *dstC, int64_t rankD, void *dstD,
                                        int64_t rankVar, void *dstVar, int64_t rankMean,
                                        void *dstMean, float alpha, float beta,
                                        int64_t activation);
HOM_EXPORT void cutlassLayernormGemmF16(int64_t rankA, void *dstA, int64_t rankB, void *dstB,
                                        int64_t rankC, void *dstC, int64_t rankD, void *dstD,
                                        int64_t rankVar, void *dstVar, int64_t rankMean,
                                        void *dstMean, float alpha, float beta,
                                        int64_t activation);

/* In-place x <- (x - mean) * rsqrt(var + eps) over the last dimension, biased variance,
 * fp32 statistics, no affine; rank 2 or 3.
 * Replaces HandsOnNVGPURunnerUtils.cu:300-310 and include/NVGPUKernels/Layernorm.h:584-694. */
HOM_EXPORT void nvteLayernormF32(int64_t rankA, void *dstA, float eps);
HOM_EXPORT void nvteLayernormF16(int64_t rankA, void *dstA, float eps);

/* O = softmax(scale * Q.K^T + padding mask).V per (batch, head), bidirectional.
 * A = packed QKV [bs, seq, 3*heads*d] with innermost order [3][heads][d];
 * Seqlen = int32 [bs+1] prefix sums of valid lengths; Out [bs, seq, heads*d].
 * Rows at padded query positions are written as zeros.
 * Replaces HandsOnNVGPURunnerUtils.cu:312-328 and
 * include/NVGPUKernels/BertAttentionRunner.h:19-137. */
HOM_EXPORT void nvteBertAttentionF32(int64_t rankA, void *dstA, int64_t rankSeqlen,
                                     void *dstSeqlen, int64_t rankOut, void *dstOut, float scale,
                                     int64_t headNum);
HOM_EXPORT void nvteBertAttentionF16(int64_t rankA, void *dstA, int64_t rankSeqlen,
                                     void *dstSeqlen, int64_t rankOut, void *dstOut, float scale,
                                     int64_t headNum);

/* Device allocation.  The descriptor is malloc()ed (callers free() it); the buffer is
 * released by dealloc*.  allocConstant* reads "<dir>/<idx>.txt" (first line: three
 * dimensions; then the values as text) and uploads it, converting to fp16 with
 * round-to-nearest-even for the F16 variant.
 * Replaces HandsOnNVGPURunnerUtils.cu:224-355 and allocHelper,
 * include/ExecutionEngine/HandsOnRunnerUtils.h:46-73. */
HOM_EXPORT HomUnrankedMemRef allocConstantNVGPUF32(int32_t idx);
HOM_EXPORT HomUnrankedMemRef allocConstantNVGPUF16(int32_t idx);
HOM_EXPORT HomUnrankedMemRef alloc3DMemRefNVGPUF32(int32_t a, int32_t b, int32_t c);
HOM_EXPORT HomUnrankedMemRef alloc3DMemRefNVGPUF16(int32_t a, int32_t b, int32_t c);
HOM_EXPORT HomUnrankedMemRef alloc1DMemRefNVGPUI32(int32_t n);
HOM_EXPORT void deallocNVGPUF32(int64_t rank, void *dst);
HOM_EXPORT void deallocNVGPUF16(int64_t rank, void *dst);
HOM_EXPORT void deallocNVGPUI32(int64_t rank, void *dst);

/* Out = A op B; same rank; B may have size-1 (broadcast) dimensions; arithmetic in the
 * element type.  Replaces HandsOnNVGPURunnerUtils.cu:357-365 and
 * include/NVGPUKernels/ElementwiseRunner.h:120-153. */
HOM_EXPORT void thrustElementwiseAddF32(int64_t, void *, int64_t, void *, int64_t, void *);
HOM_EXPORT void thrustElementwiseSubF32(int64_t, void *, int64_t, void *, int64_t, void *);
HOM_EXPORT void thrustElementwiseMulF32(int64_t, void *, int64_t, void *, int64_t, void *);
HOM_EXPORT void thrustElementwiseDivF32(int64_t, void *, int64_t, void *, int64_t, void *);
HOM_EXPORT void thrustElementwiseAddF16(int64_t, void *, int64_t, void *, int64_t, void *);
HOM_EXPORT void thrustElementwiseSubF16(int64_t, void *, int64_t, void *, int64_t, void *);
HOM_EXPORT void thrustElementwiseMulF16(int64_t, void *, int64_t, void *, int64_t, void *);
HOM_EXPORT void thrustElementwiseDivF16(int64_t, void *, int64_t, void *, int64_t, void *);

/* out[b,s,:] = table[0, indices[b,s], :]; indices int64 [bs,seq]; table [1,V,H].
 * Replaces HandsOnNVGPURunnerUtils.cu:367-368 and include/NVGPUKernels/GatherRunner.h:46-77. */
HOM_EXPORT void thrustGatherF32(int64_t rankIndices, void *desIndices, int64_t rankValue,
                                void *desValue, int64_t rankOut, void *desOut);
HOM_EXPORT void thrustGatherF16(int64_t rankIndices, void *desIndices, int64_t rankValue,
                                void *desValue, int64_t rankOut, void *desOut);

/* out[0] = 0; out[b+1] = sum over rows <= b of sum_j mask[row][j]; mask [bs,seq] int32/int64,
 * out int32 [bs+1].  Replaces HandsOnNVGPURunnerUtils.cu:370-371 and
 * include/NVGPUKernels/CuSeqLen.h:48-74. */
HOM_EXPORT void thrustCuSeqLenI32(int64_t rankInput, void *desInput, int64_t rankOut, void *desOut);
HOM_EXPORT void thrustCuSeqLenI64(int64_t rankInput, void *desInput, int64_t rankOut, void *desOut);

/* Prints "Print inside: <sizes>" to stderr (HandsOnNVGPURunnerUtils.h:58-68). */
HOM_EXPORT void printMemrefSizeF32(int64_t rank, void *descriptor);
HOM_EXPORT void printMemrefSizeF16(int64_t rank, void *descriptor);
HOM_EXPORT void printMemrefSizeI64(int64_t rank, void *descriptor);
HOM_EXPORT void printMemrefSizeI32(int64_t rank, void *descriptor);

/* ===================================================================== Part 2 */

/* Error side channel (per host thread).  Codes: 0 ok, 1 invalid argument, 2 unsupported,
 * 3 CUDA runtime error, 4 device-side wait expired, 5 I/O error. */
enum {
  HOM_OK = 0,
  HOM_ERR_INVALID = 1,
  HOM_ERR_UNSUPPORTED = 2,
  HOM_ERR_CUDA = 3,
  HOM_ERR_DEVICE_TIMEOUT = 4,
  HOM_ERR_IO = 5
};
HOM_EXPORT int homGetLastError(void);
HOM_EXPORT const char *homGetLastErrorString(void);
HOM_EXPORT void homClearLastError(void);

/* Stream used by this host thread's subsequent calls (a cudaStream_t; NULL = null stream). */
HOM_EXPORT void homSetStream(void *stream);
HOM_EXPORT void *homGetStream(void);
/* Waits for the stream, then folds the device status word into the error channel.
 * Returns the error code. */
HOM_EXPORT int homSynchronize(void);

/* Declares that no kernel will write [ptr, ptr + bytes) while GEMMs read it as their B operand
 * (model weights).  Kernels of this library are launched so that one may start while the previous
 * kernel of the stream is still finishing; a GEMM requests its first tiles of a DECLARED B before
 * that previous kernel is known to be complete, and those of any other B only afterwards, so a B
 * that an earlier call on the stream produced is always read after it was written.  Buffers
 * returned by allocConstantNVGPU* are declared by the library; callers that bring their own
 * weight buffers may declare them to get the earlier prefetch.  homForgetWeights() withdraws a
 * declaration (call it before the buffer is freed or reused).  What the library derives from a
 * declared weight and keeps (a re-pitched copy for N % 8 != 0, column sums for the deferred
 * LayerNorm) is dropped when the weight is forgotten and when it is declared again: declare a
 * buffer again after rewriting its contents.  No counterpart in the reference, whose launches
 * are fully serialised on the null stream. */
HOM_EXPORT void homDeclareWeights(const void *ptr, int64_t bytes);
HOM_EXPORT void homForgetWeights(const void *ptr);

/* Directory that allocConstantNVGPU* reads "<idx>.txt" from (default: $HOM_CONSTANT_DIR,
 * else the current directory). */
HOM_EXPORT void homSetConstantDir(const char *dir);
/* Opt-in binary cache of parsed constants: with enable != 0 (or HOM_CONSTANT_CACHE=1)
 * allocConstantNVGPU* writes `<idx>.txt.homcache` (parsed fp32 values) beside the text file on
 * first use and reads it afterwards while the text file's size and modification time are
 * unchanged.  A weight directory that cannot be written just runs uncached. */
HOM_EXPORT void homSetConstantCache(int enable);

/* D = LayerNorm(fp16(A.B + R)) over the last dimension, no affine: what a GEMM with the
 * residual as C (beta 1) followed by nvteLayernormF16 leaves in D, in one launch.  The CTAs that
 * hold the column tiles of the same 128 rows form a thread-block cluster and exchange their row
 * sums through distributed shared memory, so the normalised rows are the only thing written.
 * A [.., M, K] fp16; B [1, K, N] (weightsNK false) or [1, N, K] (true); R [.., M, N] or a rank-0
 * descriptor (absent), may alias D; N must be c x {64,128,192,256} with c in {1,2,4,8} (256, 512,
 * 768, 1024, 1536, 2048, ...).  Statistics in fp32 from the fp16-rounded values (sum and sum of
 * squares).  No counterpart in the reference: it fuses the call pairs out-projection + LayerNorm
 * and FFN2 + LayerNorm of the lowered encoder layer. */
HOM_EXPORT void homGemmResidualLayernormF16(int64_t rankA, void *dstA, int64_t rankB, void *dstB,
                                            bool weightsNK, int64_t rankR, void *dstR, int64_t rankD,
                                            void *dstD, float eps);

/* The embedding stage of the lowered BERT in one launch: what the five calls
 * thrustGatherF16(ids, word) ; thrustGatherF16(types, typeEmb) ; thrustElementwiseAddF16 x2 ;
 * nvteLayernormF16 leave in Out, bit for bit (each fp16 addition rounded, fp32 statistics, no
 * affine).  ids, types int64 [bs,seq]; word [1,V,H], pos [1,seq,H], typeEmb [1,T,H], Out
 * [bs,seq,H] fp16; out-of-range indices read as zero rows.  No counterpart in the reference:
 * a compiler pass would have to emit it in place of the five calls. */
HOM_EXPORT void homBertEmbeddingF16(int64_t rankIds, void *dstIds, int64_t rankTypes, void *dstTypes,
                                    int64_t rankWord, void *dstWord, int64_t rankPos, void *dstPos,
                                    int64_t rankTypeEmb, void *dstTypeEmb, int64_t rankOut,
                                    void *dstOut, float eps);

/* GEMM with the LayerNorms around it deferred into its epilogue, so that a post-LayerNorm
 * transformer layer needs no LayerNorm launch at all:
 *   D = act( LN?(A).B + LN?(R) ),  and optionally the row statistics of D for the next call.
 * Every tensor that is "raw" (not yet normalised) travels with fp32 partial sums of its rows,
 * shape [ceil(width / 64), rows, 2] = {sum, sum of squares} per 64-column group, exactly what a
 * previous call wrote through StatsD.  StatsA given: A is raw and the epilogue computes
 * LN(A).B as rstd * (A.B) - mean * rstd * colsum(B) (column sums of a declared weight are kept).
 * StatsR given: the residual added is LN(R) = rstd * R - mean * rstd (R raw; R may alias D).
 * StatsD given: the epilogue writes D's partial sums (of the fp16-rounded values) there.  Absent
 * operands are rank-0 / null descriptors.  LayerNorm is the reference's (no affine, biased
 * variance, eps inside the square root); statistics stay in fp32 - the sm_100a form of the
 * reference's experimental cutlassGemmWithVarMeanF16 / cutlassLayernormGemmF16 pair
 * (include/NVGPUKernels/LayernormGemmRunner.h:17-361), which stores them in fp16 and cannot
 * express BERT's normalised residual.  A [.., M, K], B [1, K, N] or [1, N, K] (weightsNK),
 * R, D [.., M, N], N % 8 == 0; activation 0 or 1 (erf GELU).  StatsD must not be the buffer
 * of StatsA or StatsR (other tiles still read them).  With StatsA, the first call for a declared
 * weight computes and caches its column sums (allocates device memory and waits for the stream):
 * make that call outside of any stream capture; for any other B the sums are recomputed by an
 * extra launch on every call (N <= 65536). */
HOM_EXPORT void homGemmDeferredLayernormF16(int64_t rankA, void *dstA, int64_t rankStatsA, void *dstStatsA,
                                            int64_t rankB, void *dstB, bool weightsNK, int64_t rankR,
                                            void *dstR, int64_t rankStatsR, void *dstStatsR, int64_t rankD,
                                            void *dstD, int64_t rankStatsD, void *dstStatsD,
                                            int64_t activation, float eps);

/* Out = LayerNorm(X + R) * gamma + beta over the last dimension; X, R, Out [rows.., H]
 * fp16 (R, gamma, beta may be rank-0 descriptors = absent), fp32 sum and statistics,
 * one fp16 rounding at the store.  Out may alias X. */
HOM_EXPORT void homResidualLayernormF16(int64_t rankX, void *dstX, int64_t rankR, void *dstR,
                                        int64_t rankGamma, void *dstGamma, int64_t rankBeta,
                                        void *dstBeta, int64_t rankOut, void *dstOut, float eps);

/* cutlassLayernormGemmF16 for callers that must not allocate device memory - a process whose
 * memory was budgeted once at start-up, a plug-in running under a framework where cudaMalloc
 * would stall every stream of the device, a latency-critical loop.  Same operands and result:
 * D = alpha * (A * Var[r] + Mean[r]).B + beta * C (A [Bs,M,K], B [1,K,N], C [Bs,M,N] or
 * [1,1,N] or unused when beta == 0, D [Bs,M,N], Var/Mean fp16 [>= Bs*M]).  The column sums of
 * B that the computation needs live in a fixed 64 KB array inside the library image instead
 * of a cudaMalloc'ed buffer, so N is limited to 16384 columns (larger N: error 2, nothing is
 * launched) and every GPU that loads the library carries those 64 KB until the process ends.
 * The call performs no cudaMalloc / cudaFree / cudaHostAlloc and uses no allocating library.
 * The first call on each device looks up the array's device address (with that device
 * current); make that first call outside of any stream capture.  All calls share the one
 * array: each call rewrites the entries it uses before reading them, so nothing needs
 * clearing between calls, but two calls whose kernels overlap on the GPU (different streams,
 * or host threads on one device) would overwrite each other's sums - issue them on one stream.
 * Its launches are counted but never timed by homOpTimingEnable (timing allocates events), and
 * an expired device-side wait is reported by homSynchronize() only if some other entry point of
 * this library has run on the device before (that is what creates the status word; this one
 * will not allocate it).  This entry point has no counterpart in the reference. */
HOM_EXPORT void homLayernormGemmF16NoAlloc(int64_t rankA, void *dstA, int64_t rankB, void *dstB,
                                           int64_t rankC, void *dstC, int64_t rankD, void *dstD,
                                           int64_t rankVar, void *dstVar, int64_t rankMean,
                                           void *dstMean, float alpha, float beta);

/* Number of kernels this library has launched since load (all threads). */
HOM_EXPORT int64_t homKernelLaunchCount(void);

/* Per-launch timing: while enabled every entry point brackets its kernel with events on
 * the current stream.  homOpTimingCollect() synchronises, writes up to `capacity` records
 * (kind: 1 gemm, 2 layernorm, 3 attention, 4 elementwise, 5 gather, 6 cu_seqlen; ms; and
 * the algorithmic flop and byte counts of that launch), clears the log and returns the
 * number of records that were available. */
typedef struct HomOpTiming {
  int32_t kind;
  float ms;
  double flops;
  double bytes;
} HomOpTiming;
HOM_EXPORT void homOpTimingEnable(int enable);
HOM_EXPORT int64_t homOpTimingCollect(HomOpTiming *out, int64_t capacity);
/* The same read-out without releasing the records: for launches that were captured into a CUDA
 * graph while timing was enabled (their event records became graph nodes), call it after each
 * replay; call homOpTimingCollect once the graph is gone. */
HOM_EXPORT int64_t homOpTimingPeek(HomOpTiming *out, int64_t capacity);

/* The tile the GEMM family would run for (M, N, K, activation): the tile's N extent,
 * pipeline stages and split-K.  Returns the tile-table row number (usable as gemmNum). */
HOM_EXPORT int32_t homGemmQueryTile(int64_t m, int64_t n, int64_t k, int64_t activation,
                                    int32_t *bn, int32_t *stages, int32_t *splitK);

/* Run-time tuner with the contract of GemmProfiler::profile
 * (lib/NVGPUKernels/GemmProfiler.cu:143-236, include/NVGPUKernels/GemmProfiler.h:39-57): times every
 * row of the tile table for fp16 (M, N, K, activation, alpha, beta) on scratch operands it
 * allocates and frees (beta != 0 reads C = D), returns the fastest row in *tile_row (usable as
 * gemmNum; the autotune pass writes it to `kernel_name`) and 1 in *split_k, and remembers the
 * result so that later calls with an automatic gemmNum use it.  weights_nk != 0 times the
 * [1,N,K] weight layout.  row_us, if not null, receives the six per-row times in microseconds.
 * Blocks until the measurements are done; call it outside stream capture.  Returns the error
 * code (0 = ok). */
HOM_EXPORT int32_t homGemmTune(int64_t m, int64_t n, int64_t k, int64_t activation, float alpha,
                               float beta, int32_t weights_nk, int32_t iterations,
                               int32_t *tile_row, int32_t *split_k, float *best_us, float *row_us);
/* The tuned table as text, one "M N K activation row" line per shape (the reference keeps its
 * timing cache in memory only).  Return the number of entries, or -1 if the file cannot be
 * opened.  $HOM_TUNE_CACHE names a file that is loaded on first use. */
HOM_EXPORT int32_t homGemmTuneSave(const char *path);
HOM_EXPORT int32_t homGemmTuneLoad(const char *path);

#ifdef __cplusplus
}
#endif

#endif /* HOM_NVGPU_RUNNER_UTILS_H */

/* MLIR memref calling convention as seen by the runner-utils C ABI.
 *
 * The compiled model passes every `memref<*xT>` as two scalar arguments
 * `(int64_t rank, void *descriptor)`; `descriptor` points at a ranked strided
 * memref record: {T *basePtr; T *data; int64 offset; int64 sizes[rank];
 * int64 strides[rank]}.  Allocation entry points return the pair by value as a
 * trivially copyable 16-byte struct whose descriptor was obtained with malloc(),
 * because MLIR-generated callers release it with free().
 *
 * Reference: include/ExecutionEngine/HandsOnRunnerUtils.h:27-73
 * (C_UnrankedMemRefType, convertToDynamicMemRefType, allocHelper) and the type
 * converter in lib/Conversions/Function/FunctionUtils.cpp:349-357.  The layout
 * is that of StridedMemRefType / UnrankedMemRefType in MLIR's CRunnerUtils.h,
 * restated here so that no LLVM header is needed.
 */
#ifndef HOM_MEMREF_H
#define HOM_MEMREF_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Largest rank any entry point accepts (the elementwise kernels pass shapes by value). */
#define HOM_MAX_RANK 8

/* {rank, descriptor}: what alloc* entry points return by value. */
typedef struct HomUnrankedMemRef {
  int64_t rank;
  void *descriptor;
} HomUnrankedMemRef;

/* Fixed-rank descriptor records.  `sizes` is followed immediately by `strides`. */
#define HOM_DECLARE_STRIDED_MEMREF(N)                                                              \
  typedef struct HomStridedMemRef##N {                                                             \
    void *basePtr;                                                                                 \
    void *data;                                                                                    \
    int64_t offset;                                                                                \
    int64_t sizes[N];                                                                              \
    int64_t strides[N];                                                                            \
  } HomStridedMemRef##N

HOM_DECLARE_STRIDED_MEMREF(1);
HOM_DECLARE_STRIDED_MEMREF(2);
HOM_DECLARE_STRIDED_MEMREF(3);
HOM_DECLARE_STRIDED_MEMREF(4);
HOM_DECLARE_STRIDED_MEMREF(5);

#ifdef __cplusplus
}
#endif

#endif /* HOM_MEMREF_H */

// Minimal stand-in for MLIR's CRunnerUtils.h, sufficient to compile the reference's
// lib/ExecutionEngine/HandsOnRunnerUtils.cpp unchanged as a CPU checker (oracle/_ref).
// TEST INFRASTRUCTURE ONLY.  It restates the public memref ABI records (ranked strided
// memref, unranked memref, and the dynamic-rank view over an unranked memref); LLVM itself
// is not vendored in the reference tree (thirdparty/llvm-project is an empty directory).
#ifndef HOM_ORACLE_SHIM_CRUNNERUTILS_H
#define HOM_ORACLE_SHIM_CRUNNERUTILS_H

#include <cassert>
#include <cstdint>
#include <vector>

template <typename T, int N>
struct StridedMemRefType {
  T *basePtr;
  T *data;
  int64_t offset;
  int64_t sizes[N];
  int64_t strides[N];
};

template <typename T>
struct StridedMemRefType<T, 0> {
  T *basePtr;
  T *data;
  int64_t offset;
};

template <typename T>
struct UnrankedMemRefType {
  int64_t rank;
  void *descriptor;
};

// Rank-erased view: reads {basePtr, data, offset, sizes[rank], strides[rank]} from the
// record an unranked memref points at.
template <typename T>
class DynamicMemRefType {
public:
  explicit DynamicMemRefType(const UnrankedMemRefType<T> &memRef) : rank(memRef.rank) {
    auto *desc = static_cast<StridedMemRefType<T, 1> *>(memRef.descriptor);
    basePtr = desc->basePtr;
    data = desc->data;
    offset = desc->offset;
    sizes = rank == 0 ? nullptr : desc->sizes;
    strides = rank == 0 ? nullptr : sizes + rank;
  }

  int64_t rank;
  T *basePtr;
  T *data;
  int64_t offset;
  const int64_t *sizes;
  const int64_t *strides;
};

#endif

// Minimal stand-in for MLIR's RunnerUtils.h (see CRunnerUtils.h beside it).
// TEST INFRASTRUCTURE ONLY.
#ifndef HOM_ORACLE_SHIM_RUNNERUTILS_H
#define HOM_ORACLE_SHIM_RUNNERUTILS_H

#include <ostream>

#include "mlir/ExecutionEngine/CRunnerUtils.h"

template <typename StreamType, typename T>
void printMemRefMetaData(StreamType &os, const DynamicMemRefType<T> &v) {
  os << "base@ = " << reinterpret_cast<void *>(v.data) << " rank = " << v.rank
     << " offset = " << v.offset;
  os << " sizes = [";
  for (int64_t i = 0; i < v.rank; ++i) os << (i ? ", " : "") << v.sizes[i];
  os << "] strides = [";
  for (int64_t i = 0; i < v.rank; ++i) os << (i ? ", " : "") << v.strides[i];
  os << "]";
}

#endif

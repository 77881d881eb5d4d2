// LLVM-free loader for model libraries compiled by Hands-on-MLIR: the protocol of the
// reference's ExecutionEngine (include/ExecutionEngine/ExecutionEngine.h:114-166,
// lib/ExecutionEngine/ExecutionEngine.cpp:44-97) restated with dlopen/dlsym only.
//
// A compiled model exports, per function <fn>, three wrappers that all take one `void **`:
//   _hom_ciface_<fn>_argNum  stores an int32 through args[0]: how many tensors the compiler
//                            hoisted out of <fn> (weights and pre-allocated activations);
//   _hom_ciface_<fn>_initFn  stores that many {int64 rank, void *descriptor} pairs,
//                            contiguously, through args[0] (each descriptor is malloc'ed);
//   _hom_ciface_<fn>         args[i] points at the i-th scalar argument of <fn> - an unranked
//                            memref contributes two slots (&rank, &descriptor) - with the hoisted
//                            tensors first, then the caller's arguments; the slot after the
//                            last argument points at storage for the result
//                            (lib/Conversions/Function/UnifyLLVMFuncInterface.cpp:74-122).
// The first invocation of <fn> runs argNum + initFn once and caches the hoisted tensors.
#include <dlfcn.h>

#include <cstdlib>
#include <cstring>
#include <map>
#include <string>
#include <vector>

#include "hom_bert_replay.h"

namespace {

struct InitTensors {
  std::vector<HomUnrankedMemRef> tensors;
};

struct Model {
  void *handle = nullptr;
  std::map<std::string, InitTensors> init;
  std::string error;
  bool synchronous = false;  // homModelInvoke waits for the stream and reports device-side errors
};

using InvokeFn = void (*)(void **);

InvokeFn lookup(Model &m, const std::string &name) {
  dlerror();
  void *sym = dlsym(m.handle, ("_hom_ciface_" + name).c_str());
  if (!sym) {
    const char *e = dlerror();
    m.error = e ? e : ("symbol _hom_ciface_" + name + " not found");
  }
  return reinterpret_cast<InvokeFn>(sym);
}

}  // namespace

extern "C" {

void *homModelOpen(const char *path) {
  if (!path) return nullptr;
  void *h = dlopen(path, RTLD_NOW | RTLD_GLOBAL);
  if (!h) return nullptr;
  auto *m = new Model();
  m->handle = h;
  return m;
}

const char *homModelLastError(void *model) {
  auto *m = static_cast<Model *>(model);
  return m ? m->error.c_str() : dlerror();
}

int32_t homModelInitTensorCount(void *model, const char *fn) {
  auto *m = static_cast<Model *>(model);
  if (!m || !fn) return -1;
  auto it = m->init.find(fn);
  return it == m->init.end() ? -1 : static_cast<int32_t>(it->second.tensors.size());
}

int homModelInvoke(void *model, const char *fn, int32_t n_user_slots, void **user_slots,
                   void *result_storage) {
  auto *m = static_cast<Model *>(model);
  if (!m || !fn || n_user_slots < 0 || (n_user_slots > 0 && !user_slots)) return HOM_ERR_INVALID;
  const std::string name(fn);
  auto it = m->init.find(name);
  if (it == m->init.end()) {
    InvokeFn arg_num_fn = lookup(*m, name + "_argNum");
    InvokeFn init_fn = lookup(*m, name + "_initFn");
    if (!arg_num_fn || !init_fn) return HOM_ERR_INVALID;
    int32_t count = 0;
    void *slot0[1] = {&count};
    arg_num_fn(slot0);
    if (count < 0) {
      m->error = "negative init-tensor count";
      return HOM_ERR_INVALID;
    }
    InitTensors init;
    init.tensors.resize(static_cast<size_t>(count));
    void *slot1[1] = {init.tensors.data()};
    if (count > 0) init_fn(slot1);
    it = m->init.emplace(name, std::move(init)).first;
  }
  InvokeFn forward = lookup(*m, name);
  if (!forward) return HOM_ERR_INVALID;
  std::vector<void *> args;
  args.reserve(2 * it->second.tensors.size() + static_cast<size_t>(n_user_slots) + 1);
  for (HomUnrankedMemRef &t : it->second.tensors) {
    args.push_back(&t.rank);
    args.push_back(&t.descriptor);
  }
  for (int32_t i = 0; i < n_user_slots; ++i) args.push_back(user_slots[i]);
  args.push_back(result_storage);
  forward(args.data());
  // A device-side wait that expired only shows once the stream has drained: callers that
  // asked for it get the stream synchronised and the status word folded in before returning.
  if (m->synchronous) return homSynchronize();
  return homGetLastError();
}

void homModelSetSynchronous(void *model, int enable) {
  auto *m = static_cast<Model *>(model);
  if (m) m->synchronous = enable != 0;
}

void homModelClose(void *model) {
  auto *m = static_cast<Model *>(model);
  if (!m) return;
  // Like the reference's loader, only the descriptors are released here; the buffers belong
  // to the model's dealloc function (ExecutionEngine.h:37-45).
  for (auto &kv : m->init)
    for (HomUnrankedMemRef &t : kv.second.tensors) std::free(t.descriptor);
  if (m->handle) dlclose(m->handle);
  delete m;
}

}  // extern "C"

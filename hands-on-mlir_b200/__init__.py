"""Python binding of the B200 runner-utils C ABI (tests and benchmarks use it).

The product is `lib/libhands_on_mlir_nvgpu_runner_utils.so`; this module only loads it with
ctypes, packs tensors into MLIR memref descriptors (see include/hom_memref.h) and turns the
library's error side channel into exceptions.  Entry points keep the reference's names
(include/ExecutionEngine/HandsOnNVGPURunnerUtils.h:70-164) so that a test reads like a call
from the compiled model.  There is no CPU fallback: a missing library raises.
"""
from __future__ import annotations

import ctypes
from ctypes import c_bool, c_char_p, c_double, c_float, c_int32, c_int64, c_void_p
from pathlib import Path

import os

PKG_DIR = Path(__file__).resolve().parent
# HOM_LIB_DIR selects another build of the same two libraries (e.g. lib/diagnostics).
_LIB_DIR = Path(os.environ["HOM_LIB_DIR"]).resolve() if os.environ.get("HOM_LIB_DIR") else PKG_DIR / "lib"
RUNNER_LIB = _LIB_DIR / "libhands_on_mlir_nvgpu_runner_utils.so"
REPLAY_LIB = _LIB_DIR / "libhom_bert_replay.so"


class HomError(RuntimeError):
    """An entry point recorded an error (code, message) instead of launching."""

    def __init__(self, code: int, message: str):
        super().__init__(f"[hom error {code}] {message}")
        self.code = code
        self.message = message


class UnrankedMemRef(ctypes.Structure):
    """{rank, descriptor} as returned by value from the alloc* entry points."""

    _fields_ = [("rank", c_int64), ("descriptor", c_void_p)]


class OpTiming(ctypes.Structure):
    _fields_ = [("kind", c_int32), ("ms", c_float), ("flops", c_double), ("bytes", c_double)]


class MemRef:
    """A ranked strided memref descriptor {basePtr, data, offset, sizes[], strides[]}.

    Build it from a torch tensor (`MemRef.of(t)`), from a raw pointer and a shape, or wrap a
    descriptor returned by the library (`MemRef.from_unranked`).  `args` yields the
    `(rank, descriptor*)` pair the C ABI takes.
    """

    def __init__(self, data_ptr: int, shape, strides=None, offset: int = 0, keepalive=None):
        shape = [int(s) for s in shape]
        rank = len(shape)
        if strides is None:
            strides, acc = [0] * rank, 1
            for i in range(rank - 1, -1, -1):
                strides[i] = acc
                acc *= shape[i]
        self.rank = rank
        self.shape = shape
        self.strides = [int(s) for s in strides]
        self._words = (c_int64 * (3 + 2 * rank))()
        self._words[0] = data_ptr or 0
        self._words[1] = data_ptr or 0
        self._words[2] = offset
        for i in range(rank):
            self._words[3 + i] = shape[i]
            self._words[3 + rank + i] = self.strides[i]
        self._keepalive = keepalive

    @classmethod
    def of(cls, tensor) -> "MemRef":
        return cls(tensor.data_ptr(), tensor.shape, tensor.stride(), 0, keepalive=tensor)

    @classmethod
    def from_unranked(cls, um: UnrankedMemRef) -> "MemRef":
        rank = int(um.rank)
        words = ctypes.cast(um.descriptor, ctypes.POINTER(c_int64))
        shape = [words[3 + i] for i in range(rank)]
        strides = [words[3 + rank + i] for i in range(rank)]
        return cls(words[1], shape, strides, words[2])

    @property
    def data_ptr(self) -> int:
        return int(self._words[1])

    @property
    def args(self):
        return c_int64(self.rank), ctypes.cast(self._words, c_void_p)


NULL_MEMREF = (c_int64(0), c_void_p(None))


def _as_args(x):
    if x is None:
        return NULL_MEMREF
    if isinstance(x, MemRef):
        return x.args
    return MemRef.of(x).args


_MEMREF = [c_int64, c_void_p]
_GEMM_ARGS = (_MEMREF + [c_bool] + _MEMREF + [c_bool] + _MEMREF + _MEMREF +
              [c_int64, c_float, c_float, c_int32, c_int32])

_SIGNATURES = {
    "cutlassGemmF16": (None, _GEMM_ARGS),
    "nvteGemmF16": (None, _GEMM_ARGS),
    "cutlassGemmF32": (None, _MEMREF + [c_bool] + _MEMREF + [c_bool] + _MEMREF + _MEMREF +
                       [c_int64, c_float, c_float]),
    "cutlassGemmWithVarMeanF16": (None, _MEMREF * 6 + [c_float, c_float, c_int64, c_float]),
    "cutlassLayernormGemmF32": (None, _MEMREF * 6 + [c_float, c_float, c_int64]),
    "cutlassLayernormGemmF16": (None, _MEMREF * 6 + [c_float, c_float, c_int64]),
    "nvteLayernormF32": (None, _MEMREF + [c_float]),
    "nvteLayernormF16": (None, _MEMREF + [c_float]),
    "nvteBertAttentionF32": (None, _MEMREF * 3 + [c_float, c_int64]),
    "nvteBertAttentionF16": (None, _MEMREF * 3 + [c_float, c_int64]),
    "allocConstantNVGPUF32": (UnrankedMemRef, [c_int32]),
    "allocConstantNVGPUF16": (UnrankedMemRef, [c_int32]),
    "alloc3DMemRefNVGPUF32": (UnrankedMemRef, [c_int32] * 3),
    "alloc3DMemRefNVGPUF16": (UnrankedMemRef, [c_int32] * 3),
    "alloc1DMemRefNVGPUI32": (UnrankedMemRef, [c_int32]),
    "deallocNVGPUF32": (None, _MEMREF),
    "deallocNVGPUF16": (None, _MEMREF),
    "deallocNVGPUI32": (None, _MEMREF),
    "thrustGatherF32": (None, _MEMREF * 3),
    "thrustGatherF16": (None, _MEMREF * 3),
    "thrustCuSeqLenI32": (None, _MEMREF * 2),
    "thrustCuSeqLenI64": (None, _MEMREF * 2),
    "printMemrefSizeF32": (None, _MEMREF),
    "printMemrefSizeF16": (None, _MEMREF),
    "printMemrefSizeI64": (None, _MEMREF),
    "printMemrefSizeI32": (None, _MEMREF),
    "homGetLastError": (ctypes.c_int, []),
    "homGetLastErrorString": (c_char_p, []),
    "homClearLastError": (None, []),
    "homSetStream": (None, [c_void_p]),
    "homGetStream": (c_void_p, []),
    "homSynchronize": (ctypes.c_int, []),
    "homSetConstantDir": (None, [c_char_p]),
    "homDeclareWeights": (None, [c_void_p, c_int64]),
    "homForgetWeights": (None, [c_void_p]),
    "homResidualLayernormF16": (None, _MEMREF * 5 + [c_float]),
    "homBertEmbeddingF16": (None, _MEMREF * 6 + [c_float]),
    "homGemmResidualLayernormF16": (None, _MEMREF * 2 + [ctypes.c_bool] + _MEMREF * 2 + [c_float]),
    "homLayernormGemmF16NoAlloc": (None, _MEMREF * 6 + [c_float, c_float]),
    "homGemmDeferredLayernormF16": (None, _MEMREF * 3 + [ctypes.c_bool] + _MEMREF * 4 + [c_int64, c_float]),
    "homKernelLaunchCount": (c_int64, []),
    "homOpTimingEnable": (None, [ctypes.c_int]),
    "homOpTimingCollect": (c_int64, [ctypes.POINTER(OpTiming), c_int64]),
    "homOpTimingPeek": (c_int64, [ctypes.POINTER(OpTiming), c_int64]),
    "homGemmQueryTile": (c_int32, [c_int64, c_int64, c_int64, c_int64,
                                   ctypes.POINTER(c_int32), ctypes.POINTER(c_int32),
                                   ctypes.POINTER(c_int32)]),
    "homGemmTune": (c_int32, [c_int64, c_int64, c_int64, c_int64, c_float, c_float, c_int32, c_int32,
                              ctypes.POINTER(c_int32), ctypes.POINTER(c_int32),
                              ctypes.POINTER(c_float), ctypes.POINTER(c_float)]),
    "homSetConstantCache": (None, [ctypes.c_int]),
    "homGemmTuneSave": (c_int32, [ctypes.c_char_p]),
    "homGemmTuneLoad": (c_int32, [ctypes.c_char_p]),
}
for _op in ("Add", "Sub", "Mul", "Div"):
    for _ty in ("F32", "F16"):
        _SIGNATURES[f"thrustElementwise{_op}{_ty}"] = (None, _MEMREF * 3)

#: every symbol include/hom_nvgpu_runner_utils.h declares
EXPORTED_SYMBOLS = tuple(sorted(_SIGNATURES))


class RunnerUtils:
    """ctypes view of libhands_on_mlir_nvgpu_runner_utils.so with error checking."""

    def __init__(self, path: Path | str = RUNNER_LIB):
        path = Path(path)
        if not path.exists():
            raise FileNotFoundError(
                f"{path} is missing: build it with `python hands-on-mlir_b200/build.py` "
                "(there is no fallback path)")
        self.path = path
        self.lib = ctypes.CDLL(str(path), mode=ctypes.RTLD_GLOBAL)
        for name, (restype, argtypes) in _SIGNATURES.items():
            fn = getattr(self.lib, name)
            fn.restype = restype
            fn.argtypes = argtypes

    # ------------------------------------------------------------ error channel
    def check(self):
        code = self.lib.homGetLastError()
        if code != 0:
            msg = (self.lib.homGetLastErrorString() or b"").decode()
            self.lib.homClearLastError()
            raise HomError(code, msg)

    def last_error(self):
        return self.lib.homGetLastError(), (self.lib.homGetLastErrorString() or b"").decode()

    def clear_error(self):
        self.lib.homClearLastError()

    def synchronize(self):
        self.lib.homSynchronize()
        self.check()

    def set_stream(self, cuda_stream_handle: int | None):
        self.lib.homSetStream(c_void_p(cuda_stream_handle or None))

    def use_torch_stream(self):
        import torch
        self.set_stream(torch.cuda.current_stream().cuda_stream)

    def declare_weights(self, tensor):
        """Tell the library that no kernel writes `tensor` (a GEMM weight): its tiles may then be
        prefetched before the previous kernel of the stream has finished."""
        self.lib.homDeclareWeights(c_void_p(tensor.data_ptr()), tensor.numel() * tensor.element_size())

    def forget_weights(self, tensor):
        self.lib.homForgetWeights(c_void_p(tensor.data_ptr()))

    # ------------------------------------------------------------------ compute
    def _gemm(self, fn, A, B, C, D, transa, transb, act, alpha, beta, gemm_num, split_k):
        fn(*_as_args(A), transa, *_as_args(B), transb, *_as_args(C), *_as_args(D), act, alpha,
           beta, gemm_num, split_k)
        self.check()

    def cutlassGemmF16(self, A, B, C, D, activation=0, alpha=1.0, beta=0.0, gemmNum=0,
                       splitKFactor=1, transa=False, transb=False):
        self._gemm(self.lib.cutlassGemmF16, A, B, C, D, transa, transb, activation, alpha, beta,
                   gemmNum, splitKFactor)

    def nvteGemmF16(self, A, B, C, D, activation=0, alpha=1.0, beta=0.0, transa=False,
                    transb=True, gemmNum=0):
        self._gemm(self.lib.nvteGemmF16, A, B, C, D, transa, transb, activation, alpha, beta,
                   gemmNum, 0)

    def cutlassGemmWithVarMeanF16(self, A, B, C, D, Var, Mean, alpha=1.0, beta=0.0, activation=0,
                                  eps=1e-5):
        self.lib.cutlassGemmWithVarMeanF16(*_as_args(A), *_as_args(B), *_as_args(C), *_as_args(D),
                                           *_as_args(Var), *_as_args(Mean), alpha, beta, activation,
                                           eps)
        self.check()

    def cutlassLayernormGemmF16(self, A, B, C, D, Var, Mean, alpha=1.0, beta=0.0, activation=0):
        self.lib.cutlassLayernormGemmF16(*_as_args(A), *_as_args(B), *_as_args(C), *_as_args(D),
                                         *_as_args(Var), *_as_args(Mean), alpha, beta, activation)
        self.check()

    def homLayernormGemmF16NoAlloc(self, A, B, C, D, Var, Mean, alpha=1.0, beta=0.0):
        self.lib.homLayernormGemmF16NoAlloc(*_as_args(A), *_as_args(B), *_as_args(C), *_as_args(D),
                                            *_as_args(Var), *_as_args(Mean), alpha, beta)
        self.check()

    def nvteLayernormF16(self, A, eps=1e-6):
        self.lib.nvteLayernormF16(*_as_args(A), eps)
        self.check()

    def nvteLayernormF32(self, A, eps=1e-6):
        self.lib.nvteLayernormF32(*_as_args(A), eps)
        self.check()

    def homGemmDeferredLayernormF16(self, A, statsA, B, R, statsR, D, statsD, activation=0, eps=1e-12,
                                    weights_nk=False):
        self.lib.homGemmDeferredLayernormF16(*_as_args(A), *_as_args(statsA), *_as_args(B), weights_nk,
                                             *_as_args(R), *_as_args(statsR), *_as_args(D),
                                             *_as_args(statsD), activation, eps)
        self.check()

    def homResidualLayernormF16(self, X, R, gamma, beta, Out, eps=1e-12):
        self.lib.homResidualLayernormF16(*_as_args(X), *_as_args(R), *_as_args(gamma),
                                         *_as_args(beta), *_as_args(Out), eps)
        self.check()

    def homGemmResidualLayernormF16(self, A, B, R, D, eps=1e-12, weights_nk=False):
        self.lib.homGemmResidualLayernormF16(*_as_args(A), *_as_args(B), bool(weights_nk), *_as_args(R),
                                             *_as_args(D), eps)
        self.check()

    def homBertEmbeddingF16(self, ids, types, word, pos, type_emb, Out, eps=1e-12):
        self.lib.homBertEmbeddingF16(*_as_args(ids), *_as_args(types), *_as_args(word), *_as_args(pos),
                                     *_as_args(type_emb), *_as_args(Out), eps)
        self.check()

    def nvteBertAttentionF16(self, qkv, cu_seqlens, out, scale, headNum):
        self.lib.nvteBertAttentionF16(*_as_args(qkv), *_as_args(cu_seqlens), *_as_args(out), scale,
                                      headNum)
        self.check()

    def elementwise(self, op: str, dtype: str, A, B, Out):
        getattr(self.lib, f"thrustElementwise{op}{dtype}")(*_as_args(A), *_as_args(B),
                                                           *_as_args(Out))
        self.check()

    def thrustElementwiseAddF16(self, A, B, Out):
        self.elementwise("Add", "F16", A, B, Out)

    def gather(self, dtype: str, indices, table, out):
        getattr(self.lib, f"thrustGather{dtype}")(*_as_args(indices), *_as_args(table),
                                                  *_as_args(out))
        self.check()

    def thrustGatherF16(self, indices, table, out):
        self.gather("F16", indices, table, out)

    def cu_seqlen(self, dtype: str, mask, out):
        getattr(self.lib, f"thrustCuSeqLen{dtype}")(*_as_args(mask), *_as_args(out))
        self.check()

    def thrustCuSeqLenI64(self, mask, out):
        self.cu_seqlen("I64", mask, out)

    # --------------------------------------------------------------- allocation
    def alloc3DMemRefNVGPUF16(self, a, b, c) -> MemRef:
        um = self.lib.alloc3DMemRefNVGPUF16(a, b, c)
        self.check()
        return MemRef.from_unranked(um)

    def alloc1DMemRefNVGPUI32(self, n) -> MemRef:
        um = self.lib.alloc1DMemRefNVGPUI32(n)
        self.check()
        return MemRef.from_unranked(um)

    def allocConstantNVGPUF16(self, idx) -> MemRef:
        um = self.lib.allocConstantNVGPUF16(idx)
        self.check()
        return MemRef.from_unranked(um)

    def allocConstantNVGPUF32(self, idx) -> MemRef:
        um = self.lib.allocConstantNVGPUF32(idx)
        self.check()
        return MemRef.from_unranked(um)

    def dealloc(self, dtype: str, memref: MemRef):
        getattr(self.lib, f"deallocNVGPU{dtype}")(*memref.args)
        self.check()

    # -------------------------------------------------------------- measurement
    def launch_count(self) -> int:
        return int(self.lib.homKernelLaunchCount())

    def op_timing(self, enable: bool):
        self.lib.homOpTimingEnable(1 if enable else 0)

    def collect_op_timings(self, capacity: int = 1 << 16):
        buf = (OpTiming * capacity)()
        n = int(self.lib.homOpTimingCollect(buf, capacity))
        return [(buf[i].kind, buf[i].ms, buf[i].flops, buf[i].bytes) for i in range(min(n, capacity))]

    def peek_op_timings(self, capacity: int = 1 << 16):
        """Durations of the recorded launches without releasing them (graph replays re-record)."""
        buf = (OpTiming * capacity)()
        n = int(self.lib.homOpTimingPeek(buf, capacity))
        return [(buf[i].kind, buf[i].ms, buf[i].flops, buf[i].bytes) for i in range(min(n, capacity))]

    def gemm_query_tile(self, m, n, k, activation=0):
        bn, st, sk = c_int32(), c_int32(), c_int32()
        row = self.lib.homGemmQueryTile(m, n, k, activation, ctypes.byref(bn), ctypes.byref(st),
                                        ctypes.byref(sk))
        return {"row": int(row), "bn": bn.value, "stages": st.value, "split_k": sk.value}

    def gemm_tune(self, m, n, k, activation=0, alpha=1.0, beta=0.0, weights_nk=False, iterations=20):
        """Time the tile-table rows for one shape (GemmProfiler::profile's contract); the winner
        is remembered for automatic selection.  Returns row, split_k, best_us and the row times."""
        row, sk, best = c_int32(), c_int32(), c_float()
        times = (c_float * 6)()
        rc = self.lib.homGemmTune(m, n, k, activation, alpha, beta, int(weights_nk), iterations,
                                  ctypes.byref(row), ctypes.byref(sk), ctypes.byref(best), times)
        if rc != 0:
            self.check()
            raise HomError(rc, "homGemmTune failed")
        return {"row": row.value, "split_k": sk.value, "best_us": best.value, "row_us": list(times)}

    def gemm_tune_save(self, path) -> int:
        return int(self.lib.homGemmTuneSave(str(path).encode()))

    def gemm_tune_load(self, path) -> int:
        return int(self.lib.homGemmTuneLoad(str(path).encode()))


_runner: RunnerUtils | None = None


def runner() -> RunnerUtils:
    """The process-wide library handle (loaded on first use)."""
    global _runner
    if _runner is None:
        _runner = RunnerUtils()
    return _runner

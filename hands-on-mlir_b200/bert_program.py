"""ctypes binding of libhom_bert_replay.so (include/hom_bert_replay.h): the hand-written
stand-in for the model library Hands-on-MLIR compiles from BERT.  The program itself is
C++ and drives the kernels only through the runner-utils C ABI; this file just loads it,
hands it weights and inputs, and exposes the batch-sharding helpers the multi-GPU runs use.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_int32, c_int64, c_void_p
from dataclasses import dataclass

from . import REPLAY_LIB, HomError, MemRef, UnrankedMemRef, runner


class _Config(ctypes.Structure):
    _fields_ = [("layers", c_int32), ("hidden", c_int32), ("heads", c_int32), ("ffn", c_int32),
                ("vocab", c_int32), ("type_vocab", c_int32), ("batch", c_int32), ("seq", c_int32),
                ("eps", c_float), ("weights_nk", c_int32), ("fused_embedding", c_int32),
                ("fused_layernorm", c_int32)]


@dataclass(frozen=True)
class BertConfig:
    layers: int = 12
    hidden: int = 768
    heads: int = 12
    ffn: int = 3072
    vocab: int = 30522
    type_vocab: int = 2
    max_pos: int = 512
    eps: float = 1e-12

    @staticmethod
    def base() -> "BertConfig":
        return BertConfig()

    @staticmethod
    def large() -> "BertConfig":
        return BertConfig(layers=24, hidden=1024, heads=16, ffn=4096)

    def gemm_flops_per_sequence(self, seq: int) -> float:
        h, f = self.hidden, self.ffn
        return self.layers * 2.0 * seq * (h * 3 * h + h * h + 2 * h * f)

    def attention_flops_per_sequence(self, seq: int) -> float:
        return self.layers * 4.0 * seq * seq * self.hidden

    def weight_names(self):
        names = ["word_emb", "pos_emb", "type_emb"]
        for i in range(self.layers):
            names += [f"wqkv_{i}", f"wo_{i}", f"w1_{i}", f"w2_{i}"]
        return names

    def weight_shape(self, name: str, seq: int, nk: bool = False):
        h, f = self.hidden, self.ffn
        if name == "word_emb":
            return (1, self.vocab, h)
        if name == "pos_emb":
            return (1, seq, h)
        if name == "type_emb":
            return (1, self.type_vocab, h)
        k, n = {"wqkv": (h, 3 * h), "wo": (h, h), "w1": (h, f), "w2": (f, h)}[name.split("_")[0]]
        return (1, n, k) if nk else (1, k, n)


def shard_batch(total: int, world_size: int, rank: int) -> tuple[int, int]:
    """Even split of `total` sequences over ranks: [start, stop) for `rank`.  The batch must
    divide evenly (the benchmark configurations do)."""
    if total % world_size != 0:
        raise ValueError(f"batch {total} does not split evenly over {world_size} ranks")
    per = total // world_size
    return rank * per, (rank + 1) * per


_lib = None


def _replay_lib():
    global _lib
    if _lib is None:
        runner()  # the runner library must be loaded (RTLD_GLOBAL) first
        if not REPLAY_LIB.exists():
            raise FileNotFoundError(f"{REPLAY_LIB} is missing: run hands-on-mlir_b200/build.py")
        lib = ctypes.CDLL(str(REPLAY_LIB))
        lib.homBertWeightCount.restype = c_int32
        lib.homBertWeightCount.argtypes = [ctypes.POINTER(_Config)]
        lib.homBertCreate.restype = c_void_p
        lib.homBertCreate.argtypes = [ctypes.POINTER(_Config)]
        lib.homBertDestroy.argtypes = [c_void_p]
        lib.homBertSetWeight.restype = c_int
        lib.homBertSetWeight.argtypes = [c_void_p, c_int32, c_int64, c_void_p]
        lib.homBertLoadConstants.restype = c_int
        lib.homBertLoadConstants.argtypes = [c_void_p, c_int32]
        lib.homBertForward.restype = c_int
        lib.homBertForward.argtypes = [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64,
                                       c_void_p, ctypes.POINTER(UnrankedMemRef), c_int]
        lib.homBertForwardHost.restype = c_int
        lib.homBertForwardHost.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int]
        lib.homBertForwardHostAsync.restype = c_int
        lib.homBertForwardHostAsync.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int]
        lib.homBertWaitHost.restype = c_int
        lib.homBertWaitHost.argtypes = [c_void_p]
        lib.homBertHostTraffic.argtypes = [c_void_p, ctypes.POINTER(c_int64),
                                           ctypes.POINTER(c_int64)]
        lib.homBertLaunchesPerForward.restype = c_int32
        lib.homBertLaunchesPerForward.argtypes = [c_void_p]
        _lib = lib
    return _lib


class BertProgram:
    """One replay program: a model configuration at a fixed [batch, seq] on the current GPU."""

    def __init__(self, cfg: BertConfig, batch: int, seq: int, weights_nk: bool = False,
                 fused_embedding: bool = False, fused_layernorm: bool | int = False):
        self.cfg, self.batch, self.seq, self.weights_nk = cfg, batch, seq, weights_nk
        self.fused_embedding, self.fused_layernorm = fused_embedding, fused_layernorm
        self._lib = _replay_lib()
        self._hom = runner()
        c = _Config(cfg.layers, cfg.hidden, cfg.heads, cfg.ffn, cfg.vocab, cfg.type_vocab, batch,
                    seq, cfg.eps, int(weights_nk), int(fused_embedding), int(fused_layernorm))
        self._handle = self._lib.homBertCreate(ctypes.byref(c))
        if not self._handle:
            self._hom.check()
            raise HomError(1, "homBertCreate failed")
        self._weights = {}

    def close(self):
        if self._handle:
            self._lib.homBertDestroy(self._handle)
            self._handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _rc(self, rc: int):
        if rc != 0:
            self._hom.check()
            raise HomError(rc, "bert replay call failed")

    def set_weights(self, tensors: dict):
        """`tensors`: name -> fp16 CUDA tensor, names and shapes as BertConfig.weight_names()."""
        for i, name in enumerate(self.cfg.weight_names()):
            t = tensors[name]
            want = self.cfg.weight_shape(name, self.seq, self.weights_nk)
            if tuple(t.shape) != want:
                raise ValueError(f"{name}: shape {tuple(t.shape)} != {want}")
            m = MemRef.of(t)
            self._rc(self._lib.homBertSetWeight(self._handle, i, *m.args))
            self._weights[name] = t  # keep the storage alive

    def load_constants(self, first_idx: int = 0):
        self._rc(self._lib.homBertLoadConstants(self._handle, first_idx))

    def forward(self, ids, mask, types, use_graph: bool = False) -> MemRef:
        """Enqueue one forward on device tensors (int64 [batch, seq]); returns the memref of
        the program-owned fp16 [batch, seq, hidden] result."""
        out = UnrankedMemRef()
        mi, mm, mt = MemRef.of(ids), MemRef.of(mask), MemRef.of(types)
        self._rc(self._lib.homBertForward(self._handle, *mi.args, *mm.args, *mt.args,
                                          ctypes.byref(out), int(use_graph)))
        return MemRef.from_unranked(out)

    def forward_host(self, ids, mask, types, out, use_graph: bool = False):
        """End-to-end step on HOST tensors (pinned torch tensors or numpy arrays): H2D copies,
        forward, D2H copy of the hidden states into `out`, and wait."""
        def ptr(x):
            return x.data_ptr() if hasattr(x, "data_ptr") else x.ctypes.data
        self._rc(self._lib.homBertForwardHost(self._handle, ptr(ids), ptr(mask), ptr(types),
                                              ptr(out), int(use_graph)))

    def forward_host_async(self, ids, mask, types, out, use_graph: bool = False):
        """Like forward_host but returns once the step is enqueued; `out` is filled by a copy
        stream while later steps run.  Alternate between two `out` buffers; call wait_host()
        before reading them."""
        def ptr(x):
            return x.data_ptr() if hasattr(x, "data_ptr") else x.ctypes.data
        self._rc(self._lib.homBertForwardHostAsync(self._handle, ptr(ids), ptr(mask), ptr(types),
                                                   ptr(out), int(use_graph)))

    def wait_host(self):
        self._rc(self._lib.homBertWaitHost(self._handle))

    def host_traffic(self) -> tuple[int, int]:
        a, b = c_int64(), c_int64()
        self._lib.homBertHostTraffic(self._handle, ctypes.byref(a), ctypes.byref(b))
        return a.value, b.value

    def launches_per_forward(self) -> int:
        return int(self._lib.homBertLaunchesPerForward(self._handle))

    def result_to_torch(self, memref: MemRef):
        """Copy the program-owned result into a fresh torch tensor (identity gather on the
        library's stream keeps ordering with the forward)."""
        import torch
        b, s, h = memref.shape
        out = torch.empty((b, s, h), dtype=torch.float16, device="cuda")
        table = MemRef(memref.data_ptr, (1, b * s, h))
        rows = torch.arange(b * s, dtype=torch.int64, device="cuda").reshape(b, s)
        self._hom.gather("F16", rows, table, out)
        return out


class ModelLibrary:
    """A model library compiled by Hands-on-MLIR, driven through the LLVM-free loader
    (homModelOpen / homModelInvoke in include/hom_bert_replay.h)."""

    def __init__(self, so_path):
        lib = _replay_lib()
        lib.homModelOpen.restype = c_void_p
        lib.homModelOpen.argtypes = [ctypes.c_char_p]
        lib.homModelInvoke.restype = c_int
        lib.homModelInvoke.argtypes = [c_void_p, ctypes.c_char_p, c_int32, ctypes.POINTER(c_void_p),
                                       c_void_p]
        lib.homModelInitTensorCount.restype = c_int32
        lib.homModelInitTensorCount.argtypes = [c_void_p, ctypes.c_char_p]
        lib.homModelLastError.restype = ctypes.c_char_p
        lib.homModelLastError.argtypes = [c_void_p]
        lib.homModelClose.argtypes = [c_void_p]
        lib.homModelSetSynchronous.argtypes = [c_void_p, c_int]
        self._lib = lib
        self._handle = lib.homModelOpen(str(so_path).encode())
        if not self._handle:
            raise OSError(f"cannot load model library {so_path}")

    def invoke(self, fn: str, args, result=None):
        """`args`: MemRef objects (two slots each) or ctypes scalars (one slot each).
        Returns the result as an UnrankedMemRef (or fills `result` if given)."""
        slots, keep = [], []
        for a in args:
            if isinstance(a, MemRef):
                rank, desc = a.args
                keep += [rank, desc]
                slots += [ctypes.addressof(rank), ctypes.addressof(desc)]
            else:
                keep.append(a)
                slots.append(ctypes.addressof(a))
        arr = (c_void_p * max(1, len(slots)))(*slots)
        res = result if result is not None else UnrankedMemRef()
        rc = self._lib.homModelInvoke(self._handle, fn.encode(), len(slots), arr, ctypes.byref(res))
        if rc != 0:
            runner().check()
            raise HomError(rc, (self._lib.homModelLastError(self._handle) or b"").decode())
        return res

    def set_synchronous(self, enable: bool = True):
        """Make invoke() wait for the stream and surface device-side errors (homSynchronize)."""
        self._lib.homModelSetSynchronous(self._handle, int(enable))

    def init_tensor_count(self, fn: str) -> int:
        return int(self._lib.homModelInitTensorCount(self._handle, fn.encode()))

    def close(self):
        if self._handle:
            self._lib.homModelClose(self._handle)
            self._handle = None

"""numpy front end of the CPU oracle (oracle/hom_oracle.cpp).  TEST INFRASTRUCTURE ONLY.

Only tests, the smoke check and the benchmark's CPU-baseline leg may import this module;
the product (the CUDA library and its binding) never does.

Arrays are numpy; fp16 tensors are `np.float16`.  Function names mirror the runner-utils
entry points they check.  `bert_encoder` composes the per-op functions in the order the
lowered BERT model calls them (examples/torch/bert/bert.cu:81-125 drives `forward`; the
per-layer op order is the one the lowering emits, lib/Conversions/Function/HOMNVGPUToFunc.cpp).
"""
from __future__ import annotations

import ctypes
import subprocess
from ctypes import c_float, c_int, c_int64, c_void_p
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
ORACLE_LIB = HERE / "libhom_oracle.so"
REF_CPU_LIB = HERE / "_ref" / "libhom_ref_cpu.so"

_lib = None


def build() -> None:
    """(Re)build libhom_oracle.so and, when the reference checkout is present, _ref/."""
    import os
    cand = os.environ.get("HOM_REFERENCE_DIR") or str(HERE.parent.parent / "reference")
    extra = [f"REFERENCE_DIR={cand}"] if (Path(cand) / "lib" / "ExecutionEngine").is_dir() else []
    subprocess.run(["make", "-C", str(HERE)] + extra, check=True, capture_output=True)


def lib():
    global _lib
    if _lib is None:
        if not ORACLE_LIB.exists():
            build()
        _lib = ctypes.CDLL(str(ORACLE_LIB))
        _lib.oracle_set_threads.restype = c_int
    return _lib


def set_threads(n: int = 0) -> int:
    return int(lib().oracle_set_threads(c_int(n)))


def _p(a):
    return None if a is None else a.ctypes.data_as(c_void_p)


def _f16(a):
    a = np.ascontiguousarray(a)
    assert a.dtype == np.float16, a.dtype
    return a


def gemm_f16(A, B, C=None, *, b_is_nk=False, alpha=1.0, beta=0.0, act=0):
    """D = epilogue(alpha * A.B + beta * C); A [..., K]; B [K, N] (or [N, K] if b_is_nk)."""
    A, B = _f16(A), _f16(B)
    K = A.shape[-1]
    M = A.size // K
    B2 = B.reshape(B.shape[-2], B.shape[-1])
    N = B2.shape[0] if b_is_nk else B2.shape[1]
    assert (B2.shape[1] if b_is_nk else B2.shape[0]) == K
    c_mode = 0
    if C is not None and beta != 0.0:
        C = _f16(C)
        c_mode = 1 if C.size == M * N else 2
        assert C.size in (M * N, N)
    D = np.empty(A.shape[:-1] + (N,), dtype=np.float16)
    lib().oracle_gemm_f16(_p(A), _p(B2), c_int(int(b_is_nk)), _p(C) if c_mode else None,
                          c_int(c_mode), _p(D), c_int64(M), c_int64(N), c_int64(K),
                          c_float(alpha), c_float(beta), c_int(act))
    return D


def layernorm_f16(x, eps, res=None, gamma=None, beta=None):
    x = _f16(x)
    hidden = x.shape[-1]
    rows = x.size // hidden
    out = np.empty_like(x)
    res = None if res is None else _f16(res)
    gamma = None if gamma is None else _f16(gamma)
    beta = None if beta is None else _f16(beta)
    lib().oracle_layernorm_f16(_p(x), _p(res), _p(gamma), _p(beta), _p(out), c_int64(rows),
                               c_int64(hidden), c_float(eps))
    return out


def row_stats_f16(x, eps):
    """(rstd, shift) per row of x, fp16: the Var / Mean outputs of cutlassGemmWithVarMeanF16."""
    x = _f16(x)
    n = x.shape[-1]
    rows = x.size // n
    rstd = np.empty(rows, dtype=np.float16)
    shift = np.empty(rows, dtype=np.float16)
    lib().oracle_row_stats_f16(_p(x), _p(rstd), _p(shift), c_int64(rows), c_int64(n), c_float(eps))
    return rstd, shift


def layernorm_gemm_f16(A, rstd, shift, B, C=None, *, alpha=1.0, beta=0.0):
    """D = alpha * (A * rstd[r] + shift[r]).B + beta * C  (cutlassLayernormGemmF16)."""
    A, B = _f16(A), _f16(B)
    K = A.shape[-1]
    M = A.size // K
    B2 = B.reshape(B.shape[-2], B.shape[-1])
    N = B2.shape[1]
    c_mode = 0
    if C is not None and beta != 0.0:
        C = _f16(C)
        c_mode = 1 if C.size == M * N else 2
    D = np.empty(A.shape[:-1] + (N,), dtype=np.float16)
    lib().oracle_layernorm_gemm_f16(_p(A), _p(_f16(rstd)), _p(_f16(shift)), _p(B2),
                                    _p(C) if c_mode else None, c_int(c_mode), _p(D), c_int64(M),
                                    c_int64(N), c_int64(K), c_float(alpha), c_float(beta))
    return D


def layernorm_f32(x, eps):
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty_like(x)
    hidden = x.shape[-1]
    lib().oracle_layernorm_f32(_p(x), _p(out), c_int64(x.size // hidden), c_int64(hidden),
                               c_float(eps))
    return out


def attention_f16(qkv, cu_seqlens, heads, scale):
    """qkv [bs, seq, 3*heads*d] fp16, cu_seqlens int32 [bs+1] -> out [bs, seq, heads*d]."""
    qkv = _f16(qkv)
    bs, seq, three_hd = qkv.shape
    d = three_hd // (3 * heads)
    cu = np.ascontiguousarray(cu_seqlens, dtype=np.int32)
    out = np.empty((bs, seq, heads * d), dtype=np.float16)
    lib().oracle_attention_f16(_p(qkv), _p(cu), _p(out), c_int64(bs), c_int64(seq),
                               c_int64(heads), c_int64(d), c_float(scale))
    return out


def cu_seqlen(mask):
    mask = np.ascontiguousarray(mask)
    bs, seq = mask.shape
    out = np.empty(bs + 1, dtype=np.int32)
    if mask.dtype == np.int64:
        lib().oracle_cu_seqlen_i64(_p(mask), _p(out), c_int64(bs), c_int64(seq))
    else:
        assert mask.dtype == np.int32
        lib().oracle_cu_seqlen_i32(_p(mask), _p(out), c_int64(bs), c_int64(seq))
    return out


_OPS = {"Add": 0, "Sub": 1, "Mul": 2, "Div": 3}


def elementwise(op: str, a, b):
    a, b = np.ascontiguousarray(a), np.ascontiguousarray(b)
    assert a.ndim == b.ndim and a.dtype == b.dtype
    out = np.empty_like(a)
    sa = (c_int64 * a.ndim)(*a.shape)
    sb = (c_int64 * a.ndim)(*b.shape)
    fn = lib().oracle_elementwise_f16 if a.dtype == np.float16 else lib().oracle_elementwise_f32
    fn(c_int(_OPS[op]), _p(a), _p(b), _p(out), c_int(a.ndim), sa, sb)
    return out


def gather(indices, table):
    """indices int64 [bs, seq]; table [1, V, H] -> [bs, seq, H]."""
    idx = np.ascontiguousarray(indices, dtype=np.int64)
    table = np.ascontiguousarray(table)
    vocab, hidden = table.shape[-2], table.shape[-1]
    out = np.empty(idx.shape + (hidden,), dtype=table.dtype)
    lib().oracle_gather(_p(idx), _p(table), _p(out), c_int64(idx.size), c_int64(vocab),
                        c_int64(hidden), c_int64(table.dtype.itemsize))
    return out


def f32_to_f16(x):
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, dtype=np.float16)
    lib().oracle_f32_to_f16(_p(x), _p(out), c_int64(x.size))
    return out


def gelu_tosa_poly_f32(x):
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty_like(x)
    lib().oracle_gelu_tosa_poly_f32(_p(x), _p(out), c_int64(x.size))
    return out


def parse_constant_text(path) -> np.ndarray:
    """Weight text file: first line three dimensions, then the values
    (writer lib/WeightsEngine/WeightsEngine.cpp:22-39)."""
    with open(path) as f:
        dims = [int(t) for t in f.readline().split()]
        vals = np.array(f.read().split(), dtype=np.float32)
    return vals.reshape(dims)


def bert_encoder(weights: dict, input_ids, attention_mask, token_type_ids, *, heads: int,
                 eps: float = 1e-12, layers: int | None = None):
    """BERT encoder forward as the lowered model runs it, every op output rounded to fp16.

    Per forward: cu_seqlens from the mask; embeddings = (gather(word) + gather(type)) + position
    then LayerNorm; per layer: QKV GEMM, attention, output GEMM with the residual as C
    (beta = 1), LayerNorm in place, FFN1 GEMM with erf GELU, FFN2 GEMM with the residual as
    C, LayerNorm in place.  There are no biases and no LayerNorm affine (the lowering has no
    pattern for them).  `weights` holds fp16 arrays: word_emb [1,V,H], pos_emb [1,S,H],
    type_emb [1,2,H], and per layer i: wqkv_i [1,H,3H], wo_i [1,H,H], w1_i [1,H,F], w2_i [1,F,H].
    """
    ids = np.ascontiguousarray(input_ids, dtype=np.int64)
    bs, seq = ids.shape
    cu = cu_seqlen(np.ascontiguousarray(attention_mask, dtype=np.int64))
    x = gather(ids, weights["word_emb"])
    t = gather(np.ascontiguousarray(token_type_ids, dtype=np.int64), weights["type_emb"])
    x = elementwise("Add", x, t)
    x = elementwise("Add", x, np.ascontiguousarray(weights["pos_emb"][:, :seq, :]))
    x = layernorm_f16(x, eps)
    n_layers = layers if layers is not None else sum(1 for k in weights if k.startswith("wqkv_"))
    hidden = x.shape[-1]
    scale = 1.0 / float(np.sqrt(hidden // heads))
    for i in range(n_layers):
        qkv = gemm_f16(x, weights[f"wqkv_{i}"])
        ctx = attention_f16(qkv, cu, heads, scale)
        y = gemm_f16(ctx, weights[f"wo_{i}"], x, beta=1.0)
        y = layernorm_f16(y, eps)
        z = gemm_f16(y, weights[f"w1_{i}"], act=1)
        y2 = gemm_f16(z, weights[f"w2_{i}"], y, beta=1.0)
        x = layernorm_f16(y2, eps)
    return x


# ----------------------------------------------------------------- oracle/_ref

class _Memref3(ctypes.Structure):
    _fields_ = [("basePtr", c_void_p), ("data", c_void_p), ("offset", c_int64),
                ("sizes", c_int64 * 3), ("strides", c_int64 * 3)]


def _memref3(a: np.ndarray) -> _Memref3:
    assert a.ndim == 3 and a.dtype == np.float32 and a.flags.c_contiguous
    m = _Memref3()
    m.basePtr = m.data = a.ctypes.data
    m.offset = 0
    for i in range(3):
        m.sizes[i] = a.shape[i]
        m.strides[i] = a.strides[i] // 4
    return m


def ref_available() -> bool:
    return REF_CPU_LIB.exists()


def ref_matmul_add_f32(A, B, C):
    """The reference's own CPU matmulAddF32 (lib/ExecutionEngine/HandsOnRunnerUtils.cpp:230-277),
    compiled from its source into oracle/_ref: D = broadcast(C) + A[0].B[0]; fp32, rank 3.
    Note that it always reads A's batch 0 (line 272), so callers use batch 1."""
    ref = ctypes.CDLL(str(REF_CPU_LIB))
    A = np.ascontiguousarray(A, dtype=np.float32)
    B = np.ascontiguousarray(B, dtype=np.float32)
    C = np.ascontiguousarray(C, dtype=np.float32)
    D = np.zeros((A.shape[0], A.shape[1], B.shape[2]), dtype=np.float32)
    ms = [_memref3(t) for t in (A, B, C, D)]
    args = []
    for m in ms:
        args += [c_int64(3), ctypes.byref(m)]
    ref.matmulAddF32(*args)
    return D

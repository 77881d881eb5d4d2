"""Randomised shapes (hypothesis, derandomised so every run sees the same cases) through the C
ABI against the CPU oracle: tails in M / N / K, every tile-table row, both weight layouts,
ragged and empty sequences, odd hidden sizes, every broadcast pattern."""
import numpy as np
import pytest
from hypothesis import HealthCheck, given, settings, strategies as st

from util import assert_bits_equal, assert_close_f16, to_dev

pytestmark = pytest.mark.gpu

# The `cuda` fixture only selects the device and binds the library to torch's stream; nothing in
# it needs resetting between generated inputs.
settings.register_profile("hom-gpu", max_examples=30, deadline=None, derandomize=True,
                          suppress_health_check=[HealthCheck.function_scoped_fixture])
settings.load_profile("hom-gpu")


def _rng(seed):
    return np.random.Generator(np.random.PCG64(seed))


@given(bs=st.integers(1, 3), m=st.integers(1, 300), n8=st.integers(1, 80), k8=st.integers(1, 70),
       tile=st.integers(0, 6), nk=st.booleans(), act=st.integers(0, 1),
       cmode=st.sampled_from(["none", "full", "alias", "bias"]), seed=st.integers(0, 2 ** 31))
def test_gemm_random_shapes(hom, cuda, oracle, bs, m, n8, k8, tile, nk, act, cmode, seed):
    import torch
    n, k = 8 * n8, 8 * k8
    rng = _rng(seed)
    A = rng.uniform(-1, 1, (bs, m, k)).astype(np.float16)
    B = rng.normal(0, 0.05, (1, n, k) if nk else (1, k, n)).astype(np.float16)
    C = None
    if cmode in ("full", "alias"):
        C = rng.uniform(-1, 1, (bs, m, n)).astype(np.float16)
    elif cmode == "bias":
        C = rng.uniform(-1, 1, (1, 1, n)).astype(np.float16)
    beta = 0.0 if C is None else 1.0
    alpha = 1.0 if nk else float(rng.choice([1.0, 0.5, -2.0]))
    tA, tB = to_dev(A, cuda), to_dev(B, cuda)
    if cmode == "alias":
        tD = to_dev(C, cuda)
        tC = tD
    else:
        tD = torch.full((bs, m, n), float("nan"), dtype=torch.float16, device=cuda)
        tC = to_dev(C, cuda) if C is not None else tD
    fn = hom.nvteGemmF16 if nk else hom.cutlassGemmF16
    fn(tA, tB, tC, tD, activation=act, alpha=alpha, beta=beta, gemmNum=tile)
    hom.synchronize()
    want = oracle.gemm_f16(A, B, C, b_is_nk=nk, alpha=alpha, beta=beta, act=act)
    assert_close_f16(tD.cpu().numpy(), want, f"gemm {bs}x{m}x{n}x{k} tile {tile} nk {nk} act {act} C {cmode}")


@given(m=st.integers(1, 200), n=st.integers(1, 300), k8=st.integers(1, 40), tile=st.integers(0, 6),
       seed=st.integers(0, 2 ** 31))
def test_gemm_nk_layout_any_n(hom, cuda, oracle, m, n, k8, tile, seed):
    """B as [1,N,K] takes every N (rows of D need not be 16-byte aligned)."""
    import torch
    k = 8 * k8
    rng = _rng(seed)
    A = rng.uniform(-1, 1, (1, m, k)).astype(np.float16)
    B = rng.normal(0, 0.05, (1, n, k)).astype(np.float16)
    C = rng.uniform(-1, 1, (1, m, n)).astype(np.float16)
    tD = to_dev(C, cuda)
    hom.nvteGemmF16(to_dev(A, cuda), to_dev(B, cuda), tD, tD, activation=0, alpha=1.0, beta=1.0, gemmNum=tile)
    hom.synchronize()
    want = oracle.gemm_f16(A, B, C, b_is_nk=True, beta=1.0)
    assert_close_f16(tD.cpu().numpy(), want, f"nk gemm {m}x{n}x{k} tile {tile}")


@given(bs=st.integers(1, 5), seq=st.integers(1, 300), heads=st.integers(1, 4), seed=st.integers(0, 2 ** 31))
def test_attention_random_shapes(hom, cuda, oracle, bs, seq, heads, seed):
    import torch
    rng = _rng(seed)
    qkv = rng.standard_normal((bs, seq, 3 * heads * 64)).astype(np.float16)
    lens = rng.integers(0, seq + 1, bs)  # empty sequences included
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    out = torch.full((bs, seq, heads * 64), float("nan"), dtype=torch.float16, device=cuda)
    hom.nvteBertAttentionF16(to_dev(qkv, cuda), to_dev(cu, cuda), out, 0.125, heads)
    hom.synchronize()
    want = oracle.attention_f16(qkv, cu, heads=heads, scale=0.125)
    assert_close_f16(out.cpu().numpy(), want, f"attention bs {bs} seq {seq} heads {heads} lens {lens}")


@given(rows=st.integers(1, 700), hidden=st.integers(1, 1100), rank3=st.booleans(), seed=st.integers(0, 2 ** 31))
def test_layernorm_random_shapes(hom, cuda, oracle, rows, hidden, rank3, seed):
    rng = _rng(seed)
    x = (rng.standard_normal((rows, hidden)) * rng.uniform(0.1, 4) + rng.uniform(-2, 2)).astype(np.float16)
    shape = (1, rows, hidden) if rank3 else (rows, hidden)
    t = to_dev(x.reshape(shape), cuda)
    hom.nvteLayernormF16(t, 1e-5)
    hom.synchronize()
    want = oracle.layernorm_f16(x, eps=1e-5).reshape(shape)
    assert_close_f16(t.cpu().numpy(), want, f"layernorm {rows}x{hidden}")


@given(op=st.sampled_from(["Add", "Sub", "Mul", "Div"]), dtype=st.sampled_from(["F16", "F32"]),
       dims=st.tuples(st.integers(1, 5), st.integers(1, 40), st.integers(1, 70)),
       bcast=st.tuples(st.booleans(), st.booleans(), st.booleans()), seed=st.integers(0, 2 ** 31))
def test_elementwise_random_broadcasts(hom, cuda, oracle, op, dtype, dims, bcast, seed):
    import torch
    rng = _rng(seed)
    npdt = np.float16 if dtype == "F16" else np.float32
    a = rng.uniform(-4, 4, dims).astype(npdt)
    bshape = tuple(1 if f else d for f, d in zip(bcast, dims))
    b = (rng.uniform(0.5, 4, bshape) * rng.choice([-1, 1], bshape)).astype(npdt)
    out = torch.empty(dims, dtype=torch.float16 if dtype == "F16" else torch.float32, device=cuda)
    hom.elementwise(op, dtype, to_dev(a, cuda), to_dev(b, cuda), out)
    hom.synchronize()
    assert_bits_equal(out.cpu().numpy(), oracle.elementwise(op, a, b), f"{op}{dtype} {dims} <- {bshape}")


@given(bs=st.integers(1, 6), seq=st.integers(1, 50), vocab=st.integers(1, 300), hidden=st.integers(1, 200),
       dtype=st.sampled_from(["F16", "F32"]), seed=st.integers(0, 2 ** 31))
def test_gather_random_shapes(hom, cuda, oracle, bs, seq, vocab, hidden, dtype, seed):
    import torch
    rng = _rng(seed)
    npdt = np.float16 if dtype == "F16" else np.float32
    table = rng.standard_normal((1, vocab, hidden)).astype(npdt)
    idx = rng.integers(-1, vocab + 1, (bs, seq)).astype(np.int64)  # one below / above the range too
    out = torch.empty((bs, seq, hidden), dtype=torch.float16 if dtype == "F16" else torch.float32, device=cuda)
    hom.gather(dtype, to_dev(idx, cuda), to_dev(table, cuda), out)
    hom.synchronize()
    assert_bits_equal(out.cpu().numpy(), oracle.gather(idx, table), f"gather{dtype} {bs}x{seq} V{vocab} H{hidden}")

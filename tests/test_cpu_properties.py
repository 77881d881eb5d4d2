"""Property tests (hypothesis) of the CPU checker and of the host-side helpers: the oracle's
integer / byte paths against numpy on arbitrary shapes, algebraic properties of its
floating-point paths, and the batch sharding used by the multi-GPU runs."""
import numpy as np
import pytest
from hypothesis import given, settings, strategies as st

settings.register_profile("hom", max_examples=40, deadline=None)
settings.load_profile("hom")


@given(st.integers(1, 40), st.integers(1, 70), st.integers(0, 2 ** 32 - 1))
def test_cu_seqlens_is_the_running_sum_of_row_sums(oracle, bs, seq, seed):
    rng = np.random.Generator(np.random.PCG64(seed))
    lens = rng.integers(0, seq + 1, bs)
    mask = (np.arange(seq)[None, :] < lens[:, None]).astype(np.int64)
    got = oracle.cu_seqlen(mask)
    assert got.dtype == np.int32 and got.shape == (bs + 1,)
    assert got[0] == 0 and np.array_equal(np.diff(got), lens)


@given(st.integers(0, 2 ** 32 - 1))
def test_f32_to_f16_is_round_to_nearest_even(oracle, seed):
    rng = np.random.Generator(np.random.PCG64(seed))
    bits = rng.integers(0, 2 ** 32, 4096, dtype=np.uint64).astype(np.uint32)
    x = bits.view(np.float32)
    x = np.concatenate([x, np.float32([0.0, -0.0, 65504.0, 65520.0, 65519.99, 5.96e-8, 2.98e-8, 2.99e-8,
                                      np.inf, -np.inf, 6.1e-5, 6.097e-5])])
    x = x[~np.isnan(x)]
    with np.errstate(over="ignore"):
        want = x.astype(np.float16)
    got = oracle.f32_to_f16(x)
    assert np.array_equal(got.view(np.uint16), want.view(np.uint16))


@given(st.sampled_from(["Add", "Sub", "Mul", "Div"]), st.integers(1, 4), st.integers(1, 5), st.integers(1, 9),
       st.tuples(st.booleans(), st.booleans(), st.booleans()), st.integers(0, 2 ** 32 - 1))
def test_elementwise_broadcast_matches_numpy_fp16(oracle, op, d0, d1, d2, bcast, seed):
    rng = np.random.Generator(np.random.PCG64(seed))
    a = rng.uniform(-4, 4, (d0, d1, d2)).astype(np.float16)
    bshape = tuple(1 if b else d for b, d in zip(bcast, (d0, d1, d2)))
    b = rng.uniform(0.5, 4, bshape).astype(np.float16) * rng.choice([-1, 1], bshape).astype(np.float16)
    fn = {"Add": np.add, "Sub": np.subtract, "Mul": np.multiply, "Div": np.divide}[op]
    want = fn(a.astype(np.float32), np.broadcast_to(b, a.shape).astype(np.float32)).astype(np.float16)
    got = oracle.elementwise(op, a, b)
    # one rounding of the exact result: fp32 holds fp16 sums / products / quotients exactly enough
    assert np.array_equal(got.view(np.uint16), want.view(np.uint16))


@given(st.integers(1, 6), st.integers(1, 17), st.integers(1, 50), st.integers(1, 33), st.integers(0, 2 ** 32 - 1))
def test_gather_copies_rows_and_zeroes_out_of_range(oracle, bs, seq, vocab, hidden, seed):
    rng = np.random.Generator(np.random.PCG64(seed))
    table = rng.standard_normal((1, vocab, hidden)).astype(np.float16)
    idx = rng.integers(-2, vocab + 2, (bs, seq)).astype(np.int64)
    got = oracle.gather(idx, table)
    ok = (idx >= 0) & (idx < vocab)
    want = np.where(ok[..., None], table[0][np.clip(idx, 0, vocab - 1)], np.float16(0))
    assert np.array_equal(got.view(np.uint16), want.view(np.uint16))


@given(st.integers(1, 9), st.integers(8, 96), st.floats(0.25, 8.0), st.floats(-3.0, 3.0), st.integers(0, 2 ** 32 - 1))
def test_layernorm_is_invariant_to_affine_changes_of_its_input(oracle, rows, hidden, scale, shift, seed):
    """LayerNorm(a*x + b) = LayerNorm(x) for a > 0 (up to the fp16 rounding of the inputs, which
    the test removes by choosing a, b as powers of two / small integers where it matters)."""
    rng = np.random.Generator(np.random.PCG64(seed))
    x = rng.standard_normal((rows, hidden)).astype(np.float16)
    base = oracle.layernorm_f16(x, eps=0.0).astype(np.float32)
    a = np.float32(2.0 ** np.round(np.log2(scale)))
    b = np.float32(np.round(shift))
    moved = (x.astype(np.float32) * a + b).astype(np.float16)
    # only rows whose transformed values are still exact in fp16 are comparable bit-tight
    exact = (moved.astype(np.float32) == x.astype(np.float32) * a + b).all(axis=1)
    got = oracle.layernorm_f16(moved, eps=0.0).astype(np.float32)
    assert np.allclose(got[exact], base[exact], rtol=2e-3, atol=2e-3)
    # rows of a LayerNorm output have mean 0 and variance 1 up to fp16 rounding
    assert np.all(np.abs(base.mean(axis=1)) < 5e-3)
    if hidden >= 16:
        keep = x.astype(np.float32).std(axis=1) > 0.2
        assert np.all(np.abs(base.var(axis=1)[keep] - 1.0) < 2e-2)


@given(st.integers(1, 5), st.integers(1, 40), st.integers(8, 64), st.integers(1, 48), st.integers(0, 2 ** 32 - 1))
def test_gemm_is_linear_in_c_and_matches_float64(oracle, bs, m, k8, n, seed):
    rng = np.random.Generator(np.random.PCG64(seed))
    k = (k8 // 8) * 8
    a = rng.uniform(-1, 1, (bs, m, k)).astype(np.float16)
    b = rng.normal(0, 0.1, (1, k, n)).astype(np.float16)
    c = rng.uniform(-1, 1, (bs, m, n)).astype(np.float16)
    exact = a.astype(np.float64) @ b[0].astype(np.float64)
    plain = oracle.gemm_f16(a, b).astype(np.float64)
    assert np.allclose(plain, exact, rtol=1e-3, atol=1e-3)
    with_c = oracle.gemm_f16(a, b, c, alpha=0.5, beta=2.0).astype(np.float64)
    assert np.allclose(with_c, 0.5 * exact + 2.0 * c.astype(np.float64), rtol=1e-3, atol=2e-3)
    nk = oracle.gemm_f16(a, np.ascontiguousarray(b.transpose(0, 2, 1)), b_is_nk=True)
    assert np.array_equal(nk.view(np.uint16), oracle.gemm_f16(a, b).view(np.uint16))


@given(st.integers(1, 4), st.integers(1, 3), st.integers(2, 40), st.integers(0, 2 ** 32 - 1))
def test_attention_rows_are_convex_combinations_of_the_valid_values(oracle, bs, heads, seq, seed):
    rng = np.random.Generator(np.random.PCG64(seed))
    d = 64
    qkv = rng.standard_normal((bs, seq, 3 * heads * d)).astype(np.float16)
    lens = rng.integers(1, seq + 1, bs)
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    out = oracle.attention_f16(qkv, cu, heads=heads, scale=0.125).astype(np.float32)
    v = qkv.reshape(bs, seq, 3, heads, d)[:, :, 2].astype(np.float32)
    for b in range(bs):
        n = lens[b]
        o = out[b, :n].reshape(n, heads, d)
        lo, hi = v[b, :n].min(axis=0), v[b, :n].max(axis=0)
        assert np.all(o >= lo[None] - 2e-3) and np.all(o <= hi[None] + 2e-3)
        assert not out[b, n:].any()  # padded query rows are zeros


@given(st.integers(1, 64), st.integers(1, 8))
def test_shard_batch_partitions_the_batch(pkg, per_rank, world):
    from hands_on_mlir_b200.bert_program import shard_batch
    total = per_rank * world
    spans = [shard_batch(total, world, r) for r in range(world)]
    assert spans[0][0] == 0 and spans[-1][1] == total
    assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
    assert all(hi - lo == per_rank for lo, hi in spans)
    if world > 1:
        with pytest.raises(ValueError):
            shard_batch(total + 1, world, 0)

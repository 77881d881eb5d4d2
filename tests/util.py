"""Helpers shared by the parity tests."""
import numpy as np

RTOL = 1e-3  # fp16 parity tolerance stated for this path: rtol 1e-3 / atol 1e-3
ATOL = 1e-3


def to_dev(x, dev):
    import torch
    return torch.from_numpy(np.ascontiguousarray(x)).to(dev)


def assert_close_f16(got, want, what="", rtol=RTOL, atol=ATOL):
    got = np.asarray(got).astype(np.float64)
    want = np.asarray(want).astype(np.float64)
    assert got.shape == want.shape, (got.shape, want.shape)
    err = np.abs(got - want)
    tol = atol + rtol * np.abs(want)
    bad = ~(err <= tol)
    if bad.any():
        idx = np.unravel_index(np.argmax(np.where(bad, err, 0)), err.shape)
        raise AssertionError(
            f"{what}: {bad.sum()} of {bad.size} elements outside rtol={rtol} atol={atol}; "
            f"worst at {idx}: got {got[idx]!r} want {want[idx]!r} (max abs err {err.max():.3e})")


def assert_bits_equal(got, want, what=""):
    got, want = np.asarray(got), np.asarray(want)
    assert got.shape == want.shape and got.dtype == want.dtype, (got.shape, want.shape)
    g = got.view(np.uint16 if got.dtype == np.float16 else np.uint32 if got.dtype == np.float32 else got.dtype)
    w = want.view(g.dtype)
    if not np.array_equal(g, w):
        bad = np.argwhere(g != w)
        i = tuple(bad[0])
        raise AssertionError(f"{what}: {len(bad)} elements differ bitwise; first at {i}: "
                             f"got {got[i]!r} want {want[i]!r}")


def assert_end_to_end_close(got, want, what=""):
    """End-to-end criterion for final hidden states after several layers.

    rtol 1e-3 is one fp16 ulp, so two correct implementations that round an intermediate
    differently (fp32 tensor-core accumulation here, double accumulation in the oracle) drift
    by a few ulps after a few layers.  Required: at least 99.9 % of the elements within
    rtol 1e-3 / atol 1e-3, and every element within the reference's own end-to-end bound
    (abs <= 1e-2 or rel <= 1e-2, examples/torch/bert/bert.cu:148-153)."""
    got = np.asarray(got).astype(np.float64)
    want = np.asarray(want).astype(np.float64)
    assert got.shape == want.shape
    assert np.isfinite(got).all(), f"{what}: non-finite output"
    err = np.abs(got - want)
    tight = err <= ATOL + RTOL * np.abs(want)
    frac = 1.0 - tight.mean()
    assert frac <= 1e-3, f"{what}: {frac:.2%} of elements outside rtol/atol 1e-3 (max err {err.max():.3e})"
    loose = (err <= 1e-2) | (err <= 1e-2 * np.abs(want))
    assert loose.all(), f"{what}: max abs err {err.max():.3e} exceeds the 1e-2 end-to-end bound"


def drift_fractions(got, want):
    """Fractions of elements outside rtol/atol 1e-3, outside 2e-3, and outside the reference's
    own end-to-end bound (abs <= 1e-2 or rel <= 1e-2, examples/torch/bert/bert.cu:148-153)."""
    got = np.asarray(got).astype(np.float64)
    want = np.asarray(want).astype(np.float64)
    assert got.shape == want.shape and np.isfinite(got).all()
    err, mag = np.abs(got - want), np.abs(want)
    return (float(np.mean(err > 1e-3 + 1e-3 * mag)), float(np.mean(err > 2e-3 + 2e-3 * mag)),
            float(np.mean((err > 1e-2) & (err > 1e-2 * mag))))


def encoder_fp64(weights, input_ids, attention_mask, token_type_ids, *, heads, eps=1e-12, layers=None,
                 return_layers=False):
    """The encoder in float64 with no intermediate rounding at all (weights and embeddings are
    the given fp16 values): the mathematical result both fp16 pipelines approximate.  Same op
    order as the oracle's `bert_encoder`; padded key columns are excluded from the softmax and
    padded query rows come back as zeros."""
    from scipy.special import erf
    ids = np.asarray(input_ids)
    bs, seq = ids.shape
    mask = np.asarray(attention_mask).astype(bool)
    w = {k: np.asarray(v).astype(np.float64) for k, v in weights.items()}

    def ln(z):
        mu = z.mean(-1, keepdims=True)
        var = ((z - mu) ** 2).mean(-1, keepdims=True)
        return (z - mu) / np.sqrt(var + eps)

    x = ln(w["word_emb"][0][ids] + w["type_emb"][0][np.asarray(token_type_ids)] + w["pos_emb"][0][None, :seq])
    n_layers = layers if layers is not None else sum(1 for k in w if k.startswith("wqkv_"))
    hidden = x.shape[-1]
    d = hidden // heads
    outs = []
    for i in range(n_layers):
        qkv = (x @ w[f"wqkv_{i}"][0]).reshape(bs, seq, 3, heads, d)
        q, k, v = (qkv[:, :, j].transpose(0, 2, 1, 3) for j in range(3))
        s = q @ k.transpose(0, 1, 3, 2) / np.sqrt(d)
        s = np.where(mask[:, None, None, :], s, -np.inf)
        s = s - s.max(-1, keepdims=True)
        p = np.exp(s)
        p /= p.sum(-1, keepdims=True)
        ctx = (p @ v).transpose(0, 2, 1, 3).reshape(bs, seq, hidden) * mask[:, :, None]
        y = ln(ctx @ w[f"wo_{i}"][0] + x)
        h = y @ w[f"w1_{i}"][0]
        h = 0.5 * h * (1.0 + erf(h / np.sqrt(2.0)))
        x = ln(h @ w[f"w2_{i}"][0] + y)
        if return_layers:
            outs.append(x)
    return outs if return_layers else x

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

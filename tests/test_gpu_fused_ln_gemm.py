"""The GEMM <-> LayerNorm-statistics pair (cutlassGemmWithVarMeanF16, cutlassLayernormGemmF16)
against the values the reference's own verify.py computes and against the CPU oracle."""
from pathlib import Path

import numpy as np
import pytest

from util import assert_close_f16, to_dev

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden"


def f16(x):
    return np.asarray(x, dtype=np.float32).astype(np.float16)


def run_pair(hom, dev, A, B, C2, eps, beta1=0.0, Cres=None):
    """D1 = A.B (+ Cres) with row statistics, then D2 = LN(D1).C2."""
    import torch
    bs, m, _ = A.shape
    n, n2 = B.shape[-1], C2.shape[-1]
    tD1 = to_dev(Cres, dev) if Cres is not None else torch.empty((bs, m, n), dtype=torch.float16, device=dev)
    var = torch.full((bs * m,), float("nan"), dtype=torch.float16, device=dev)
    mean = torch.full((bs * m,), float("nan"), dtype=torch.float16, device=dev)
    hom.cutlassGemmWithVarMeanF16(to_dev(A, dev), to_dev(B, dev), tD1, tD1, var, mean, 1.0, beta1, 0, eps)
    tD2 = torch.empty((bs, m, n2), dtype=torch.float16, device=dev)
    hom.cutlassLayernormGemmF16(tD1, to_dev(C2, dev), tD2, tD2, var, mean, 1.0, 0.0, 0)
    hom.synchronize()
    return tD1.cpu().numpy(), var.cpu().numpy(), mean.cpu().numpy(), tD2.cpu().numpy()


def test_verify_py_literals(hom, cuda, oracle):
    """A[4x32].B[32x8] with statistics (eps 1e-5), then LN(A.B).C[8x16]: the numbers
    examples/torch/layernorm/cuda/verify.py prints."""
    g = np.load(GOLDEN / "verify_gemm_ln_gemm.npz")
    a, b, c = f16(g["a"])[None], f16(g["b"])[None], f16(g["c"])[None]
    d1, var, mean, d2 = run_pair(hom, cuda, a, b, c, 1e-5)
    assert_close_f16(d1[0], g["ab"], "A.B")
    assert_close_f16(var, g["rstd"], "rstd", rtol=2e-3, atol=2e-3)
    assert_close_f16(mean, g["shift"], "-mean*rstd", rtol=4e-3, atol=4e-3)
    # the statistics are stored in fp16 (as in the reference): |shift| ~ 10 has an ulp of 8e-3,
    # which the second GEMM multiplies by the column sums of C (~4)
    assert_close_f16(d2[0], g["ln_ab_c"], "LN(A.B).C", rtol=1e-2, atol=4e-2)


@pytest.mark.parametrize("shape", [(2, 128, 256, 128, 320), (1, 300, 264, 72, 136), (32, 128, 768, 768, 3072)])
def test_against_oracle(hom, cuda, oracle, shape):
    bs, m, n, k, n2 = shape
    rng = np.random.Generator(np.random.PCG64(17))
    A = f16(rng.normal(0, 1, (bs, m, k)))
    B = f16(rng.normal(0, 0.05, (1, k, n)))
    R = f16(rng.normal(0.5, 1, (bs, m, n)))
    C2 = f16(rng.normal(0, 0.03, (1, n, n2)))
    d1, var, mean, d2 = run_pair(hom, cuda, A, B, C2, 1e-5, beta1=1.0, Cres=R)
    want1 = oracle.gemm_f16(A, B, R, beta=1.0)
    rows = np.arange(0, bs * m, 7) if bs * m > 1000 else np.arange(bs * m)
    assert_close_f16(d1.reshape(-1, n)[rows], want1.reshape(-1, n)[rows], "D1")
    # statistics and the second GEMM are checked on the GPU's own D1 (their input)
    w_var, w_mean = oracle.row_stats_f16(d1, 1e-5)
    assert_close_f16(var, w_var, "Var", rtol=2e-3, atol=2e-3)
    assert_close_f16(mean, w_mean, "Mean", rtol=2e-3, atol=2e-3)
    want2 = oracle.layernorm_gemm_f16(d1.reshape(-1, n)[rows], var[rows], mean[rows], C2)
    assert_close_f16(d2.reshape(-1, n2)[rows], want2, "D2", rtol=2e-3, atol=2e-3)


def test_rejects_bad_statistics_operands(hom, cuda, pkg):
    import torch
    A = torch.zeros((1, 128, 64), dtype=torch.float16, device=cuda)
    B = torch.zeros((1, 64, 64), dtype=torch.float16, device=cuda)
    D = torch.zeros((1, 128, 64), dtype=torch.float16, device=cuda)
    short = torch.zeros((100,), dtype=torch.float16, device=cuda)
    ok = torch.zeros((128,), dtype=torch.float16, device=cuda)
    with pytest.raises(pkg.HomError):
        hom.cutlassGemmWithVarMeanF16(A, B, D, D, short, ok)
    with pytest.raises(pkg.HomError):
        hom.cutlassLayernormGemmF16(A, B, D, D, ok, short)

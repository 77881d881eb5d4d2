"""homLayernormGemmF16NoAlloc - the LayerNorm-on-A GEMM for callers that cannot allocate device
memory (fixed memory budget, allocator locked, cudaMalloc would stall other streams).

It must give what cutlassLayernormGemmF16 gives.  Two calls in a row with different shapes
are checked, because the entry point keeps its column sums in one array built into the
library that every call shares and that still holds the previous call's values.  This file
is collected last so that a run stopping at the first failure has already run everything
else; the test does not depend on any other test having run.
"""
import numpy as np
import pytest

from util import assert_close_f16, to_dev

pytestmark = pytest.mark.gpu


def _case(hom, dev, oracle, seed, bs, m, k, n, with_c):
    import torch
    rng = np.random.Generator(np.random.PCG64(seed))
    f16 = lambda x: x.astype(np.float32).astype(np.float16)
    A = f16(rng.normal(0.3, 1.0, (bs, m, k)))
    B = f16(rng.normal(0.0, 0.05, (1, k, n)))
    C = f16(rng.normal(0.0, 1.0, (bs, m, n))) if with_c else None
    rstd, shift = oracle.row_stats_f16(A, 1e-5)
    tA, tB = to_dev(A, dev), to_dev(B, dev)
    tV, tM = to_dev(rstd, dev), to_dev(shift, dev)
    beta = 1.0 if with_c else 0.0
    # existing entry point (allocates its scratch with cudaMalloc on first use)
    d_ref = to_dev(C, dev) if with_c else torch.full((bs, m, n), float("nan"), dtype=torch.float16, device=dev)
    hom.cutlassLayernormGemmF16(tA, tB, d_ref, d_ref, tV, tM, 1.0, beta, 0)
    # the entry point under test
    d_new = to_dev(C, dev) if with_c else torch.full((bs, m, n), float("nan"), dtype=torch.float16, device=dev)
    hom.homLayernormGemmF16NoAlloc(tA, tB, d_new, d_new, tV, tM, 1.0, beta)
    hom.synchronize()
    got, ref = d_new.cpu().numpy(), d_ref.cpu().numpy()
    assert_close_f16(got, ref, f"no-alloc vs cutlassLayernormGemmF16 ({bs}x{m}x{n}x{k})")
    want = oracle.layernorm_gemm_f16(A, rstd, shift, B, C, beta=beta)
    assert_close_f16(got, want, "no-alloc vs oracle", rtol=2e-3, atol=2e-3)


def test_two_calls_in_a_row_match_the_allocating_entry_point(hom, cuda, oracle):
    # first call: wide N fills many scratch entries; second call: narrower N and other data,
    # so stale sums from the first call would show up if they were ever read
    _case(hom, cuda, oracle, seed=1, bs=2, m=128, k=256, n=1024, with_c=False)
    _case(hom, cuda, oracle, seed=2, bs=1, m=200, k=136, n=328, with_c=True)


def test_rejects_n_beyond_the_built_in_scratch(hom, cuda, pkg):
    import torch
    n = 16384 + 64
    A = torch.zeros((1, 8, 64), dtype=torch.float16, device=cuda)
    B = torch.zeros((1, 64, n), dtype=torch.float16, device=cuda)
    D = torch.zeros((1, 8, n), dtype=torch.float16, device=cuda)
    s = torch.zeros((8,), dtype=torch.float16, device=cuda)
    before = hom.launch_count()
    with pytest.raises(pkg.HomError) as e:
        hom.homLayernormGemmF16NoAlloc(A, B, D, D, s, s)
    assert e.value.code == 2 and "16384" in e.value.message
    assert hom.launch_count() == before

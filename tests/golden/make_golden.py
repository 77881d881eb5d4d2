"""Generates the committed golden fixtures under tests/golden/.

Run where a checkout of the reference and PyTorch are available:

    python tests/golden/make_golden.py REFERENCE_DIR

* verify_gemm_ln_gemm.npz — produced by EXECUTING the reference's own
  examples/torch/layernorm/cuda/verify.py (its literal A[4x32], B[32x8], C[8x16] and the
  values it computes with PyTorch: A.B, the fused-statistics form rstd / -mean*rstd, and
  LayerNorm(A.B).C).  Nothing of that script is copied into this repository; only its
  numeric inputs and outputs are stored.
* torch_ops.npz — seeded inputs (fp16-representable) and PyTorch CPU fp32 results for the
  ops of the hot path: GEMM + bias + erf GELU, LayerNorm (plain and residual + affine),
  padded packed-QKV attention.
"""
import contextlib
import io
import runpy
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def from_reference_verify(ref_dir: Path):
    script = ref_dir / "examples/torch/layernorm/cuda/verify.py"
    with contextlib.redirect_stdout(io.StringIO()):
        g = runpy.run_path(str(script))
    a, b, c, ab = g["a_tensor"], g["b_tensor"], g["c_tensor"], g["ab"]
    with torch.no_grad():
        out = g["ln"](ab) @ c
    np.savez(HERE / "verify_gemm_ln_gemm.npz", a=a.numpy(), b=b.numpy(), c=c.numpy(),
             ab=ab.numpy(), rstd=g["var"].numpy(), shift=g["new_mean"].numpy(),
             ln_ab_c=out.numpy())


def torch_ops():
    rng = np.random.Generator(np.random.PCG64(2024))
    f16 = lambda x: x.astype(np.float32).astype(np.float16)
    d = {}
    # GEMM + bias + erf GELU (distributions of the single-GEMM benchmark configuration)
    A = f16(rng.uniform(-1, 1, (2, 24, 64)))
    B = f16(rng.normal(0, 0.02, (1, 64, 48)))
    bias = f16(rng.uniform(-1, 1, (1, 1, 48)))
    tA, tB, tb = (torch.from_numpy(x.astype(np.float32)) for x in (A, B, bias))
    d.update(gemm_A=A, gemm_B=B, gemm_bias=bias,
             gemm_plain=(tA @ tB[0]).numpy(),
             gemm_bias_gelu=torch.nn.functional.gelu(tA @ tB[0] + tb).numpy())
    # LayerNorm
    x = f16(rng.normal(0, 1, (16, 768)))
    r = f16(rng.normal(0, 1, (16, 768)))
    gm = f16(1 + rng.normal(0, 0.1, 768))
    bt = f16(rng.normal(0, 0.1, 768))
    tx, tr, tg, tbt = (torch.from_numpy(v.astype(np.float32)) for v in (x, r, gm, bt))
    d.update(ln_x=x, ln_r=r, ln_gamma=gm, ln_beta=bt,
             ln_plain=torch.nn.functional.layer_norm(tx, (768,), eps=1e-12).numpy(),
             ln_res_affine=torch.nn.functional.layer_norm(tx + tr, (768,), tg, tbt, eps=1e-12).numpy())
    # Attention, packed QKV [bs, seq, 3, heads, 64], padding by valid length, scale 1/8
    bs, seq, heads, hd = 3, 128, 2, 64
    lens = np.array([128, 77, 1])
    qkv = f16(rng.normal(0, 1, (bs, seq, 3 * heads * hd)))
    t = torch.from_numpy(qkv.astype(np.float32)).view(bs, seq, 3, heads, hd)
    q, k, v = (t[:, :, i].permute(0, 2, 1, 3) for i in range(3))
    m = torch.from_numpy((np.arange(seq)[None, :] < lens[:, None]).astype(np.float32))
    add_mask = (1.0 - m)[:, None, None, :] * torch.finfo(torch.float32).min
    att = torch.softmax(q @ k.transpose(-1, -2) * 0.125 + add_mask, -1) @ v
    att = att.permute(0, 2, 1, 3).reshape(bs, seq, heads * hd) * m[:, :, None]
    d.update(attn_qkv=qkv, attn_lens=lens, attn_out=att.numpy())
    np.savez_compressed(HERE / "torch_ops.npz", **d)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: make_golden.py REFERENCE_DIR (the reference checkout to execute verify.py from)")
    ref = Path(sys.argv[1])
    from_reference_verify(ref)
    torch_ops()
    for f in sorted(HERE.glob("*.npz")):
        print(f.name, f.stat().st_size, "bytes")

"""The CPU oracle against everything that can pin it without a GPU: the values the
reference's own verify.py computes, its literal harness inputs, its own CPU GEMM compiled
from source (oracle/_ref), PyTorch CPU fp32 fixtures, and numpy's fp16 arithmetic."""
from pathlib import Path

import numpy as np
import pytest

from util import assert_bits_equal, assert_close_f16

GOLDEN = Path(__file__).resolve().parent / "golden"


def f16(x):
    return np.asarray(x, dtype=np.float32).astype(np.float16)


def test_verify_py_gemm_ln_gemm_chain(oracle):
    """A[4x32].B[32x8] -> LayerNorm(eps 1e-6) -> .C[8x16] with the literals of
    examples/torch/layernorm/cuda/verify.py; expected values are what that script computes."""
    g = np.load(GOLDEN / "verify_gemm_ln_gemm.npz")
    a, b, c = f16(g["a"]), f16(g["b"]), f16(g["c"])
    # the literals were printed from half tensors with 6 digits: fp16 casts reproduce them
    np.testing.assert_allclose(a.astype(np.float32), g["a"], rtol=1e-5)
    ab = oracle.gemm_f16(a[None], b[None])
    assert_close_f16(ab[0], g["ab"], "A.B", rtol=1e-3, atol=1e-3)
    ln = oracle.layernorm_f16(ab, 1e-6)
    out = oracle.gemm_f16(ln, c[None])
    # two fp16 roundings upstream of an 8-term dot product of O(1) values
    assert_close_f16(out[0], g["ln_ab_c"], "LN(A.B).C", rtol=4e-3, atol=4e-3)
    # the fused-statistics form: rstd = 1/sqrt(E[x^2] - mean^2 + 1e-5), shift = -mean * rstd
    abf = g["ab"].astype(np.float64)
    mean, sq = abf.mean(-1), (abf * abf).mean(-1)
    np.testing.assert_allclose(1 / np.sqrt(sq - mean * mean + 1e-5), g["rstd"], rtol=1e-5)
    np.testing.assert_allclose(-mean / np.sqrt(sq - mean * mean + 1e-5), g["shift"], rtol=1e-4)


def test_fused_statistics_pair_against_verify_py(oracle):
    """row_stats + layernorm_gemm (the cutlassGemmWithVarMeanF16 / cutlassLayernormGemmF16 pair)
    against verify.py's rstd, -mean*rstd and LN(A.B).C; the statistics are fp16 like the
    reference's, which bounds the accuracy of the second product."""
    g = np.load(GOLDEN / "verify_gemm_ln_gemm.npz")
    ab = oracle.gemm_f16(f16(g["a"])[None], f16(g["b"])[None])
    rstd, shift = oracle.row_stats_f16(ab, 1e-5)
    assert_close_f16(rstd, g["rstd"], "rstd", rtol=2e-3, atol=2e-3)
    assert_close_f16(shift, g["shift"], "shift", rtol=2e-3, atol=8e-3)
    d2 = oracle.layernorm_gemm_f16(ab, rstd, shift, f16(g["c"])[None])
    assert_close_f16(d2[0], g["ln_ab_c"], "LN(A.B).C", rtol=1e-2, atol=4e-2)
    # with exact fp32 statistics the same formula reproduces the golden values tightly
    abf = ab[0].astype(np.float64)
    mean, sq = abf.mean(-1), (abf * abf).mean(-1)
    r = 1 / np.sqrt(sq - mean * mean + 1e-6)
    want = ((abf - mean[:, None]) * r[:, None]) @ g["c"].astype(np.float64)
    np.testing.assert_allclose(want, g["ln_ab_c"], rtol=5e-3, atol=5e-3)


def test_gemm_against_torch_fixture(oracle):
    g = np.load(GOLDEN / "torch_ops.npz")
    A, B, bias = g["gemm_A"], g["gemm_B"], g["gemm_bias"]
    assert_close_f16(oracle.gemm_f16(A, B), g["gemm_plain"], "gemm")
    assert_close_f16(oracle.gemm_f16(A, B, bias, beta=1.0, act=1), g["gemm_bias_gelu"], "bias+gelu")
    Bt = np.ascontiguousarray(B.transpose(0, 2, 1))
    assert_bits_equal(oracle.gemm_f16(A, Bt, b_is_nk=True), oracle.gemm_f16(A, B), "[N,K] weights")


def test_layernorm_against_torch_fixture(oracle):
    g = np.load(GOLDEN / "torch_ops.npz")
    assert_close_f16(oracle.layernorm_f16(g["ln_x"], 1e-12), g["ln_plain"], "ln")
    got = oracle.layernorm_f16(g["ln_x"], 1e-12, g["ln_r"], g["ln_gamma"], g["ln_beta"])
    assert_close_f16(got, g["ln_res_affine"], "ln residual+affine")


def test_layernorm_reference_literal(oracle):
    import torch
    from golden.reference_literals import LAYERNORM_2x10
    want = torch.nn.functional.layer_norm(torch.from_numpy(LAYERNORM_2x10), (10,), eps=1e-5).numpy()
    np.testing.assert_allclose(oracle.layernorm_f32(LAYERNORM_2x10, 1e-5), want, rtol=1e-5, atol=1e-6)


def test_attention_against_torch_fixture(oracle):
    g = np.load(GOLDEN / "torch_ops.npz")
    lens = g["attn_lens"]
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    got = oracle.attention_f16(g["attn_qkv"], cu, 2, 0.125)
    assert_close_f16(got, g["attn_out"], "attention")
    for b, n in enumerate(lens):
        assert not got[b, n:].any()  # padded query rows are zeros


def test_matmul_add_matches_reference_cpu_kernel(oracle):
    """The reference's own matmulAddF32 (compiled from its source) on fp16-representable
    inputs, bias broadcast [1,1,N]."""
    if not oracle.ref_available():
        pytest.skip("oracle/_ref was not built (no reference checkout at build time)")
    rng = np.random.Generator(np.random.PCG64(5))
    A, B, C = f16(rng.uniform(-1, 1, (1, 40, 72))), f16(rng.normal(0, 0.1, (1, 72, 56))), \
        f16(rng.uniform(-1, 1, (1, 1, 56)))
    want = oracle.ref_matmul_add_f32(A.astype(np.float32), B.astype(np.float32), C.astype(np.float32))
    assert_close_f16(oracle.gemm_f16(A, B, C, beta=1.0), want, "matmulAddF32 bias")
    Cfull = f16(rng.uniform(-1, 1, (1, 40, 56)))
    want = oracle.ref_matmul_add_f32(A.astype(np.float32), B.astype(np.float32),
                                     Cfull.astype(np.float32))
    assert_close_f16(oracle.gemm_f16(A, B, Cfull, beta=1.0), want, "matmulAddF32 full C")


def test_fp16_rounding_is_round_to_nearest_even(oracle):
    rng = np.random.Generator(np.random.PCG64(6))
    x = (rng.standard_normal(200000) * np.exp(rng.uniform(-20, 11, 200000))).astype(np.float32)
    x = np.concatenate([x, np.array([0.0, -0.0, 65504.0, 65519.9, 65520.0, 1e6, -1e6, 2.0 ** -24,
                                     2.0 ** -25, 2.0 ** -25 * 1.0001, 6.1e-5, np.inf, -np.inf],
                                    dtype=np.float32)])
    with np.errstate(over="ignore"):
        want = x.astype(np.float16)
    assert_bits_equal(oracle.f32_to_f16(x), want, "f32->f16")


@pytest.mark.parametrize("op,fn", [("Add", np.add), ("Sub", np.subtract), ("Mul", np.multiply),
                                   ("Div", np.divide)])
def test_elementwise_matches_numpy_half_arithmetic(oracle, op, fn):
    rng = np.random.Generator(np.random.PCG64(7))
    a = f16(rng.normal(0, 4, (5, 7, 16)))
    for bshape in [(5, 7, 16), (1, 7, 16), (5, 1, 16), (5, 7, 1), (1, 1, 1)]:
        b = f16(rng.normal(0, 4, bshape) + 0.5)
        assert_bits_equal(oracle.elementwise(op, a, b), fn(a, b).astype(np.float16), f"{op} {bshape}")


def test_elementwise_reference_literal(oracle):
    from golden.reference_literals import ADD_A_3x3x3, ADD_B_3x1x3
    assert_bits_equal(oracle.elementwise("Add", ADD_A_3x3x3, ADD_B_3x1x3), ADD_A_3x3x3 + ADD_B_3x1x3)


def test_cu_seqlen_reference_table(oracle):
    from golden.reference_literals import CU_SEQLEN_VALID_LENGTHS
    lens = np.array(CU_SEQLEN_VALID_LENGTHS * 2)
    mask = (np.arange(64)[None, :] < lens[:, None]).astype(np.int64)
    np.testing.assert_array_equal(oracle.cu_seqlen(mask), np.concatenate([[0], np.cumsum(lens)]))
    np.testing.assert_array_equal(oracle.cu_seqlen(mask.astype(np.int32)),
                                  np.concatenate([[0], np.cumsum(lens)]))
    assert oracle.cu_seqlen(np.zeros((0, 5), dtype=np.int64)).tolist() == [0]


def test_gather_and_out_of_range(oracle):
    table = f16(np.arange(40).reshape(1, 5, 8))
    idx = np.array([[4, 0, 7], [1, 1, -1]], dtype=np.int64)
    got = oracle.gather(idx, table)
    np.testing.assert_array_equal(got[0, 0], table[0, 4])
    assert not got[0, 2].any() and not got[1, 2].any()


def test_gelu_tosa_polynomial_is_close_to_erf_gelu(oracle):
    import math
    x = np.linspace(-6, 6, 2001).astype(np.float32)
    want = np.array([0.5 * v * (1 + math.erf(v / math.sqrt(2))) for v in x], dtype=np.float32)
    assert np.abs(oracle.gelu_tosa_poly_f32(x) - want).max() < 2e-3


def test_constant_text_parser(oracle, tmp_path):
    vals = np.arange(24, dtype=np.float32).reshape(1, 4, 6) / 7
    (tmp_path / "3.txt").write_text("1 4 6\n" + " ".join(repr(float(v)) for v in vals.ravel()) + "\n")
    np.testing.assert_array_equal(oracle.parse_constant_text(tmp_path / "3.txt"), vals)


def test_encoder_composition_matches_torch_fp32(oracle):
    """The oracle's whole-encoder composition against a PyTorch fp32 encoder with the same
    (bias-free, affine-free) weights; tolerance 1e-2 as in the reference's own end-to-end
    check (examples/torch/bert/bert.cu:148-153)."""
    import torch
    rng = np.random.Generator(np.random.PCG64(8))
    L, H, heads, F, V, S, B = 2, 128, 2, 256, 50, 128, 2
    w = {"word_emb": f16(rng.normal(0, 0.02, (1, V, H))), "pos_emb": f16(rng.normal(0, 0.02, (1, S, H))),
         "type_emb": f16(rng.normal(0, 0.02, (1, 2, H)))}
    for i in range(L):
        w[f"wqkv_{i}"] = f16(rng.normal(0, 0.02, (1, H, 3 * H)))
        w[f"wo_{i}"] = f16(rng.normal(0, 0.02, (1, H, H)))
        w[f"w1_{i}"] = f16(rng.normal(0, 0.02, (1, H, F)))
        w[f"w2_{i}"] = f16(rng.normal(0, 0.02, (1, F, H)))
    lens = np.array([128, 90])
    ids = rng.integers(0, V, (B, S)).astype(np.int64)
    mask = (np.arange(S)[None, :] < lens[:, None]).astype(np.int64)
    types = np.zeros((B, S), dtype=np.int64)
    got = oracle.bert_encoder(w, ids, mask, types, heads=heads, eps=1e-12).astype(np.float32)

    t = {k: torch.from_numpy(v.astype(np.float32)) for k, v in w.items()}
    ln = lambda z: torch.nn.functional.layer_norm(z, (H,), eps=1e-12)
    x = ln(t["word_emb"][0][torch.from_numpy(ids)] + t["type_emb"][0][0] + t["pos_emb"][0][None])
    add_mask = (1.0 - torch.from_numpy(mask).float())[:, None, None, :] * torch.finfo(torch.float32).min
    for i in range(L):
        qkv = (x @ t[f"wqkv_{i}"][0]).view(B, S, 3, heads, H // heads)
        q, k, v = (qkv[:, :, j].permute(0, 2, 1, 3) for j in range(3))
        a = torch.softmax(q @ k.transpose(-1, -2) / (H // heads) ** 0.5 + add_mask, -1) @ v
        a = a.permute(0, 2, 1, 3).reshape(B, S, H) * torch.from_numpy(mask).float()[:, :, None]
        x = ln(a @ t[f"wo_{i}"][0] + x)
        x = ln(torch.nn.functional.gelu(x @ t[f"w1_{i}"][0]) @ t[f"w2_{i}"][0] + x)
    want = x.numpy()
    for b, n in enumerate(lens):  # the reference compares valid tokens only
        assert_close_f16(got[b, :n], want[b, :n], f"encoder seq {b}", rtol=1e-2, atol=1e-2)


def test_encoder_composition_matches_huggingface_bert_model(oracle):
    """The oracle's encoder against the model class the reference exports
    (examples/torch/bert/convert_hf.py:44-45 builds a Hugging Face BERT and lowers it): a
    randomly initialised `BertModel` in fp32 with its weights rounded to fp16 and handed to the
    oracle in the layout the lowering produces (Wq|Wk|Wv concatenated along the output
    dimension, lib/Conversions/HOM/HOMFusionPass.cpp:317-346).  Pins the embedding order, the
    position ids, the post-LayerNorm placement and the packed-QKV head order.  Valid tokens
    only, tolerance 1e-2 as in the reference's end-to-end check (bert.cu:148-153)."""
    import torch
    transformers = pytest.importorskip("transformers")
    L, H, heads, F, V, S, B = 2, 128, 2, 256, 60, 64, 3
    cfg = transformers.BertConfig(vocab_size=V, hidden_size=H, num_hidden_layers=L, num_attention_heads=heads,
                                  intermediate_size=F, max_position_embeddings=S, type_vocab_size=2,
                                  hidden_act="gelu", layer_norm_eps=1e-12, hidden_dropout_prob=0.0,
                                  attention_probs_dropout_prob=0.0)
    torch.manual_seed(3)
    model = transformers.BertModel(cfg, add_pooling_layer=False).eval()
    with torch.no_grad():
        for name, prm in model.named_parameters():
            if name.endswith("LayerNorm.weight"):
                prm.fill_(1.0)
            elif name.endswith(".bias"):
                prm.zero_()  # the lowered model has neither biases nor LayerNorm affine
            else:
                prm.copy_(prm.half().float())  # both sides see the same fp16 weights
    sd = {k: v.detach().numpy() for k, v in model.state_dict().items()}
    w = {"word_emb": f16(sd["embeddings.word_embeddings.weight"][None]),
         "pos_emb": f16(sd["embeddings.position_embeddings.weight"][None]),
         "type_emb": f16(sd["embeddings.token_type_embeddings.weight"][None])}
    for i in range(L):
        pre = f"encoder.layer.{i}."
        wq, wk, wv = (sd[pre + f"attention.self.{n}.weight"].T for n in ("query", "key", "value"))
        w[f"wqkv_{i}"] = f16(np.concatenate([wq, wk, wv], axis=1)[None])
        w[f"wo_{i}"] = f16(sd[pre + "attention.output.dense.weight"].T[None])
        w[f"w1_{i}"] = f16(sd[pre + "intermediate.dense.weight"].T[None])
        w[f"w2_{i}"] = f16(sd[pre + "output.dense.weight"].T[None])
    rng = np.random.Generator(np.random.PCG64(21))
    lens = np.array([64, 40, 17])
    ids = rng.integers(0, V, (B, S)).astype(np.int64)
    mask = (np.arange(S)[None, :] < lens[:, None]).astype(np.int64)
    types = rng.integers(0, 2, (B, S)).astype(np.int64)
    got = oracle.bert_encoder(w, ids, mask, types, heads=heads, eps=1e-12).astype(np.float32)
    with torch.no_grad():
        want = model(input_ids=torch.from_numpy(ids), attention_mask=torch.from_numpy(mask),
                     token_type_ids=torch.from_numpy(types)).last_hidden_state.numpy()
    for b, n in enumerate(lens):
        assert_close_f16(got[b, :n], want[b, :n], f"HF BertModel seq {b}", rtol=1e-2, atol=1e-2)

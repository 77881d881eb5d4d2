"""Child process of test_gpu_cold_start.py: runs a few cases once each in a fresh process (first
launch of every kernel, freshly allocated device memory filled with NaNs beforehand) and prints
one checksum per case on the last line of stdout."""
import hashlib
import sys
from pathlib import Path

import numpy as np
import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
import __graft_entry__ as entry  # noqa: E402

pkg = entry.load_package()
from hands_on_mlir_b200.bert_program import BertConfig, BertProgram  # noqa: E402

hom = pkg.runner()
dev = torch.device("cuda:0")
torch.cuda.set_device(0)
hom.use_torch_stream()
junk = [torch.full((32 << 20,), float("nan"), dtype=torch.float16, device=dev) for _ in range(4)]
del junk
torch.cuda.empty_cache()
gen = torch.Generator(device=dev)
gen.manual_seed(5)


def mk(*shape, scale=1.0):
    return (torch.randn(*shape, generator=gen, device=dev) * scale).half()


def digest(t):
    return hashlib.md5(t.detach().cpu().numpy().tobytes()).hexdigest()[:8]


out = []
# GEMMs: CTA-pair tile, one-CTA tile with residual, GELU, a K split, an odd shape
for (m, n, k, act, res, split) in [(4096, 2304, 768, 0, False, 1), (4096, 768, 3072, 0, True, 1),
                                   (4096, 3072, 768, 1, False, 1), (1024, 1024, 4096, 0, False, 3),
                                   (300, 264, 200, 1, True, 1)]:
    A, B = mk(1, m, k), mk(1, k, n, scale=0.03)
    D = mk(1, m, n) if res else torch.empty(1, m, n, dtype=torch.half, device=dev)
    hom.cutlassGemmF16(A, B, D, D, beta=1.0 if res else 0.0, activation=act, splitKFactor=split)
    hom.synchronize()
    out.append(digest(D))
# attention: one KV tile, and several with a last tile of one or a few valid keys
for (S, H, lens) in [(128, 12, [128, 64, 100, 17, 1, 0, 77, 128]), (512, 16, [512, 257, 384, 300, 411, 256, 129, 1])]:
    qkv = mk(len(lens), S, 3 * H * 64)
    cu = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32, device=dev)
    o = torch.empty(len(lens), S, H * 64, dtype=torch.half, device=dev)
    hom.nvteBertAttentionF16(qkv, cu, o, 0.125, H)
    hom.synchronize()
    valid = torch.arange(S, device=dev)[None, :] < torch.tensor(lens, device=dev)[:, None]
    out.append(digest(o[valid]))
# an encoder at BERT-large width with ragged lengths, eagerly and as a replayed graph
rng = np.random.Generator(np.random.PCG64(12))
cfg = BertConfig(layers=3, hidden=1024, heads=16, ffn=4096)
B, S, lens = 3, 512, np.array([257, 512, 300])
w = {n: torch.from_numpy(rng.normal(0, 0.02, cfg.weight_shape(n, S)).astype(np.float16)).to(dev)
     for n in cfg.weight_names()}
ids = torch.from_numpy(rng.integers(0, cfg.vocab, (B, S)).astype(np.int64)).to(dev)
mask = torch.from_numpy((np.arange(S)[None, :] < lens[:, None]).astype(np.int64)).to(dev)
types = torch.zeros_like(ids)
prog = BertProgram(cfg, B, S)
prog.set_weights(w)
res = prog.forward(ids, mask, types, use_graph=False)
eager = prog.result_to_torch(res)[mask.bool()].clone()
hom.synchronize()
for _ in range(3):
    res = prog.forward(ids, mask, types, use_graph=True)
replay = prog.result_to_torch(res)[mask.bool()].clone()
hom.synchronize()
out.append(digest(eager) + ("=" if torch.equal(eager, replay) else "/" + digest(replay)))
prog.close()
print(" ".join(out), flush=True)

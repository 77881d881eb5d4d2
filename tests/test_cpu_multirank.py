"""The multi-GPU plan on CPU: world_size 2 over gloo.  Each rank runs its shard of the batch
(here through the CPU oracle, since there is no GPU) and the final gather reassembles the
global result; it must equal the single-process result bit for bit, because sequences are
independent and there is no collective on the data path."""
import os
import sys
from pathlib import Path

import numpy as np
import pytest

REPO = Path(__file__).resolve().parents[1]


def _tiny_weights(rng, L, H, F, V, S):
    f16 = lambda x: x.astype(np.float32).astype(np.float16)
    w = {"word_emb": f16(rng.normal(0, 0.02, (1, V, H))), "pos_emb": f16(rng.normal(0, 0.02, (1, S, H))),
         "type_emb": f16(rng.normal(0, 0.02, (1, 2, H)))}
    for i in range(L):
        w[f"wqkv_{i}"] = f16(rng.normal(0, 0.02, (1, H, 3 * H)))
        w[f"wo_{i}"] = f16(rng.normal(0, 0.02, (1, H, H)))
        w[f"w1_{i}"] = f16(rng.normal(0, 0.02, (1, H, F)))
        w[f"w2_{i}"] = f16(rng.normal(0, 0.02, (1, F, H)))
    return w


def _worker(rank, world, port, out_path):
    sys.path.insert(0, str(REPO))
    sys.path.insert(0, str(REPO / "tests"))
    import torch
    import torch.distributed as dist
    from __graft_entry__ import load_package
    load_package()
    from hands_on_mlir_b200.bert_program import shard_batch
    from oracle import hom_oracle
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    hom_oracle.set_threads(2)
    rng = np.random.Generator(np.random.PCG64(3))
    w = _tiny_weights(rng, 1, 128, 256, 64, 128)
    B = 4
    lens = np.array([128, 64, 100, 1])
    ids = rng.integers(0, 64, (B, 128)).astype(np.int64)
    mask = (np.arange(128)[None, :] < lens[:, None]).astype(np.int64)
    types = np.zeros((B, 128), dtype=np.int64)
    lo, hi = shard_batch(B, world, rank)
    local = hom_oracle.bert_encoder(w, ids[lo:hi], mask[lo:hi], types[lo:hi], heads=2)
    t = torch.from_numpy(local.view(np.int16).astype(np.int32))
    bufs = [torch.empty_like(t) for _ in range(world)]
    dist.all_gather(bufs, t)
    if rank == 0:
        full = hom_oracle.bert_encoder(w, ids, mask, types, heads=2)
        got = torch.cat(bufs, 0).numpy().astype(np.int16).view(np.float16)
        np.save(out_path, np.array([np.array_equal(got.view(np.uint16), full.view(np.uint16))]))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_shard_and_gather(tmp_path):
    import torch.multiprocessing as mp
    out = tmp_path / "ok.npy"
    port = 29500 + (os.getpid() % 500)
    mp.spawn(_worker, args=(2, port, str(out)), nprocs=2, join=True)
    assert np.load(out)[0]


def test_bench_refuses_mismatched_world_size(monkeypatch):
    """bench.py must be launched with one process per GPU."""
    import bench
    monkeypatch.setenv("WORLD_SIZE", "1")
    class A:  # noqa: D401 - minimal argparse stand-in
        gpus, steps, warmup, workload, no_cpu_baseline = 2, 1, 0, "bert-base", True
    with pytest.raises(SystemExit):
        bench.run_gpu_arm(A, None, bench.WORKLOADS["bert-base"])

#!/usr/bin/env python
"""Benchmark of the BERT runtime-kernel path: fp16 encoder sequences/s on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload bert-base|bert-large]
                    [--impl reference] [--op NAME [--l2-resident]]

A step is one encoder forward over one batch of synthetic input (random-init weights
N(0, 0.02), LayerNorm without affine, no biases; ids uniform in [1000, 30522)):
  bert-base   12 layers, hidden 768, 32 sequences x 128 tokens PER GPU (weak scaling);
  bert-large  24 layers, hidden 1024, 256 sequences x 512 tokens split evenly over the GPUs,
              valid lengths uniform in [256, 512] (strong scaling).
One process per GPU (launch N > 1 with torch.distributed.run); batches are independent, so
there is no collective on the data path - only the final gather of the hidden states, which
is timed separately.

Rank 0 prints one JSON line:
  value      sequences/s of the whole job with inputs resident in HBM (CUDA-graph replay of
             the forward, CUDA events on the launching stream, max over ranks);
  e2e        the same metric through the host-buffer entry point: every step copies the
             int64 ids / mask / token types from pinned host memory to the device and the
             fp16 hidden states back, and waits for them;
  roofline   the GEMM family (the dominant kernel): algorithmic FLOPs of every GEMM launch
             of a step / their summed CUDA-event durations, against the measured dense
             bf16/fp16 tensor peak;
  cpu_baseline  the CPU oracle's encoder on a bounded sample, host threads stated.

`--impl reference` times the CPU restatement of the same path on the host cores only (the
reference has no CPU implementation of LayerNorm / GELU / attention to run instead; its one
CPU kernel, matmulAddF32, is timed beside it when oracle/_ref was built).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time
from pathlib import Path

import numpy as np

REPO = Path(__file__).resolve().parent
sys.path.insert(0, str(REPO))

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}

WORKLOADS = {
    "bert-base": dict(model="base", batch=32, seq=128, scaling="weak", lens=None),
    "bert-large": dict(model="large", batch=256, seq=512, scaling="strong", lens=(256, 512)),
}


# DRAM bytes (read + written) per launch from the ncu captures summarised under profiles/
# (dram__bytes_read.sum + dram__bytes_write.sum); keyed by the --op case, "bert-base" is the mean
# over the 48 GEMM launches of one step with caches as the preceding kernels leave them.
NCU_TRAFFIC_BYTES = {
    "bert-base": {"bytes": 8.32e6, "source": "profiles/launch_list_bert_base_b32_s128.txt"},
    "gemm-ffn1": {"bytes": 11.05e6, "source": "profiles/gemm_pair_256x256_bert_base_ffn1.txt"},
    "gemm-qkv": {"bytes": 9.86e6, "source": "profiles/gemm_pair_256x256_bert_base_qkv.txt"},
    "gemm-ffn2": {"bytes": 36.22e6, "source": "profiles/gemm_1cta_128x192_bert_base_ffn2.txt"},
    "gemm-large-ffn1": {"bytes": 122.0e6, "source": "profiles/gemm_pair_256x256_bert_large_ffn1_m16384.txt"},
    "ln-c2": {"bytes": 12.60e6, "source": "profiles/layernorm_residual_affine_4096x768.txt"},
    "ln-large": {"bytes": 480.6e6, "source": "profiles/layernorm_inplace_131072x1024.txt"},
    "attn-c3": {"bytes": 18.90e6, "source": "profiles/attention_single_tile_bs32_seq128_h12.txt"},
    "attn-large": {"bytes": 101.6e6, "source": "profiles/attention_two_query_tiles_bs32_seq512_h16.txt"},
}


def ncu_traffic(key):
    t = NCU_TRAFFIC_BYTES.get(key)
    return (t["bytes"], t["source"]) if t else (None, None)


def load_peaks():
    p = REPO / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            d = json.loads(p.read_text())
            return {k: float(d[k]) for k in FALLBACK_PEAKS}, "measured"
        except Exception:
            pass
    return dict(FALLBACK_PEAKS), "fallback"


# ------------------------------------------------------------------ synthetic data

def make_inputs(workload: dict, n_seq: int, first_seq: int, seed: int = 0):
    """ids / mask / token types (int64 [n_seq, seq]) for sequences [first_seq, first_seq+n_seq)
    of the workload's global batch; each sequence's data depends only on its global index."""
    seq = workload["seq"]
    ids = np.zeros((n_seq, seq), dtype=np.int64)
    mask = np.zeros((n_seq, seq), dtype=np.int64)
    for i in range(n_seq):
        rng = np.random.Generator(np.random.PCG64([seed, first_seq + i]))
        length = seq if workload["lens"] is None else int(
            rng.integers(workload["lens"][0], workload["lens"][1] + 1))
        ids[i, :length] = rng.integers(1000, 30522, length)
        mask[i, :length] = 1
    types = np.zeros((n_seq, seq), dtype=np.int64)
    return ids, mask, types


def make_weights_numpy(cfg, seq: int, seed: int = 0, layers: int | None = None):
    """Random-init encoder weights, N(0, 0.02), fp16, as numpy (for the CPU arms)."""
    rng = np.random.Generator(np.random.PCG64(seed))
    out = {}
    n_layers = cfg.layers if layers is None else layers
    for name in cfg.weight_names():
        if name.split("_")[-1].isdigit() and int(name.split("_")[-1]) >= n_layers:
            continue
        shape = cfg.weight_shape(name, seq)
        out[name] = (rng.standard_normal(shape, dtype=np.float32) * 0.02).astype(np.float16)
    return out


def make_weights_torch(cfg, seq: int, device, seed: int = 0):
    import torch
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    out = {}
    for name in cfg.weight_names():
        shape = cfg.weight_shape(name, seq)
        out[name] = (torch.randn(shape, generator=g, device=device, dtype=torch.float32) * 0.02).half()
    return out


# ------------------------------------------------------------------- clock sampling

class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU while the timed region runs
    (read-only NVML queries)."""

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown",
               0x4: "sw_power_cap"}

    def __init__(self, index: int, period_s: float = 0.02):
        self.index, self.period = index, period_s
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nvml = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self._nvml = None

    def _run(self):
        n = self._nvml
        while not self._stop.is_set():
            try:
                self.samples.append(float(n.nvmlDeviceGetClockInfo(self._h, n.NVML_CLOCK_SM)))
                bits = int(n.nvmlDeviceGetCurrentClocksThrottleReasons(self._h))
                for bit, name in self.REASONS.items():
                    if bits & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(self.period)

    def __enter__(self):
        if self._nvml is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread:
            self._thread.join(timeout=2.0)  # a stuck NVML query must not hold up the benchmark

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


# ------------------------------------------------------------------------ CPU arms

class CpuEncoder:
    """The CPU oracle's encoder on a bounded sample of the workload: `n_seq` sequences through
    the first `layers` layers; rates are reported in full-model sequence equivalents."""

    def __init__(self, cfg, workload):
        from oracle import hom_oracle
        self.oracle, self.cfg, self.workload = hom_oracle, cfg, workload
        self.threads = hom_oracle.set_threads(0)
        self.weights = make_weights_numpy(cfg, workload["seq"])

    def run(self, n_seq: int, layers: int) -> float:
        ids, mask, types = make_inputs(self.workload, n_seq, 0)
        t0 = time.perf_counter()
        self.oracle.bert_encoder(self.weights, ids, mask, types, heads=self.cfg.heads,
                                 eps=self.cfg.eps, layers=layers)
        return time.perf_counter() - t0

    def plan(self, step_budget_s: float):
        """(n_seq, layers) whose run takes about `step_budget_s`."""
        per_layer_seq = min(self.run(1, 1), self.run(1, 1))
        full_seq = per_layer_seq * self.cfg.layers
        if step_budget_s >= full_seq:
            return int(min(self.workload["batch"], step_budget_s // full_seq)), self.cfg.layers
        return 1, int(max(1, step_budget_s // per_layer_seq))

    def describe(self, n_seq, layers):
        return (f"{n_seq} of {self.workload['batch']} sequences x {self.workload['seq']} tokens, "
                f"{layers} of {self.cfg.layers} layers per step (rate scaled to the full depth)")


def run_reference_arm(args, cfg, workload):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    enc = CpuEncoder(cfg, workload)
    n_seq, layers = enc.plan(120.0 / max(1, args.steps + min(args.warmup, 2)))
    for _ in range(min(args.warmup, 2)):
        enc.run(n_seq, layers)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        enc.run(n_seq, layers)
    dt = time.perf_counter() - t0
    value = args.steps * n_seq * (layers / cfg.layers) / dt
    line = {
        "impl": "reference", "metric": "bert_fp16_sequences_per_s", "value": value,
        "unit": "sequences/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * dt / args.steps, "higher_is_better": True,
        "scaling": workload["scaling"], "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": f"{args.workload} encoder, CPU restatement of the runner-utils "
                               "call sequence on the host cores"},
        "cpu_baseline": {"value": value, "unit": "sequences/s", "cores": enc.threads,
                         "kind": "port", "sample": enc.describe(n_seq, layers)},
        "e2e": {"value": value, "unit": "sequences/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
    }
    extra = reference_matmul_rate()
    if extra:
        line["cpu_baseline"]["reference_matmulAddF32"] = extra
    try:
        line["cpu_baseline"]["torch_cpu_fp32"] = torch_cpu_baseline(cfg, workload, budget_s=8.0)
    except Exception as exc:
        line["cpu_baseline"]["torch_cpu_fp32"] = {"unavailable": repr(exc)}
    print(json.dumps(line), flush=True)


def reference_matmul_rate():
    """GFLOP/s of the reference's own CPU GEMM (matmulAddF32 compiled into oracle/_ref) on a
    128 x 768 x 768 slice, 1 thread; None when oracle/_ref was not built."""
    try:
        from oracle import hom_oracle
        if not hom_oracle.ref_available():
            return None
        rng = np.random.default_rng(0)
        A = rng.standard_normal((1, 128, 768), dtype=np.float32)
        B = rng.standard_normal((1, 768, 768), dtype=np.float32)
        C = np.zeros((1, 1, 768), dtype=np.float32)
        t0 = time.perf_counter()
        hom_oracle.ref_matmul_add_f32(A, B, C)
        dt = time.perf_counter() - t0
        return {"gflops": 2 * 128 * 768 * 768 / dt / 1e9, "cores": 1, "shape": "128x768x768"}
    except Exception:
        return None



# ------------------------------------------------------------------ op-level arm

OP_CASES = {
    # name: (kind, parameters)
    "gemm-c1": ("gemm", dict(m=512, n=3072, k=768, act=1, c="bias")),      # GEMM+bias+GELU config
    "gemm-qkv": ("gemm", dict(m=4096, n=2304, k=768, act=0, c=None)),
    "gemm-out": ("gemm", dict(m=4096, n=768, k=768, act=0, c="residual")),
    "gemm-ffn1": ("gemm", dict(m=4096, n=3072, k=768, act=1, c=None)),
    "gemm-ffn2": ("gemm", dict(m=4096, n=768, k=3072, act=0, c="residual")),
    "gemm-large-ffn1": ("gemm", dict(m=16384, n=4096, k=1024, act=1, c=None)),
    "gemm-large-ffn2": ("gemm", dict(m=16384, n=1024, k=4096, act=0, c="residual")),
    "ln-c2": ("ln", dict(rows=4096, hidden=768, residual=True, affine=True)),  # residual+LN config
    "ln-inplace": ("ln", dict(rows=4096, hidden=768, residual=False, affine=False)),
    "ln-large": ("ln", dict(rows=131072, hidden=1024, residual=False, affine=False)),
    "attn-c3": ("attn", dict(bs=32, seq=128, heads=12, lens=(64, 128))),    # attention config
    "attn-large": ("attn", dict(bs=32, seq=512, heads=16, lens=(256, 512))),
}


def run_op_arm(args):
    """One kernel of the path on its own: rotating buffer sets larger than L2, CUDA events on
    the launching stream around `steps` launches, per-launch average."""
    import torch
    from __graft_entry__ import load_package

    pkg = load_package()
    hom = pkg.runner()
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    hom.use_torch_stream()
    kind, prm = OP_CASES[args.op]
    g = torch.Generator(device=dev)
    g.manual_seed(0)
    randn = lambda *shape, std=1.0: (torch.randn(shape, generator=g, device=dev) * std).half()
    peaks, peak_src = load_peaks()
    sets, launch = [], None
    if kind == "gemm":
        if args.shape:
            prm = dict(prm)
            prm["m"], prm["n"], prm["k"] = (int(v) for v in args.shape.split(","))
        m, n, k = prm["m"], prm["n"], prm["k"]
        per_set = 2 * (m * k + k * n + m * n)
        nsets = max(2, min(16, -(-300_000_000 // per_set))) if not args.l2_resident else 1
        for _ in range(nsets):
            A = (torch.rand((1, m, k), generator=g, device=dev) * 2 - 1).half()
            B = randn(1, k, n, std=0.02)
            D = randn(1, m, n) if prm["c"] == "residual" else torch.empty((1, m, n), dtype=torch.float16, device=dev)
            C = (torch.rand((1, 1, n), generator=g, device=dev) * 2 - 1).half() if prm["c"] == "bias" else D
            hom.declare_weights(B)  # weights, as in the model: never written by a kernel
            sets.append((A, B, C, D))
        beta = 1.0 if prm["c"] else 0.0
        launch = lambda s: hom.cutlassGemmF16(s[0], s[1], s[2], s[3], activation=prm["act"], beta=beta,
                                              gemmNum=args.tile, splitKFactor=args.split)
        flops = 2.0 * m * n * k
        nbytes = per_set + (2 * m * n if prm["c"] == "residual" else 2 * n if prm["c"] else 0)
        bound, work, unit, peak = "tensor", flops, "TFLOP/s", peaks["bf16_tflops"]
        peak_note = f"{peak_src} (burst dense bf16/fp16; kernel timed alone)"
        desc = f"GEMM {m}x{n}x{k} act={prm['act']} C={prm['c']} tile={hom.gemm_query_tile(m, n, k, prm['act'])}"
    elif kind == "ln":
        rows, hidden = prm["rows"], prm["hidden"]
        per_set = 2 * rows * hidden * (3 if prm["residual"] else 2)
        nsets = max(2, min(32, -(-300_000_000 // per_set))) if not args.l2_resident else 1
        gamma = (1 + torch.randn(hidden, generator=g, device=dev) * 0.1).half()
        beta_t = (torch.randn(hidden, generator=g, device=dev) * 0.1).half()
        for _ in range(nsets):
            X = randn(rows, hidden)
            R = randn(rows, hidden) if prm["residual"] else None
            O = torch.empty_like(X) if prm["residual"] else X
            sets.append((X, R, O))
        if prm["residual"]:
            launch = lambda s: hom.homResidualLayernormF16(s[0], s[1], gamma, beta_t, s[2], 1e-12)
        else:
            launch = lambda s: hom.nvteLayernormF16(s[0], 1e-12)
        nbytes = per_set + (4 * hidden if prm["affine"] else 0)
        bound, work, unit, peak = "hbm", float(nbytes), "GB/s", peaks["hbm_gbs"]
        peak_note = f"{peak_src} (HBM copy)"
        desc = f"LayerNorm rows={rows} hidden={hidden} residual={prm['residual']} affine={prm['affine']}"
    else:
        bs, seq, heads = prm["bs"], prm["seq"], prm["heads"]
        rng = np.random.Generator(np.random.PCG64(0))
        lens = rng.integers(prm["lens"][0], prm["lens"][1] + 1, bs)
        cu = torch.from_numpy(np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)).to(dev)
        per_set = 2 * bs * seq * heads * 64 * 4
        nsets = max(2, min(16, -(-300_000_000 // per_set))) if not args.l2_resident else 1
        for _ in range(nsets):
            sets.append((randn(bs, seq, 3 * heads * 64), torch.empty((bs, seq, heads * 64), dtype=torch.float16, device=dev)))
        launch = lambda s: hom.nvteBertAttentionF16(s[0], cu, s[1], 0.125, heads)
        nbytes = per_set + 4 * (bs + 1)
        flops = 4.0 * 64 * heads * float((lens.astype(np.float64) ** 2).sum())
        bound, work, unit, peak = "hbm", float(nbytes), "GB/s", peaks["hbm_gbs"]
        peak_note = f"{peak_src} (HBM copy)"
        desc = f"attention bs={bs} seq={seq} heads={heads} valid lengths U{prm['lens']}"

    for i in range(max(args.warmup, 3)):
        launch(sets[i % len(sets)])
    hom.synchronize()
    # One pass over the buffer sets is captured into a CUDA graph so that short kernels are
    # not limited by the Python call overhead; `steps` launches = steps / len(sets) replays.
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        for st in sets:
            launch(st)
    replays = max(1, args.steps // len(sets))
    args.steps = replays * len(sets)
    graph.replay()
    torch.cuda.synchronize()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(0) as clocks:
        ev0.record(stream)
        for _ in range(replays):
            graph.replay()
        ev1.record(stream)
        torch.cuda.synchronize()
    hom.synchronize()
    ms = ev0.elapsed_time(ev1) / args.steps
    achieved = work / (ms / 1e3) / (1e12 if bound == "tensor" else 1e9)
    line = {
        "metric": f"{args.op}_{'tflops' if bound == 'tensor' else 'gbs'}", "value": achieved,
        "unit": unit, "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f16", "data": "synthetic",
        "config": {"workload": desc,
                   "l2": ("single buffer set, L2 resident" if args.l2_resident else
                          f"{len(sets)} rotating buffer sets, {len(sets) * per_set / 1e6:.0f} MB > 126 MB L2")},
        "gpu_launches": args.steps,
        "roofline": {"bound": bound, "achieved": achieved, "peak": peak, "unit": unit,
                     "frac": achieved / peak, "peak_source": peak_note,
                     "traffic": ncu_traffic(args.op)[0], "traffic_source": ncu_traffic(args.op)[1],
                     "algorithmic_bytes": nbytes,
                     "algorithmic_flops": flops if kind != "ln" else 0.0},
        "clocks": clocks.summary(),
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------- GPU arm

MIN_TIMED_SECONDS = 1.0  # every throughput figure is averaged over at least this much GPU time


class Ranks:
    """The process group of the run (or a stand-in for one process)."""

    def __init__(self, device):
        import torch
        import torch.distributed as dist
        self.torch, self.dist, self.device = torch, dist, device
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))

    def barrier(self):
        self.torch.cuda.synchronize()
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max(self, x: float) -> float:
        if self.world == 1:
            return x
        t = self.torch.tensor([x], dtype=self.torch.float64, device=self.device)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())


def timed_region(ranks, stream, step, steps: int, min_seconds: float | None = None):
    """Times `steps` calls of `step()` per round, as many rounds back to back as it takes to fill
    `min_seconds` (the same number on every rank), between two CUDA events on the launching
    stream with a barrier + synchronize on both sides.  Returns (ms per step = max over ranks of
    the whole region / steps run, steps run, seconds)."""
    import torch
    if min_seconds is None:
        min_seconds = MIN_TIMED_SECONDS
    min_seconds = min(min_seconds, MIN_TIMED_SECONDS)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ranks.barrier()
    ev0.record(stream)
    for _ in range(steps):
        step()
    ev1.record(stream)
    ranks.barrier()
    probe_ms = ranks.max(ev0.elapsed_time(ev1))
    rounds = max(1, int(np.ceil(min_seconds * 1e3 / max(probe_ms, 1e-3))))
    ranks.barrier()
    ev0.record(stream)
    for _ in range(rounds * steps):
        step()
    ev1.record(stream)
    ranks.barrier()
    total_ms = ranks.max(ev0.elapsed_time(ev1))
    return total_ms / (rounds * steps), rounds * steps, total_ms / 1e3


def gemm_chain(hom, cfg, weights, batch, seq, device, stream):
    """The GEMM launches of one forward, in order and on the model's own weights, with nothing
    in between: what the dominant kernel family costs when only it runs (neighbouring launches
    overlap through programmatic dependent launch exactly as in the full step).  Returns a
    callable that replays the captured chain once, the launch count and the FLOPs."""
    import torch
    g = torch.Generator(device=device)
    g.manual_seed(1)
    h = cfg.hidden
    mk = lambda *shape: (torch.randn(shape, generator=g, device=device)).half()
    x, res, ctx = mk(batch, seq, h), mk(batch, seq, h), mk(batch, seq, h)
    qkv = torch.empty((batch, seq, 3 * h), dtype=torch.float16, device=device)
    mid = torch.empty((batch, seq, cfg.ffn), dtype=torch.float16, device=device)

    def issue():
        for i in range(cfg.layers):
            hom.cutlassGemmF16(x, weights[f"wqkv_{i}"], None, qkv)
            hom.cutlassGemmF16(ctx, weights[f"wo_{i}"], res, x, beta=1.0)
            hom.cutlassGemmF16(x, weights[f"w1_{i}"], None, mid, activation=1)
            hom.cutlassGemmF16(mid, weights[f"w2_{i}"], res, x, beta=1.0)

    issue()
    hom.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        issue()
    keep = (x, res, ctx, qkv, mid)
    return (lambda: (graph.replay(), keep)[0]), 4 * cfg.layers, cfg.gemm_flops_per_sequence(seq) * batch


def per_kernel_breakdown(hom, prog_factory, inputs, n_prof=5):
    """Per-launch CUDA-event durations of one step: a second replay program is captured with the
    library's per-launch events switched on, so every launch of its graph is bracketed by
    event-record nodes on the launching stream.  The event nodes stand between the kernels, so
    launches are serialised here (no overlap of a kernel's ramp with its predecessor's tail):
    the SHARES are meaningful, the sum exceeds the step time measured without them."""
    prog_t = prog_factory()
    ids_d, mask_d, types_d = inputs
    prog_t.forward(ids_d, mask_d, types_d, use_graph=True)  # first call runs eagerly (set-up)
    hom.synchronize()
    hom.op_timing(True)
    prog_t.forward(ids_d, mask_d, types_d, use_graph=True)  # capture + first launch
    hom.op_timing(False)
    hom.synchronize()
    records = []
    for _ in range(n_prof):
        prog_t.forward(ids_d, mask_d, types_d, use_graph=True)
        hom.synchronize()
        records += hom.peek_op_timings()
    prog_t.close()
    hom.collect_op_timings()  # releases the events
    kinds = {1: "gemm", 2: "layernorm", 3: "attention", 4: "elementwise", 5: "gather", 6: "cu_seqlen"}
    per_kind, gemm_shapes = {}, {}
    for kind, ms, flops, nbytes in records:
        d = per_kind.setdefault(kinds.get(kind, str(kind)), {"launches": 0, "ms": 0.0, "flops": 0.0, "bytes": 0.0})
        d["launches"] += 1
        d["ms"] += ms
        d["flops"] += flops
        d["bytes"] += nbytes
        if kind == 1:
            d = gemm_shapes.setdefault(f"{flops / 1e9:.2f}_gflop", {"launches": 0, "ms": 0.0, "flops": flops})
            d["launches"] += 1
            d["ms"] += ms
    total_ms = sum(v["ms"] for v in per_kind.values()) or 1.0
    kernels = {k: {"launches_per_step": v["launches"] // n_prof, "serialised_ms_per_step": v["ms"] / n_prof,
                   "share": v["ms"] / total_ms,
                   "tflops": (v["flops"] / (v["ms"] / 1e3) / 1e12) if v["ms"] > 0 and v["flops"] else None,
                   "gbs": (v["bytes"] / (v["ms"] / 1e3) / 1e9) if v["ms"] > 0 else None}
               for k, v in per_kind.items()}
    by_shape = {k: {"launches_per_step": v["launches"] // n_prof, "serialised_avg_us": 1e3 * v["ms"] / v["launches"],
                    "tflops": v["flops"] * v["launches"] / (v["ms"] / 1e3) / 1e12}
                for k, v in gemm_shapes.items()}
    gemm_bytes = per_kind.get("gemm", {}).get("bytes", 0.0) / max(1, per_kind.get("gemm", {}).get("launches", 1))
    return kernels, by_shape, gemm_bytes


def measure_workload(args, ranks, hom, stream, cfg, workload, name, *, full: bool):
    """Everything that is measured for one workload on this rank's GPU; `full` adds the
    end-to-end, eager, per-kernel, GEMM-chain and gather measurements to the device-resident
    throughput."""
    import torch
    from hands_on_mlir_b200.bert_program import BertProgram, shard_batch
    world, rank, device = ranks.world, ranks.rank, ranks.device
    if workload["scaling"] == "weak":
        local_batch, first = workload["batch"], rank * workload["batch"]
        global_batch = workload["batch"] * world
    else:
        lo, hi = shard_batch(workload["batch"], world, rank)
        local_batch, first, global_batch = hi - lo, lo, workload["batch"]
    seq = workload["seq"]
    factory = lambda: _program(BertProgram, cfg, local_batch, seq, args, weights)
    weights = make_weights_torch(cfg, seq, device)
    prog = factory()
    ids_np, mask_np, types_np = make_inputs(workload, local_batch, first)
    ids_h, mask_h, types_h = (torch.from_numpy(x).pin_memory() for x in (ids_np, mask_np, types_np))
    ids_d, mask_d, types_d = (x.to(device) for x in (ids_h, mask_h, types_h))
    steps = args.steps
    out = {"local_batch": local_batch, "global_batch": global_batch, "seq": seq}

    # ---- device-resident throughput (value): CUDA-graph replay, inputs already in HBM
    for _ in range(max(args.warmup, 3)):
        prog.forward(ids_d, mask_d, types_d, use_graph=True)
    hom.synchronize()
    with ClockSampler(torch.cuda.current_device()) as clocks:
        ms, n_run, secs = timed_region(ranks, stream, lambda: prog.forward(ids_d, mask_d, types_d, use_graph=True), steps)
    hom.synchronize()
    out.update(ms_per_step=ms, value=global_batch / (ms / 1e3), timed_steps_total=n_run, timed_region_s=secs,
               clocks=clocks.summary(), launches_per_forward=prog.launches_per_forward())
    mhz = out["clocks"]["sm_mhz"]
    out["ms_x_ghz"] = ms * mhz / 1e3 if mhz else None  # step time in millions of SM cycles: clock-independent
    if not full:
        kernels, _, _ = per_kernel_breakdown(hom, factory, (ids_d, mask_d, types_d), n_prof=2)
        out["kernels"] = kernels
        prog.close()
        return out

    # ---- the same call sequence issued eagerly (one host call per kernel, no graph): what a
    # model library compiled by the reference does (examples/torch/bert/bert.cu:107-127)
    for _ in range(3):
        prog.forward(ids_d, mask_d, types_d, use_graph=False)
    hom.synchronize()
    ms_e, n_e, _ = timed_region(ranks, stream, lambda: prog.forward(ids_d, mask_d, types_d, use_graph=False),
                                steps, min_seconds=0.5)
    t0 = time.perf_counter()
    for _ in range(20):
        prog.forward(ids_d, mask_d, types_d, use_graph=False)
    host_us = (time.perf_counter() - t0) / (20 * prog.launches_per_forward()) * 1e6
    hom.synchronize()
    out["eager"] = {"value": global_batch / (ms_e / 1e3), "unit": "sequences/s", "ms_per_step": ms_e,
                    "steps_timed": n_e, "host_us_per_call": host_us,
                    "note": "no CUDA graph: every runner-utils call is made from the host each step"}

    # ---- end to end with host buffers (e2e): every step copies its inputs from pinned host
    # memory and delivers its hidden states to pinned host memory; the delivery of step i
    # overlaps the compute of step i+1 (two result slots), and the clock stops only after the
    # last step's result is on the host.
    outs = tuple(torch.empty((local_batch, seq, cfg.hidden), dtype=torch.float16).pin_memory() for _ in range(2))
    for i in range(4):
        prog.forward_host_async(ids_h, mask_h, types_h, outs[i & 1], use_graph=True)
    prog.wait_host()
    e2e_steps = max(steps, int(np.ceil(MIN_TIMED_SECONDS * 1e3 / ms)))
    ranks.barrier()
    t0 = time.perf_counter()
    for i in range(e2e_steps):
        prog.forward_host_async(ids_h, mask_h, types_h, outs[i & 1], use_graph=True)
    prog.wait_host()
    torch.cuda.synchronize()
    e2e_s = ranks.max(time.perf_counter() - t0)
    ranks.barrier()
    h2d, d2h = prog.host_traffic()
    out["e2e"] = {"value": global_batch * e2e_steps / e2e_s, "unit": "sequences/s", "h2d_bytes_per_step": h2d,
                  "d2h_bytes_per_step": d2h, "ms_per_step": 1e3 * e2e_s / e2e_steps, "steps_timed": e2e_steps}

    # ---- the two LayerNorm-fusion extensions of the replay program, same inputs, same timing:
    # reported beside the headline (which stays the reference's call sequence), never as it
    if args.fused_layernorm == 0 and not args.no_extensions:
        ext = {}
        try:
            for mode, label in ((1, "gemm_residual_layernorm_fused"), (2, "deferred_layernorm")):
                prog_x = BertProgram(cfg, local_batch, seq, fused_embedding=args.fused_embedding, fused_layernorm=mode)
                prog_x.set_weights(weights)
                for _ in range(3):
                    prog_x.forward(ids_d, mask_d, types_d, use_graph=True)
                hom.synchronize()
                ms_x, n_x, _ = timed_region(ranks, stream,
                                            lambda: prog_x.forward(ids_d, mask_d, types_d, use_graph=True),
                                            steps, min_seconds=0.5)
                hom.synchronize()
                ext[label] = {"value": global_batch / (ms_x / 1e3), "unit": "sequences/s", "ms_per_step": ms_x,
                              "steps_timed": n_x, "launches_per_forward": prog_x.launches_per_forward()}
                prog_x.close()
        except Exception as e:  # an option of the replay program must not take the headline down with it
            if ranks.world > 1:
                raise  # the other ranks are inside the timed region's barriers: fail the whole job instead
            ext["error"] = f"{type(e).__name__}: {e}"
            hom.clear_error()
        ext["note"] = ("replay-program options that change the call sequence: GEMM + residual + LayerNorm in one "
                       "cluster kernel (same rounding points as the sequence), and LayerNorm deferred into the "
                       "consumers' epilogues (no fp16 rounding of the LayerNorm output)")
        out["extensions"] = ext

    # ---- the GEMM family alone (roofline) and the per-kernel shares
    replay_chain, n_gemm, chain_flops = gemm_chain(hom, cfg, weights, local_batch, seq, device, stream)
    for _ in range(3):
        replay_chain()
    with ClockSampler(torch.cuda.current_device()) as chain_clocks:
        ms_chain, _, _ = timed_region(ranks, stream, replay_chain, max(10, steps // 4))
    kernels, by_shape, gemm_bytes = per_kernel_breakdown(hom, factory, (ids_d, mask_d, types_d))
    out.update(kernels=kernels, gemm_by_shape=by_shape)
    peaks, peak_src = load_peaks()
    achieved = chain_flops / (ms_chain / 1e3) / 1e12
    cc = chain_clocks.summary()
    capped = bool(cc["sm_mhz"] and cc["sm_max_mhz"] and cc["sm_mhz"] < 0.95 * cc["sm_max_mhz"])
    peak = peaks["bf16_tflops_sustained"] if capped else peaks["bf16_tflops"]
    out["roofline"] = {
        "bound": "tensor", "kernel": "gemm_f16_pair_kernel / gemm_f16_kernel (all GEMM launches of a step)",
        "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
        "peak_source": f"{peak_src}: " + ("sustained dense bf16/fp16 (SM clock below 95 % of max while timed)"
                                         if capped else "burst dense bf16/fp16 (SM clock at max while timed)"),
        "frac_of_burst": achieved / peaks["bf16_tflops"],
        "frac_of_sustained": achieved / peaks["bf16_tflops_sustained"],
        "how": f"the step's {n_gemm} GEMM launches replayed as one CUDA graph with nothing in between, "
               f">= {MIN_TIMED_SECONDS:.0f} s between two CUDA events on the launching stream; "
               "achieved = algorithmic FLOPs / that time",
        "gemm_ms_per_step": ms_chain, "launches_per_step": n_gemm, "avg_launch_us": 1e3 * ms_chain / n_gemm,
        "clocks": cc, "traffic": ncu_traffic(name)[0], "traffic_source": ncu_traffic(name)[1],
        "algorithmic_bytes_per_launch": gemm_bytes,
    }

    # ---- final gather of the hidden states (the only collective): warm, on a side stream, the
    # gather of step i overlapping the compute of step i+1
    if world > 1:
        dist = ranks.dist
        side = torch.cuda.Stream()
        res0 = prog.result_to_torch(prog.forward(ids_d, mask_d, types_d, use_graph=True))
        slots = [torch.empty_like(res0) for _ in range(2)]
        gathered = [torch.empty((world,) + tuple(res0.shape), dtype=res0.dtype, device=device) for _ in range(2)]
        done = [torch.cuda.Event() for _ in range(2)]

        def step_with_gather(i):
            mem = prog.forward(ids_d, mask_d, types_d, use_graph=True)
            slot = slots[i & 1]
            if i >= 2:
                stream.wait_event(done[i & 1])  # the gather that last read this slot has finished
            # the program's result buffer is overwritten by the next forward: park the result
            slot.copy_(_device_view(torch, mem, res0), non_blocking=True)
            ready = torch.cuda.Event()
            ready.record(stream)
            with torch.cuda.stream(side):
                side.wait_event(ready)
                dist.all_gather_into_tensor(gathered[i & 1], slot)
                done[i & 1].record(side)

        for i in range(4):
            step_with_gather(i)
        torch.cuda.synchronize()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(side):
            g0.record(side)
            dist.all_gather_into_tensor(gathered[0], slots[0])
            g1.record(side)
        torch.cuda.synchronize()
        out["output_gather_ms"] = ranks.max(g0.elapsed_time(g1))
        n_g = max(steps, int(np.ceil(MIN_TIMED_SECONDS * 1e3 / ms)))
        ranks.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for i in range(n_g):
            step_with_gather(i)
        stream.wait_stream(side)
        e1.record(stream)
        ranks.barrier()
        ms_g = ranks.max(e0.elapsed_time(e1)) / n_g
        out["value_with_gather"] = global_batch / (ms_g / 1e3)
        out["with_gather"] = {"ms_per_step": ms_g, "steps_timed": n_g,
                              "bytes_gathered_per_rank_per_step": int(res0.numel() * 2 * world),
                              "how": "NCCL all-gather of every step's hidden states on a side stream, "
                                     "overlapping the next step's compute; the clock stops after the last gather"}
    prog.close()
    return out


def _device_view(torch, memref, like):
    """A torch view (no copy) of the program-owned fp16 result buffer."""
    return torch.as_tensor(_CudaArray(memref.data_ptr, tuple(like.shape)), device=like.device)


class _CudaArray:
    """Minimal __cuda_array_interface__ wrapper around a device pointer holding fp16 values."""

    def __init__(self, ptr: int, shape):
        self.__cuda_array_interface__ = {"shape": shape, "typestr": "<f2", "data": (int(ptr), False),
                                         "version": 3, "strides": None}


def _program(BertProgram, cfg, batch, seq, args, weights):
    prog = BertProgram(cfg, batch, seq, fused_embedding=args.fused_embedding,
                       fused_layernorm=args.fused_layernorm)
    prog.set_weights(weights)
    return prog


def torch_cpu_baseline(cfg, workload, budget_s: float = 10.0):
    """PyTorch CPU fp32 encoder (all host cores) on a bounded sample: the same math as the
    oracle without the fp16 rounding points, as an optimised-CPU-library figure beside the
    scalar port."""
    import torch
    seq, h, heads = workload["seq"], cfg.hidden, cfg.heads
    g = torch.Generator().manual_seed(0)
    w = {n: torch.randn(cfg.weight_shape(n, seq), generator=g) * 0.02 for n in cfg.weight_names()}

    def run(n_seq):
        ids, mask, types = (torch.from_numpy(x) for x in make_inputs(workload, n_seq, 0))
        ln = lambda z: torch.nn.functional.layer_norm(z, (h,), eps=cfg.eps)
        t0 = time.perf_counter()
        with torch.no_grad():
            x = ln(w["word_emb"][0][ids] + w["type_emb"][0][types] + w["pos_emb"][0][None, :seq])
            add_mask = (1.0 - mask.float())[:, None, None, :] * torch.finfo(torch.float32).min
            for i in range(cfg.layers):
                qkv = (x @ w[f"wqkv_{i}"][0]).view(n_seq, seq, 3, heads, h // heads)
                q, k, v = (qkv[:, :, j].permute(0, 2, 1, 3) for j in range(3))
                a = torch.softmax(q @ k.transpose(-1, -2) / (h // heads) ** 0.5 + add_mask, -1) @ v
                a = a.permute(0, 2, 1, 3).reshape(n_seq, seq, h)
                x = ln(a @ w[f"wo_{i}"][0] + x)
                x = ln(torch.nn.functional.gelu(x @ w[f"w1_{i}"][0]) @ w[f"w2_{i}"][0] + x)
        return time.perf_counter() - t0

    run(1)
    one = run(1)
    n_seq = int(max(1, min(workload["batch"], budget_s // max(one, 1e-3))))
    secs = run(n_seq)
    return {"value": n_seq / secs, "unit": "sequences/s", "cores": torch.get_num_threads(), "kind": "torch-cpu-fp32",
            "sample": f"{n_seq} of {workload['batch']} sequences x {seq} tokens, all {cfg.layers} layers, {secs:.1f} s"}


def run_gpu_arm(args, cfg, workload):
    import faulthandler
    import torch
    import torch.distributed as dist
    from __graft_entry__ import load_package

    # A GPU arm that makes no progress must not sit in a synchronize call for ever: after 20
    # minutes the Python stacks are dumped to stderr and the process exits non-zero.
    faulthandler.dump_traceback_later(1200, exit=True)

    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with "
                         "python -m torch.distributed.run --nproc-per-node N")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback path)")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        # NCCL may print a version banner on stdout while the communicator comes up; stdout is
        # reserved for the one JSON line, so it is pointed at stderr during initialisation.
        sys.stdout.flush()
        saved_stdout = os.dup(1)
        os.dup2(2, 1)
        try:
            dist.init_process_group("nccl", device_id=device)
            warm = torch.zeros(1, device=device)
            dist.all_reduce(warm)
            torch.cuda.synchronize()
        finally:
            sys.stdout.flush()
            os.dup2(saved_stdout, 1)
            os.close(saved_stdout)

    pkg = load_package()
    from hands_on_mlir_b200.bert_program import BertConfig
    hom = pkg.runner()
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    hom.use_torch_stream()
    ranks = Ranks(device)
    rank = ranks.rank

    m = measure_workload(args, ranks, hom, stream, cfg, workload, args.workload, full=True)

    # ---- the split configuration (BERT-large 256 x 512 divided over the GPUs) beside the headline
    config5 = None
    if args.workload == "bert-base" and not args.no_config5:
        wl5 = WORKLOADS["bert-large"]
        saved = args.steps
        args.steps = max(10, min(saved, 20))
        r5 = measure_workload(args, ranks, hom, stream, BertConfig.large(), wl5, "bert-large", full=False)
        args.steps = saved
        cfg5 = BertConfig.large()
        fl5 = cfg5.gemm_flops_per_sequence(wl5["seq"]) + cfg5.attention_flops_per_sequence(wl5["seq"])
        config5 = {"workload": f"bert-large encoder (24 layers, hidden 1024), global batch {r5['global_batch']} x seq "
                               f"{wl5['seq']} split evenly: {r5['local_batch']} sequences per GPU, valid lengths U[256, 512]",
                   "metric": "bert_fp16_sequences_per_s", "value": r5["value"], "unit": "sequences/s",
                   "n_gpus": world, "scaling": "strong", "ms_per_step": r5["ms_per_step"],
                   "steps_timed": r5["timed_steps_total"], "timed_region_s": r5["timed_region_s"],
                   "model_tflops": r5["value"] * fl5 / 1e12, "clocks": r5["clocks"],
                   "kernel_shares": {k: round(v["share"], 4) for k, v in r5["kernels"].items()}}

    # ---- CPU baselines on bounded samples (rank 0, N = 1 only)
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        enc = CpuEncoder(cfg, workload)
        n_seq, layers = enc.plan(12.0)
        secs = enc.run(n_seq, layers)
        cpu = {"value": n_seq * (layers / cfg.layers) / secs, "unit": "sequences/s",
               "cores": enc.threads, "kind": "port",
               "sample": enc.describe(n_seq, layers) + f", {secs:.1f} s"}
        try:
            cpu["torch_cpu_fp32"] = torch_cpu_baseline(cfg, workload)
        except Exception as exc:  # a baseline, never a reason to lose the GPU line
            cpu["torch_cpu_fp32"] = {"unavailable": repr(exc)}
        ref = reference_matmul_rate()
        if ref:
            cpu["reference_matmulAddF32"] = ref

    if rank == 0:
        seq = workload["seq"]
        flops_per_seq = cfg.gemm_flops_per_sequence(seq) + cfg.attention_flops_per_sequence(seq)
        line = {
            "metric": "bert_fp16_sequences_per_s", "value": m["value"], "unit": "sequences/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": m["ms_per_step"], "higher_is_better": True,
            "scaling": workload["scaling"], "vs_baseline": None, "dtype": "f16",
            "data": "synthetic",
            "config": {
                "workload": f"{args.workload} encoder ({cfg.layers} layers, hidden {cfg.hidden}, "
                            f"{cfg.heads} heads, FFN {cfg.ffn}), global batch {m['global_batch']} x seq "
                            f"{seq}, {m['local_batch']} sequences per GPU",
                "parallelism": f"batch-sharded replicas x{world}, no data-path collective",
                "l2": "no explicit flush: the per-step working set (all layer weights + "
                      "activations) exceeds the 126 MB L2",
                "launch": "CUDA-graph replay of the runner-utils call sequence"
                          + (" with the fused embedding extension" if args.fused_embedding else "")
                          + (" with the deferred-LayerNorm extension" if args.fused_layernorm == 2 else
                             " with the fused GEMM+LayerNorm extension" if args.fused_layernorm else ""),
                "timing": f"{args.steps}-step rounds repeated back to back for >= {MIN_TIMED_SECONDS:.0f} s "
                          "between one pair of CUDA events; ms_per_step is the mean over all of them",
            },
            "timed_steps_total": m["timed_steps_total"], "timed_region_s": m["timed_region_s"],
            "ms_per_step_x_sm_ghz": m["ms_x_ghz"],
            "model_tflops": m["value"] * flops_per_seq / 1e12,
            "e2e": m["e2e"],
            "eager": m["eager"],
            "gpu_launches": m["timed_steps_total"] * m["launches_per_forward"],
            "gpu_launches_per_step": m["launches_per_forward"],
            "roofline": m["roofline"],
            "kernels": m["kernels"],
            "kernels_note": ("per-launch CUDA events serialise the launches; the floor of this measurement is "
                             f"{1e3 * m['kernels'].get('cu_seqlen', {}).get('serialised_ms_per_step', 0.0):.1f} us, what the "
                             "one-block cu_seqlen kernel takes in it: compare shares, not absolutes"),
            "gemm_by_shape": m["gemm_by_shape"],
            "extensions": m.get("extensions"),
            "clocks": m["clocks"],
            "output_gather_ms": m.get("output_gather_ms"),
        }
        if "value_with_gather" in m:
            line["value_with_gather"] = m["value_with_gather"]
            line["with_gather"] = m["with_gather"]
        if config5:
            line["config5"] = config5
        if cpu:
            line["cpu_baseline"] = cpu
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_grid_arm(args):
    """The reference's own benchmark grid (examples/torch/bert/benchmark_bert.py:50-52: batch
    {1, 8, 16, 32} x seq {64, 128}) for BERT-base and BERT-large on one GPU: CUDA-graph replay,
    inputs in HBM, >= 0.3 s per cell; prints one JSON line with a row per cell, each with the
    tile-table row and K split the library picked for the layer's four GEMM shapes."""
    import torch
    from __graft_entry__ import load_package
    pkg = load_package()
    from hands_on_mlir_b200.bert_program import BertConfig, BertProgram
    hom = pkg.runner()
    torch.cuda.set_device(0)
    device = torch.device("cuda", 0)
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    hom.use_torch_stream()
    ranks = Ranks(device)
    rows = []
    for model, cfg in (("bert-base", BertConfig.base()), ("bert-large", BertConfig.large())):
        for seq in (64, 128):
            weights = make_weights_torch(cfg, seq, device)
            for batch in (1, 8, 16, 32):
                wl = dict(model=model, batch=batch, seq=seq, scaling="weak", lens=None)
                prog = BertProgram(cfg, batch, seq, fused_embedding=args.fused_embedding,
                                   fused_layernorm=args.fused_layernorm)
                prog.set_weights(weights)
                ids, mask, types = (torch.from_numpy(x).to(device) for x in make_inputs(wl, batch, 0))
                for _ in range(3):
                    prog.forward(ids, mask, types, use_graph=True)
                hom.synchronize()
                ms, n_run, _ = timed_region(ranks, stream, lambda: prog.forward(ids, mask, types, use_graph=True),
                                            20, min_seconds=0.3)
                for _ in range(3):
                    prog.forward(ids, mask, types, use_graph=False)
                hom.synchronize()
                ms_e, _, _ = timed_region(ranks, stream, lambda: prog.forward(ids, mask, types, use_graph=False),
                                          20, min_seconds=0.2)
                m, h, f = batch * seq, cfg.hidden, cfg.ffn
                shapes = {"qkv": (m, 3 * h, h, 0), "out": (m, h, h, 0), "ffn1": (m, f, h, 1), "ffn2": (m, h, f, 0)}
                tiles = {}
                for name, shp in shapes.items():
                    q = hom.gemm_query_tile(*shp)
                    tiles[name] = f"row {q['row']} ({'256' if q['row'] >= 5 else '128'}x{q['bn']}), split {q['split_k']}"
                flops = (cfg.gemm_flops_per_sequence(seq) + cfg.attention_flops_per_sequence(seq)) * batch
                rows.append({"model": model, "batch": batch, "seq": seq, "ms_per_step": ms,
                             "sequences_per_s": batch / (ms / 1e3), "model_tflops": flops / (ms / 1e3) / 1e12,
                             "eager_ms_per_step": ms_e, "steps_timed": n_run, "gemm_tiles": tiles})
                prog.close()
            del weights
    print(json.dumps({"metric": "bert_fp16_sequences_per_s", "unit": "sequences/s", "n_gpus": 1,
                      "grid": "batch {1, 8, 16, 32} x seq {64, 128}, bert-base and bert-large, CUDA-graph replay",
                      "rows": rows}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--workload", choices=sorted(WORKLOADS), default="bert-base")
    ap.add_argument("--impl", choices=["b200", "reference"], default="b200")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-config5", action="store_true",
                    help="skip the bert-large (batch 256 x seq 512, split over the GPUs) sub-record")
    ap.add_argument("--no-extensions", action="store_true",
                    help="skip timing the two LayerNorm-fusion options of the replay program beside the headline")
    ap.add_argument("--fused-layernorm", type=int, nargs="?", const=2, default=0, choices=[0, 1, 2],
                    help="extensions, off by default like --fused-embedding: 2 (the flag alone) = deferred "
                         "LayerNorm, every GEMM applies the LayerNorm of its operands in its epilogue "
                         "(homGemmDeferredLayernormF16, no LayerNorm launch inside the layers); 1 = "
                         "homGemmResidualLayernormF16 in place of the GEMM + LayerNorm call pairs")
    ap.add_argument("--fused-embedding", action="store_true",
                    help="replace the five embedding calls by homBertEmbeddingF16 (same bits; not "
                         "the call sequence the reference's lowering emits, so off by default)")
    ap.add_argument("--op", choices=sorted(OP_CASES), default=None,
                    help="time one kernel of the path on its own instead of the whole encoder")
    ap.add_argument("--tile", type=int, default=0,
                    help="with --op gemm-*: force tile-table row 1..4 (0 = automatic)")
    ap.add_argument("--split", type=int, default=1,
                    help="with --op gemm-*: K parts per output tile (1 = the library's choice)")
    ap.add_argument("--shape", default=None, help="with --op gemm-*: override M,N,K")
    ap.add_argument("--l2-resident", action="store_true",
                    help="with --op: reuse one buffer set (L2-resident figure)")
    ap.add_argument("--min-seconds", type=float, default=None,
                    help="GPU time every throughput figure is averaged over (default 1.0; lower it only "
                         "for a profiler capture, whose numbers are never bench values)")
    ap.add_argument("--grid", action="store_true",
                    help="time the reference's benchmark grid (batch 1/8/16/32 x seq 64/128, base and large)")
    args = ap.parse_args()
    if args.min_seconds is not None:
        global MIN_TIMED_SECONDS
        MIN_TIMED_SECONDS = max(0.0, args.min_seconds)
    if args.op:
        run_op_arm(args)
        return
    if args.grid:
        run_grid_arm(args)
        return

    from __graft_entry__ import load_package
    load_package()
    from hands_on_mlir_b200.bert_program import BertConfig
    workload = WORKLOADS[args.workload]
    cfg = BertConfig.base() if workload["model"] == "base" else BertConfig.large()
    if args.impl == "reference":
        run_reference_arm(args, cfg, workload)
    else:
        run_gpu_arm(args, cfg, workload)


if __name__ == "__main__":
    main()

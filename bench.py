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
    "gemm-ffn1": {"bytes": 11.07e6, "source": "profiles/gemm_pair_256x256_bert_base_ffn1.txt"},
    "gemm-qkv": {"bytes": 9.89e6, "source": "profiles/gemm_pair_256x256_bert_base_qkv.txt"},
    "gemm-ffn2": {"bytes": 36.24e6, "source": "profiles/gemm_1cta_128x192_bert_base_ffn2.txt"},
    "gemm-large-ffn1": {"bytes": 122.0e6, "source": "profiles/gemm_pair_256x256_bert_large_ffn1_m16384.txt"},
    "ln-c2": {"bytes": 12.60e6, "source": "profiles/layernorm_residual_affine_4096x768.txt"},
    "ln-large": {"bytes": 480.6e6, "source": "profiles/layernorm_inplace_131072x1024.txt"},
    "attn-c3": {"bytes": 18.90e6, "source": "profiles/attention_single_tile_bs32_seq128_h12.txt"},
    "attn-large": {"bytes": 105.8e6, "source": "profiles/attention_multi_tile_bs32_seq512_h16.txt"},
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
            self._thread.join()

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
        line["reference_matmulAddF32"] = extra
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

def run_gpu_arm(args, cfg, workload):
    import torch
    import torch.distributed as dist
    from __graft_entry__ import load_package

    rank = int(os.environ.get("RANK", "0"))
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
    from hands_on_mlir_b200.bert_program import BertProgram, shard_batch
    hom = pkg.runner()
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    hom.use_torch_stream()

    if workload["scaling"] == "weak":
        local_batch, first = workload["batch"], rank * workload["batch"]
        global_batch = workload["batch"] * world
    else:
        lo, hi = shard_batch(workload["batch"], world, rank)
        local_batch, first, global_batch = hi - lo, lo, workload["batch"]
    seq = workload["seq"]

    prog = BertProgram(cfg, local_batch, seq, fused_embedding=args.fused_embedding,
                       fused_layernorm=args.fused_layernorm)
    weights = make_weights_torch(cfg, seq, device)
    prog.set_weights(weights)
    ids_np, mask_np, types_np = make_inputs(workload, local_batch, first)
    ids_h, mask_h, types_h = (torch.from_numpy(x).pin_memory() for x in (ids_np, mask_np, types_np))
    out_h = torch.empty((local_batch, seq, cfg.hidden), dtype=torch.float16).pin_memory()
    ids_d, mask_d, types_d = (x.to(device) for x in (ids_h, mask_h, types_h))

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- device-resident throughput (value)
    for _ in range(max(args.warmup, 3)):
        prog.forward(ids_d, mask_d, types_d, use_graph=True)
    hom.synchronize()
    barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as clocks:
        ev0.record(stream)
        for _ in range(args.steps):
            prog.forward(ids_d, mask_d, types_d, use_graph=True)
        ev1.record(stream)
        barrier()
    hom.synchronize()
    ms_total = max_over_ranks(ev0.elapsed_time(ev1))
    value = global_batch * args.steps / (ms_total / 1e3)

    # ---- end to end with host buffers (e2e): every step copies its inputs from pinned host
    # memory and delivers its hidden states to pinned host memory; the delivery of step i
    # overlaps the compute of step i+1 (two result slots), and the clock stops only after the
    # last step's result is on the host.
    out_h2 = torch.empty_like(out_h).pin_memory()
    outs = (out_h, out_h2)
    for i in range(4):
        prog.forward_host_async(ids_h, mask_h, types_h, outs[i & 1], use_graph=True)
    prog.wait_host()
    barrier()
    t0 = time.perf_counter()
    for i in range(args.steps):
        prog.forward_host_async(ids_h, mask_h, types_h, outs[i & 1], use_graph=True)
    prog.wait_host()
    torch.cuda.synchronize()
    e2e_s = max_over_ranks(time.perf_counter() - t0)
    barrier()
    h2d, d2h = prog.host_traffic()
    e2e_value = global_batch * args.steps / e2e_s

    # ---- per-launch durations of a step (roofline): a second replay program is captured with
    # the library's per-launch CUDA events switched on, so every launch of its graph is bracketed
    # by event-record nodes on the launching stream; the graph is replayed and read out n_prof
    # times.  (The event nodes stand between the kernels, so this pass runs without the
    # programmatic overlap of neighbouring launches that the timed region above has.)
    prog_t = BertProgram(cfg, local_batch, seq, fused_embedding=args.fused_embedding,
                         fused_layernorm=args.fused_layernorm)
    prog_t.set_weights(weights)
    prog_t.forward(ids_d, mask_d, types_d, use_graph=True)  # first call runs eagerly (set-up)
    hom.synchronize()
    hom.op_timing(True)
    prog_t.forward(ids_d, mask_d, types_d, use_graph=True)  # capture + first launch
    hom.op_timing(False)
    hom.synchronize()
    n_prof = 5
    records = []
    for _ in range(n_prof):
        prog_t.forward(ids_d, mask_d, types_d, use_graph=True)
        hom.synchronize()
        records += hom.peek_op_timings()
    prog_t.close()
    hom.collect_op_timings()  # releases the events
    kinds = {1: "gemm", 2: "layernorm", 3: "attention", 4: "elementwise", 5: "gather", 6: "cu_seqlen"}
    per_kind = {}
    for kind, ms, flops, nbytes in records:
        d = per_kind.setdefault(kinds.get(kind, str(kind)), {"launches": 0, "ms": 0.0, "flops": 0.0,
                                                              "bytes": 0.0})
        d["launches"] += 1
        d["ms"] += ms
        d["flops"] += flops
        d["bytes"] += nbytes
    # GEMM launches grouped by their algorithmic FLOPs (= by shape)
    gemm_shapes = {}
    for kind, ms, flops, nbytes in records:
        if kind == 1:
            d = gemm_shapes.setdefault(f"{flops / 1e9:.2f}_gflop", {"launches": 0, "ms": 0.0, "flops": flops})
            d["launches"] += 1
            d["ms"] += ms
    gemm_by_shape = {k: {"launches_per_step": v["launches"] // n_prof,
                         "avg_us": 1e3 * v["ms"] / v["launches"],
                         "tflops": v["flops"] * v["launches"] / (v["ms"] / 1e3) / 1e12}
                     for k, v in gemm_shapes.items()}
    peaks, peak_src = load_peaks()
    gemm = per_kind.get("gemm", {"launches": 1, "ms": float("nan"), "flops": 0.0})
    gemm_tflops = gemm["flops"] / (gemm["ms"] / 1e3) / 1e12 if gemm["ms"] > 0 else float("nan")
    tensor_peak = peaks["bf16_tflops_sustained"]
    roofline = {
        "bound": "tensor", "kernel": "gemm_f16_kernel (all GEMM launches of a step)",
        "achieved": gemm_tflops, "peak": tensor_peak, "unit": "TFLOP/s",
        "frac": gemm_tflops / tensor_peak, "peak_source": f"{peak_src} (sustained dense bf16/fp16)",
        "traffic": ncu_traffic(args.workload)[0],
        "traffic_source": ncu_traffic(args.workload)[1],
        "algorithmic_bytes_per_launch": gemm["bytes"] / max(1, gemm["launches"]),
        "launches_per_step": gemm["launches"] // n_prof,
        "avg_launch_us": 1e3 * gemm["ms"] / max(1, gemm["launches"]),
    }
    kernel_share = {k: {"launches_per_step": v["launches"] // n_prof,
                        "ms_per_step": v["ms"] / n_prof,
                        "tflops": (v["flops"] / (v["ms"] / 1e3) / 1e12) if v["ms"] > 0 and v["flops"] else None,
                        "gbs": (v["bytes"] / (v["ms"] / 1e3) / 1e9) if v["ms"] > 0 else None}
                    for k, v in per_kind.items()}

    # ---- final gather of the hidden states (the only collective; not on the data path)
    gather_ms = None
    if world > 1:
        res = prog.result_to_torch(prog.forward(ids_d, mask_d, types_d, use_graph=True))
        bufs = [torch.empty_like(res) for _ in range(world)]
        barrier()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        g0.record(stream)
        dist.all_gather(bufs, res)
        g1.record(stream)
        torch.cuda.synchronize()
        gather_ms = max_over_ranks(g0.elapsed_time(g1))

    # ---- CPU baseline on a bounded sample (rank 0, N = 1 only)
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        enc = CpuEncoder(cfg, workload)
        n_seq, layers = enc.plan(12.0)
        secs = enc.run(n_seq, layers)
        cpu = {"value": n_seq * (layers / cfg.layers) / secs, "unit": "sequences/s",
               "cores": enc.threads, "kind": "port",
               "sample": enc.describe(n_seq, layers) + f", {secs:.1f} s"}

    if rank == 0:
        flops_per_seq = cfg.gemm_flops_per_sequence(seq) + cfg.attention_flops_per_sequence(seq)
        line = {
            "metric": "bert_fp16_sequences_per_s", "value": value, "unit": "sequences/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms_total / args.steps, "higher_is_better": True,
            "scaling": workload["scaling"], "vs_baseline": None, "dtype": "f16",
            "data": "synthetic",
            "config": {
                "workload": f"{args.workload} encoder ({cfg.layers} layers, hidden {cfg.hidden}, "
                            f"{cfg.heads} heads, FFN {cfg.ffn}), global batch {global_batch} x seq "
                            f"{seq}, {local_batch} sequences per GPU",
                "parallelism": f"batch-sharded replicas x{world}, no data-path collective",
                "l2": "no explicit flush: the per-step working set (all layer weights + "
                      "activations) exceeds the 126 MB L2",
                "launch": "CUDA-graph replay of the runner-utils call sequence"
                          + (" with the fused embedding extension" if args.fused_embedding else "")
                          + (" with the fused GEMM+LayerNorm extension" if args.fused_layernorm else ""),
            },
            "model_tflops": value * flops_per_seq / 1e12,
            "e2e": {"value": e2e_value, "unit": "sequences/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": 1e3 * e2e_s / args.steps},
            "gpu_launches": args.steps * prog.launches_per_forward(),
            "roofline": roofline,
            "kernels": kernel_share,
            "gemm_by_shape": gemm_by_shape,
            "clocks": clocks.summary(),
            "output_gather_ms": gather_ms,
        }
        if cpu:
            line["cpu_baseline"] = cpu
        print(json.dumps(line), flush=True)
    prog.close()
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--workload", choices=sorted(WORKLOADS), default="bert-base")
    ap.add_argument("--impl", choices=["b200", "reference"], default="b200")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--fused-layernorm", action="store_true",
                    help="replace the GEMM + LayerNorm call pairs (out-projection, FFN2) by "
                         "homGemmResidualLayernormF16 (an extension; off by default like "
                         "--fused-embedding)")
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
    args = ap.parse_args()
    if args.op:
        run_op_arm(args)
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

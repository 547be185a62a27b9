#!/usr/bin/env python
"""Benchmark of the block-sparse attention hot path: fwd+bwd Mtokens/s at L=4096.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Workload (default ``sweep_L4096_bs64_d05``): one attention layer, forward + backward, of the
isolated-kernel sweep shape B=8, H=8, L=4096, d_head=64, bf16, block 64, mask = diagonal band of
2 blocks + uniformly random blocks to 5 % density; Q, K, V, dO ~ N(0,1) from a seed.  A step is
one fwd+bwd over that batch; tokens per step = B*L per rank.  With N > 1 (torchrun, one rank per
GPU) every rank runs its own shard of the batch*head work with no data-path collective (weak
scaling); time = max over ranks.

One JSON line on stdout (rank 0).  ``value``: inputs resident in HBM, C ABI called directly.
``e2e``: same metric through the public module with pinned host buffers, host<->device copies
inside the timed region.  ``roofline``: the dominant kernel, timed live with CUDA events on the
launch stream (``spion_profile``).  ``cpu_baseline``: the oracle's dense-masked PyTorch path on
the host cores, on a bounded sample (N=1 only).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (B, H, L, d, bs, density, dtype)
    "sweep_L4096_bs64_d05": (8, 8, 4096, 64, 64, 0.05, "bf16"),
    "sweep_L4096_bs32_d05": (8, 8, 4096, 64, 32, 0.05, "bf16"),
    "sweep_L4096_bs64_d10": (8, 8, 4096, 64, 64, 0.10, "bf16"),
    "sweep_L4096_bs64_d30": (8, 8, 4096, 64, 64, 0.30, "bf16"),
    "sweep_L1024_bs64_d10": (8, 8, 1024, 64, 64, 0.10, "bf16"),
    "sweep_L16384_bs64_d02": (8, 8, 16384, 64, 64, 0.02, "bf16"),
    "config1_L1024_fp32": (8, 2, 1024, 32, 32, 0.15, "fp32"),
    "image_L1024_fp32_B256": (256, 2, 1024, 32, 32, 0.15, "fp32"),   # attention layer of the image-shaped training step
    "retrieval_L4096_d32_B128": (128, 2, 4096, 32, 64, 0.10, "bf16"),  # ... of the retrieval-shaped step (64 pairs)
    "tiny": (2, 2, 512, 64, 64, 0.25, "bf16"),
}

# End-to-end training-step workloads (benchmark configs 2, 3, 5): name -> (task, batch, dtype,
# quantile threshold chosen to land near the config's block density, scaling).  The batch of the
# "strong" workload is the GLOBAL batch, split evenly across ranks.
TRAIN_WORKLOADS = {
    "train_image_L1024": ("image", 256, "fp32", 0.80, "weak"),
    "train_text_L4096": ("text", 32, "bf16", 0.90, "weak"),
    "train_retrieval_L4096": ("retrieval", 64, "bf16", 0.90, "strong"),
    "train_retrieval_L4096_b8": ("retrieval", 8, "bf16", 0.90, "weak"),     # the per-GPU share of the 8-GPU run, per rank
    "train_tiny": ("text", 2, "bf16", 0.85, "weak"),
}


# dram__bytes_read.sum + dram__bytes_write.sum per launch, from one ncu capture of the same workload and
# kernels (the summaries are kept under profiles/; NCU_TRAFFIC_SOURCE names the one each entry comes from)
NCU_TRAFFIC = {
    # workload: {stage: bytes}; the forward entry depends on whether P is stored ("fused_fwd+P" / "fused_fwd")
    "sweep_L4096_bs64_d05": {"fused_fwd+P": 248.9e6, "bwd_row": 420.3e6, "spmm_dkdv": 336.4e6,
                             "fused_fwd": 134.4e6, "bwd_row_rc": 228.4e6, "bwd_col_rc": 174.9e6},
    "image_L1024_fp32_B256": {"fused_fwd+P": 581.9e6, "bwd_row": 971.0e6, "spmm_dkdv": 903.6e6},
}


NCU_TRAFFIC_SOURCE = {
    "sweep_L4096_bs64_d05": "ncu dram bytes per launch, profiles/tcgen05_kernels_sweep_L4096_bs64_d05.md",
    "image_L1024_fp32_B256": "ncu dram bytes per launch, profiles/simt_fused_fp32_image_L1024_bs32.md",
}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.idx), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for ln in self.proc.stdout:
            self.lines.append(ln.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for n, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def algorithmic(B, H, L, d, bs, nnzb, esz):
    """Algorithmic work of one fwd+bwd step (per rank)."""
    BH = B * H
    nnz = nnzb * bs * bs
    flops = 12.0 * nnz * d * BH                                     # 2 SDDMM + 4 SpMM, 2*nnz*d each
    fused_bytes = 12.0 * L * d * esz * BH                            # Q,K,V,O fwd; Q,K,V,O,dO in, dQ,dK,dV out bwd
    return flops, fused_bytes, nnz


# per-launch algorithmic bytes of each stage (p = bytes of a stored P/dS element, 4 for fp32 scratch)
def stage_bytes(stage, BH, L, d, nnz, esz, psz, p_stored=False):
    ld = BH * L * d * esz
    v = BH * nnz
    return {
        "sddmm_s": 2 * ld + 4 * v, "softmax_fwd": 4 * v + psz * v, "spmm_o": psz * v + 2 * ld,
        "sddmm_dp": 2 * ld + 4 * v, "softmax_bwd": 4 * v + psz * v + psz * v, "spmm_dq": psz * v + 2 * ld,
        "spmm_dk": psz * v + 2 * ld, "spmm_dv": psz * v + 2 * ld,
        "fused_dp_ds": 2 * ld + 2 * psz * v + 4 * BH * L,
        "spmm_dkdv": 2 * psz * v + 4 * ld, "structure": 0,
        # fused kernels: operands once, no S/P/dP/dS (P written only when the staged backward needs it)
        "fused_fwd": 4 * ld + 4 * BH * L + (psz * v if p_stored else 0),
        "bwd_row": 5 * ld + 2 * psz * v,
        # recompute backward: Q, K, V, dO, O in, dQ out (+ lse in, delta out) / Q, K, V, dO in, dK, dV out (+ lse, delta in)
        "bwd_row_rc": 6 * ld + 8 * BH * L,
        "bwd_col_rc": 6 * ld + 8 * BH * L,
    }[stage]


def stage_flops(stage, BH, d, nnz):
    if stage in ("sddmm_s", "spmm_o", "sddmm_dp", "spmm_dq", "spmm_dk", "spmm_dv", "fused_dp_ds"):
        return 2.0 * nnz * d * BH
    if stage in ("spmm_dkdv", "fused_fwd", "bwd_row"):
        return 4.0 * nnz * d * BH
    if stage == "bwd_row_rc":
        return 6.0 * nnz * d * BH
    if stage == "bwd_col_rc":
        return 8.0 * nnz * d * BH
    return 0.0


def time_c_port(Q, K, V, dO, mat, bs, reps=3):
    """Seconds per fwd+bwd of the plain-C restatement (row-wise, selected blocks only, OpenMP over the host cores),
    or None when the library cannot be built or loaded.  A second CPU figure beside the dense-masked torch path."""
    try:
        from oracle import c_oracle
        lib = c_oracle.load()
    except Exception:
        return None
    if lib is None:
        return None
    q, k, v, g = [t.numpy() for t in (Q, K, V, dO)]
    c_oracle.attention_step(q, k, v, mat, bs, g)
    t0 = time.perf_counter()
    for _ in range(reps):
        c_oracle.attention_step(q, k, v, mat, bs, g)
    return {"s_per_step": (time.perf_counter() - t0) / reps, "threads": int(lib.oracle_threads())}


def time_cpu_oracle(step, want_warmup: int, want_steps: int, budget_s: float = 25.0):
    """Bounded timing of the CPU oracle: up to 3 warm-up and 10 timed steps (what the measurement plan asks for),
    fewer when one step is so long that the whole leg would exceed the budget.  Returns (s per step, warm-up, steps)."""
    step()                                                   # cold start (thread pool, allocator): not representative
    t0 = time.perf_counter()
    step()
    first = time.perf_counter() - t0
    warm = 2
    while warm < min(max(want_warmup, 2), 3) and (warm + 1) * first < 0.3 * budget_s:
        step()
        warm += 1
    steps = max(1, min(want_steps, 10, int(0.7 * budget_s / max(first, 1e-9))))
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    return (time.perf_counter() - t0) / steps, warm, steps


def run_reference(args, rank):
    """--impl reference: the oracle's dense-masked PyTorch path on the host cores (the reference has
    no CPU implementation of the sparse kernels; this restates models/block_attn.cu:453-545)."""
    if rank != 0:
        return
    from oracle import attention as oatt
    from spion_b200 import synthetic
    B, H, L, d, bs, dens, dt = WORKLOADS[args.workload]
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    Bs = 1                                                   # bounded sample: one batch element (H heads)
    mat = synthetic.band_random_mask(2024, L // bs, dens)
    M = oatt.expand_mask(mat, bs)
    Q, K, V, dO = synthetic.qkv(99, Bs, H, L, d)
    dt_s, warm, steps = time_cpu_oracle(lambda: oatt.fwd_bwd_step(Q, K, V, dO, M), args.warmup, args.steps)
    val = Bs * L / dt_s / 1e6
    sample = f"B={Bs} of {B} batch elements (H={H}, L={L}, d={d}), fp32, {warm} warm-up + {steps} timed steps"
    cport = time_c_port(Q, K, V, dO, mat, bs)
    if cport:
        cport["value"] = Bs * L / cport["s_per_step"] / 1e6
        cport["unit"] = "Mtokens/s"
    print(json.dumps({
        "impl": "reference", "metric": "sparse-attn fwd+bwd Mtokens/s at L=%d" % L, "value": val, "unit": "Mtokens/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": warm, "ms_per_step": dt_s * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, "B": Bs, "H": H, "L": L, "d_head": d, "block": bs, "density": dens},
        "cpu_baseline": {"value": val, "unit": "Mtokens/s", "cores": cores, "kind": "port", "sample": sample,
                         "c_port": cport},
        "e2e": {"value": val, "unit": "Mtokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def run_training(args, rank, world, local_rank):
    """One optimizer step of the 2-layer SPION-CF encoder classifier per step: dense warm-up step,
    pattern discovery per layer, then timed sparse steps (fwd + bwd + gradient all-reduce + AdamW)."""
    from spion_b200 import dp, harness, synthetic
    import torch.distributed as dist
    task, batch, dt, thr, scaling = TRAIN_WORKLOADS[args.workload]
    dev = torch.device("cuda", local_rank)
    per_rank = batch // world if scaling == "strong" else batch
    cfg = harness.task_config(task, per_rank, native=True, dtype=dt)
    for kv in args.harness:                                   # e.g. --harness fused_bias_grad=1 batch_towers=0
        k, v = kv.split("=", 1)
        cfg[k] = bool(int(v))
    if args.workload == "train_tiny":
        cfg["max_seq_len"] = 512
    cfg["threshold"] = thr
    L, dual = cfg["max_seq_len"], cfg["dual"]
    tr = harness.Trainer(cfg, lr=1e-4, device=dev, seed=0)

    def host_batch(seed):
        a = synthetic.token_ids(seed + 100 * rank, per_rank, L).pin_memory()
        b = synthetic.token_ids(seed + 100 * rank + 50, per_rank, L).pin_memory() if dual else None
        return a, b, synthetic.labels(seed + rank, per_rank, cfg["num_classes"]).pin_memory()

    def to_dev(hb):
        a, b, y = hb
        ids = (a.to(dev, non_blocking=True), b.to(dev, non_blocking=True)) if dual else a.to(dev, non_blocking=True)
        return ids, y.to(dev, non_blocking=True)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    hb = host_batch(1)
    ids, y = to_dev(hb)
    _, maps = tr.step(ids, y, is_attn=True)                      # dense warm-up step (untimed)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    mat_lst = tr.discover(maps)
    torch.cuda.synchronize()
    pattern_ms = (time.perf_counter() - t0) * 1e3
    dens = [float(m.mean()) for m in mat_lst[0]]
    del maps
    torch.cuda.empty_cache()
    # A capture never holds a collective: with more than one rank the step is two graphs (forward + backward;
    # clipping + optimizer) around an eager gradient all-reduce.
    use_graph = not args.no_graph
    if use_graph:
        tr.capture_sparse_step(ids, y)
    run_step = (lambda a, b: tr.step_graph(a, b)) if use_graph else (lambda a, b: tr.step(a, b)[0])
    sampler = ClockSampler(local_rank)
    if rank == 0 and not args.no_clocks:
        sampler.start()
    for _ in range(args.warmup):
        run_step(ids, y)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        run_step(ids, y)
    e1.record()
    barrier()
    # keep rank 0 under the same load until nvidia-smi has produced a few samples (steps outside the timed region)
    t_load = time.perf_counter()
    while rank == 0 and world == 1 and sampler.proc and len(sampler.lines) < 4 and time.perf_counter() - t_load < 3.0:
        run_step(ids, y)
        torch.cuda.synchronize()
    clocks = sampler.stop() if rank == 0 and not args.no_clocks else None
    ms_local = e0.elapsed_time(e1) / args.steps
    t = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step = float(t.item()) / args.steps
    tokens = per_rank * world * L * (2 if dual else 1)
    # e2e: ids and labels from pinned host memory every step, the loss read back every step
    for _ in range(2):
        ids2, y2 = to_dev(hb); float(run_step(ids2, y2))
    barrier()
    e0.record()
    for _ in range(args.steps):
        ids2, y2 = to_dev(hb)
        loss = run_step(ids2, y2)
        lv = float(loss)                                          # device -> host read of the step's result
    e1.record()
    barrier()
    t = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_ms = float(t.item()) / args.steps
    # Where the step's time goes on every rank: CUDA events inside a few extra steps -- forward + backward,
    # the gradient all-reduce (which also absorbs the wait for the slowest rank), clipping + optimizer.
    parts = None
    ar_ms = None
    if world > 1:
        tr.allreduce_events = []
        for _ in range(10):
            run_step(ids, y)
        torch.cuda.synchronize()
        evs = tr.allreduce_events
        tr.allreduce_events = None
        if use_graph:
            med = [statistics.median(e[k].elapsed_time(e[k + 1]) for e in evs) for k in range(3)]
        else:
            med = [float("nan"), statistics.median(a.elapsed_time(b) for a, b in evs), float("nan")]
        mine = torch.tensor(med + [ms_local], device=dev, dtype=torch.float64)
        allr = [torch.zeros_like(mine) for _ in range(world)]
        dist.all_gather(allr, mine)
        parts = {"fwd_bwd_ms": [round(float(t[0]), 3) for t in allr], "allreduce_ms": [round(float(t[1]), 3) for t in allr],
                 "clip_opt_ms": [round(float(t[2]), 3) for t in allr], "step_ms": [round(float(t[3]), 3) for t in allr]}
        ar_ms = max(float(t[1]) for t in allr)
    launches = sum(int(layer.mha.block_attn.launch_count()) for layer in tr.model.model.layers)
    if rank == 0:
        print(json.dumps({
            "metric": "training-step Mtokens/s (2-layer SPION-CF encoder, L=%d)" % L, "value": tokens / (ms_step * 1e-3) / 1e6,
            "unit": "Mtokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": scaling, "vs_baseline": None, "dtype": "bf16" if dt == "bf16" else "f32",
            "data": "synthetic",
            "config": {"workload": args.workload, "task": cfg["task"], "batch_per_gpu": per_rank, "L": L,
                       "block": cfg["block_size"], "threshold": thr, "density_per_layer": dens,
                       "grad_bucket_bytes": tr.bucket.nbytes, "cuda_graph": use_graph, "pattern_discovery_ms": pattern_ms,
                       "allreduce_ms_per_step": ar_ms, "allreduce_share": (ar_ms / ms_step) if ar_ms else None,
                       "per_rank": parts,
                       "l2_policy": "activations of one step exceed L2"},
            "e2e": {"value": tokens / (e2e_ms * 1e-3) / 1e6, "unit": "Mtokens/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": int((2 if dual else 1) * per_rank * L * 8 + per_rank * 8), "d2h_bytes_per_step": 4},
            "gpu_launches": launches, "loss": lv, "clocks": clocks}))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_pattern(args, rank, local_rank):
    """Pattern discovery of one layer (conv + pool + quantile + walkers + CSR/CSC) at L=4096, block 64."""
    if rank != 0:
        return
    from spion_b200 import pattern, synthetic
    L, bs, q = (4096, 64, 0.96) if args.workload == "pattern_L4096_bs64" else (1024, 32, 0.96)
    dev = torch.device("cuda", local_rank)
    A = synthetic.structured_map(25, L).to(dev)
    for _ in range(args.warmup):
        pat = pattern.discover_pattern(A, bs, q)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        pat = pattern.discover_pattern(A, bs, q)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    peaks = load_peaks()
    by = 4.0 * L * L
    cpu = None
    if not args.no_cpu_baseline:
        from oracle import pattern as opat
        cores = os.cpu_count() or 1
        torch.set_num_threads(cores)
        An = A.cpu().numpy()
        t0 = time.perf_counter()
        opat.discover_block_mask(An, bs, q, float_path="torch")       # the reference's calls + restated walkers
        cs = time.perf_counter() - t0
        cpu = {"value": 1.0 / cs, "unit": "maps/s", "cores": cores, "kind": "port",
               "sample": "one [%d,%d] map, torch conv2d/avg_pool2d/quantile + iterative walkers" % (L, L), "s_per_map": cs}
    print(json.dumps({
        "metric": "pattern discovery maps/s at L=%d" % L, "value": 1e3 / ms, "unit": "maps/s", "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32 in, f64 accumulate, u8/int32 out", "data": "synthetic",
        "config": {"workload": args.workload, "L": L, "block": bs, "quantile": q, "nnzb": pat.nnzb,
                   "includes": "one host sync per call to return the block count"},
        "roofline": {"bound": "hbm", "achieved": by / (ms * 1e-3) / 1e9, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": by / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"], "traffic": None, "peak_source": peaks["source"],
                     "algorithmic_bytes_per_launch": by},
        "cpu_baseline": cpu, "gpu_launches": 3 * args.steps}))


def run_meanmap(args, rank, local_rank):
    """The head / batch mean of the attention map that feeds pattern discovery (models/model_transformer.py:137).
    meanmap_dense_*: the reduction of a stored [B, H, L, L] fp32 tensor (what the reference-layout warm-up path
    leaves).  meanmap_recompute_*: the native warm-up path, which stores no probability: the map is rebuilt from
    Q, K and the forward's log-sum-exp on the tensor cores (spion_mean_map_recompute; full mask)."""
    if rank != 0:
        return
    from spion_b200 import pattern, synthetic
    dev = torch.device("cuda", local_rank)
    peaks = load_peaks()
    dense = args.workload.startswith("meanmap_dense")
    if dense:
        B, H, L = 256, 2, 1024                                   # image encoder shape: 2.1 GB of probabilities
        g = torch.Generator().manual_seed(3)
        attn = torch.rand(B, H, L, L, generator=g).to(dev)
        run = lambda: pattern.mean_attention_map(attn)
        by, cfg = 4.0 * B * H * L * L + 4.0 * L * L, {"B": B, "H": H, "L": L, "stored": "fp32 [B, H, L, L]"}
    else:
        from spion_b200.native import DenseViaBlocks
        B, H, L, d, bs = 32, 2, 4096, 32, 64                     # text encoder shape
        cfg_m = {"head_dim": d, "num_head": H, "max_seq_len": L, "batch_size": B, "block_size": bs,
                 "transformer_dim": H * d, "task": "bench"}
        mod = DenseViaBlocks(cfg_m, dtype=torch.bfloat16)
        Q, K, V, _ = [t.to(torch.bfloat16).to(dev) for t in synthetic.qkv(5, B, H, L, d)]
        out, handle = mod(Q, K, V)
        run = lambda: mod.mean_attention_map(handle)
        by = 2.0 * 2 * B * H * L * d + 4.0 * B * H * L + 4.0 * L * L       # Q, K, lse in; the map out
        cfg = {"B": B, "H": H, "L": L, "d_head": d, "block": bs, "stored": "nothing (rebuilt from Q, K, lse)",
               "flops": 2.0 * B * H * L * L * d}
    for _ in range(args.warmup):
        A = run()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        A = run()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    rows = float(A.sum(-1).mean())
    line = {"metric": "mean attention maps/s at L=%d" % L, "value": 1e3 / ms, "unit": "maps/s", "n_gpus": 1,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32" if dense else "bf16 in, f32 out", "data": "synthetic",
            "config": dict(cfg, workload=args.workload, mean_row_sum=rows),
            "roofline": {"bound": "hbm", "achieved": by / (ms * 1e-3) / 1e9, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": by / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"], "traffic": None, "peak_source": peaks["source"],
                         "algorithmic_bytes_per_launch": by},
            "gpu_launches": args.steps}
    if not dense:
        line["tensor"] = {"TFLOPs": cfg["flops"] / (ms * 1e-3) / 1e12, "peak": peaks["bf16_tflops"],
                          "frac": cfg["flops"] / (ms * 1e-3) / 1e12 / peaks["bf16_tflops"]}
    print(json.dumps(line))


REFCUDA_WORKLOADS = {
    # name: (B, H, L, d, bs, density) -- fp32, the reference's own layouts
    "refcuda_config1_L1024": (8, 2, 1024, 32, 32, 0.15),
    "refcuda_L4096_bs64_d05": (4, 2, 4096, 64, 64, 0.05),
    # dense warm-up path (models/attn.cu: cuBLAS tensor-op GEMMs + its softmax kernels); block = 0 marks it
    "refcuda_dense_L1024": (8, 2, 1024, 32, 0, 1.0),
    "refcuda_dense_L4096": (2, 2, 4096, 64, 0, 1.0),
}


def run_refcuda(args, rank, local_rank):
    """The reference's own CUDA path (its four .cu files compiled unchanged for sm_100a into oracle/_ref:
    cuSPARSE SDDMM / SpMM + its softmax kernels, models/block_attn.cu:453-545) and this library, behind the
    same entry points (init / attn_forward / attn_backward) with the same fp32 buffers, timed back to back
    with CUDA events.  Operand copies the reference's Python makes per call are outside the timed loop for
    both; the zero-fill of the dP scratch, which its caller does on every backward, is inside for both."""
    if rank != 0:
        return
    import ctypes
    from spion_b200 import synthetic
    from spion_b200.attention import Attention
    from spion_b200.pattern import pattern_from_mask
    B, H, L, d, bs, dens = REFCUDA_WORKLOADS[args.workload]
    if bs == 0:
        return run_refcuda_dense(args, local_rank, B, H, L, d)
    line = {"metric": "sparse-attn fwd+bwd Mtokens/s at L=%d (reference entry points, fp32)" % L, "unit": "Mtokens/s",
            "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": args.workload, "B": B, "H": H, "L": L, "d_head": d, "block": bs}}
    ref_path = os.path.join(ROOT, "oracle", "_ref", "block_attn.so")
    if not os.path.exists(ref_path):
        line.update({"value": None, "reference_cuda": {"unavailable": "oracle/_ref/block_attn.so was not built "
                                                                       "(needs the reference checkout at build time)"}})
        print(json.dumps(line))
        return
    dev = torch.device("cuda", local_rank)
    BH = B * H
    P = ctypes.c_void_p
    ref = ctypes.CDLL(ref_path)
    ref.init.argtypes = [ctypes.c_int] * 4
    ref.init.restype = P
    ref.attn_forward.argtypes = [P] * 9 + [ctypes.c_int]
    ref.attn_backward.argtypes = [P] * 14 + [ctypes.c_int]
    ref.attn_forward.restype = None
    ref.attn_backward.restype = None
    mine = Attention._blockcuda_compile_module()
    Q, K, V, dO = [t.to(dev).contiguous() for t in synthetic.qkv(3, B, H, L, d)]
    mat = synthetic.band_random_mask(77, L // bs, dens)
    pat = pattern_from_mask(torch.as_tensor(mat).to(dev), bs)
    sm, off, col, nnz = pat.element_csr(BH)                       # Columns repeated per (b,h), as the reference passes them
    Kt = K.permute(0, 1, 3, 2).contiguous()
    Vt = V.permute(0, 1, 3, 2).contiguous()
    f32 = dict(dtype=torch.float32, device=dev)
    attn = torch.empty(BH * nnz, **f32); out = torch.empty(BH * L * d, **f32)
    dP = torch.zeros(BH * nnz, **f32); dS = torch.empty(BH * nnz, **f32)
    dQ, dK, dV = [torch.empty(BH * L * d, **f32) for _ in range(3)]
    p = lambda t: P(t.data_ptr())

    def step(lib, handle):
        lib.attn_forward(handle, p(Q), p(Kt), p(V), p(attn), p(out), p(off), p(col), p(sm), nnz)
        dP.zero_()
        lib.attn_backward(handle, p(Q), p(K), p(Vt), p(attn), p(dO), p(dP), p(dS), p(dQ), p(dK), p(dV),
                          p(off), p(col), p(sm), nnz)

    res, outs = {}, {}
    for name, lib in (("reference_cuda", ref), ("spion_b200", mine)):
        h = lib.init(d, L, BH, bs)
        for _ in range(args.warmup):
            step(lib, h)
        torch.cuda.synchronize()
        reps = []
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for _ in range(args.repeats):
            e0.record()
            for _ in range(args.steps):
                step(lib, h)
            e1.record()
            torch.cuda.synchronize()
            reps.append(e0.elapsed_time(e1) / args.steps)
        ms = statistics.median(reps)
        res[name] = {"ms_per_step": ms, "min_ms": min(reps), "max_ms": max(reps), "Mtokens_per_s": B * L / (ms * 1e-3) / 1e6}
        outs[name] = [t.clone() for t in (out, dQ, dK, dV)]
        if lib is mine:
            lib.destroy(h)
    diff = max(float((a - b).abs().max()) for a, b in zip(outs["reference_cuda"], outs["spion_b200"]))
    line.update({"value": res["spion_b200"]["Mtokens_per_s"], "ms_per_step": res["spion_b200"]["ms_per_step"],
                 "reference_cuda": res["reference_cuda"], "spion_b200": res["spion_b200"],
                 "speedup_over_reference_cuda": res["reference_cuda"]["ms_per_step"] / res["spion_b200"]["ms_per_step"],
                 "max_abs_difference_of_outputs_and_gradients": diff})
    line["config"]["density"] = float(mat.mean())
    line["config"]["l2_policy"] = "working set %.0f MB" % ((4 * Q.numel() * 4 + 3 * attn.numel() * 4) / 1e6)
    print(json.dumps(line))


def run_refcuda_dense(args, local_rank, B, H, L, d):
    """The dense warm-up path behind the reference's entry points (models/attn.cu:265-280, called as
    models/attention_cuda.py:17-74 does): the reference's file compiled unchanged (cuBLAS strided-batched GEMMs
    with fp16 tensor-op compute, its row softmax kernels) against this library's shim, same buffers."""
    import ctypes
    from spion_b200 import synthetic
    from spion_b200.attention import Attention
    line = {"metric": "dense-attn fwd+bwd Mtokens/s at L=%d (reference entry points, fp32 storage)" % L, "unit": "Mtokens/s",
            "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": args.workload, "B": B, "H": H, "L": L, "d_head": d, "block": None, "density": 1.0}}
    ref_path = os.path.join(ROOT, "oracle", "_ref", "attn.so")
    if not os.path.exists(ref_path):
        line.update({"value": None, "reference_cuda": {"unavailable": "oracle/_ref/attn.so was not built "
                                                                       "(needs the reference checkout at build time)"}})
        print(json.dumps(line))
        return
    dev = torch.device("cuda", local_rank)
    BH = B * H
    P = ctypes.c_void_p
    ref = ctypes.CDLL(ref_path)
    ref.init.argtypes = [ctypes.c_int] * 3
    ref.init.restype = P
    ref.attn_forward.argtypes = [P] * 6
    ref.attn_backward.argtypes = [P] * 12
    ref.attn_forward.restype = None
    ref.attn_backward.restype = None
    mine = Attention._cuda_compile_module()
    Q, K, V, dO = [t.to(dev).contiguous() for t in synthetic.qkv(3, B, H, L, d)]
    Qt = Q.permute(0, 1, 3, 2).contiguous(); Kt = K.permute(0, 1, 3, 2).contiguous(); Vt = V.permute(0, 1, 3, 2).contiguous()
    dOt = dO.permute(0, 1, 3, 2).contiguous()
    f32 = dict(dtype=torch.float32, device=dev)
    attn = torch.empty(BH * L * L, **f32); out = torch.empty(BH * L * d, **f32)
    s1 = torch.zeros(BH * L * L, **f32); s2 = torch.empty(BH * L * L, **f32); s3 = torch.empty(BH * L * L, **f32)
    dQ, dK, dV = [torch.empty(BH * L * d, **f32) for _ in range(3)]
    p = lambda t: P(t.data_ptr())

    def step(lib, handle):
        lib.attn_forward(handle, p(Qt), p(K), p(Vt), p(attn), p(out))
        s1.zero_()                                            # the reference's caller zero-fills it on every backward
        lib.attn_backward(handle, p(Qt), p(Kt), p(V), p(attn), p(dOt), p(s1), p(s2), p(s3), p(dQ), p(dK), p(dV))

    res, outs = {}, {}
    for name, lib in (("reference_cuda", ref), ("spion_b200", mine)):
        h = lib.init(d, L, BH)
        for _ in range(args.warmup):
            step(lib, h)
        torch.cuda.synchronize()
        reps = []
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for _ in range(args.repeats):
            e0.record()
            for _ in range(args.steps):
                step(lib, h)
            e1.record()
            torch.cuda.synchronize()
            reps.append(e0.elapsed_time(e1) / args.steps)
        ms = statistics.median(reps)
        res[name] = {"ms_per_step": ms, "min_ms": min(reps), "max_ms": max(reps), "Mtokens_per_s": B * L / (ms * 1e-3) / 1e6}
        outs[name] = [t.clone() for t in (out, dQ, dK, dV)]
        if lib is mine:
            lib.destroy(h)
    diff = max(float((a - b).abs().max()) for a, b in zip(outs["reference_cuda"], outs["spion_b200"]))
    line.update({"value": res["spion_b200"]["Mtokens_per_s"], "ms_per_step": res["spion_b200"]["ms_per_step"],
                 "reference_cuda": res["reference_cuda"], "spion_b200": res["spion_b200"],
                 "speedup_over_reference_cuda": res["reference_cuda"]["ms_per_step"] / res["spion_b200"]["ms_per_step"],
                 "max_abs_difference_of_outputs_and_gradients": diff,
                 "note": "the reference multiplies with fp16 tensor-op compute (CUBLAS_COMPUTE_32F_FAST_16F), this library's "
                         "dense entry points in fp32 on the FMA pipes: the difference of the results is the reference's rounding"})
    line["config"]["l2_policy"] = "working set %.0f MB" % ((4 * Q.numel() * 4 + 4 * attn.numel() * 4) / 1e6)
    print(json.dumps(line))


def run_sweep_table(args, rank, world, local_rank):
    """Benchmark config 4 in full: L x block x density grid (B=8, H=8, d=64, bf16), fwd+bwd of one layer through
    the C ABI with inputs resident in HBM, CUDA events; one JSON line whose "sweep" key holds the table.  Every
    rank runs the same grid on its own shard (no collective); the value reported per cell is rank 0's."""
    from spion_b200 import _lib, synthetic
    from spion_b200._lib import check, lib, ptr
    from spion_b200.native import BlockSparseAttention
    dev = torch.device("cuda", local_rank)
    B, H, d = 8, 8, 64
    steps = min(args.steps, 20)
    rows = []
    for L in (1024, 2048, 4096, 8192, 16384):
        g = torch.Generator().manual_seed(7 + L)
        Q, K, V, dO = [torch.randn(B, H, L, d, generator=g).to(torch.bfloat16).to(dev) for _ in range(4)]
        O = torch.empty_like(Q); dQ = torch.empty_like(Q); dK = torch.empty_like(Q); dV = torch.empty_like(Q)
        lse = torch.empty(B * H * L, dtype=torch.float32, device=dev)
        for bs in (32, 64):
            cfg = {"head_dim": d, "num_head": H, "max_seq_len": L, "batch_size": B, "block_size": bs,
                   "transformer_dim": H * d, "task": "sweep"}
            mod = BlockSparseAttention(cfg, dtype=torch.bfloat16, device=dev, block32=args.block32)
            check(lib.spion_set_stream(mod.handle, _lib.current_stream_ptr()))
            for dens in (0.02, 0.05, 0.10, 0.30):
                mat = synthetic.band_random_mask(2024 + bs, L // bs, dens)
                nnzb = mod.set_mask(torch.as_tensor(mat).to(dev))
                n = B * H * nnzb * bs * bs
                stored = args.mode == "stored"
                P = dS = None
                if stored:
                    P = torch.empty(n, dtype=torch.bfloat16, device=dev); dS = torch.empty_like(P)

                def step():
                    check(lib.spion_attn_forward_fused(mod.handle, ptr(Q), ptr(K), ptr(V), None, ptr(O), ptr(lse), ptr(P)))
                    if stored:
                        check(lib.spion_attn_backward_ex(mod.handle, ptr(Q), ptr(K), ptr(V), ptr(P), ptr(O), ptr(dO),
                                                         ptr(dS), None, None, ptr(dQ), ptr(dK), ptr(dV)))
                    else:
                        check(lib.spion_attn_backward_fused(mod.handle, ptr(Q), ptr(K), ptr(V), ptr(O), ptr(dO), ptr(lse),
                                                            None, ptr(dQ), ptr(dK), ptr(dV)))
                for _ in range(3):
                    step()
                mod.check_device_status()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                torch.cuda.synchronize()
                e0.record()
                for _ in range(steps):
                    step()
                e1.record()
                torch.cuda.synchronize()
                ms = e0.elapsed_time(e1) / steps
                rows.append({"L": L, "block": bs, "density": round(nnzb / float((L // bs) ** 2), 4), "nnzb": nnzb,
                             "ms_per_step": round(ms, 4), "Mtokens_per_s": round(B * L / (ms * 1e-3) / 1e6, 2)})
                del P, dS
            del mod
        del Q, K, V, dO, O, dQ, dK, dV
        torch.cuda.empty_cache()
    if rank == 0:
        head = next(r for r in rows if r["L"] == 4096 and r["block"] == 64 and abs(r["density"] - 0.05) < 0.01)
        print(json.dumps({"metric": "sparse-attn fwd+bwd Mtokens/s", "value": head["Mtokens_per_s"] * world,
                          "unit": "Mtokens/s", "n_gpus": world, "steps": steps, "warmup": 3,
                          "ms_per_step": head["ms_per_step"], "higher_is_better": True, "scaling": "weak",
                          "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                          "config": {"workload": "sweep_table", "B": B, "H": H, "d_head": d,
                                     "mode": "stored P / dS" if args.mode == "stored" else "recompute backward",
                                     "timing": "inputs resident in HBM; working set of every cell larger than L2 "
                                               "except L=1024"},
                          "sweep": rows}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=500)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="sweep_L4096_bs64_d05",
                    choices=sorted(WORKLOADS) + sorted(TRAIN_WORKLOADS) + sorted(REFCUDA_WORKLOADS) +
                    ["pattern_L4096_bs64", "pattern_L1024_bs32", "sweep_table", "meanmap_dense_L1024", "meanmap_recompute_L4096"])
    ap.add_argument("--engine", default="auto", choices=["auto", "simt", "tcgen05", "staged"])
    ap.add_argument("--mode", default="auto", choices=["auto", "fused", "stored", "staged"],
                    help="fused: S, P, dP, dS stay on chip, the backward rebuilds its tiles (tcgen05 engine); "
                         "stored: fused forward that stores P, backward kernels that read P and write dS; "
                         "staged: one kernel per stage")
    ap.add_argument("--block32", default="auto", choices=["auto", "own", "super"],
                    help="32-wide masks on the tensor-core engine: kernels on the mask's own blocks, on 64-wide super-blocks, or chosen per mask")
    ap.add_argument("--repeats", type=int, default=5, help="how often the timed loop of --steps steps is repeated")
    ap.add_argument("--no-graph", action="store_true", help="training workloads: launch the step eagerly")
    ap.add_argument("--harness", nargs="*", default=[], metavar="KEY=0|1",
                    help="training workloads: switches of the harness (fused_layernorm, fused_bias_grad, batch_towers)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-clocks", action="store_true", help="do not sample nvidia-smi (profiler runs)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    args.repeats = max(args.repeats, 1)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference(args, rank)
        return

    from spion_b200 import _lib, dp, synthetic
    from spion_b200._lib import check, lib, ptr
    from spion_b200.native import BlockSparseAttention
    import torch.distributed as dist

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: spion_b200 has no CPU path")
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    if world > 1:
        dp.init_from_env("nccl")
    dev = torch.device("cuda", local_rank)
    if args.workload in TRAIN_WORKLOADS:
        run_training(args, rank, world, local_rank)
        return
    if args.workload.startswith("pattern_"):
        run_pattern(args, rank, local_rank)
        return
    if args.workload.startswith("meanmap_"):
        run_meanmap(args, rank, local_rank)
        return
    if args.workload == "sweep_table":
        run_sweep_table(args, rank, world, local_rank)
        return
    if args.workload in REFCUDA_WORKLOADS:
        run_refcuda(args, rank, local_rank)
        return

    B, H, L, d, bs, dens, dt = WORKLOADS[args.workload]
    tdt = torch.bfloat16 if dt == "bf16" else torch.float32
    esz = 2 if dt == "bf16" else 4
    BH, nb = B * H, L // bs
    cfg = {"head_dim": d, "num_head": H, "max_seq_len": L, "batch_size": B, "block_size": bs,
           "transformer_dim": H * d, "task": "sweep"}
    engine = {"auto": _lib.ENGINE_AUTO, "simt": _lib.ENGINE_SIMT, "tcgen05": _lib.ENGINE_TCGEN05,
              "staged": _lib.ENGINE_SIMT_STAGED}[args.engine]
    mod = BlockSparseAttention(cfg, dtype=tdt, engine=engine, device=dev,
                               fused=None if args.mode == "auto" else (args.mode in ("fused", "stored")),
                               return_probs=False, recompute={"fused": True, "stored": False}.get(args.mode),
                               block32=args.block32)
    fused_fwd = mod.fused
    mat = synthetic.band_random_mask(2024, nb, dens)          # same mask on every rank (one layer)
    nnzb = mod.set_mask(torch.as_tensor(mat).to(dev))
    fused_bwd = mod.recompute    # neither P nor dS in HBM (chosen per mask when --mode auto)
    flops, fused_bytes, nnz = algorithmic(B, H, L, d, bs, nnzb, esz)

    # rank-specific shard of the batch*head work
    hQ, hK, hV, hdO = [t.to(tdt).pin_memory() for t in synthetic.qkv(99 + rank, B, H, L, d)]
    Q, K, V, dO = [t.to(dev) for t in (hQ, hK, hV, hdO)]
    n = BH * nnz
    P = dS = None
    if not mod.recompute:
        P = torch.empty(n, dtype=tdt, device=dev); dS = torch.empty(n, dtype=tdt, device=dev)
    O = torch.empty_like(Q); dQ = torch.empty_like(Q); dK = torch.empty_like(Q); dV = torch.empty_like(Q)
    scr = torch.empty(n, dtype=torch.float32, device=dev) if mod.needs_scratch else None
    check(lib.spion_set_stream(mod.handle, _lib.current_stream_ptr()))

    lse = torch.empty(BH * L, dtype=torch.float32, device=dev)

    def step_device():
        if fused_bwd:
            check(lib.spion_attn_forward_fused(mod.handle, ptr(Q), ptr(K), ptr(V), None, ptr(O), ptr(lse), None))
            check(lib.spion_attn_backward_fused(mod.handle, ptr(Q), ptr(K), ptr(V), ptr(O), ptr(dO), ptr(lse), None,
                                                ptr(dQ), ptr(dK), ptr(dV)))
            return
        if fused_fwd:
            check(lib.spion_attn_forward_fused(mod.handle, ptr(Q), ptr(K), ptr(V), None, ptr(O), ptr(lse), ptr(P)))
        else:
            check(lib.spion_attn_forward_ex(mod.handle, ptr(Q), ptr(K), ptr(V), None, ptr(P), ptr(O), ptr(scr)))
        check(lib.spion_attn_backward_ex(mod.handle, ptr(Q), ptr(K), ptr(V), ptr(P), ptr(O), ptr(dO), ptr(dS),
                                         ptr(scr), None, ptr(dQ), ptr(dK), ptr(dV)))

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        if world == 1:
            return ms
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---------------- value: inputs resident in HBM, C ABI -------------------------------------
    sampler = ClockSampler(local_rank)
    if rank == 0 and not args.no_clocks:
        sampler.start()
    for _ in range(args.warmup):
        step_device()
    mod.check_device_status()
    # keep the GPU under the same load until nvidia-smi has produced a few samples
    t_load = time.perf_counter()
    while rank == 0 and sampler.proc and len(sampler.lines) < 4 and time.perf_counter() - t_load < 3.0:
        for _ in range(20):
            step_device()
        torch.cuda.synchronize()
    barrier()
    l0 = mod.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    # the timed loop of `steps` steps is repeated; the line reports the median repeat and the spread
    rep_ms = []
    for _ in range(args.repeats):
        barrier()
        e0.record()
        for _ in range(args.steps):
            step_device()
        e1.record()
        barrier()
        rep_ms.append(max_over_ranks(e0.elapsed_time(e1)) / args.steps)
    launches = mod.launch_count() - l0
    clocks = sampler.stop() if rank == 0 else None
    ms_step = statistics.median(rep_ms)
    spread = {"repeats": args.repeats, "min_ms": min(rep_ms), "max_ms": max(rep_ms), "median_ms": ms_step}
    value = world * B * L / (ms_step * 1e-3) / 1e6

    # ---------------- per-kernel times, live, CUDA events on the launch stream -----------------
    check(lib.spion_profile_reset(mod.handle)); check(lib.spion_profile(mod.handle, 1))
    for _ in range(args.steps):
        step_device()
    stages = {}
    for s in range(_lib.STAGE_COUNT):
        tot = _lib.ctypes.c_double(0); cnt = _lib.ctypes.c_longlong(0)
        check(lib.spion_profile_get(mod.handle, s, _lib.ctypes.byref(tot), _lib.ctypes.byref(cnt)))
        if cnt.value:
            stages[lib.spion_stage_name(s).decode()] = tot.value / cnt.value
    check(lib.spion_profile(mod.handle, 0))
    peaks = load_peaks()
    psz = esz
    kern = {}
    for name, ms in stages.items():
        by = stage_bytes(name, BH, L, d, nnz, esz, psz, p_stored=not fused_bwd)
        fl = stage_flops(name, BH, d, nnz)
        kern[name] = {"ms": ms, "GBps": by / (ms * 1e-3) / 1e9 if ms > 0 else None,
                      "TFLOPs": fl / (ms * 1e-3) / 1e12 if ms > 0 else None}
    dom = max((k for k in stages if k != "structure"), key=lambda k: stages[k])
    dom_bytes = stage_bytes(dom, BH, L, d, nnz, esz, psz, p_stored=not fused_bwd)
    achieved = dom_bytes / (stages[dom] * 1e-3) / 1e9
    roofline = {"kernel": dom, "bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": achieved / peaks["hbm_gbs"],
                "traffic": NCU_TRAFFIC.get(args.workload, {}).get(dom + "+P" if (dom == "fused_fwd" and not fused_bwd) else dom),
                "traffic_source": NCU_TRAFFIC_SOURCE.get(args.workload),
                "peak_source": peaks["source"],
                "algorithmic_bytes_per_launch": dom_bytes, "ms_per_launch": stages[dom]}
    step_bound_ms = max(flops / (peaks["bf16_tflops"] * 1e12), fused_bytes / (peaks["hbm_gbs"] * 1e9)) * 1e3

    # ---------------- e2e: public module, pinned host buffers, copies inside the timed region ---
    hO = torch.empty_like(hQ).pin_memory(); hdQ = torch.empty_like(hQ).pin_memory()
    hdK = torch.empty_like(hQ).pin_memory(); hdV = torch.empty_like(hQ).pin_memory()

    # Three streams, two sets of device buffers: while step i computes, step i+1's inputs come up
    # over PCIe and step i-1's results go down, as a data loader feeding this module would do.
    main_stream = torch.cuda.current_stream()
    s_in, s_cmp, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
    dbuf = [[torch.empty_like(Q) for _ in range(4)] for _ in range(2)]
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_cmp = [torch.cuda.Event() for _ in range(2)]
    ev_out = [torch.cuda.Event() for _ in range(2)]
    keep = [None, None]

    def step_e2e(i):
        b = i & 1
        with torch.cuda.stream(s_in):
            s_in.wait_event(ev_cmp[b])                      # the compute that last read this buffer set
            for dst, src in zip(dbuf[b], (hQ, hK, hV, hdO)):
                dst.copy_(src, non_blocking=True)
            ev_in[b].record()
        with torch.cuda.stream(s_cmp):
            s_cmp.wait_event(ev_in[b])
            s_cmp.wait_event(ev_out[b])                     # results of step i-2 have left their tensors
            q = dbuf[b][0].detach().requires_grad_(True)
            k = dbuf[b][1].detach().requires_grad_(True)
            v = dbuf[b][2].detach().requires_grad_(True)
            out, _ = mod(q, k, v)
            out.backward(dbuf[b][3])
            ev_cmp[b].record()
            res = (out.detach(), q.grad, k.grad, v.grad)
            for t in res:
                t.record_stream(s_out)
            keep[b] = res
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_cmp[b])
            for dst, src in zip((hO, hdQ, hdK, hdV), keep[b]):
                dst.copy_(src, non_blocking=True)
            ev_out[b].record()

    def e2e_sync():
        for st in (s_in, s_cmp, s_out):
            main_stream.wait_stream(st)

    def timed(fn_step, n):
        """n calls of fn_step(i) on the three streams between two events on the main stream; ms per call, max over ranks"""
        barrier()
        for st in (s_in, s_cmp, s_out):
            st.wait_stream(main_stream)
        e0.record()
        for st in (s_in, s_cmp, s_out):
            st.wait_stream(main_stream)
        for i in range(n):
            fn_step(i)
        e2e_sync()
        e1.record()
        barrier()
        return max_over_ranks(e0.elapsed_time(e1)) / n

    for st in (s_in, s_cmp, s_out):
        st.wait_stream(main_stream)
    for i in range(4):
        step_e2e(i)
    e2e_sync()
    e2e_steps = min(args.steps, 100)
    e2e_rep = [timed(step_e2e, e2e_steps) for _ in range(min(args.repeats, 3))]
    e2e_ms = statistics.median(e2e_rep)
    h2d = 4 * hQ.numel() * esz
    d2h = 4 * hQ.numel() * esz

    # The same copies with no compute between them (every rank at once): what the host <-> device path
    # alone allows for this step's bytes, to read the e2e figure against.
    def step_copies(i):
        b = i & 1
        with torch.cuda.stream(s_in):
            for dst, src in zip(dbuf[b], (hQ, hK, hV, hdO)):
                dst.copy_(src, non_blocking=True)
        with torch.cuda.stream(s_out):
            for dst, src in zip((hO, hdQ, hdK, hdV), dbuf[b ^ 1]):
                dst.copy_(src, non_blocking=True)

    copy_ms = timed(step_copies, min(e2e_steps, 50))
    e2e = {"value": world * B * L / (e2e_ms * 1e-3) / 1e6, "unit": "Mtokens/s", "ms_per_step": e2e_ms,
           "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": e2e_steps,
           "spread": {"repeats": len(e2e_rep), "min_ms": min(e2e_rep), "max_ms": max(e2e_rep)},
           "host_copy_ceiling": {"ms_per_step": copy_ms, "value": world * B * L / (copy_ms * 1e-3) / 1e6,
                                 "unit": "Mtokens/s", "GBps_each_way_per_rank": h2d / (copy_ms * 1e-3) / 1e9,
                                 "note": "the step's pinned H2D and D2H copies alone, both directions at once, all ranks together"},
           "note": "public module (autograd); copies of step i+1 / i-1 overlap the compute of step i on separate streams"}
    mod.check_device_status()

    # ---------------- CPU baseline (rank 0, N=1 only): bounded sample of the same workload ------
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        from oracle import attention as oatt
        cores = os.cpu_count() or 1
        torch.set_num_threads(cores)
        Bs = 1
        M = oatt.expand_mask(mat, bs)
        cQ, cK, cV, cdO = synthetic.qkv(99, Bs, H, L, d)
        cs, cwarm, reps = time_cpu_oracle(lambda: oatt.fwd_bwd_step(cQ, cK, cV, cdO, M), 3, 10)
        cport = time_c_port(cQ, cK, cV, cdO, mat, bs)
        if cport:
            cport["value"] = Bs * L / cport["s_per_step"] / 1e6
            cport["unit"] = "Mtokens/s"
        cpu = {"value": Bs * L / cs / 1e6, "unit": "Mtokens/s", "cores": cores, "kind": "port",
               "sample": f"B={Bs} of {B} batch elements (H={H}, L={L}, d={d}), fp32 dense-masked torch, {cwarm} warm-up + {reps} timed steps",
               "s_per_step": cs, "c_port": cport}

    if rank == 0:
        line = {
            "metric": "sparse-attn fwd+bwd Mtokens/s at L=%d" % L, "value": value, "unit": "Mtokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "spread": spread,
            "dtype": "bf16" if dt == "bf16" else "f32", "data": "synthetic",
            "config": {"workload": args.workload, "B_per_gpu": B, "H": H, "L": L, "d_head": d, "block": bs,
                       "density": nnzb / float(nb * nb), "nnzb": nnzb, "engine": args.engine,
                       "mode": ("fused forward + recompute backward (no P / dS in HBM)" if fused_bwd else
                                "fused forward (P stored) + row / column backward kernels" if fused_fwd else "one kernel per stage"),
                       "l2_policy": "inputs and outputs larger than L2 (Q,K,V,dO + O,dQ,dK,dV = %.0f MB%s per step)"
                                    % (8 * hQ.numel() * esz / 1e6, "" if fused_bwd else ", P+dS = %.0f MB" % (2 * n * esz / 1e6))},
            "roofline": roofline, "kernels": kern,
            "step_bound": {"ms": step_bound_ms, "frac": step_bound_ms / ms_step,
                           "note": "max(12*nnz*d*BH flop / bf16 peak, 12*L*d*e*BH bytes / HBM peak): fully fused bound"},
            "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": int(launches), "clocks": clocks,
        }
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()

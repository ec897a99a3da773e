"""Benchmark of the full-attention mixer hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload decode|verify|prefill8k] [--impl reference]

Prints ONE JSON line.  The default workload is BASELINE.json's decode configuration (16
sequences, one query token each, 8192 cached tokens, 24/4 heads, head_dim 256, bf16).  A step
is one fused mixer call over the whole batch: rope(q,k), KV append, attention, sigmoid gate.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

KV_BYTES_PER_TOKEN = 4096  # K + V, 4 heads x 256 x bf16, for the full (unsharded) layer
FLOPS_PER_PAIR = 24576     # 4 * head_dim * q_heads per (query, key) pair


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d.get("hbm_gbs", 6650.0), d.get("bf16_tflops", 1590.0), "measured"
    return 6650.0, 1590.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for l in self.lines:
            f = [x.strip() for x in l.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for n, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def dist_env():
    return int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))


def shard_plan(n_gpus, rank):
    """KV-head sharding at 2 and 4 GPUs; at 8, one KV head per GPU pair and the pair splits the
    sequences.  Returns (kv_heads_local, seq_share) where seq_share = fraction of the global
    batch's sequences this rank serves."""
    if n_gpus == 1:
        return 4, 1.0
    if n_gpus == 2:
        return 2, 1.0
    if n_gpus == 4:
        return 1, 1.0
    if n_gpus == 8:
        return 1, 0.5
    raise SystemExit("--gpus must be 1, 2, 4 or 8")


def build_decode_workload(name, n_gpus, rank, seed):
    """Weak scaling: the global batch grows with N so that every GPU streams the same KV bytes
    as the single-GPU configuration."""
    kvh, share = shard_plan(n_gpus, rank)
    g = torch.Generator(device="cuda").manual_seed(seed + 1000 * rank)
    if name == "decode":
        n_seq_global, n_new = 16 * n_gpus, 1
        hist_global = np.full(n_seq_global, 8192, np.int32)
    else:  # verify: BASELINE config 3
        n_seq_global, n_new = 8 * n_gpus, 4
        hist_global = np.random.default_rng(seed).integers(2048, 32769 - n_new, n_seq_global).astype(np.int32)
    n_local = int(round(n_seq_global * share))
    first = (rank // 4) * n_local if n_gpus == 8 else 0
    hist = hist_global[first:first + n_local]
    cap = hist.astype(np.int64) + n_new
    cache_row = np.concatenate([[0], np.cumsum(cap)[:-1]]).astype(np.int64)
    rows = int(cap.sum())
    kvdim = kvh * 256
    dev = "cuda"
    w = {
        "n_seq": n_local, "n_new": n_new, "kv_heads": kvh, "hist": hist,
        "kc": torch.randn(rows, kvdim, device=dev, dtype=torch.bfloat16, generator=g),
        "vc": torch.randn(rows, kvdim, device=dev, dtype=torch.bfloat16, generator=g),
        "pos": torch.from_numpy(hist).to(dev), "cache_row": torch.from_numpy(cache_row).to(dev),
    }
    for k_, heads in (("q", 6 * kvh), ("gate", 6 * kvh), ("k_new", kvh), ("v_new", kvh)):
        w[k_] = torch.randn(n_local, n_new, heads, 256, device=dev, dtype=torch.bfloat16, generator=g)
    w["out"] = torch.empty_like(w["q"])
    w["lse"] = torch.empty(n_local, n_new, 6 * kvh, device=dev, dtype=torch.float32)
    # algorithmic KV bytes of this rank: every row b reads pos + b + 1 tokens, but the n_new rows of
    # a sequence share one pass over the cache, so bytes = (hist + n_new) tokens * K+V * local heads
    w["kv_bytes"] = float((hist.astype(np.int64) + n_new).sum()) * KV_BYTES_PER_TOKEN * kvh / 4
    pairs = sum(int(h) * n_new + n_new * (n_new + 1) // 2 for h in hist)
    w["flops"] = float(pairs) * FLOPS_PER_PAIR * kvh / 4
    return w


def run_ours(args, rank, local_rank, world):
    from qwengine_b200 import api
    torch.cuda.set_device(local_rank)
    if world > 1:
        torch.distributed.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    hbm_peak, tc_peak, peak_kind = measured_peaks()
    w = build_decode_workload(args.workload, world, rank, args.seed)
    mx = api.Mixer(w["n_seq"], w["n_new"], kv_heads=w["kv_heads"])
    mx.bind(w["q"], w["kc"], w["vc"], w["pos"], w["out"], k_new=w["k_new"], v_new=w["v_new"], gate=w["gate"],
            lse=w["lse"], cache_row=w["cache_row"])
    api.profile_enable(True)

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        mx.forward()
    barrier()
    mx.check_status()
    launches_per_step = mx.launches()

    # ---- timed region 1: device-resident inputs -------------------------------------------------
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    kernel_ms = []
    barrier()
    ev[0].record()
    for _ in range(args.steps):
        mx.forward()
    ev[1].record()
    barrier()
    total_ms = ev[0].elapsed_time(ev[1])
    # dominant-kernel time, one event pair per step around the split-KV kernel itself
    for _ in range(args.steps):
        mx.forward()
        kernel_ms.append(api.profile_last_kernel_ms())
    barrier()

    # ---- timed region 2: end to end through the public call with host buffers -------------------
    names = ("q", "k_new", "v_new", "gate")
    host_in = {k: w[k].cpu().pin_memory() for k in names}
    host_pos = w["pos"].cpu().pin_memory()
    host_out = torch.empty(w["out"].shape, dtype=w["out"].dtype).pin_memory()
    h2d = sum(t.numel() * t.element_size() for t in host_in.values()) + host_pos.numel() * 4
    d2h = host_out.numel() * host_out.element_size()

    def e2e_step():
        for k in names:
            w[k].copy_(host_in[k], non_blocking=True)
        w["pos"].copy_(host_pos, non_blocking=True)
        mx.forward()
        host_out.copy_(w["out"], non_blocking=True)

    for _ in range(3):
        e2e_step()
    barrier()
    ev2 = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    ev2[0].record()
    for _ in range(args.steps):
        e2e_step()
    ev2[1].record()
    barrier()
    e2e_ms = ev2[0].elapsed_time(ev2[1])
    clocks = sampler.stop() if rank == 0 else None

    # ---- reduce over ranks ---------------------------------------------------------------------------
    stats = torch.tensor([total_ms, e2e_ms, float(np.mean(kernel_ms))], device="cuda", dtype=torch.float64)
    sums = torch.tensor([w["kv_bytes"], w["flops"]], device="cuda", dtype=torch.float64)
    if world > 1:
        torch.distributed.all_reduce(stats, op=torch.distributed.ReduceOp.MAX)
        torch.distributed.all_reduce(sums, op=torch.distributed.ReduceOp.SUM)
    total_ms, e2e_ms, k_ms = [float(x) for x in stats.cpu()]
    kv_bytes_all, flops_all = [float(x) for x in sums.cpu()]
    if rank != 0:
        return
    ms_per_step = total_ms / args.steps
    value = kv_bytes_all / (ms_per_step * 1e-3) / 1e9
    achieved = w["kv_bytes"] / (k_ms * 1e-3) / 1e9
    line = {
        "metric": "decode_attn_kv_GBps", "value": round(value, 1), "unit": "GB/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(ms_per_step, 5),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: seeded N(0,1) bf16 q/k/v/gate and KV cache, no dataset",
        "config": {"workload": "%s: %d seqs x %d query token(s), kv history %s, 24q/4kv heads, head_dim 256, "
                               "partial RoPE 64, sigmoid gate" % (args.workload, (16 if args.workload == "decode" else 8) * world, w["n_new"],
                                                             "8192" if args.workload == "decode" else "U[2048,32768]"),
                   "sharding": {1: "none", 2: "kv-head (2 per GPU)", 4: "kv-head (1 per GPU)",
                                8: "kv-head x 2-way sequence split"}[world],
                   "l2_policy": "inputs larger than L2: %.0f MB of KV per GPU per step vs 126 MB L2" % (w["kv_bytes"] / 1e6)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": hbm_peak, "unit": "GB/s",
                     "frac": round(achieved / hbm_peak, 4), "traffic": None, "peak_kind": peak_kind,
                     "kernel": "splitkv_kernel", "kernel_ms": round(k_ms, 5)},
        "e2e": {"value": round(kv_bytes_all / (e2e_ms / args.steps * 1e-3) / 1e9, 1), "unit": "GB/s",
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": launches_per_step * args.steps,
        "clocks": clocks,
    }
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(w, args)
    print(json.dumps(line))


def cpu_baseline(w, args, max_seqs=4):
    """The CPU oracle timed on a bounded sample of the same workload (first sequences of the batch)."""
    from oracle import pyoracle as O
    n = min(max_seqs, w["n_seq"])
    hist = w["hist"][:n]
    rows = int((hist.astype(np.int64) + w["n_new"]).sum())
    f = lambda t: t.float().cpu().numpy()
    kc = w["kc"][:rows].view(torch.int16).cpu().numpy().view(np.uint16)
    vc = w["vc"][:rows].view(torch.int16).cpu().numpy().view(np.uint16)
    cap = hist.astype(np.int64) + w["n_new"]
    cache_row = np.concatenate([[0], np.cumsum(cap)[:-1]])
    t0 = time.perf_counter()
    O.mixer(f(w["q"][:n]), f(w["k_new"][:n]), f(w["v_new"][:n]), f(w["gate"][:n]), kc, vc, hist, cache_row,
            kv_heads=w["kv_heads"])
    dt = time.perf_counter() - t0
    nbytes = float(cap.sum()) * KV_BYTES_PER_TOKEN * w["kv_heads"] / 4
    return {"value": round(nbytes / dt / 1e9, 4), "unit": "GB/s", "cores": O.num_threads(), "kind": "port",
            "sample": "first %d of %d sequences of the same batch, one pass, %.2f s" % (n, w["n_seq"], dt)}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="decode", choices=["decode", "verify"])
    ap.add_argument("--seed", type=int, default=1234)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    rank, local_rank, world = dist_env()
    if world != args.gpus and world == 1 and args.gpus > 1:
        raise SystemExit("launch with torchrun --nproc-per-node %d for --gpus %d" % (args.gpus, args.gpus))
    if args.impl == "reference":
        from bench_reference import run_reference
        run_reference(args, rank, local_rank, world)
        return
    run_ours(args, rank, local_rank, world)
    if world > 1:
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()

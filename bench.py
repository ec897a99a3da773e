"""Benchmark of the full-attention mixer hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload decode|verify|prefill8k|prefill32k]
                    [--impl reference]

Prints ONE JSON line.  The headline workload is BASELINE.json's decode configuration (16
sequences x 1 query token against 8192 cached tokens, 24/4 heads, head_dim 256, bf16); the same
line carries, under "prefill", the other half of the metric: causal prefill attention at 8K
context on the tcgen05 kernel, and under "verify" the MTP-verify batch (8 ragged sequences x 4
query tokens) on the tcgen05 split-KV kernel.  A step is one fused mixer call over the whole batch: rope(q, k),
KV append, attention, sigmoid gate.
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
FLOPS_PER_PAIR = 24576     # 4 * head_dim * q_heads per unmasked (query, key) pair


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d.get("hbm_gbs", 6650.0), d.get("bf16_tflops", 1590.0), "measured"
    return 6650.0, 1590.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed regions run."""
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
        sm, mx, pw, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for l in self.lines:
            f = [x.strip() for x in l.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2])); pw.append(float(f[3]))
            except ValueError:
                continue
            for n, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        # the median over samples taken under load (power above the idle floor)
        busy = [c for c, w in zip(sm, pw) if w > 250.0] or sm
        return {"sm_mhz": float(np.median(busy)) if busy else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm), "power_w_max": max(pw) if pw else None}


def dist_env():
    return int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))


def shard_plan(n_gpus):
    """KV-head sharding at 2 and 4 GPUs; at 8, one KV head per GPU pair and the pair splits the
    sequences.  Returns (kv_heads_local, sequence share)."""
    plan = {1: (4, 1.0), 2: (2, 1.0), 4: (1, 1.0), 8: (1, 0.5)}
    if n_gpus not in plan:
        raise SystemExit("--gpus must be 1, 2, 4 or 8")
    return plan[n_gpus]


WORKLOADS = {
    # name: (sequences per GPU-equivalent, new tokens, description of the history)
    "decode": (16, 1, "8192"),
    "verify": (8, 4, "U[2048,32768]"),
    "prefill8k": (1, 8192, "0 (single shot, 8K context)"),
    "prefill32k": (1, 2048, "30720 (last 2048-token chunk of a 32K prefill)"),
}


def build_workload(name, n_gpus, rank, seed):
    """Weak scaling: the global batch grows with N so that every GPU does the work of the
    single-GPU configuration; ranks own disjoint KV heads (and, at 8, disjoint sequences)."""
    kvh, share = shard_plan(n_gpus)
    per, n_new, _ = WORKLOADS[name]
    n_seq_global = per * n_gpus
    if name == "decode":
        hist_global = np.full(n_seq_global, 8192, np.int32)
    elif name == "verify":
        hist_global = np.random.default_rng(seed).integers(2048, 32769 - n_new, n_seq_global).astype(np.int32)
    elif name == "prefill8k":
        hist_global = np.zeros(n_seq_global, np.int32)
    else:
        hist_global = np.full(n_seq_global, 30720, np.int32)
    n_local = int(round(n_seq_global * share))
    first = (rank // 4) * n_local if n_gpus == 8 else 0
    hist = hist_global[first:first + n_local]
    cap = hist.astype(np.int64) + n_new
    cache_row = np.concatenate([[0], np.cumsum(cap)[:-1]]).astype(np.int64)
    rows = int(cap.sum())
    kvdim = kvh * 256
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(seed + 1000 * rank)
    w = {"name": name, "n_seq": n_local, "n_seq_global": n_seq_global, "n_new": n_new, "kv_heads": kvh, "hist": hist,
         "kc": torch.randn(rows, kvdim, device=dev, dtype=torch.bfloat16, generator=g),
         "vc": torch.randn(rows, kvdim, device=dev, dtype=torch.bfloat16, generator=g),
         "pos": torch.from_numpy(hist).to(dev), "cache_row": torch.from_numpy(cache_row).to(dev)}
    for k_, heads in (("q", 6 * kvh), ("gate", 6 * kvh), ("k_new", kvh), ("v_new", kvh)):
        w[k_] = torch.randn(n_local, n_new, heads, 256, device=dev, dtype=torch.bfloat16, generator=g)
    w["out"] = torch.empty_like(w["q"])
    w["lse"] = torch.empty(n_local, n_new, 6 * kvh, device=dev, dtype=torch.float32)
    # Algorithmic work of this rank.  KV bytes: the n_new rows of a sequence share one pass over
    # its cache, (hist + n_new) tokens x 4096 B x (local heads / 4).  FLOPs: 24576 per unmasked pair.
    w["kv_bytes"] = float((hist.astype(np.int64) + n_new).sum()) * KV_BYTES_PER_TOKEN * kvh / 4
    pairs = sum(int(h) * n_new + n_new * (n_new + 1) // 2 for h in hist)
    w["flops"] = float(pairs) * FLOPS_PER_PAIR * kvh / 4
    return w


def measure(name, args, rank, world, flags_extra=0, with_e2e=True, fused_rows=False):
    """Times `steps` fused-mixer calls on workload `name`.  Returns a dict of rank-reduced results.
    fused_rows: feed the call with the fused q/k/v projection rows (fp32, as the reference's GEMM emits
    them) through qw_mixer_forward_fused instead of separate q, k, v and gate tensors."""
    from qwengine_b200 import api
    w = build_workload(name, world, rank, args.seed)
    mx = api.Mixer(w["n_seq"], w["n_new"], kv_heads=w["kv_heads"])
    if fused_rows:
        g = torch.Generator(device="cuda").manual_seed(args.seed + 7)
        kvh = w["kv_heads"]
        rows = torch.randn(w["n_seq"] * w["n_new"], 6 * kvh * 512 + 2 * kvh * 256, device="cuda", generator=g)
        nw = [(0.2 * torch.randn(256, device="cuda", generator=g)).to(torch.bfloat16) for _ in range(2)]
        mx.bind(w["q"], w["kc"], w["vc"], w["pos"], w["out"], gate=w["gate"], lse=w["lse"], cache_row=w["cache_row"],
                flags=api.F_ROPE | api.F_APPEND | api.F_GATE | flags_extra, fused=True)
        mx.forward = lambda: mx.forward_fused(rows, nw[0], nw[1])
        with_e2e = False
    else:
        mx.bind(w["q"], w["kc"], w["vc"], w["pos"], w["out"], k_new=w["k_new"], v_new=w["v_new"], gate=w["gate"],
                lse=w["lse"], cache_row=w["cache_row"], flags=api.F_ROPE | api.F_APPEND | api.F_GATE | flags_extra)
    steps = args.steps if w["n_new"] < 64 else max(3, min(args.steps, 20))
    warm = max(args.warmup, 3)

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    for _ in range(warm):
        mx.forward()
    barrier()
    mx.check_status()
    launches = mx.launches()

    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    barrier()
    ev[0].record()
    for _ in range(steps):
        mx.forward()
    ev[1].record()
    barrier()
    total_ms = ev[0].elapsed_time(ev[1])
    kernel_ms = []
    api.profile_enable(True)  # only here: the event pair sits between the two launches of a step
    for _ in range(steps):  # dominant-kernel time: an event pair around that kernel alone, every step
        mx.forward()
        kernel_ms.append(api.profile_last_kernel_ms())
    api.profile_enable(False)
    barrier()

    e2e_ms, h2d, d2h = None, 0, 0
    if with_e2e:
        # The step's inputs (q, k, v, gate of the new tokens and the positions) live in ONE pinned host
        # block and ONE device block of the same layout, so a step is one host->device copy, the call,
        # and one device->host copy of the result.  Two sets of blocks alternate, each copy engine has
        # its own stream, and events order them: the copy-in of step i+1 and the copy-out of step i-1
        # run while step i computes (every step still copies its own inputs in and its result out).
        names = ("q", "k_new", "v_new", "gate")
        sizes = [w[k].numel() * w[k].element_size() for k in names] + [w["pos"].numel() * 4]
        offs = np.concatenate([[0], np.cumsum([(b + 255) // 256 * 256 for b in sizes])]).astype(np.int64)
        view = lambda blk, i, like: blk[int(offs[i]):int(offs[i]) + sizes[i]].view(like.dtype).view(like.shape)
        host_block = torch.empty(int(offs[-1]), dtype=torch.uint8).pin_memory()
        for i, k in enumerate(names):
            view(host_block, i, w[k]).copy_(w[k].cpu())
        view(host_block, 4, w["pos"]).copy_(w["pos"].cpu())
        h2d = int(offs[-1])  # bytes the copy moves (each part padded to 256 B)
        d2h = w["out"].numel() * w["out"].element_size()
        s_in, s_out, s_comp = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.current_stream()
        sets = []
        for _ in range(2):
            blk = torch.empty(int(offs[-1]), dtype=torch.uint8, device="cuda")
            dv = {k: view(blk, i, w[k]) for i, k in enumerate(names)}
            dv["pos"] = view(blk, 4, w["pos"])
            out_d = torch.empty_like(w["out"])
            m2 = api.Mixer(w["n_seq"], w["n_new"], kv_heads=w["kv_heads"])
            m2.bind(dv["q"], w["kc"], w["vc"], dv["pos"], out_d, k_new=dv["k_new"], v_new=dv["v_new"], gate=dv["gate"],
                    lse=w["lse"], cache_row=w["cache_row"], flags=api.F_ROPE | api.F_APPEND | api.F_GATE | flags_extra)
            sets.append({"blk": blk, "out": out_d, "host_out": torch.empty(w["out"].shape, dtype=w["out"].dtype).pin_memory(),
                         "mx": m2, "ev_in": torch.cuda.Event(), "ev_comp": torch.cuda.Event(), "ev_out": torch.cuda.Event()})
        for st_ in sets:  # so that the first waits below find completed events
            st_["ev_comp"].record(s_comp)
            st_["ev_out"].record(s_out)

        def e2e_step(i):
            z = sets[i & 1]
            s_in.wait_event(z["ev_comp"])            # the block's previous step has consumed it
            with torch.cuda.stream(s_in):
                z["blk"].copy_(host_block, non_blocking=True)
                z["ev_in"].record(s_in)
            s_comp.wait_event(z["ev_in"])
            s_comp.wait_event(z["ev_out"])           # the previous result in this out buffer has left
            z["mx"].forward()
            z["ev_comp"].record(s_comp)
            s_out.wait_event(z["ev_comp"])
            with torch.cuda.stream(s_out):
                z["host_out"].copy_(z["out"], non_blocking=True)
                z["ev_out"].record(s_out)

        for i in range(4):
            e2e_step(i)
        barrier()
        ev2 = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
        ev2[0].record()
        for i in range(steps):
            e2e_step(i)
        for st_ in sets:                             # the timed region ends when the last results are on the host
            s_comp.wait_event(st_["ev_out"])
        ev2[1].record()
        barrier()
        e2e_ms = ev2[0].elapsed_time(ev2[1])
        for st_ in sets:
            st_["mx"].check_status()
    mx.check_status()

    stats = torch.tensor([total_ms, e2e_ms or 0.0, float(np.mean(kernel_ms))], device="cuda", dtype=torch.float64)
    sums = torch.tensor([w["kv_bytes"], w["flops"]], device="cuda", dtype=torch.float64)
    if world > 1:
        torch.distributed.all_reduce(stats, op=torch.distributed.ReduceOp.MAX)
        torch.distributed.all_reduce(sums, op=torch.distributed.ReduceOp.SUM)
    total_ms, e2e_ms, k_ms = [float(x) for x in stats.cpu()]
    kv_all, flops_all = [float(x) for x in sums.cpu()]
    return {"w": w, "steps": steps, "warmup": warm, "ms_per_step": total_ms / steps,
            "e2e_ms_per_step": (e2e_ms / steps) if with_e2e else None,
            "kernel_ms": k_ms, "kv_bytes_all": kv_all, "flops_all": flops_all, "launches": launches * steps,
            "h2d": h2d, "d2h": d2h}


def describe(name, world, w):
    _, n_new, hist = WORKLOADS[name]
    return ("%s: %d seq(s) x %d new token(s), kv history %s, 24q/4kv heads, head_dim 256, partial RoPE 64, "
            "sigmoid gate" % (name, w["n_seq_global"], n_new, hist))


SHARDING = {1: "none", 2: "kv-head (2 per GPU)", 4: "kv-head (1 per GPU)", 8: "kv-head x 2-way sequence split"}


def hbm_line(name, r, world, peaks):
    hbm_peak, _, kind = peaks
    w = r["w"]
    achieved = w["kv_bytes"] / (r["kernel_ms"] * 1e-3) / 1e9
    return {
        "metric": "decode_attn_kv_GBps", "value": round(r["kv_bytes_all"] / (r["ms_per_step"] * 1e-3) / 1e9, 1),
        "unit": "GB/s", "n_gpus": world, "steps": r["steps"], "warmup": r["warmup"],
        "ms_per_step": round(r["ms_per_step"], 5), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: seeded N(0,1) bf16 q/k/v/gate and KV cache, no dataset",
        "config": {"workload": describe(name, world, w), "sharding": SHARDING[world],
                   "l2_policy": "inputs larger than L2: %.0f MB of KV per GPU per step vs 126 MB L2" % (w["kv_bytes"] / 1e6)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": hbm_peak, "unit": "GB/s",
                     "frac": round(achieved / hbm_peak, 4),
                     "traffic": ({"decode": 545.4e6, "verify": 689.2e6}[name] if world == 1 else None),
                     "traffic_source": "ncu dram read+write bytes per launch, profiles/%s.txt"
                                       % ("splitkv_decode_config2" if name == "decode" else "splitkv_umma_verify"),
                     "algorithmic_bytes": w["kv_bytes"], "peak_kind": kind,
                     "kernel": "splitkv_kernel" if name == "decode" else "splitkv_umma_kernel",
                     "kernel_ms": round(r["kernel_ms"], 5),
                     "kernel_ms_how": "CUDA event pair around the attention kernel on its stream, in separate steps: the "
                                      "events sit between the step's two launches and switch their overlap off, so "
                                      "kernel_ms can exceed ms_per_step"},
        "e2e": {"value": round(r["kv_bytes_all"] / (r["e2e_ms_per_step"] * 1e-3) / 1e9, 1), "unit": "GB/s",
                "h2d_bytes_per_step": r["h2d"], "d2h_bytes_per_step": r["d2h"],
                "how": "qw_mixer_forward with host buffers: per step one pinned host->device copy of q/k/v/gate/pos, the "
                       "call, one device->host copy of the output; two buffer sets alternate so that the copies of "
                       "neighbouring steps overlap the call"},
        "gpu_launches": r["launches"],
    }


def tensor_line(name, r, world, peaks, mode):
    _, tc_peak, kind = peaks
    w = r["w"]
    achieved = w["flops"] / (r["kernel_ms"] * 1e-3) / 1e12
    return {
        "metric": "prefill_attn_TFLOPs", "value": round(r["flops_all"] / (r["ms_per_step"] * 1e-3) / 1e12, 1),
        "unit": "TFLOP/s", "n_gpus": world, "steps": r["steps"], "warmup": r["warmup"],
        "ms_per_step": round(r["ms_per_step"], 5), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: seeded N(0,1) bf16 q/k/v/gate, no dataset",
        "config": {"workload": describe(name, world, w), "sharding": SHARDING[world], "p_operand": mode,
                   "l2_policy": "L2 flushed by the q/gate/out streams of the step (%.0f MB) plus KV"
                                % (3 * w["q"].numel() * 2 / 1e6)},
        "roofline": {"bound": "tensor", "achieved": round(achieved, 1), "peak": tc_peak, "unit": "TFLOP/s",
                     "frac": round(achieved / tc_peak, 4),
                     "traffic": 319.5e6 if (name == "prefill8k" and world == 1) else None,
                     "traffic_source": "ncu dram read+write bytes per launch, profiles/prefill_umma_pair_8k.txt",
                     "algorithmic_flops": w["flops"], "peak_kind": kind,
                     "kernel": "prefill_umma_pair_kernel", "kernel_ms": round(r["kernel_ms"], 5),
                     "flops_counted": "4*256*24 per unmasked (query,key) pair; the bf16 lo pass of P is not counted"},
        "e2e": {"value": round(r["flops_all"] / (r["e2e_ms_per_step"] * 1e-3) / 1e12, 1) if r["e2e_ms_per_step"] else None,
                "unit": "TFLOP/s", "h2d_bytes_per_step": r["h2d"], "d2h_bytes_per_step": r["d2h"]},
        "gpu_launches": r["launches"],
    }


def cpu_baseline(w, min_seconds=10.0):
    """The CPU oracle timed on a bounded sample of the same workload: whole sequences of the batch,
    repeated until `min_seconds` of CPU work have been done."""
    from oracle import pyoracle as O
    n = min(4, w["n_seq"])
    hist = w["hist"][:n]
    cap = hist.astype(np.int64) + w["n_new"]
    rows = int(cap.sum())
    f = lambda t: t.float().cpu().numpy()
    kc = w["kc"][:rows].view(torch.int16).cpu().numpy().view(np.uint16)
    vc = w["vc"][:rows].view(torch.int16).cpu().numpy().view(np.uint16)
    cache_row = np.concatenate([[0], np.cumsum(cap)[:-1]])
    q, k, v, g = f(w["q"][:n]), f(w["k_new"][:n]), f(w["v_new"][:n]), f(w["gate"][:n])
    passes, t0 = 0, time.perf_counter()
    while True:
        O.mixer(q, k, v, g, kc, vc, hist, cache_row, kv_heads=w["kv_heads"])
        passes += 1
        dt = time.perf_counter() - t0
        if dt >= min_seconds or passes >= 5000:
            break
    nbytes = float(cap.sum()) * KV_BYTES_PER_TOKEN * w["kv_heads"] / 4 * passes
    return {"value": round(nbytes / dt / 1e9, 4), "unit": "GB/s", "cores": O.num_threads(), "kind": "port",
            "sample": "%d of %d sequences of the same batch, %d passes, %.1f s" % (n, w["n_seq"], passes, dt)}


def run_ours(args, rank, local_rank, world):
    from qwengine_b200 import api
    torch.cuda.set_device(local_rank)
    if world > 1:
        torch.distributed.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    peaks = measured_peaks()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    if args.workload in ("decode", "verify"):
        r = measure(args.workload, args, rank, world)
        line = hbm_line(args.workload, r, world, peaks) if rank == 0 else None
        if args.workload == "decode" and not args.no_prefill:
            rp = measure("prefill8k", args, rank, world)
            rf = measure("prefill8k", args, rank, world, flags_extra=api.F_FAST_P, with_e2e=False)
            if rank == 0:
                line["prefill"] = tensor_line("prefill8k", rp, world, peaks, "bf16 hi+lo pair (meets rel-L2 1e-3)")
                fast = tensor_line("prefill8k", rf, world, peaks, "single bf16 (rel-L2 ~1.4e-3)")
                line["prefill"]["fast_p"] = {"value": fast["value"], "unit": "TFLOP/s", "ms_per_step": fast["ms_per_step"],
                                             "roofline_frac": fast["roofline"]["frac"]}
            rq = measure("decode", args, rank, world, fused_rows=True)
            if rank == 0:
                line["fused_rows"] = {
                    "what": "the decode step fed by fp32 fused q/k/v projection rows (qw_mixer_forward_fused): scatter, "
                            "query/gate de-interleave, q/k RMSNorm, rope(k) and append in one launch before attention",
                    "value": round(rq["kv_bytes_all"] / (rq["ms_per_step"] * 1e-3) / 1e9, 1), "unit": "GB/s",
                    "ms_per_step": round(rq["ms_per_step"], 5), "gpu_launches_per_step": rq["launches"] // rq["steps"]}
            rv = measure("verify", args, rank, world, with_e2e=False)
            if rank == 0:
                v = hbm_line("verify", dict(rv, e2e_ms_per_step=rv["ms_per_step"]), world, peaks)
                line["verify"] = {"value": v["value"], "unit": v["unit"], "ms_per_step": v["ms_per_step"],
                                  "workload": v["config"]["workload"], "roofline": v["roofline"]}
    else:
        r = measure(args.workload, args, rank, world, flags_extra=api.F_FAST_P if args.fast_p else 0)
        line = tensor_line(args.workload, r, world, peaks,
                           "single bf16" if args.fast_p else "bf16 hi+lo pair") if rank == 0 else None
    if rank == 0:
        line["clocks"] = sampler.stop()
        if world == 1 and not args.no_cpu_baseline and args.workload in ("decode", "verify"):
            line["cpu_baseline"] = cpu_baseline(r["w"])
        print(json.dumps(line))
    if world > 1:
        torch.distributed.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="decode", choices=sorted(WORKLOADS))
    ap.add_argument("--seed", type=int, default=1234)
    ap.add_argument("--fast-p", action="store_true", help="prefill workloads: single-bf16 P operand")
    ap.add_argument("--no-prefill", action="store_true", help="decode workload: skip the prefill8k and verify sub-measurements")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    rank, local_rank, world = dist_env()
    if world == 1 and args.gpus > 1:
        raise SystemExit("launch with torchrun --nproc-per-node %d for --gpus %d" % (args.gpus, args.gpus))
    if args.impl == "reference":
        from bench_reference import run_reference
        run_reference(args, rank, local_rank, world)
        return
    run_ours(args, rank, local_rank, world)


if __name__ == "__main__":
    main()

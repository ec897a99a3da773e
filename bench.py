"""Benchmark of the full-attention mixer hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--repeats R] [--impl reference]
                    [--workload decode|verify|prefill8k|prefill32k|mixed|prefill32k_full]

Prints ONE JSON line.  The headline workload is BASELINE.json's decode configuration (16 sequences x 1
query token against 8192 cached tokens, 24/4 heads, head_dim 256, bf16); the same line carries, as
sub-objects, the other half of the metric and the neighbouring routes:
  prefill          causal prefill attention at 8K context on the tcgen05 CTA-pair kernel
  verify           the MTP-verify batch (8 ragged sequences x 4 query tokens) on the tcgen05 split-KV kernel
  fused_rows       the decode step fed by the fused q/k/v projection rows
  dropin           the reference's own launch sites (rope / kv_append / attn_decode|attn_prefill / gate_sigmoid,
                   one sequence at a time) through the per-kernel launchers
  decode_b1        one sequence alone, the reference's serving case
and, with more than one GPU,
  multi_gpu_check  one sequence's KV range split over all ranks, partials merged over NVLink, against the unsplit call
  mixed            BASELINE configuration 5 (64 decode sequences partitioned by KV bytes + 2 prefill chunks)
  prefill32k_full  BASELINE configuration 4 (one 32768-token prompt in 2048-token chunks), strong-scaled.
A step is one pass of the path over one batch: rope(q, k), KV append, attention, sigmoid gate.  Every
timed region is `steps` back-to-back steps between CUDA events, repeated `repeats` times; the per-step
figures are the median (and min / max) over the repeats of the slowest rank's time.
"""
import argparse
import datetime
import hashlib
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
    """(HBM GB/s, bf16 TFLOP/s burst, kind, bf16 TFLOP/s sustained under the power cap)."""
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d.get("hbm_gbs", 6650.0), d.get("bf16_tflops", 1590.0), "measured", d.get("bf16_tflops_sustained", 1400.0)
    return 6650.0, 1590.0, "fallback", 1400.0


def recorded_traffic(kernel, workload=None):
    """DRAM bytes per launch of `kernel` from the committed ncu capture (profiles/traffic.json), or None with a
    reason when the kernel's sources have changed since the capture (the figure would be stale) or the capture
    was of another workload than the one being reported."""
    p = os.path.join(ROOT, "profiles", "traffic.json")
    if not os.path.exists(p):
        return None, "no profiles/traffic.json"
    e = json.load(open(p)).get(kernel)
    if not e:
        return None, "no capture of this kernel recorded"
    if workload is not None and not e.get("workload", "").startswith(workload + ":"):
        return None, "the recorded capture is of another workload (%s)" % e.get("workload", "?")
    h = hashlib.sha256()
    for f in e["sources"]:
        with open(os.path.join(ROOT, "qwengine_b200", "csrc", f), "rb") as fh:
            h.update(fh.read())
    if h.hexdigest()[:16] != e["sources_sha16"]:
        return None, "kernel sources changed since the capture (%s)" % e.get("profile", "?")
    return e["dram_bytes_per_launch"], "ncu dram read+write bytes per launch, %s (%s)" % (e["profile"], e["workload"])


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
                "reasons": sorted(reasons), "samples": len(sm), "samples_under_load": len([w for w in pw if w > 250.0]),
                "power_w_max": max(pw) if pw else None}


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
SHARDING = {1: "none", 2: "kv-head (2 per GPU)", 4: "kv-head (1 per GPU)", 8: "kv-head x 2-way sequence split"}


# ---- timing ------------------------------------------------------------------------------------------
def barrier(world):
    if world > 1:
        torch.distributed.barrier()
    torch.cuda.synchronize()


def rank_max(values, world):
    t = torch.tensor(values, device="cuda", dtype=torch.float64)
    if world > 1:
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    return [float(x) for x in t.cpu()]


def rank_sum(values, world):
    t = torch.tensor(values, device="cuda", dtype=torch.float64)
    if world > 1:
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.SUM)
    return [float(x) for x in t.cpu()]


def timed(step, steps, warm, repeats, world):
    """`repeats` timed regions of exactly `steps` calls of step() each, after `warm` untimed calls: barrier and
    synchronize on both sides, CUDA events on the launching stream, the slowest rank's time per region.
    Returns ms per step for every region."""
    for _ in range(warm):
        step()
    out = []
    for _ in range(repeats):
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
        barrier(world)
        ev[0].record()
        for _ in range(steps):
            step()
        ev[1].record()
        barrier(world)
        out.append(ev[0].elapsed_time(ev[1]) / steps)
    return rank_max(out, world)


def stats(ms):
    return {"median": round(float(np.median(ms)), 5), "min": round(float(min(ms)), 5), "max": round(float(max(ms)), 5),
            "repeats": len(ms)}


# ---- the weak-scaled workloads (decode, verify, prefill) ------------------------------------------------
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
    return make_batch(name, hist_global[first:first + n_local], n_new, kvh, seed + 1000 * rank, n_seq_global)


def make_batch(name, hist, n_new, kvh, seed, n_seq_global=None):
    hist = np.asarray(hist, np.int32)
    n_local = len(hist)
    cap = hist.astype(np.int64) + n_new
    cache_row = np.concatenate([[0], np.cumsum(cap)[:-1]]).astype(np.int64)
    rows = int(cap.sum())
    kvdim = kvh * 256
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(seed)
    w = {"name": name, "n_seq": n_local, "n_seq_global": n_seq_global or n_local, "n_new": n_new, "kv_heads": kvh,
         "hist": hist,
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


def bind_fused(api, w, flags_extra=0):
    mx = api.Mixer(w["n_seq"], w["n_new"], kv_heads=w["kv_heads"])
    mx.bind(w["q"], w["kc"], w["vc"], w["pos"], w["out"], k_new=w["k_new"], v_new=w["v_new"], gate=w["gate"],
            lse=w["lse"], cache_row=w["cache_row"], flags=api.F_ROPE | api.F_APPEND | api.F_GATE | flags_extra)
    return mx


def kernel_time(api, step, n=10):
    """Duration of the step's dominant kernel: the library records an event pair around it on the launching
    stream; n steps, each waited for before the next is launched (the kernel timed alone, as the peaks in
    MEASURED_PEAKS.json were), median.  The pair sits between the step's two launches and so switches off their
    overlap: these are extra steps, and the figure is reported beside ms_per_step, not instead of it."""
    ms = []
    api.profile_enable(True)
    for _ in range(n):
        step()
        ms.append(api.profile_last_kernel_ms())
    api.profile_enable(False)
    return float(np.median(ms))


def measure(name, args, rank, world, flags_extra=0, with_e2e=True, fused_rows=False):
    """Times the fused mixer call on workload `name`.  Returns a dict of rank-reduced results.
    fused_rows: feed the call with the fused q/k/v projection rows (fp32, as the reference's GEMM emits
    them) through qw_mixer_forward_fused instead of separate q, k, v and gate tensors."""
    from qwengine_b200 import api
    w = build_workload(name, world, rank, args.seed)
    mx = bind_fused(api, w, flags_extra)
    step = mx.forward
    if fused_rows:
        g = torch.Generator(device="cuda").manual_seed(args.seed + 7)
        kvh = w["kv_heads"]
        rows = torch.randn(w["n_seq"] * w["n_new"], 6 * kvh * 512 + 2 * kvh * 256, device="cuda", generator=g)
        nw = [(0.2 * torch.randn(256, device="cuda", generator=g)).to(torch.bfloat16) for _ in range(2)]
        mx.bind(w["q"], w["kc"], w["vc"], w["pos"], w["out"], gate=w["gate"], lse=w["lse"], cache_row=w["cache_row"],
                flags=api.F_ROPE | api.F_APPEND | api.F_GATE | flags_extra, fused=True)
        step = lambda: mx.forward_fused(rows, nw[0], nw[1])
        with_e2e = False
    steps = args.steps if w["n_new"] < 64 else max(3, min(args.steps, 20))
    warm = max(args.warmup, 3)
    for _ in range(warm):
        step()
    torch.cuda.synchronize()
    mx.check_status()
    launches = mx.launches()
    kernel = api.last_attention_kernel()
    k_alone = rank_max([kernel_time(api, step)], world)[0]              # the kernel timed alone, before the long regions
    ms = timed(step, steps, warm, args.repeats, world)
    k_after = rank_max([kernel_time(api, step, 5)], world)[0]           # and again right after them (clocks under the power cap)
    k_mean = k_alone

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
        counter = [0]

        def e2e_step():
            z = sets[counter[0] & 1]
            counter[0] += 1
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

        for _ in range(4):
            e2e_step()
        e2e = []
        for _ in range(args.repeats):
            ev2 = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
            barrier(world)
            ev2[0].record()
            for _ in range(steps):
                e2e_step()
            for st_ in sets:                         # the timed region ends when the last results are on the host
                s_comp.wait_event(st_["ev_out"])
            ev2[1].record()
            barrier(world)
            e2e.append(ev2[0].elapsed_time(ev2[1]) / steps)
        e2e_ms = rank_max(e2e, world)
        for st_ in sets:
            st_["mx"].check_status()
    mx.check_status()
    kv_all, flops_all = rank_sum([w["kv_bytes"], w["flops"]], world)
    return {"w": w, "steps": steps, "warmup": warm, "ms": ms, "ms_per_step": float(np.median(ms)),
            "e2e_ms": e2e_ms, "e2e_ms_per_step": float(np.median(e2e_ms)) if e2e_ms else None,
            "kernel_ms": k_mean, "kernel_ms_after": k_after, "kernel": kernel, "kv_bytes_all": kv_all, "flops_all": flops_all,
            "launches": launches * steps, "h2d": h2d, "d2h": d2h}


def describe(name, world, w):
    _, n_new, hist = WORKLOADS[name]
    return ("%s: %d seq(s) x %d new token(s), kv history %s, 24q/4kv heads, head_dim 256, partial RoPE 64, "
            "sigmoid gate" % (name, w["n_seq_global"], n_new, hist))


KERNEL_MS_HOW = ("CUDA event pair around the attention kernel on its stream: 10 extra steps before the timed regions, each "
                 "waited for before the next (the kernel alone, as the measured peaks were taken), median.  The events sit "
                 "between the step's two launches and switch their overlap off, so kernel_ms can exceed ms_per_step; "
                 "frac_of_step uses ms_per_step (back-to-back steps, clocks as the power cap leaves them) instead")


def hbm_roofline(algorithmic_bytes, kernel_ms, step_ms, kernel, peaks, world, workload=None):
    hbm_peak, _, kind = peaks[:3]
    achieved = algorithmic_bytes / (kernel_ms * 1e-3) / 1e9
    traffic, src = recorded_traffic(kernel, workload) if world == 1 else (None, "captured on one GPU only")
    return {"bound": "hbm", "achieved": round(achieved, 1), "peak": hbm_peak, "unit": "GB/s",
            "frac": round(achieved / hbm_peak, 4),
            "frac_of_step": round(algorithmic_bytes / (step_ms * 1e-3) / 1e9 / hbm_peak, 4),
            "traffic": traffic, "traffic_source": src, "algorithmic_bytes": algorithmic_bytes, "peak_kind": kind,
            "kernel": kernel, "kernel_ms": round(kernel_ms, 5), "kernel_ms_how": KERNEL_MS_HOW}


def tensor_roofline(flops, kernel_ms, step_ms, kernel, peaks, world, kernel_ms_after=None, workload=None):
    _, tc_peak, kind, tc_sustained = peaks
    achieved = flops / (kernel_ms * 1e-3) / 1e12
    traffic, src = recorded_traffic(kernel, workload) if world == 1 else (None, "captured on one GPU only")
    return {"bound": "tensor", "achieved": round(achieved, 1), "peak": tc_peak, "unit": "TFLOP/s",
            "frac": round(achieved / tc_peak, 4),
            "frac_of_step": round(flops / (step_ms * 1e-3) / 1e12 / tc_peak, 4),
            "traffic": traffic, "traffic_source": src, "algorithmic_flops": flops, "peak_kind": kind,
            "kernel": kernel, "kernel_ms": round(kernel_ms, 5), "kernel_ms_how": KERNEL_MS_HOW,
            "sustained": None if kernel_ms_after is None else {
                "kernel_ms": round(kernel_ms_after, 5), "peak": tc_sustained,
                "frac": round(flops / (kernel_ms_after * 1e-3) / 1e12 / tc_sustained, 4),
                "what": "the same kernel right after the back-to-back regions, against the sustained (power-capped) "
                        "cuBLAS figure of MEASURED_PEAKS.json"},
            "flops_counted": "4*256*24 per unmasked (query,key) pair; the bf16 lo pass of P is not counted"}


def hbm_line(name, r, world, peaks):
    w = r["w"]
    line = {
        "metric": "decode_attn_kv_GBps", "value": round(r["kv_bytes_all"] / (r["ms_per_step"] * 1e-3) / 1e9, 1),
        "unit": "GB/s", "n_gpus": world, "steps": r["steps"], "warmup": r["warmup"],
        "ms_per_step": round(r["ms_per_step"], 5), "ms_per_step_stats": stats(r["ms"]), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: seeded N(0,1) bf16 q/k/v/gate and KV cache, no dataset",
        "config": {"workload": describe(name, world, w), "sharding": SHARDING[world],
                   "l2_policy": "inputs larger than L2: %.0f MB of KV per GPU per step vs 126 MB L2" % (w["kv_bytes"] / 1e6)},
        "roofline": hbm_roofline(w["kv_bytes"], r["kernel_ms"], r["ms_per_step"], r["kernel"], peaks, world, name),
        "gpu_launches": r["launches"],
    }
    if r["e2e_ms_per_step"]:
        line["e2e"] = {"value": round(r["kv_bytes_all"] / (r["e2e_ms_per_step"] * 1e-3) / 1e9, 1), "unit": "GB/s",
                       "h2d_bytes_per_step": r["h2d"], "d2h_bytes_per_step": r["d2h"], "ms_per_step_stats": stats(r["e2e_ms"]),
                       "how": "qw_mixer_forward with host buffers: per step one pinned host->device copy of q/k/v/gate/pos, "
                              "the call, one device->host copy of the output; two buffer sets alternate so that the copies "
                              "of neighbouring steps overlap the call"}
    return line


def tensor_line(name, r, world, peaks, mode):
    w = r["w"]
    line = {
        "metric": "prefill_attn_TFLOPs", "value": round(r["flops_all"] / (r["ms_per_step"] * 1e-3) / 1e12, 1),
        "unit": "TFLOP/s", "n_gpus": world, "steps": r["steps"], "warmup": r["warmup"],
        "ms_per_step": round(r["ms_per_step"], 5), "ms_per_step_stats": stats(r["ms"]), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: seeded N(0,1) bf16 q/k/v/gate, no dataset",
        "config": {"workload": describe(name, world, w), "sharding": SHARDING[world], "p_operand": mode,
                   "l2_policy": "L2 flushed by the q/gate/out streams of the step (%.0f MB) plus KV"
                                % (3 * w["q"].numel() * 2 / 1e6)},
        "roofline": tensor_roofline(w["flops"], r["kernel_ms"], r["ms_per_step"], r["kernel"], peaks, world, r["kernel_ms_after"], name),
        "gpu_launches": r["launches"],
    }
    if r["e2e_ms_per_step"]:
        line["e2e"] = {"value": round(r["flops_all"] / (r["e2e_ms_per_step"] * 1e-3) / 1e12, 1), "unit": "TFLOP/s",
                       "h2d_bytes_per_step": r["h2d"], "d2h_bytes_per_step": r["d2h"]}
    return line


# ---- the reference's launch sites through the per-kernel launchers ----------------------------------------
def measure_dropin(args, peaks):
    """One GPU.  (a) BASELINE configuration 2 served as the reference serves it -- one sequence at a time, the five
    launches of src/model.cu:228-240 per sequence; (b) one 2048-token chunk behind 30720 cached tokens through
    the five launches of src/prefill.cu:142-156.  bf16 activations (the measured flavour)."""
    from qwengine_b200 import api
    out = {}
    # (a) decode, 16 sequences, each its own contiguous cache of ctx rows and its own device position
    n_seq, hist, ctx = 16, 8192, 8448
    g = torch.Generator(device="cuda").manual_seed(args.seed + 11)
    rn = lambda *s: torch.randn(*s, device="cuda", dtype=torch.bfloat16, generator=g)
    seqs = []
    for s in range(n_seq):
        seqs.append({"kc": rn(ctx, 1024), "vc": rn(ctx, 1024), "q0": rn(1, 24, 256), "k0": rn(1, 4, 256), "v": rn(1, 4, 256),
                     "gate": rn(1, 24, 256), "q": torch.empty(1, 24, 256, device="cuda", dtype=torch.bfloat16),
                     "k": torch.empty(1, 4, 256, device="cuda", dtype=torch.bfloat16),
                     "out": torch.empty(1, 24, 256, device="cuda", dtype=torch.bfloat16),
                     "dpos": torch.tensor([hist], dtype=torch.int32, device="cuda")})
    scratch = torch.empty(api.attn_decode_scratch_floats(24, 4, ctx, 1), dtype=torch.float32, device="cuda")
    launches = [0]

    def decode_step():
        n = 0
        for z in seqs:
            z["q"].copy_(z["q0"]); z["k"].copy_(z["k0"])      # rope works in place: start from un-rotated rows
            api.rope(z["q"], 24, 256, 64, z["dpos"], 1e7, B=1)
            api.rope(z["k"], 4, 256, 64, z["dpos"], 1e7, B=1)
            api.kv_append(z["k"], z["v"], z["kc"], z["vc"], z["dpos"], 1024, B=1)
            api.attn_decode(z["q"], z["kc"], z["vc"], z["out"], z["dpos"], 256, 4, 24, 1.0 / 16.0, scratch, ctx, B=1)
            n += api.lib().qw_last_launch_count()
            api.gate_sigmoid(z["out"], z["gate"], 24 * 256)
            n += 4
        launches[0] = n

    ms = timed(decode_step, max(3, args.steps // 5), 3, args.repeats, 1)
    kernel = api.last_attention_kernel()
    kv_bytes = float(n_seq * (hist + 1)) * KV_BYTES_PER_TOKEN
    api.profile_enable(True)
    kms = []
    for _ in range(3):
        for z in seqs:
            api.attn_decode(z["q"], z["kc"], z["vc"], z["out"], z["dpos"], 256, 4, 24, 1.0 / 16.0, scratch, ctx, B=1)
            kms.append(api.profile_last_kernel_ms())
    api.profile_enable(False)
    per_seq_kernel = float(np.mean(kms))
    hbm_peak = peaks[0]
    out["decode"] = {
        "what": "16 sequences x 1 token x 8192 cached, one sequence at a time: qw_rope x2, qw_kv_append, "
                "qw_attn_decode, qw_gate_sigmoid per sequence (bf16), scratch of the reference's size",
        "value": round(kv_bytes / (float(np.median(ms)) * 1e-3) / 1e9, 1), "unit": "GB/s",
        "ms_per_step": round(float(np.median(ms)), 5), "ms_per_step_stats": stats(ms), "gpu_launches_per_step": launches[0],
        "roofline": {"bound": "hbm", "kernel": kernel, "kernel_ms": round(per_seq_kernel, 5),
                     "algorithmic_bytes": kv_bytes / n_seq, "achieved": round(kv_bytes / n_seq / (per_seq_kernel * 1e-3) / 1e9, 1),
                     "peak": hbm_peak, "unit": "GB/s", "frac": round(kv_bytes / n_seq / (per_seq_kernel * 1e-3) / 1e9 / hbm_peak, 4),
                     "note": "one sequence per launch, as the reference serves (README.md:365-367): 33.6 MB per launch "
                             "cannot fill the machine; the batched fused call above is the measured path"}}
    del seqs
    # (b) prefill chunk
    T, pos0, ctx = 2048, 30720, 32768
    kc, vc = rn(ctx, 1024), rn(ctx, 1024)
    q0, k0, v, gate = rn(T, 24, 256), rn(T, 4, 256), rn(T, 4, 256), rn(T, 24, 256)
    q, k, o = torch.empty_like(q0), torch.empty_like(k0), torch.empty_like(q0)
    dpos = torch.tensor([pos0], dtype=torch.int32, device="cuda")
    scratch = torch.empty(api.attn_prefill_scratch_floats(24, 4, ctx, T), dtype=torch.float32, device="cuda")

    def prefill_step():
        q.copy_(q0); k.copy_(k0)
        api.rope(q, 24, 256, 64, dpos, 1e7, B=T)
        api.rope(k, 4, 256, 64, dpos, 1e7, B=T)
        api.kv_append(k, v, kc, vc, dpos, 1024, B=T)
        api.attn_prefill(q, kc, vc, o, dpos, 256, 4, 24, 1.0 / 16.0, scratch, ctx, T)
        api.gate_sigmoid(o, gate, T * 24 * 256)

    for _ in range(3):
        prefill_step()
    torch.cuda.synchronize()
    api.profile_enable(True)
    kms = []
    for _ in range(10):   # the attention kernel alone, each launch waited for, before the back-to-back regions
        api.attn_prefill(q, kc, vc, o, dpos, 256, 4, 24, 1.0 / 16.0, scratch, ctx, T)
        kms.append(api.profile_last_kernel_ms())
        kernel = api.last_attention_kernel()
    api.profile_enable(False)
    ms = timed(prefill_step, max(3, min(args.steps, 10)), 3, args.repeats, 1)
    flops = float(T * pos0 + T * (T + 1) // 2) * FLOPS_PER_PAIR
    out["prefill_chunk"] = {
        "what": "one 2048-token chunk behind 30720 cached tokens: qw_rope x2, qw_kv_append, qw_attn_prefill, "
                "qw_gate_sigmoid (bf16), as src/prefill.cu:142-156 launches them",
        "value": round(flops / (float(np.median(ms)) * 1e-3) / 1e12, 1), "unit": "TFLOP/s",
        "ms_per_step": round(float(np.median(ms)), 5), "ms_per_step_stats": stats(ms), "gpu_launches_per_step": 5,
        "roofline": tensor_roofline(flops, float(np.median(kms)), float(np.median(ms)), kernel, peaks, 1, workload="prefill_chunk")}
    return out


def measure_decode_b1(args, peaks):
    """One sequence alone, one new token: the reference's actual serving case (grid (24, 1) at src/model.cu:236).
    Timed twice: launched from Python every step, and as a replayed CUDA graph of the two-launch step, which is how
    the reference runs its decode step (src/model.cu:318-327) and takes the host's launch cost out."""
    from qwengine_b200 import api
    res = {}
    for hist, n_new in ((8192, 1), (32768, 1), (8192, 4), (32768, 4)):
        # One sequence's KV (33.6 MB at 8K) fits the 126 MB L2, and the reference runs this call once per full-attention
        # layer, each with a cache of its own: so the steps rotate over enough caches ("layers") to stream more than
        # 600 MB before one is read again, and every step finds its KV in HBM, not in L2.
        w0 = make_batch("decode_b1", [hist], n_new, 4, args.seed + 21)
        n_rot = int(600e6 // w0["kv_bytes"]) + 1
        ws = [w0] + [make_batch("decode_b1", [hist], n_new, 4, args.seed + 21 + i) for i in range(1, n_rot)]
        mxs = [bind_fused(api, w) for w in ws]
        w = w0

        def sweep(stream=None):
            for m in mxs:
                m.forward(stream=stream)

        steps = max(1, args.steps // n_rot + 1)
        ms = [t / n_rot for t in timed(sweep, steps, 2, args.repeats, 1)]
        for m in mxs:
            m.check_status()
        s = torch.cuda.Stream()
        with torch.cuda.stream(s):
            sweep(s)
            s.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=s):
                sweep(s)
        torch.cuda.synchronize()
        ms_g = [t / n_rot for t in timed(g.replay, steps, 2, args.repeats, 1)]
        for m in mxs:
            m.check_status()
        us, us_g = float(np.median(ms)) * 1e3, float(np.median(ms_g)) * 1e3
        res[("hist_%d" if n_new == 1 else "verify4_hist_%d") % hist] = {
                                 "us_per_step": round(us_g, 2), "us_per_step_python_launch": round(us, 2),
                                 "us_stats": {k: (round(v * 1e3, 2) if k != "repeats" else v) for k, v in stats(ms_g).items()},
                                 "kv_GBps": round(w["kv_bytes"] / (us_g * 1e-6) / 1e9, 1),
                                 "hbm_frac": round(w["kv_bytes"] / (us_g * 1e-6) / 1e9 / peaks[0], 4),
                                 "kernel": api.last_attention_kernel(), "caches_rotated": n_rot}
        del mxs, ws
    res["what"] = ("one sequence x 1 new token (hist_*) or x 4 draft tokens (verify4_hist_*, the reference's MTP verify), "
                   "fused call (2 launches per step); the steps rotate over caches_rotated caches of that length (more than "
                   "600 MB: every step streams its KV from HBM, as one layer after another does in the reference's decode "
                   "graph); us_per_step = a CUDA graph of one such rotation replayed, per step; us_per_step_python_launch = "
                   "the same steps launched from the host; latency-bound: 33.6 MB / 134 MB of KV per step")
    return res


# ---- multi-GPU sub-benchmarks ----------------------------------------------------------------------------------
def multi_gpu_check(args, rank, world, ex_cls):
    """One sequence's KV range cut into `world` ranges, one per rank; every rank attends to its range (q rotated in
    the kernel from q_pos), the partials are merged in the combine kernel over NVLink peer memory, and the result
    is compared with the unsplit call on rank 0's copy of the same data."""
    from qwengine_b200 import api
    hist, B = 20000 + 128 * world, 4
    g = torch.Generator(device="cpu").manual_seed(args.seed + 31)     # the same data on every rank
    rn = lambda *s: torch.randn(*s, generator=g).to(torch.bfloat16).cuda()
    L = hist + B
    kc, vc = rn(L, 1024), rn(L, 1024)
    q, k, v, gate = rn(1, B, 24, 256), rn(1, B, 4, 256), rn(1, B, 4, 256), rn(1, B, 24, 256)
    cuts = [min(hist, (hist // world // 128) * 128 * i) for i in range(world)] + [L]
    lo, hi = cuts[rank], cuts[rank + 1]
    ex = ex_cls(B, 24)
    mx = api.Mixer(1, B)
    crow = torch.tensor([lo], dtype=torch.int64, device="cuda")
    q_pos = torch.tensor([hist], dtype=torch.int32, device="cuda")
    scratch_out = torch.empty(1, B, 24, 256, dtype=torch.bfloat16, device="cuda")
    if rank == world - 1:   # owns the new rows: appends them, causal among them
        pos = torch.tensor([hi - lo - B], dtype=torch.int32, device="cuda")
        mx.bind(q, kc, vc, pos, scratch_out, k_new=k, v_new=v, cache_row=crow, flags=api.F_ROPE | api.F_APPEND, q_pos=q_pos)
    else:
        pos = torch.tensor([hi - lo], dtype=torch.int32, device="cuda")
        mx.bind(q, kc, vc, pos, scratch_out, cache_row=crow, flags=api.F_ROPE | api.F_NO_CAUSAL, q_pos=q_pos)
    out = torch.zeros(B, 24, 256, dtype=torch.float32, device="cuda")
    lse = torch.zeros(B, 24, dtype=torch.float32, device="cuda")
    mx.forward_partial(ex.partial())
    kernel = api.last_attention_kernel()
    ex.combine(out, gate=gate.view(B, 24, 256), lse=lse)
    torch.cuda.synchronize()
    mx.check_status()
    ex.check_status()
    # every rank must hold the same bits (same parts, merged in the same order)
    everyone = torch.empty((world,) + tuple(out.shape), dtype=out.dtype, device="cuda")
    torch.distributed.all_gather_into_tensor(everyone, out.contiguous())
    same = all(bool(torch.equal(everyone[i], everyone[0])) for i in range(1, world))
    res = None
    if rank == 0:
        kc1, vc1 = kc.clone(), vc.clone()
        m1 = api.Mixer(1, B)
        ref = torch.zeros(1, B, 24, 256, dtype=torch.float32, device="cuda")
        lse1 = torch.zeros(1, B, 24, dtype=torch.float32, device="cuda")
        m1.bind(q, kc1, vc1, torch.tensor([hist], dtype=torch.int32, device="cuda"), ref, k_new=k, v_new=v, gate=gate, lse=lse1)
        m1.forward()
        torch.cuda.synchronize()
        m1.check_status()
        d = (out - ref.view(B, 24, 256)).double()
        rel = float(torch.sqrt((d ** 2).sum() / (ref.double() ** 2).sum()))
        res = {"what": "KV range of one %d-token sequence (4 new rows) cut over %d GPUs, partials merged over NVLink peer "
                       "memory inside the combine kernel, against the unsplit call" % (L, world),
               "max_abs_vs_unsplit": float(d.abs().max()), "rel_l2_vs_unsplit": rel,
               "lse_max_abs_vs_unsplit": float((lse - lse1.view(B, 24)).abs().max()),
               "ranks_bit_identical": same, "kernel": kernel,
               "ok": bool(same and float(d.abs().max()) <= 2e-2 and rel <= 1e-3)}
    return res, ex


def measure_mixed(args, rank, world, peaks, ex_cls):
    """BASELINE configuration 5, strong-scaled: 64 decode sequences with log-uniform histories in [512, 131072],
    partitioned over the ranks by KV bytes (sharding.partition_for_exchange; sequences of more than 32768 tokens
    are cut into ranges on different ranks and merged over NVLink), plus two prefill chunks of 4096 tokens split
    over the ranks by chunk and KV head."""
    from qwengine_b200 import api, sharding
    rng = np.random.default_rng(args.seed + 41)
    n_seq = 64
    hist = np.exp(rng.uniform(np.log(512), np.log(131072), n_seq)).astype(np.int64)
    lens = hist + 1                                              # the new token is appended
    bins = sharding.partition_for_exchange(lens, world, max_piece=32768)
    owners = {}
    for r, b in enumerate(bins):
        for s, a, e in b:
            owners.setdefault(s, []).append(r)
    split = sorted(s for s, o in owners.items() if len(o) > 1)
    slot_of = {s: j for j, s in enumerate(split)}
    mine = bins[rank]
    whole = [s for s, a, e in mine if (a, e) == (0, int(lens[s]))]
    pieces = [(s, a, e) for s, a, e in mine if (a, e) != (0, int(lens[s]))]
    g = torch.Generator(device="cuda").manual_seed(args.seed + 100 * rank + 43)
    rn = lambda *s: torch.randn(*s, device="cuda", dtype=torch.bfloat16, generator=g)
    # -- whole sequences: one fused decode call
    calls = []
    if whole:
        wb = make_batch("mixed-whole", hist[whole], 1, 4, args.seed + 100 * rank + 44)
        mw = bind_fused(api, wb)
        calls.append(mw.forward)
    # -- split sequences: one partial call over every split sequence (pos = 0 where this rank holds no range)
    n_split = len(split)
    ex = None
    if world > 1 and n_split:
        ex = ex_cls(n_split, 24)
        rows = sum(e - a for _, a, e in pieces)
        kcp, vcp = rn(max(rows, 128), 1024), rn(max(rows, 128), 1024)
        pos_p = np.zeros(n_split, np.int32)
        crow_p = np.zeros(n_split, np.int64)
        tails, r0 = [], 0
        for s, a, e in pieces:
            j = slot_of[s]
            pos_p[j], crow_p[j] = e - a, r0
            if e == int(lens[s]):
                tails.append((j, r0 + e - a - 1))
            r0 += e - a
        qs, gs = rn(n_split, 1, 24, 256), rn(n_split, 1, 24, 256)
        q_pos = torch.from_numpy(hist[split].astype(np.int32)).cuda()
        mp = api.Mixer(n_split, 1)
        scratch_out = torch.empty(n_split, 1, 24, 256, dtype=torch.bfloat16, device="cuda")
        mp.bind(qs, kcp, vcp, torch.from_numpy(pos_p).cuda(), scratch_out, cache_row=torch.from_numpy(crow_p).cuda(),
                flags=api.F_ROPE | api.F_NO_CAUSAL, q_pos=q_pos)
        out_s = torch.empty(n_split, 24, 256, dtype=torch.bfloat16, device="cuda")
        ma = None
        if tails:   # the ranges that end their sequence append its new row first (rope(k) from the absolute position)
            ma = api.Mixer(len(tails), 1)
            ma.bind_append_only(kcp, vcp, torch.tensor([t[1] for t in tails], dtype=torch.int32, device="cuda") * 0,
                                rn(len(tails), 1, 4, 256), rn(len(tails), 1, 4, 256),
                                cache_row=torch.tensor([t[1] for t in tails], dtype=torch.int64, device="cuda"),
                                q_pos=q_pos[[t[0] for t in tails]].contiguous())

        # This rank's partials are published FIRST and merged LAST, with the whole sequences' call in between: by the
        # time a rank reads its peers' partials they have long been written, so the combine does not wait for the
        # slowest rank (merged right after publishing it took 31 us at 2 GPUs and 76 us at 4, nearly all of it waiting).
        def split_publish():
            if ma is not None:
                ma.forward()
            part = ex.partial()
            part.zero_()                              # ranks without a range of a sequence contribute l = 0
            mp.forward_partial(part)

        def split_combine():
            ex.combine(out_s, gate=gs.view(n_split, 24, 256))

        calls.insert(0, split_publish)
        calls.append(split_combine)
    # -- prefill chunks: 2 x 4096 tokens; chunk and KV heads by rank
    per_chunk = max(1, world // 2)
    kvh_p = 4 // per_chunk if world > 1 else 4
    n_chunks_local = 2 if world == 1 else 1
    wp = make_batch("mixed-prefill", [0] * n_chunks_local, 4096, kvh_p, args.seed + 100 * rank + 45)
    mpf = bind_fused(api, wp)

    def decode_part():
        for c in calls:
            c()

    def whole_step():
        decode_part()
        mpf.forward()

    steps = max(3, args.steps // 5)
    ms_dec = timed(decode_part, steps, 3, args.repeats, world)
    ms_pre = timed(mpf.forward, steps, 3, args.repeats, world)
    ms_all = timed(whole_step, steps, 3, args.repeats, world)
    comb_ms = comb_ms_last = None
    if ex is not None:   # the combine's share: an event pair around it, in its place at the end of the step
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t = []
        for _ in range(5):
            for c in calls[:-1]:
                c()
            e0.record(); calls[-1](); e1.record()
            torch.cuda.synchronize()
            t.append(e0.elapsed_time(e1))
        comb_ms = rank_max([float(np.median(t))], world)[0]
        comb_ms_last = -rank_max([-float(np.median(t))], world)[0]   # the rank that arrives last waits for nobody
        ex.check_status()
    kv_total = float(lens.sum()) * KV_BYTES_PER_TOKEN
    flops_total = 2 * float(4096 * 4097 // 2) * FLOPS_PER_PAIR
    d, pf, al = float(np.median(ms_dec)), float(np.median(ms_pre)), float(np.median(ms_all))
    load = [sum(e - a for _, a, e in b) for b in bins]
    return {"what": "64 decode sequences, histories log-uniform [512, 131072] (%.2f GB of KV), partitioned by KV bytes; "
                    "%d sequences of more than 32768 tokens cut into ranges on different GPUs and merged over NVLink peer "
                    "memory; plus 2 prefill chunks of 4096 tokens split by chunk and KV head" % (kv_total / 1e9, n_split if world > 1 else 0),
            "scaling": "strong", "n_gpus": world,
            "decode_part": {"value": round(kv_total / (d * 1e-3) / 1e9, 1), "unit": "GB/s", "ms_per_step": round(d, 5),
                            "ms_per_step_stats": stats(ms_dec), "hbm_frac_of_step": round(kv_total / (d * 1e-3) / 1e9 / (peaks[0] * world), 4),
                            "includes": "append, attention, partial exchange and combine (partials published first, merged last)"},
            "combine_ms": None if comb_ms is None else round(comb_ms, 5),
            "combine_ms_what": "max over ranks: a rank that reaches its combine early waits there for the slowest rank's flag",
            "combine_ms_of_the_last_rank": None if comb_ms is None else round(comb_ms_last, 5),
            "combine_share_of_decode_part": None if comb_ms is None else round(comb_ms / d, 4),
            "nvlink_bytes_read_per_rank_per_step": 0 if ex is None else n_split * 24 * 260 * 4 * (world - 1),
            "prefill_part": {"value": round(flops_total / (pf * 1e-3) / 1e12, 1), "unit": "TFLOP/s", "ms_per_step": round(pf, 5)},
            "whole_step_ms": round(al, 5), "whole_step_ms_stats": stats(ms_all),
            "partition_max_over_mean": round(max(load) / (sum(load) / world), 4)}


def measure_prefill32k_full(args, rank, world, peaks):
    """BASELINE configuration 4, strong-scaled: one 32768-token prompt in 16 chunks of 2048, append then attend.
    1 GPU: all four KV heads; 2 and 4 GPUs: KV-head shards (no exchange); 8 GPUs: one KV head per GPU pair and
    the pair splits every chunk's query rows zig-zag (rows [0, 512) and [1536, 2048) on one GPU -- one call of two
    "sequences" over the same cache rows -- and [512, 1536) on the other: equal causal work), both GPUs appending the
    whole chunk's K/V: no exchange either."""
    from qwengine_b200 import api
    T, CH = 32768, 2048
    kvh = {1: 4, 2: 2, 4: 1, 8: 1}[world]
    half = rank // 4 if world == 8 else -1
    g = torch.Generator(device="cuda").manual_seed(args.seed + 100 * rank + 51)
    rn = lambda *s: torch.randn(*s, device="cuda", dtype=torch.bfloat16, generator=g)
    kc, vc = torch.empty(T, kvh * 256, device="cuda", dtype=torch.bfloat16), torch.empty(T, kvh * 256, device="cuda", dtype=torch.bfloat16)
    q, gate = rn(T, 6 * kvh, 256), rn(T, 6 * kvh, 256)
    k, v = rn(T, kvh, 256), rn(T, kvh, 256)
    out = torch.empty_like(q)
    blocks = {-1: [(0, CH)], 0: [(0, 512), (1536, 512)], 1: [(512, 1024)]}[half]
    plan = []   # per chunk: optional append-only call, then attention calls
    for c0 in range(0, T, CH):
        calls = []
        if half >= 0:
            ma = api.Mixer(1, CH, kv_heads=kvh)
            ma.bind_append_only(kc, vc, torch.tensor([c0], dtype=torch.int32, device="cuda"), k[c0:c0 + CH].view(1, CH, kvh, 256),
                                v[c0:c0 + CH].view(1, CH, kvh, 256))
            calls.append(ma)
        if half == 0:
            # This GPU's two row blocks go out as ONE call of two "sequences" that share the cache rows and differ in
            # position: a launch of one 512-row block is 12 items for 74 CTA pairs, and two launches one after the
            # other took twice as long as the 4-GPU plan's whole chunk.  The rank holds just its own rows, packed.
            mx = api.Mixer(2, 512, kv_heads=kvh)
            sl = slice(c0, c0 + 1024)   # (synthetic data: any 1024 rows of the rank's tensors stand for its two blocks)
            mx.bind(q[sl].view(2, 512, 6 * kvh, 256), kc, vc,
                    torch.tensor([c0, c0 + 1536], dtype=torch.int32, device="cuda"), out[sl].view(2, 512, 6 * kvh, 256),
                    gate=gate[sl].view(2, 512, 6 * kvh, 256), cache_row=torch.zeros(2, dtype=torch.int64, device="cuda"),
                    flags=api.F_ROPE | api.F_GATE)
            calls.append(mx)
            plan.append(calls)
            continue
        for off, n in blocks:
            r0 = c0 + off
            mx = api.Mixer(1, n, kv_heads=kvh)
            sl = slice(r0, r0 + n)
            if half >= 0:
                mx.bind(q[sl].view(1, n, 6 * kvh, 256), kc, vc, torch.tensor([r0], dtype=torch.int32, device="cuda"),
                        out[sl].view(1, n, 6 * kvh, 256), gate=gate[sl].view(1, n, 6 * kvh, 256),
                        flags=api.F_ROPE | api.F_GATE)
            else:
                mx.bind(q[sl].view(1, n, 6 * kvh, 256), kc, vc, torch.tensor([r0], dtype=torch.int32, device="cuda"),
                        out[sl].view(1, n, 6 * kvh, 256), k_new=k[sl].view(1, n, kvh, 256), v_new=v[sl].view(1, n, kvh, 256),
                        gate=gate[sl].view(1, n, 6 * kvh, 256))
            calls.append(mx)
        plan.append(calls)
    n_launch = [0]
    for calls in plan:          # one untimed pass that also counts the kernels of a step
        for m in calls:
            m.forward()
            n_launch[0] += m.launches()

    def step():
        for calls in plan:
            for m in calls:
                m.forward()

    ms = timed(step, 3, 2, args.repeats, world)
    for calls in plan:
        for m in calls:
            m.check_status()
    flops_total = float(T * (T + 1) // 2) * FLOPS_PER_PAIR
    t = float(np.median(ms))
    return {"what": "one 32768-token prompt in 16 chunks of 2048 (append, then attend): %s" %
                    {1: "all four KV heads on one GPU", 2: "KV-head shards, 2 heads per GPU", 4: "KV-head shards, 1 head per GPU",
                     8: "1 KV head per GPU pair, the pair splits each chunk's query rows zig-zag, both append the chunk"}[world],
            "scaling": "strong", "n_gpus": world, "value": round(flops_total / (t * 1e-3) / 1e12, 1), "unit": "TFLOP/s",
            "ms_per_step": round(t, 4), "ms_per_step_stats": stats(ms), "gpu_launches_per_step": n_launch[0],
            "tensor_frac_of_step": round(flops_total / (t * 1e-3) / 1e12 / (peaks[1] * world), 4),
            "exchange": "none: outputs are disjoint head slices / row blocks"}


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


def guarded(fn, world, what):
    """Runs a sub-benchmark; a failure on any rank turns into an error entry on all of them instead of leaving
    the other ranks waiting in a collective."""
    err = None
    try:
        res = fn()
    except Exception as e:  # noqa: BLE001 -- the line must still be printed
        res, err = None, "%s: %s" % (type(e).__name__, str(e)[:300])
    bad = rank_max([1.0 if err else 0.0], world)[0] if torch.cuda.is_available() else (1.0 if err else 0.0)
    if bad:
        return {"error": err or "failed on another rank", "what": what}
    return res


def run_ours(args, rank, local_rank, world):
    from qwengine_b200 import api
    torch.cuda.set_device(local_rank)
    ex_cls = None
    if world > 1:
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")   # plain peer loads only: no multicast binding
        # a short collective timeout: ranks that stop agreeing on the next collective end with an error within
        # minutes instead of holding eight GPUs for the default ten
        torch.distributed.init_process_group("nccl", device_id=torch.device("cuda", local_rank),
                                             timeout=datetime.timedelta(seconds=180))
        from qwengine_b200 import sharding
        ex_cls = sharding.PeerExchange
    peaks = measured_peaks()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    line = None
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
                v = hbm_line("verify", rv, world, peaks)
                line["verify"] = {"value": v["value"], "unit": v["unit"], "ms_per_step": v["ms_per_step"],
                                  "ms_per_step_stats": v["ms_per_step_stats"], "workload": v["config"]["workload"],
                                  "roofline": v["roofline"]}
            if world == 1:
                d = guarded(lambda: measure_dropin(args, peaks), world, "dropin")
                b1 = guarded(lambda: measure_decode_b1(args, peaks), world, "decode_b1")
                line["dropin"], line["decode_b1"] = d, b1
            else:
                chk = guarded(lambda: multi_gpu_check(args, rank, world, ex_cls)[0], world, "multi_gpu_check")
                mixed = guarded(lambda: measure_mixed(args, rank, world, peaks, ex_cls), world, "mixed")
                full = guarded(lambda: measure_prefill32k_full(args, rank, world, peaks), world, "prefill32k_full")
                if rank == 0:
                    line["multi_gpu_check"], line["mixed"], line["prefill32k_full"] = chk, mixed, full
    elif args.workload == "mixed":
        res = guarded(lambda: measure_mixed(args, rank, world, peaks, ex_cls), world, "mixed")
        if rank == 0:
            ok = "decode_part" in res
            line = {"metric": "decode_attn_kv_GBps", "value": res["decode_part"]["value"] if ok else None, "unit": "GB/s",
                    "n_gpus": world, "steps": max(3, args.steps // 5), "warmup": 3, "ms_per_step": res["decode_part"]["ms_per_step"] if ok else None,
                    "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
                    "data": "synthetic: seeded N(0,1) bf16, no dataset", "config": {"workload": "mixed: " + res.get("what", "")},
                    "mixed": res}
    elif args.workload == "prefill32k_full":
        res = guarded(lambda: measure_prefill32k_full(args, rank, world, peaks), world, "prefill32k_full")
        if rank == 0:
            ok = "value" in res
            line = {"metric": "prefill_attn_TFLOPs", "value": res.get("value"), "unit": "TFLOP/s", "n_gpus": world, "steps": 3,
                    "warmup": 2, "ms_per_step": res.get("ms_per_step"), "higher_is_better": True, "scaling": "strong",
                    "vs_baseline": None, "dtype": "bf16", "data": "synthetic: seeded N(0,1) bf16, no dataset",
                    "config": {"workload": "prefill32k_full: " + res.get("what", "")}, "prefill32k_full": res}
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
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--repeats", type=int, default=5, help="timed regions of `steps` steps each; median / min / max are reported")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="decode", choices=sorted(WORKLOADS) + ["mixed", "prefill32k_full"])
    ap.add_argument("--seed", type=int, default=1234)
    ap.add_argument("--fast-p", action="store_true", help="prefill workloads: single-bf16 P operand")
    ap.add_argument("--no-prefill", action="store_true", help="decode workload: skip the sub-measurements")
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

"""The reference arm of bench.py: `python bench.py --impl reference ...`.

The reference engine has no CPU implementation of attention; its implementation of this path IS
five CUDA kernels.  When the test-only library built from the reference's own sources for sm_100a
(oracle/_ref/libref_attn.so) is present, this arm times those kernels, launched exactly as the
reference launches them (src/model.cu:228-240 for decode, src/prefill.cu:142-156 for prefill):
fp32 tensors, one sequence per launch sequence, the `rows x 24 x ctx` fp32 score scratch.  If
the library is absent it times the CPU oracle port instead.  Either way the line also carries the
oracle's CPU timing under "cpu_baseline".  Only rank 0 works; other ranks exit at once.
"""
import ctypes as C
import json
import os
import sys
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
REF_LIB = os.path.join(ROOT, "oracle", "_ref", "libref_attn.so")


def _load_ref():
    l = C.CDLL(REF_LIB)
    vp, i, f = C.c_void_p, C.c_int, C.c_float
    l.ref_rope.argtypes = [vp, i, i, i, vp, f, vp, i, vp]
    l.ref_kv_append.argtypes = [vp, vp, vp, vp, vp, i, i, vp]
    l.ref_attn_decode.argtypes = [vp, vp, vp, vp, vp, i, i, i, f, vp, i, i, vp]
    l.ref_attn_prefill.argtypes = [vp, vp, vp, vp, vp, i, i, i, f, vp, i, i, vp]
    l.ref_gate_sigmoid.argtypes = [vp, vp, i, vp]
    return l


def _reference_gpu(args, w):
    """Times the reference kernels on fp32 copies of workload w (built by bench.build_workload)."""
    l = _load_ref()
    p = lambda t: C.c_void_p(t.data_ptr())
    n_seq, n_new = w["n_seq"], w["n_new"]
    prefill = n_new >= 64
    seqs = []
    row0 = w["cache_row"].cpu().numpy()
    for s in range(n_seq):
        h = int(w["hist"][s])
        ctx = h + n_new
        kc = torch.zeros(ctx, 1024, device="cuda")
        vc = torch.zeros(ctx, 1024, device="cuda")
        kc[:h] = w["kc"][row0[s]:row0[s] + h].float()
        vc[:h] = w["vc"][row0[s]:row0[s] + h].float()
        seqs.append(dict(ctx=ctx, kc=kc, vc=vc, q0=w["q"][s].float(), k0=w["k_new"][s].float(), v=w["v_new"][s].float(),
                         gate=w["gate"][s].float(), out=torch.empty(n_new, 24, 256, device="cuda"),
                         dpos=torch.tensor([h], dtype=torch.int32, device="cuda")))
    max_ctx = max(s["ctx"] for s in seqs)
    scratch = torch.empty(n_new * 24 * max_ctx, dtype=torch.float32, device="cuda")
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)

    prefill_like = prefill
    steps = max(1, min(args.steps, 3 if prefill_like else 20))
    warm = max(1, min(args.warmup, 1 if prefill_like else 5))
    # rope works in place: every step needs its own un-rotated copy of q and k, made outside the timed region
    for s in seqs:
        s["qs"] = [s["q0"].clone() for _ in range(steps + warm)]
        s["ks"] = [s["k0"].clone() for _ in range(steps + warm)]

    def step(i):
        for s in seqs:
            q, k = s["qs"][i], s["ks"][i]
            l.ref_rope(p(q), 24, 256, 64, p(s["dpos"]), 1e7, st, n_new, None)
            l.ref_rope(p(k), 4, 256, 64, p(s["dpos"]), 1e7, st, n_new, None)
            l.ref_kv_append(p(k), p(s["v"]), p(s["kc"]), p(s["vc"]), p(s["dpos"]), 1024, n_new, st)
            if prefill:
                l.ref_attn_prefill(p(q), p(s["kc"]), p(s["vc"]), p(s["out"]), p(s["dpos"]), 256, 4, 24, 1.0 / 16.0,
                                   p(scratch), s["ctx"], n_new, st)
            else:
                l.ref_attn_decode(p(q), p(s["kc"]), p(s["vc"]), p(s["out"]), p(s["dpos"]), 256, 4, 24, 1.0 / 16.0,
                                  p(scratch), s["ctx"], n_new, st)
            l.ref_gate_sigmoid(p(s["out"]), p(s["gate"]), n_new * 6144, st)

    for i in range(warm):
        step(i)
    torch.cuda.synchronize()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    ev[0].record()
    for i in range(steps):
        step(warm + i)
    ev[1].record()
    torch.cuda.synchronize()
    return ev[0].elapsed_time(ev[1]) / steps, steps, warm


def run_reference(args, rank, local_rank, world):
    if rank != 0:
        return
    sys.path.insert(0, ROOT)
    import bench
    name = args.workload
    have_gpu = torch.cuda.is_available()
    if not have_gpu:
        print(json.dumps({"impl": "reference", "unavailable": "no CUDA device: the reference's implementation of this path is CUDA kernels"}))
        return
    torch.cuda.set_device(local_rank)
    w = bench.build_workload(name, 1, 0, args.seed)
    is_hbm = name in ("decode", "verify")
    cpu = bench.cpu_baseline(w) if is_hbm else None
    if os.path.exists(REF_LIB):
        ms, steps, warm = _reference_gpu(args, w)
        kind = "reference"
        how = "the reference's own CUDA kernels (k_rope, k_kv_append, k_attn_%s, k_gate_sigmoid) rebuilt for sm_100a, fp32, one sequence per launch" % ("prefill" if not is_hbm else "decode")
        cores = 0
    else:
        # no reference build on this box: the CPU oracle port stands in
        t0 = time.perf_counter()
        cpu = bench.cpu_baseline(w, min_seconds=5.0)
        ms = None
        kind, how, cores = "port", "CPU oracle port (reference library not built on this box)", cpu["cores"]
        steps, warm = 1, 0
    if is_hbm:
        value = (w["kv_bytes"] / (ms * 1e-3) / 1e9) if ms else cpu["value"]
        metric, unit = "decode_attn_kv_GBps", "GB/s"
    else:
        value = w["flops"] / (ms * 1e-3) / 1e12 if ms else None
        metric, unit = "prefill_attn_TFLOPs", "TFLOP/s"
    line = {
        "impl": "reference", "metric": metric, "value": round(value, 4) if value else None, "unit": unit, "n_gpus": int(getattr(args, "gpus", 1) or 1), "ranks_used": 1,
        "steps": steps, "warmup": warm, "ms_per_step": round(ms, 5) if ms else None, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32" if kind == "reference" else "f64",
        "data": "synthetic: the same seeded tensors as the B200 arm, widened to fp32",
        "config": {"workload": bench.describe(name, 1, w), "how": how,
                   "ranks": "rank 0 alone runs one GPU's share of the weak-scaled batch: the reference serves one sequence on one GPU (README.md:365-367), so its rate does not grow with N",
                   "note": "algorithmic unit is the same as the B200 arm's (4096 B of bf16 K+V per cached token, "
                           "24576 FLOP per pair); the reference itself moves fp32"},
        "cpu_baseline": dict(cpu, kind="port") if cpu else {"kind": kind, "cores": cores, "sample": how, "value": round(value, 4) if value else None, "unit": unit},
        "reference_kind": kind,
        "e2e": {"value": round(value, 4) if value else None, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))

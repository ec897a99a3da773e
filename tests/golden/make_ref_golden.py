"""Generates tests/golden/ref_*.npz by RUNNING THE REFERENCE ENGINE'S OWN KERNELS (k_rope,
k_kv_append, k_attn_decode / k_attn_prefill, k_gate_sigmoid, launched in the order of
src/model.cu:228-240 and src/prefill.cu:142-156) on seeded inputs.  The kernels come from
oracle/_ref/libref_attn.so, which oracle/Makefile compiles for sm_100a from the reference
sources where they lie.  Needs a CUDA device:
    python tests/golden/make_ref_golden.py [output_dir]
Inputs are bf16-exact N(0,1) values stored as bf16 bit patterns; everything the kernels see
and produce is fp32, as in the reference.
"""
import ctypes as C
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
from oracle import pyoracle as O  # noqa: E402  (bf16 bit helpers only)

REF_LIB = os.path.join(ROOT, "oracle", "_ref", "libref_attn.so")


def load_ref():
    l = C.CDLL(REF_LIB)
    vp, i, f = C.c_void_p, C.c_int, C.c_float
    l.ref_rope.argtypes = [vp, i, i, i, vp, f, vp, i, vp]
    l.ref_kv_append.argtypes = [vp, vp, vp, vp, vp, i, i, vp]
    l.ref_attn_decode.argtypes = [vp, vp, vp, vp, vp, i, i, i, f, vp, i, i, vp]
    l.ref_attn_prefill.argtypes = [vp, vp, vp, vp, vp, i, i, i, f, vp, i, i, vp]
    l.ref_gate_sigmoid.argtypes = [vp, vp, i, vp]
    return l


def run_reference_layer(l, q, k, v, gate, kc, vc, pos0, kv_heads, ctx, prefill, mpos=None):
    """q [B, Hq, 256], k/v [B, Hkv, 256], gate like q, kc/vc [ctx, Hkv*256]: fp32 CUDA tensors.
    Runs the reference launch sequence in place; returns the gated output [B, Hq, 256]."""
    B, Hq = q.shape[0], q.shape[1]
    p = lambda t: C.c_void_p(t.data_ptr()) if t is not None else None
    dpos = torch.tensor([pos0], dtype=torch.int32, device="cuda")
    out = torch.empty_like(q)
    scratch = torch.zeros(B * Hq * ctx, dtype=torch.float32, device="cuda")
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = l.ref_rope(p(q), Hq, 256, 64, p(dpos), 1e7, st, B, p(mpos))
    rc |= l.ref_rope(p(k), kv_heads, 256, 64, p(dpos), 1e7, st, B, p(mpos))
    rc |= l.ref_kv_append(p(k), p(v), p(kc), p(vc), p(dpos), kv_heads * 256, B, st)
    if prefill:
        rc |= l.ref_attn_prefill(p(q), p(kc), p(vc), p(out), p(dpos), 256, kv_heads, Hq, 1.0 / 16.0, p(scratch),
                                 ctx, B, st)
    else:
        rc |= l.ref_attn_decode(p(q), p(kc), p(vc), p(out), p(dpos), 256, kv_heads, Hq, 1.0 / 16.0, p(scratch),
                                ctx, B, st)
    rc |= l.ref_gate_sigmoid(p(out), p(gate), out.numel(), st)
    torch.cuda.synchronize()
    assert rc == 0, "a reference launch failed: %d" % rc
    return out


def case(l, outdir, name, seed, kv_heads, hist, B, prefill, mrope=False):
    rng = np.random.default_rng(seed)
    bf = lambda shape: O.bf16_bits_to_f32(O.f32_to_bf16_bits(rng.standard_normal(shape, dtype=np.float32)))
    Hq, ctx = 6 * kv_heads, hist + B
    q, k, v, gate = bf((B, Hq, 256)), bf((B, kv_heads, 256)), bf((B, kv_heads, 256)), bf((B, Hq, 256))
    kc0, vc0 = bf((hist, kv_heads * 256)), bf((hist, kv_heads * 256))
    mpos = None
    if mrope:
        t = hist + np.arange(B)
        mpos = np.stack([t, t // 3 + 5, (t * 7) % 11], -1).astype(np.int32)
    dev = lambda a: torch.from_numpy(a.copy()).cuda()
    kc = torch.zeros(ctx, kv_heads * 256, device="cuda")
    vc = torch.zeros(ctx, kv_heads * 256, device="cuda")
    kc[:hist], vc[:hist] = dev(kc0), dev(vc0)
    dq, dk = dev(q), dev(k)
    out = run_reference_layer(l, dq, dk, dev(v), dev(gate), kc, vc, hist, kv_heads, ctx, prefill,
                              None if mpos is None else dev(mpos))
    np.savez(os.path.join(outdir, name + ".npz"), kv_heads=kv_heads, hist=hist, n_new=B, prefill=int(prefill),
             q=O.f32_to_bf16_bits(q), k=O.f32_to_bf16_bits(k), v=O.f32_to_bf16_bits(v),
             gate=O.f32_to_bf16_bits(gate), kc0=O.f32_to_bf16_bits(kc0), vc0=O.f32_to_bf16_bits(vc0),
             mpos=mpos if mpos is not None else np.zeros((0, 3), np.int32),
             q_rot=dq.cpu().numpy(), k_rows=kc[hist:].cpu().numpy(), v_rows=vc[hist:].cpu().numpy(),
             out=out.cpu().numpy())


if __name__ == "__main__":
    outdir = sys.argv[1] if len(sys.argv) > 1 else HERE
    os.makedirs(outdir, exist_ok=True)
    lib = load_ref()
    case(lib, outdir, "ref_decode", 21, 1, 40, 1, False)
    case(lib, outdir, "ref_verify", 22, 1, 33, 4, False)
    case(lib, outdir, "ref_prefill_scratch", 23, 1, 0, 20, True)
    case(lib, outdir, "ref_prefill_hist", 24, 1, 13, 11, True)
    case(lib, outdir, "ref_mrope_prefill", 25, 1, 6, 9, True, mrope=True)
    case(lib, outdir, "ref_decode_4kv", 26, 4, 70, 2, False)
    print("wrote", sorted(f for f in os.listdir(outdir) if f.startswith("ref_")))

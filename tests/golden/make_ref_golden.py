"""Generates tests/golden/ref_*.npz by RUNNING THE REFERENCE ENGINE'S OWN KERNELS (k_rope,
k_kv_append, k_attn_decode / k_attn_prefill, k_gate_sigmoid, launched in the order of
src/model.cu:228-240 and src/prefill.cu:142-156; for the ref_fused_* cases also k_unpack3,
k_split_qgate and k_rmsnorm_head in front of them, src/model.cu:219-226) on seeded inputs.  The kernels come from
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
    l.ref_unpack3.argtypes = [vp, vp, vp, vp, i, i, i, i, vp]
    l.ref_split_qgate.argtypes = [vp, vp, vp, i, i, vp]
    l.ref_rmsnorm_head.argtypes = [vp, vp, i, i, f, vp]
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


def fused_case(l, outdir, name, seed, kv_heads, hist, B, prefill, eps=1e-6):
    """The steps in front of the mixer as well, in the order of src/model.cu:219-240: the fused
    projection row [ (q|gate) x heads | k | v ] goes through unpack3, k_split_qgate and the two
    k_rmsnorm_head launches, then through the launch sequence of run_reference_layer."""
    rng = np.random.default_rng(seed)
    bf = lambda shape: O.bf16_bits_to_f32(O.f32_to_bf16_bits(rng.standard_normal(shape, dtype=np.float32)))
    Hq, ctx, kvd = 6 * kv_heads, hist + B, kv_heads * 256
    fused = (1.5 * rng.standard_normal((B, Hq * 512 + 2 * kvd))).astype(np.float32)  # raw GEMM output: plain fp32
    qw = O.f32_to_bf16_bits((0.2 * rng.standard_normal(256)).astype(np.float32))
    kw = O.f32_to_bf16_bits((0.2 * rng.standard_normal(256)).astype(np.float32))
    kc0, vc0 = bf((hist, kvd)), bf((hist, kvd))
    dev = lambda a: torch.from_numpy(a.copy()).cuda()
    p = lambda t: C.c_void_p(t.data_ptr())
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    dfused, dqw, dkw = dev(fused), dev(qw.view(np.int16)), dev(kw.view(np.int16))
    qproj = torch.empty(B, Hq * 512, device="cuda")
    q = torch.empty(B, Hq, 256, device="cuda")
    gate = torch.empty(B, Hq, 256, device="cuda")
    k = torch.empty(B, kv_heads, 256, device="cuda")
    v = torch.empty(B, kv_heads, 256, device="cuda")
    rc = l.ref_unpack3(p(dfused), p(qproj), p(k), p(v), Hq * 512, kvd, kvd, B, st)
    rc |= l.ref_split_qgate(p(qproj), p(q), p(gate), B * Hq, 256, st)
    rc |= l.ref_rmsnorm_head(p(q), p(dqw), B * Hq, 256, eps, st)
    rc |= l.ref_rmsnorm_head(p(k), p(dkw), B * kv_heads, 256, eps, st)
    torch.cuda.synchronize()
    assert rc == 0
    q_norm, k_norm = q.cpu().numpy().copy(), k.cpu().numpy().copy()
    kc = torch.zeros(ctx, kvd, device="cuda")
    vc = torch.zeros(ctx, kvd, device="cuda")
    kc[:hist], vc[:hist] = dev(kc0), dev(vc0)
    out = run_reference_layer(l, q, k, v, gate, kc, vc, hist, kv_heads, ctx, prefill)
    np.savez(os.path.join(outdir, name + ".npz"), kv_heads=kv_heads, hist=hist, n_new=B, prefill=int(prefill), eps=eps,
             fused=fused, q_norm_w=qw, k_norm_w=kw, kc0=O.f32_to_bf16_bits(kc0), vc0=O.f32_to_bf16_bits(vc0),
             q_norm=q_norm, k_norm=k_norm, gate=gate.cpu().numpy(), k_rows=kc[hist:].cpu().numpy(),
             v_rows=vc[hist:].cpu().numpy(), out=out.cpu().numpy())


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
    fused_case(lib, outdir, "ref_fused_decode", 31, 4, 37, 1, False)
    fused_case(lib, outdir, "ref_fused_verify", 32, 1, 50, 4, False)
    fused_case(lib, outdir, "ref_fused_prefill", 33, 1, 9, 14, True)
    print("wrote", sorted(f for f in os.listdir(outdir) if f.startswith("ref_")))

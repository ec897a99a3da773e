"""Parity at the benchmark's FULL sizes, where the oracle cannot be run over everything in seconds: properties
that do not depend on size (a batch equals its sequences run alone, verify rows equal sequential decode steps,
chunked prefill equals one shot, repeated runs are bit-identical) plus the oracle on a sample of rows."""
import numpy as np
import pytest
import torch

from oracle import pyoracle as O
from qwengine_b200 import api
from tests.gpu_util import dev_bf16, dev_bits, host_bits, host_f32, run_case
from tests.util import Case, check_lse, check_out, rel_l2

pytestmark = pytest.mark.gpu


def _sample_rows_vs_oracle(c, out, lse, rows, what):
    ref, lse_ref, _, _ = c.oracle(rows=rows)
    check_out(out[rows], ref, what)
    check_lse(lse[rows], lse_ref, what)


def _alone(c, s):
    """Sequence s of Case c as a batch of one (same tensors, own cache pool)."""
    d = Case.__new__(Case)
    d.n_seq, d.n_new, d.kv_heads, d.q_heads = 1, c.n_new, c.kv_heads, c.q_heads
    d.hist = c.hist[s:s + 1].copy()
    d.cache_row = np.zeros(1, np.int64)
    r0 = int(c.cache_row[s])
    r1 = int(c.cache_row[s + 1]) if s + 1 < c.n_seq else c.rows_total
    d.rows_total = r1 - r0
    d.q, d.k, d.v, d.gate = c.q[s:s + 1], c.k[s:s + 1], c.v[s:s + 1], c.gate[s:s + 1]
    d.kc0, d.vc0 = c.kc0[r0:r1], c.vc0[r0:r1]
    d.mpos = None
    return d


def test_decode_configuration_full_size():
    """16 sequences x 1 token against 8192 cached tokens (the bench's headline workload)."""
    c = Case(301, [8192] * 16, 1)
    out, lse, kc, vc, mx = run_case(c, out_f32=True)
    out2, lse2, _, _, _ = run_case(c, out_f32=True)
    assert np.array_equal(out, out2) and np.array_equal(lse, lse2), "not bit-repeatable"
    for s in (0, 7, 15):  # a batch is its sequences run alone (other partition, other merge order: not bit-equal)
        o1, l1, _, _, _ = run_case(_alone(c, s), out_f32=True)
        assert np.abs(o1[0] - out[s]).max() <= 1e-5 and np.abs(l1[0] - lse[s]).max() <= 1e-5
    _sample_rows_vs_oracle(c, out, lse, [0, 5, 15], "decode full size")
    _, _, kc_ref, vc_ref = c.oracle(rows=[0])  # appends every new row before it evaluates the one asked for
    assert np.array_equal(kc, kc_ref) and np.array_equal(vc, vc_ref)


def test_verify_configuration_full_size_rows_equal_sequential_decode():
    """8 sequences x 4 draft tokens, ragged histories up to 32K: row b of a verify batch is what a decode step at
    position pos + b gives once rows 0..b are in the cache (test/test_spec.cu:64-98, at the bench's size)."""
    hist = np.random.default_rng(302).integers(2048, 32769 - 4, 8).tolist()
    c = Case(302, hist, 4)
    out, lse, kc, vc, _ = run_case(c, out_f32=True)
    out = out.reshape(8, 4, 24, 256)
    lse = lse.reshape(8, 4, 24)
    # sequential decode over the cache the verify call left behind (rows pos .. pos+3 appended): no append
    mx = api.Mixer(8, 1)
    kcd, vcd = dev_bits(kc), dev_bits(vc)
    crow = torch.from_numpy(c.cache_row).cuda()
    for b in range(4):
        o = torch.empty(8, 1, 24, 256, dtype=torch.float32, device="cuda")
        l = torch.empty(8, 1, 24, dtype=torch.float32, device="cuda")
        pos = torch.from_numpy(c.hist + b).cuda()
        # q rotated at position pos + b inside the call; the key rows are already in the cache, so no append
        mx.bind(dev_bf16(c.q[:, b:b + 1]), kcd, vcd, pos, o, gate=dev_bf16(c.gate[:, b:b + 1]), lse=l, cache_row=crow,
                flags=api.F_ROPE | api.F_GATE)
        # a decode row at position p sees keys [0, p]: without the append flag the call reads pos[s] + n_new rows
        mx.forward()
        torch.cuda.synchronize()
        mx.check_status()
        got = host_f32(o).reshape(8, 24, 256)
        assert np.abs(got - out[:, b]).max() <= 2e-5, "verify row %d differs from the decode step" % b
        assert np.abs(l.cpu().numpy().reshape(8, 24) - lse[:, b]).max() <= 2e-5
    flat = out.reshape(32, 24, 256)
    _sample_rows_vs_oracle(c, flat, lse.reshape(32, 24), [int(np.argmin(hist)) * 4 + 3], "verify full size")


def test_prefill_8k_chunked_equals_single_shot_and_samples_match_oracle():
    """8192-token causal prefill (the bench's prefill workload, one KV head's share): four chunks of 2048 appended to
    the cache give the bits of one shot; a sample of rows is checked against the oracle."""
    c = Case(303, [0], 8192, kv_heads=1)
    out, lse, kc, vc, _ = run_case(c, out_f32=True)
    mx = api.Mixer(1, 2048, kv_heads=1)
    kcd, vcd = dev_bits(c.kc0), dev_bits(c.vc0)
    pos = torch.zeros(1, dtype=torch.int32, device="cuda")
    outs = []
    for t0 in range(0, 8192, 2048):
        sl = slice(t0, t0 + 2048)
        o = torch.empty(1, 2048, 6, 256, dtype=torch.float32, device="cuda")
        pos.fill_(t0)
        mx.bind(dev_bf16(c.q[:, sl]), kcd, vcd, pos, o, k_new=dev_bf16(c.k[:, sl]), v_new=dev_bf16(c.v[:, sl]),
                gate=dev_bf16(c.gate[:, sl]))
        mx.forward()
        torch.cuda.synchronize()
        mx.check_status()
        outs.append(host_f32(o).reshape(2048, 6, 256))
    assert np.array_equal(host_bits(kcd), kc) and np.array_equal(host_bits(vcd), vc)
    assert np.array_equal(np.concatenate(outs), out), "chunked prefill differs from the single shot"
    _sample_rows_vs_oracle(c, out, lse, [0, 127, 128, 4095, 8191], "prefill 8K")


def test_maximum_context_decode():
    """One sequence at the model's native maximum position (262144, qwen38.h:30; the engine itself caps a
    context at 32768, qwen38.h:31): the last decode step, one KV head's share."""
    n = 262143
    c = Case(304, [n], 1, kv_heads=1)
    out, lse, kc, vc, _ = run_case(c, out_f32=True)
    ref, lse_ref, kc_ref, _ = c.oracle()
    assert np.array_equal(kc[n], kc_ref[n])
    check_out(out, ref, "max context")
    check_lse(lse, lse_ref, "max context")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_dropin_prefill_last_chunk_of_a_32k_prompt(dtype):
    """The reference's own prefill launch site (src/prefill.cu:142-154) at its hardest shape: a 2048-token chunk
    behind 30720 cached tokens, all four KV heads, through qw_rope / qw_kv_append / qw_attn_prefill.  It must run
    on the tcgen05 kernel, agree with the oracle on sampled rows, and agree with the fused call on everything."""
    T, pos0, ctx = 2048, 30720, 32768
    c = Case(310, [pos0], T)
    q = torch.from_numpy(c.q[0]).cuda().to(dtype)
    k = torch.from_numpy(c.k[0]).cuda().to(dtype)
    v = torch.from_numpy(c.v[0]).cuda().to(dtype)
    kc, vc = dev_bits(c.kc0), dev_bits(c.vc0)
    dpos = torch.tensor([pos0], dtype=torch.int32, device="cuda")
    out = torch.full_like(q, float("nan"))
    scratch = torch.empty(api.attn_prefill_scratch_floats(24, 4, ctx, T), dtype=torch.float32, device="cuda")
    api.rope(q, 24, 256, 64, dpos, 1e7, B=T)
    api.rope(k, 4, 256, 64, dpos, 1e7, B=T)
    api.kv_append(k, v, kc, vc, dpos, 1024, B=T)
    api.attn_prefill(q, kc, vc, out, dpos, 256, 4, 24, 1.0 / 16.0, scratch, ctx, T)
    torch.cuda.synchronize()
    assert api.last_attention_kernel() == "prefill_umma_pair_kernel"
    got = host_f32(out)
    assert np.isfinite(got).all()
    rows = [0, 127, 128, 1000, 2047]
    ref, _, kc_ref, vc_ref = c.oracle(rows=rows, do_gate=False)
    assert np.array_equal(host_bits(kc), kc_ref) and np.array_equal(host_bits(vc), vc_ref)
    # attention alone, on the q the tensor cores read
    q_seen = host_f32(q.to(torch.bfloat16))[None]
    ref_attn, _ = O.mixer(q_seen, None, None, None, kc_ref.copy(), vc_ref.copy(), [pos0], rows=rows, do_rope=False,
                          do_append=False, do_gate=False)
    assert np.abs(got[rows] - ref_attn).max() <= 2e-2 and rel_l2(got[rows], ref_attn) <= (1e-3 if dtype == torch.float32 else 2e-3)
    assert np.abs(got[rows] - ref).max() <= 2e-2 and rel_l2(got[rows], ref) <= (2e-3 if dtype == torch.float32 else 4e-3)
    # the fused call (q rotated inside, in fp32) on the same inputs, gate off
    import copy
    cg = copy.copy(c)
    cg.gate = None
    fused, _, _, _, _ = run_case(cg, out_f32=True)
    assert np.abs(got - fused).max() <= 2e-2 and rel_l2(got, fused) <= (2e-3 if dtype == torch.float32 else 4e-3)

"""The two multi-GPU configurations of the benchmark plan at their full sizes, on one GPU: the 32768-token
prefill in 2048-token chunks (one KV head's share, as a rank of the 4-GPU head sharding sees it) and the mixed
serving step (64 decode sequences with log-uniform histories up to 131072 partitioned into eight shares by KV
bytes, long sequences cut into KV ranges whose partials are merged, plus two 4096-token prefill chunks).  The
eight shares run one after the other here; tests/test_gpu_multi.py runs the exchange between real processes."""
import numpy as np
import pytest
import torch

from oracle import pyoracle as O
from qwengine_b200 import api, sharding
from tests.gpu_util import dev_bf16, dev_bits, host_bits, host_f32
from tests.util import Case, check_lse, check_out, rel_l2

pytestmark = pytest.mark.gpu


def test_long_context_prefill_32k_in_2048_token_chunks():
    T, CH = 32768, 2048
    c = Case(501, [0], T, kv_heads=1)
    mx = api.Mixer(1, CH, kv_heads=1)
    kc, vc = dev_bits(c.kc0), dev_bits(c.vc0)
    pos = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = torch.empty(T, 6, 256, dtype=torch.float32, device="cuda")
    lse = torch.empty(T, 6, dtype=torch.float32, device="cuda")
    for t0 in range(0, T, CH):
        sl = slice(t0, t0 + CH)
        pos.fill_(t0)
        mx.bind(dev_bf16(c.q[:, sl]), kc, vc, pos, out[sl].view(1, CH, 6, 256), k_new=dev_bf16(c.k[:, sl]),
                v_new=dev_bf16(c.v[:, sl]), gate=dev_bf16(c.gate[:, sl]), lse=lse[sl].view(1, CH, 6))
        mx.forward()
    torch.cuda.synchronize()
    mx.check_status()
    rows = [0, 2047, 2048, 16383, 30000, 32767]
    ref, lse_ref, kc_ref, vc_ref = c.oracle(rows=rows)
    assert np.array_equal(host_bits(kc), kc_ref) and np.array_equal(host_bits(vc), vc_ref)
    check_out(host_f32(out[rows]), ref, "32K chunked prefill")
    check_lse(lse[rows].cpu().numpy(), lse_ref, "32K chunked prefill")
    # one 32768-token call gives the same bits: a row's tiles are visited in the same order either way
    one = torch.empty(1, T, 6, 256, dtype=torch.float32, device="cuda")
    kc1, vc1 = dev_bits(c.kc0), dev_bits(c.vc0)
    m1 = api.Mixer(1, T, kv_heads=1)
    pos.fill_(0)
    m1.bind(dev_bf16(c.q), kc1, vc1, pos, one, k_new=dev_bf16(c.k), v_new=dev_bf16(c.v), gate=dev_bf16(c.gate))
    m1.forward()
    torch.cuda.synchronize()
    m1.check_status()
    assert torch.equal(one.view(T, 6, 256), out)


def test_mixed_serving_step_partitioned_by_kv_bytes():
    rng = np.random.default_rng(502)
    n_seq = 64
    hist = np.exp(rng.uniform(np.log(512), np.log(131072), n_seq)).astype(np.int64)
    cap = hist + 1
    crow = np.concatenate([[0], np.cumsum(cap)[:-1]])
    rows_total = int(cap.sum())
    g = torch.Generator(device="cuda").manual_seed(502)
    bf = lambda *shape: torch.randn(*shape, device="cuda", generator=g).to(torch.bfloat16)
    kc, vc = bf(rows_total, 1024), bf(rows_total, 1024)
    q, k, v, gate = bf(n_seq, 1, 24, 256), bf(n_seq, 1, 4, 256), bf(n_seq, 1, 4, 256), bf(n_seq, 1, 24, 256)
    kc_before = {}
    out = torch.full((n_seq, 24, 256), float("nan"), dtype=torch.float32, device="cuda")
    lse = torch.full((n_seq, 24), float("nan"), dtype=torch.float32, device="cuda")

    bins = sharding.partition_by_kv_bytes(cap, 8, max_share=32768)
    pieces_of = {}
    for b in bins:
        for s, a, e in b:
            pieces_of.setdefault(s, []).append((a, e))
    split = sorted(s for s, p in pieces_of.items() if len(p) > 1)
    assert split, "the plan should cut the longest sequences"
    sample = [int(np.argmin(hist)), int(np.argsort(hist)[n_seq // 2]), split[0], split[-1]]
    for s in sample:  # the oracle's inputs: this sequence's history before the step
        r0 = int(crow[s])
        kc_before[s] = (host_bits(kc[r0:r0 + int(cap[s])]), host_bits(vc[r0:r0 + int(cap[s])]))

    # split sequences: one partial per KV range.  The range that holds the new row appends it (rope(k) from the
    # absolute position in q_pos); every range rotates q itself from q_pos, in fp32 like an unsplit call.
    parts = {s: [] for s in split}
    for b in bins:  # one share after the other
        whole = [s for s, a, e in b if (a, e) == (0, int(cap[s]))]
        if whole:
            idx = torch.tensor(whole, device="cuda")
            mx = api.Mixer(len(whole), 1)
            o = torch.empty(len(whole), 1, 24, 256, dtype=torch.float32, device="cuda")
            l = torch.empty(len(whole), 1, 24, dtype=torch.float32, device="cuda")
            mx.bind(q[idx].contiguous(), kc, vc, torch.from_numpy(hist[whole].astype(np.int32)).cuda(), o,
                    k_new=k[idx].contiguous(), v_new=v[idx].contiguous(), gate=gate[idx].contiguous(), lse=l,
                    cache_row=torch.from_numpy(crow[whole]).cuda())
            mx.forward()
            torch.cuda.synchronize()
            mx.check_status()
            out[idx], lse[idx] = o[:, 0], l[:, 0]
        for s, a, e in b:
            if s not in parts:
                continue
            L = int(cap[s])
            mx = api.Mixer(1, 1)
            part = torch.zeros(1, 24, api.PARTIAL_FLOATS, dtype=torch.float32, device="cuda")
            scratch_out = torch.empty(1, 1, 24, 256, dtype=torch.bfloat16, device="cuda")
            cr = torch.tensor([int(crow[s]) + a], dtype=torch.int64, device="cuda")
            qp = torch.tensor([int(hist[s])], dtype=torch.int32, device="cuda")
            if e == L:   # the tail range holds the new row: it appends it and attends causally
                mx.bind(q[s:s + 1], kc, vc, torch.tensor([e - a - 1], dtype=torch.int32, device="cuda"), scratch_out,
                        k_new=k[s:s + 1], v_new=v[s:s + 1], cache_row=cr, flags=api.F_ROPE | api.F_APPEND, q_pos=qp)
            else:
                mx.bind(q[s:s + 1], kc, vc, torch.tensor([e - a], dtype=torch.int32, device="cuda"), scratch_out,
                        cache_row=cr, flags=api.F_ROPE | api.F_NO_CAUSAL, q_pos=qp)
            mx.forward_partial(part)
            torch.cuda.synchronize()
            mx.check_status()
            parts[s].append((a, part))
    for s in split:  # merged in range order, the order a rank-ordered exchange gives
        ps = torch.stack([p for _, p in sorted(parts[s], key=lambda t: t[0])])
        assert ps.shape[0] == len(pieces_of[s])
        o = torch.empty(1, 24, 256, dtype=torch.float32, device="cuda")
        l = torch.empty(1, 24, dtype=torch.float32, device="cuda")
        api.combine_partials(ps, ps.shape[0], 1, 24, o, gate=gate[s, 0:1].contiguous().view(1, 24, 256), lse=l)
        torch.cuda.synchronize()
        out[s], lse[s] = o[0], l[0]
    assert bool(torch.isfinite(out).all()) and bool(torch.isfinite(lse).all())

    f32 = lambda t: t.float().cpu().numpy()
    for s in sample:
        kc_h, vc_h = kc_before[s][0].copy(), kc_before[s][1].copy()
        ref, lse_ref = O.mixer(f32(q[s:s + 1]), f32(k[s:s + 1]), f32(v[s:s + 1]), f32(gate[s:s + 1]), kc_h, vc_h,
                               [int(hist[s])])
        got = host_f32(out[s:s + 1])
        # split or not, the same bounds: max-abs 2e-2, rel-L2 1e-3, LSE 1e-3
        check_out(got, ref, "mixed step, sequence %d" % s)
        check_lse(lse[s:s + 1].cpu().numpy(), lse_ref, "mixed step, sequence %d" % s)
        r0 = int(crow[s]) + int(hist[s])
        assert np.array_equal(host_bits(kc[r0:r0 + 1]), kc_h[int(hist[s]):int(hist[s]) + 1]), "appended K row"

    # the two prefill chunks of the step (4096 tokens each, from scratch), all four KV heads
    c = Case(503, [0, 0], 4096)
    mx = api.Mixer(2, 4096)
    kcp, vcp = dev_bits(c.kc0), dev_bits(c.vc0)
    o = torch.empty(2, 4096, 24, 256, dtype=torch.float32, device="cuda")
    l = torch.empty(2, 4096, 24, dtype=torch.float32, device="cuda")
    mx.bind(dev_bf16(c.q), kcp, vcp, torch.zeros(2, dtype=torch.int32, device="cuda"), o, k_new=dev_bf16(c.k),
            v_new=dev_bf16(c.v), gate=dev_bf16(c.gate), lse=l, cache_row=torch.from_numpy(c.cache_row).cuda())
    mx.forward()
    torch.cuda.synchronize()
    mx.check_status()
    rows = [0, 4095, 4096, 4096 + 2500, 8191]
    ref, lse_ref, kc_ref, _ = c.oracle(rows=rows)
    assert np.array_equal(host_bits(kcp), kc_ref)
    check_out(host_f32(o).reshape(-1, 24, 256)[rows], ref, "prefill chunks of the mixed step")
    check_lse(l.cpu().numpy().reshape(-1, 24)[rows], lse_ref, "prefill chunks of the mixed step")


@pytest.mark.parametrize("hist,CH", [(0, 256), (700, 512)])
def test_query_rows_of_a_chunk_split_zigzag_between_two_shares(hist, CH):
    """The 8-GPU plan of the long prefill: two GPUs share a KV head, both append the whole chunk (rope(k) + store,
    no attention) and each attends for its query-row blocks only -- rows [0, CH/4) and [3CH/4, CH) on one,
    [CH/4, 3CH/4) on the other -- with the position set to the block's first row and nothing appended.  Run here one
    share after the other on one GPU; every row must match the oracle, the cache must be the chunk call's cache."""
    c = Case(520 + CH, [hist], CH, kv_heads=1)
    ref, lse_ref, kc_ref, vc_ref = c.oracle()
    q, gate = dev_bf16(c.q), dev_bf16(c.gate)
    out = torch.zeros(1, CH, 6, 256, dtype=torch.float32, device="cuda")
    lse = torch.zeros(1, CH, 6, dtype=torch.float32, device="cuda")
    for blocks in ([(0, CH // 4), (3 * CH // 4, CH // 4)], [(CH // 4, CH // 2)]):
        kc, vc = dev_bits(c.kc0), dev_bits(c.vc0)   # each share holds its own copy of the cache
        ma = api.Mixer(1, CH, kv_heads=1)
        ma.bind_append_only(kc, vc, torch.tensor([hist], dtype=torch.int32, device="cuda"), dev_bf16(c.k), dev_bf16(c.v))
        ma.forward()
        if len(blocks) == 2:
            # the share with two row blocks sends them as ONE call of two "sequences" over the same cache rows
            n = blocks[0][1]
            pack = lambda x: torch.stack([x[0, off:off + n] for off, _ in blocks]).contiguous()
            o2 = torch.zeros(2, n, 6, 256, dtype=torch.float32, device="cuda")
            l2 = torch.zeros(2, n, 6, dtype=torch.float32, device="cuda")
            mx = api.Mixer(2, n, kv_heads=1)
            mx.bind(pack(q), kc, vc, torch.tensor([hist + off for off, _ in blocks], dtype=torch.int32, device="cuda"), o2,
                    gate=pack(gate), lse=l2, cache_row=torch.zeros(2, dtype=torch.int64, device="cuda"),
                    flags=api.F_ROPE | api.F_GATE)
            mx.forward()
            torch.cuda.synchronize()
            mx.check_status()
            for i, (off, _) in enumerate(blocks):
                out[0, off:off + n] = o2[i]
                lse[0, off:off + n] = l2[i]
            blocks = []
        for off, n in blocks:
            mx = api.Mixer(1, n, kv_heads=1)
            sl = slice(off, off + n)
            mx.bind(q[:, sl].contiguous(), kc, vc, torch.tensor([hist + off], dtype=torch.int32, device="cuda"),
                    out[:, sl], gate=gate[:, sl].contiguous(), lse=lse[:, sl], flags=api.F_ROPE | api.F_GATE)
            mx.forward()
            torch.cuda.synchronize()
            mx.check_status()
        ma.check_status()
        assert np.array_equal(host_bits(kc), kc_ref) and np.array_equal(host_bits(vc), vc_ref)
    check_out(host_f32(out), ref, "zig-zag row split")
    check_lse(lse.cpu().numpy(), lse_ref, "zig-zag row split")

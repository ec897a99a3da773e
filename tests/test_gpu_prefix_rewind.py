"""What a serving loop does to the cache between steps, on the paged and the contiguous layout.

Prefix sharing: the reference keeps the cache of the last conversation and re-reads only the new tail when the
next prompt extends it (src/server.cpp:283-306,460-476).  With a block table the same idea serves several
sequences at once: their tables name the SAME pages for the common prefix.  Nothing may be written into a
shared page, and the results must be the bits of sequences that own private copies.

Speculative rewind: a verify step appends D draft rows; if only k are accepted the position is set back to
pos + 1 + k and the next step overwrites the rejected slots (src/spec.cu:104-106; "the KV cache heals itself",
src/model.cu:77-79).  The second step must give the bits of a sequence that never held the rejected rows."""
import numpy as np
import pytest
import torch

from qwengine_b200 import api
from tests.gpu_util import dev_bf16, dev_bits, host_bits, host_f32, run_case
from tests.test_gpu_paged import _paged
from tests.util import Case, check_lse, check_out

pytestmark = pytest.mark.gpu

PAGE = 128


def _bind_paged(c, kc, vc, table, out, lse, pos=None):
    mx = api.Mixer(c.n_seq, c.n_new, kv_heads=c.kv_heads)
    mx.bind(dev_bf16(c.q), kc, vc, torch.from_numpy(c.hist).cuda() if pos is None else pos, out, k_new=dev_bf16(c.k),
            v_new=dev_bf16(c.v), gate=dev_bf16(c.gate), lse=lse, block_table=torch.from_numpy(table).cuda(),
            page_rows=PAGE)
    return mx


@pytest.mark.parametrize("n_new", [1, 4, 160])
def test_two_sequences_share_their_prefix_pages(n_new):
    shared_pages = 3
    c = Case(600 + n_new, [shared_pages * PAGE + 57, shared_pages * PAGE + 300, 90], n_new)
    r0, r1 = int(c.cache_row[0]), int(c.cache_row[1])
    n_shared = shared_pages * PAGE
    c.kc0[r1:r1 + n_shared] = c.kc0[r0:r0 + n_shared]          # sequences 0 and 1 start with the same tokens
    c.vc0[r1:r1 + n_shared] = c.vc0[r0:r0 + n_shared]
    ref, lse_ref, _, _ = c.oracle()
    out_c, lse_c, _, _, _ = run_case(c, out_f32=True)           # private copies, contiguous layout
    kc_h, vc_h, table = _paged(c, PAGE, seed=n_new)
    orphan = table[1, :shared_pages].copy()
    table[1, :shared_pages] = table[0, :shared_pages]           # sequence 1 names sequence 0's prefix pages
    for pg in orphan:                                           # its own former copies now belong to nobody
        kc_h[pg * PAGE:(pg + 1) * PAGE] = 0x7FC0                # NaN: reading them would show
        vc_h[pg * PAGE:(pg + 1) * PAGE] = 0x7FC0
    kc, vc = dev_bits(kc_h), dev_bits(vc_h)
    out = torch.full((c.n_seq, n_new, 24, 256), float("nan"), dtype=torch.float32, device="cuda")
    lse = torch.full((c.n_seq, n_new, 24), float("nan"), dtype=torch.float32, device="cuda")
    mx = _bind_paged(c, kc, vc, table, out, lse)
    mx.forward()
    torch.cuda.synchronize()
    mx.check_status()
    got, got_lse = host_f32(out).reshape(-1, 24, 256), lse.cpu().numpy().reshape(-1, 24)
    assert np.array_equal(got, out_c) and np.array_equal(got_lse, lse_c), "shared prefix pages change the result"
    check_out(got, ref, "shared prefix")
    check_lse(got_lse, lse_ref, "shared prefix")
    kc_after, vc_after = host_bits(kc), host_bits(vc)
    for pg in table[0, :shared_pages]:                          # nobody wrote into a shared page
        sl = slice(int(pg) * PAGE, (int(pg) + 1) * PAGE)
        assert np.array_equal(kc_after[sl], kc_h[sl]) and np.array_equal(vc_after[sl], vc_h[sl])


def _rows_of(c, lo, hi):
    return slice(int(c.cache_row[0]) + lo, int(c.cache_row[0]) + hi)


@pytest.mark.parametrize("layout", ["contiguous", "paged"])
@pytest.mark.parametrize("hist,accepted", [(253, 1), (700, 0), (1021, 2)])
def test_verify_rewind_then_overwrite(layout, hist, accepted):
    D = 4
    consumed = 1 + accepted                                      # src/spec.cu:96
    first = Case(700 + hist, [hist], D, pad_rows=2 * D)         # room for the second step's rows
    second = Case(701 + hist, [hist + consumed], D)             # only its q / k / v / gate are used

    def run_two_steps(with_rejected_rows):
        """Step 1 appends D rows; the position is set back to hist + consumed; step 2 appends D rows there.
        with_rejected_rows=False builds the cache a sequence has that never saw the rejected rows."""
        kc_h, vc_h = first.kc0.copy(), first.vc0.copy()
        table = None
        if layout == "paged":
            kc_h, vc_h, table = _paged(first, PAGE, seed=hist)   # sized for hist + D rows: add spare pages
            spare = np.arange(kc_h.shape[0] // PAGE, kc_h.shape[0] // PAGE + 2, dtype=np.int32)
            kc_h = np.concatenate([kc_h, np.full((2 * PAGE, kc_h.shape[1]), 0x4F00, np.uint16)])
            vc_h = np.concatenate([vc_h, np.full((2 * PAGE, vc_h.shape[1]), 0x4F00, np.uint16)])
            need = (hist + consumed + D + PAGE - 1) // PAGE
            if need > table.shape[1]:
                table = np.concatenate([table, spare[None, :need - table.shape[1]]], axis=1)
        kc, vc = dev_bits(kc_h), dev_bits(vc_h)
        pos = torch.tensor([hist], dtype=torch.int32, device="cuda")
        out = torch.full((1, D, 24, 256), float("nan"), dtype=torch.float32, device="cuda")
        lse = torch.full((1, D, 24), float("nan"), dtype=torch.float32, device="cuda")

        def step(c):
            mx = api.Mixer(1, D)
            if table is None:
                mx.bind(dev_bf16(c.q), kc, vc, pos, out, k_new=dev_bf16(c.k), v_new=dev_bf16(c.v), gate=dev_bf16(c.gate),
                        lse=lse)
            else:
                mx = _bind_paged(c, kc, vc, table, out, lse, pos=pos)
            mx.forward()
            torch.cuda.synchronize()
            mx.check_status()

        if with_rejected_rows:
            step(first)                                          # rows hist .. hist+3, all four drafts
        else:                                                    # only the rows that were kept ever existed
            kept = Case.__new__(Case)
            kept.__dict__.update(first.__dict__)
            kept.n_new = consumed
            kept.q, kept.k, kept.v, kept.gate = (a[:, :consumed] for a in (first.q, first.k, first.v, first.gate))
            mxk = api.Mixer(1, consumed)
            o2 = torch.empty(1, consumed, 24, 256, dtype=torch.float32, device="cuda")
            if table is None:
                mxk.bind(dev_bf16(kept.q), kc, vc, pos, o2, k_new=dev_bf16(kept.k), v_new=dev_bf16(kept.v),
                         gate=dev_bf16(kept.gate))
            else:
                mxk.bind(dev_bf16(kept.q), kc, vc, pos, o2, k_new=dev_bf16(kept.k), v_new=dev_bf16(kept.v),
                         gate=dev_bf16(kept.gate), block_table=torch.from_numpy(table).cuda(), page_rows=PAGE)
            mxk.forward()
            torch.cuda.synchronize()
            mxk.check_status()
        pos.fill_(hist + consumed)                               # k_set_pos(rt.dpos, pos_before + consumed)
        step(second)
        return host_f32(out).reshape(D, 24, 256), lse.cpu().numpy().reshape(D, 24), host_bits(kc), host_bits(vc), table

    o_a, l_a, kc_a, vc_a, table = run_two_steps(True)
    o_b, l_b, kc_b, vc_b, _ = run_two_steps(False)
    assert np.isfinite(o_a).all()
    assert np.array_equal(o_a, o_b) and np.array_equal(l_a, l_b), "rejected draft rows leak into the next step"
    # every live row of the cache is the same either way
    live = hist + consumed + D
    for t in range(live):
        r = t if table is None else int(table[0, t // PAGE]) * PAGE + t % PAGE
        assert np.array_equal(kc_a[r], kc_b[r]) and np.array_equal(vc_a[r], vc_b[r]), "cache row %d" % t
    # and the second step agrees with the oracle run over the kept history
    hist_k = np.concatenate([first.kc0[_rows_of(first, 0, hist)], np.zeros((consumed + D, 1024), np.uint16)])
    hist_v = np.concatenate([first.vc0[_rows_of(first, 0, hist)], np.zeros((consumed + D, 1024), np.uint16)])
    from oracle import pyoracle as O
    O.mixer(first.q[:, :consumed], first.k[:, :consumed], first.v[:, :consumed], first.gate[:, :consumed], hist_k, hist_v,
            [hist])
    ref, lse_ref = O.mixer(second.q, second.k, second.v, second.gate, hist_k, hist_v, [hist + consumed])
    check_out(o_a, ref, "verify after rewind")
    check_lse(l_a, lse_ref, "verify after rewind")

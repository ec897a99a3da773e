"""Paged KV cache (qw_mixer_desc.block_table): the same batch served from a pool of shuffled pages must give
bit-identical outputs to the contiguous layout, and the new rows must land in the pages the block table names.
The reference keeps one contiguous cache for one sequence (src/model.cu:182-184, README.md:365-367); the block
table is what its multi-sequence serving step needs."""
import numpy as np
import pytest
import torch

from qwengine_b200 import api
from tests.gpu_util import dev_bf16, dev_bits, host_bits, host_f32, run_case
from tests.util import Case, check_out

pytestmark = pytest.mark.gpu


def _paged(c, page_rows, seed):
    """Scatters Case c's contiguous cache into shuffled pages.  Returns (kc, vc pools, table, pool rows)."""
    rng = np.random.default_rng(seed)
    need = [(int(h) + c.n_new + page_rows - 1) // page_rows for h in c.hist]
    n_pages = sum(need) + 3                                   # a few pages belong to nobody
    order = rng.permutation(n_pages)
    table = np.full((c.n_seq, max(need)), -1, np.int32)
    kvd = c.kv_heads * 256
    kc = np.full((n_pages * page_rows, kvd), 0x4F00, np.uint16)  # large finite value everywhere else
    vc = kc.copy()
    nxt = 0
    for s in range(c.n_seq):
        r0, h = int(c.cache_row[s]), int(c.hist[s])
        for pg in range(need[s]):
            page = int(order[nxt]); nxt += 1
            table[s, pg] = page
            lo, hi = pg * page_rows, min((pg + 1) * page_rows, h)
            if hi > lo:
                kc[page * page_rows:page * page_rows + hi - lo] = c.kc0[r0 + lo:r0 + hi]
                vc[page * page_rows:page * page_rows + hi - lo] = c.vc0[r0 + lo:r0 + hi]
    table[table < 0] = 0
    return kc, vc, table


def _run_paged(c, page_rows, seed, flags=None):
    kc_h, vc_h, table = _paged(c, page_rows, seed)
    mx = api.Mixer(c.n_seq, c.n_new, kv_heads=c.kv_heads)
    q, k, v, gate = dev_bf16(c.q), dev_bf16(c.k), dev_bf16(c.v), dev_bf16(c.gate)
    kc, vc = dev_bits(kc_h), dev_bits(vc_h)
    out = torch.full((c.n_seq, c.n_new, c.q_heads, 256), float("nan"), dtype=torch.float32, device="cuda")
    lse = torch.full((c.n_seq, c.n_new, c.q_heads), float("nan"), dtype=torch.float32, device="cuda")
    kw = {} if flags is None else {"flags": flags}
    mx.bind(q, kc, vc, torch.from_numpy(c.hist).cuda(), out, k_new=k, v_new=v, gate=gate, lse=lse,
            block_table=torch.from_numpy(table).cuda(), page_rows=page_rows, **kw)
    mx.forward()
    torch.cuda.synchronize()
    mx.check_status()
    return host_f32(out).reshape(-1, c.q_heads, 256), lse.cpu().numpy().reshape(-1, c.q_heads), host_bits(kc), host_bits(vc), table


CASES = {
    "decode_ragged": (Case, (201, [700, 130, 1, 2049], 1), {}),
    "verify": (Case, (202, [513, 90, 1300], 4), {}),
    "short_chunk_2kv": (Case, (203, [260], 20), {"kv_heads": 2}),
    "prefill_chunk_hist": (Case, (204, [300], 160), {"kv_heads": 2}),
    "prefill_scratch": (Case, (205, [0], 384), {"kv_heads": 2}),
    # the last 128-row tile of the first sequence is part empty, and another sequence's rows lie behind it
    "prefill_two_sequences_ragged_tile": (Case, (206, [114, 134], 300), {"kv_heads": 1}),
}


@pytest.mark.parametrize("page_rows", [128, 256])
@pytest.mark.parametrize("name", sorted(CASES))
def test_paged_cache_equals_contiguous(name, page_rows):
    cls, args, kw = CASES[name]
    c = cls(*args, **kw)
    ref, ref_lse, kc_o, vc_o = c.oracle()
    out_c, lse_c, _, _, _ = run_case(c, out_f32=True)
    out_p, lse_p, kc_p, vc_p, table = _run_paged(c, page_rows, seed=args[0])
    assert np.array_equal(out_p, out_c) and np.array_equal(lse_p, lse_c), "paged and contiguous outputs differ"
    check_out(out_p, ref, name)
    for s in range(c.n_seq):                                  # the new rows, where the table says
        for b in range(c.n_new):
            t = int(c.hist[s]) + b
            row = int(table[s, t // page_rows]) * page_rows + t % page_rows
            assert np.array_equal(kc_p[row], kc_o[int(c.cache_row[s]) + t])
            assert np.array_equal(vc_p[row], vc_o[int(c.cache_row[s]) + t])


def test_paged_cache_argument_errors():
    c = Case(207, [10], 1)
    mx = api.Mixer(1, 1)
    q = dev_bf16(c.q)
    kc, vc = dev_bits(c.kc0), dev_bits(c.vc0)
    table = torch.zeros((1, 1), dtype=torch.int32, device="cuda")
    mx.bind(q, kc, vc, torch.from_numpy(c.hist).cuda(), torch.empty_like(q), k_new=dev_bf16(c.k), v_new=dev_bf16(c.v),
            gate=None, block_table=table, page_rows=96)  # not a multiple of 128
    with pytest.raises(api.QwError):
        mx.forward()

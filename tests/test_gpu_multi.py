"""Split of one sequence's KV range across ranks: each rank attends to its sub-range and emits
(o, m, l) partials, the partials are gathered and merged in rank order.  On one GPU the two
sub-ranges are run one after the other (same kernels, same merge); with two or more GPUs the
exchange is a real NCCL all-gather between processes, and also the peer-memory merge that needs no
collective (sharding.PeerExchange)."""
import os
import socket

import numpy as np
import pytest
import torch

from oracle import pyoracle as O
from qwengine_b200 import api, sharding
from tests.gpu_util import dev_bf16, dev_bits, host_f32
from tests.util import Case, check_lse, check_out

pytestmark = pytest.mark.gpu


def _partial_for_range(c, q, kc, vc, lo, hi, owns_new_rows, hist):
    """Partials of the (un-rotated) rows q over cache rows [lo, hi) of the single sequence, whose new rows sit
    at absolute positions hist, hist + 1, ...: the call rotates q itself from q_pos, in fp32, like an unsplit
    call does."""
    B = c.n_new
    mx = api.Mixer(1, B, kv_heads=c.kv_heads)
    part = torch.zeros(B, c.q_heads, api.PARTIAL_FLOATS, dtype=torch.float32, device="cuda")
    crow = torch.tensor([lo], dtype=torch.int64, device="cuda")
    q_pos = torch.tensor([hist], dtype=torch.int32, device="cuda")
    out = torch.empty(1, B, c.q_heads, 256, dtype=torch.bfloat16, device="cuda")
    if owns_new_rows:   # tail range: causal among the new rows, which are its last B rows
        pos = torch.tensor([hi - lo - B], dtype=torch.int32, device="cuda")
        mx.bind(q, kc, vc, pos, out, cache_row=crow, flags=api.F_ROPE, q_pos=q_pos)
    else:               # head range: every row sees all of it
        pos = torch.tensor([hi - lo], dtype=torch.int32, device="cuda")
        mx.bind(q, kc, vc, pos, out, cache_row=crow, flags=api.F_ROPE | api.F_NO_CAUSAL, q_pos=q_pos)
    mx.forward_partial(part)
    torch.cuda.synchronize()
    mx.check_status()
    # two or more rows per sequence run on the tcgen05 split-KV kernel, partials included
    assert api.last_attention_kernel() == ("splitkv_umma_kernel" if B >= 2 else "splitkv_kernel")
    return part


@pytest.mark.parametrize("hist,B,cut", [(700, 1, 384), (3000, 4, 1000), (129, 2, 64), (20000, 4, 12032), (9000, 8, 4096)])
def test_kv_range_split_and_combine_on_one_gpu(hist, B, cut):
    c = Case(300 + B, [hist], B)
    ref, lse_ref, kc_ref, vc_ref = c.oracle()          # also gives the cache with the new rows appended
    kc, vc = dev_bits(kc_ref), dev_bits(vc_ref)
    q = dev_bf16(c.q[0])
    L = hist + B
    parts = torch.stack([_partial_for_range(c, q, kc, vc, 0, cut, False, hist),
                         _partial_for_range(c, q, kc, vc, cut, L, True, hist)])
    out = torch.empty(B, c.q_heads, 256, dtype=torch.float32, device="cuda")
    lse = torch.empty(B, c.q_heads, dtype=torch.float32, device="cuda")
    api.combine_partials(parts, 2, B, c.q_heads, out, gate=dev_bf16(c.gate[0]), lse=lse)
    torch.cuda.synchronize()
    # the split route is held to the same bounds as an unsplit call: max-abs 2e-2, rel-L2 1e-3, LSE 1e-3
    got = host_f32(out)
    check_out(got, ref, "KV-range split")
    check_lse(lse.cpu().numpy(), lse_ref, "KV-range split")
    # the merge on the GPU equals its host specification bit for bit in structure: compare loosely
    o_host, lse_host = sharding.merge_partials_reference(parts.cpu())
    gate = 1.0 / (1.0 + np.exp(-c.gate[0].astype(np.float64)))
    assert np.abs(o_host.numpy() * gate - got).max() < 1e-5


def _nccl_worker(rank, world, port, hist, B, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    torch.distributed.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        c = Case(400, [hist], B)
        ref, lse_ref, kc_ref, vc_ref = c.oracle()
        kc, vc = dev_bits(kc_ref), dev_bits(vc_ref)   # every rank holds the cache here; it reads only its range
        q = dev_bf16(c.q[0])
        L = hist + B
        cut = (L // 2 // 64) * 64
        lo, hi = (0, cut) if rank == 0 else (cut, L)
        part = _partial_for_range(c, q, kc, vc, lo, hi, rank == world - 1, hist)
        parts = sharding.gather_partials(part)
        out = torch.empty(B, c.q_heads, 256, dtype=torch.float32, device="cuda")
        api.combine_partials(parts, world, B, c.q_heads, out, gate=dev_bf16(c.gate[0]))
        torch.cuda.synchronize()
        from tests.util import MAX_ABS, REL_L2, rel_l2
        got = host_f32(out)
        ok = bool(np.abs(got - ref).max() <= MAX_ABS and rel_l2(got, ref) <= REL_L2)
        # the same merge with the exchange inside the kernel, over peer memory: three steps in a row (both buffer
        # sets, and the first one again), each bit-identical to the all-gather + combine result
        ex = sharding.PeerExchange(B, c.q_heads)
        for _ in range(3):
            ex.partial().copy_(part)
            out2 = torch.zeros(B, c.q_heads, 256, dtype=torch.float32, device="cuda")
            ex.combine(out2, gate=dev_bf16(c.gate[0]))
            torch.cuda.synchronize()
            ex.check_status()
            ok = ok and bool(np.array_equal(host_f32(out2), got))
        ret[rank] = ok
    finally:
        torch.distributed.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_kv_range_split_across_two_gpus_with_nccl():
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ret = mp.Manager().dict()
    mp.spawn(_nccl_worker, args=(2, port, 2500, 4, ret), nprocs=2, join=True)
    assert dict(ret) == {0: True, 1: True}


def test_peer_combine_gives_up_when_a_peer_never_publishes():
    """Failure detection without a fault: rank 1's flag word is never set, so the bounded wait in the kernel runs
    out, the status word receives the device error code and the output is left untouched; the context stays usable."""
    rows, heads = 2, 24
    parts = torch.zeros(2, rows, heads, api.PARTIAL_FLOATS, dtype=torch.float32, device="cuda")
    parts[..., 257] = 1.0
    flags = torch.zeros(2, dtype=torch.int32, device="cuda")
    part_ptrs = torch.tensor([parts[0].data_ptr(), parts[1].data_ptr()], dtype=torch.int64, device="cuda")
    flag_ptrs = torch.tensor([flags[0:1].data_ptr(), flags[1:2].data_ptr()], dtype=torch.int64, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = torch.full((rows, heads, 256), 7.0, dtype=torch.float32, device="cuda")
    api.combine_partials_peer(part_ptrs, flag_ptrs, 0, 2, 1, rows, heads, out, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 106
    assert int(flags[0].item()) == 1 and int(flags[1].item()) == 0
    assert bool((out == 7.0).all())
    # once the "peer" has published, the same call goes through
    flags[1] = 1
    status.zero_()
    api.combine_partials_peer(part_ptrs, flag_ptrs, 0, 2, 1, rows, heads, out, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0 and bool((out == 0.0).all())

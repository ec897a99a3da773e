"""World-size-2 tests of the multi-GPU host logic on CPU (gloo): sharding plans, the KV-bytes
partitioner, and the gather + fixed-order merge of split-KV partials against the oracle."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import pyoracle as O
from qwengine_b200 import sharding
from tests.util import Case, rel_l2


def test_shard_plans_cover_all_heads_and_sequences():
    for world in (1, 2, 4, 8):
        seen = {}
        for r in range(world):
            n, first, groups, g = sharding.shard_plan(world, r)
            for h in range(first, first + n):
                seen.setdefault((h, g), 0)
                seen[(h, g)] += 1
        groups = 2 if world == 8 else 1
        assert sorted(seen) == [(h, g) for h in range(4) for g in range(groups)] and set(seen.values()) == {1}
    with pytest.raises(ValueError):
        sharding.shard_plan(3, 0)


def test_partition_for_exchange_gives_every_rank_at_most_one_range_of_a_sequence():
    """The partition behind the one-exchange merge: exact cover, cuts on tile boundaries, a cut sequence's ranges on
    distinct ranks, balanced loads; and the query-row split of a chunk over a GPU pair has equal causal work."""
    rng = np.random.default_rng(6)
    lens = np.exp(rng.uniform(np.log(512), np.log(131072), 64)).astype(int) + 1
    for world in (1, 2, 4, 8):
        bins = sharding.partition_for_exchange(lens, world, max_piece=32768)
        assert len(bins) == world
        per_seq = {}
        for r, b in enumerate(bins):
            for s, a, e in b:
                assert 0 <= a < e <= lens[s] and (a % 128 == 0)
                per_seq.setdefault(s, []).append((a, e, r))
        for s, L in enumerate(lens):
            rs = sorted(per_seq[s])
            assert rs[0][0] == 0 and rs[-1][1] == L and all(rs[i][1] == rs[i + 1][0] for i in range(len(rs) - 1))
            assert len({r for _, _, r in rs}) == len(rs), "two ranges of one sequence on one rank"
            if world == 1:
                assert len(rs) == 1
        load = [sum(e - a for _, a, e in b) for b in bins]
        assert max(load) <= 1.02 * sum(load) / world
    # zig-zag query-row split of a 2048-row chunk behind h cached tokens: rows [0,512) + [1536,2048) vs [512,1536)
    pairs = lambda h, off, n: n * (h + off) + n * (n + 1) // 2
    for h in (0, 2048, 30720):
        assert pairs(h, 0, 512) + pairs(h, 1536, 512) == pairs(h, 512, 1024)


def test_partition_by_kv_bytes_is_exact_and_balanced():
    rng = np.random.default_rng(5)
    lens = np.exp(rng.uniform(np.log(512), np.log(131072), 64)).astype(int)  # BASELINE config 5 lengths
    bins = sharding.partition_by_kv_bytes(lens, 8)
    covered = {}
    for b in bins:
        for s, a, e in b:
            assert 0 <= a < e <= lens[s]
            covered.setdefault(s, []).append((a, e))
    for s, L in enumerate(lens):
        rs = sorted(covered[s])
        assert rs[0][0] == 0 and rs[-1][1] == L and all(x[1] == y[0] for x, y in zip(rs, rs[1:]))
    load = [sum(e - a for _, a, e in b) for b in bins]
    assert max(load) <= 1.05 * sum(load) / 8 + 64
    assert sharding.partition_by_kv_bytes([], 4) == [[], [], [], []]
    assert sharding.partition_by_kv_bytes([10], 2, max_share=4) == [[(0, 0, 4), (0, 8, 10)], [(0, 4, 8)]]


def _partial_numpy(q_rot, K, V, scale_log2):
    """(o, m, l) of rows q_rot [R, D] over keys K, V [n, D], in the library's partial format."""
    s = (q_rot.astype(np.float64) @ K.astype(np.float64).T) * scale_log2
    m = s.max(axis=1)
    p = np.exp2(s - m[:, None])
    out = np.zeros((q_rot.shape[0], sharding.PARTIAL_FLOATS), np.float32)
    out[:, :256] = p @ V.astype(np.float64)
    out[:, 256], out[:, 257] = m, p.sum(axis=1)
    return out


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # one sequence, 1 KV head, its KV range cut in two; rank 1 owns the tail with the new row
        c = Case(77, [300], 1, kv_heads=1)
        ref, lse_ref, kc, vc = c.oracle()
        L, cut = 301, 192
        K = O.bf16_bits_to_f32(kc[:L]).reshape(L, 256)
        V = O.bf16_bits_to_f32(vc[:L]).reshape(L, 256)
        q = c.q[0].copy()
        O.rope_f32(q, 300)
        lo, hi = (0, cut) if rank == 0 else (cut, L)
        part = _partial_numpy(q[0], K[lo:hi], V[lo:hi], (1.0 / 16.0) * 1.4426950408889634)
        parts = sharding.gather_partials(torch.from_numpy(part)[None])      # [world, 1, 6, 260]
        o, lse = sharding.merge_partials_reference(parts)
        gate = 1.0 / (1.0 + np.exp(-c.gate[0, 0].astype(np.float64)))
        got = o[0].numpy().astype(np.float64) * gate
        ok = rel_l2(got, ref[0]) < 1e-5 and np.abs(lse[0].numpy() - lse_ref[0]).max() < 1e-4
        # a rank whose sub-range is empty contributes l = 0 and must be ignored by the merge
        empty = torch.zeros_like(parts[0])
        empty[..., 256] = float("-inf")
        o2, _ = sharding.merge_partials_reference(torch.cat([parts, empty[None]]))
        ok = ok and torch.equal(o2, o)
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_split_kv_partials_gathered_over_gloo_match_the_oracle():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(2, port, ret), nprocs=2, join=True)
    assert dict(ret) == {0: True, 1: True}

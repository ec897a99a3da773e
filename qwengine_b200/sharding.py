"""Host-side partitioning of the attention path across the GPUs of one box (one process per GPU).

The reference is single-GPU; this is new design.  Three partitions are used:
  * KV-head sharding (2 and 4 GPUs): a rank owns kv_heads/N KV heads and their 6x query heads of
    every sequence; outputs are disjoint head slices and no data crosses GPUs.
  * KV head x sequence split (8 GPUs): 4 KV heads x 2 groups of sequences.
  * KV-range split of one long sequence across ranks: each rank attends to its sub-range and
    produces (o, m, l) partials; the partials are all-gathered and merged in rank order.
Functions here are pure host logic (lists, torch.distributed calls); they run on CPU with the gloo
backend in the tests and with NCCL on the GPUs.
"""
import torch
import torch.distributed as dist

PARTIAL_FLOATS = 260


def shard_plan(world, rank):
    """(kv_heads_local, first_kv_head, seq_groups, seq_group) for KV-head sharding of 4 KV heads."""
    if world == 1:
        return 4, 0, 1, 0
    if world == 2:
        return 2, 2 * rank, 1, 0
    if world == 4:
        return 1, rank, 1, 0
    if world == 8:
        return 1, rank % 4, 2, rank // 4
    raise ValueError("world size must be 1, 2, 4 or 8")


def partition_by_kv_bytes(kv_lens, n_bins, max_share=None):
    """Greedy longest-first assignment of sequences to bins by KV bytes (proportional to length).
    A sequence longer than `max_share` (default: total / n_bins, rounded up to 64) is cut into
    KV sub-ranges of at most that size first.  Returns a list of n_bins lists of
    (seq, start, end) ranges; every token of every sequence appears exactly once."""
    total = sum(int(x) for x in kv_lens)
    if max_share is None:
        max_share = -(-max(1, -(-total // n_bins)) // 64) * 64
    pieces = []
    for s, L in enumerate(kv_lens):
        L = int(L)
        a = 0
        while L - a > max_share:
            pieces.append((s, a, a + max_share))
            a += max_share
        if L > a:
            pieces.append((s, a, L))
    pieces.sort(key=lambda r: (-(r[2] - r[1]), r[0], r[1]))
    bins, load = [[] for _ in range(n_bins)], [0] * n_bins
    for pc in pieces:
        b = min(range(n_bins), key=lambda i: (load[i], i))
        bins[b].append(pc)
        load[b] += pc[2] - pc[1]
    for b in bins:
        b.sort()
    return bins


def partition_for_exchange(kv_lens, n_bins, align=128, max_piece=None):
    """Partition for a step whose split sequences are merged by one exchange of per-rank partials: greedy
    longest-first by KV bytes like partition_by_kv_bytes, but a sequence longer than the per-bin share
    (total / n_bins) is cut into ceil(len / share) nearly equal ranges (cuts on multiples of `align`, so that no
    K/V tile or cache page straddles a cut) which go to DISTINCT bins -- every rank then holds at most one
    range of a sequence and contributes one partial row per split sequence.  `max_piece` lowers the length
    above which a sequence is cut (a serving step bounds the latency of its longest sequence that way).
    Returns n_bins lists of (seq, start, end); every token of every sequence appears exactly once."""
    lens = [int(x) for x in kv_lens]
    total = sum(lens)
    share = max(align, -(-total // n_bins))
    if max_piece is not None:
        share = max(align, min(share, int(max_piece)))
    bins, load = [[] for _ in range(n_bins)], [0] * n_bins
    for s in sorted(range(len(lens)), key=lambda i: (-lens[i], i)):
        L = lens[s]
        n_cut = min(n_bins, -(-L // share)) if (L > share and n_bins > 1) else 1
        if n_cut <= 1:
            b = min(range(n_bins), key=lambda i: (load[i], i))
            bins[b].append((s, 0, L))
            load[b] += L
            continue
        step = -(-(-(-L // n_cut)) // align) * align          # ceil(L / n_cut) rounded up to the alignment
        cuts = [min(L, i * step) for i in range(n_cut + 1)]
        cuts[-1] = L
        pieces = [(cuts[i], cuts[i + 1]) for i in range(n_cut) if cuts[i + 1] > cuts[i]]
        targets = sorted(range(n_bins), key=lambda i: (load[i], i))[:len(pieces)]
        for b, (a, e) in zip(targets, sorted(pieces, key=lambda r: -(r[1] - r[0]))):
            bins[b].append((s, a, e))
            load[b] += e - a
    for b in bins:
        b.sort()
    return bins


def gather_partials(partial, group=None):
    """All-gathers one rank's partials [rows, q_heads, 260] into [world, rows, q_heads, 260],
    ordered by rank, which is also the order the merge uses (fixed => bit-stable)."""
    world = dist.get_world_size(group)
    partial = partial.contiguous()
    out = torch.empty((world * partial.shape[0],) + tuple(partial.shape[1:]), dtype=partial.dtype,
                      device=partial.device)
    dist.all_gather_into_tensor(out, partial, group=group)
    return out.view((world,) + tuple(partial.shape))


def merge_partials_reference(parts):
    """Merge [n_parts, rows, heads, 260] partials on the host (torch, any device), in index order.
    The GPU path uses qw_combine_partials; this is its specification for the CPU tests.
    Returns (o [rows, heads, 256] normalised, lse [rows, heads] natural log)."""
    o, m, l = parts[..., :256], parts[..., 256], parts[..., 257]
    live = l > 0
    m_eff = torch.where(live, m, torch.full_like(m, float("-inf")))
    mg = m_eff.max(dim=0).values
    m_use = torch.where(torch.isinf(mg), torch.zeros_like(mg), mg)
    f = torch.where(live, torch.exp2(m - m_use), torch.zeros_like(m))
    lg = torch.zeros_like(mg)
    acc = torch.zeros_like(o[0])
    for k in range(parts.shape[0]):   # fixed order
        lg = lg + l[k] * f[k]
        acc = acc + o[k] * f[k][..., None]
    return acc / lg[..., None], (mg + torch.log2(lg)) * 0.6931471805599453


class PeerExchange:
    """Cross-GPU merge of split-KV partials without a collective: every rank writes its partials into a buffer
    that its peers have mapped (torch symmetric memory over NVLink) and the combine kernel of each rank reads
    the others' partials in place, after a flag handshake inside the kernel (qw_combine_partials_peer).
    Two buffer / flag sets alternate by step so that a fast rank never overwrites what a slow one still reads.

        ex = PeerExchange(rows, q_heads)             # collective: call on every rank of the group
        mixer.forward_partial(ex.partial())          # this rank's (o, m, l) for its KV sub-range
        ex.combine(out, gate=gate, lse=lse)          # merged, normalised, gated output
    """

    def __init__(self, rows, q_heads, group=None, device=None):
        import torch.distributed._symmetric_memory as symm
        from . import api
        self._api = api
        group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.rows, self.q_heads = rows, q_heads
        self.n = rows * q_heads * api.PARTIAL_FLOATS
        device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        # [two partial buffers | 64 ints of flags]; float32 storage, the flags are viewed as int32
        self.buf = symm.empty(2 * self.n + 64, dtype=torch.float32, device=device)
        self.buf.zero_()
        hdl = symm.rendezvous(self.buf, group)
        ptrs = [int(p) for p in hdl.buffer_ptrs]
        torch.cuda.synchronize(device)
        dist.barrier(group)                          # every flag word is zero before anyone publishes a step
        self._hdl = hdl
        self.part_ptrs = [torch.tensor([p + par * self.n * 4 for p in ptrs], dtype=torch.int64, device=device)
                          for par in (0, 1)]
        self.flag_ptrs = [torch.tensor([p + (2 * self.n + par) * 4 for p in ptrs], dtype=torch.int64, device=device)
                          for par in (0, 1)]
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        self.step = 0

    def partial(self):
        """This rank's partial buffer for the NEXT combine: [rows, q_heads, 260] float32 (a view, no copy)."""
        par = (self.step + 1) & 1
        return self.buf[par * self.n:(par + 1) * self.n].view(self.rows, self.q_heads, self._api.PARTIAL_FLOATS)

    def combine(self, out, gate=None, lse=None, stream=None):
        self.step += 1
        par = self.step & 1
        self._api.combine_partials_peer(self.part_ptrs[par], self.flag_ptrs[par], self.rank, self.world, self.step,
                                        self.rows, self.q_heads, out, gate=gate, lse=lse, status=self.status,
                                        stream=stream)

    def check_status(self):
        code = int(self.status.item())
        if code:
            raise RuntimeError("peer combine reported device error code %d" % code)

"""The allocation-free decode entry point (qw_attn_decode_bf16_noalloc) against the regular one.

Collected last on purpose: a run that stops at the first failure has then already run every
other test.  The entry point exists for callers that cannot give the library any scratch
memory -- an engine that took all its device memory in one block at start-up, a plugin slot
with tensors but no allocator, a loop where cudaMalloc is banned because it may synchronise --
so its split-KV partials live in a fixed array inside the library.  Two calls in a row are
checked because that array keeps the first call's partials when the second one starts.
"""
import numpy as np
import pytest
import torch

from qwengine_b200 import api
from tests.gpu_util import dev_bf16, dev_bits, host_f32
from oracle import pyoracle as O
from tests.util import MAX_ABS, REL_L2, Case, bf16_floor, rel_l2

pytestmark = pytest.mark.gpu


def _both(c, ctx, pos0, B):
    """Runs the scratch-taking entry point and the allocation-free one on the same inputs."""
    q = dev_bf16(c.q[0][:B])
    kc, vc = dev_bits(c.kc0), dev_bits(c.vc0)
    dpos = torch.tensor([pos0], dtype=torch.int32, device="cuda")
    want = torch.empty_like(q)
    got = torch.full_like(q, float("nan"))
    scratch = torch.empty(B * 24 * ctx, dtype=torch.float32, device="cuda")
    api.attn_decode(q, kc, vc, want, dpos, 256, 4, 24, 1.0 / 16.0, scratch, ctx, B=B)
    before = torch.cuda.memory_allocated()
    api.attn_decode_noalloc(q, kc, vc, got, dpos, 256, 4, 24, 1.0 / 16.0, ctx, B=B)
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == before
    # and against the oracle itself, not only against the scratch-taking entry: attention of the given (already
    # rotated) rows over the first pos0 + b + 1 cache rows, no gate; bf16 output, hence the rounding floor
    ref, _ = O.mixer(c.q[:, :B], None, None, None, c.kc0.copy(), c.vc0.copy(), [pos0], do_rope=False, do_append=False,
                     do_gate=False)
    g = host_f32(got)
    assert np.abs(g - ref).max() <= MAX_ABS
    assert rel_l2(g, ref) <= float(np.hypot(REL_L2, bf16_floor(ref)))
    return host_f32(want), g


def test_noalloc_decode_matches_regular_entry_on_two_calls_in_a_row():
    ctx = 4096
    # history of 3000 rows is drawn; rows the attention may touch beyond it are finite poison
    c = Case(123, [3000], 8, pad_rows=ctx - 3008)
    # first call: 4 verify rows deep in the cache (many CTAs leave partials in the built-in array)
    want, got = _both(c, ctx, 2900, 4)
    assert np.isfinite(got).all()
    assert np.abs(got - want).max() <= MAX_ABS and rel_l2(got, want) <= REL_L2
    # second call, straight after: one row, a short history -- far fewer partials than the array
    # still holds from the first call
    want2, got2 = _both(c, ctx, 70, 1)
    assert np.isfinite(got2).all()
    assert np.abs(got2 - want2).max() <= MAX_ABS and rel_l2(got2, want2) <= REL_L2
    # and a third shape with two unit blocks (B = 8)
    want3, got3 = _both(c, ctx, 1500, 8)
    assert np.abs(got3 - want3).max() <= MAX_ABS and rel_l2(got3, want3) <= REL_L2


def test_noalloc_decode_rejects_what_its_array_cannot_hold():
    l = api.lib()
    buf = torch.zeros(64, dtype=torch.int32, device="cuda")
    p = buf.data_ptr()
    rc = l.qw_attn_decode_bf16_noalloc(p, p, p, p, p, 256, 4, 24, 0.0625, 128, 9, None)
    assert rc == 6 and b"capacity" in l.qw_strerror(rc)

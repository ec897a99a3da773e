"""On a GPU box: the reference engine's own kernels (oracle/_ref, built from the reference sources)
against the oracle and against the B200 path.  Skipped when the test-only library is absent."""
import os
import sys

import numpy as np
import pytest
import torch

from oracle import pyoracle as O
from tests.conftest import ROOT
from tests.util import Case, check_out, rel_l2

sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))
pytestmark = pytest.mark.gpu

REF_LIB = os.path.join(ROOT, "oracle", "_ref", "libref_attn.so")


@pytest.mark.skipif(not os.path.exists(REF_LIB), reason="oracle/_ref/libref_attn.so not built")
@pytest.mark.parametrize("hist,B,prefill", [(500, 1, False), (129, 4, False), (0, 40, True), (77, 19, True)])
def test_reference_kernels_agree_with_oracle_and_b200_path(hist, B, prefill):
    import make_ref_golden as R
    from tests.gpu_util import run_case
    l = R.load_ref()
    c = Case(90 + B, [hist], B)
    ctx = hist + B
    kc = torch.zeros(ctx, 1024, device="cuda")
    vc = torch.zeros(ctx, 1024, device="cuda")
    kc[:hist] = torch.from_numpy(O.bf16_bits_to_f32(c.kc0[:hist])).cuda()
    vc[:hist] = torch.from_numpy(O.bf16_bits_to_f32(c.vc0[:hist])).cuda()
    dev = lambda a: torch.from_numpy(a.copy()).cuda()
    out_ref = R.run_reference_layer(l, dev(c.q[0]), dev(c.k[0]), dev(c.v[0]), dev(c.gate[0]), kc, vc, hist, 4, ctx,
                                    prefill).cpu().numpy()
    # oracle in the reference's own storage mode (fp32 cache)
    kc32 = np.zeros((ctx, 1024), np.float32)
    vc32 = np.zeros((ctx, 1024), np.float32)
    kc32[:hist], vc32[:hist] = O.bf16_bits_to_f32(c.kc0[:hist]), O.bf16_bits_to_f32(c.vc0[:hist])
    o32, _ = O.mixer(c.q, c.k, c.v, c.gate, kc32, vc32, [hist])
    assert np.abs(o32 - out_ref).max() < 5e-4 and rel_l2(o32, out_ref) < 2e-4
    # B200 path (bf16 cache) against the reference kernels: only the K rounding separates them
    ours, _, _, _, _ = run_case(c, out_f32=True)
    assert np.abs(ours - out_ref).max() <= 2e-2 and rel_l2(ours, out_ref) < 5e-3

"""The fused mixer fed by the fused q/k/v projection rows (qw_mixer_forward_fused): what the reference does
with unpack3, k_split_qgate and k_rmsnorm_head between the GEMM and attention (src/model.cu:219-226) runs
inside the call.  Checked against the oracle's restatement of those steps and, from the committed
fixtures, against the reference's own kernels."""
import glob
import os

import numpy as np
import pytest
import torch

from oracle import pyoracle as O
from qwengine_b200 import api
from tests.gpu_util import dev_bits, host_bits, host_f32
from tests.util import GOLDEN, check_lse, check_out, check_out_bf16, rel_l2

pytestmark = pytest.mark.gpu


def _problem(seed, hist, n_new, kv_heads):
    rng = np.random.default_rng(seed)
    hist = np.asarray(hist, np.int32)
    n_seq, hq, kvd = len(hist), 6 * kv_heads, kv_heads * 256
    cap = hist.astype(np.int64) + n_new
    cache_row = np.concatenate([[0], np.cumsum(cap)[:-1]]).astype(np.int64)
    kc0 = np.full((int(cap.sum()), kvd), 0x4F00, np.uint16)  # slots to be appended hold a large finite value
    vc0 = kc0.copy()
    for s in range(n_seq):
        r0, h = int(cache_row[s]), int(hist[s])
        kc0[r0:r0 + h] = O.f32_to_bf16_bits(rng.standard_normal((h, kvd), dtype=np.float32))
        vc0[r0:r0 + h] = O.f32_to_bf16_bits(rng.standard_normal((h, kvd), dtype=np.float32))
    fused = (1.7 * rng.standard_normal((n_seq * n_new, hq * 512 + 2 * kvd))).astype(np.float32)
    qw = O.f32_to_bf16_bits((0.25 * rng.standard_normal(256)).astype(np.float32))
    kw = O.f32_to_bf16_bits((0.25 * rng.standard_normal(256)).astype(np.float32))
    return dict(hist=hist, n_seq=n_seq, n_new=n_new, kv_heads=kv_heads, hq=hq, cache_row=cache_row, kc0=kc0, vc0=vc0,
                fused=fused, qw=qw, kw=kw)


def _oracle(p, fused=None, eps=1e-6):
    q, gate, k, v = O.fused_rows(p["fused"] if fused is None else fused, p["qw"], p["kw"], q_heads=p["hq"],
                                 kv_heads=p["kv_heads"], eps=eps, round_bf16=True)
    shp = lambda a, h: a.reshape(p["n_seq"], p["n_new"], h, 256)
    kc, vc = p["kc0"].copy(), p["vc0"].copy()
    out, lse = O.mixer(shp(q, p["hq"]), shp(k, p["kv_heads"]), shp(v, p["kv_heads"]), shp(gate, p["hq"]), kc, vc,
                       p["hist"], p["cache_row"], kv_heads=p["kv_heads"])
    return out, lse, kc, vc, q, gate


def _run(p, fused_t, out_dtype, eps=1e-6):
    mx = api.Mixer(p["n_seq"], p["n_new"], kv_heads=p["kv_heads"])
    n = p["n_seq"] * p["n_new"]
    q = torch.full((n, p["hq"], 256), float("nan"), dtype=torch.bfloat16, device="cuda")
    gate = torch.full_like(q, float("nan"))
    kc, vc = dev_bits(p["kc0"]), dev_bits(p["vc0"])
    out = torch.full((n, p["hq"], 256), float("nan"), dtype=out_dtype, device="cuda")
    lse = torch.full((n, p["hq"]), float("nan"), dtype=torch.float32, device="cuda")
    mx.bind(q, kc, vc, torch.from_numpy(p["hist"]).cuda(), out, gate=gate, lse=lse,
            cache_row=torch.from_numpy(p["cache_row"]).cuda(), fused=True)
    mx.forward_fused(fused_t, dev_bits(p["qw"]), dev_bits(p["kw"]), eps=eps)
    torch.cuda.synchronize()
    mx.check_status()
    return host_f32(out), lse.cpu().numpy(), host_bits(kc), host_bits(vc), host_bits(q), host_bits(gate), mx


CASES = {
    "decode_ragged": (101, [300, 17, 1029], 1, 4),
    "verify": (102, [513, 64], 4, 4),
    "short_chunk_1kv": (103, [40], 9, 1),
    "prefill_chunk": (104, [130], 200, 2),   # tcgen05 CTA-pair kernel
    "prefill_scratch": (105, [0], 128, 4),
}


@pytest.mark.parametrize("name", sorted(CASES))
def test_fused_rows_fp32_input_matches_oracle(name):
    p = _problem(*CASES[name])
    ref, ref_lse, kc_ref, vc_ref, q_ref, gate_ref = _oracle(p)
    out, lse, kc, vc, q, gate, mx = _run(p, torch.from_numpy(p["fused"]).cuda(), torch.float32)
    assert mx.launches() == 2, "one prologue launch + one attention launch"
    assert np.array_equal(vc, vc_ref), "appended V rows"
    assert np.array_equal(kc, kc_ref), "normalised, rotated K rows are bit-exact (double arithmetic on both sides)"
    assert np.array_equal(gate, O.f32_to_bf16_bits(gate_ref)), "gate"
    # q is normalised in fp32 on the GPU and in double in the oracle: a bf16 rounding may flip, rarely
    qd = O.bf16_bits_to_f32(q) - q_ref
    assert np.mean(qd != 0) < 2e-3 and np.abs(qd).max() <= np.abs(q_ref).max() * 2.0 ** -7
    check_out(out, ref, name)
    check_lse(lse, ref_lse, name)
    # Attention alone, against the oracle fed with the very q rows the prologue wrote: this is the tight comparison.
    # (One flipped bf16 rounding of q moves a logit by about 1e-3, so over random shapes the end-to-end LSE above can
    # pass its 1e-3 bound by a little: 1.15e-3 was seen once in 670 random draws, all of which kept this one.)
    shp = lambda a, h: a.reshape(p["n_seq"], p["n_new"], h, 256)
    _, _, k_ref, v_ref = O.fused_rows(p["fused"], p["qw"], p["kw"], q_heads=p["hq"], kv_heads=p["kv_heads"], eps=1e-6,
                                      round_bf16=True)
    kc2, vc2 = p["kc0"].copy(), p["vc0"].copy()
    ref2, lse2 = O.mixer(shp(O.bf16_bits_to_f32(q), p["hq"]), shp(k_ref, p["kv_heads"]), shp(v_ref, p["kv_heads"]),
                         shp(gate_ref, p["hq"]), kc2, vc2, p["hist"], p["cache_row"], kv_heads=p["kv_heads"])
    check_out(out, ref2, name + ", q as written")
    check_lse(lse, lse2, name + ", q as written")


def test_fused_rows_bf16_input_and_bf16_output():
    p = _problem(110, [700, 5], 2, 4)
    fused_bf = O.bf16_bits_to_f32(O.f32_to_bf16_bits(p["fused"]))
    ref, ref_lse, kc_ref, vc_ref, _, _ = _oracle(p, fused=fused_bf)
    out, lse, kc, vc, _, _, _ = _run(p, torch.from_numpy(fused_bf).cuda().to(torch.bfloat16), torch.bfloat16)
    assert np.array_equal(kc, kc_ref) and np.array_equal(vc, vc_ref)
    check_out_bf16(out, ref, "bf16 rows")
    check_lse(lse, ref_lse, "bf16 rows")


_REF_FUSED = sorted(glob.glob(os.path.join(GOLDEN, "ref_fused_*.npz")))


@pytest.mark.skipif(not _REF_FUSED, reason="no fused-row fixtures committed yet")
@pytest.mark.parametrize("path", _REF_FUSED, ids=os.path.basename)
def test_fused_rows_against_reference_kernel_golden(path):
    """Against what the reference's own kernels produced from the same fused rows (fp32 end to end there).
    The gap is the bf16 storage of q, gate and the cache rows on this side: bounded, not bit-exact."""
    z = np.load(path)
    kvh, hist, n_new = int(z["kv_heads"]), int(z["hist"]), int(z["n_new"])
    p = dict(hist=np.asarray([hist], np.int32), n_seq=1, n_new=n_new, kv_heads=kvh, hq=6 * kvh,
             cache_row=np.zeros(1, np.int64), fused=z["fused"], qw=z["q_norm_w"], kw=z["k_norm_w"])
    p["kc0"] = np.full((hist + n_new, kvh * 256), 0x4F00, np.uint16)
    p["vc0"] = p["kc0"].copy()
    p["kc0"][:hist], p["vc0"][:hist] = z["kc0"], z["vc0"]
    out, _, kc, vc, _, _, _ = _run(p, torch.from_numpy(z["fused"]).cuda(), torch.float32, eps=float(z["eps"]))
    assert np.array_equal(vc[hist:], O.f32_to_bf16_bits(z["v_rows"]))
    assert np.abs(O.bf16_bits_to_f32(kc[hist:]) - z["k_rows"]).max() <= np.abs(z["k_rows"]).max() * 2.0 ** -8
    got = out.reshape(z["out"].shape)
    assert np.abs(got - z["out"]).max() <= 2e-2 and rel_l2(got, z["out"]) <= 4e-3


def test_fused_rows_argument_errors():
    p = _problem(120, [8], 1, 4)
    mx = api.Mixer(1, 1)
    q = torch.zeros((1, 24, 256), dtype=torch.bfloat16, device="cuda")
    kc, vc = dev_bits(p["kc0"]), dev_bits(p["vc0"])
    mx.bind(q, kc, vc, torch.from_numpy(p["hist"]).cuda(), torch.empty_like(q), gate=None, fused=True)
    with pytest.raises(api.QwError):  # no gate buffer to write the de-interleaved gate into
        mx.forward_fused(torch.from_numpy(p["fused"]).cuda(), dev_bits(p["qw"]), dev_bits(p["kw"]))

"""CPU tests of the oracle: rounding rule, golden vectors, internal consistency."""
import glob
import os

import numpy as np
import pytest

from oracle import pyoracle as O
from tests.util import GOLDEN, Case, rel_l2


def test_bf16_rounding_rule():
    l = O.lib()
    # ties to even, carry into the exponent, sign symmetry
    cases = {0x3F808000: 0x3F80, 0x3F818000: 0x3F82, 0x3F808001: 0x3F81, 0x3F7FFFFF: 0x3F80,
             0xBF808000: 0xBF80, 0x00000000: 0x0000, 0x7F7FFFFF: 0x7F80}
    for bits, want in cases.items():
        f = np.array([bits], np.uint32).view(np.float32)[0]
        assert l.oracle_f32_to_bf16(float(f)) == want
        assert int(O.f32_to_bf16_bits(np.array([f]))[0]) == want
    a = np.random.default_rng(0).standard_normal(4096).astype(np.float32)
    b = O.f32_to_bf16_bits(a)
    assert all(l.oracle_f32_to_bf16(float(x)) == int(y) for x, y in zip(a[:256], b[:256]))
    assert np.array_equal(O.f32_to_bf16_bits(O.bf16_bits_to_f32(b)), b)


@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(GOLDEN, "hf_*.npz"))), ids=os.path.basename)
def test_oracle_matches_hf_golden(path):
    """The oracle reproduces vectors computed with the Hugging Face Qwen3.5 attention functions."""
    z = np.load(path)
    kvh, hist, n_new = int(z["kv_heads"]), int(z["hist"]), int(z["n_new"])
    f = O.bf16_bits_to_f32
    kc = np.zeros((hist + n_new, kvh * 256), np.uint16)
    vc = np.zeros_like(kc)
    kc[:hist] = z["kc0"].reshape(hist, kvh * 256)
    vc[:hist] = z["vc0"].reshape(hist, kvh * 256)
    mpos = z["mpos"][None] if z["mpos"].size else None
    out, lse = O.mixer(f(z["q"])[None], f(z["k"])[None], f(z["v"])[None], f(z["gate"])[None], kc, vc, [hist],
                       mpos=mpos, kv_heads=kvh)
    assert np.array_equal(kc[hist:].reshape(n_new, kvh, 256), z["k_rot"]), "appended K rows differ"
    assert np.array_equal(vc[hist:].reshape(n_new, kvh, 256), z["v"]), "appended V rows differ"
    assert np.abs(out - z["out"]).max() < 2e-6
    assert np.abs(lse - z["lse"]).max() < 2e-6


_REF = sorted(p for p in glob.glob(os.path.join(GOLDEN, "ref_*.npz")) if "ref_fused" not in p)
_REF_FUSED = sorted(glob.glob(os.path.join(GOLDEN, "ref_fused_*.npz")))


@pytest.mark.skipif(not _REF, reason="no reference-kernel fixtures committed yet")
@pytest.mark.parametrize("path", _REF, ids=os.path.basename)
def test_oracle_matches_reference_kernel_golden(path):
    """The oracle (fp32-cache mode) reproduces what the reference engine's own kernels produced.
    The reference evaluates pow / sincos / exp with fast intrinsics, so agreement is to ~1e-5."""
    z = np.load(path)
    kvh, hist, n_new = int(z["kv_heads"]), int(z["hist"]), int(z["n_new"])
    f = O.bf16_bits_to_f32
    kc = np.zeros((hist + n_new, kvh * 256), np.float32)
    vc = np.zeros_like(kc)
    kc[:hist] = f(z["kc0"]).reshape(hist, kvh * 256)
    vc[:hist] = f(z["vc0"]).reshape(hist, kvh * 256)
    mpos = z["mpos"][None] if z["mpos"].size else None
    out, _ = O.mixer(f(z["q"])[None], f(z["k"])[None], f(z["v"])[None], f(z["gate"])[None], kc, vc, [hist],
                     mpos=mpos, kv_heads=kvh)
    assert np.array_equal(vc[hist:], z["v_rows"])
    assert np.abs(kc[hist:] - z["k_rows"]).max() < 2e-4, "rotated K rows"
    assert np.abs(out - z["out"]).max() < 2e-4 and rel_l2(out, z["out"]) < 1e-4


@pytest.mark.skipif(not _REF_FUSED, reason="no fused-row fixtures committed yet")
@pytest.mark.parametrize("path", _REF_FUSED, ids=os.path.basename)
def test_oracle_fused_rows_match_reference_kernel_golden(path):
    """From the fused projection row on: k_unpack3, k_split_qgate and k_rmsnorm_head as the reference's own
    kernels ran them (src/model.cu:219-226), then the layer.  fp32 everywhere, as in the reference."""
    z = np.load(path)
    kvh, hist, n_new = int(z["kv_heads"]), int(z["hist"]), int(z["n_new"])
    q, gate, k, v = O.fused_rows(z["fused"], z["q_norm_w"], z["k_norm_w"], q_heads=6 * kvh, kv_heads=kvh,
                                 eps=float(z["eps"]), round_bf16=False)
    assert np.array_equal(gate, z["gate"]) and np.array_equal(v.reshape(n_new, -1), z["v_rows"])
    assert np.abs(q - z["q_norm"]).max() < 2e-5 and np.abs(k - z["k_norm"]).max() < 2e-5
    f = O.bf16_bits_to_f32
    kc = np.zeros((hist + n_new, kvh * 256), np.float32)
    vc = np.zeros_like(kc)
    kc[:hist] = f(z["kc0"]).reshape(hist, kvh * 256)
    vc[:hist] = f(z["vc0"]).reshape(hist, kvh * 256)
    out, _ = O.mixer(q[None], k[None], v[None], gate[None], kc, vc, [hist], kv_heads=kvh)
    assert np.abs(kc[hist:] - z["k_rows"]).max() < 2e-4, "normalised, rotated K rows"
    assert np.abs(out - z["out"]).max() < 2e-4 and rel_l2(out, z["out"]) < 1e-4


def test_verify_rows_equal_sequential_decode():
    """A verify batch of B rows gives what B single-token decode steps give: the property the
    reference's end-to-end spec test relies on (test/test_spec.cu:64-98)."""
    c = Case(3, [50], 4, kv_heads=1)
    out_b, lse_b, kc_b, _ = c.oracle()
    kc, vc = c.kc0.copy(), c.vc0.copy()
    for b in range(4):
        o, l = O.mixer(c.q[:, b:b + 1], c.k[:, b:b + 1], c.v[:, b:b + 1], c.gate[:, b:b + 1], kc, vc,
                       c.hist + b, c.cache_row, kv_heads=1)
        assert np.array_equal(o[0], out_b[b]) and np.array_equal(l[0], lse_b[b])
    assert np.array_equal(kc, kc_b)


def test_chunked_prefill_equals_single_shot():
    """Prefilling in chunks that append to the cache equals one shot (src/prefill.cu:231-240)."""
    c = Case(4, [0], 48, kv_heads=1, gate=True)
    out1, lse1, kc1, vc1 = c.oracle()
    kc, vc = c.kc0.copy(), c.vc0.copy()
    outs = []
    for t0 in range(0, 48, 16):
        o, _ = O.mixer(c.q[:, t0:t0 + 16], c.k[:, t0:t0 + 16], c.v[:, t0:t0 + 16], c.gate[:, t0:t0 + 16], kc, vc,
                       [t0], c.cache_row, kv_heads=1)
        outs.append(o)
    assert np.array_equal(np.concatenate(outs), out1)
    assert np.array_equal(kc, kc1) and np.array_equal(vc, vc1)


def test_row_subset_and_fp32_cache():
    c = Case(5, [20, 7], 3, kv_heads=2)
    out, lse, _, _ = c.oracle()
    sub, lsub, _, _ = c.oracle(rows=[4, 1])
    assert np.array_equal(sub[0], out[4]) and np.array_equal(sub[1], out[1]) and np.array_equal(lsub[1], lse[1])
    # reference-literal fp32 cache: same maths, K not rounded on store
    kc = O.bf16_bits_to_f32(c.kc0)
    vc = O.bf16_bits_to_f32(c.vc0)
    o32, _ = O.mixer(c.q, c.k, c.v, c.gate, kc, vc, c.hist, c.cache_row, kv_heads=2)
    assert 0 < rel_l2(o32, out) < 5e-3


def test_rope_and_gate_helpers():
    rng = np.random.default_rng(6)
    v = rng.standard_normal((3, 2, 256)).astype(np.float32)
    r = O.rope_f32(v.copy(), 100)
    inv = 1e7 ** (-2.0 * np.arange(32) / 64.0)
    for b in range(3):
        a = (100 + b) * inv
        want0 = v[b, :, :32] * np.cos(a) - v[b, :, 32:64] * np.sin(a)
        want1 = v[b, :, :32] * np.sin(a) + v[b, :, 32:64] * np.cos(a)
        assert np.abs(r[b, :, :32] - want0).max() < 1e-6 and np.abs(r[b, :, 32:64] - want1).max() < 1e-6
    assert np.array_equal(r[:, :, 64:], v[:, :, 64:])
    # norm is preserved by a rotation
    assert np.allclose((r[..., :64] ** 2).sum(-1), (v[..., :64] ** 2).sum(-1), rtol=1e-5)
    x = rng.standard_normal(64).astype(np.float32)
    g = rng.standard_normal(64).astype(np.float32)
    assert np.allclose(O.gate_sigmoid_f32(x.copy(), g), x / (1 + np.exp(-g.astype(np.float64))), atol=1e-6)

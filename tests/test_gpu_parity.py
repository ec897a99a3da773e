"""Parity of the CUDA path against the CPU oracle, through the C ABI.  Needs a B200."""
import numpy as np
import pytest
import torch

from oracle import pyoracle as O
from qwengine_b200 import api
from tests.gpu_util import dev_bf16, dev_bits, host_bits, host_f32, run_case
from tests.util import Case, bf16_exact, check_lse, check_out, check_out_bf16, rel_l2

pytestmark = pytest.mark.gpu


def _full_check(c, what):
    ref, lse_ref, kc_ref, vc_ref = c.oracle()
    o32, lse, kc, vc, _ = run_case(c, out_f32=True)
    assert np.array_equal(kc, kc_ref), what + ": appended K rows differ from the oracle (bit-exact expected)"
    assert np.array_equal(vc, vc_ref), what + ": appended V rows differ"
    check_out(o32, ref, what + " fp32 out")
    check_lse(lse, lse_ref, what)
    o16, lse16, _, _, _ = run_case(c, out_f32=False)
    check_out_bf16(o16, ref, what + " bf16 out")
    # the bf16 output is the rounding of the fp32 output
    assert np.array_equal(O.f32_to_bf16_bits(o32), O.f32_to_bf16_bits(o16))
    assert np.array_equal(lse, lse16)


# ---- small kernels ---------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("pos0,B,use_mpos", [(0, 1, False), (8192, 4, False), (131071, 3, False), (17, 5, True)])
def test_rope(dtype, pos0, B, use_mpos):
    rng = np.random.default_rng(1)
    v = bf16_exact(rng, (B, 24, 256))
    mpos = None
    if use_mpos:
        t = pos0 + np.arange(B)
        mpos = np.stack([t, t + 2, 3 * t], -1).astype(np.int32)
    ref = O.rope_f32(v.copy(), pos0, mpos=mpos)
    t = torch.from_numpy(v).cuda().to(dtype)
    dpos = torch.tensor([pos0], dtype=torch.int32, device="cuda")
    api.rope(t, 24, 256, 64, dpos, 1e7, B=B, mpos=None if mpos is None else torch.from_numpy(mpos).cuda())
    got = host_f32(t)
    if dtype == torch.float32:
        assert np.abs(got - ref).max() <= 2e-7 * max(1.0, np.abs(ref).max())
    else:
        assert np.array_equal(O.f32_to_bf16_bits(got), O.f32_to_bf16_bits(ref))
    assert np.array_equal(got[..., 64:], v[..., 64:])


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_kv_append(dtype):
    rng = np.random.default_rng(2)
    B, ctx, pos0 = 5, 64, 37
    k, v = bf16_exact(rng, (B, 1024)), bf16_exact(rng, (B, 1024))
    kc = torch.zeros(ctx, 1024, dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros_like(kc)
    dpos = torch.tensor([pos0], dtype=torch.int32, device="cuda")
    api.kv_append(torch.from_numpy(k).cuda().to(dtype), torch.from_numpy(v).cuda().to(dtype), kc, vc, dpos, 1024, B=B)
    want_k = np.zeros((ctx, 1024), np.float32)
    want_k[pos0:pos0 + B] = k
    want_v = np.zeros((ctx, 1024), np.float32)
    want_v[pos0:pos0 + B] = v
    assert np.array_equal(host_f32(kc), want_k) and np.array_equal(host_f32(vc), want_v)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_gate_sigmoid(dtype):
    rng = np.random.default_rng(3)
    x, g = bf16_exact(rng, (3 * 6144,)), bf16_exact(rng, (3 * 6144,))
    ref = O.gate_sigmoid_f32(x.copy(), g)
    t = torch.from_numpy(x).cuda().to(dtype)
    api.gate_sigmoid(t, torch.from_numpy(g).cuda().to(dtype), x.size)
    got = host_f32(t)
    tol = 1e-6 if dtype == torch.float32 else 2 ** -8
    assert np.abs(got - ref).max() <= tol * max(1.0, np.abs(ref).max())


# ---- fused mixer: decode and verify --------------------------------------------------------------------
@pytest.mark.parametrize("hist", [[0], [1], [62], [63], [64], [65], [127, 128, 129], [1000, 3, 517, 64]])
def test_decode_small(hist):
    _full_check(Case(10 + len(hist), hist, 1), "decode hist=%s" % hist)


@pytest.mark.parametrize("n_new", [2, 3, 4, 5, 6, 8])
def test_verify_rows(n_new):
    _full_check(Case(20 + n_new, [300, 61, 0, 1999], n_new), "verify B=%d" % n_new)


@pytest.mark.parametrize("kv_heads", [1, 2])
def test_kv_head_shards(kv_heads):
    _full_check(Case(31, [700, 129], 4, kv_heads=kv_heads), "kv_heads=%d" % kv_heads)


def test_mrope_positions():
    _full_check(Case(32, [40, 7], 3, mrope=True), "mrope")


def test_no_gate_no_lse_and_flags():
    c = Case(33, [200], 2, gate=False)
    ref, _, _, _ = c.oracle(do_gate=False)
    o32, lse, _, _, _ = run_case(c, out_f32=True, lse=False)
    check_out(o32, ref, "no gate")


def test_config2_shape_reduced():
    """BASELINE config 2 at a history the oracle finishes quickly: 16 sequences, 1 query each."""
    _full_check(Case(40, [2048] * 16, 1), "config2-reduced")


@pytest.mark.parametrize("n_seq,hist", [(13, 333), (18, 1), (16, 1000)])
def test_uniform_batches_that_give_every_unit_two_ctas(n_seq, hist):
    """50 to 74 equally long units on 148 SMs: the grid is trimmed to two CTAs per unit (one-tile units leave every
    other CTA without work).  Checked against the oracle and for run-to-run identity."""
    c = Case(43 + n_seq, [hist] * n_seq, 1)
    _full_check(c, "uniform %d x %d" % (n_seq, hist))
    a, b = run_case(c), run_case(c)
    assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1])


@pytest.mark.parametrize("hist", [[5000], [3000, 2000], [40000]])
def test_few_long_sequences_merge_sliced_or_by_the_last_cta(hist):
    """One to four sequences decoding alone: every KV head is cut into eight parts or more and all of its CTAs merge
    it together, a slice of the channels each.  With QW_F_NO_GRID_WAIT the CTA that arrives last merges alone.  Both
    against the oracle; each bit-identical from run to run."""
    c = Case(60 + len(hist), hist, 1)
    _full_check(c, "sliced merge hist=%s" % hist)
    ref, lse_ref, _, _ = c.oracle()
    fl = api.F_ROPE | api.F_APPEND | api.F_GATE | api.F_NO_GRID_WAIT
    a = run_case(c, out_f32=True, flags=fl)
    b = run_case(c, out_f32=True, flags=fl)
    check_out(a[0], ref, "no grid wait")
    check_lse(a[1], lse_ref, "no grid wait")
    assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1])
    s1, s2 = run_case(c, out_f32=True), run_case(c, out_f32=True)
    assert np.array_equal(s1[0], s2[0]) and np.array_equal(s1[1], s2[1])


@pytest.mark.parametrize("hist,n_new", [([6000], 4), ([2500, 4000], 3), ([9000], 12)])
def test_few_long_sequences_with_draft_tokens_both_merge_routes(hist, n_new):
    """The tcgen05 split-KV kernel with few long units: all CTAs of a unit merge it together, or (QW_F_NO_GRID_WAIT)
    the CTA that arrives last does; both against the oracle, each bit-identical from run to run."""
    c = Case(70 + n_new, hist, n_new)
    _full_check(c, "verify, sliced merge hist=%s" % hist)
    ref, lse_ref, _, _ = c.oracle()
    fl = api.F_ROPE | api.F_APPEND | api.F_GATE | api.F_NO_GRID_WAIT
    a = run_case(c, out_f32=True, flags=fl)
    b = run_case(c, out_f32=True, flags=fl)
    assert api.last_attention_kernel() == "splitkv_umma_kernel"
    check_out(a[0], ref, "verify, no grid wait")
    check_lse(a[1], lse_ref, "verify, no grid wait")
    assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1])
    s1, s2 = run_case(c, out_f32=True), run_case(c, out_f32=True)
    assert np.array_equal(s1[0], s2[0]) and np.array_equal(s1[1], s2[1])


def test_config3_shape_reduced():
    """BASELINE config 3 shape: 8 sequences x 4 draft tokens, ragged histories."""
    rng = np.random.default_rng(41)
    _full_check(Case(41, rng.integers(256, 4096, 8).tolist(), 4), "config3-reduced")


def test_bitwise_repeatable():
    c = Case(42, [3000, 500, 64, 9000], 4)
    a = run_case(c)
    b = run_case(c)
    d = run_case(c)
    assert np.array_equal(a[0], b[0]) and np.array_equal(a[0], d[0]) and np.array_equal(a[1], b[1])


def test_stale_rows_beyond_position_are_never_read():
    """Cache rows past a sequence's position hold anything (the reference never clears them,
    src/model.cu:77-79,195-202); NaN patterns there must not leak into the result."""
    c = Case(43, [100, 64], 2, pad_rows=130)
    c.kc0[c.kc0 == 0x4F00] = 0x7FC0  # NaN
    c.vc0[c.vc0 == 0x4F00] = 0x7FC0
    ref, lse_ref, _, _ = c.oracle()
    o32, lse, _, _, _ = run_case(c, out_f32=True)
    assert np.isfinite(o32).all()
    check_out(o32, ref, "stale rows")
    check_lse(lse, lse_ref, "stale rows")


# ---- prefill through the split-KV kernel (short chunks and the forced fallback) ------------------------
@pytest.mark.parametrize("hist,T", [(0, 16), (0, 64), (100, 40), (0, 129)])
def test_prefill_chunk_splitkv(hist, T):
    c = Case(50 + T, [hist], T, kv_heads=2)
    ref, lse_ref, kc_ref, _ = c.oracle()
    o32, lse, kc, _, _ = run_case(c, out_f32=True, flags=api.F_ROPE | api.F_APPEND | api.F_GATE | api.F_NO_UMMA)
    assert np.array_equal(kc, kc_ref)
    check_out(o32, ref, "prefill splitkv")
    check_lse(lse, lse_ref, "prefill splitkv")


# ---- prefill on the tcgen05 kernels (chunks of >= 64 rows) ------------------------------------------------
_FUSED = api.F_ROPE | api.F_APPEND | api.F_GATE


@pytest.mark.parametrize("hist,T,kvh", [([0], 128, 1), ([0], 64, 2), ([0], 256, 1), ([100], 200, 2), ([37], 333, 1),
                                        ([500, 3], 96, 1), ([0], 512, 4), ([1000], 128, 4), ([3000], 640, 1)])
def test_prefill_umma(hist, T, kvh):
    c = Case(55 + T, hist, T, kv_heads=kvh)
    ref, lse_ref, kc_ref, vc_ref = c.oracle()
    o32, lse, kc, vc, mx = run_case(c, out_f32=True, flags=_FUSED)
    assert mx.launches() == 2, "expected rope_append + the tcgen05 kernel"
    assert np.array_equal(kc, kc_ref) and np.array_equal(vc, vc_ref)
    check_out(o32, ref, "prefill umma")
    check_lse(lse, lse_ref, "prefill umma")
    o16, _, _, _, _ = run_case(c, out_f32=False, flags=_FUSED)
    check_out_bf16(o16, ref, "prefill umma bf16")
    assert np.array_equal(O.f32_to_bf16_bits(o32), O.f32_to_bf16_bits(o16))


def test_prefill_umma_fast_p_mode():
    """QW_F_FAST_P drops the bf16 lo pass of P: still inside max-abs, rel-L2 up to ~2e-3 by design."""
    c = Case(57, [700], 384, kv_heads=1)
    ref, lse_ref, _, _ = c.oracle()
    o32, lse, _, _, _ = run_case(c, out_f32=True, flags=_FUSED | api.F_FAST_P)
    assert np.abs(o32 - ref).max() <= 2e-2 and 5e-4 < rel_l2(o32, ref) <= 2.5e-3
    check_lse(lse, lse_ref, "fast p")


def test_prefill_umma_mrope_and_stale_rows():
    """mrope positions, a ragged last tile, and NaN bit patterns in the cache rows past the end."""
    c = Case(58, [70], 130, kv_heads=1, mrope=True, pad_rows=200)
    c.kc0[c.kc0 == 0x4F00] = 0x7FC0
    c.vc0[c.vc0 == 0x4F00] = 0x7FC0
    ref, lse_ref, kc_ref, _ = c.oracle()
    o32, lse, kc, _, _ = run_case(c, out_f32=True, flags=_FUSED)
    n = (70 + 130) * 256
    assert np.array_equal(kc.reshape(-1)[:n], kc_ref.reshape(-1)[:n])
    assert np.isfinite(o32).all()
    check_out(o32, ref, "prefill umma mrope")
    check_lse(lse, lse_ref, "prefill umma mrope")


def test_prefill_umma_bitwise_repeatable():
    c = Case(56, [260], 512, kv_heads=2)
    a = run_case(c, flags=_FUSED)
    b = run_case(c, flags=_FUSED)
    assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1])


def test_chunked_prefill_equals_single_shot_gpu():
    """Config 4 in miniature: 4 chunks of 128 appended to the cache equal one 512-token shot."""
    c = Case(59, [0], 512, kv_heads=1)
    o_full, lse_full, kc_full, vc_full, _ = run_case(c, out_f32=True)
    mx = api.Mixer(1, 128, kv_heads=1)
    kc, vc = dev_bits(c.kc0), dev_bits(c.vc0)
    pos = torch.zeros(1, dtype=torch.int32, device="cuda")
    outs = []
    for t0 in range(0, 512, 128):
        sl = slice(t0, t0 + 128)
        out = torch.empty(1, 128, 6, 256, dtype=torch.float32, device="cuda")
        pos.fill_(t0)
        mx.bind(dev_bf16(c.q[:, sl]), kc, vc, pos, out, k_new=dev_bf16(c.k[:, sl]), v_new=dev_bf16(c.v[:, sl]),
                gate=dev_bf16(c.gate[:, sl]))
        mx.forward()
        torch.cuda.synchronize()
        mx.check_status()
        outs.append(host_f32(out).reshape(128, 6, 256))
    got = np.concatenate(outs)
    assert np.array_equal(host_bits(kc), kc_full)
    # same kernel, same tile order per row => identical bits
    assert np.array_equal(got, o_full)


# ---- drop-in launchers with the reference's argument lists ------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("B", [1, 4, 8])
def test_dropin_sequence_like_model_cu(dtype, B):
    """rope(q), rope(k), k_kv_append, k_attn_decode, k_gate_sigmoid in the order of
    src/model.cu:228-240, one sequence, device-resident position."""
    ctx, pos0 = 2048, 777
    c = Case(60 + B, [pos0], B, pad_rows=ctx - pos0 - B)
    ref, _, kc_ref, vc_ref = c.oracle()
    q = torch.from_numpy(c.q[0]).cuda().to(dtype)
    k = torch.from_numpy(c.k[0]).cuda().to(dtype)
    v = torch.from_numpy(c.v[0]).cuda().to(dtype)
    gate = torch.from_numpy(c.gate[0]).cuda().to(dtype)
    kc, vc = dev_bits(c.kc0), dev_bits(c.vc0)
    dpos = torch.tensor([pos0], dtype=torch.int32, device="cuda")
    out = torch.empty_like(q)
    scratch = torch.empty(B * 24 * ctx, dtype=torch.float32, device="cuda")  # the reference's size
    api.rope(q, 24, 256, 64, dpos, 1e7, B=B)
    api.rope(k, 4, 256, 64, dpos, 1e7, B=B)
    api.kv_append(k, v, kc, vc, dpos, 1024, B=B)
    api.attn_decode(q, kc, vc, out, dpos, 256, 4, 24, 1.0 / 16.0, scratch, ctx, B=B)
    api.gate_sigmoid(out, gate, out.numel())
    torch.cuda.synchronize()
    got = host_f32(out)
    assert np.array_equal(host_bits(kc), kc_ref) and np.array_equal(host_bits(vc), vc_ref)
    if dtype == torch.float32:
        check_out(got, ref, "drop-in f32")
    else:
        # q is rounded to bf16 after RoPE and the attention output before the gate: two extra
        # roundings the fused path does not have
        assert np.abs(got - ref).max() <= 2e-2 and rel_l2(got, ref) <= 4e-3


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("B", [1, 4, 8])
def test_dropin_decode_uses_no_more_scratch_than_documented(dtype, B):
    """The decode launcher may use B * q_heads * ctx floats of scratch (what the reference's kernel needs at the
    same launch) and not one more: sentinel words behind that size stay untouched."""
    ctx, pos0 = 1024, 900
    c = Case(65 + B, [pos0], B, pad_rows=ctx - pos0 - B)
    _, _, kc_ref, vc_ref = c.oracle()
    q = torch.from_numpy(c.q[0]).cuda().to(dtype)
    kc, vc = dev_bits(kc_ref), dev_bits(vc_ref)
    dpos = torch.tensor([pos0], dtype=torch.int32, device="cuda")
    out = torch.empty_like(q)
    n = api.attn_decode_scratch_floats(24, 4, ctx, B)
    assert n == B * 24 * ctx
    guard = 1 << 20
    scratch = torch.full((n + guard,), -7.25, dtype=torch.float32, device="cuda")
    api.attn_decode(q, kc, vc, out, dpos, 256, 4, 24, 1.0 / 16.0, scratch, ctx, B=B)
    torch.cuda.synchronize()
    assert bool((scratch[n:] == -7.25).all()), "the launcher wrote past the documented scratch size"
    assert bool(torch.isfinite(out.float()).all())
    want = "splitkv_umma_kernel" if (dtype == torch.bfloat16 and B >= 2) else "splitkv_kernel"
    assert api.last_attention_kernel() == want


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("pos0,B,ctx", [(0, 1, 1), (5, 1, 45), (30, 3, 45), (0, 8, 8), (150, 8, 200), (299, 1, 300)])
def test_dropin_decode_with_a_cache_of_a_few_rows(dtype, pos0, B, ctx):
    """The reference sizes its cache as prompt + new tokens + 8 rows (src/main.cu:38), so a short run has a score
    buffer of a few hundred floats, less than one set of split-KV partials.  The launcher then keeps the partials
    in the library's own array: the result still matches the oracle and the caller's scratch is not written."""
    c = Case(80 + B + ctx, [pos0], B, pad_rows=ctx - pos0 - B)
    ref, _, kc_ref, vc_ref = c.oracle(do_gate=False)
    q = torch.from_numpy(c.q[0]).cuda().to(dtype)
    k = torch.from_numpy(c.k[0]).cuda().to(dtype)
    v = torch.from_numpy(c.v[0]).cuda().to(dtype)
    kc, vc = dev_bits(c.kc0), dev_bits(c.vc0)
    dpos = torch.tensor([pos0], dtype=torch.int32, device="cuda")
    out = torch.full_like(q, float("nan"))
    n = api.attn_decode_scratch_floats(24, 4, ctx, B)
    assert n == B * 24 * ctx
    scratch = torch.full((n + 4096,), -7.25, dtype=torch.float32, device="cuda")
    api.rope(q, 24, 256, 64, dpos, 1e7, B=B)
    api.rope(k, 4, 256, 64, dpos, 1e7, B=B)
    api.kv_append(k, v, kc, vc, dpos, 1024, B=B)
    api.attn_decode(q, kc, vc, out, dpos, 256, 4, 24, 1.0 / 16.0, scratch, ctx, B=B)
    torch.cuda.synchronize()
    assert api.last_attention_kernel() == "splitkv_kernel"
    assert bool((scratch == -7.25).all()), "the launcher wrote into a scratch it had judged too small"
    assert np.array_equal(host_bits(kc), kc_ref) and np.array_equal(host_bits(vc), vc_ref)
    got = host_f32(out)
    if dtype == torch.float32:
        check_out(got, ref, "drop-in decode, short cache, f32")
    else:
        assert np.abs(got - ref).max() <= 2e-2 and rel_l2(got, ref) <= 4e-3


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("pos0,T,ctx", [(0, 5, 45), (0, 40, 80), (7, 63, 70), (0, 64, 104), (10, 100, 120), (0, 127, 127)])
def test_dropin_prefill_with_a_reference_sized_scratch_in_a_small_cache(dtype, pos0, T, ctx):
    """The prefill launcher is not told the size of its scratch.  A caller that kept the reference's allocation
    (T * q_heads * ctx floats, src/prefill.cu:75) has, in a cache of a few rows, less than the split-KV partials of a
    short chunk or (fp32, T >= 64, ctx < 128) the bf16 copy of q need: the launcher must then not write into it."""
    c = Case(90 + T + ctx, [pos0], T, pad_rows=ctx - pos0 - T)
    ref, _, kc_ref, vc_ref = c.oracle(do_gate=False)
    q = torch.from_numpy(c.q[0]).cuda().to(dtype)
    k = torch.from_numpy(c.k[0]).cuda().to(dtype)
    v = torch.from_numpy(c.v[0]).cuda().to(dtype)
    kc, vc = dev_bits(c.kc0), dev_bits(c.vc0)
    dpos = torch.tensor([pos0], dtype=torch.int32, device="cuda")
    out = torch.full_like(q, float("nan"))
    n = T * 24 * ctx                      # the reference's size
    scratch = torch.full((n + (1 << 21),), -7.25, dtype=torch.float32, device="cuda")
    api.rope(q, 24, 256, 64, dpos, 1e7, B=T)
    api.rope(k, 4, 256, 64, dpos, 1e7, B=T)
    api.kv_append(k, v, kc, vc, dpos, 1024, B=T)
    api.attn_prefill(q, kc, vc, out, dpos, 256, 4, 24, 1.0 / 16.0, scratch, ctx, T)
    torch.cuda.synchronize()
    assert bool((scratch[n:] == -7.25).all()), "the launcher wrote past the reference's scratch size"
    assert api.last_attention_kernel() == ("prefill_umma_pair_kernel" if T >= 64 else "splitkv_kernel")
    assert np.array_equal(host_bits(kc), kc_ref) and np.array_equal(host_bits(vc), vc_ref)
    got = host_f32(out)
    assert np.isfinite(got).all()
    assert np.abs(got - ref).max() <= 2e-2 and rel_l2(got, ref) <= 4e-3


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("pos0,T,ctx", [(0, 64, 256), (300, 256, 1024), (1000, 333, 2048)])
def test_dropin_prefill_reaches_the_tcgen05_kernel(dtype, pos0, T, ctx):
    """qw_attn_prefill_* with a chunk of 64 rows or more, as src/prefill.cu:142-154 would call it: rope, append,
    attention (no gate).  The attention is compared with the oracle fed with the very q the kernel got (tight), and
    the whole sequence with the oracle's own fp32 pipeline (the bf16 roundings of this route on top)."""
    c = Case(170 + T, [pos0], T, pad_rows=ctx - pos0 - T)
    ref, _, kc_ref, vc_ref = c.oracle(do_gate=False)
    q = torch.from_numpy(c.q[0]).cuda().to(dtype)
    k = torch.from_numpy(c.k[0]).cuda().to(dtype)
    v = torch.from_numpy(c.v[0]).cuda().to(dtype)
    kc, vc = dev_bits(c.kc0), dev_bits(c.vc0)
    dpos = torch.tensor([pos0], dtype=torch.int32, device="cuda")
    out = torch.full_like(q, float("nan"))
    scratch = torch.empty(api.attn_prefill_scratch_floats(24, 4, ctx, T), dtype=torch.float32, device="cuda")
    api.rope(q, 24, 256, 64, dpos, 1e7, B=T)
    api.rope(k, 4, 256, 64, dpos, 1e7, B=T)
    api.kv_append(k, v, kc, vc, dpos, 1024, B=T)
    api.attn_prefill(q, kc, vc, out, dpos, 256, 4, 24, 1.0 / 16.0, scratch, ctx, T)
    torch.cuda.synchronize()
    assert api.last_attention_kernel() == "prefill_umma_pair_kernel"
    assert np.array_equal(host_bits(kc), kc_ref) and np.array_equal(host_bits(vc), vc_ref)
    got = host_f32(out)
    # (1) attention alone: the oracle on the rotated q as the tensor cores read it (bf16), same cache
    q_seen = host_f32(q.to(torch.bfloat16))[None]
    kcn, vcn = kc_ref.copy(), vc_ref.copy()
    ref_attn, _ = O.mixer(q_seen, None, None, None, kcn, vcn, [pos0], do_rope=False, do_append=False, do_gate=False)
    if dtype == torch.float32:
        check_out(got, ref_attn, "drop-in prefill f32, attention alone")
        # (2) end to end against the fp32 pipeline: q was rounded to bf16 on its way to the tensor cores
        assert np.abs(got - ref).max() <= 2e-2 and rel_l2(got, ref) <= 2e-3
    else:
        check_out_bf16(got, ref_attn, "drop-in prefill bf16, attention alone")
        assert np.abs(got - ref).max() <= 2e-2 and rel_l2(got, ref) <= 4e-3


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_dropin_prefill_like_prefill_cu(dtype):
    ctx, pos0, T = 512, 100, 50
    c = Case(70, [pos0], T, pad_rows=ctx - pos0 - T)
    ref, _, _, _ = c.oracle(do_gate=False)
    q = torch.from_numpy(c.q[0]).cuda().to(dtype)
    k = torch.from_numpy(c.k[0]).cuda().to(dtype)
    v = torch.from_numpy(c.v[0]).cuda().to(dtype)
    kc, vc = dev_bits(c.kc0), dev_bits(c.vc0)
    dpos = torch.tensor([pos0], dtype=torch.int32, device="cuda")
    out = torch.empty_like(q)
    scratch = torch.empty(api.attn_prefill_scratch_floats(24, 4, ctx, T), dtype=torch.float32, device="cuda")
    api.rope(q, 24, 256, 64, dpos, 1e7, B=T)
    api.rope(k, 4, 256, 64, dpos, 1e7, B=T)
    api.kv_append(k, v, kc, vc, dpos, 1024, B=T)
    api.attn_prefill(q, kc, vc, out, dpos, 256, 4, 24, 1.0 / 16.0, scratch, ctx, T)
    torch.cuda.synchronize()
    got = host_f32(out)
    if dtype == torch.float32:
        check_out(got, ref, "drop-in prefill f32")
    else:
        assert np.abs(got - ref).max() <= 2e-2 and rel_l2(got, ref) <= 4e-3


def test_graph_capture_and_replay_advances_with_device_position():
    """The decode launch is legal inside a stream capture and reads its position on the device,
    like the reference's replayed decode graph (src/model.cu:318-327)."""
    ctx = 1024
    c = Case(80, [300], 1, pad_rows=ctx - 301)
    q = dev_bf16(c.q[0])
    kc, vc = dev_bits(c.kc0), dev_bits(c.vc0)
    dpos = torch.tensor([300], dtype=torch.int32, device="cuda")
    out = torch.empty_like(q)
    scratch = torch.empty(24 * ctx, dtype=torch.float32, device="cuda")
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        api.attn_decode(q, kc, vc, out, dpos, 256, 4, 24, 1.0 / 16.0, scratch, ctx, B=1, stream=s)  # warm-up
        s.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            api.attn_decode(q, kc, vc, out, dpos, 256, 4, 24, 1.0 / 16.0, scratch, ctx, B=1, stream=s)
    outs = []
    for p in (300, 150, 299):
        dpos.fill_(p)
        g.replay()
        torch.cuda.synchronize()
        outs.append(host_f32(out).copy())
    for p, got in zip((300, 150, 299), outs):
        cc = Case(80, [300], 1, pad_rows=ctx - 301)
        kcn, vcn = cc.kc0.copy(), cc.vc0.copy()
        ref, _ = O.mixer(cc.q, None, None, None, kcn, vcn, [p], do_rope=False, do_append=False, do_gate=False)
        # row sees keys [0, p]: slot p must hold data, so only p < 300 is meaningful with this cache
        if p < 300:
            assert np.abs(got - ref).max() <= 2e-2 and rel_l2(got, ref) <= 4e-3
    assert not np.array_equal(outs[1], outs[2])


def test_fused_mixer_step_in_a_cuda_graph():
    """The two-launch decode step (append kernel, then the attention kernel launched as its programmatic
    dependent) is capturable and a replay gives the bits of the eager call."""
    c = Case(81, [900, 131, 4000], 1)
    eager, lse_eager, kc_eager, _, _ = run_case(c, out_f32=True)
    mx = api.Mixer(c.n_seq, 1)
    q, k, v, gate = dev_bf16(c.q), dev_bf16(c.k), dev_bf16(c.v), dev_bf16(c.gate)
    kc, vc = dev_bits(c.kc0), dev_bits(c.vc0)
    out = torch.zeros(c.n_seq, 1, 24, 256, dtype=torch.float32, device="cuda")
    lse = torch.zeros(c.n_seq, 1, 24, dtype=torch.float32, device="cuda")
    mx.bind(q, kc, vc, torch.from_numpy(c.hist).cuda(), out, k_new=k, v_new=v, gate=gate, lse=lse,
            cache_row=torch.from_numpy(c.cache_row).cuda())
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        mx.forward(stream=s)  # warm-up: one-time kernel attributes are set outside the capture
        s.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            mx.forward(stream=s)
    out.zero_()
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    mx.check_status()
    assert np.array_equal(host_f32(out).reshape(-1, 24, 256), eager)
    assert np.array_equal(lse.cpu().numpy().reshape(-1, 24), lse_eager)
    assert np.array_equal(host_bits(kc), kc_eager)


@pytest.mark.parametrize("hist,n_new", [([3000, 700], 1), ([2500], 4), ([600], 300)])
def test_growing_logits_force_rescales(hist, n_new):
    """Keys whose scale grows along the sequence (and one late outlier) make the running maximum rise tile after
    tile, so every kernel's deferred rescale of O and l is exercised, far from the N(0,1) comfort zone."""
    c = Case(90 + n_new, hist, n_new)
    for s in range(c.n_seq):
        r0, h = int(c.cache_row[s]), int(c.hist[s])
        k = O.bf16_bits_to_f32(c.kc0[r0:r0 + h])
        ramp = (0.25 + 3.0 * np.arange(h, dtype=np.float32) / max(h, 1))[:, None]
        k = k * ramp
        k[h - 7] *= 3.0  # a late outlier key
        c.kc0[r0:r0 + h] = O.f32_to_bf16_bits(k.astype(np.float32))
    _full_check(c, "growing logits")


@pytest.mark.parametrize("n_new", [1, 3])
def test_many_short_sequences_per_cta(n_new):
    """Far more units than CTAs: every CTA walks through many whole units (and shares at most its first and its
    last with a neighbour), which exercises the unit-change path and the ring phases of both split-KV kernels."""
    rng = np.random.default_rng(95)
    hist = rng.integers(0, 700, 311).tolist()
    hist[5], hist[77] = 0, 1
    _full_check(Case(95 + n_new, hist, n_new), "many short sequences")


@pytest.mark.parametrize("n_new", [10, 11, 21, 22, 63])
def test_short_chunks_all_tile_layouts(n_new):
    """Chunk lengths around the row-tile limits of the tcgen05 split-KV kernel: 10 / 11 tokens (60 / 66 rows: the
    64- and 128-row Q tiles), 21 (126 rows, one block) and 22, 63 (two and three blocks per sequence and KV head)."""
    _full_check(Case(120 + n_new, [513, 64, 1290], n_new, kv_heads=2), "chunk of %d" % n_new)


# ---- a launch that finds the status word already set leaves at once --------------------------------------
@pytest.mark.parametrize("hist,n_new", [([900, 70], 4), ([300], 256)])
def test_launch_with_status_word_already_set_does_nothing(hist, n_new):
    """After a kernel has reported a failure through the status word, later launches that share the word must not
    keep the GPU busy with further waits: the tcgen05 kernels read it first and leave (no output, no hang)."""
    c = Case(180 + n_new, hist, n_new)
    mx = api.Mixer(c.n_seq, n_new)
    kc, vc = dev_bits(c.kc0), dev_bits(c.vc0)
    out = torch.full((c.n_seq, n_new, 24, 256), 3.0, dtype=torch.float32, device="cuda")
    mx.bind(dev_bf16(c.q), kc, vc, torch.from_numpy(c.hist).cuda(), out, k_new=dev_bf16(c.k), v_new=dev_bf16(c.v),
            gate=dev_bf16(c.gate), cache_row=torch.from_numpy(c.cache_row).cuda())
    mx.status.fill_(103)
    mx.forward()
    torch.cuda.synchronize()
    assert api.last_attention_kernel() in ("splitkv_umma_kernel", "prefill_umma_pair_kernel")
    assert int(mx.status.item()) == 103
    assert bool((out == 3.0).all()), "a launch that found the status word set still wrote output"
    with pytest.raises(api.QwError):
        mx.check_status()
    # cleared, the same call goes through
    mx.status.zero_()
    kc2, vc2 = dev_bits(c.kc0), dev_bits(c.vc0)
    mx.bind(dev_bf16(c.q), kc2, vc2, torch.from_numpy(c.hist).cuda(), out, k_new=dev_bf16(c.k), v_new=dev_bf16(c.v),
            gate=dev_bf16(c.gate), cache_row=torch.from_numpy(c.cache_row).cuda())
    mx.forward()
    torch.cuda.synchronize()
    mx.check_status()
    ref, _, _, _ = c.oracle()
    check_out(host_f32(out).reshape(-1, 24, 256), ref, "after clearing the status word")


@pytest.mark.parametrize("seed", [11, 12])
def test_seeded_random_shapes_against_the_oracle(seed):
    """Forty seeded draws of (sequences, new tokens, KV heads, histories, M-RoPE, QW_F_NO_GRID_WAIT) through the fused
    call: appended rows bit-exact, output and LSE within the stated tolerance, and a second run bit-identical.  The
    draws reach both split-KV kernels and every merge route (direct, bulk, row, sliced)."""
    rng = np.random.default_rng(seed)
    kernels = set()
    for _ in range(40):
        n_seq = int(rng.choice([1, 1, 2, 3, 4, 7, 16]))
        n_new = int(rng.choice([1, 1, 1, 2, 4, 5, 6, 12, 21, 40, 63]))
        kvh = int(rng.choice([4, 4, 2, 1]))
        top = int(rng.choice([300, 3000, 12000])) if n_seq <= 4 else int(rng.choice([300, 2000]))
        hist = rng.integers(0, top, n_seq).tolist()
        if n_seq * (max(hist) + n_new) * n_new > 1.5e6:  # keeps the oracle to a fraction of a second
            hist = [h % 1500 for h in hist]
        flags = api.F_ROPE | api.F_APPEND | api.F_GATE | api.F_NO_GRID_WAIT if rng.random() < 0.3 else None
        c = Case(int(rng.integers(1 << 30)), hist, n_new, kv_heads=kvh, mrope=bool(rng.random() < 0.2))
        what = "n_seq=%d n_new=%d kv_heads=%d hist=%s flags=%s" % (n_seq, n_new, kvh, hist, flags)
        ref, lse_ref, kc_ref, vc_ref = c.oracle()
        o, lse, kc, vc, _ = run_case(c, out_f32=True, flags=flags)
        assert np.array_equal(kc, kc_ref) and np.array_equal(vc, vc_ref), what
        check_out(o, ref, what)
        check_lse(lse, lse_ref, what)
        again = run_case(c, out_f32=True, flags=flags)
        assert np.array_equal(o, again[0]) and np.array_equal(lse, again[1]), "not repeatable: " + what
        kernels.add(api.last_attention_kernel())
    assert kernels == {"splitkv_kernel", "splitkv_umma_kernel"}

"""Generates tests/golden/hf_*.npz: golden vectors for the gated-attention mixer computed with the
Hugging Face Qwen3.5 attention functions (the module the reference engine cites as its source,
src/mixers.cu:19-20,381,652), evaluated in float64.

Only these transformers functions do the arithmetic: apply_rotary_pos_emb (rotate_half pairing),
Qwen3_5TextRotaryEmbedding.apply_interleaved_mrope (which position component each frequency slot
uses), eager_attention_forward (GQA repeat, scaling, mask, softmax, PV) and torch.sigmoid for the
gate.  Inputs are seeded N(0,1) values rounded to bf16; the cache convention is the B200 one
(K stored post-RoPE, rounded to bf16).  Run from the repo root:
    python tests/golden/make_hf_golden.py
"""
import os
import types

import numpy as np
import torch
from transformers.models.qwen3_5 import modeling_qwen3_5 as hf

HERE = os.path.dirname(os.path.abspath(__file__))
D, ROT, THETA, SCALE = 256, 64, 1e7, 1.0 / 16.0


def bf16_round(t):
    return t.to(torch.bfloat16).to(torch.float64)


def bits(t):
    return t.to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)


def cos_sin(pos3):
    """pos3: [3, T] integer positions (t, h, w).  Returns cos, sin [1, T, ROT] in float64."""
    inv_freq = 1.0 / (THETA ** (torch.arange(0, ROT, 2, dtype=torch.float64) / ROT))
    freqs = pos3.to(torch.float64)[:, None, :, None] * inv_freq[None, None, None, :]  # [3, 1, T, 32]
    freqs = hf.Qwen3_5TextRotaryEmbedding.apply_interleaved_mrope(None, freqs, [11, 11, 10])
    emb = torch.cat((freqs, freqs), dim=-1)
    return emb.cos(), emb.sin()


def case(name, seed, kv_heads, hist, n_new, mrope):
    g = torch.Generator().manual_seed(seed)
    Hq = 6 * kv_heads
    q = bf16_round(torch.randn(n_new, Hq, D, generator=g))
    k = bf16_round(torch.randn(n_new, kv_heads, D, generator=g))
    v = bf16_round(torch.randn(n_new, kv_heads, D, generator=g))
    gate = bf16_round(torch.randn(n_new, Hq, D, generator=g))
    kc0 = bf16_round(torch.randn(hist, kv_heads, D, generator=g))
    vc0 = bf16_round(torch.randn(hist, kv_heads, D, generator=g))
    if mrope:
        t = torch.arange(hist, hist + n_new)
        pos3 = torch.stack([t, t // 3 + 5, (t * 7) % 11])
    else:
        t = torch.arange(hist, hist + n_new)
        pos3 = torch.stack([t, t, t])
    cos, sin = cos_sin(pos3)
    # HF layout [batch, heads, seq, dim]
    qh, kh = q.transpose(0, 1)[None], k.transpose(0, 1)[None]
    q_rot, k_rot = hf.apply_rotary_pos_emb(qh, kh, cos, sin)
    q_rot = q_rot.to(torch.float32).to(torch.float64)  # the mixer holds rotated q in fp32
    k_rot = bf16_round(k_rot.to(torch.float32))        # and stores rotated k as bf16
    keys = torch.cat([kc0.transpose(0, 1)[None], k_rot], dim=2)
    vals = torch.cat([vc0.transpose(0, 1)[None], v.transpose(0, 1)[None]], dim=2)
    L = hist + n_new
    mask = torch.full((n_new, L), float("-inf"), dtype=torch.float64)
    for b in range(n_new):
        mask[b, : hist + b + 1] = 0.0
    module = types.SimpleNamespace(num_key_value_groups=6, training=False)
    attn, _ = hf.eager_attention_forward(module, q_rot, keys, vals, mask[None, None], scaling=SCALE)
    out = attn[0] * torch.sigmoid(gate)  # [n_new, Hq, D]
    scores = torch.matmul(q_rot, hf.repeat_kv(keys, 6).transpose(2, 3)) * SCALE + mask[None, None]
    lse = torch.logsumexp(scores, dim=-1)[0].transpose(0, 1)  # [n_new, Hq]
    np.savez(os.path.join(HERE, name + ".npz"),
             kv_heads=kv_heads, hist=hist, n_new=n_new,
             q=bits(q), k=bits(k), v=bits(v), gate=bits(gate), kc0=bits(kc0), vc0=bits(vc0),
             mpos=pos3.t().contiguous().numpy().astype(np.int32) if mrope else np.zeros((0, 3), np.int32),
             k_rot=bits(k_rot[0].transpose(0, 1)), out=out.to(torch.float32).numpy(),
             lse=lse.to(torch.float32).numpy())


if __name__ == "__main__":
    case("hf_prefill_text", 11, 1, 0, 16, False)
    case("hf_verify_hist", 12, 1, 37, 3, False)
    case("hf_mrope", 13, 1, 9, 12, True)
    case("hf_decode_4kv", 14, 4, 130, 1, False)
    print("wrote", sorted(f for f in os.listdir(HERE) if f.endswith(".npz")))

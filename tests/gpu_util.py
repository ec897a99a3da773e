"""GPU-side glue for the parity tests: moves a tests.util.Case to the device and calls the C ABI."""
import numpy as np
import torch

from oracle import pyoracle as O
from qwengine_b200 import api


def dev_bf16(a_f32):
    """float32 numpy (bf16-exact) -> bf16 CUDA tensor."""
    return torch.from_numpy(np.ascontiguousarray(a_f32)).cuda().to(torch.bfloat16)


def dev_bits(a_u16):
    """uint16 bf16 bit patterns -> bf16 CUDA tensor."""
    return torch.from_numpy(np.ascontiguousarray(a_u16).view(np.int16)).cuda().view(torch.bfloat16)


def host_bits(t_bf16):
    return t_bf16.view(torch.int16).cpu().numpy().view(np.uint16)


def host_f32(t):
    return t.float().cpu().numpy()


def run_case(c, out_f32=False, flags=None, lse=True):
    """Runs the fused mixer on Case c.  Returns (out fp32 numpy, lse numpy, kc bits, vc bits, mixer)."""
    mx = api.Mixer(c.n_seq, c.n_new, kv_heads=c.kv_heads)
    q, k, v = dev_bf16(c.q), dev_bf16(c.k), dev_bf16(c.v)
    gate = dev_bf16(c.gate) if c.gate is not None else None
    kc, vc = dev_bits(c.kc0), dev_bits(c.vc0)
    pos = torch.from_numpy(c.hist).cuda()
    crow = torch.from_numpy(c.cache_row).cuda()
    mpos = torch.from_numpy(c.mpos).cuda() if c.mpos is not None else None
    out = torch.full((c.n_seq, c.n_new, c.q_heads, 256), float("nan"),
                     dtype=torch.float32 if out_f32 else torch.bfloat16, device="cuda")
    lse_t = torch.full((c.n_seq, c.n_new, c.q_heads), float("nan"), dtype=torch.float32, device="cuda") if lse else None
    kw = {} if flags is None else {"flags": flags}
    mx.bind(q, kc, vc, pos, out, k_new=k, v_new=v, gate=gate, lse=lse_t, cache_row=crow, mpos=mpos, **kw)
    mx.forward()
    torch.cuda.synchronize()
    mx.check_status()
    return (host_f32(out).reshape(-1, c.q_heads, 256), None if lse_t is None else lse_t.cpu().numpy().reshape(-1, c.q_heads),
            host_bits(kc), host_bits(vc), mx)

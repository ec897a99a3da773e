"""ctypes binding of libqwengine_attn.so plus thin torch conveniences.

The functions mirror the reference engine's launch sites by name and argument order
(rope, kv_append, attn_decode, attn_prefill, gate_sigmoid: reference src/elem.cu:255,
src/mixers.cu:416/436/546/653) and add the fused batched mixer.  torch is used only to
hold device memory and streams; every computation happens inside the CUDA library, and
there is no fallback: a missing or unloadable library raises.
"""
import ctypes as C
import os
import shutil

import torch

from . import build as _build

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libqwengine_attn.so")

QW_OK = 0
F_ROPE, F_APPEND, F_GATE, F_OUT_F32, F_NO_UMMA, F_FAST_P, F_NO_CAUSAL, F_NO_ATTENTION, F_NO_GRID_WAIT = 1, 2, 4, 8, 16, 32, 128, 256, 512
PARTIAL_FLOATS = 260
HEAD_DIM, ROTARY_DIM, GROUP = 256, 64, 6

_vp, _i, _f = C.c_void_p, C.c_int, C.c_float


class MixerDesc(C.Structure):
    _fields_ = [
        ("n_seq", _i), ("n_new", _i), ("q_heads", _i), ("kv_heads", _i), ("head_dim", _i),
        ("rotary_dim", _i), ("theta", _f), ("scale", _f), ("flags", _i),
        ("q", _vp), ("k_new", _vp), ("v_new", _vp), ("gate", _vp), ("out", _vp), ("lse", _vp),
        ("kc", _vp), ("vc", _vp), ("cache_rows", C.c_int64), ("cache_row", _vp), ("pos", _vp),
        ("mpos", _vp), ("workspace", _vp), ("workspace_bytes", C.c_size_t), ("status", _vp),
        ("block_table", _vp), ("block_table_stride", _i), ("page_rows", _i), ("q_pos", _vp),
    ]


# name -> (restype, argtypes); the list doubles as the symbol inventory checked by the tests.
_SIGS = {
    "qw_strerror": (C.c_char_p, [_i]),
    "qw_abi_version": (_i, []),
    "qw_last_cuda_error": (C.c_char_p, []),
    "qw_last_launch_count": (_i, []),
    "qw_last_attention_kernel": (C.c_char_p, []),
    "qw_profile_enable": (_i, [_i]),
    "qw_profile_last_kernel_ms": (_i, [C.POINTER(C.c_float)]),
    "qw_rope_bf16": (_i, [_vp, _i, _i, _i, _vp, _f, _vp, _i, _vp]),
    "qw_rope_f32": (_i, [_vp, _i, _i, _i, _vp, _f, _vp, _i, _vp]),
    "qw_kv_append_bf16": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _vp]),
    "qw_kv_append_f32": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _vp]),
    "qw_attn_decode_bf16": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _f, _vp, _i, _i, _vp]),
    "qw_attn_decode_f32": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _f, _vp, _i, _i, _vp]),
    "qw_attn_decode_bf16_noalloc": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _f, _i, _i, _vp]),
    "qw_attn_decode_scratch_floats": (C.c_size_t, [_i, _i, _i, _i]),
    "qw_attn_prefill_bf16": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _f, _vp, _i, _i, _vp]),
    "qw_attn_prefill_f32": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _f, _vp, _i, _i, _vp]),
    "qw_attn_prefill_scratch_floats": (C.c_size_t, [_i, _i, _i, _i]),
    "qw_gate_sigmoid_bf16": (_i, [_vp, _vp, _i, _vp]),
    "qw_gate_sigmoid_f32": (_i, [_vp, _vp, _i, _vp]),
    "qw_mixer_workspace_bytes": (C.c_size_t, [C.POINTER(MixerDesc)]),
    "qw_mixer_forward": (_i, [C.POINTER(MixerDesc), _vp]),
    "qw_mixer_forward_partial": (_i, [C.POINTER(MixerDesc), _vp, _vp]),
    "qw_mixer_forward_fused": (_i, [C.POINTER(MixerDesc), _vp, _i, _vp, _vp, _f, _vp]),
    "qw_combine_partials": (_i, [_vp, _i, C.c_int64, _i, _vp, _vp, _vp, _i, _vp]),
    "qw_combine_partials_peer": (_i, [_vp, _vp, _i, _i, _i, C.c_int64, _i, _vp, _vp, _vp, _i, _vp, _vp]),
}

_lib = None


def lib():
    """The loaded C-ABI library.  Builds it when nvcc is available and it is stale; raises if
    it can be neither found nor built -- there is deliberately no other implementation."""
    global _lib
    if _lib is None:
        # build() is a no-op when the library is newer than every source; without a compiler (a box that
        # only received the prebuilt file) the existing library is used as it is
        if shutil.which(os.environ.get("NVCC", "nvcc")) or not os.path.exists(LIB_PATH):
            _build.build()
        l = C.CDLL(LIB_PATH)
        for name, (res, args) in _SIGS.items():
            fn = getattr(l, name)
            fn.restype, fn.argtypes = res, args
        _lib = l
    return _lib


class QwError(RuntimeError):
    pass


def _check(rc):
    if rc != QW_OK:
        l = lib()
        raise QwError("%s [%s]" % (l.qw_strerror(rc).decode(), l.qw_last_cuda_error().decode()))


def _p(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def _stream(stream=None):
    s = stream if stream is not None else torch.cuda.current_stream()
    return C.c_void_p(s.cuda_stream)


def _suffix(t):
    if t.dtype == torch.bfloat16:
        return "bf16"
    if t.dtype == torch.float32:
        return "f32"
    raise TypeError("activations must be bfloat16 or float32")


# ---- per-kernel launchers, named and ordered like the reference's --------------------------------
def rope(v, heads, dim, rot, dpos, theta, stream=None, B=1, mpos=None):
    _check(getattr(lib(), "qw_rope_" + _suffix(v))(_p(v), heads, dim, rot, _p(dpos), theta, _stream(stream), B, _p(mpos)))


def kv_append(k, v, kc, vc, dpos, kvdim, B=1, stream=None):
    _check(getattr(lib(), "qw_kv_append_" + _suffix(k))(_p(k), _p(v), _p(kc), _p(vc), _p(dpos), kvdim, B, _stream(stream)))


def attn_decode(q, kc, vc, out, dpos, dim, kv_heads, q_heads, scale, scratch, ctx, B=1, stream=None):
    _check(getattr(lib(), "qw_attn_decode_" + _suffix(q))(
        _p(q), _p(kc), _p(vc), _p(out), _p(dpos), dim, kv_heads, q_heads, scale, _p(scratch), ctx, B, _stream(stream)))


def attn_decode_noalloc(q, kc, vc, out, dpos, dim, kv_heads, q_heads, scale, ctx, B=1, stream=None):
    """attn_decode without a scratch argument: partials go to an array built into the library
    (bf16 only, B <= 8).  The first call on a device must happen outside stream capture."""
    _check(lib().qw_attn_decode_bf16_noalloc(_p(q), _p(kc), _p(vc), _p(out), _p(dpos), dim, kv_heads, q_heads, scale,
                                             ctx, B, _stream(stream)))


def attn_prefill(q, kc, vc, out, dpos, dim, kv_heads, q_heads, scale, scratch, ctx, T, stream=None):
    _check(getattr(lib(), "qw_attn_prefill_" + _suffix(q))(
        _p(q), _p(kc), _p(vc), _p(out), _p(dpos), dim, kv_heads, q_heads, scale, _p(scratch), ctx, T, _stream(stream)))


def gate_sigmoid(x, gate, n, stream=None):
    _check(getattr(lib(), "qw_gate_sigmoid_" + _suffix(x))(_p(x), _p(gate), n, _stream(stream)))


def attn_decode_scratch_floats(q_heads, kv_heads, ctx, B):
    return lib().qw_attn_decode_scratch_floats(q_heads, kv_heads, ctx, B)


def attn_prefill_scratch_floats(q_heads, kv_heads, ctx, T):
    return lib().qw_attn_prefill_scratch_floats(q_heads, kv_heads, ctx, T)


# ---- fused batched mixer ------------------------------------------------------------------------------
class Mixer:
    """Holds the descriptor and workspace of one fused-mixer call shape so that repeated calls
    (a decode loop, a benchmark) do no host allocation.  Tensors are bf16 on one CUDA device."""

    def __init__(self, n_seq, n_new, kv_heads=4, theta=1e7, scale=1.0 / 16.0, device="cuda"):
        self.n_seq, self.n_new, self.kv_heads, self.q_heads = n_seq, n_new, kv_heads, GROUP * kv_heads
        d = MixerDesc()
        d.n_seq, d.n_new, d.q_heads, d.kv_heads = n_seq, n_new, self.q_heads, kv_heads
        d.head_dim, d.rotary_dim, d.theta, d.scale = HEAD_DIM, ROTARY_DIM, theta, scale
        self.desc = d
        nbytes = lib().qw_mixer_workspace_bytes(C.byref(d))
        self.workspace = torch.empty(nbytes, dtype=torch.uint8, device=device)
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        d.workspace, d.workspace_bytes, d.status = self.workspace.data_ptr(), nbytes, self.status.data_ptr()
        self._keep = None

    def bind_append_only(self, kc, vc, pos, k_new, v_new, cache_row=None, mpos=None, block_table=None, page_rows=0,
                         q_pos=None, rope=True):
        """Descriptor for QW_F_NO_ATTENTION: forward() then only rotates k_new and stores k_new / v_new."""
        d = self.desc
        d.flags = F_APPEND | F_NO_ATTENTION | (F_ROPE if rope else 0)
        d.q = d.gate = d.out = d.lse = None
        d.k_new, d.v_new, d.kc, d.vc = k_new.data_ptr(), v_new.data_ptr(), kc.data_ptr(), vc.data_ptr()
        d.cache_rows = kc.numel() // (self.kv_heads * HEAD_DIM)
        d.cache_row, d.pos, d.mpos = _addr(cache_row), pos.data_ptr(), _addr(mpos)
        d.block_table = _addr(block_table)
        d.block_table_stride = 0 if block_table is None else int(block_table.shape[-1])
        d.page_rows = int(page_rows)
        d.q_pos = _addr(q_pos)
        self._keep = (kc, vc, pos, k_new, v_new, cache_row, mpos, block_table, q_pos)
        return self

    def bind(self, q, kc, vc, pos, out, k_new=None, v_new=None, gate=None, lse=None, cache_row=None,
             mpos=None, flags=F_ROPE | F_APPEND | F_GATE, fused=False, block_table=None, page_rows=0, q_pos=None):
        d = self.desc
        if out.dtype == torch.float32:
            flags |= F_OUT_F32
        if gate is None:
            flags &= ~F_GATE
        if k_new is None and not fused:  # forward_fused() takes k and v from the fused rows
            flags &= ~F_APPEND
        d.flags = flags
        d.q, d.k_new, d.v_new, d.gate = q.data_ptr(), _addr(k_new), _addr(v_new), _addr(gate)
        d.out, d.lse, d.kc, d.vc = out.data_ptr(), _addr(lse), kc.data_ptr(), vc.data_ptr()
        d.cache_rows = kc.numel() // (self.kv_heads * HEAD_DIM)
        d.cache_row, d.pos, d.mpos = _addr(cache_row), pos.data_ptr(), _addr(mpos)
        # paged cache: int32 block table [n_seq, pages per sequence], pages of page_rows (multiple of 128) rows
        d.block_table = _addr(block_table)
        d.block_table_stride = 0 if block_table is None else int(block_table.shape[-1])
        d.page_rows = int(page_rows)
        # absolute position of each sequence's first new row, when pos counts keys of a KV sub-range only
        d.q_pos = _addr(q_pos)
        self._keep = (q, kc, vc, pos, out, k_new, v_new, gate, lse, cache_row, mpos, block_table, q_pos)
        return self

    def forward(self, stream=None):
        _check(lib().qw_mixer_forward(C.byref(self.desc), _stream(stream)))

    def forward_fused(self, fused, q_norm_w, k_norm_w, eps=1e-6, stream=None):
        """The same call fed by the fused q/k/v projection rows [n_seq * n_new, q_heads*512 + 2*kv_heads*256]
        (float32 or bf16): scatter, query/gate de-interleave and per-head RMSNorm with (1 + w) run inside.
        The q and gate tensors given to bind() are overwritten with the normalised query and the gate."""
        assert fused.dtype in (torch.float32, torch.bfloat16) and fused.is_contiguous()
        assert fused.numel() == self.n_seq * self.n_new * (self.q_heads * 2 + 2 * self.kv_heads) * HEAD_DIM
        _check(lib().qw_mixer_forward_fused(C.byref(self.desc), _p(fused), 1 if fused.dtype == torch.float32 else 0,
                                            _p(q_norm_w), _p(k_norm_w), float(eps), _stream(stream)))

    def forward_partial(self, partial, stream=None):
        _check(lib().qw_mixer_forward_partial(C.byref(self.desc), _p(partial), _stream(stream)))

    def launches(self):
        return lib().qw_last_launch_count()

    def check_status(self):
        code = int(self.status.item())
        if code:
            raise QwError("kernel reported device error code %d" % code)


def last_attention_kernel():
    """Name of the attention kernel that the last attention call on this thread launched."""
    return lib().qw_last_attention_kernel().decode()


def profile_enable(on=True):
    _check(lib().qw_profile_enable(1 if on else 0))


def profile_last_kernel_ms():
    ms = C.c_float()
    _check(lib().qw_profile_last_kernel_ms(C.byref(ms)))
    return ms.value


def _addr(t):
    return None if t is None else t.data_ptr()


def combine_partials_peer(part_ptrs, flag_ptrs, rank, n_parts, step, rows, q_heads, out, gate=None, lse=None, status=None,
                          stream=None):
    """Merge with the exchange inside the kernel: part_ptrs / flag_ptrs are int64 CUDA tensors holding this
    process's mappings of every rank's partial buffer and flag word (see qwengine_b200.sharding.PeerExchange)."""
    flags = (F_GATE if gate is not None else 0) | (F_OUT_F32 if out.dtype == torch.float32 else 0)
    _check(lib().qw_combine_partials_peer(_p(part_ptrs), _p(flag_ptrs), rank, n_parts, step, rows, q_heads, _p(gate),
                                          _p(out), _p(lse), flags, _p(status), _stream(stream)))


def combine_partials(parts, n_parts, rows, q_heads, out, gate=None, lse=None, stream=None):
    flags = (F_GATE if gate is not None else 0) | (F_OUT_F32 if out.dtype == torch.float32 else 0)
    _check(lib().qw_combine_partials(_p(parts), n_parts, rows, q_heads, _p(gate), _p(out), _p(lse), flags,
                                     _stream(stream)))

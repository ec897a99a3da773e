"""ctypes loader for the CPU oracle (oracle/attn_oracle.c).  TEST INFRASTRUCTURE ONLY:
imported by tests/, the smoke entry and the benchmark's cpu-baseline leg, never by the
qwengine_b200 package."""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = os.path.join(_HERE, "liboracle.so")


class Geom(C.Structure):
    _fields_ = [("n_seq", C.c_int), ("n_new", C.c_int), ("q_heads", C.c_int), ("kv_heads", C.c_int),
                ("head_dim", C.c_int), ("rotary_dim", C.c_int), ("theta", C.c_double), ("scale", C.c_double),
                ("cache_is_bf16", C.c_int), ("do_rope", C.c_int), ("do_append", C.c_int), ("do_gate", C.c_int)]


_lib = None


def lib():
    global _lib
    if _lib is None:
        src = os.path.join(_HERE, "attn_oracle.c")
        if not os.path.exists(_LIB) or os.path.getmtime(_LIB) < os.path.getmtime(src):
            subprocess.check_call(["make", "-C", _HERE, "liboracle.so"], stdout=subprocess.DEVNULL)
        l = C.CDLL(_LIB)
        l.oracle_mixer.restype = C.c_int
        l.oracle_mixer.argtypes = [C.POINTER(Geom)] + [C.c_void_p] * 10 + [C.c_int64, C.c_void_p, C.c_void_p]
        l.oracle_rope_f32.restype = None
        l.oracle_rope_f32.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_double, C.c_void_p]
        l.oracle_gate_sigmoid_f32.restype = None
        l.oracle_gate_sigmoid_f32.argtypes = [C.c_void_p, C.c_void_p, C.c_int64]
        l.oracle_num_threads.restype = C.c_int
        l.oracle_fused_rows.argtypes = [C.c_void_p, C.c_int64, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p,
                                        C.c_double, C.c_int] + [C.c_void_p] * 4
        l.oracle_fused_rows.restype = None
        l.oracle_set_threads.argtypes = [C.c_int]
        l.oracle_f32_to_bf16.restype = C.c_uint16
        l.oracle_f32_to_bf16.argtypes = [C.c_float]
        l.oracle_bf16_to_f32.restype = C.c_float
        l.oracle_bf16_to_f32.argtypes = [C.c_uint16]
        _lib = l
    return _lib


def _ptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def bf16_bits_to_f32(a):
    """uint16 array of bf16 bit patterns -> float32 array (exact)."""
    return (a.astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16_bits(a):
    """float32 array -> uint16 bf16 bit patterns, round-to-nearest-even (finite inputs)."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    u = u + 0x7FFF + ((u >> 16) & 1)
    return (u >> 16).astype(np.uint16)


def mixer(q, k_new, v_new, gate, kc, vc, pos, cache_row=None, mpos=None, rows=None, kv_heads=4,
          theta=1e7, scale=1.0 / 16.0, rot=64, do_rope=True, do_append=True, do_gate=True):
    """Runs the oracle.  q/k_new/v_new/gate: float32 numpy arrays shaped [n_seq, n_new, heads, dim]
    (already exactly representable in bf16 when they model bf16 inputs).  kc/vc: uint16 (bf16
    cache) or float32 (reference-literal cache) arrays [rows, kv_heads*dim], updated in place.
    Returns (out [n_eval, q_heads, dim] float32, lse [n_eval, q_heads] float32)."""
    n_seq, n_new, q_heads, dim = q.shape
    g = Geom(n_seq, n_new, q_heads, kv_heads, dim, rot, theta, scale, int(kc.dtype == np.uint16),
             int(do_rope), int(do_append), int(do_gate and gate is not None))
    pos = np.ascontiguousarray(pos, dtype=np.int32)
    cache_row = np.zeros(n_seq, np.int64) if cache_row is None else np.ascontiguousarray(cache_row, dtype=np.int64)
    if mpos is not None:
        mpos = np.ascontiguousarray(mpos, dtype=np.int32)
    if rows is not None:
        rows = np.ascontiguousarray(rows, dtype=np.int64)
    n_eval = n_seq * n_new if rows is None else len(rows)
    out = np.empty((n_eval, q_heads, dim), np.float32)
    lse = np.empty((n_eval, q_heads), np.float32)
    q = np.ascontiguousarray(q, np.float32)
    k_new = None if k_new is None else np.ascontiguousarray(k_new, np.float32)
    v_new = None if v_new is None else np.ascontiguousarray(v_new, np.float32)
    gate = None if gate is None else np.ascontiguousarray(gate, np.float32)
    assert kc.flags.c_contiguous and vc.flags.c_contiguous
    rc = lib().oracle_mixer(C.byref(g), _ptr(q), _ptr(k_new), _ptr(v_new), _ptr(gate), _ptr(kc), _ptr(vc),
                            _ptr(pos), _ptr(cache_row), _ptr(mpos), _ptr(rows), n_eval, _ptr(out), _ptr(lse))
    if rc:
        raise RuntimeError("oracle_mixer failed: %d" % rc)
    return out, lse


def fused_rows(fused, q_norm_w, k_norm_w, q_heads=24, kv_heads=4, dim=256, eps=1e-6, round_bf16=True):
    """Fused projection rows [n_rows, q_heads*2*dim + 2*kv_heads*dim] (float32) -> (q, gate, k, v) float32
    arrays [n_rows, heads, dim]: scatter, query/gate de-interleave and per-head RMSNorm with (1 + w);
    q_norm_w / k_norm_w are bf16 bit patterns (uint16) of length dim."""
    fused = np.ascontiguousarray(fused, np.float32)
    n_rows = fused.shape[0]
    assert fused.shape[1] == q_heads * 2 * dim + 2 * kv_heads * dim
    qw = np.ascontiguousarray(q_norm_w, np.uint16)
    kw = np.ascontiguousarray(k_norm_w, np.uint16)
    q = np.empty((n_rows, q_heads, dim), np.float32)
    gate = np.empty((n_rows, q_heads, dim), np.float32)
    k = np.empty((n_rows, kv_heads, dim), np.float32)
    v = np.empty((n_rows, kv_heads, dim), np.float32)
    lib().oracle_fused_rows(_ptr(fused), n_rows, q_heads, kv_heads, dim, _ptr(qw), _ptr(kw), float(eps),
                            int(round_bf16), _ptr(q), _ptr(gate), _ptr(k), _ptr(v))
    return q, gate, k, v


def rope_f32(v, pos0, theta=1e7, rot=64, mpos=None):
    """In-place partial RoPE on float32 v[B, heads, dim]."""
    B, heads, dim = v.shape
    assert v.dtype == np.float32 and v.flags.c_contiguous
    if mpos is not None:
        mpos = np.ascontiguousarray(mpos, dtype=np.int32)
    lib().oracle_rope_f32(_ptr(v), B, heads, dim, rot, int(pos0), theta, _ptr(mpos))
    return v


def gate_sigmoid_f32(x, gate):
    assert x.dtype == np.float32 and gate.dtype == np.float32
    lib().oracle_gate_sigmoid_f32(_ptr(x), _ptr(gate), x.size)
    return x


def num_threads():
    return lib().oracle_num_threads()

"""CPU tests of the C-ABI library: it builds, loads, and exports every declared symbol.
No compute entry point is called here (no GPU)."""
import ctypes
import os
import re

import pytest

from qwengine_b200 import api, build
from tests.conftest import ROOT


def _declared():
    names = set()
    for fn in os.listdir(os.path.join(ROOT, "include")):
        text = open(os.path.join(ROOT, "include", fn)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names |= set(re.findall(r"\b(qw_[a-z0-9_]+)\s*\(", text))
    return names


def test_library_builds_and_exports_every_declared_symbol():
    path = build.build()
    assert os.path.exists(path)
    l = ctypes.CDLL(path)
    declared = _declared()
    assert len(declared) >= 20
    missing = [n for n in sorted(declared) if not hasattr(l, n)]
    assert not missing, "declared in include/ but not exported: %s" % missing
    # the binding covers the same set
    assert declared == set(api._SIGS), (declared ^ set(api._SIGS))


def test_host_only_entry_points():
    l = api.lib()
    assert l.qw_abi_version() == 3
    assert l.qw_strerror(0) == b"ok" and b"geometry" in l.qw_strerror(2)
    assert l.qw_attn_decode_scratch_floats(24, 4, 8192, 1) <= 1 * 24 * 8192
    assert l.qw_attn_decode_scratch_floats(24, 4, 512, 8) <= 8 * 24 * 512


def test_argument_validation_needs_no_gpu():
    l = api.lib()
    assert l.qw_rope_bf16(None, 24, 256, 64, None, 1e7, None, 1, None) == 1       # null pointers
    assert l.qw_gate_sigmoid_f32(None, None, 8, None) == 1
    d = api.MixerDesc()
    assert l.qw_mixer_forward(ctypes.byref(d), None) == 1
    buf = (ctypes.c_float * 16)()
    p = ctypes.cast(buf, ctypes.c_void_p)
    assert l.qw_rope_f32(p, 24, 128, 64, p, 1e7, None, 1, None) == 2               # head_dim 128 unsupported
    assert l.qw_attn_decode_f32(p, p, p, p, p, 256, 3, 18, 0.0625, p, 64, 1, None) == 2   # 3 kv heads
    assert l.qw_attn_decode_f32(p, p, p, p, p, 256, 4, 24, 0.0625, p, 64, 9, None) == 2   # B > 8


def test_header_is_plain_c_and_cpp_mirror_compiles():
    """include/qwengine_attn.h must parse as C99 (the boundary is a C ABI) and the C++ mirror of the
    reference's launchers must compile against it."""
    import shutil
    import subprocess
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    if shutil.which("gcc") is None or shutil.which("g++") is None:
        pytest.skip("no host compiler")
    hdr = os.path.join(root, "include", "qwengine_attn.h")
    subprocess.check_call(["gcc", "-std=c99", "-fsyntax-only", "-x", "c", hdr])
    cuda_inc = "/usr/local/cuda/include"
    if not os.path.isdir(cuda_inc):
        pytest.skip("no CUDA headers for the C++ mirror")
    src = "#include \"%s\"\nint main() { qwengine_b200::Mixer m(1, 1); return m.workspace_bytes() == 0; }\n" % os.path.join(
        root, "qwengine_b200", "csrc", "mixer.hpp")
    subprocess.run(["g++", "-std=c++17", "-fsyntax-only", "-I", os.path.join(root, "include"), "-I", cuda_inc, "-x", "c++", "-"],
                   input=src.encode(), check=True)


def test_workspace_errors_come_before_any_launch():
    """A call that returns QW_ERR_WORKSPACE has enqueued nothing: the workspace is checked in front of the append
    kernel, so a caller may fix the workspace and repeat the call without appending its rows twice.  Needs no GPU:
    the call returns before it touches the CUDA runtime."""
    l = api.lib()
    buf = (ctypes.c_float * 64)()
    p = ctypes.cast(buf, ctypes.c_void_p).value
    d = api.MixerDesc()
    d.n_seq, d.n_new, d.q_heads, d.kv_heads, d.head_dim, d.rotary_dim = 2, 4, 24, 4, 256, 64
    d.theta, d.scale, d.flags = 1e7, 0.0625, api.F_ROPE | api.F_APPEND | api.F_GATE
    d.q = d.k_new = d.v_new = d.gate = d.out = d.kc = d.vc = d.pos = p
    d.cache_rows = 1024
    need = l.qw_mixer_workspace_bytes(ctypes.byref(d))
    assert need > 4096
    for ws, nbytes in ((None, need), (p, 64), (p, 4096), (p + 4, need)):   # missing, tiny, one slot short, misaligned
        d.workspace, d.workspace_bytes = ws, nbytes
        assert l.qw_mixer_forward(ctypes.byref(d), None) == 4
        assert l.qw_last_launch_count() == 0
    # (the drop-in decode launcher has no such error: with a scratch too small for one set of partials it uses the
    # library's own array, tests/test_gpu_parity.py::test_dropin_decode_with_a_cache_of_a_few_rows)


def test_flag_values_of_the_binding_match_the_header():
    """qwengine_b200/api.py repeats the QW_F_* values of include/qwengine_attn.h: they must agree, and no two flags
    may share a bit."""
    text = open(os.path.join(ROOT, "include", "qwengine_attn.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    header = {m.group(1): int(m.group(2)) for m in re.finditer(r"\bQW_F_([A-Z0-9_]+)\s*=\s*(\d+)", text)}
    assert len(header) >= 9
    for name, value in header.items():
        assert getattr(api, "F_" + name) == value, name
    bits = sorted(header.values())
    assert all(v & (v - 1) == 0 for v in bits) and len(set(bits)) == len(bits)

"""The reference's three attention call sites rebuilt in C++ against this library (oracle/callsite_check.cu).

The program includes the reference's own qwen38.h, holds fp32 activations and a device-resident position as the
engine's Runtime does, replaces the inline launches of src/model.cu:228-240 (inside a captured, replayed graph, as
src/model.cu:318-327 runs them), src/mtp.cu:172-179 and src/prefill.cu:142-156 with the C++ mirror of the reference
launchers (qwengine_b200/csrc/mixer.hpp), and compares every site's attention output with the reference's own kernels
rebuilt for sm_100a.  It is compiled where the reference tree is present (oracle/Makefile, into oracle/_ref/) and
travels as a binary; the token-exact end-to-end check of test/test_spec.cu needs the model weights and is not run."""
import os
import subprocess

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BIN = os.path.join(ROOT, "oracle", "_ref", "callsite_check")


def test_reference_call_sites_built_against_the_cpp_mirror():
    if not os.path.exists(BIN):
        pytest.skip("oracle/_ref/callsite_check was not built (it needs the reference tree at build time)")
    from qwengine_b200 import api
    api.lib()                                   # the product library the binary links must be current
    r = subprocess.run([BIN], capture_output=True, text=True, timeout=300)
    print(r.stdout)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "CALLSITE_CHECK ok" in r.stdout
    assert r.stdout.count(" ok") >= 18          # 3 batch sizes x 3 graph replays, 2 x 3 short-run steps, 2 prefill chunks, the summary

"""B200 (sm_100a) implementation of qwengine's gated GQA full-attention mixer.

The product is the C-ABI shared library built from csrc/ (see include/qwengine_attn.h);
`qwengine_b200.api` is its ctypes binding for Python callers and tests.
"""
__all__ = ["api", "build"]

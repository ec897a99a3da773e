"""Builds libqwengine_attn.so (the C-ABI library) in-tree with nvcc for sm_100a.

Usage: python -m qwengine_b200.build [--verbose]
The library has no Python or torch dependency; it links only the CUDA runtime.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libqwengine_attn.so")
SOURCES = ["capi.cu", "prefill_umma2.cu", "splitkv_umma.cu"]


def nvcc_cmd(verbose=False):
    cmd = [
        os.environ.get("NVCC", "nvcc"), "-O3", "-std=c++17",
        "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
        "-Xcompiler", "-fPIC", "-shared",
        "-o", LIB,
    ]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += [os.path.join(CSRC, s) for s in SOURCES]
    return cmd


def needs_build():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    deps.append(os.path.join(HERE, "..", "include", "qwengine_attn.h"))
    return any(os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False):
    """Compiles the library if a source is newer than it.  Safe when several processes (one rank per GPU) call it
    at once: one of them compiles under a file lock into a temporary name and renames it into place, the others
    wait for the lock and find the library up to date."""
    if not force and not needs_build():
        return LIB
    import fcntl
    with open(LIB + ".lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if not force and not needs_build():
                return LIB
            tmp = "%s.%d.tmp" % (LIB, os.getpid())
            cmd = nvcc_cmd(verbose)
            cmd[cmd.index("-o") + 1] = tmp
            r = subprocess.run(cmd, capture_output=True, text=True)
            if verbose or r.returncode:
                sys.stderr.write(r.stdout + r.stderr)
            if r.returncode:
                if os.path.exists(tmp):
                    os.remove(tmp)
                raise RuntimeError("nvcc failed building libqwengine_attn.so")
            os.replace(tmp, LIB)
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)
    return LIB


if __name__ == "__main__":
    build(force=True, verbose="--verbose" in sys.argv)
    print(LIB)

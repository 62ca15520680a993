"""Builds what whole Soliton training steps need on top of this repository's library -- into fullstep/_ref/, which is
not part of the source tree (git-ignored):

    fullstep/_ref/soliton/libsoliton.so           this library's sources + fullstep/ops_dispatch.cpp: all 55 `sl_*`
    fullstep/_ref/soliton/libsoliton_ref_cuda.so  the reference's CUDA backend (a copy of the build in oracle/_ref/)
    fullstep/_ref/soliton/*.pyc                   the reference's Python package, compiled, unmodified
    fullstep/_ref/gpt2.pyc                        the reference's example model and trainer, compiled, unmodified
    fullstep/_ref/reftests/*.pyc                  the reference's own tests, compiled, unmodified

The Python parts need a reference checkout (environment variable SOLITON_REFERENCE): nothing of it is copied as
source, only compiled. Where no checkout is present the existing outputs are used as they are.

    python fullstep/build.py
"""
import os
import py_compile
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
OUT = os.path.join(HERE, "_ref")
PKG = os.path.join(OUT, "soliton")
LIB = os.path.join(PKG, "libsoliton.so")
REFERENCE = os.environ.get("SOLITON_REFERENCE", "/root/reference")
sys.path.insert(0, ROOT)


def _stale(target, sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def build_library(force=False):
    from soliton_b200 import build as b
    sources = [os.path.join(b.CSRC, f) for f in b.SOURCES] + [os.path.join(HERE, "ops_dispatch.cpp")]
    headers = [os.path.join(b.CSRC, f) for f in b.HEADERS]
    if force or _stale(LIB, sources + headers):
        os.makedirs(PKG, exist_ok=True)
        nvcc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
        tmp = LIB + ".tmp"
        subprocess.check_call([nvcc] + b.NVCC_FLAGS + ["-o", tmp] + sources + ["-ldl"])
        os.replace(tmp, LIB)
    return LIB


def build_backend():
    from oracle import build as ob
    src = ob.build_ref(REFERENCE)
    dst = os.path.join(PKG, "libsoliton_ref_cuda.so")
    if src and os.path.exists(src) and _stale(dst, [src]):
        os.makedirs(PKG, exist_ok=True)
        shutil.copyfile(src, dst)
    return dst if os.path.exists(dst) else None


def compile_reference_python():
    """Byte-compiles the reference's package, example and tests where they lie; returns False without a checkout."""
    pkg_src = os.path.join(REFERENCE, "python", "soliton")
    if not os.path.isdir(pkg_src):
        return os.path.exists(os.path.join(PKG, "__init__.pyc"))
    jobs = [(os.path.join(pkg_src, f), os.path.join(PKG, f + "c")) for f in sorted(os.listdir(pkg_src)) if f.endswith(".py")]
    jobs.append((os.path.join(REFERENCE, "examples", "gpt2.py"), os.path.join(OUT, "gpt2.pyc")))
    tests = os.path.join(REFERENCE, "tests")
    jobs += [(os.path.join(tests, f), os.path.join(OUT, "reftests", f + "c")) for f in sorted(os.listdir(tests))
             if f.startswith("test_") and f.endswith(".py")]
    for src, dst in jobs:
        if _stale(dst, [src]):
            os.makedirs(os.path.dirname(dst), exist_ok=True)
            py_compile.compile(src, cfile=dst, dfile=os.path.relpath(src, REFERENCE), doraise=True)
    return True


def _compiled_files():
    found = []
    for base, _, files in os.walk(OUT):
        found += [os.path.join(base, f) for f in files if f.endswith(".pyc") or f.endswith(".pyc.bin")]
    return found


def keep_travel_copies():
    """Tools that ship a source tree tend to leave *.pyc behind; every compiled file also exists as *.pyc.bin."""
    for path in _compiled_files():
        if path.endswith(".pyc") and _stale(path + ".bin", [path]):
            shutil.copyfile(path, path + ".bin")


def ensure_importable():
    """Where only the *.pyc.bin copies arrived, puts the *.pyc files back. Called by everything that imports them."""
    for path in _compiled_files():
        if path.endswith(".pyc.bin") and not os.path.exists(path[:-4]):
            shutil.copyfile(path, path[:-4])
    return os.path.exists(os.path.join(PKG, "__init__.pyc"))


def build(force=False):
    out = build_library(force), build_backend(), compile_reference_python()
    keep_travel_copies()
    return out


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))

"""Build recipe for the test oracle (test infrastructure, not product code).

`build_oracle()`  compiles oracle/oracle.c with gcc into oracle/liboracle.so.
`build_ref()`     compiles the reference's own CUDA backend (core/cuda/kernels.cu, where it lies in the reference
                  checkout, unmodified) with nvcc into oracle/_ref/libsoliton_ref_cuda.so. It exports the
                  reference's `sl_cuda_*` functions, among them `sl_cuda_adamw` and the NCCL calls; the GPU
                  tests use it as the ground truth for bit parity and the benchmark as the same-box GPU baseline.
                  Nothing is copied out of the reference; only the built library lands under oracle/_ref/.

Run as a script to build both:  python oracle/build.py [reference checkout]
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "liboracle.so")
REF_DIR = os.path.join(HERE, "_ref")
REF_SO = os.path.join(REF_DIR, "libsoliton_ref_cuda.so")
DEFAULT_REFERENCE = os.environ.get("SOLITON_REFERENCE", "/root/reference")


def _stale(target, sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def build_oracle(force=False):
    src = os.path.join(HERE, "oracle.c")
    if force or _stale(ORACLE_SO, [src]):
        tmp = ORACLE_SO + ".tmp"
        subprocess.check_call(["gcc", "-O3", "-ffp-contract=off", "-fno-fast-math", "-shared", "-fPIC",
                               "-o", tmp, src, "-lm", "-lpthread"])
        os.replace(tmp, ORACLE_SO)
    return ORACLE_SO


def build_ref(reference=DEFAULT_REFERENCE, force=False):
    """Returns the path of the built reference backend, or None when no reference checkout is present."""
    src = os.path.join(reference, "core", "cuda", "kernels.cu")
    if not os.path.exists(src):
        return REF_SO if os.path.exists(REF_SO) else None
    if force or _stale(REF_SO, [src]):
        os.makedirs(REF_DIR, exist_ok=True)
        cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
        tmp = REF_SO + ".tmp"
        # The reference's Makefile line (Makefile:16-18) with its CUDA_ARCH set for B200, plus the link step
        # its D link line would have done (Makefile:10-13).
        subprocess.check_call([os.path.join(cuda, "bin", "nvcc"), "-O3", "-std=c++17", "-arch=sm_100",
                               "-Xcompiler", "-fPIC", "-shared", "-o", tmp, src,
                               "-lcublas", "-lnccl", "-lnvrtc", "-lcuda"])
        os.replace(tmp, REF_SO)
    return REF_SO


if __name__ == "__main__":
    print(build_oracle())
    print(build_ref(*(sys.argv[1:2] or [DEFAULT_REFERENCE])))

"""Build recipe of libsoliton_b200.so: nvcc, sm_100a only, in-tree output next to this file.

    python -m soliton_b200.build          # build if stale
    python -m soliton_b200.build --force
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libsoliton_b200.so")
SOURCES = ["pool.cpp", "rendezvous.cpp", "dp_kernels.cu", "dp_engine.cu", "api.cu", "fabric_probe.cu", "step_kernels.cu", "attention_kernels.cu", "xent_kernels.cu", "elementwise_kernels.cu"]
HEADERS = ["pool.hpp", "rendezvous.hpp", "dp_types.h", "dp_launch.h", "dp_engine.hpp", "foreign_path.h",
           os.path.join("..", "..", "include", "soliton_b200.h")]
NVCC_FLAGS = ["-std=c++17", "-O3", "-lineinfo", "-gencode", "arch=compute_100a,code=sm_100a",
              "-Xcompiler", "-fPIC", "-shared"]


def stale():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    return any(os.path.getmtime(os.path.join(CSRC, f)) > t for f in SOURCES + HEADERS)


def build(force=False, verbose=False):
    """Compiles the library when a source is newer than it. Returns the library path."""
    if force or stale():
        nvcc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
        tmp = LIB + ".tmp"
        cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-o", tmp] + SOURCES
        subprocess.check_call(cmd, cwd=CSRC)
        os.replace(tmp, LIB)  # running processes keep the old library
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))

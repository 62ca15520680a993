"""Generates tests/golden/config0.npz: the single-rank flat-buffer configuration (1,048,576 parameters,
p ~ N(0, 0.02) seed 0, g ~ N(0, 1e-3) seed 1, m = v = 0, step 1, lr 3e-4, betas (0.9, 0.999), eps 1e-8, wd 0.1)
pushed through the CPU restatement of the reference's host AdamW (oracle/oracle.c: oracle_adamw).

The fixture keeps the SHA-256 of the full p, m, v outputs plus every 1024th element, small enough to commit.
Run from the repository root:  python tests/golden/make_golden.py
"""
import hashlib
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import pyoracle  # noqa: E402
from soliton_b200 import workload  # noqa: E402

N = 1 << 20


def compute():
    p, g = workload.flat_case(N)
    m, v = np.zeros(N, np.float32), np.zeros(N, np.float32)
    h = workload.HYPER
    pyoracle.adamw(p, g, m, v, h["lr"], h["b1"], h["b2"], h["eps"], h["wd"], 1)
    return p, m, v


if __name__ == "__main__":
    p, m, v = compute()
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "config0.npz")
    np.savez(out, n=N, stride=1024, p=p[::1024], m=m[::1024], v=v[::1024],
             sha_p=hashlib.sha256(p.tobytes()).hexdigest(), sha_m=hashlib.sha256(m.tobytes()).hexdigest(),
             sha_v=hashlib.sha256(v.tobytes()).hexdigest())
    print(out, os.path.getsize(out), "bytes")

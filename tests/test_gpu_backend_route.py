"""The backend-level entry points a Soliton build links in place of its own (core/soliton/api.d:47-48,58-62 declares
them; core/cuda/kernels.cu:251-254,756-779 defines the originals): sl_cuda_dp_set_workspace, sl_cuda_adamw,
sl_cuda_nccl_*. Driven the way that build would drive them: device memory that does NOT come from this library's
allocator (plain cudaMalloc), no sl_init_device, in a process of its own."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

SCRIPT = r'''
import ctypes as C, sys
import numpy as np
from oracle import pyoracle
from soliton_b200._C import lib
from tests.cudart import Cudart
eager = int(sys.argv[1])
rt = Cudart()
rt.set_device(0)
if eager:
    assert lib.slb_set_option(b"eager", 1) == 0
ws_bytes = lib.slb_workspace_bytes()
ws = rt.malloc(ws_bytes)
assert lib.sl_cuda_dp_set_workspace(ws, ws_bytes) == 0          # as api.d would after its own pool.alloc
sizes = [5, 2048, 70001, 3 * 2048 + 1]
wds = [0.0, 0.1, 0.1, 0.0]
rng = np.random.default_rng(3)
host = [[(rng.standard_normal(n) * 0.02).astype(np.float32), np.zeros(n, np.float32), np.zeros(n, np.float32)] for n in sizes]
dev = [[rt.malloc(4 * n) for _ in range(4)] for n in sizes]   # p, m, v, g
for d, h in zip(dev, host):
    for ptr, a in zip(d[:3], h):
        rt.h2d(ptr, a)
lr, b1, b2, eps = 3e-4, 0.9, 0.999, 1e-8
for step in (1, 2, 3):
    grads = [(rng.standard_normal(n) * 1e-3).astype(np.float32) for n in sizes]
    for d, g in zip(dev, grads):
        rt.h2d(d[3], g)
    before = lib.slb_get_counter(b"launches")
    for d, n, wd in zip(dev, sizes, wds):
        lib.sl_cuda_adamw(d[0], d[3], d[1], d[2], n, lr, b1, b2, eps, wd, step)
    if not eager:
        lib.slb_flush()                                            # what a deferred build adds before it reads
    launches = lib.slb_get_counter(b"launches") - before
    assert launches == (len(sizes) if eager else 1), launches
    rt.sync()
    for h, g, wd in zip(host, grads, wds):
        pyoracle.adamw(h[0], g, h[1], h[2], lr, b1, b2, eps, wd, step, fma=True)
    for d, h, n in zip(dev, host, sizes):
        for ptr, want in zip(d[:3], h):
            got = np.empty(n, np.float32)
            rt.d2h(got, ptr)
            assert np.array_equal(got, want)
# the small ops around the path at backend level: Sum x^2 (blocking), in-place scale, axpy
g = grads[2]
got = lib.sl_cuda_sumsq(dev[2][3], sizes[2])
assert abs(got - float(np.sum(g.astype(np.float64) ** 2))) <= 1e-12 * got
lib.sl_cuda_scale(dev[2][3], dev[2][3], sizes[2], 0.5)
lib.sl_cuda_axpy(dev[2][3], dev[2][3], sizes[2], 2.0)             # g <- 0.5 g + 2 (0.5 g)
lib.slb_flush()
out = np.empty(sizes[2], np.float32)
rt.d2h(out, dev[2][3])
half = g * np.float32(0.5)
assert np.array_equal(out, half + np.float32(2.0) * half)
assert lib.sl_check(2) == 0
print("route ok")
'''


@pytest.mark.parametrize("eager", [0, 1], ids=["deferred", "eager"])
def test_backend_entry_points_on_memory_from_plain_cudamalloc(built, eager):
    env = dict(os.environ, PYTHONPATH=ROOT)
    r = subprocess.run([sys.executable, "-c", SCRIPT, str(eager)], env=env, cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "route ok" in r.stdout, r.stdout + r.stderr

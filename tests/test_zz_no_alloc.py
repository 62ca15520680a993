"""slb_adamw_step_static: the fused AdamW step for callers that cannot let the library allocate (a host runtime that
owns and plans all device memory, and has given the library no workspace). Its segment table lives in a fixed device
array inside the library. Checked through the C ABI against the regular entry point (sl_adamw), bit for bit, on two
calls in a row that use different tensor lists, so that what the first call left in the shared array is shown not
to matter. Collected last on purpose: a run that stops at the first failure has then already run everything else."""
import ctypes as C

import numpy as np
import pytest

from soliton_b200 import workload
from soliton_b200._C import lib, longs
from tests.gpu_util import CUDA, DevBuf, check_ok, ptr_array, zeros

pytestmark = pytest.mark.gpu
H = workload.HYPER


def static_step(bufs, wds, step):
    """bufs: [(p, g, m, v)] DevBufs."""
    n = len(bufs)
    wd = (C.c_float * n)(*wds)
    return lib.slb_adamw_step_static(n, ptr_array([b[0] for b in bufs]), ptr_array([b[1] for b in bufs]),
                                     ptr_array([b[2] for b in bufs]), ptr_array([b[3] for b in bufs]),
                                     longs([b[0].n for b in bufs]), wd, H["lr"], H["b1"], H["b2"], H["eps"], step)


def pool_stats():
    buf = (C.c_int64 * 7)()
    lib.sl_stats(CUDA, buf)
    return list(buf)


def test_static_step_matches_regular_entry_point_on_two_calls_in_a_row(cuda):
    sizes = [1, 5, 2047, 2048, 2049, 100003, 3 * 2048]
    wds = [0.1, 0.0, 0.1, 0.0, 0.1, 0.1, 0.0]
    rng = np.random.default_rng(31)
    p0 = [(rng.standard_normal(n) * 0.02).astype(np.float32) for n in sizes]
    regular = [(DevBuf(x), None, zeros(x.size), zeros(x.size)) for x in p0]
    static = [(DevBuf(x), None, zeros(x.size), zeros(x.size)) for x in p0]
    # call 1: all seven tensors; call 2: a shorter, reordered list (tensors 5, 0, 3) with new gradients
    for step, picks in ((1, list(range(len(sizes)))), (2, [5, 0, 3])):
        grads = {i: (rng.standard_normal(sizes[i]) * 1e-3).astype(np.float32) for i in picks}
        dg = {i: DevBuf(grads[i]) for i in picks}
        for i in picks:
            r = regular[i]
            lib.sl_adamw(CUDA, r[0].ptr, dg[i].ptr, r[2].ptr, r[3].ptr, sizes[i], H["lr"], H["b1"], H["b2"], H["eps"],
                         wds[i], step)
        check_ok()
        before = pool_stats()
        rc = static_step([(static[i][0], dg[i], static[i][2], static[i][3]) for i in picks], [wds[i] for i in picks], step)
        assert rc == 0
        check_ok()
        assert pool_stats() == before  # not one byte through the allocator
        for i in range(len(sizes)):
            for a, b in ((regular[i][0], static[i][0]), (regular[i][2], static[i][2]), (regular[i][3], static[i][3])):
                np.testing.assert_array_equal(a.get().view(np.uint32), b.get().view(np.uint32))


def test_static_step_rejects_what_does_not_fit_or_make_sense(cuda):
    n = 513
    one = zeros(4)
    arr = ptr_array([one] * n)
    rc = lib.slb_adamw_step_static(n, arr, arr, arr, arr, longs([4] * n), None, 1e-3, 0.9, 0.999, 1e-8, 1)
    assert rc == -2  # the fixed table holds 512 tensors
    arr1 = ptr_array([one])
    assert lib.slb_adamw_step_static(0, arr1, arr1, arr1, arr1, longs([4]), None, 1e-3, 0.9, 0.999, 1e-8, 1) == -1
    assert lib.slb_adamw_step_static(1, arr1, arr1, arr1, arr1, longs([-1]), None, 1e-3, 0.9, 0.999, 1e-8, 1) == -1
    none = (C.c_void_p * 1)()
    assert lib.slb_adamw_step_static(1, none, arr1, arr1, arr1, longs([4]), None, 1e-3, 0.9, 0.999, 1e-8, 1) == -1
    check_ok()


def mem_free():
    free, total = C.c_size_t(), C.c_size_t()
    lib.sl_mem_info(C.byref(free), C.byref(total))
    return free.value


def test_static_step_comes_after_work_the_library_has_recorded_but_not_launched(cuda):
    """An in-place clip scale (sl_scale with x == y) is only recorded until something consumes the gradient. The
    static step must see the scaled gradient, exactly as sl_adamw after the same sl_scale does."""
    n = 70001
    rng = np.random.default_rng(41)
    p0 = (rng.standard_normal(n) * 0.02).astype(np.float32)
    g0 = (rng.standard_normal(n) * 1e-3).astype(np.float32)
    a = (DevBuf(p0), DevBuf(g0), zeros(n), zeros(n))
    b = (DevBuf(p0), DevBuf(g0), zeros(n), zeros(n))
    check_ok()
    lib.sl_scale(CUDA, a[1].ptr, a[1].ptr, n, 0.25)
    lib.sl_adamw(CUDA, a[0].ptr, a[1].ptr, a[2].ptr, a[3].ptr, n, H["lr"], H["b1"], H["b2"], H["eps"], 0.1, 1)
    check_ok()
    lib.sl_scale(CUDA, b[1].ptr, b[1].ptr, n, 0.25)
    assert static_step([b], [0.1], 1) == 0
    check_ok()
    for x, y in zip(a, b):
        np.testing.assert_array_equal(x.get().view(np.uint32), y.get().view(np.uint32))


def test_static_step_unaligned_pointers_empty_tensors_full_table_and_device_memory(cuda):
    rng = np.random.default_rng(43)
    # 4-byte aligned but not 32-byte aligned pointers (the scalar path), and an empty tensor in the middle
    sizes = [3000, 0, 2048 * 2 + 5]
    p0 = [(rng.standard_normal(n) * 0.02).astype(np.float32) for n in sizes]
    g0 = [(rng.standard_normal(n) * 1e-3).astype(np.float32) for n in sizes]
    reg = [(DevBuf(p, skew=1), DevBuf(g, skew=1), zeros(len(p), skew=1), zeros(len(p), skew=1)) for p, g in zip(p0, g0)]
    sta = [(DevBuf(p, skew=1), DevBuf(g, skew=1), zeros(len(p), skew=1), zeros(len(p), skew=1)) for p, g in zip(p0, g0)]
    for r in reg:
        if r[0].n:
            lib.sl_adamw(CUDA, r[0].ptr, r[1].ptr, r[2].ptr, r[3].ptr, r[0].n, H["lr"], H["b1"], H["b2"], H["eps"], 0.1, 1)
    check_ok()
    assert static_step(sta, [0.1] * len(sizes), 1) == 0     # warm call: the array's address is looked up here
    check_ok()
    for r, s in zip(reg, sta):
        for x, y in zip(r, s):
            if x.n:
                np.testing.assert_array_equal(x.get().view(np.uint32), y.get().view(np.uint32))
    # exactly 512 tensors fit; and the driver's free-memory figure does not move across a call
    many = [(zeros(16), DevBuf(np.full(16, 1e-3, np.float32)), zeros(16), zeros(16)) for _ in range(512)]
    check_ok()
    free_before = mem_free()
    assert static_step(many, [0.0] * 512, 1) == 0
    check_ok()
    assert mem_free() == free_before
    want = [np.zeros(16, np.float32), np.full(16, 1e-3, np.float32), np.zeros(16, np.float32), np.zeros(16, np.float32)]
    from oracle import pyoracle
    pyoracle.adamw(want[0], want[1], want[2], want[3], H["lr"], H["b1"], H["b2"], H["eps"], 0.0, 1, fma=True)
    for k in (0, 255, 511):
        np.testing.assert_array_equal(many[k][0].get(), want[0])
        np.testing.assert_array_equal(many[k][3].get(), want[3])


NO_INIT = r'''
import ctypes as C
import numpy as np
from oracle import pyoracle
from soliton_b200._C import lib
from tests.cudart import Cudart
rt = Cudart()
rt.set_device(0)
n = 100003
rng = np.random.default_rng(47)
host = [(rng.standard_normal(n) * 0.02).astype(np.float32), (rng.standard_normal(n) * 1e-3).astype(np.float32),
        np.zeros(n, np.float32), np.zeros(n, np.float32)]
dev = [rt.malloc(4 * n) for _ in range(4)]
for ptr, a in zip(dev, host):
    rt.h2d(ptr, a)
one = lambda x: (C.c_void_p * 1)(x)
for step in (1, 2):
    rc = lib.slb_adamw_step_static(1, one(dev[0]), one(dev[1]), one(dev[2]), one(dev[3]), (C.c_int64 * 1)(n),
                                   (C.c_float * 1)(0.1), 3e-4, 0.9, 0.999, 1e-8, step)
    assert rc == 0, rc
    rt.sync()
    pyoracle.adamw(host[0], host[1], host[2], host[3], 3e-4, 0.9, 0.999, 1e-8, 0.1, step, fma=True)
    for ptr, want in zip((dev[0], dev[2], dev[3]), (host[0], host[2], host[3])):
        got = np.empty(n, np.float32)
        rt.d2h(got, ptr)
        assert np.array_equal(got, want)
print("static ok")
'''


def test_static_step_in_a_process_that_never_initialised_the_library(built):
    """The caller this entry point exists for has given the library neither a device initialisation nor a
    workspace: only its own cudaMalloc memory."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-c", NO_INIT], env=dict(os.environ, PYTHONPATH=root), cwd=root,
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "static ok" in r.stdout, r.stdout + r.stderr

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

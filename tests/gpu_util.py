"""Helpers of the GPU tests: device buffers from the library's own allocator and the sim entry point."""
import ctypes as C

import numpy as np

from soliton_b200._C import lib, longs

CUDA = 2


class DevBuf:
    """A float32 device buffer from sl_alloc, optionally starting `skew` floats into the allocation (to make
    pointers that are 4- but not 16-byte aligned)."""

    def __init__(self, array=None, n=None, skew=0):
        if array is not None:
            array = np.ascontiguousarray(array, np.float32).ravel()
            n = array.size
        self.n, self.skew = int(n), skew
        self.nbytes = (self.n + skew) * 4
        self.base = lib.sl_alloc(CUDA, self.nbytes)
        assert self.base, "device allocation failed"
        self.ptr = self.base + 4 * skew
        if array is not None:
            self.put(array)

    def put(self, array):
        a = np.ascontiguousarray(array, np.float32).ravel()
        assert a.size == self.n
        lib.sl_from_host(CUDA, self.ptr, a.ctypes.data, a.nbytes)

    def get(self):
        out = np.empty(self.n, np.float32)
        lib.sl_to_host(CUDA, out.ctypes.data, self.ptr, out.nbytes)
        return out

    def free(self):
        if self.base:
            lib.sl_free(CUDA, self.base, self.nbytes)
            self.base = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


def zeros(n, skew=0):
    return DevBuf(np.zeros(n, np.float32), skew=skew)


def check_ok():
    lib.sl_sync(CUDA)
    err = lib.sl_check(CUDA)
    assert err == 0, f"sticky error {err}"


def ptr_array(bufs):
    return (C.c_void_p * len(bufs))(*[b.ptr if b is not None else None for b in bufs])


def sim_step(world, ns, p, g, m, v, wd, hyper, step, adam=True, mode=0, blocks_per_rank=0, timeout_ms=0,
             active_mask=None, sumsq=None):
    """p, g, m, v: [rank][segment] DevBuf lists. Returns (rc, [status per rank]). `sumsq`: a float64 array of
    shape (world, segments) that receives, per rank, the sums of squares of the mean (two-shot, adam=False)."""
    nseg = len(ns)
    flat = lambda xs: ptr_array([xs[r][s] for r in range(world) for s in range(nseg)])  # noqa: E731
    status = (C.c_int * world)()
    wd_arr = (C.c_float * nseg)(*wd)
    none = (C.c_void_p * (world * nseg))()
    rc = lib.slb_sim_step(world, nseg, longs(ns), flat(p) if adam else none, flat(g), flat(m) if adam else none,
                          flat(v) if adam else none, wd_arr, hyper["lr"], hyper["b1"], hyper["b2"], hyper["eps"], step,
                          1 if adam else 0, mode, blocks_per_rank, timeout_ms,
                          (1 << world) - 1 if active_mask is None else active_mask, status,
                          sumsq.ctypes.data if sumsq is not None else None)
    return rc, list(status)

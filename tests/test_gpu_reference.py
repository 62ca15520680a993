"""Bit parity with the reference's own CUDA AdamW: core/cuda/kernels.cu compiled unmodified into oracle/_ref/ and
driven through its `sl_cuda_*` functions in the same process, on the same device buffers' contents."""
import ctypes as C
import os

import numpy as np
import pytest

from oracle import build as obuild
from oracle import pyoracle
from soliton_b200 import workload
from soliton_b200._C import lib
from tests.gpu_util import CUDA, DevBuf, check_ok, zeros

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ref(cuda):
    path = obuild.build_ref()
    if not path or not os.path.exists(path):
        pytest.skip("reference CUDA backend not built (no reference checkout at build time)")
    r = C.CDLL(path)
    assert r.sl_cuda_set_device(0) == 0
    r.sl_cuda_adamw.argtypes = [C.c_void_p] * 4 + [C.c_int64] + [C.c_float] * 5 + [C.c_int]
    r.sl_cuda_adamw.restype = None
    return r


@pytest.mark.parametrize("hyper", [dict(lr=3e-4, b1=0.9, b2=0.999, eps=1e-8, wd=0.1),
                                   dict(lr=1e-2, b1=0.9, b2=0.95, eps=1e-8, wd=0.1),
                                   dict(lr=6e-4, b1=0.9, b2=0.95, eps=1e-8, wd=0.0)])
def test_five_steps_bit_identical_to_reference_kernel(ref, hyper):
    n = 300_007
    rng = np.random.default_rng(9)
    p0 = (rng.standard_normal(n) * 0.02).astype(np.float32)
    ours = [DevBuf(p0), zeros(n), zeros(n)]
    theirs = [DevBuf(p0), zeros(n), zeros(n)]
    host = [p0.copy(), np.zeros(n, np.float32), np.zeros(n, np.float32)]
    for step in range(1, 6):
        g0 = (rng.standard_normal(n) * 1e-3).astype(np.float32)
        g = DevBuf(g0)
        lib.sl_adamw(CUDA, ours[0].ptr, g.ptr, ours[1].ptr, ours[2].ptr, n, hyper["lr"], hyper["b1"], hyper["b2"],
                     hyper["eps"], hyper["wd"], step)
        check_ok()
        ref.sl_cuda_adamw(theirs[0].ptr, g.ptr, theirs[1].ptr, theirs[2].ptr, n, hyper["lr"], hyper["b1"], hyper["b2"],
                          hyper["eps"], hyper["wd"], step)
        assert ref.sl_cuda_check() == 0
        ref.sl_cuda_sync()
        pyoracle.adamw(host[0], g0, host[1], host[2], hyper["lr"], hyper["b1"], hyper["b2"], hyper["eps"], hyper["wd"], step, fma=True)
        for a, b, c in zip(ours, theirs, host):
            got, want = a.get(), b.get()
            np.testing.assert_array_equal(got, want)  # this library == the reference's kernel, every bit
            np.testing.assert_array_equal(c, want)    # and the GPU-shaped oracle restates that kernel exactly


def test_special_values_bit_identical_to_reference_kernel(ref):
    # Zero gradients (v = 0: square root of zero), gradients whose square is a float denormal, very large
    # gradients: the inputs on which a hand-written division / square root would first differ from IEEE.
    n = 1 << 20
    rng = np.random.default_rng(21)
    p0 = (rng.standard_normal(n) * 0.02).astype(np.float32)
    p0[::13] = 0
    g0 = (rng.standard_normal(n) * 1e-3).astype(np.float32)
    g0[::7] = 0
    g0[1::1001] = 1e-22
    g0[2::1003] = 3e4
    g0[3::1007] = -1e-30
    g0[4::1009] = 1e15
    h = dict(lr=3e-4, b1=0.9, b2=0.999, eps=1e-8, wd=0.1)
    g = DevBuf(g0)
    ours, theirs = [DevBuf(p0), zeros(n), zeros(n)], [DevBuf(p0), zeros(n), zeros(n)]
    for step in (1, 2, 3):
        lib.sl_adamw(CUDA, ours[0].ptr, g.ptr, ours[1].ptr, ours[2].ptr, n, h["lr"], h["b1"], h["b2"], h["eps"], h["wd"], step)
        check_ok()
        ref.sl_cuda_adamw(theirs[0].ptr, g.ptr, theirs[1].ptr, theirs[2].ptr, n, h["lr"], h["b1"], h["b2"], h["eps"], h["wd"], step)
        ref.sl_cuda_sync()
        for a, b in zip(ours, theirs):
            np.testing.assert_array_equal(a.get().view(np.uint32), b.get().view(np.uint32))


def test_overflowing_second_moment_bit_identical_to_reference_kernel(ref):
    # |g| above about 1.8e19: (1 - b2) * g * g overflows float, v becomes +inf. IEEE arithmetic then gives
    # sqrt(inf) = inf and m / (inf + eps) = 0, so p only sees the weight decay; an infinite gradient gives NaN.
    n = 4096 + 17
    rng = np.random.default_rng(23)
    p0 = (rng.standard_normal(n) * 0.02).astype(np.float32)
    g0 = (rng.standard_normal(n) * 1e-3).astype(np.float32)
    g0[::5] = 1e20
    g0[1::7] = -3e25
    g0[2::11] = np.float32(3.0e38)
    g0[3::13] = np.inf
    g0[4::17] = -np.inf
    h = dict(lr=3e-4, b1=0.9, b2=0.999, eps=1e-8, wd=0.1)
    g = DevBuf(g0)
    ours, theirs = [DevBuf(p0), zeros(n), zeros(n)], [DevBuf(p0), zeros(n), zeros(n)]
    for step in (1, 2):
        lib.sl_adamw(CUDA, ours[0].ptr, g.ptr, ours[1].ptr, ours[2].ptr, n, h["lr"], h["b1"], h["b2"], h["eps"], h["wd"], step)
        check_ok()
        ref.sl_cuda_adamw(theirs[0].ptr, g.ptr, theirs[1].ptr, theirs[2].ptr, n, h["lr"], h["b1"], h["b2"], h["eps"], h["wd"], step)
        ref.sl_cuda_sync()
        for a, b in zip(ours, theirs):
            x, y = a.get(), b.get()
            both_nan = np.isnan(x) & np.isnan(y)       # NaN payloads are not part of the contract
            np.testing.assert_array_equal(np.where(both_nan, 0, x).view(np.uint32), np.where(both_nan, 0, y).view(np.uint32))
        overflowed = np.abs(g0) == np.float32(1e20)
        assert overflowed.any() and np.isfinite(ours[0].get()[overflowed]).all()   # v = inf, m finite: p stays finite


def test_config0_against_reference_kernel(ref):
    n = 1 << 20
    p0, g0 = workload.flat_case(n)
    h = workload.HYPER
    g = DevBuf(g0)
    ours, theirs = [DevBuf(p0), zeros(n), zeros(n)], [DevBuf(p0), zeros(n), zeros(n)]
    lib.sl_adamw(CUDA, ours[0].ptr, g.ptr, ours[1].ptr, ours[2].ptr, n, h["lr"], h["b1"], h["b2"], h["eps"], h["wd"], 1)
    check_ok()
    ref.sl_cuda_adamw(theirs[0].ptr, g.ptr, theirs[1].ptr, theirs[2].ptr, n, h["lr"], h["b1"], h["b2"], h["eps"], h["wd"], 1)
    ref.sl_cuda_sync()
    for a, b in zip(ours, theirs):
        np.testing.assert_array_equal(a.get(), b.get())

"""Single-rank path on a B200 through the C ABI: sl_adamw (batched into one multi-tensor launch) against the CPU
oracle, the golden fixture, and size-independent properties at the full GPT-2 124M parameter set."""
import hashlib
import os

import numpy as np
import pytest

from oracle import pyoracle
from soliton_b200 import workload
from soliton_b200._C import counter, lib, set_option
from tests.gpu_util import CUDA, DevBuf, check_ok, zeros

pytestmark = pytest.mark.gpu
H = workload.HYPER
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "config0.npz")


def dev_adamw(p, g, m, v, wd, step, h=H):
    lib.sl_adamw(CUDA, p.ptr, g.ptr, m.ptr, v.ptr, p.n, h["lr"], h["b1"], h["b2"], h["eps"], wd, step)


def max_rel(a, b):
    return float(np.max(np.abs(a.astype(np.float64) - b) / np.maximum(np.abs(b.astype(np.float64)), 1e-30)))


def test_config0_flat_buffer_matches_oracle_and_golden(cuda):
    n = 1 << 20
    p0, g0 = workload.flat_case(n)
    p, g, m, v = DevBuf(p0), DevBuf(g0), zeros(n), zeros(n)
    dev_adamw(p, g, m, v, H["wd"], 1)
    check_ok()
    got = [p.get(), m.get(), v.get()]
    ref = [p0.copy(), np.zeros(n, np.float32), np.zeros(n, np.float32)]
    pyoracle.adamw(ref[0], g0, ref[1], ref[2], H["lr"], H["b1"], H["b2"], H["eps"], H["wd"], 1)
    np.testing.assert_array_equal(got[1], ref[1])     # moments: bit-exact
    np.testing.assert_array_equal(got[2], ref[2])
    assert max_rel(got[0], ref[0]) <= 1e-6            # parameters: the stated tolerance ...
    fma = [p0.copy(), np.zeros(n, np.float32), np.zeros(n, np.float32)]
    pyoracle.adamw(fma[0], g0, fma[1], fma[2], H["lr"], H["b1"], H["b2"], H["eps"], H["wd"], 1, fma=True)
    np.testing.assert_array_equal(got[0], fma[0])     # ... and bit-exact against the GPU-shaped restatement
    gold = np.load(GOLDEN)
    s = int(gold["stride"])
    np.testing.assert_array_equal(got[1][::s], gold["m"])
    np.testing.assert_array_equal(got[2][::s], gold["v"])
    assert hashlib.sha256(got[1].tobytes()).hexdigest() == str(gold["sha_m"])
    assert hashlib.sha256(got[2].tobytes()).hexdigest() == str(gold["sha_v"])
    assert max_rel(got[0][::s], gold["p"]) <= 1e-6


@pytest.mark.parametrize("skew", [0, 1, 3])
def test_ragged_tensors_in_one_launch_over_three_steps(cuda, skew):
    # empty-ish, sub-tile, tile-boundary and multi-tile sizes; skew != 0 makes pointers 4- but not 16-byte aligned
    sizes = [1, 3, 4, 5, 255, 2047, 2048, 2049, 4096 + 7, 100000, 3 * 2048]
    wds = [0.0 if i % 3 == 0 else 0.1 for i in range(len(sizes))]
    rng = np.random.default_rng(11)
    host = [[(rng.standard_normal(n) * 0.02).astype(np.float32), np.zeros(n, np.float32), np.zeros(n, np.float32)]
            for n in sizes]
    dev = [[DevBuf(h[0], skew=skew), DevBuf(h[1], skew=skew), DevBuf(h[2], skew=skew)] for h in host]
    for step in (1, 2, 3):
        grads = [(rng.standard_normal(n) * 1e-3).astype(np.float32) for n in sizes]
        dg = [DevBuf(g, skew=skew) for g in grads]
        before = counter("launches")
        for d, g, wd in zip(dev, dg, wds):
            dev_adamw(d[0], g, d[1], d[2], wd, step)
        check_ok()
        assert counter("launches") - before == 1      # eleven tensors, one kernel
        for h, g, wd in zip(host, grads, wds):
            pyoracle.adamw(h[0], g, h[1], h[2], H["lr"], H["b1"], H["b2"], H["eps"], wd, step, fma=True)
        for d, h in zip(dev, host):
            for a, b in zip(d, h):
                np.testing.assert_array_equal(a.get(), b)


def test_reference_test_recipe_five_steps(cuda):
    # tests/test_ops.py:121-134 of the reference, with torch replaced by the pinned oracle
    rng = np.random.default_rng(3)
    p0 = rng.standard_normal(20).astype(np.float32)
    hp = dict(lr=1e-2, b1=0.9, b2=0.95, eps=1e-8)
    p, m, v = DevBuf(p0), zeros(20), zeros(20)
    ref = [p0.copy(), np.zeros(20, np.float32), np.zeros(20, np.float32)]
    for step in range(1, 6):
        g0 = rng.standard_normal(20).astype(np.float32)
        g = DevBuf(g0)
        lib.sl_adamw(CUDA, p.ptr, g.ptr, m.ptr, v.ptr, 20, hp["lr"], hp["b1"], hp["b2"], hp["eps"], 0.1, step)
        pyoracle.adamw(ref[0], g0, ref[1], ref[2], hp["lr"], hp["b1"], hp["b2"], hp["eps"], 0.1, step)
        got = p.get()  # reading the parameter launches the pending update first
        np.testing.assert_allclose(got, ref[0], rtol=1e-5, atol=1e-6)


def test_same_parameter_twice_is_two_launches_in_order(cuda):
    n = 5000
    p0, g0 = workload.flat_case(n)
    p, g, m, v = DevBuf(p0), DevBuf(g0), zeros(n), zeros(n)
    before = counter("launches")
    dev_adamw(p, g, m, v, 0.1, 1)
    dev_adamw(p, g, m, v, 0.1, 2)
    check_ok()
    assert counter("launches") - before == 2
    ref = [p0.copy(), np.zeros(n, np.float32), np.zeros(n, np.float32)]
    for step in (1, 2):
        pyoracle.adamw(ref[0], g0, ref[1], ref[2], H["lr"], H["b1"], H["b2"], H["eps"], 0.1, step, fma=True)
    np.testing.assert_array_equal(p.get(), ref[0])


def test_bad_arguments_set_sticky_error_12(cuda):
    check_ok()
    b = zeros(16)
    lib.sl_adamw(CUDA, None, b.ptr, b.ptr, b.ptr, 16, 1e-3, 0.9, 0.999, 1e-8, 0.0, 1)
    assert lib.sl_check(CUDA) == 12
    lib.slb_clear_error()
    lib.sl_adamw(CUDA, b.ptr + 2, b.ptr, b.ptr, b.ptr, 8, 1e-3, 0.9, 0.999, 1e-8, 0.0, 1)  # not float-aligned
    assert lib.sl_check(CUDA) == 12
    lib.slb_clear_error()
    lib.sl_adamw(CUDA, b.ptr, b.ptr, b.ptr, b.ptr, 0, 1e-3, 0.9, 0.999, 1e-8, 0.0, 1)       # empty: nothing to do
    check_ok()


def test_gpt2_124m_parameter_set_single_rank(cuda):
    """The benchmark workload at full size: 148 tensors, 124,439,808 parameters, one launch, bit-compared."""
    shapes = workload.param_shapes("124M")
    params = workload.init_params("124M", seed=0)
    grads = workload.rank_grads("124M", rank=0)
    dev = []
    for prm, grd in zip(params, grads):
        dev.append((DevBuf(prm), DevBuf(grd), zeros(prm.size), zeros(prm.size)))
    before = counter("launches")
    for (p, g, m, v), (_, shape, _) in zip(dev, shapes):
        dev_adamw(p, g, m, v, H["wd"] if len(shape) >= 2 else 0.0, 1)
    check_ok()
    assert counter("launches") - before == 1
    worst = 0.0
    for (p, g, m, v), prm, grd, (_, shape, _) in zip(dev, params, grads, shapes):
        wd = H["wd"] if len(shape) >= 2 else 0.0
        rp, rm, rv = prm.ravel().copy(), np.zeros(prm.size, np.float32), np.zeros(prm.size, np.float32)
        rp2 = rp.copy()
        pyoracle.adamw(rp, grd.ravel(), rm, rv, H["lr"], H["b1"], H["b2"], H["eps"], wd, 1)
        got_p = p.get()
        np.testing.assert_array_equal(m.get(), rm)
        np.testing.assert_array_equal(v.get(), rv)
        worst = max(worst, max_rel(got_p, rp))
        pyoracle.adamw(rp2, grd.ravel(), np.zeros_like(rm), np.zeros_like(rv), H["lr"], H["b1"], H["b2"], H["eps"], wd, 1, fma=True)
        np.testing.assert_array_equal(got_p, rp2)
    assert worst <= 1e-6

    # property: one fused launch over all tensors == one launch per tensor (the partition never changes bits)
    set_option("eager", 1)
    try:
        sample = [0, 1, 2, 6, 8, 147]
        fresh = [(DevBuf(params[i]), zeros(params[i].size), zeros(params[i].size)) for i in sample]
        for (p2, m2, v2), i in zip(fresh, sample):
            wd = H["wd"] if len(shapes[i][1]) >= 2 else 0.0
            lib.sl_adamw(CUDA, p2.ptr, dev[i][1].ptr, m2.ptr, v2.ptr, p2.n, H["lr"], H["b1"], H["b2"], H["eps"], wd, 1)
        check_ok()
        for (p2, m2, v2), i in zip(fresh, sample):
            np.testing.assert_array_equal(p2.get(), dev[i][0].get())
            np.testing.assert_array_equal(v2.get(), dev[i][3].get())
    finally:
        set_option("eager", 0)

    # property: a zero gradient without weight decay leaves p, m, v untouched
    i = 2  # blocks.0.ln1.weight
    p3, g3, m3, v3 = DevBuf(params[i]), zeros(params[i].size), zeros(params[i].size), zeros(params[i].size)
    dev_adamw(p3, g3, m3, v3, 0.0, 1)
    check_ok()
    np.testing.assert_array_equal(p3.get(), params[i].ravel())
    assert not m3.get().any() and not v3.get().any()


def test_scale_axpy_fill_sumsq_next_to_the_path(cuda):
    rng = np.random.default_rng(2)
    n = 1_000_003
    x0, y0 = rng.standard_normal(n, dtype=np.float32), rng.standard_normal(n, dtype=np.float32)
    x, y = DevBuf(x0), DevBuf(y0)
    lib.sl_axpy(CUDA, x.ptr, y.ptr, n, 0.5)
    ry = y0.copy()
    pyoracle.axpy(x0, ry, 0.5)
    np.testing.assert_allclose(y.get(), ry, rtol=0, atol=1e-7)  # the device fuses the multiply-add (one rounding)
    lib.sl_scale(CUDA, x.ptr, x.ptr, n, 0.25)
    np.testing.assert_array_equal(x.get(), x0 * np.float32(0.25))
    s1 = lib.sl_sumsq(CUDA, y.ptr, n)
    s2 = lib.sl_sumsq(CUDA, y.ptr, n)
    assert s1 == s2                                              # run-to-run identical
    assert s1 == pytest.approx(pyoracle.sumsq(y.get()), rel=1e-12)
    lib.sl_fill(CUDA, x.ptr, n, 1.5)
    assert (x.get() == 1.5).all()
    check_ok()


def test_pending_update_goes_out_before_anything_can_touch_its_memory(cuda):
    """The recorded (not yet launched) update must behave as if it had run at the call: freeing and reusing the
    gradient's block, copying the parameter, filling a moment -- each has to see or preserve the right values."""
    n = 70000
    p0, g0 = workload.flat_case(n)
    ref = [p0.copy(), np.zeros(n, np.float32), np.zeros(n, np.float32)]
    pyoracle.adamw(ref[0], g0, ref[1], ref[2], H["lr"], H["b1"], H["b2"], H["eps"], 0.1, 1, fma=True)

    # (a) the gradient's block is freed and handed out again before any launch was forced
    p, g, m, v = DevBuf(p0), DevBuf(g0), zeros(n), zeros(n)
    before = counter("launches")
    dev_adamw(p, g, m, v, 0.1, 1)
    assert counter("launches") == before            # recorded only
    old_ptr = g.ptr
    g.free()                                         # launches the update, then releases the block
    assert counter("launches") == before + 1
    g2 = DevBuf(np.full(n, 123.0, np.float32))       # same size: the pool hands the same block out again
    assert g2.ptr == old_ptr
    check_ok()
    np.testing.assert_array_equal(p.get(), ref[0])

    # (b) a device-to-device copy of the parameter sees the updated values
    p, g, m, v, q = DevBuf(p0), DevBuf(g0), zeros(n), zeros(n), zeros(n)
    dev_adamw(p, g, m, v, 0.1, 1)
    lib.sl_copy(CUDA, q.ptr, p.ptr, 4 * n)
    np.testing.assert_array_equal(q.get(), ref[0])

    # (c) filling the second moment after the call does not reach back into the update
    p, g, m, v = DevBuf(p0), DevBuf(g0), zeros(n), zeros(n)
    dev_adamw(p, g, m, v, 0.1, 1)
    lib.sl_fill(CUDA, v.ptr, n, 7.0)
    np.testing.assert_array_equal(p.get(), ref[0])
    assert (v.get() == 7.0).all()
    check_ok()


def test_eager_option_launches_at_every_call(cuda):
    n = 3000
    p0, g0 = workload.flat_case(n)
    bufs = [(DevBuf(p0), DevBuf(g0), zeros(n), zeros(n)) for _ in range(3)]
    set_option("eager", 1)
    try:
        before = counter("launches")
        for p, g, m, v in bufs:
            dev_adamw(p, g, m, v, 0.1, 1)
        assert counter("launches") == before + 3
    finally:
        set_option("eager", 0)
    check_ok()
    ref = [p0.copy(), np.zeros(n, np.float32), np.zeros(n, np.float32)]
    pyoracle.adamw(ref[0], g0, ref[1], ref[2], H["lr"], H["b1"], H["b2"], H["eps"], 0.1, 1, fma=True)
    for p, g, m, v in bufs:
        np.testing.assert_array_equal(p.get(), ref[0])

"""Gradient clipping next to the path (python/soliton/optim.py:31-39: sumsq per tensor, host sqrt, in-place scale)
through the Soliton-shaped interface: the per-tensor sumsq calls are answered from one batched launch, the scales
ride along with the AdamW launch, and the results equal the oracle's clip + AdamW bit for bit."""
import math

import numpy as np
import pytest

from oracle import pyoracle
from soliton_b200 import tensor as T, workload
from soliton_b200._C import counter, lib
from soliton_b200.optim import AdamW, clip_grad_norm

pytestmark = pytest.mark.gpu
H = workload.HYPER
SHAPES = [(300, 70), (70,), (2048,), (5, 2049), (1,), (130000,), (64, 1024)]


def run_steps(max_norm, steps, grad_std):
    rng = np.random.default_rng(17)
    p0 = [(rng.standard_normal(s) * 0.02).astype(np.float32) for s in SHAPES]
    params = [T.tensor(a, "cuda") for a in p0]
    opt = AdamW(params, lr=H["lr"], betas=(H["b1"], H["b2"]), eps=H["eps"], weight_decay=H["wd"])
    ref = [[a.ravel().copy(), np.zeros(a.size, np.float32), np.zeros(a.size, np.float32)] for a in p0]
    launches = []
    for step in range(1, steps + 1):
        grads = [(rng.standard_normal(s) * grad_std).astype(np.float32) for s in SHAPES]
        for p, g in zip(params, grads):
            p.grad = T.tensor(g, "cuda")
        T.synchronize()
        before = counter("launches")
        norm = clip_grad_norm(opt.params, max_norm)
        opt.step()
        T.synchronize()
        launches.append(counter("launches") - before)
        # oracle: same clip on the host kernels, with the scale the device's norm produced
        want_norm = math.sqrt(sum(pyoracle.sumsq(g.ravel()) for g in grads))
        assert norm == pytest.approx(want_norm, rel=1e-12)
        hg = [g.ravel().copy() for g in grads]
        if norm > max_norm:
            s = max_norm / (norm + 1e-6)
            for g in hg:
                pyoracle.scale(g, g, s)
        for i, shape in enumerate(SHAPES):
            wd = H["wd"] if len(shape) >= 2 else 0.0
            pyoracle.adamw(ref[i][0], hg[i], ref[i][1], ref[i][2], H["lr"], H["b1"], H["b2"], H["eps"], wd, step, fma=True)
        for i, p in enumerate(params):
            np.testing.assert_array_equal(p.grad.numpy().ravel(), hg[i])       # gradients are clipped in place
            np.testing.assert_array_equal(p.numpy().ravel(), ref[i][0])
            np.testing.assert_array_equal(opt.state[i][0].numpy().ravel(), ref[i][1])
            np.testing.assert_array_equal(opt.state[i][1].numpy().ravel(), ref[i][2])
        opt.zero_grad()
    return launches


def test_clip_that_scales_is_two_launches_once_the_tensor_list_is_known(cuda):
    launches = run_steps(max_norm=0.05, steps=4, grad_std=1e-3)   # norm ~ 0.49 > 0.05: every step scales
    assert launches[0] == len(SHAPES) + 1      # first clip: one sumsq launch per tensor, then one fused AdamW
    # The second clip meets two gradients whose (equal-sized) blocks swapped places, which it cannot have seen yet.
    assert launches[1] <= 4
    assert launches[2:] == [2, 2]              # from then on: one batched sumsq + one AdamW that applies the scale


def test_clip_below_threshold_changes_nothing(cuda):
    launches = run_steps(max_norm=10.0, steps=3, grad_std=1e-3)
    assert launches[2] == 2


def test_scale_then_read_sees_the_scaled_values(cuda):
    # a deferred in-place scale must be visible to anything that looks at the memory
    x0 = np.arange(1, 1001, dtype=np.float32)
    x = T.tensor(x0, "cuda")
    lib.sl_scale(T.CUDA, x.ptr, x.ptr, x.numel, 0.5)
    np.testing.assert_array_equal(x.numpy(), x0 * np.float32(0.5))
    lib.sl_scale(T.CUDA, x.ptr, x.ptr, x.numel, 0.5)
    lib.sl_scale(T.CUDA, x.ptr, x.ptr, x.numel, 4.0)
    assert lib.sl_sumsq(T.CUDA, x.ptr, x.numel) == float(np.sum(x0.astype(np.float64) ** 2))

"""Pins the CPU oracle: against torch.optim.AdamW with the reference's own recipe, against the committed golden
fixture, and its two AdamW shapes against each other."""
import hashlib
import os

import numpy as np
import pytest
import torch

from oracle import pyoracle
from soliton_b200 import workload

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "config0.npz")


@pytest.mark.parametrize("fma", [False, True])
def test_oracle_adamw_matches_torch_reference_recipe(built, fma):
    # The reference's test_adamw_matches_torch (tests/test_ops.py:121-134): (4,5) tensor, default_rng(3), 5 steps,
    # lr 1e-2, wd 0.1, betas (0.9, 0.95), eps 1e-8, against torch.optim.AdamW, rtol 1e-5 / atol 1e-6.
    rng = np.random.default_rng(3)
    p0 = rng.standard_normal((4, 5)).astype(np.float32)
    p, m, v = p0.copy().ravel(), np.zeros(20, np.float32), np.zeros(20, np.float32)
    tp = torch.nn.Parameter(torch.tensor(p0))
    topt = torch.optim.AdamW([tp], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    for step in range(1, 6):
        g = rng.standard_normal(p0.shape).astype(np.float32)
        pyoracle.adamw(p, g.ravel().copy(), m, v, 1e-2, 0.9, 0.95, 1e-8, 0.1, step, fma=fma)
        tp.grad = torch.tensor(g)
        topt.step()
    np.testing.assert_allclose(p.reshape(4, 5), tp.detach().numpy(), rtol=1e-5, atol=1e-6)


def test_oracle_matches_torch_at_benchmark_hyperparameters(built):
    n = 1 << 16
    p, g = workload.flat_case(n)
    m, v = np.zeros(n, np.float32), np.zeros(n, np.float32)
    h = workload.HYPER
    tp = torch.nn.Parameter(torch.tensor(p.copy()))
    topt = torch.optim.AdamW([tp], lr=h["lr"], betas=(h["b1"], h["b2"]), eps=h["eps"], weight_decay=h["wd"])
    for step in range(1, 4):
        pyoracle.adamw(p, g, m, v, h["lr"], h["b1"], h["b2"], h["eps"], h["wd"], step)
        tp.grad = torch.tensor(g)
        topt.step()
    np.testing.assert_allclose(p, tp.detach().numpy(), rtol=1e-5, atol=1e-6)


def test_oracle_reproduces_golden_fixture(built):
    from tests.golden.make_golden import compute
    gold = np.load(GOLDEN)
    p, m, v = compute()
    s = int(gold["stride"])
    for name, arr in (("p", p), ("m", m), ("v", v)):
        assert hashlib.sha256(arr.tobytes()).hexdigest() == str(gold["sha_" + name])
        np.testing.assert_array_equal(arr[::s], gold[name])


def test_fma_shape_equals_plain_at_step_one_and_within_one_ulp_later(built):
    n = 1 << 14
    p, g = workload.flat_case(n)
    h = workload.HYPER
    a = [p.copy(), np.zeros(n, np.float32), np.zeros(n, np.float32)]
    b = [p.copy(), np.zeros(n, np.float32), np.zeros(n, np.float32)]
    pyoracle.adamw(a[0], g, a[1], a[2], h["lr"], h["b1"], h["b2"], h["eps"], h["wd"], 1, fma=False)
    pyoracle.adamw(b[0], g, b[1], b[2], h["lr"], h["b1"], h["b2"], h["eps"], h["wd"], 1, fma=True)
    for x, y in zip(a[1:], b[1:]):
        np.testing.assert_array_equal(x, y)  # m = v = 0 makes the two shapes the same arithmetic
    np.testing.assert_allclose(a[0], b[0], rtol=2e-7, atol=0)
    for step in (2, 3):
        pyoracle.adamw(a[0], g, a[1], a[2], h["lr"], h["b1"], h["b2"], h["eps"], h["wd"], step, fma=False)
        pyoracle.adamw(b[0], g, b[1], b[2], h["lr"], h["b1"], h["b2"], h["eps"], h["wd"], step, fma=True)
    # From the second step on the two shapes round m and v differently by at most one float ulp. p follows
    # within 1e-6 relative except where the update nearly cancels the parameter, hence the absolute floor.
    for x, y in zip(a[1:], b[1:]):
        np.testing.assert_allclose(x, y, rtol=3e-7, atol=0)
    np.testing.assert_allclose(a[0], b[0], rtol=1e-6, atol=1e-9)


@pytest.mark.parametrize("world", [1, 2, 3, 4, 8])
def test_mean_ranks_is_rank_ordered_float_sum_times_inverse(built, world):
    rng = np.random.default_rng(5)
    gs = [rng.standard_normal(1000, dtype=np.float32) for _ in range(world)]
    acc = gs[0].copy()
    for g in gs[1:]:
        acc = (acc + g).astype(np.float32)
    want = (acc * np.float32(1.0 / world)).astype(np.float32)
    np.testing.assert_array_equal(pyoracle.mean_ranks(gs), want)
    if world == 2:  # a + b commutes, so any two-rank all-reduce must give these bits
        np.testing.assert_array_equal(pyoracle.mean_ranks(gs[::-1]), want)


def test_axpy_scale_sumsq_clip(built):
    rng = np.random.default_rng(6)
    x, y = rng.standard_normal(777, dtype=np.float32), rng.standard_normal(777, dtype=np.float32)
    y2 = y.copy()
    pyoracle.axpy(x, y2, 0.5)
    np.testing.assert_array_equal(y2, (y + np.float32(0.5) * x).astype(np.float32))
    z = np.empty_like(x)
    pyoracle.scale(x, z, 0.25)
    np.testing.assert_array_equal(z, x * np.float32(0.25))
    assert pyoracle.sumsq(x) == pytest.approx(float(np.sum(x.astype(np.float64) ** 2)), rel=1e-12)
    gs = [x.copy(), y.copy()]
    norm = pyoracle.clip(gs, 1.0)
    assert norm == pytest.approx(np.sqrt(np.sum(x.astype(np.float64) ** 2) + np.sum(y.astype(np.float64) ** 2)))
    s = np.float32(1.0 / (norm + 1e-6))
    np.testing.assert_array_equal(gs[0], x * s)

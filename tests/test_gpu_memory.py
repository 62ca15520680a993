"""The zero-error memory claim for this path: the same calls on meta and on cuda leave identical allocator traces
(as tests/test_memory.py:26-32 of the reference checks for whole training runs), and the path takes nothing from
the pool per step."""
import ctypes

import numpy as np
import pytest

from soliton_b200 import tensor as T
from soliton_b200.optim import AdamW, clip_grad_norm
from soliton_b200 import distributed

pytestmark = pytest.mark.gpu
SHAPES = [(50, 32), (32,), (32,), (96, 32), (96,), (3000, 700), (700,), (1,)]


def run(device, steps=3):
    T.empty_cache(device)
    base = T.memory_stats(device)
    T.reset_peak_stats(device)
    rng = np.random.default_rng(0)
    params = [T.tensor(rng.standard_normal(s, dtype=np.float32) * 0.02, device) if device != "meta" else T.empty(s, device)
              for s in SHAPES]
    opt = AdamW(params, lr=1e-3)
    for _ in range(steps):
        for p in params:
            p.grad = T.empty(p.shape, device) if device == "meta" else T.tensor(rng.standard_normal(p.shape, dtype=np.float32), device)
        distributed.all_reduce_grads(opt.params)  # single process: no-op, as in the reference
        if device != "meta":
            clip_grad_norm(opt.params, 1.0)
        opt.step()
        opt.zero_grad()
    if device == "cuda":
        T.synchronize()
    s = T.memory_stats(device)
    out = {k: s[k] - base["allocated"] if k.startswith("peak_") else s[k] for k in ("peak_allocated", "trace", "n_alloc")}
    out["reserved_growth"] = s["reserved"] - base["reserved"]
    del opt, params
    return out


def test_meta_trace_matches_cuda(cuda):
    meta = run("meta")
    real = run("cuda")
    assert real == meta


def test_steps_take_nothing_from_the_pool(cuda):
    n = 10000
    p, g, m, v = (T.zeros((n,), "cuda") for _ in range(4))
    T.synchronize()
    before = T.memory_stats("cuda")
    from soliton_b200._C import lib
    for step in range(1, 4):
        lib.sl_adamw(T.CUDA, p.ptr, g.ptr, m.ptr, v.ptr, n, 1e-3, 0.9, 0.999, 1e-8, 0.1, step)
    T.synchronize()
    after = T.memory_stats("cuda")
    assert after == before


def run_with_marks(device, values, steps=3):
    """The step loop with a mark at every step boundary, as the reference's trainer runs it (examples/gpt2.py:108)."""
    from soliton_b200 import arena
    rng = np.random.default_rng(1)
    params = [T.tensor(a, device) for a in values]
    opt = AdamW(params, lr=1e-3)
    for _ in range(steps):
        arena.mark(device)
        for p in params:
            g = rng.standard_normal(p.shape, dtype=np.float32)
            p.grad = T.empty(p.shape, device) if device == "meta" else T.tensor(g, device)
        distributed.all_reduce_grads(opt.params)
        opt.step()
        opt.zero_grad()
    if device == "cuda":
        T.synchronize()
    return params, opt


def test_arena_run_is_bit_equal_to_pool_run_and_its_size_is_predicted(cuda):
    # tests/test_arena.py:29-50 of the reference, for this path: allocator mode must not change a bit
    from soliton_b200 import arena
    rng = np.random.default_rng(0)
    values = [rng.standard_normal(s, dtype=np.float32) * 0.02 for s in SHAPES]
    params, opt = run_with_marks("cuda", values)
    want = [p.numpy() for p in params] + [m.numpy() for m, _ in opt.state]
    del params, opt
    T.empty_cache("cuda")
    plan = arena.plan(lambda dev: run_with_marks(dev, values))
    before = T.memory_stats("cuda")["reserved"]
    arena.install(plan, "cuda")
    assert T.memory_stats("cuda")["reserved"] - before == plan.bytes      # 0 bytes of prediction error
    params, opt = run_with_marks("cuda", values, steps=3)
    arena.check("cuda")
    got = [p.numpy() for p in params] + [m.numpy() for m, _ in opt.state]
    for a, b in zip(got, want):
        np.testing.assert_array_equal(a, b)
    arena.off("cuda")
    del params, opt
    # As in the reference (core/soliton/alloc.d:202-213) the arena goes back to the driver only once nothing at all
    # is allocated; the device's fixed workspaces stay allocated, so it stays reserved here.
    assert T.memory_stats("cuda")["reserved"] in (before, before + plan.bytes)

"""The offset solver of soliton_b200.arena and record -> plan -> replay on the cpu pool (no GPU)."""
import numpy as np

from soliton_b200 import arena, tensor as T


def test_solver_never_overlaps_blocks_that_are_alive_together():
    rng = np.random.default_rng(0)
    n = 300
    sizes = [int(s) * 512 for s in rng.integers(1, 200, n)]
    starts = list(range(n))
    ends = [int(min(n + 1, i + 1 + rng.integers(1, 40))) if rng.random() < 0.8 else -1 for i in range(n)]
    offsets, total, peak = arena.solve(sizes, starts, ends)
    death = [e if e >= 0 else n + 1 for e in ends]
    for i in range(n):
        for j in range(i):
            if starts[i] < death[j] and starts[j] < death[i]:
                assert offsets[i] + sizes[i] <= offsets[j] or offsets[j] + sizes[j] <= offsets[i]
    assert peak <= total <= 1.5 * peak


def step_like(device, steps=3):
    """The allocation pattern of a training step around the optimizer path: persistent p, m, v; per-step gradients."""
    shapes = [(64, 32), (32,), (200, 100), (100,)]
    params = [T.empty(s, device) for s in shapes]
    state = [(T.zeros(s, device), T.zeros(s, device)) for s in shapes]
    for _ in range(steps):
        arena.mark(device)
        grads = [T.empty(s, device) for s in shapes]
        del grads
    return params, state


def test_plan_predicts_the_arena_and_the_replay_follows_it(lib):
    p = arena.plan(lambda dev: step_like(dev))
    assert p.body == 12 + 2 * 4 and len(p.sizes) == 12 + 3 * 4   # the body is the last recorded step
    T.empty_cache("cpu")
    before = T.memory_stats("cpu")["reserved"]
    arena.install(p, "cpu")
    assert T.memory_stats("cpu")["reserved"] - before == p.bytes   # predicted bytes == reserved bytes
    keep = step_like("cpu", steps=5)                               # more steps than planned: the body repeats
    arena.check("cpu")
    arena.off("cpu")
    del keep
    assert T.memory_stats("cpu")["reserved"] == before

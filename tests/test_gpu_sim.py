"""The multi-rank kernels with all ranks emulated on one GPU (one cooperative launch, blocks of every rank
resident together), through the C ABI test hook. Checks the fixed summation order, bit-identical ranks, the
one-shot/two-shot equivalence and the bounded waits -- none of which needs a second GPU."""
import numpy as np
import pytest

from oracle import pyoracle
from soliton_b200 import workload
from soliton_b200._C import counter, set_option
from tests.gpu_util import DevBuf, sim_step, zeros

pytestmark = pytest.mark.gpu
H = workload.HYPER
SIZES = [1, 5, 2047, 2048, 2049, 3 * 2048 + 17, 70001, 4]
WDS = [0.1, 0.0, 0.1, 0.1, 0.0, 0.1, 0.1, 0.0]


def make_case(world, sizes, seed=0, skew=0):
    rng = np.random.default_rng(seed)
    p0 = [(rng.standard_normal(n) * 0.02).astype(np.float32) for n in sizes]
    g0 = [[(np.random.default_rng(100 + 17 * r + s).standard_normal(n) * 1e-3).astype(np.float32)
           for s, n in enumerate(sizes)] for r in range(world)]
    p = [[DevBuf(x, skew=skew) for x in p0] for _ in range(world)]
    g = [[DevBuf(x, skew=skew) for x in g0[r]] for r in range(world)]
    m = [[zeros(n, skew=skew) for n in sizes] for _ in range(world)]
    v = [[zeros(n, skew=skew) for n in sizes] for _ in range(world)]
    return p0, g0, p, g, m, v


def oracle_steps(p0, g_by_step, sizes, wds, world):
    """Reference state after len(g_by_step) steps: rank-ordered mean, then the GPU-shaped AdamW."""
    ref = [[x.copy(), np.zeros_like(x), np.zeros_like(x)] for x in p0]
    means = None
    for step, g0 in enumerate(g_by_step, 1):
        means = [pyoracle.mean_ranks([g0[r][s] for r in range(world)]) for s in range(len(sizes))]
        for s in range(len(sizes)):
            pyoracle.adamw(ref[s][0], means[s], ref[s][1], ref[s][2], H["lr"], H["b1"], H["b2"], H["eps"], wds[s], step, fma=True)
    return ref, means


@pytest.fixture
def large_kernel():
    """The kernel that takes large steps (two-shot); kept as a fixture so that variants can be run side by side."""
    return "k_twoshot"


@pytest.mark.parametrize("mode", [1, 2], ids=["oneshot", "twoshot"])
@pytest.mark.parametrize("world", [2, 3, 4, 8])
def test_fused_step_matches_oracle_and_ranks_agree(cuda, world, mode, large_kernel):
    p0, g0, p, g, m, v = make_case(world, SIZES)
    rc, status = sim_step(world, SIZES, p, g, m, v, WDS, H, 1, adam=True, mode=mode)
    assert rc == 0 and status == [0] * world
    assert counter("last_mode") == mode
    ref, means = oracle_steps(p0, [g0], SIZES, WDS, world)
    for r in range(world):
        for s in range(len(SIZES)):
            np.testing.assert_array_equal(g[r][s].get(), means[s])     # every rank holds the mean, same bits
            np.testing.assert_array_equal(p[r][s].get(), ref[s][0])
            np.testing.assert_array_equal(m[r][s].get(), ref[s][1])
            np.testing.assert_array_equal(v[r][s].get(), ref[s][2])


@pytest.mark.parametrize("world", [2, 8])
def test_bare_allreduce_mean_without_optimizer(cuda, world, large_kernel):
    _, g0, p, g, m, v = make_case(world, SIZES)
    for mode in (1, 2):
        for r in range(world):
            for s in range(len(SIZES)):
                g[r][s].put(g0[r][s])
        rc, status = sim_step(world, SIZES, p, g, m, v, WDS, H, 1, adam=False, mode=mode)
        assert rc == 0 and status == [0] * world
        for s in range(len(SIZES)):
            want = pyoracle.mean_ranks([g0[r][s] for r in range(world)])
            for r in range(world):
                np.testing.assert_array_equal(g[r][s].get(), want)


def test_three_steps_unaligned_pointers_and_block_counts(cuda, large_kernel):
    world, sizes, wds = 4, [2048 * 5 + 3, 999, 2048], [0.1, 0.0, 0.1]
    results = []
    for skew, blocks, mode in [(0, 0, 2), (1, 1, 2), (0, 3, 2), (3, 2, 1), (0, 0, 1)]:
        p0, g0, p, g, m, v = make_case(world, sizes, seed=4, skew=skew)
        steps = []
        for step in (1, 2, 3):
            gs = [[(np.random.default_rng(1000 * step + 17 * r + s).standard_normal(n) * 1e-3).astype(np.float32)
                   for s, n in enumerate(sizes)] for r in range(world)]
            for r in range(world):
                for s in range(len(sizes)):
                    g[r][s].put(gs[r][s])
            steps.append(gs)
            rc, status = sim_step(world, sizes, p, g, m, v, wds, H, step, mode=mode, blocks_per_rank=blocks)
            assert rc == 0 and status == [0] * world
        ref, _ = oracle_steps(p0, steps, sizes, wds, world)
        for r in range(world):
            for s in range(len(sizes)):
                np.testing.assert_array_equal(p[r][s].get(), ref[s][0])
                np.testing.assert_array_equal(v[r][s].get(), ref[s][2])
        results.append([p[0][s].get() for s in range(len(sizes))])
    for other in results[1:]:  # alignment, block count and one-shot/two-shot never change a bit
        for a, b in zip(results[0], other):
            np.testing.assert_array_equal(a, b)


def test_large_single_buffer_two_shot_world_8(cuda, large_kernel):
    world, n = 8, 3_000_000
    p0, g0, p, g, m, v = make_case(world, [n])
    rc, status = sim_step(world, [n], p, g, m, v, [0.1], H, 1, mode=0)
    assert rc == 0 and status == [0] * world
    assert counter("last_mode") == 2  # too large for the staging slots: the size rule picked two-shot
    ref, means = oracle_steps(p0, [g0], [n], [0.1], world)
    for r in range(world):
        np.testing.assert_array_equal(g[r][0].get(), means[0])
        np.testing.assert_array_equal(p[r][0].get(), ref[0][0])


def test_missing_rank_makes_waits_run_out_and_the_device_stays_usable(cuda, large_kernel):
    world = 2
    p0, g0, p, g, m, v = make_case(world, [5000])
    for mode, code in ((2, 21), (1, 22)):
        rc, status = sim_step(world, [5000], p, g, m, v, [0.1], H, 1, mode=mode, timeout_ms=50, active_mask=0b01)
        assert rc == 0           # the kernel returned by itself
        assert status[0] == code  # start barrier (two-shot) / staged-gradients barrier (one-shot) ran out
    # the context is intact: the same buffers go through a complete step afterwards
    for r in range(world):
        g[r][0].put(g0[r][0])
        p[r][0].put(p0[0])
        m[r][0].put(np.zeros(5000, np.float32))
        v[r][0].put(np.zeros(5000, np.float32))
    rc, status = sim_step(world, [5000], p, g, m, v, [0.1], H, 1, mode=2)
    assert rc == 0 and status == [0, 0]
    ref, _ = oracle_steps(p0, [g0], [5000], [0.1], world)
    np.testing.assert_array_equal(p[1][0].get(), ref[0][0])


@pytest.mark.parametrize("world", [2, 3, 4, 5, 8])
def test_two_shot_mean_leaves_the_sum_of_squares_of_every_tensor(cuda, world, large_kernel):
    """The clip that follows a gradient mean needs sum(x^2) per tensor of the MEAN; the owner of each chunk has it in
    registers. Every rank must end up with the same bits, equal to the oracle's piece-wise restatement."""
    sizes = SIZES + [2048 * 37, 9, 2048 * 3]
    for skew, blocks in ((0, 0), (0, 3), (1, 2)):
        _, g0, p, g, m, v = make_case(world, sizes, seed=9, skew=skew)
        got = np.zeros((world, len(sizes)), np.float64)
        rc, status = sim_step(world, sizes, p, g, m, v, [0.0] * len(sizes), H, 1, adam=False, mode=2,
                              blocks_per_rank=blocks, sumsq=got)
        assert rc == 0 and status == [0] * world
        means = [pyoracle.mean_ranks([g0[r][s] for r in range(world)]) for s in range(len(sizes))]
        want = pyoracle.sumsq_pieces(means, world, counter("last_blocks"), vec=(skew == 0))
        for r in range(world):
            for s in range(len(sizes)):
                np.testing.assert_array_equal(g[r][s].get(), means[s])
            assert list(got[r]) == want, (r, list(got[r]), want)
        exact = [float(np.sum(x.astype(np.float64) ** 2)) for x in means]
        np.testing.assert_allclose(want, exact, rtol=1e-13)

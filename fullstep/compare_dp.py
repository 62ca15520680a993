"""Runs the training function of the reference's own distributed test (tests/test_distributed.py:22-38, compiled
unmodified) -- two ranks, three steps of the tiny GPT -- once on this library's data-parallel path and once on the
reference's own (NCCL ncclAvg + k_adamw, selected with SOLITON_FULLSTEP_DP=reference), plus the single-process run
the test compares with, and reports how the three relate.

With two ranks the mean is (a + b) / 2 whoever computes it, so the two paths must give the same bits. The
reference's assertion (2 ranks == 1 process within rtol 1e-4, atol 1e-6) is evaluated for both: whether it holds
depends on the GEMM library's numerics on the GPU at hand, not on the path.

    python fullstep/compare_dp.py        # one JSON line: "COMPARE {...}"
"""
import json
import multiprocessing as mp
import os
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")
sys.path[:0] = [REF, os.path.join(REF, "reftests"), os.path.dirname(HERE)]
from fullstep.build import ensure_importable  # noqa: E402
ensure_importable()


def run_mode(mode):
    """Parameters after the reference test's training: {(rank, world): [arrays]} for 2 ranks and for 1 process."""
    import test_distributed as td
    os.environ["SOLITON_FULLSTEP_DP"] = mode      # inherited by the spawned ranks
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    init_file = os.path.join(tempfile.mkdtemp(), "group_id")
    procs = [ctx.Process(target=td.train, args=(r, 2, init_file, q)) for r in range(2)]
    procs.append(ctx.Process(target=td.train, args=(0, 1, None, q)))
    for p in procs:
        p.start()
    results = {(r, w): params for r, w, params in (q.get(timeout=300) for _ in procs)}
    for p in procs:
        p.join(timeout=60)
    return results


def outside_tolerance(a, b):
    return int(np.sum(np.abs(a - b) > 1e-6 + 1e-4 * np.abs(b)))   # numpy.testing.assert_allclose(rtol=1e-4, atol=1e-6)


def main():
    ours, theirs = run_mode("ours"), run_mode("reference")
    same_bits = all(np.array_equal(x, y) for key in ours for x, y in zip(ours[key], theirs[key]))
    ranks_equal = all(np.array_equal(x, y) for x, y in zip(ours[(0, 2)], ours[(1, 2)]))
    out = {"paths_bit_identical": bool(same_bits), "ranks_bit_identical": bool(ranks_equal),
           "elements": int(sum(a.size for a in ours[(0, 1)])),
           "outside_reference_tolerance_ours": sum(outside_tolerance(a, s) for a, s in zip(ours[(0, 2)], ours[(0, 1)])),
           "outside_reference_tolerance_reference_path": sum(outside_tolerance(a, s) for a, s in zip(theirs[(0, 2)], theirs[(0, 1)])),
           "max_abs_difference_two_ranks_vs_one_process": float(max(np.max(np.abs(a - s)) for a, s in zip(ours[(0, 2)], ours[(0, 1)])))}
    print("COMPARE " + json.dumps(out), flush=True)


if __name__ == "__main__":
    main()

"""Whole training steps: the UNMODIFIED Soliton Python package and its example trainer (compiled into fullstep/_ref/)
on top of this repository's library -- forward and backward on the reference's own CUDA backend, gradient mean and
AdamW on this library's kernels. The reference's own tests are run as they are (its cpu-device cases left out: this
library has no host kernels), and its trainer is run with the memory plan checked against the pool."""
import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "fullstep", "_ref")
# Tests of the reference that build their model on the "cpu" device inside the test body.
NEEDS_HOST_KERNELS = {"test_memory::test_checkpoint_gives_same_grads_and_less_memory[]"}


def ready():
    sys.path.insert(0, ROOT)
    from fullstep.build import ensure_importable
    ensure_importable()
    return all(os.path.exists(os.path.join(REF, p)) for p in
               ("soliton/__init__.pyc", "soliton/libsoliton.so", "soliton/libsoliton_ref_cuda.so", "gpt2.pyc", "reftests"))


def run(script, *args, timeout=1500):
    r = subprocess.run([sys.executable, os.path.join(ROOT, "fullstep", script), *args], capture_output=True, text=True,
                       timeout=timeout, cwd=ROOT)
    assert r.returncode == 0, (r.stdout[-2000:], r.stderr[-3000:])
    return r.stdout


def tagged(out, tag):
    return json.loads([l for l in out.splitlines() if l.startswith(tag + " ")][-1][len(tag) + 1:])


@pytest.fixture(scope="module")
def fullstep(cuda):
    if not ready():
        pytest.skip("fullstep/_ref is not built (no reference checkout at build time)")
    return True


def test_the_reference_own_tests_pass_on_this_library(fullstep):
    res = tagged(run("run_reftests.py", "test_ops", "test_fusion", "test_memory", "test_arena", "test_preflight"), "REFTESTS")
    unexpected = [f for f in res["failed"] if f["test"] not in NEEDS_HOST_KERNELS]
    assert not unexpected, unexpected
    assert res["passed"] >= 35 and res["left_out_cpu_device"] > 0


def test_single_rank_training_steps_and_exact_memory_prediction(fullstep):
    for extra in ([], ["--no-arena"]):
        res = tagged(run("run_gpt2.py", "--config", "tiny", "--batch", "4", "--seq", "64", "--steps", "6", "--hash", *extra), "FULLSTEP")
        assert res["prediction_error_bytes"] == 0, res     # the meta dry run predicted the real peak to the byte
        assert res["loss_last"] < res["loss_first"] and res["tokens_per_s"] > 0


def test_the_reference_distributed_test_gives_the_bits_of_the_reference_path(fullstep, lib):
    """tests/test_distributed.py of the reference: two ranks against one process on the tiny GPT. Its training function
    runs on this library's path and on the reference's own NCCL + k_adamw path: same bits. Its tolerance check is
    evaluated for both and must come out alike (on a B200 a single bias element misses atol 1e-6 by 1.6e-7 with
    either path: the forward and backward GEMMs of batch 4 and batch 8 round differently)."""
    if lib.sl_cuda_count() < 2:
        pytest.skip("needs 2 GPUs")
    res = tagged(run("compare_dp.py"), "COMPARE")
    assert res["paths_bit_identical"] and res["ranks_bit_identical"], res
    assert res["outside_reference_tolerance_ours"] == res["outside_reference_tolerance_reference_path"], res
    assert res["max_abs_difference_two_ranks_vs_one_process"] < 1e-5, res


@pytest.mark.parametrize("world", [2, 8])
def test_data_parallel_training_steps_are_bit_identical_across_ranks(fullstep, lib, world):
    if lib.sl_cuda_count() < world:
        pytest.skip(f"needs {world} GPUs")
    res = tagged(run("run_gpt2.py", "--config", "tiny", "--batch", "4", "--seq", "64", "--steps", "10", "--hash",
                     "--nproc", str(world)), "FULLSTEP")
    assert res["bit_identical_across_ranks"] is True, res["sha256_per_rank"]
    assert set(res["prediction_error_bytes_per_rank"]) == {0}

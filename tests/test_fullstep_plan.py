"""The allocator and the scratch order of every op, pinned against numbers the reference itself published.

The unmodified Soliton Python package (compiled into fullstep/_ref/ by fullstep/build.py) runs its own GPT-2 example
on the meta device on top of this repository's library: every parameter, activation, gradient and per-op scratch
buffer goes through csrc/pool.cpp and fullstep/ops_dispatch.cpp. The sizes that come out are compared with the
reference's own published measurements on its own core (bench/results/fp32/e1.json of the reference: GPT-2 124M,
sequence 1024, `predicted` of the "soliton+arena" rows, which equals what its GPU run then reserved). No GPU needed."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "fullstep", "_ref")

# batch -> arena bytes, bench/results/fp32/e1.json (framework "soliton+arena", key "predicted")
PUBLISHED_ARENA = {1: 2791476224, 2: 3735997440, 4: 5780229120, 8: 9872886784}
# batch -> pool peak reserved / peak allocated (framework "soliton", keys "predicted" / "predicted_alloc")
PUBLISHED_POOL = {1: (3563441152, 2825031168), 4: (6807277056, 5813784064), 8: (11025126400, 9906441728)}

SCRIPT = r'''
import json, sys
sys.path.insert(0, sys.argv[1])
import soliton as sl, gpt2
out = {"arena": {}, "pool": {}}
for b in (1, 2, 4, 8):
    p = sl.arena.plan(lambda d: gpt2.run(d, "124M", b, 1024, 1, 2))
    out["arena"][b] = [p.bytes, p.live_peak, len(p.sizes)]
for b in (1, 4, 8):
    s = sl.plan(lambda d: gpt2.run(d, "124M", b, 1024, 1, 2))
    out["pool"][b] = [s["peak_reserved"], s["peak_allocated"]]
print("PLAN " + json.dumps(out))
'''


@pytest.fixture(scope="module")
def plans(built):
    sys.path.insert(0, ROOT)
    from fullstep import build as fb
    fb.build()
    fb.ensure_importable()
    if not os.path.exists(os.path.join(REF, "soliton", "__init__.pyc")):
        pytest.skip("the reference's Python package is not compiled (no reference checkout at build time)")
    r = subprocess.run([sys.executable, "-c", SCRIPT, REF], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    line = [l for l in r.stdout.splitlines() if l.startswith("PLAN ")][-1]
    return json.loads(line[5:])


def test_arena_bytes_equal_the_reference_published_numbers(plans):
    for batch, want in PUBLISHED_ARENA.items():
        got, live_peak, blocks = plans["arena"][str(batch)]
        assert got == want, (batch, got, want)
        assert got >= live_peak and blocks > 1000


def test_pool_peaks_differ_from_the_published_ones_by_the_fixed_workspace_only(plans):
    """The pool numbers contain what device initialisation reserves: the reference 32 MiB for cuBLAS, this library
    18 MiB more for the data-parallel path. The published runs differ from that by one further 512-byte block, the
    same at every batch size and in both counters: a constant of device initialisation in the build that produced
    them, not of any step."""
    deltas = set()
    for batch, (reserved, allocated) in PUBLISHED_POOL.items():
        got_r, got_a = plans["pool"][str(batch)]
        deltas.add(got_r - reserved)
        deltas.add(got_a - allocated)
    assert deltas == {(18 << 20) - 512}

"""The hardened launcher (soliton_b200/launch.py) against what examples/gpt2.py:153-159 of the reference leaves open:
a rank that fails must end the job, a time limit must hold, and nothing may stay behind. CPU only: the ranks here
are small Python scripts."""
import os
import sys
import time

from soliton_b200.launch import TIMEOUT_EXIT, launch_workers


def script(body):
    return [sys.executable, "-c", "import os, sys, time\n" + body]


def test_all_ranks_succeed_and_the_group_directory_is_removed(tmp_path):
    out = tmp_path / "seen"
    out.mkdir()
    body = (f"r = os.environ['RANK']; w = os.environ['WORLD_SIZE']; f = os.environ['SOLITON_INIT_FILE']\n"
            f"open(os.path.join({str(out)!r}, r), 'w').write(w + ' ' + f + ' ' + os.environ['LOCAL_RANK'])\n")
    assert launch_workers(3, script(body), timeout=30) == 0
    seen = {name: (out / name).read_text().split() for name in os.listdir(out)}
    assert sorted(seen) == ["0", "1", "2"]
    files = {v[1] for v in seen.values()}
    assert len(files) == 1 and all(v[0] == "3" for v in seen.values())      # same world size and id file everywhere
    assert [seen[str(r)][2] for r in range(3)] == ["0", "1", "2"]
    assert not os.path.exists(os.path.dirname(files.pop()))                   # the temporary directory is gone


def test_a_failing_rank_ends_the_others_and_its_code_is_returned(tmp_path):
    marker = tmp_path / "survivor_finished"
    body = (f"if os.environ['RANK'] == '1':\n    sys.exit(7)\n"
            f"time.sleep(60)\nopen({str(marker)!r}, 'w').write('x')\n")
    t0 = time.monotonic()
    assert launch_workers(2, script(body), timeout=120, grace=2.0) == 7
    assert time.monotonic() - t0 < 30          # did not wait for the sleeping rank
    assert not marker.exists()


def test_time_limit(tmp_path):
    t0 = time.monotonic()
    assert launch_workers(2, script("time.sleep(60)\n"), timeout=1.0, grace=2.0) == TIMEOUT_EXIT
    assert time.monotonic() - t0 < 30


def test_a_rank_that_ignores_sigterm_is_killed(tmp_path):
    body = ("import signal\nsignal.signal(signal.SIGTERM, signal.SIG_IGN)\n"
            "if os.environ['RANK'] == '0':\n    time.sleep(0.5); sys.exit(3)\ntime.sleep(60)\n")
    t0 = time.monotonic()
    assert launch_workers(2, script(body), timeout=120, grace=1.0) == 3
    assert time.monotonic() - t0 < 30

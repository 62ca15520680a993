"""One process per GPU on one box: the launcher of Soliton's example (examples/gpt2.py:153-159), hardened.

The reference starts the ranks and waits for each in turn, whatever happens: a rank that dies leaves its peers
blocked in their next collective for good, the group-id directory is never removed, and nothing bounds the run.
Here the ranks are watched together: the first failure, or the time limit, ends the others (first SIGTERM to exactly
the processes started here, SIGKILL after a grace period), the exit code says what happened, and the temporary
directory of the group id goes away in every case. The environment contract is the reference's: RANK, WORLD_SIZE,
SOLITON_INIT_FILE (and LOCAL_RANK, which python/soliton/tensor.py:26 reads).
"""
import os
import shutil
import signal
import subprocess
import sys
import tempfile
import time

TIMEOUT_EXIT = 124   # like timeout(1)


def _stop(procs, grace):
    """Ends the given children: SIGTERM, then SIGKILL for those still alive after `grace` seconds."""
    alive = [p for p in procs if p.poll() is None]
    for p in alive:
        p.terminate()
    deadline = time.monotonic() + grace
    for p in alive:
        try:
            p.wait(timeout=max(0.0, deadline - time.monotonic()))
        except subprocess.TimeoutExpired:
            p.kill()
            p.wait()


def launch_workers(nproc, argv=None, timeout=None, grace=10.0, env=None, poll=0.05):
    """Runs `argv` (default: this script again) once per rank and returns the job's exit code: 0 when every rank
    returned 0; the first non-zero code a rank returned (the other ranks are stopped at that moment); TIMEOUT_EXIT
    when `timeout` seconds passed first. A rank killed by a signal counts as 128 + signal."""
    argv = [sys.executable, *sys.argv] if argv is None else list(argv)
    workdir = tempfile.mkdtemp(prefix="soliton_group_")
    init_file = os.path.join(workdir, "group_id")
    base = dict(os.environ if env is None else env)
    procs = []
    try:
        for rank in range(nproc):
            procs.append(subprocess.Popen(argv, env=dict(base, RANK=str(rank), LOCAL_RANK=str(rank),
                                                         WORLD_SIZE=str(nproc), SOLITON_INIT_FILE=init_file)))
        deadline = None if timeout is None else time.monotonic() + timeout
        while True:
            codes = [p.poll() for p in procs]
            failed = [c for c in codes if c not in (None, 0)]
            if failed:
                _stop(procs, grace)
                return failed[0] if failed[0] > 0 else 128 - failed[0]
            if all(c == 0 for c in codes):
                return 0
            if deadline is not None and time.monotonic() > deadline:
                _stop(procs, grace)
                return TIMEOUT_EXIT
            time.sleep(poll)
    except BaseException:
        _stop(procs, grace)   # the launcher itself is going down (Ctrl-C, an exception): take the ranks along
        raise
    finally:
        shutil.rmtree(workdir, ignore_errors=True)


def rank_env():
    """(rank, world, init_file) of this process as the launcher set them; (0, 1, None) outside a launched job."""
    return int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), os.environ.get("SOLITON_INIT_FILE")


if __name__ == "__main__":
    # python -m soliton_b200.launch NPROC [--timeout S] -- command ...
    args = sys.argv[1:]
    n = int(args.pop(0))
    limit = None
    if args and args[0] == "--timeout":
        limit = float(args[1])
        args = args[2:]
    if args and args[0] == "--":
        args = args[1:]
    sys.exit(launch_workers(n, args, timeout=limit))

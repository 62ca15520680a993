"""Runs the reference's OWN tests (compiled unmodified into fullstep/_ref/reftests/ by fullstep/build.py) against the
unmodified Soliton Python package on top of this repository's library.

The reference parametrises its tests over the devices "cpu" and "cuda" (tests/test_ops.py:9 and the like). This
library has no host kernels, so the cases that run on "cpu" are left out and counted as such; everything that runs on
"meta" and "cuda" is called exactly as pytest would call it, with the arguments of the test's own parametrize marks.

    python fullstep/run_reftests.py [module ...]        # prints one JSON line: passed / failed / left out
"""
import importlib
import itertools
import json
import os
import sys
import traceback

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")
sys.path[:0] = [REF, os.path.join(REF, "reftests"), os.path.dirname(HERE)]   # the first two: what the reference's tests/conftest.py:4-5 puts on the path
from fullstep.build import ensure_importable  # noqa: E402
ensure_importable()


def cases_of(fn):
    """Argument dicts of a test function, from its parametrize marks (the cartesian product, as pytest forms it)."""
    axes = []
    for mark in getattr(fn, "pytestmark", []):
        if mark.name != "parametrize":
            continue
        names = [n.strip() for n in mark.args[0].split(",")]
        values = [v if len(names) > 1 else (v,) for v in mark.args[1]]
        axes.append([dict(zip(names, v)) for v in values])
    out = []
    for combo in itertools.product(*axes):
        merged = {}
        for part in combo:
            merged.update(part)
        out.append(merged)
    return out or [{}]


def clear_sticky_error():
    from soliton._C import lib
    try:
        lib.slb_clear_error()
    except AttributeError:   # another build of libsoliton.so
        pass


def skipped_by_module(mod):
    mark = getattr(mod, "pytestmark", None)
    marks = mark if isinstance(mark, list) else [mark] if mark is not None else []
    return any(m.name == "skipif" and m.args and m.args[0] for m in marks)


def run(modules):
    passed, failed, left_out, skipped = [], [], [], []
    for name in modules:
        mod = importlib.import_module(name)
        if skipped_by_module(mod):
            skipped.append(name)
            continue
        for attr in sorted(dir(mod)):
            fn = getattr(mod, attr)
            if not attr.startswith("test_") or not callable(fn):
                continue
            for kwargs in cases_of(fn):
                label = f"{name}::{attr}[{'-'.join(str(v) for v in kwargs.values())}]"
                if kwargs.get("device") == "cpu":
                    left_out.append(label)
                    continue
                try:
                    fn(**kwargs)
                    passed.append(label)
                except BaseException as e:   # a failing assert must not hide the tests after it
                    failed.append({"test": label, "error": "".join(traceback.format_exception_only(type(e), e)).strip()[-400:]})
                    clear_sticky_error()     # nor may the library's sticky error code fail them in its wake
    return {"passed": len(passed), "failed": failed, "left_out_cpu_device": len(left_out), "skipped_modules": skipped,
            "passed_tests": passed}


if __name__ == "__main__":
    mods = sys.argv[1:] or ["test_ops", "test_fusion", "test_memory", "test_arena", "test_preflight", "test_distributed"]
    print("REFTESTS " + json.dumps(run(mods)), flush=True)

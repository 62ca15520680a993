"""The shared library loads without a GPU and exports every function include/soliton_b200.h declares."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "soliton_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(sl[b]?_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported(lib):
    names = declared_functions()
    assert len(names) >= 45
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing


def test_binding_table_covers_the_header(lib):
    from soliton_b200 import _C
    assert set(_C._SIGS) == set(declared_functions())


def test_compute_on_cpu_is_refused_loudly(lib):
    buf = (ctypes.c_float * 8)()
    lib.slb_clear_error()
    lib.sl_adamw(0, buf, buf, buf, buf, 8, 1e-3, 0.9, 0.999, 1e-8, 0.0, 1)
    assert lib.sl_check(0) == 13
    lib.slb_clear_error()
    assert lib.sl_check(0) == 0


def test_meta_calls_do_no_work_and_report_success(lib):
    lib.slb_clear_error()
    assert lib.sl_dist_group(1, 1) == 0 and lib.sl_dist_allreduce_mean(1, None, 10) == 0 and lib.sl_dist_group(1, 0) == 0
    lib.sl_adamw(1, None, None, None, None, 10, 1e-3, 0.9, 0.999, 1e-8, 0.0, 1)
    assert lib.sl_check(1) == 0


def test_path_without_device_fails_instead_of_falling_back(lib):
    if lib.sl_cuda_count() > 0:
        return  # on a GPU box the device tests cover the real path
    lib.slb_clear_error()
    buf = (ctypes.c_float * 8)()
    lib.sl_adamw(2, buf, buf, buf, buf, 8, 1e-3, 0.9, 0.999, 1e-8, 0.0, 1)
    assert lib.sl_check(2) == 14  # device never initialised: no silent host path
    assert lib.sl_init_device(2, 0) == -1
    lib.slb_clear_error()

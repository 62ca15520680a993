"""ctypes bindings to libsoliton_b200.so.

Mirrors python/soliton/_C.py:5-70 for the symbols of the data-parallel optimizer path: the same names, result and
argument types, resolved eagerly at import so that a missing symbol fails here and not in the middle of a step.
There is no fallback: if the library is not built, importing this module raises.
"""
import ctypes as C
import os

_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "libsoliton_b200.so")
if not os.path.exists(_PATH):
    raise ImportError(f"soliton_b200: {_PATH} is not built; run `python -m soliton_b200.build` (needs nvcc)")
lib = C.CDLL(_PATH)

P, L, I, F, D, S = C.c_void_p, C.c_int64, C.c_int, C.c_float, C.c_double, C.c_size_t
LP = C.POINTER(C.c_int64)
PP = C.POINTER(C.c_void_p)

# Subset of python/soliton/_C.py:11-67 that lies on the path or serves its callers; identical signatures.
_SIGS = {
    "sl_alloc": (P, [I, S]),
    "sl_free": (None, [I, P, S]),
    "sl_stats": (None, [I, LP]),
    "sl_reset_stats": (None, [I]),
    "sl_empty_cache": (None, [I]),
    "sl_set_limit": (None, [I, L]),
    "sl_record_start": (None, [I]),
    "sl_record_stop": (None, [I]),
    "sl_record_mark": (None, [I]),
    "sl_record_count": (L, [I]),
    "sl_record_body": (L, [I]),
    "sl_record_get": (None, [I, LP, LP, LP]),
    "sl_arena_install": (I, [I, LP, LP, L, L, L]),
    "sl_arena_diverged": (I, [I]),
    "sl_arena_off": (None, [I]),
    "sl_init_device": (I, [I, I]),
    "sl_cuda_count": (I, []),
    "sl_check": (I, [I]),
    "sl_sync": (None, [I]),
    "sl_mem_info": (None, [C.POINTER(S), C.POINTER(S)]),
    "sl_from_host": (None, [I, P, P, S]),
    "sl_to_host": (None, [I, P, P, S]),
    "sl_copy": (None, [I, P, P, S]),
    "sl_fill": (None, [I, P, L, F]),
    "sl_axpy": (None, [I, P, P, L, F]),
    "sl_scale": (None, [I, P, P, L, F]),
    "sl_sumsq": (D, [I, P, L]),
    "sl_adamw": (None, [I, P, P, P, P, L, F, F, F, F, F, I]),
    "sl_dist_unique_id": (I, [C.c_char_p]),
    "sl_dist_init": (I, [I, I, C.c_char_p]),
    "sl_dist_group": (I, [I, I]),
    "sl_dist_allreduce_mean": (I, [I, P, L]),
    "sl_dist_destroy": (None, []),
    # backend level (core/soliton/api.d:47-48,58-62)
    "sl_cuda_adamw": (None, [P, P, P, P, L, F, F, F, F, F, I]),
    "sl_cuda_nccl_unique_id": (I, [C.c_char_p]),
    "sl_cuda_nccl_init": (I, [I, I, C.c_char_p]),
    "sl_cuda_nccl_group": (I, [I]),
    "sl_cuda_nccl_allreduce_mean": (I, [P, L]),
    "sl_cuda_nccl_destroy": (None, []),
    "sl_cuda_dp_set_workspace": (I, [P, S]),
    # additions of this library
    "slb_workspace_bytes": (S, []),
    "slb_set_option": (I, [C.c_char_p, L]),
    "slb_get_counter": (L, [C.c_char_p]),
    "slb_flush": (None, []),
    "slb_clear_error": (None, []),
    "slb_tile_count": (L, [LP, I]),
    "slb_run_range": (None, [L, I, I, I, I, LP, LP]),
    "slb_adamw_step_static": (I, [I, PP, PP, PP, PP, LP, C.POINTER(F), F, F, F, F, I]),
    "slb_sim_step": (I, [I, I, LP, PP, PP, PP, PP, C.POINTER(F), F, F, F, F, I, I, I, I, L, C.c_uint, C.POINTER(I)]),
    "slb_rdv_selftest": (I, [C.c_char_p, I, I, I]),
    "slb_rdv_create_id": (I, [C.c_char_p]),
}
for _name, (_res, _args) in _SIGS.items():
    _fn = getattr(lib, _name)
    _fn.restype, _fn.argtypes = _res, _args


def longs(xs):
    xs = list(xs)
    return (C.c_int64 * max(len(xs), 1))(*xs)


def set_option(name, value):
    if lib.slb_set_option(name.encode(), int(value)) != 0:
        raise KeyError(f"soliton_b200: unknown option {name!r}")


def counter(name):
    return lib.slb_get_counter(name.encode())

"""ctypes front end of oracle/liboracle.so (the CPU restatement in oracle/oracle.c). Test infrastructure only."""
import ctypes as C
import os

import numpy as np

from . import build as _build

_lib = None
FP = C.POINTER(C.c_float)
FPP = C.POINTER(FP)


def lib():
    global _lib
    if _lib is None:
        path = _build.ORACLE_SO if os.path.exists(_build.ORACLE_SO) and not _stale() else _build.build_oracle()
        _lib = C.CDLL(path)
        _lib.oracle_sumsq.restype = C.c_double
        _lib.oracle_clip.restype = C.c_double
        _lib.oracle_bench.restype = C.c_double
        _lib.oracle_sumsq_piece.restype = C.c_double
    return _lib


def _stale():
    src = os.path.join(_build.HERE, "oracle.c")
    return os.path.getmtime(src) > os.path.getmtime(_build.ORACLE_SO)


def _fp(a):
    assert a.dtype == np.float32 and a.flags.c_contiguous
    return a.ctypes.data_as(FP)


def adamw(p, g, m, v, lr, b1, b2, eps, wd, step, fma=False):
    """In place on float32 arrays. fma=False: the host kernel (cpu.d); fma=True: the shape nvcc gives k_adamw."""
    fn = lib().oracle_adamw_fma if fma else lib().oracle_adamw
    fn(_fp(p), _fp(g), _fp(m), _fp(v), C.c_int64(p.size), C.c_float(lr), C.c_float(b1), C.c_float(b2),
       C.c_float(eps), C.c_float(wd), C.c_int(step))


def mean_ranks(grads):
    """Mean of per-rank float32 arrays in rank order: ((g0 + g1) + ...) * (1 / world)."""
    out = np.empty_like(grads[0])
    arr = (FP * len(grads))(*[_fp(np.ascontiguousarray(g)) for g in grads])
    lib().oracle_mean_ranks(arr, C.c_int(len(grads)), C.c_int64(out.size), _fp(out))
    return out


def sumsq(x):
    return lib().oracle_sumsq(_fp(x), C.c_int64(x.size))


def axpy(x, y, alpha):
    lib().oracle_axpy(_fp(x), _fp(y), C.c_int64(x.size), C.c_float(alpha))


def scale(x, y, alpha):
    lib().oracle_scale(_fp(x), _fp(y), C.c_int64(x.size), C.c_float(alpha))


def clip(grads, max_norm):
    arr = (FP * len(grads))(*[_fp(g) for g in grads])
    ns = (C.c_int64 * len(grads))(*[g.size for g in grads])
    return lib().oracle_clip(arr, ns, C.c_int(len(grads)), C.c_double(max_norm))


def bench(p0, grads, reps, threads):
    """Seconds for `reps` host steps (sum ranks, scale, adamw) on each of `threads` threads; the slowest thread."""
    arr = (FP * len(grads))(*[_fp(g) for g in grads])
    return lib().oracle_bench(_fp(p0), arr, C.c_int(len(grads)), C.c_int64(p0.size), C.c_int(reps), C.c_int(threads))


TILE = 2048


def sumsq_pieces(tensors, world, blocks, vec=True):
    """Per-tensor sum of squares as the two-shot gradient mean leaves it behind: the step's tensors, each padded to
    whole tiles, form one tile sequence; rank c's chunk is tiles [T*c//world, T*(c+1)//world), block b's run inside a
    chunk of length L starts at L*b//blocks. A piece starts where a run starts and where a tensor starts; a tensor's
    pieces are added in tile order. `vec`: per tensor (or one flag for all) whether it is 32-byte aligned."""
    ns = [int(t.size) for t in tensors]
    prefix = [0]
    for n in ns:
        prefix.append(prefix[-1] + (n + TILE - 1) // TILE)
    total = prefix[-1]
    starts = set(prefix[i] for i in range(len(ns)) if prefix[i + 1] > prefix[i])
    for c in range(world):
        cb = total * c // world
        length = total * (c + 1) // world - cb
        for b in range(blocks):
            r0, r1 = cb + length * b // blocks, cb + length * (b + 1) // blocks
            if r1 > r0:
                starts.add(r0)
    bounds = sorted(starts) + [total]
    flags = [vec] * len(ns) if isinstance(vec, bool) else list(vec)
    sums = [0.0] * len(ns)
    seg = 0
    for lo, hi in zip(bounds[:-1], bounds[1:]):
        while prefix[seg + 1] <= lo:
            seg += 1
        x = np.ascontiguousarray(tensors[seg], np.float32).ravel()
        sums[seg] += lib().oracle_sumsq_piece(_fp(x), C.c_int64(x.size), C.c_int64(lo - prefix[seg]),
                                              C.c_int64(hi - prefix[seg]), C.c_int(1 if flags[seg] else 0))
    return sums

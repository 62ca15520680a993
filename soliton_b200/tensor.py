"""The slice of python/soliton/tensor.py the optimizer path touches: devices, pool statistics, storage, and a plain
contiguous float32 tensor with `.ptr/.numel/.ndim/.grad` -- enough for soliton's AdamW, clip_grad_norm and
all_reduce_grads to run unchanged in meaning. No autograd, no ops: those are not part of this path.
"""
import ctypes
import os

import numpy as np

from ._C import lib

DEVICES = ("cpu", "meta", "cuda")
CPU, META, CUDA = 0, 1, 2

_ordinal = int(os.environ.get("LOCAL_RANK", 0))
_ready = set()


def set_device(ordinal):
    """python/soliton/tensor.py:31-36"""
    global _ordinal
    if CUDA in _ready and ordinal != _ordinal:
        raise RuntimeError("soliton: CUDA device already initialized")
    _ordinal = ordinal


def _dev(device):
    """python/soliton/tensor.py:39-47: first use of a device initialises it (and makes its fixed reservations)."""
    d = device if isinstance(device, int) else DEVICES.index(device)
    if d not in _ready:
        if d == CUDA and lib.sl_cuda_count() <= _ordinal:
            raise RuntimeError(f"soliton: no CUDA device {_ordinal}")
        if lib.sl_init_device(d, _ordinal) != 0:
            raise RuntimeError(f"soliton: cannot initialize {DEVICES[d]}")
        _ready.add(d)
    return d


def _check(d):
    """python/soliton/tensor.py:50-53"""
    err = lib.sl_check(d)
    if err:
        raise RuntimeError(f"soliton: {DEVICES[d]} error code {err}")


_STAT_KEYS = ("allocated", "reserved", "peak_allocated", "peak_reserved", "n_alloc", "n_raw", "trace")


def memory_stats(device="cuda"):
    buf = (ctypes.c_int64 * 7)()
    lib.sl_stats(_dev(device), buf)
    return dict(zip(_STAT_KEYS, buf))


def reset_peak_stats(device="cuda"):
    lib.sl_reset_stats(_dev(device))


def empty_cache(device="cuda"):
    lib.sl_empty_cache(_dev(device))


def set_memory_limit(device, nbytes):
    lib.sl_set_limit(_dev(device), int(nbytes))


def synchronize():
    """python/soliton/tensor.py:106-109"""
    if CUDA in _ready:
        lib.sl_sync(CUDA)
        _check(CUDA)


class Storage:
    """python/soliton/tensor.py:130-147: sl_alloc on construction, sl_free with the unrounded size on collection."""
    __slots__ = ("dev", "ptr", "nbytes")

    def __init__(self, dev, nbytes):
        ptr = lib.sl_alloc(dev, nbytes)
        if not ptr:
            raise MemoryError(f"soliton: out of memory on {DEVICES[dev]} allocating {nbytes} bytes")
        self.dev, self.ptr, self.nbytes = dev, ptr, nbytes

    def __del__(self):
        try:
            lib.sl_free(self.dev, self.ptr, self.nbytes)
        except Exception:  # interpreter shutdown, or __init__ failed
            pass


class Tensor:
    """Contiguous float32 tensor on one of the three devices."""
    __slots__ = ("storage", "shape", "grad")

    def __init__(self, storage, shape):
        self.storage, self.shape, self.grad = storage, tuple(int(s) for s in shape), None

    dev = property(lambda self: self.storage.dev)
    ptr = property(lambda self: self.storage.ptr)
    ndim = property(lambda self: len(self.shape))

    @property
    def numel(self):
        n = 1
        for s in self.shape:
            n *= s
        return n

    def numpy(self):
        """python/soliton/tensor.py:194-200: blocking copy to the host, then the sticky error check."""
        if self.dev == META:
            raise RuntimeError("soliton: meta tensors have no data")
        out = np.empty(self.shape, np.float32)
        lib.sl_to_host(self.dev, out.ctypes.data, self.ptr, out.nbytes)
        _check(self.dev)
        return out

    def copy_from(self, array):
        a = np.ascontiguousarray(array, np.float32)
        assert a.size == self.numel
        lib.sl_from_host(self.dev, self.ptr, a.ctypes.data, a.nbytes)
        return self


def empty(shape, device="cpu"):
    d = _dev(device)
    shape = tuple(shape) if hasattr(shape, "__len__") else (int(shape),)
    n = 1
    for s in shape:
        n *= int(s)
    return Tensor(Storage(d, n * 4), shape)


def zeros(shape, device="cpu"):
    t = empty(shape, device)
    lib.sl_fill(t.dev, t.ptr, t.numel, 0.0)
    return t


def tensor(array, device="cpu"):
    a = np.asarray(array, np.float32)
    t = empty(a.shape, device)
    if t.dev != META:
        t.copy_from(a)
    return t


def sumsq(t):
    return lib.sl_sumsq(t.dev, t.ptr, t.numel)

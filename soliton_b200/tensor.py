"""Devices, pool statistics, storage and a plain float32 tensor: the part of Soliton's `tensor` module
(python/soliton/tensor.py:22-147,194-200) that the optimizer path and its callers touch. Same public names and
behaviour; no autograd and no ops, which are not on this path.

A `Runtime` object keeps what the reference keeps in module globals (chosen CUDA ordinal, which device kinds have
been initialised); the module-level functions are its methods.
"""
import ctypes
import os

import numpy as np

from ._C import lib

DEVICES = ("cpu", "meta", "cuda")
CPU, META, CUDA = range(3)
_STATS = ("allocated", "reserved", "peak_allocated", "peak_reserved", "n_alloc", "n_raw", "trace")


def _count(shape):
    total = 1
    for extent in shape:
        total *= int(extent)
    return total


class Runtime:
    def __init__(self):
        self.ordinal = int(os.environ.get("LOCAL_RANK", 0))  # tensor.py:26
        self.ready = set()

    def set_device(self, ordinal):
        """tensor.py:31-36: pick the CUDA device of this process, before its first CUDA use."""
        if CUDA in self.ready and ordinal != self.ordinal:
            raise RuntimeError("soliton: CUDA device already initialized")
        self.ordinal = ordinal

    def device(self, spec):
        """tensor.py:39-47: device kind of a name or number; the first use initialises the device, which is when
        its fixed reservations (BLAS workspace, data-parallel workspace) are taken from the pool."""
        kind = DEVICES.index(spec) if isinstance(spec, str) else int(spec)
        if kind in self.ready:
            return kind
        if kind == CUDA and lib.sl_cuda_count() <= self.ordinal:
            raise RuntimeError(f"soliton: no CUDA device {self.ordinal}")
        if lib.sl_init_device(kind, self.ordinal) != 0:
            raise RuntimeError(f"soliton: cannot initialize {DEVICES[kind]}")
        self.ready.add(kind)
        return kind

    def check(self, kind):
        """tensor.py:50-53: the library's sticky error as an exception."""
        code = lib.sl_check(kind)
        if code:
            raise RuntimeError(f"soliton: {DEVICES[kind]} error code {code}")

    def stats(self, spec):
        raw = (ctypes.c_int64 * len(_STATS))()
        lib.sl_stats(self.device(spec), raw)
        return {name: raw[i] for i, name in enumerate(_STATS)}


_rt = Runtime()
set_device = _rt.set_device
_dev = _rt.device
_check = _rt.check
_ready = _rt.ready


def memory_stats(device="cuda"):
    return _rt.stats(device)


def reset_peak_stats(device="cuda"):
    lib.sl_reset_stats(_dev(device))


def empty_cache(device="cuda"):
    lib.sl_empty_cache(_dev(device))


def set_memory_limit(device, nbytes):
    """Cap on reserved bytes, 0 for none; on meta this plays a smaller GPU (tensor.py:83-85)."""
    lib.sl_set_limit(_dev(device), int(nbytes))


def synchronize():
    """tensor.py:106-109: wait for the device (pending launches go out first), then raise on a sticky error."""
    if CUDA not in _rt.ready:
        return
    lib.sl_sync(CUDA)
    _check(CUDA)


class Storage:
    """A block from the deterministic pool: sl_alloc when made, sl_free with the unrounded size when collected
    (tensor.py:130-147)."""
    __slots__ = ("dev", "ptr", "nbytes")

    def __init__(self, dev, nbytes):
        self.dev, self.nbytes = dev, nbytes
        self.ptr = lib.sl_alloc(dev, nbytes)
        if not self.ptr:
            raise MemoryError(f"soliton: out of memory on {DEVICES[dev]} allocating {nbytes} bytes")

    def __del__(self):
        ptr = getattr(self, "ptr", None)
        if ptr:
            try:
                lib.sl_free(self.dev, ptr, self.nbytes)
            except Exception:  # interpreter shutdown
                pass


class Tensor:
    """Contiguous float32 data on one device kind; `grad` is whatever the caller hangs on it."""
    __slots__ = ("storage", "shape", "grad")

    def __init__(self, storage, shape):
        self.storage = storage
        self.shape = tuple(int(extent) for extent in shape)
        self.grad = None

    @property
    def dev(self):
        return self.storage.dev

    @property
    def ptr(self):
        return self.storage.ptr

    @property
    def ndim(self):
        return len(self.shape)

    @property
    def numel(self):
        return _count(self.shape)

    def numpy(self):
        """Blocking copy to the host followed by the error check (tensor.py:194-200)."""
        if self.dev == META:
            raise RuntimeError("soliton: meta tensors have no data")
        host = np.empty(self.shape, np.float32)
        lib.sl_to_host(self.dev, host.ctypes.data, self.ptr, host.nbytes)
        _check(self.dev)
        return host

    def copy_from(self, array):
        host = np.ascontiguousarray(array, np.float32)
        if host.size != self.numel:
            raise ValueError("soliton: size mismatch in copy_from")
        lib.sl_from_host(self.dev, self.ptr, host.ctypes.data, host.nbytes)
        return self


def empty(shape, device="cpu"):
    shape = tuple(shape) if hasattr(shape, "__len__") else (int(shape),)
    return Tensor(Storage(_dev(device), 4 * _count(shape)), shape)


def zeros(shape, device="cpu"):
    out = empty(shape, device)
    lib.sl_fill(out.dev, out.ptr, out.numel, 0.0)
    return out


def tensor(array, device="cpu"):
    host = np.asarray(array, np.float32)
    out = empty(host.shape, device)
    return out if out.dev == META else out.copy_from(host)


def sumsq(t):
    return lib.sl_sumsq(t.dev, t.ptr, t.numel)

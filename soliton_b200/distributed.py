"""Data parallel behind the interface of Soliton's `distributed` module (python/soliton/distributed.py:16-53): one
process per GPU, gradients averaged after backward.

What differs underneath: the collective is this library's NVSwitch peer-memory kernel family, not NCCL, and the
128-byte group id names a shared-memory file through which the ranks of one box meet. What does not differ: like
the reference's collective it takes nothing from the pool per step (its workspace is reserved when the device is
initialised, on meta as on cuda), so a single-rank meta dry run remains the exact per-rank memory plan.
"""
import ctypes
import os
import time

from . import tensor as T
from ._C import lib

ID_BYTES = 128


class _Group:
    """The process group of this process: its size, and how to enter and leave it."""
    size = 1

    @classmethod
    def enter(cls, rank, world, blob):
        T.set_device(rank)
        T._dev(T.CUDA)  # the device's workspace must exist before the group maps it for the peers
        if lib.sl_dist_init(rank, world, ctypes.create_string_buffer(bytes(blob), ID_BYTES)) != 0:
            raise RuntimeError(f"soliton: process group init failed on rank {rank}")
        cls.size = world

    @classmethod
    def leave(cls):
        lib.sl_dist_destroy()
        cls.size = 1


def unique_id():
    """The 128 bytes that name a new process group: rank 0 makes them, every rank joins with them."""
    raw = ctypes.create_string_buffer(ID_BYTES)
    if lib.sl_dist_unique_id(raw) != 0:
        raise RuntimeError("soliton: cannot create the process group id")
    return raw.raw


def _publish(path, blob):
    # under a temporary name first: a reader either finds no file or a whole id
    with open(path + ".tmp", "wb") as out:
        out.write(blob)
    os.replace(path + ".tmp", path)


def _await_file(path, rank, timeout):
    deadline = time.monotonic() + timeout
    while not os.path.exists(path):
        if time.monotonic() > deadline:
            raise RuntimeError(f"soliton: rank {rank} waited {timeout:.0f}s for {path}")
        time.sleep(0.05)
    with open(path, "rb") as src:
        return src.read(ID_BYTES)


def init(rank, world, init_file, timeout=300.0):
    """distributed.py:16-35: rank 0 creates the group id and publishes it through `init_file`; the other ranks wait
    for the file -- at most `timeout` seconds, where the reference polls without limit -- and everybody joins."""
    if rank == 0:
        T.set_device(rank)
        T._dev(T.CUDA)
        blob = unique_id()
        _publish(init_file, blob)
    else:
        blob = _await_file(init_file, rank, timeout)
    _Group.enter(rank, world, blob)


def init_with_id(rank, world, id_bytes):
    """Joins a group whose id travelled by other means (for instance a torch.distributed broadcast)."""
    _Group.enter(rank, world, id_bytes)


def world_size():
    return _Group.size


def destroy():
    _Group.leave()


def all_reduce_grads(params):
    """distributed.py:42-53: one group around one in-place mean per gradient; nothing to do for a single process.
    If any call fails the whole all-reduce fails with a RuntimeError, after the group has been closed."""
    grads = [p.grad for p in params if p.grad is not None]
    if _Group.size == 1 or not grads:
        return
    dev = grads[0].dev
    failed = lib.sl_dist_group(dev, 1) != 0
    for g in grads:
        failed |= lib.sl_dist_allreduce_mean(dev, g.ptr, g.numel) != 0
    failed |= lib.sl_dist_group(dev, 0) != 0
    if failed:
        raise RuntimeError("soliton: all-reduce failed")

"""Data parallel with the interface of python/soliton/distributed.py: one process per GPU, gradients averaged
after backward. The collective is this library's own NVSwitch peer-memory kernel family instead of NCCL; like the
reference's, it takes nothing from the pool per step (its workspace is reserved when the device is initialised, on
meta as on cuda), so a single-rank meta dry run stays the exact per-rank memory plan.
"""
import ctypes
import os
import time

from . import tensor as T
from ._C import lib

_world = 1


def init(rank, world, init_file, timeout=300.0):
    """python/soliton/distributed.py:16-35. Rank 0 creates the group id and publishes it through init_file; the
    other ranks wait for it -- for at most `timeout` seconds, where the reference polls forever."""
    global _world
    T.set_device(rank)
    T._dev(T.CUDA)
    buf = ctypes.create_string_buffer(128)
    if rank == 0:
        if lib.sl_dist_unique_id(buf):
            raise RuntimeError("soliton: cannot create the process group id")
        with open(init_file + ".tmp", "wb") as f:
            f.write(buf.raw)
        os.replace(init_file + ".tmp", init_file)  # readers never see a partial id
    else:
        t0 = time.time()
        while not os.path.exists(init_file):
            if time.time() - t0 > timeout:
                raise RuntimeError(f"soliton: rank {rank} waited {timeout:.0f}s for {init_file}")
            time.sleep(0.05)
        with open(init_file, "rb") as f:
            ctypes.memmove(buf, f.read(128), 128)
    if lib.sl_dist_init(rank, world, buf):
        raise RuntimeError(f"soliton: process group init failed on rank {rank}")
    _world = world


def init_with_id(rank, world, id_bytes):
    """Joins a group whose 128-byte id was distributed by other means (e.g. a torch.distributed broadcast)."""
    global _world
    T.set_device(rank)
    T._dev(T.CUDA)
    buf = ctypes.create_string_buffer(bytes(id_bytes), 128)
    if lib.sl_dist_init(rank, world, buf):
        raise RuntimeError(f"soliton: process group init failed on rank {rank}")
    _world = world


def unique_id():
    buf = ctypes.create_string_buffer(128)
    if lib.sl_dist_unique_id(buf):
        raise RuntimeError("soliton: cannot create the process group id")
    return buf.raw


def world_size():
    return _world


def destroy():
    global _world
    lib.sl_dist_destroy()
    _world = 1


def all_reduce_grads(params):
    """python/soliton/distributed.py:42-53. Average gradients across ranks in one group. No-op for one process."""
    grads = [p.grad for p in params if p.grad is not None]
    if _world == 1 or not grads:
        return
    dev = grads[0].dev
    ok = lib.sl_dist_group(dev, 1) == 0
    for g in grads:
        ok = lib.sl_dist_allreduce_mean(dev, g.ptr, g.numel) == 0 and ok
    ok = lib.sl_dist_group(dev, 0) == 0 and ok
    if not ok:
        raise RuntimeError("soliton: all-reduce failed")

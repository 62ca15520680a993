"""Static memory planning with the interface of Soliton's `arena` module (python/soliton/arena.py:37-110): record a
trace on meta, give every block a fixed offset, install one arena, mark step boundaries. Recording and replay are
the allocator's (sl_record_*, sl_arena_*); the packing below is this package's own.

For the optimizer path arena mode means: all gradients, parameters and moments of a rank live in one device
allocation, at offsets that are the same on every rank, so a peer maps a rank's whole gradient memory through a
single IPC handle; and since the path takes nothing from the allocator per step, the plan stays exact.
"""
import ctypes
from dataclasses import dataclass, field

from . import tensor as T
from ._C import lib, longs


@dataclass
class Plan:
    offsets: list
    sizes: list
    body: int           # index of the first block of the repeating step
    bytes: int          # size of the arena
    live_peak: int      # most bytes alive at once: the lower bound no packing can beat
    _keep: tuple = field(default=None, repr=False)  # the C arrays the pool points at while installed

    @property
    def waste(self):
        return 1.0 - self.live_peak / self.bytes if self.bytes else 0.0


def record(fn):
    """Runs fn("meta") with the block cache bypassed; returns (sizes, starts, ends, body) of the recorded blocks
    (end -1: still alive when the trace stopped)."""
    meta = T._dev("meta")
    lib.sl_record_start(meta)
    try:
        fn("meta")
    finally:
        lib.sl_record_stop(meta)
    count = lib.sl_record_count(meta)
    columns = [(ctypes.c_int64 * max(count, 1))() for _ in range(3)]
    lib.sl_record_get(meta, *columns)
    sizes, starts, ends = ([int(x) for x in col[:count]] for col in columns)
    return sizes, starts, ends, lib.sl_record_body(meta)


class _Packer:
    """Greedy interval packing. Blocks are taken largest first; a block goes to the lowest address at which no
    block that is alive at any time during its lifetime sits."""

    def __init__(self, sizes, starts, ends):
        horizon = len(sizes) + 1
        self.sizes = sizes
        self.span = [(born, gone if gone >= 0 else horizon) for born, gone in zip(starts, ends)]
        self.where = [0] * len(sizes)
        self.settled = []

    def _neighbours(self, i):
        born, gone = self.span[i]
        for j in self.settled:
            if self.span[j][0] < gone and born < self.span[j][1]:
                yield self.where[j], self.where[j] + self.sizes[j]

    def place(self, i):
        need, at = self.sizes[i], 0
        for lo, hi in sorted(self._neighbours(i)):
            if lo - at >= need:
                break
            at = max(at, hi)
        self.where[i] = at
        self.settled.append(i)

    def run(self):
        order = sorted(range(len(self.sizes)), key=lambda k: (-self.sizes[k], self.span[k][0]))
        for i in order:
            self.place(i)
        return self.where

    def extent(self):
        return max((self.where[i] + self.sizes[i] for i in self.settled), default=0)

    def live_peak(self):
        deltas = sorted([(self.span[i][0], 1, self.sizes[i]) for i in self.settled] +
                        [(self.span[i][1], 0, -self.sizes[i]) for i in self.settled])
        alive = peak = 0
        for _, _, change in deltas:
            alive += change
            peak = max(peak, alive)
        return peak


def solve(sizes, starts, ends):
    """Offsets for the recorded blocks. Returns (offsets, arena bytes, peak of live bytes)."""
    packer = _Packer(list(sizes), list(starts), list(ends))
    offsets = packer.run()
    return offsets, packer.extent(), packer.live_peak()


def plan(fn):
    """Record on meta and pack; no GPU involved."""
    sizes, starts, ends, body = record(fn)
    offsets, arena_bytes, peak = solve(sizes, starts, ends)
    return Plan(offsets, sizes, body, arena_bytes, peak)


def install(p, device):
    """One allocation of p.bytes on `device`; from here on the k-th allocation of the run gets the k-th offset."""
    dev = T._dev(device)
    p._keep = (longs(p.offsets), longs(p.sizes))
    if lib.sl_arena_install(dev, p._keep[0], p._keep[1], len(p.sizes), p.body, p.bytes) != 0:
        raise MemoryError(f"soliton: cannot allocate a {p.bytes / 2**30:.2f} GiB arena on {device}")


def mark(device="cuda"):
    """Step boundary: recorded while planning, a rewind to the repeating body while replaying."""
    lib.sl_record_mark(T._dev(device))


def check(device="cuda"):
    if lib.sl_arena_diverged(T._dev(device)):
        raise RuntimeError("soliton: the run diverged from its memory plan (an unplanned allocation)")


def off(device="cuda"):
    lib.sl_arena_off(T._dev(device))

"""Static memory planning with the interface of python/soliton/arena.py (record on meta, solve offsets, install one
arena, mark step boundaries). The recording and the replay are the allocator's (sl_record_*, sl_arena_*); the offset
solver here is this package's own: blocks sorted by size, each placed at the lowest offset that is free for its
whole lifetime, found by sweeping the already placed blocks that are alive at the same time.

What it means for the optimizer path: in arena mode every gradient, parameter and moment of a rank lives in one
device allocation at offsets that are the same on every rank, so peers map a rank's whole gradient memory through a
single IPC handle; and the path itself takes nothing from the allocator per step, so the plan stays exact.
"""
import ctypes

from . import tensor as T
from ._C import lib, longs


class Plan:
    """python/soliton/arena.py:19-35"""
    __slots__ = ("offsets", "sizes", "body", "bytes", "live_peak", "_keep")

    def __init__(self, offsets, sizes, body, nbytes, live_peak):
        self.offsets, self.sizes, self.body = offsets, sizes, body
        self.bytes, self.live_peak = nbytes, live_peak
        self._keep = None

    @property
    def waste(self):
        return (self.bytes - self.live_peak) / self.bytes if self.bytes else 0.0


def record(fn):
    """python/soliton/arena.py:38-51: run fn("meta") with every allocation recorded as its own block."""
    meta = T.DEVICES.index("meta")
    T._dev(meta)
    lib.sl_record_start(meta)
    try:
        fn("meta")
    finally:
        lib.sl_record_stop(meta)
    n = lib.sl_record_count(meta)
    sizes, starts, ends = ((ctypes.c_int64 * max(n, 1))() for _ in range(3))
    lib.sl_record_get(meta, sizes, starts, ends)
    return list(sizes)[:n], list(starts)[:n], list(ends)[:n], lib.sl_record_body(meta)


def solve(sizes, starts, ends):
    """Offsets such that blocks alive at the same time never overlap. Returns (offsets, arena_bytes, live_peak)."""
    n = len(sizes)
    death = [e if e >= 0 else n + 1 for e in ends]  # never released: alive to the end of the trace
    offsets = [0] * n
    placed = []
    for i in sorted(range(n), key=lambda k: (-sizes[k], starts[k])):
        busy = sorted((offsets[j], offsets[j] + sizes[j]) for j in placed if starts[i] < death[j] and starts[j] < death[i])
        at = 0
        for lo, hi in busy:
            if lo - at >= sizes[i]:
                break
            at = max(at, hi)
        offsets[i] = at
        placed.append(i)
    arena = max((offsets[i] + sizes[i] for i in range(n)), default=0)
    events = sorted([(starts[i], 1, sizes[i]) for i in range(n)] + [(death[i], 0, -sizes[i]) for i in range(n)])
    live = peak = 0
    for _, _, delta in events:
        live += delta
        peak = max(peak, live)
    return offsets, arena, peak


def plan(fn):
    sizes, starts, ends, body = record(fn)
    offsets, nbytes, live_peak = solve(sizes, starts, ends)
    return Plan(offsets, sizes, body, nbytes, live_peak)


def install(p, device):
    """python/soliton/arena.py:86-93: one allocation for the run; the plan arrays must outlive the install."""
    dev = T._dev(device)
    p._keep = (longs(p.offsets), longs(p.sizes))
    off, sz = p._keep
    if lib.sl_arena_install(dev, off, sz, len(p.sizes), p.body, p.bytes) != 0:
        raise MemoryError(f"soliton: cannot allocate a {p.bytes / 2**30:.2f} GiB arena on {device}")


def mark(device="cuda"):
    lib.sl_record_mark(T._dev(device))


def check(device="cuda"):
    if lib.sl_arena_diverged(T._dev(device)):
        raise RuntimeError("soliton: the run diverged from its memory plan (an unplanned allocation)")


def off(device="cuda"):
    lib.sl_arena_off(T._dev(device))

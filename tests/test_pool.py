"""The deterministic allocator through the C ABI on the cpu and meta pools (no GPU): the policy of
core/soliton/alloc.d that the memory plan rests on."""
import ctypes

import numpy as np
import pytest

CPU, META = 0, 1
KEYS = ("allocated", "reserved", "peak_allocated", "peak_reserved", "n_alloc", "n_raw", "trace")
FNV_SEED = 1469598103934665603
FNV_PRIME = 1099511628211


def stats(lib, dev):
    buf = (ctypes.c_int64 * 7)()
    lib.sl_stats(dev, buf)
    return dict(zip(KEYS, buf))


def rounded(n):
    n = max(n, 1)
    return (n + 511) // 512 * 512 if n < (1 << 20) else (n + (2 << 20) - 1) // (2 << 20) * (2 << 20)


@pytest.fixture()
def clean(lib):
    for dev in (CPU, META):
        lib.sl_arena_off(dev)
        lib.sl_record_stop(dev)
        lib.sl_set_limit(dev, 0)
        lib.sl_empty_cache(dev)
        lib.sl_reset_stats(dev)
    return lib


@pytest.mark.parametrize("dev", [CPU, META])
def test_size_classes_counters_and_trace_hash(clean, dev):
    lib = clean
    base = stats(lib, dev)
    sizes = [0, 1, 511, 512, 513, 3072, (1 << 20) - 1, 1 << 20, (2 << 20) + 1, 38597376 * 4]
    ptrs = [lib.sl_alloc(dev, n) for n in sizes]
    assert all(ptrs)
    s = stats(lib, dev)
    assert s["allocated"] - base["allocated"] == sum(rounded(n) for n in sizes)
    assert s["n_alloc"] == len(sizes) and s["n_raw"] == len(sizes)
    h = FNV_SEED
    for n in sizes:  # alloc.d:62-66: FNV-1a over (kind = 1 alloc / 2 free, rounded size)
        h = ((h ^ 1) * FNV_PRIME) % 2**64
        h = ((h ^ rounded(n)) * FNV_PRIME) % 2**64
    assert s["trace"] % 2**64 == h
    for p, n in zip(ptrs, sizes):
        lib.sl_free(dev, p, n)
    s2 = stats(lib, dev)
    assert s2["allocated"] == base["allocated"]
    assert s2["reserved"] == s["reserved"]  # freed blocks stay cached
    # exact-size reuse: same sizes again take nothing new from the system
    ptrs = [lib.sl_alloc(dev, n) for n in sizes]
    assert stats(lib, dev)["n_raw"] == len(sizes)
    for p, n in zip(ptrs, sizes):
        lib.sl_free(dev, p, n)
    lib.sl_empty_cache(dev)
    assert stats(lib, dev)["reserved"] == base["reserved"]


def test_meta_trace_equals_cpu_trace_for_the_same_requests(clean):
    lib = clean
    rng = np.random.default_rng(0)
    reqs = [int(x) for x in rng.integers(1, 5 << 20, size=200)]
    out = {}
    for dev in (CPU, META):
        base = stats(lib, dev)["allocated"]
        live = []
        for i, n in enumerate(reqs):
            live.append((lib.sl_alloc(dev, n), n))
            if i % 3 == 2:
                p, m = live.pop(0)
                lib.sl_free(dev, p, m)
        s = stats(lib, dev)
        out[dev] = (s["peak_allocated"] - base, s["peak_reserved"] - stats(lib, dev)["reserved"] + s["reserved"] - base,
                    s["trace"], s["n_alloc"], s["n_raw"])
        for p, m in live:
            lib.sl_free(dev, p, m)
        lib.sl_empty_cache(dev)
    assert out[CPU][0] == out[META][0] and out[CPU][2:] == out[META][2:]


@pytest.mark.parametrize("dev", [CPU, META])
def test_limit_fails_like_oom_after_one_cache_flush(clean, dev):
    lib = clean
    base = stats(lib, dev)["reserved"]
    lib.sl_set_limit(dev, base + (8 << 20))
    a = lib.sl_alloc(dev, 4 << 20)
    assert a
    lib.sl_free(dev, a, 4 << 20)           # 4 MiB now sits in the cache
    b = lib.sl_alloc(dev, 6 << 20)         # does not fit beside it: the pool flushes the cache and retries
    assert b and stats(lib, dev)["reserved"] == base + (6 << 20)
    assert not lib.sl_alloc(dev, 4 << 20)  # 6 + 4 > 8: refused, nothing to flush
    lib.sl_free(dev, b, 6 << 20)
    lib.sl_set_limit(dev, 0)


def test_record_then_arena_replay(clean):
    lib = clean
    lib.sl_record_start(META)
    a = lib.sl_alloc(META, 1000)
    lib.sl_record_mark(META)
    b = lib.sl_alloc(META, 3 << 20)
    c = lib.sl_alloc(META, 700)
    lib.sl_free(META, b, 3 << 20)
    d = lib.sl_alloc(META, 2 << 20)
    lib.sl_free(META, c, 700)
    lib.sl_free(META, d, 2 << 20)
    lib.sl_record_stop(META)
    n = lib.sl_record_count(META)
    assert n == 4 and lib.sl_record_body(META) == 1
    size, start, end = ((ctypes.c_int64 * n)() for _ in range(3))
    lib.sl_record_get(META, size, start, end)
    assert list(size) == [1024, 4 << 20, 1024, 2 << 20]
    assert list(start) == [0, 1, 2, 3] and list(end) == [-1, 3, 4, 4]
    lib.sl_free(META, a, 1000)

    # replay on the cpu pool: offsets from a trivial plan (b and d may share bytes, they never overlap in time)
    offsets = (ctypes.c_int64 * 4)(0, 1024, 1024 + (4 << 20), 1024)
    sizes = (ctypes.c_int64 * 4)(*size)
    arena_bytes = 1024 + (4 << 20) + 1024
    before = stats(lib, CPU)["reserved"]
    assert lib.sl_arena_install(CPU, offsets, sizes, 4, 1, arena_bytes) == 0
    assert stats(lib, CPU)["reserved"] == before + arena_bytes
    a = lib.sl_alloc(CPU, 1000)
    for _ in range(3):  # the body repeats: mark rewinds the cursor, the same offsets come back
        lib.sl_record_mark(CPU)
        b = lib.sl_alloc(CPU, 3 << 20)
        c = lib.sl_alloc(CPU, 700)
        assert b - a == 1024 and c - a == 1024 + (4 << 20)
        lib.sl_free(CPU, b, 3 << 20)
        d = lib.sl_alloc(CPU, 2 << 20)
        assert d == b
        lib.sl_free(CPU, c, 700)
        lib.sl_free(CPU, d, 2 << 20)
    assert lib.sl_arena_diverged(CPU) == 0
    lib.sl_record_mark(CPU)
    assert not lib.sl_alloc(CPU, 5000)  # not what the plan recorded at this position
    assert lib.sl_arena_diverged(CPU) == 1
    lib.sl_arena_off(CPU)
    lib.sl_free(CPU, a, 1000)           # last arena-backed block: the arena goes back to the system
    assert stats(lib, CPU)["reserved"] == before


def test_init_device_reserves_the_same_on_meta_each_time(clean):
    lib = clean
    before = stats(lib, META)
    assert lib.sl_init_device(META, 0) == 0
    after = stats(lib, META)
    assert after["allocated"] - before["allocated"] == (32 << 20) + lib.slb_workspace_bytes()
    assert lib.slb_workspace_bytes() == 18 << 20
    assert lib.sl_init_device(CPU, 0) == 0


@pytest.mark.parametrize("dev", [CPU, META])
@pytest.mark.parametrize("seed", [0, 1, 2])
def test_random_traces_match_the_restated_reference_policy(clean, dev, seed):
    """Differential test against oracle/pool_model.py (alloc.d restated in Python): every counter after every
    operation, including reserve-limit refusals, flush-and-retry, cache flushes and statistic resets -- and WHICH
    cached block an allocation gets (the reference takes the first of the exact size and moves the last cached
    block into its place, alloc.d:145-151), checked through a token <-> address correspondence."""
    from oracle.pool_model import PoolModel
    lib = clean
    rng = np.random.default_rng(seed)
    base = stats(lib, dev)
    model = PoolModel()
    live = []
    address_of = {}      # model token -> address the library gave for it
    sizes = [int(x) for x in rng.choice([1, 300, 512, 4096, 70000, 1 << 20, (1 << 20) + 5, 3 << 20, 9 << 20], 400)]
    for step, n in enumerate(sizes):
        op = rng.random()
        if op < 0.55 or not live:
            p, tok = lib.sl_alloc(dev, n), model.alloc(n)
            assert bool(p) == (tok is not None)
            if p:
                assert address_of.setdefault(tok, p) == p, (step, "the library reused another cached block than the reference would")
                live.append((p, tok, n))
        elif op < 0.9:
            p, tok, m = live.pop(int(rng.integers(len(live))))
            lib.sl_free(dev, p, m)
            model.release(tok, m)
        elif op < 0.94:
            lib.sl_empty_cache(dev)
            model.empty_cache()
            address_of = {tok: p for p, tok, _ in live}   # cached blocks went back to the system
        elif op < 0.97:
            lib.sl_reset_stats(dev)
            model.reset_stats()
            base = dict(base, peak_allocated=base["allocated"], peak_reserved=base["reserved"])
        else:
            cap = int(rng.choice([0, 24 << 20, 64 << 20]))
            lib.sl_set_limit(dev, base["reserved"] + cap if cap else 0)
            model.limit = cap
        got, want = stats(lib, dev), model.stats()
        rel = [got["allocated"] - base["allocated"], got["reserved"] - base["reserved"],
               got["peak_allocated"] - base["allocated"], got["peak_reserved"] - base["reserved"],
               got["n_alloc"], got["n_raw"], got["trace"]]
        # the library's pools already hold the fixed workspaces of earlier tests: compare growth, not totals
        want[2] = max(want[2], 0)
        assert rel[0] == want[0] and rel[1] == want[1] and rel[4:] == want[4:], (step, rel, want)
    for p, tok, m in live:
        lib.sl_free(dev, p, m)
    lib.sl_set_limit(dev, 0)
    lib.sl_empty_cache(dev)

"""Host-side multi-rank logic without a GPU: the shared-memory rendezvous between processes, the same bootstrapped
through torch.distributed (gloo, world size 2), and the partition every rank computes for itself."""
import ctypes
import multiprocessing as mp
import os

import numpy as np
import pytest


def _selftest(rank, world, id_bytes, rounds, q):
    from soliton_b200._C import lib
    q.put((rank, lib.slb_rdv_selftest(ctypes.create_string_buffer(id_bytes, 128), rank, world, rounds)))


@pytest.mark.parametrize("world", [2, 4])
def test_rendezvous_between_processes(lib, world):
    buf = ctypes.create_string_buffer(128)
    assert lib.slb_rdv_create_id(buf) == 0
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_selftest, args=(r, world, buf.raw, 9, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = dict(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=30)
    assert results == {r: 0 for r in range(world)}
    assert not os.path.exists(buf.raw[8:].split(b"\0")[0].decode())  # rank 0 removed the file


def _slot_selftest(rank, world, id_bytes, q):
    from soliton_b200._C import lib
    q.put((rank, lib.slb_rdv_slot_selftest(ctypes.create_string_buffer(id_bytes, 128), rank, world, 150, 64)))


def test_export_slots_are_reused_once_every_peer_has_let_go(lib):
    """A trainer that returns its gradient blocks to the driver every step publishes new allocations for ever; the
    table has 8192 slots per rank. 150 cycles x 64 allocations = 9600 pass through 64 slots."""
    world = 3
    buf = ctypes.create_string_buffer(128)
    assert lib.slb_rdv_create_id(buf) == 0
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_slot_selftest, args=(r, world, buf.raw, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = dict(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=30)
    assert results == {r: 0 for r in range(world)}


def test_missing_rank_times_out_instead_of_hanging(lib):
    buf = ctypes.create_string_buffer(128)
    assert lib.slb_rdv_create_id(buf) == 0
    path = buf.raw[8:].split(b"\0")[0].decode()
    # world of 2 with only rank 0 present: selftest uses 30 s waits, so drive the pieces with a short-lived helper
    code = ("import ctypes,sys; from soliton_b200._C import lib; "
            "lib.slb_set_option(b'host_timeout_ms',1500); b=ctypes.create_string_buffer(bytes.fromhex(sys.argv[1]),128); "
            "sys.exit(0 if lib.slb_rdv_selftest(b,0,2,1)!=0 else 1)")
    import subprocess
    import sys
    env = dict(os.environ, PYTHONPATH=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    r = subprocess.run([sys.executable, "-c", code, buf.raw.hex()], env=env, timeout=100)
    assert r.returncode == 0  # the lone rank gave up with an error
    if os.path.exists(path):
        os.unlink(path)


def _gloo_rank(rank, world, port, q):
    import torch
    import torch.distributed as dist
    from oracle import pyoracle
    from soliton_b200._C import lib
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    idt = torch.zeros(128, dtype=torch.uint8)
    if rank == 0:
        buf = ctypes.create_string_buffer(128)
        assert lib.slb_rdv_create_id(buf) == 0
        idt = torch.frombuffer(bytearray(buf.raw), dtype=torch.uint8).clone()
    dist.broadcast(idt, 0)
    rc = lib.slb_rdv_selftest(ctypes.create_string_buffer(bytes(idt.numpy().tobytes()), 128), rank, world, 5)
    # the mean two ranks must agree on: gloo's sum / 2 has the bits of the oracle's rank-ordered mean
    gs = [np.random.default_rng(1 + r).standard_normal(4096, dtype=np.float32) for r in range(world)]
    t = torch.tensor(gs[rank].copy())
    dist.all_reduce(t)
    same = bool(np.array_equal((t.numpy() * np.float32(0.5)), pyoracle.mean_ranks(gs)))
    dist.destroy_process_group()
    q.put((rank, rc, same))


def test_bootstrap_over_gloo_world_size_2(lib):
    import socket
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_gloo_rank, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = sorted(q.get(timeout=180) for _ in procs)
    for p in procs:
        p.join(timeout=30)
    assert results == [(0, 0, True), (1, 0, True)]


def test_partition_covers_every_tile_once_and_is_block_aligned_across_ranks(lib):
    from soliton_b200 import workload
    from soliton_b200._C import longs
    ns = [workload.numel(s) for _, s, _ in workload.param_shapes("124M")]
    T = lib.slb_tile_count(longs(ns), len(ns))
    assert T == sum((n + 2047) // 2048 for n in ns)
    b, e = ctypes.c_int64(), ctypes.c_int64()
    for world in (1, 2, 3, 4, 8):
        for blocks in (1, 7, 296):
            seen = 0
            prev_end = 0
            for chunk in range(world):
                for block in range(blocks):
                    lib.slb_run_range(T, world, chunk, blocks, block, ctypes.byref(b), ctypes.byref(e))
                    assert b.value == prev_end and e.value >= b.value
                    prev_end = e.value
                    seen += e.value - b.value
            assert seen == T and prev_end == T
    # chunk = -1: runs over the whole sequence (single rank and one-shot)
    lib.slb_run_range(T, 8, -1, 296, 295, ctypes.byref(b), ctypes.byref(e))
    assert e.value == T

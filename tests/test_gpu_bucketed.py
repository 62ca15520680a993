"""The step bucket by bucket (soliton_b200/bucketed.py): launches go out while later gradients do not exist yet
(gradients become final in reverse layer order, python/soliton/tensor.py:427-471), on a stream of their own when
asked, and a host-fed step moves its buckets over the library's copy streams. Whatever the bucketing and the
streams, the results are the bits of the unbucketed step (the oracle's)."""
import ctypes as C

import numpy as np
import pytest

from oracle import pyoracle
from soliton_b200 import tensor as T, workload
from soliton_b200._C import counter, lib, set_option
from soliton_b200.bucketed import BucketedAdamW, plan_buckets

pytestmark = pytest.mark.gpu
H = workload.HYPER
SHAPES = [(300, 70), (70,), (2048,), (64, 1024), (5, 2049), (1,), (130000,), (33, 1000), (4096,), (257, 129)]


def oracle_step(ref, grads, step):
    for i, shape in enumerate(SHAPES):
        pyoracle.adamw(ref[i][0], grads[i].ravel(), ref[i][1], ref[i][2], H["lr"], H["b1"], H["b2"], H["eps"],
                       H["wd"] if len(shape) >= 2 else 0.0, step, fma=True)


def make(bucket_bytes):
    rng = np.random.default_rng(5)
    p0 = [(rng.standard_normal(s) * 0.02).astype(np.float32) for s in SHAPES]
    params = [T.tensor(a, "cuda") for a in p0]
    opt = BucketedAdamW(params, bucket_bytes=bucket_bytes, lr=H["lr"], betas=(H["b1"], H["b2"]), eps=H["eps"],
                        weight_decay=H["wd"])
    ref = [[a.ravel().copy(), np.zeros(a.size, np.float32), np.zeros(a.size, np.float32)] for a in p0]
    return rng, params, opt, ref


def test_bucket_plan_covers_every_tensor_once_last_first():
    sizes = [10, 1000, 5, 700, 300, 50]
    buckets = plan_buckets(sizes, 4 * 900)
    assert [i for b in buckets for i in b] == [5, 4, 3, 2, 1, 0]
    assert buckets == [[5, 4, 3], [2, 1], [0]]


@pytest.mark.parametrize("overlap", [0, 1], ids=["legacy-stream", "own-stream"])
def test_each_bucket_launches_before_the_next_gradients_exist(cuda, overlap):
    set_option("overlap", overlap)
    try:
        rng, params, opt, ref = make(bucket_bytes=256 << 10)
        assert len(opt.buckets) >= 3
        for step in (1, 2, 3):
            grads = [(rng.standard_normal(s) * 1e-3).astype(np.float32) for s in SHAPES]
            opt.begin_step()
            for b, bucket in enumerate(opt.buckets):
                for i in bucket:                       # "backward" reaches this bucket only now
                    params[i].grad = T.tensor(grads[i], "cuda")
                before = counter("launches")
                opt.step_bucket(b)
                assert counter("launches") == before + 1   # out already; gradients of later buckets are not even allocated
            oracle_step(ref, grads, step)
            # no synchronize: a blocking read orders itself after the launch that writes what it reads
            for i, p in enumerate(params):
                np.testing.assert_array_equal(p.numpy().ravel(), ref[i][0])
            for i, (m, v) in enumerate(opt.state):
                np.testing.assert_array_equal(m.numpy().ravel(), ref[i][1])
                np.testing.assert_array_equal(v.numpy().ravel(), ref[i][2])
            opt.zero_grad()                            # frees gradient blocks a launch may still be reading
        T.synchronize()
    finally:
        set_option("overlap", 0)


class Pinned:
    def __init__(self, n):
        self.ptr = lib.slb_pinned_alloc(4 * n)
        assert self.ptr
        self.array = np.ctypeslib.as_array(C.cast(self.ptr, C.POINTER(C.c_float)), shape=(n,))

    def data_ptr(self):
        return self.ptr

    def __del__(self):
        lib.slb_pinned_free(self.ptr)


@pytest.mark.parametrize("overlap", [0, 1], ids=["legacy-stream", "own-stream"])
def test_host_fed_steps_through_the_copy_streams(cuda, overlap):
    set_option("overlap", overlap)
    try:
        rng, params, opt, ref = make(bucket_bytes=128 << 10)
        for p in params:
            p.grad = T.empty(p.shape, "cuda")
        hg = [Pinned(p.numel) for p in params]
        hp = [Pinned(p.numel) for p in params]
        opt.bind_host(hg, hp)
        for step in (1, 2, 3, 4):
            grads = [(rng.standard_normal(s) * 1e-3).astype(np.float32) for s in SHAPES]
            for buf, g in zip(hg, grads):
                buf.array[:] = g.ravel()
            for buf in hp:
                buf.array[:] = np.nan
            opt.host_step()                            # returns when the parameters are on the host
            oracle_step(ref, grads, step)
            for i, buf in enumerate(hp):
                np.testing.assert_array_equal(buf.array, ref[i][0])
        assert lib.sl_check(T.CUDA) == 0
    finally:
        set_option("overlap", 0)


def test_back_to_back_host_fed_steps_order_themselves(cuda):
    """No host wait between steps: the upload of step k+1 into a gradient must wait for the launch of step k that
    still reads it, and that launch for the download of step k-1 that still reads its parameters."""
    rng, params, opt, ref = make(bucket_bytes=64 << 10)
    for p in params:
        p.grad = T.empty(p.shape, "cuda")
    steps = 5
    hg = [[Pinned(p.numel) for p in params] for _ in range(steps)]
    hp = [[Pinned(p.numel) for p in params] for _ in range(steps)]
    all_grads = []
    for k in range(steps):
        grads = [(rng.standard_normal(s) * 1e-3).astype(np.float32) for s in SHAPES]
        all_grads.append(grads)
        for buf, g in zip(hg[k], grads):
            buf.array[:] = g.ravel()
    for k in range(steps):
        opt.bind_host(hg[k], hp[k])
        opt.begin_step()
        for b in range(len(opt.buckets)):
            opt.upload(b), opt.step_bucket(b), opt.download(b)
    assert lib.slb_wait_copies() == 0
    for k in range(steps):
        oracle_step(ref, all_grads[k], k + 1)
        for i, buf in enumerate(hp[k]):
            np.testing.assert_array_equal(buf.array, ref[i][0])
    T.synchronize()


def test_each_rank_reads_back_only_its_share_of_the_parameters(cuda):
    """Data-parallel ranks end a step with the same parameter bits; a host-fed job therefore reads every parameter
    back once, rank r its r-th share. Emulated here by binding the same optimizer as rank r of 4, for every r: the
    shares are disjoint, cover everything, and hold the right values."""
    world = 4
    rng, params, opt, ref = make(bucket_bytes=256 << 10)
    for p in params:
        p.grad = T.empty(p.shape, "cuda")
    hg = [Pinned(p.numel) for p in params]
    grads = [(rng.standard_normal(s) * 1e-3).astype(np.float32) for s in SHAPES]
    for buf, g in zip(hg, grads):
        buf.array[:] = g.ravel()
    whole = [Pinned(p.numel) for p in params]
    opt.bind_host(hg, whole)
    opt.host_step()
    oracle_step(ref, grads, 1)
    for i, buf in enumerate(whole):
        np.testing.assert_array_equal(buf.array, ref[i][0])
    written = [np.zeros(p.numel, np.int32) for p in params]
    total = 0
    for r in range(world):
        hp = [Pinned(p.numel) for p in params]
        for buf in hp:
            buf.array[:] = np.nan
        opt.bind_host(hg, hp, share=(r, world))
        total += opt.download_bytes
        for b in range(len(opt.buckets)):
            opt.download(b)
        assert lib.slb_wait_copies() == 0
        for i, buf in enumerate(hp):
            got = ~np.isnan(buf.array)
            written[i] += got
            np.testing.assert_array_equal(buf.array[got], ref[i][0][got])
    assert all((w == 1).all() for w in written)          # every element exactly once over the four ranks
    assert total == 4 * sum(p.numel for p in params)

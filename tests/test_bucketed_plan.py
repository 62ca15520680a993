"""Host-side logic of the bucketed, host-fed step without a GPU (meta device: the pool hands out addresses, nothing
runs): the bucket plan, and the split of the parameter read-back over the ranks -- every element of every parameter
must reach the host exactly once over the whole job, at the place that mirrors its device address."""
import numpy as np
import pytest

from soliton_b200 import tensor as T
from soliton_b200.bucketed import BucketedAdamW, plan_buckets

SIZES = [50000, 7, 16384, 300, 16385, 1, 40000, 16383, 123457]        # around the 64 KiB rule (16,384 floats), and odd ones


def test_buckets_take_tensors_from_the_last_to_the_first_and_each_once():
    buckets = plan_buckets(SIZES, 100000)
    flat = [i for b in buckets for i in b]
    assert flat == list(range(len(SIZES) - 1, -1, -1))
    for b in buckets[:-1]:
        held = [4 * SIZES[i] for i in b]
        assert sum(held) >= 100000 and sum(held[:-1]) < 100000        # closed by the tensor that reached the size
    assert plan_buckets(SIZES, 1) == [[i] for i in range(len(SIZES) - 1, -1, -1)]
    assert plan_buckets(SIZES, 1 << 40) == [list(range(len(SIZES) - 1, -1, -1))]
    assert plan_buckets([], 1024) == []


@pytest.mark.parametrize("world", [1, 2, 3, 4, 8])
def test_every_parameter_element_is_read_back_exactly_once_over_the_ranks(world):
    params = []
    for n in SIZES:
        p = T.zeros((n,), "meta")
        p.grad = T.zeros((n,), "meta")
        params.append(p)
    opt = BucketedAdamW(params, bucket_bytes=100000)
    host = [4_000_000 * (i + 1) for i in range(len(SIZES))]           # stand-ins for pinned buffers: addresses only
    cover = [np.zeros(n, int) for n in SIZES]
    total = 0
    for rank in range(world):
        opt.bind_host(host, host, share=(rank, world))
        assert opt.upload_bytes == 4 * sum(SIZES)                     # every rank uploads all of its own gradients
        total += opt.download_bytes
        for copies in opt._down:
            for k in range(copies.k):
                h, nbytes = copies.host[k], copies.bytes[k]
                i = next(j for j in range(len(SIZES)) if host[j] <= h < host[j] + 4 * SIZES[j])
                assert copies.dev[k] - params[i].ptr == h - host[i]   # same offset on both sides
                assert nbytes % 4 == 0 and (h - host[i]) % 4 == 0
                lo = (h - host[i]) // 4
                cover[i][lo:lo + nbytes // 4] += 1
    assert total == 4 * sum(SIZES)
    for c in cover:
        assert (c == 1).all()

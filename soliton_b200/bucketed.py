"""The optimizer step bucket by bucket, so that it can start before the last gradient exists.

Soliton's backward makes gradients final in reverse layer order (python/soliton/tensor.py:427-471; a leaf adopts or
accumulates its gradient at :451-462), yet its trainer reduces and steps only after all of backward
(examples/gpt2.py:92-94). Here the parameters are cut into buckets, last parameter first, and each bucket goes
through the same calls as the whole step -- distributed.all_reduce_grads, then one sl_adamw per tensor -- as soon
as its gradients are final: one fused launch per bucket. With the library's "overlap" option those launches run on a
stream of their own beside whatever backward still has on the legacy stream.

The same structure carries a host-fed step (gradients arriving from pinned host memory, parameters read back):
`upload` and `download` move one bucket's tensors on the library's copy streams, which order themselves against
the launches by address, so that bucket k+1 uploads and bucket k-1 downloads while bucket k computes.
"""
import ctypes

from . import distributed
from ._C import lib
from .optim import AdamW


def plan_buckets(sizes, bucket_bytes):
    """Indices of the tensors of each bucket: tensors taken from the last to the first, a bucket closed once it holds
    at least `bucket_bytes` (4 bytes per element). Every index appears exactly once."""
    buckets, current, held = [], [], 0
    for index in range(len(sizes) - 1, -1, -1):
        current.append(index)
        held += 4 * int(sizes[index])
        if held >= bucket_bytes:
            buckets.append(current)
            current, held = [], 0
    if current:
        buckets.append(current)
    return buckets


class _Copies:
    """Argument arrays for slb_from_host_async / slb_to_host_async, kept per bucket so that a step builds nothing."""

    def __init__(self, device_ptrs, host_ptrs, nbytes):
        k = len(device_ptrs)
        self.k = k
        self.dev = (ctypes.c_void_p * max(k, 1))(*device_ptrs)
        self.host = (ctypes.c_void_p * max(k, 1))(*host_ptrs)
        self.bytes = (ctypes.c_size_t * max(k, 1))(*nbytes)


class BucketedAdamW(AdamW):
    """AdamW (python/soliton/optim.py:7-28) stepped bucket by bucket. `step()` still runs the whole step; what is
    added is `begin_step()` + `step_bucket(b)` for a caller that knows when a bucket's gradients are final.

    Same arithmetic, same bits as the unbucketed step: a bucket only decides which tensors share a launch."""

    def __init__(self, params, bucket_bytes=64 << 20, **kw):
        super().__init__(params, **kw)
        self.buckets = plan_buckets([slot.param.numel for slot in self._slots], bucket_bytes)

    def begin_step(self):
        self.t += 1

    def step_bucket(self, b):
        """All gradients of bucket b are final: average them over the ranks and update their parameters."""
        slots = [self._slots[i] for i in self.buckets[b] if self._slots[i].param.grad is not None]
        if not slots:
            return
        distributed.all_reduce_grads([slot.param for slot in slots])
        hyper = (self.lr, self.betas[0], self.betas[1], self.eps)
        for slot in slots:
            p = slot.param
            lib.sl_adamw(p.dev, p.ptr, p.grad.ptr, slot.m.ptr, slot.v.ptr, p.numel, *hyper,
                         self.wd if slot.decays else 0.0, self.t)
        lib.slb_flush()  # a single rank batches sl_adamw calls until something else happens: the bucket ends here

    def step(self):
        self.begin_step()
        for b in range(len(self.buckets)):
            self.step_bucket(b)

    # --- host-fed steps

    def bind_host(self, host_grads, host_params, share=None):
        """Pinned host buffers, one per parameter (objects with data_ptr(), or addresses): where gradients come from
        and where updated parameters go. Gradient tensors must already hang on the parameters.

        `share` = (rank, world): after a data-parallel step every rank holds the same parameter bits, so the job
        needs them on the host once, not once per rank. Rank r then reads back only its share -- elements
        [n r / world, n (r + 1) / world) of every tensor of 64 KiB or more, and the whole of every world-th small
        tensor -- into the same places of its host buffers; the rest of those buffers is not written."""
        addr = lambda x: x.data_ptr() if hasattr(x, "data_ptr") else int(x)  # noqa: E731
        rank, world = share if share else (0, 1)
        self._bound = (list(host_grads), list(host_params))   # the copies run later: the buffers must outlive this call
        self._up, self._down = [], []
        self.upload_bytes = self.download_bytes = 0
        for bucket in self.buckets:
            ps = [self._slots[i].param for i in bucket]
            nb = [4 * p.numel for p in ps]
            self._up.append(_Copies([p.grad.ptr for p in ps], [addr(host_grads[i]) for i in bucket], nb))
            self.upload_bytes += sum(nb)
            dev, host, size = [], [], []
            for i, p in zip(bucket, ps):
                n = p.numel
                if 4 * n >= (64 << 10):
                    lo, hi = n * rank // world, n * (rank + 1) // world
                elif i % world == rank:
                    lo, hi = 0, n
                else:
                    continue
                if hi > lo:
                    dev.append(p.ptr + 4 * lo), host.append(addr(host_params[i]) + 4 * lo), size.append(4 * (hi - lo))
            self._down.append(_Copies(dev, host, size))
            self.download_bytes += sum(size)

    def upload(self, b):
        c = self._up[b]
        if lib.slb_from_host_async(c.k, c.dev, c.host, c.bytes) != 0:
            raise RuntimeError("soliton: asynchronous upload failed")

    def download(self, b):
        c = self._down[b]
        if c.k and lib.slb_to_host_async(c.k, c.host, c.dev, c.bytes) != 0:
            raise RuntimeError("soliton: asynchronous download failed")

    def host_step(self):
        """One step fed from and read back to the bound host buffers; returns once the parameters are on the host."""
        self.begin_step()
        for b in range(len(self.buckets)):
            self.upload(b)
            self.step_bucket(b)
            self.download(b)
        if lib.slb_wait_copies() != 0:
            raise RuntimeError("soliton: a copy stream reported an error")

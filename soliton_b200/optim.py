"""AdamW and gradient-norm clipping behind the interface of Soliton's `optim` module
(python/soliton/optim.py:7-39). All arithmetic runs in the library; this file keeps the per-parameter records and
decides which call each tensor gets.
"""
import math
from collections import namedtuple

from . import tensor as T
from ._C import lib

# One record per parameter: the tensor, its two moments, and whether weight decay applies to it.
_Slot = namedtuple("_Slot", "param m v decays")


class AdamW:
    """Constructor arguments, public attributes (`params`, `state`, `lr`, `betas`, `eps`, `wd`, `t`) and methods
    follow the reference class.

    Weight decay applies to tensors with two or more dimensions (matrices, embeddings) and not to biases or norm
    weights (optim.py:23). Both moments are created in the constructor -- first moment, then second, parameter by
    parameter -- so that they appear in a memory plan made before the first step (optim.py:14-15).

    `step` issues one `sl_adamw` per parameter that carries a gradient. On cuda the library records these calls
    and runs them as a single launch, fused with the gradient mean when the process group has just reduced the
    same gradients, and with a pending clip scale when `clip_grad_norm` ran in between.
    """

    def __init__(self, params, lr=6e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1):
        self.lr, self.betas, self.eps, self.wd, self.t = lr, betas, eps, weight_decay, 0
        self._slots = [_Slot(p, T.zeros(p.shape, p.dev), T.zeros(p.shape, p.dev), p.ndim >= 2) for p in params]

    @property
    def params(self):
        return [slot.param for slot in self._slots]

    @property
    def state(self):
        return [(slot.m, slot.v) for slot in self._slots]

    def step(self):
        self.t += 1
        hyper = (self.lr, self.betas[0], self.betas[1], self.eps)
        for slot in self._slots:
            grad = slot.param.grad
            if grad is not None:
                lib.sl_adamw(slot.param.dev, slot.param.ptr, grad.ptr, slot.m.ptr, slot.v.ptr, slot.param.numel, *hyper,
                             self.wd if slot.decays else 0.0, self.t)

    def zero_grad(self):
        for slot in self._slots:
            slot.param.grad = None


def clip_grad_norm(params, max_norm):
    """optim.py:31-39: the global L2 norm over all gradients; when it exceeds `max_norm`, every gradient is
    multiplied in place by max_norm / (norm + 1e-6). Returns the norm before clipping.

    On cuda the per-tensor sums of squares come out of one batched, deterministic launch, and the scales are applied
    by the optimizer launch that follows."""
    live = [p.grad for p in params if p.grad is not None]
    norm = math.sqrt(sum(T.sumsq(grad) for grad in live))
    if norm <= max_norm:
        return norm
    shrink = max_norm / (norm + 1e-6)
    for grad in live:
        lib.sl_scale(grad.dev, grad.ptr, grad.ptr, grad.numel, shrink)
    return norm

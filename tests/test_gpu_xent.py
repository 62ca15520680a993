"""Cross entropy, forward and backward (csrc/xent_kernels.cu), through the backend-level C ABI, against float64 and
against the reference's own kernels (core/cuda/kernels.cu:488-534, built unmodified into oracle/_ref/).

Floating point: one pass with a running maximum instead of the reference's two, fast exponentials, and a different
reduction tree, so results agree to rounding, not to the bit. Bars: the loss within 1e-5 relative of float64 (the
reference's own test bar for losses is rtol 1e-4, tests/test_ops.py), every gradient element within 1e-5 of the
largest possible magnitude dloss / n plus 1e-5 relative; and no further from float64 than twice the reference's own
distance plus one rounding of the result."""
import ctypes as C
import os

import numpy as np
import pytest

from oracle import build as obuild
from oracle import step_ops
from soliton_b200._C import lib
from tests.gpu_util import DevBuf, check_ok

pytestmark = pytest.mark.gpu
# (rows, v, skew of the logits, skew of the gradient): 50,257 is GPT-2's vocabulary -- an odd row length, so rows start
# at all four alignments; n = 1 takes the host sum; unequal skews the scalar-store path. Backward: rows from 4,096
# logits on are split over a cluster of 4 blocks (8 when a quarter exceeds 100 KB: 120,001), longer ones (250,007) and
# shorter ones are read twice by one block
SHAPES = [(64, 50257, 0, 0), (7, 1000, 0, 0), (3, 5, 0, 0), (1, 17, 0, 0), (128, 50304, 0, 0), (33, 4097, 1, 1), (33, 4097, 0, 3),
          (9, 2, 0, 0), (5, 1, 0, 0), (5, 120001, 0, 0), (3, 250007, 0, 0)]


@pytest.fixture(scope="module")
def ref(cuda):
    path = obuild.build_ref()
    if not path or not os.path.exists(path):
        pytest.skip("reference CUDA backend not built (no reference checkout at build time)")
    r = C.CDLL(path)
    assert r.sl_cuda_set_device(0) == 0
    r.sl_cuda_cross_entropy.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_void_p]
    r.sl_cuda_cross_entropy.restype = C.c_double
    r.sl_cuda_cross_entropy_bwd.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_float]
    r.sl_cuda_cross_entropy_bwd.restype = None
    return r


def truth(logits, t, dloss):
    """float64, the restatement of the reference's host twin (pinned against PyTorch in tests/test_step_ops_oracle.py)."""
    return step_ops.cross_entropy(logits, t, dloss)


def run(fns, n, v, skew_l, skew_d, logits, t, dloss):
    fwd, bwd = fns
    dl_in, dt = DevBuf(logits, skew=skew_l), DevBuf(t.view(np.float32))
    rowloss, dl = DevBuf(n=max(n, 2)), DevBuf(n=n * v, skew=skew_d)
    loss = fwd(dl_in.ptr, dt.ptr, n, v, rowloss.ptr)
    bwd(dl_in.ptr, dt.ptr, dl.ptr, n, v, dloss)
    check_ok()
    return loss, dl.get().reshape(n, v)


@pytest.mark.parametrize("n,v,skew_l,skew_d", SHAPES)
def test_cross_entropy_forward_and_backward(ref, n, v, skew_l, skew_d):
    rng = np.random.default_rng(n * 7 + v)
    logits = (rng.standard_normal((n, v)) * 3.0).astype(np.float32)
    logits[0, rng.integers(0, v)] = 40.0                              # one dominant logit: the rescaling path
    if n > 2:
        logits[2] -= 300.0                                            # a row far below zero
    t = rng.integers(0, v, n).astype(np.int32)
    t[0] = 0
    t[-1] = v - 1                                                     # targets in the scalar head and tail of a row
    dloss = 0.7
    loss, d = run((lib.sl_cuda_cross_entropy, lib.sl_cuda_cross_entropy_bwd), n, v, skew_l, skew_d, logits, t, dloss)
    loss2, d2 = run((lib.sl_cuda_cross_entropy, lib.sl_cuda_cross_entropy_bwd), n, v, skew_l, skew_d, logits, t, dloss)
    rloss, rd = run((ref.sl_cuda_cross_entropy, ref.sl_cuda_cross_entropy_bwd), n, v, skew_l, skew_d, logits, t, dloss)
    assert ref.sl_cuda_check() == 0
    assert loss == loss2 and np.array_equal(d, d2)                    # fixed orders: the same bits every run
    want_loss, want_d = truth(logits, t, dloss)
    g = dloss / n
    assert abs(loss - want_loss) <= 1e-5 * max(1.0, abs(want_loss)), (loss, rloss, want_loss)
    assert abs(loss - want_loss) <= 2 * abs(rloss - want_loss) + 1e-6 * max(1.0, abs(want_loss)), (loss, rloss, want_loss)
    err, rerr = np.abs(d - want_d), np.abs(rd - want_d)
    assert np.all(err <= 1e-5 * g + 1e-5 * np.abs(want_d)), (err.max(), rerr.max(), g)
    assert err.max() <= 2 * rerr.max() + 1e-6 * g, (err.max(), rerr.max(), g)
    assert abs(float(d.sum(dtype=np.float64))) <= 1e-4 * g * n       # each row of softmax - onehot sums to zero


def test_empty_input_is_not_a_number(cuda):
    buf = DevBuf(n=8)
    assert np.isnan(lib.sl_cuda_cross_entropy(buf.ptr, buf.ptr, 0, 5, buf.ptr))
    lib.sl_cuda_cross_entropy_bwd(buf.ptr, buf.ptr, buf.ptr, 0, 5, 1.0)
    check_ok()

"""Broadcasting binary ops, GELU and the embedding's backward (csrc/elementwise_kernels.cu), through the backend-level
C ABI, against the reference's own kernels (core/cuda/kernels.cu:139-181, 226-240, 459-487, built unmodified into
oracle/_ref/) and against numpy.

Bit-exact: a binary op is one IEEE fp32 operation per element on the same two inputs, so the reference, numpy's
float32 arithmetic and these kernels must agree in every bit; the embedding's backward adds the same rows in the same
(token) order as the reference, so its sums agree in every bit with the reference and to rounding with float64. GELU
is the same fp32 expression through the same erf and exp of the CUDA math library: the reference's bits, and float64's
(oracle/step_ops.py) to 1e-6, the reference's own bar for unary ops being rtol 1e-4 (tests/test_ops.py)."""
import ctypes as C
import os

import numpy as np
import pytest

from oracle import build as obuild
from oracle import step_ops
from soliton_b200._C import lib
from tests.gpu_util import DevBuf, check_ok

pytestmark = pytest.mark.gpu
L, P = C.c_int64, C.c_void_p


@pytest.fixture(scope="module")
def ref(cuda):
    path = obuild.build_ref()
    if not path or not os.path.exists(path):
        pytest.skip("reference CUDA backend not built (no reference checkout at build time)")
    r = C.CDLL(path)
    assert r.sl_cuda_set_device(0) == 0
    r.sl_cuda_binary.argtypes = [C.c_int, P, P, P, C.c_int, P, P, P]
    r.sl_cuda_binary.restype = None
    r.sl_cuda_embedding_bwd.argtypes = [P, P, P, L, L, L, P, P, P, P, C.c_size_t]
    r.sl_cuda_embedding_bwd.restype = None
    r.sl_cuda_gelu.argtypes = [P, P, L]
    r.sl_cuda_gelu.restype = None
    r.sl_cuda_gelu_bwd.argtypes = [P, P, P, L]
    r.sl_cuda_gelu_bwd.restype = None
    return r


def longs(values):
    return (C.c_int64 * len(values))(*values)


def strides_for(array_shape, out_shape):
    """Element strides of a dense array of `array_shape` broadcast (numpy rules) to `out_shape`; 0 where it repeats."""
    pad = (1,) * (len(out_shape) - len(array_shape)) + tuple(array_shape)
    dense, out = 1, []
    for size in reversed(pad):
        out.append(0 if size == 1 else dense)
        dense *= size
    return list(reversed(out))


# (output shape, shape of a, shape of b, skew in floats of every buffer)
BROADCASTS = [
    ((8192, 768), (8192, 768), (8192, 768), 0),     # residual add: both inputs are the output's shape
    ((8192, 3072), (8192, 3072), (3072,), 0),       # bias add: b is the trailing dimension
    ((4, 1024, 768), (4, 1024, 768), (1024, 768), 0),  # positional embedding: b is the two trailing dimensions
    ((64, 64), (64, 64), (1,), 0),                  # scalar
    ((7, 5), (7, 5), (5,), 0),                      # sizes that are no multiple of four
    ((33, 768), (33, 768), (768,), 1),              # pointers that are not 16-byte aligned
    ((6, 1, 8), (6, 1, 8), (8,), 0),
    ((4, 5, 6), (4, 5, 6), (4, 1, 6), 0),           # b repeats in the middle: general strides
    ((4, 5, 6), (5, 1), (4, 1, 6), 0),              # both inputs broadcast
    ((2, 3, 4, 5), (2, 3, 4, 5), (3, 1, 5), 0),
]


@pytest.mark.parametrize("op", [0, 1, 2, 3])
@pytest.mark.parametrize("out_shape,a_shape,b_shape,skew", BROADCASTS)
def test_binary_gives_the_reference_bits(ref, op, out_shape, a_shape, b_shape, skew):
    rng = np.random.default_rng(len(out_shape) * 100 + op)
    a = rng.standard_normal(a_shape).astype(np.float32)
    b = (rng.standard_normal(b_shape) + 3.0).astype(np.float32)      # away from zero: op 3 divides by it
    n = int(np.prod(out_shape))
    da, db = DevBuf(a, skew=skew), DevBuf(b, skew=skew)
    shape, sa, sb = longs(out_shape), longs(strides_for(a_shape, out_shape)), longs(strides_for(b_shape, out_shape))
    got = {}
    for name, fn in (("ours", lib.sl_cuda_binary), ("reference", ref.sl_cuda_binary)):
        out = DevBuf(n=n, skew=skew)
        fn(op, da.ptr, db.ptr, out.ptr, len(out_shape), shape, sa, sb)
        check_ok()
        got[name] = out.get().reshape(out_shape)
    assert ref.sl_cuda_check() == 0
    want = np.broadcast_to(step_ops.binary(op, a, b), out_shape)
    np.testing.assert_array_equal(got["ours"].view(np.uint32), got["reference"].view(np.uint32))
    np.testing.assert_array_equal(got["ours"].view(np.uint32), np.ascontiguousarray(want).view(np.uint32))


def test_binary_with_a_transposed_input(ref):
    rng = np.random.default_rng(5)
    a = rng.standard_normal((48, 20)).astype(np.float32)
    b = rng.standard_normal((20, 48)).astype(np.float32)              # read as its transpose: strides (1, 48)
    da, db, out = DevBuf(a), DevBuf(b), DevBuf(n=48 * 20)
    lib.sl_cuda_binary(0, da.ptr, db.ptr, out.ptr, 2, longs((48, 20)), longs((20, 1)), longs((1, 48)))
    check_ok()
    np.testing.assert_array_equal(out.get().reshape(48, 20), a + b.T)


def test_binary_refuses_what_it_cannot_index(cuda):
    buf = DevBuf(n=16)
    lib.sl_cuda_binary(0, buf.ptr, buf.ptr, buf.ptr, 9, longs((1,) * 9), longs((0,) * 9), longs((0,) * 9))
    lib.sl_sync(2)
    assert lib.sl_check(2) == 12                                      # more dimensions than the reference's 8
    lib.slb_clear_error()
    lib.sl_cuda_binary(0, buf.ptr, buf.ptr, buf.ptr, 2, longs((0, 4)), longs((4, 1)), longs((4, 1)))  # empty: nothing to do
    check_ok()


@pytest.mark.parametrize("n,skew", [(8192 * 3072, 0), (1000, 0), (1001, 0), (4096, 1), (3, 0)])
def test_gelu_gives_the_reference_bits(ref, n, skew):
    rng = np.random.default_rng(n)
    x = (rng.standard_normal(n) * 2.5).astype(np.float32)
    x[:3] = [0.0, -12.0, 12.0][: min(3, n)]
    dy = rng.standard_normal(n).astype(np.float32)
    dx_, ddy = DevBuf(x, skew=skew), DevBuf(dy, skew=skew)
    got = {}
    for name, L_ in (("ours", lib), ("reference", ref)):
        y, dx = DevBuf(n=n, skew=skew), DevBuf(n=n, skew=skew)
        L_.sl_cuda_gelu(dx_.ptr, y.ptr, n)
        L_.sl_cuda_gelu_bwd(dx_.ptr, ddy.ptr, dx.ptr, n)
        check_ok()
        got[name] = (y.get(), dx.get())
    assert ref.sl_cuda_check() == 0
    for mine, theirs in zip(got["ours"], got["reference"]):
        np.testing.assert_array_equal(mine.view(np.uint32), theirs.view(np.uint32))
    m = min(n, 20000)
    want_y, want_dx = step_ops.gelu(x[:m], dy[:m])
    np.testing.assert_allclose(got["ours"][0][:m], want_y, rtol=1e-6, atol=1e-6)
    np.testing.assert_allclose(got["ours"][1][:m], want_dx, rtol=1e-6, atol=1e-6)


# (tokens, vocabulary, columns, how the ids are drawn)
EMBEDDINGS = [(8192, 50257, 768, "uniform"), (8192, 1024, 768, "positions"), (7, 5, 16, "uniform"), (4096, 37, 16, "uniform"),
              (300, 11, 5, "uniform"), (64, 9, 64, "one")]


@pytest.mark.parametrize("n,vocab,c,draw", EMBEDDINGS)
def test_embedding_backward_gives_the_reference_bits(ref, n, vocab, c, draw):
    rng = np.random.default_rng(n + vocab)
    if draw == "uniform":
        idx = rng.integers(0, vocab, n).astype(np.int32)
    elif draw == "positions":
        idx = (np.arange(n) % vocab).astype(np.int32)                # every id 8 times, as a batch of 8 sequences has them
    else:
        idx = np.full(n, 3, np.int32)                                # one run holds every token
    dy = rng.standard_normal((n, c)).astype(np.float32)
    ddy, didx = DevBuf(dy), DevBuf(idx.view(np.float32))
    temp_bytes = n * 16 + (1 << 20)                                  # what the reference's host core sets aside (api.d:124-127)
    assert lib.sl_cuda_sort_temp_bytes(n) <= temp_bytes
    got = {}
    for name, fn in (("ours", lib.sl_cuda_embedding_bwd), ("reference", ref.sl_cuda_embedding_bwd)):
        dw = DevBuf(np.full(vocab * c, 7.0, np.float32))             # stale contents: the op overwrites all of dw
        keys, perm, perm_out, temp = DevBuf(n=n), DevBuf(n=n), DevBuf(n=n), DevBuf(n=temp_bytes // 4)
        fn(ddy.ptr, didx.ptr, dw.ptr, vocab, n, c, keys.ptr, perm.ptr, perm_out.ptr, temp.ptr, temp_bytes)
        check_ok()
        got[name] = dw.get().reshape(vocab, c)
    assert ref.sl_cuda_check() == 0
    np.testing.assert_array_equal(got["ours"].view(np.uint32), got["reference"].view(np.uint32))
    np.testing.assert_allclose(got["ours"], step_ops.embedding_bwd(idx, dy, vocab), rtol=1e-5, atol=1e-5 * np.sqrt(n))


def test_embedding_backward_reports_too_little_sort_space(cuda):
    n, vocab, c = 200000, 50, 4                                       # more tokens than one sorting tile: the sort needs room
    dy, idx, dw = DevBuf(n=n * c), DevBuf(np.zeros(n, np.int32).view(np.float32)), DevBuf(n=vocab * c)
    keys, perm, perm_out, temp = DevBuf(n=n), DevBuf(n=n), DevBuf(n=n), DevBuf(n=4)
    lib.sl_cuda_embedding_bwd(dy.ptr, idx.ptr, dw.ptr, vocab, n, c, keys.ptr, perm.ptr, perm_out.ptr, temp.ptr, 16)
    lib.sl_sync(2)
    assert lib.sl_cuda_sort_temp_bytes(n) > 16
    assert lib.sl_check(2) == 8                                       # the reference's code for this (core/cuda/kernels.cu:478-481)
    lib.slb_clear_error()

"""Layer normalisation, forward and backward (csrc/step_kernels.cu), through the backend-level C ABI, against the
reference's own kernels (core/cuda/kernels.cu:385-449, built unmodified into oracle/_ref/) and against float64.

Floating point: the reduction order differs from the reference's (a warp per row and a butterfly, where the reference
reduces a block in two stages; column sums in a fixed order over the blocks, where the reference calls cuBLAS), so results agree
to rounding, not to the bit. The bars are the reference's own test bars (tests/test_ops.py:17-26): outputs
rtol 1e-4 / atol 1e-4, gradients rtol 1e-3 / atol 1e-4 -- and, against the reference kernels on the same inputs, ten
times tighter than that."""
import ctypes as C
import os

import numpy as np
import pytest

from oracle import build as obuild
from oracle import step_ops
from soliton_b200._C import lib
from tests.gpu_util import DevBuf, check_ok

pytestmark = pytest.mark.gpu
F, L, P = C.c_float, C.c_int64, C.c_void_p
EPS = 1e-5
# (rows, c, skew): c a multiple of 256 up to 1024 takes the register path when the rows suffice for the per-block
# column sums; everything else (odd widths, one row, pointers that are not 32-byte aligned) the general path
SHAPES = [(8192, 768, 0), (300, 1024, 0), (64, 256, 0), (1000, 512, 0), (33, 768, 0), (1, 768, 0), (50, 32, 0), (7, 5, 0),
          (129, 1280, 0), (513, 768, 1)]


@pytest.fixture(scope="module")
def ref(cuda):
    path = obuild.build_ref()
    if not path or not os.path.exists(path):
        pytest.skip("reference CUDA backend not built (no reference checkout at build time)")
    r = C.CDLL(path)
    assert r.sl_cuda_set_device(0) == 0
    r.sl_cuda_layernorm.argtypes = [P] * 6 + [L, L, F, P]
    r.sl_cuda_layernorm.restype = None
    r.sl_cuda_layernorm_bwd.argtypes = [P] * 8 + [L, L] + [P] * 5
    r.sl_cuda_layernorm_bwd.restype = None
    return r


def truth(x, w, b, dy):
    """float64, the restatement of the reference's host twin (pinned against PyTorch in tests/test_step_ops_oracle.py)."""
    return step_ops.layernorm(x, w, b, dy, EPS)


def run(fns, rows, c, skew, x, w, b, dy):
    fwd, bwd = fns
    bufs = {k: DevBuf(v, skew=skew) for k, v in dict(x=x, w=w, b=b, dy=dy).items()}
    out = {k: DevBuf(n=n, skew=skew) for k, n in dict(y=rows * c, mean=rows, invstd=rows, dx=rows * c, dw=c, db=c,
                                                       tmp=rows * c, sg=rows, sgx=rows, ones_c=c, ones_rows=rows).items()}
    fwd(bufs["x"].ptr, bufs["w"].ptr, bufs["b"].ptr, out["y"].ptr, out["mean"].ptr, out["invstd"].ptr, rows, c, EPS, out["ones_c"].ptr)
    bwd(bufs["dy"].ptr, bufs["x"].ptr, bufs["w"].ptr, out["mean"].ptr, out["invstd"].ptr, out["dx"].ptr, out["dw"].ptr,
        out["db"].ptr, rows, c, out["tmp"].ptr, out["sg"].ptr, out["sgx"].ptr, out["ones_c"].ptr, out["ones_rows"].ptr)
    check_ok()
    return {k: out[k].get() for k in ("y", "mean", "invstd", "dx", "dw", "db")}


@pytest.mark.parametrize("rows,c,skew", SHAPES)
def test_layernorm_forward_and_backward(ref, rows, c, skew):
    rng = np.random.default_rng(rows * 31 + c)
    x = (rng.standard_normal((rows, c)) * 1.7 + 0.3).astype(np.float32)
    w = (1.0 + 0.1 * rng.standard_normal(c)).astype(np.float32)
    b = (0.1 * rng.standard_normal(c)).astype(np.float32)
    dy = rng.standard_normal((rows, c)).astype(np.float32)
    ours = run((lib.sl_cuda_layernorm, lib.sl_cuda_layernorm_bwd), rows, c, skew, x, w, b, dy)
    again = run((lib.sl_cuda_layernorm, lib.sl_cuda_layernorm_bwd), rows, c, skew, x, w, b, dy)
    theirs = run((ref.sl_cuda_layernorm, ref.sl_cuda_layernorm_bwd), rows, c, skew, x, w, b, dy)
    assert ref.sl_cuda_check() == 0
    want = dict(zip(("y", "mean", "invstd", "dx", "dw", "db"), truth(x, w, b, dy)))
    for k in ours:
        np.testing.assert_array_equal(ours[k], again[k])           # no atomics, fixed orders: the same bits every run
        t = want[k].ravel()
        scale = max(1.0, float(np.max(np.abs(t))))
        rtol = 1e-4 if k in ("y", "mean", "invstd") else 1e-3       # tests/test_ops.py:21,26 of the reference
        np.testing.assert_allclose(ours[k], t, rtol=rtol, atol=1e-4 * scale, err_msg=k)
        np.testing.assert_allclose(ours[k], theirs[k], rtol=rtol / 10, atol=1e-5 * scale, err_msg=k + " vs reference kernel")
        # at least as close to float64 as the reference kernel is, up to a small allowance
        assert np.max(np.abs(ours[k] - t)) <= 4 * np.max(np.abs(theirs[k] - t)) + 1e-5 * scale, k

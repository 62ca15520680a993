"""Fused causal attention, forward and backward (csrc/attention_kernels.cu), through the backend-level C ABI, against
float64 and against the reference's own kernels (core/cuda/kernels.cu:536-692, built unmodified into oracle/_ref/),
in both precisions of the reference's matmuls: fp32 (the default) and TF32 (sl_cuda_set_tf32(1)).

Floating point, so agreement to rounding. Both implementations are measured against a float64 evaluation of the same
formulas.
fp32 mode (split products, three TF32 products per fp32 product): the reference's own test bars for this op
(tests/test_ops.py:84-85: outputs rtol 1e-4 / atol 1e-5, gradients rtol 1e-3 / atol 1e-4) against float64, and an
error within 2^-16 of the largest value: a split product is good to about 2^-21 per operand pair where fp32 is good
to 2^-24, so the distance to float64 is some eight times the reference's fp32 path's.
TF32 mode (10-bit mantissa): at least as close to float64 as the reference's TF32 path is, with a factor 1.5 of
slack for the different operand rounding, and inside an absolute bar that follows from the operand precision, 2^-10.
The reference's TF32 path does not meet the fp32 bars either; the table printed on failure shows both."""
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
HS = 64
# (B, T, H): T a multiple of 64; 1024 is GPT-2's context, 64 a single tile, 192 an odd number of tiles
SHAPES = [(1, 64, 1), (2, 192, 3), (1, 256, 2), (2, 1024, 2), (1, 512, 12)]


@pytest.fixture(scope="module")
def ref(cuda):
    path = obuild.build_ref()
    if not path or not os.path.exists(path):
        pytest.skip("reference CUDA backend not built (no reference checkout at build time)")
    r = C.CDLL(path)
    assert r.sl_cuda_set_device(0) == 0
    r.sl_cuda_attention.argtypes = [P] * 3 + [L] * 4 + [F, L] + [P] * 8
    r.sl_cuda_attention.restype = None
    r.sl_cuda_attention_bwd.argtypes = [P] * 5 + [L] * 4 + [F, L] + [P] * 9
    r.sl_cuda_attention_bwd.restype = None
    r.sl_cuda_set_tf32.argtypes = [C.c_int]
    r.sl_cuda_set_tf32.restype = None
    yield r
    r.sl_cuda_set_tf32(0)
    lib.sl_cuda_attention_set_tf32(0)


def truth(qkv, dout, scale):
    """float64: out, L, dqkv for qkv (B, T, 3, H, hs), dout (B, T, H, hs): the restatement of the reference's host
    twin (pinned against PyTorch in tests/test_step_ops_oracle.py)."""
    return step_ops.attention(qkv, dout, scale)


def chunks_for(dim):
    c = 1
    while c * c < dim:
        c += 1
    return c


def run(fns, B, T, H, qkv, dout, scale):
    """Both passes with the scratch the reference's host core hands over (core/soliton/api.d:501-541)."""
    fwd, bwd = fns
    tile = 256 if T % 256 == 0 else T
    bh = B * H
    rows = bh * tile
    d = {k: DevBuf(v) for k, v in dict(qkv=qkv, dout=dout).items()}
    o = {k: DevBuf(n=n) for k, n in dict(out=B * T * H * HS, L=bh * T, dqkv=B * T * 3 * H * HS, s=rows * tile, dp=rows * tile,
                                         acc=rows * HS, oc=rows * HS, m=rows, l=rows, c=rows, rowbuf=rows * (chunks_for(tile) + 1),
                                         ones=max(tile, HS), ptrs=2 * 9 * bh).items()}
    fwd(d["qkv"].ptr, o["out"].ptr, o["L"].ptr, B, T, H, HS, scale, tile, o["s"].ptr, o["acc"].ptr, o["m"].ptr, o["l"].ptr,
        o["c"].ptr, o["rowbuf"].ptr, o["ones"].ptr, o["ptrs"].ptr)
    bwd(d["qkv"].ptr, o["out"].ptr, o["L"].ptr, d["dout"].ptr, o["dqkv"].ptr, B, T, H, HS, scale, tile, o["s"].ptr, o["dp"].ptr,
        o["acc"].ptr, o["oc"].ptr, o["m"].ptr, o["l"].ptr, o["rowbuf"].ptr, o["ones"].ptr, o["ptrs"].ptr)
    check_ok()
    return {k: o[k].get() for k in ("out", "L", "dqkv")}


@pytest.mark.parametrize("tf32", [0, 1])
@pytest.mark.parametrize("B,T,H", SHAPES)
def test_attention_forward_and_backward(ref, B, T, H, tf32):
    ref.sl_cuda_set_tf32(tf32)
    lib.sl_cuda_attention_set_tf32(tf32)
    rng = np.random.default_rng(B * 1000 + T + H)
    qkv = rng.standard_normal((B, T, 3, H, HS)).astype(np.float32)
    qkv[:, :, 0] *= 1.5                                               # scores of a few units: a softmax with peaks
    dout = rng.standard_normal((B, T, H, HS)).astype(np.float32)
    scale = 1.0 / np.sqrt(HS)
    ours = run((lib.sl_cuda_attention, lib.sl_cuda_attention_bwd), B, T, H, qkv, dout, scale)
    again = run((lib.sl_cuda_attention, lib.sl_cuda_attention_bwd), B, T, H, qkv, dout, scale)
    theirs = run((ref.sl_cuda_attention, ref.sl_cuda_attention_bwd), B, T, H, qkv, dout, scale)
    assert ref.sl_cuda_check() == 0
    want = dict(zip(("out", "L", "dqkv"), truth(qkv, dout, scale)))
    report = []
    for k in ("out", "L", "dqkv"):
        np.testing.assert_array_equal(ours[k], again[k])             # no atomics, fixed orders: the same bits every run
        t = want[k].ravel()
        mine, ref_err = np.abs(ours[k] - t), np.abs(theirs[k] - t)
        report.append(f"{k}: ours max {mine.max():.3e} rms {np.sqrt((mine ** 2).mean()):.3e}; "
                      f"reference max {ref_err.max():.3e} rms {np.sqrt((ref_err ** 2).mean()):.3e}")
    text = "\n".join(report)
    for k in ("out", "L", "dqkv"):
        t = want[k].ravel()
        mine, ref_err = np.abs(ours[k] - t), np.abs(theirs[k] - t)
        rms, ref_rms = np.sqrt((mine ** 2).mean()), np.sqrt((ref_err ** 2).mean())
        assert np.isfinite(ours[k]).all(), text
        top = max(1.0, float(np.abs(t).max()))
        if tf32:
            assert rms <= 1.5 * ref_rms + 1e-7, text
            # 2^-10 per operand, sums of up to T products of magnitude about one, three roundings deep for gradients
            assert mine.max() <= 2.0 ** -10 * (8 if k == "dqkv" else 4) * top, text
        else:
            rtol, atol = (1e-3, 1e-4) if k == "dqkv" else (1e-4, 1e-5)  # tests/test_ops.py:84-85 of the reference
            assert np.all(mine <= atol + rtol * np.abs(t)), text
            assert mine.max() <= 2.0 ** -16 * top, text


def test_unsupported_shapes_are_refused(cuda):
    assert lib.sl_cuda_attention_supported(1024, 64) == 1
    assert lib.sl_cuda_attention_supported(1000, 64) == 0
    assert lib.sl_cuda_attention_supported(1024, 32) == 0
    buf = DevBuf(n=4096)
    lib.sl_cuda_attention(buf.ptr, buf.ptr, buf.ptr, 1, 16, 1, 16, 0.25, 16, None, None, None, None, None, None, None, None)
    lib.sl_sync(2)
    assert lib.sl_check(2) == 2                                       # sticky launch error, nothing ran
    lib.slb_clear_error()
    assert lib.sl_check(2) == 0

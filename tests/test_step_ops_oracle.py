"""The float64 restatements of the step's compute ops (oracle/step_ops.py) pinned against PyTorch on the CPU with
the reference's own recipes: same seeds, shapes and bars as its tests/test_ops.py (gelu and layernorm :45-46 with
check() :13-27, fused attention :69-85, embedding :88-102, cross entropy :105-119), plus the shapes the GPU tests use.
No GPU: the GPU tests then hold the kernels against these functions."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

from oracle import step_ops


def test_gelu_matches_torch_with_the_reference_recipe():
    rng = np.random.default_rng(0)                                    # check(): rng(0), standard normal, then gy
    x = rng.standard_normal((4, 9)).astype(np.float32)
    gy = rng.standard_normal((4, 9)).astype(np.float32)
    tx = torch.tensor(x, requires_grad=True)
    ty = F.gelu(tx)
    ty.backward(torch.tensor(gy))
    y, dx = step_ops.gelu(x, gy)
    np.testing.assert_allclose(y, ty.detach().numpy(), rtol=1e-4, atol=1e-4)
    np.testing.assert_allclose(dx, tx.grad.numpy(), rtol=1e-3, atol=1e-4)
    np.testing.assert_allclose(y, ty.detach().numpy(), rtol=0, atol=2e-7)   # float64 against torch's fp32: one rounding
    np.testing.assert_allclose(dx, tx.grad.numpy(), rtol=0, atol=5e-7)


@pytest.mark.parametrize("shape", [(2, 3, 8), (33, 768), (7, 5)])
def test_layernorm_matches_torch_with_the_reference_recipe(shape):
    rng = np.random.default_rng(0)
    c = shape[-1]
    x, w, b = (rng.standard_normal(s).astype(np.float32) for s in (shape, (c,), (c,)))
    gy = rng.standard_normal(shape).astype(np.float32)
    tx, tw, tb = (torch.tensor(a, requires_grad=True) for a in (x, w, b))
    ty = F.layer_norm(tx, (c,), tw, tb, 1e-5)
    ty.backward(torch.tensor(gy))
    y, mean, invstd, dx, dw, db = step_ops.layernorm(x.reshape(-1, c), w, b, gy.reshape(-1, c), 1e-5)
    np.testing.assert_allclose(y.reshape(shape), ty.detach().numpy(), rtol=1e-4, atol=1e-4)
    np.testing.assert_allclose(dx.reshape(shape), tx.grad.numpy(), rtol=1e-3, atol=1e-4)
    np.testing.assert_allclose(dw, tw.grad.numpy(), rtol=1e-3, atol=1e-4)
    np.testing.assert_allclose(db, tb.grad.numpy(), rtol=1e-3, atol=1e-4)
    np.testing.assert_allclose(mean, x.reshape(-1, c).astype(np.float64).mean(axis=1), rtol=0, atol=1e-12)
    np.testing.assert_allclose(invstd ** -2, x.reshape(-1, c).astype(np.float64).var(axis=1) + 1e-5, rtol=1e-12)


@pytest.mark.parametrize("t,hs", [(6, 16), (256, 16), (512, 16), (192, 64)])
def test_attention_matches_torch_with_the_reference_recipe(t, hs):
    b, h = 2, 3
    rng = np.random.default_rng(4)                                    # tests/test_ops.py:73-75
    packed = rng.standard_normal((b, t, 3, h, hs)).astype(np.float32)
    gy = rng.standard_normal((b, t, h, hs)).astype(np.float32)
    tq = torch.tensor(packed, requires_grad=True)
    q, k, v = (tq[:, :, i].transpose(1, 2) for i in range(3))
    tout = F.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2)
    tout.backward(torch.tensor(gy))
    out, L, dqkv = step_ops.attention(packed, gy, 1.0 / np.sqrt(hs))
    np.testing.assert_allclose(out, tout.detach().numpy(), rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(dqkv, tq.grad.numpy(), rtol=1e-3, atol=1e-4)
    # L is the log of the softmax denominator of the scaled, masked scores
    s = np.einsum("bqhd,bkhd->bhqk", packed[:, :, 0].astype(np.float64), packed[:, :, 1].astype(np.float64)) / np.sqrt(hs)
    s = np.where(np.tril(np.ones((t, t), bool)), s, -np.inf)
    np.testing.assert_allclose(L, np.log(np.exp(s - s.max(-1, keepdims=True)).sum(-1)) + s.max(-1), rtol=1e-12)
    assert L.shape == (b, h, t)


@pytest.mark.parametrize("n,vocab", [(7, 5), (4096, 37)])
def test_embedding_backward_matches_torch_with_the_reference_recipe(n, vocab):
    rng = np.random.default_rng(1)                                    # tests/test_ops.py:91-94
    w = rng.standard_normal((vocab, 16)).astype(np.float32)
    idx = rng.integers(0, vocab, size=(n,)).astype(np.int32)
    gy = rng.standard_normal((n, 16)).astype(np.float32)
    tw = torch.tensor(w, requires_grad=True)
    F.embedding(torch.tensor(idx, dtype=torch.long), tw).backward(torch.tensor(gy))
    np.testing.assert_allclose(step_ops.embedding_bwd(idx, gy, vocab), tw.grad.numpy(), rtol=1e-4, atol=1e-3)


@pytest.mark.parametrize("n,vocab", [(6, 11), (512, 4099)])
def test_cross_entropy_matches_torch_with_the_reference_recipe(n, vocab):
    rng = np.random.default_rng(2)                                    # tests/test_ops.py:108-110
    logits = (rng.standard_normal((n, vocab)) * 3).astype(np.float32)
    tgt = rng.integers(0, vocab, size=(n,)).astype(np.int32)
    tx = torch.tensor(logits, requires_grad=True)
    tloss = F.cross_entropy(tx, torch.tensor(tgt, dtype=torch.long))
    tloss.backward()
    loss, d = step_ops.cross_entropy(logits, tgt, 1.0)
    assert abs(loss - tloss.item()) < 1e-4
    np.testing.assert_allclose(d, tx.grad.numpy(), rtol=1e-3, atol=1e-6)
    np.testing.assert_allclose(d.sum(axis=1), 0.0, atol=1e-12)        # softmax - onehot sums to zero in every row


@pytest.mark.parametrize("op", [0, 1, 2, 3])
def test_binary_matches_torch_with_the_reference_shapes(op):
    rng = np.random.default_rng(0)                                    # CASES add/sub/mul/div broadcast shapes, :31-34
    shapes = [((2, 3, 4), (4,)), ((2, 3, 4), (3, 1)), ((2, 1, 4), (3, 4)), ((3, 4), (4,))][op]
    a, b = (rng.standard_normal(s).astype(np.float32) for s in shapes)
    if op == 3:
        b = np.abs(b) + 0.5
    want = [torch.add, torch.sub, torch.mul, torch.div][op](torch.tensor(a), torch.tensor(b)).numpy()
    np.testing.assert_array_equal(step_ops.binary(op, a, b).view(np.uint32), want.view(np.uint32))

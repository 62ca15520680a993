"""TEST INFRASTRUCTURE ONLY. float64 restatements of the reference's host twins of the step's compute kernels.

The reference keeps a plain-loop CPU version of every op (core/soliton/cpu.d) as the thing its CUDA kernels are
tested against; its D core cannot be compiled here (no D compiler), so these are restatements in numpy, evaluated in
float64 throughout (the D code accumulates in double and stores float; the tests that use these compare with
tolerances, not bits). Each function cites the lines it follows. Pinned by tests/test_step_ops_oracle.py against
PyTorch on the CPU with the reference's own test recipes (tests/test_ops.py), which is how the reference pins them.
Nothing outside tests/ imports this module.
"""
import math

import numpy as np

_erf = np.vectorize(math.erf, otypes=[np.float64])


def binary(op, a, b):
    """core/soliton/cpu.d:38-61: out = a op b with numpy broadcasting; op 0 add, 1 subtract, 2 multiply, 3 divide.
    In float32: one IEEE operation per element, so this one is exact to the bit."""
    a, b = np.asarray(a, np.float32), np.asarray(b, np.float32)
    return [np.add, np.subtract, np.multiply, np.divide][op](a, b).astype(np.float32)


def gelu(x, dy):
    """core/soliton/cpu.d:166-181: y = x * Phi(x) with Phi through erf; dx = dy * (Phi(x) + x * phi(x))."""
    x, dy = np.asarray(x, np.float64), np.asarray(dy, np.float64)
    cdf = 0.5 * (1.0 + _erf(x / math.sqrt(2.0)))
    pdf = np.exp(-0.5 * x * x) / math.sqrt(2.0 * math.pi)
    return x * cdf, dy * (cdf + x * pdf)


def layernorm(x, w, b, dy, eps):
    """core/soliton/cpu.d:183-230: rows of c elements; biased variance; returns y, mean, 1/std, dx, dw, db."""
    x, w, b, dy = (np.asarray(a, np.float64) for a in (x, w, b, dy))
    mean = x.mean(axis=1, keepdims=True)
    invstd = 1.0 / np.sqrt(((x - mean) ** 2).mean(axis=1, keepdims=True) + eps)
    xh = (x - mean) * invstd
    g = dy * w
    dx = invstd * (g - g.mean(axis=1, keepdims=True) - xh * (g * xh).mean(axis=1, keepdims=True))
    return xh * w + b, mean.ravel(), invstd.ravel(), dx, (dy * xh).sum(axis=0), dy.sum(axis=0)


def embedding_bwd(idx, dy, vocab):
    """core/soliton/cpu.d:238-244: dw[idx[i]] += dy[i], tokens in order, from zero."""
    dy = np.asarray(dy, np.float64)
    dw = np.zeros((vocab, dy.shape[1]), np.float64)
    np.add.at(dw, np.asarray(idx), dy)
    return dw


def cross_entropy(logits, t, dloss):
    """core/soliton/cpu.d:247-276: mean over rows of log(sum exp(l - max)) + max - l[target]; gradient
    (softmax - onehot) * g with g = dloss / n formed in float32 as the reference forms it."""
    x = np.asarray(logits, np.float64)
    t = np.asarray(t)
    n = len(t)
    m = x.max(axis=1, keepdims=True)
    e = np.exp(x - m)
    z = e.sum(axis=1, keepdims=True)
    loss = (np.log(z[:, 0]) + m[:, 0] - x[np.arange(n), t]).mean()
    g = np.float64(np.float32(dloss) / np.float32(n))
    d = e / z * g
    d[np.arange(n), t] -= g
    return loss, d


def attention(qkv, dout, scale):
    """core/soliton/cpu.d:279-360: qkv packed (B, T, 3, H, hs), dout (B, T, H, hs). Scores scale * q.k, keys after
    the query masked; out = softmax(scores) v; L (B, H, T) = row maximum + log of the row's sum of exponentials;
    backward with D = rowsum(dout * out): dv = P^T dout, dS = P * (dout v^T - D) * scale, dq = dS k, dk = dS^T q.
    Returns out (B, T, H, hs), L, dqkv (B, T, 3, H, hs)."""
    qkv, dout = np.asarray(qkv, np.float64), np.asarray(dout, np.float64)
    q, k, v = (qkv[:, :, i].transpose(0, 2, 1, 3) for i in range(3))  # (B, H, T, hs)
    do = dout.transpose(0, 2, 1, 3)
    T = q.shape[2]
    s = scale * q @ k.transpose(0, 1, 3, 2)
    s = np.where(np.tril(np.ones((T, T), bool)), s, -np.inf)
    m = s.max(axis=-1, keepdims=True)
    e = np.exp(s - m)
    l = e.sum(axis=-1, keepdims=True)
    p = e / l
    o = p @ v
    dv = p.transpose(0, 1, 3, 2) @ do
    dp = do @ v.transpose(0, 1, 3, 2)
    ds = p * (dp - (do * o).sum(axis=-1, keepdims=True)) * scale
    dq, dk = ds @ k, ds.transpose(0, 1, 3, 2) @ q
    dqkv = np.stack([g.transpose(0, 2, 1, 3) for g in (dq, dk, dv)], axis=2)
    return o.transpose(0, 2, 1, 3), (m + np.log(l))[..., 0], dqkv

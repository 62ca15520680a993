"""Synthetic workloads of the optimizer path: the parameter set of Soliton's GPT-2 example and seeded values.

Shapes and order follow `Module.named_parameters` (python/soliton/nn.py:7-16) over the example model
(examples/gpt2.py:23-30,60-65): wte, wpe, then per block ln1.{weight,bias}, ln2.{weight,bias}, qkv.{weight,bias},
proj.{weight,bias}, fc.{weight,bias}, fc_proj.{weight,bias}, then ln_f.{weight,bias}. Linear weights are
(n_out, n_in) (nn.py:34). Values use the reference's RNG idiom (python/soliton/tensor.py:259-263):
`default_rng(seed).standard_normal(shape, dtype=float32) * std`, drawn in parameter order.
"""
import math

import numpy as np

MODELS = {
    # examples/gpt2.py:76-79 has "124M" and "tiny"; "medium" is GPT-2 medium in the same layout.
    "124M": dict(vocab=50257, block_size=1024, n_layer=12, n_embd=768),
    "medium": dict(vocab=50257, block_size=1024, n_layer=24, n_embd=1024),
    "tiny": dict(vocab=512, block_size=64, n_layer=2, n_embd=32),
}


def param_shapes(model="124M"):
    """[(name, shape, kind)] with kind in {"normal", "residual", "ones", "zeros"} (how the example initialises it)."""
    cfg = MODELS[model]
    c = cfg["n_embd"]
    out = [("wte.weight", (cfg["vocab"], c), "normal"), ("wpe.weight", (cfg["block_size"], c), "normal")]
    for i in range(cfg["n_layer"]):
        b = f"blocks.{i}."
        out += [(b + "ln1.weight", (c,), "ones"), (b + "ln1.bias", (c,), "zeros"),
                (b + "ln2.weight", (c,), "ones"), (b + "ln2.bias", (c,), "zeros"),
                (b + "qkv.weight", (3 * c, c), "normal"), (b + "qkv.bias", (3 * c,), "zeros"),
                (b + "proj.weight", (c, c), "residual"), (b + "proj.bias", (c,), "zeros"),
                (b + "fc.weight", (4 * c, c), "normal"), (b + "fc.bias", (4 * c,), "zeros"),
                (b + "fc_proj.weight", (c, 4 * c), "residual"), (b + "fc_proj.bias", (c,), "zeros")]
    out += [("ln_f.weight", (c,), "ones"), ("ln_f.bias", (c,), "zeros")]
    return out


def numel(shape):
    return int(np.prod(shape, dtype=np.int64))


def total_params(model="124M"):
    return sum(numel(s) for _, s, _ in param_shapes(model))


def init_params(model="124M", seed=0):
    """Parameter values as examples/gpt2.py builds them: N(0, 0.02), residual projections N(0, 0.02/sqrt(2 L)),
    layer-norm weights 1, biases 0. Returns a list of float32 arrays in parameter order."""
    rng = np.random.default_rng(seed)
    n_layer = MODELS[model]["n_layer"]
    out = []
    for _, shape, kind in param_shapes(model):
        if kind == "normal":
            out.append(rng.standard_normal(shape, dtype=np.float32) * np.float32(0.02))
        elif kind == "residual":
            out.append(rng.standard_normal(shape, dtype=np.float32) * np.float32(0.02 / math.sqrt(2 * n_layer)))
        elif kind == "ones":
            out.append(np.ones(shape, np.float32))
        else:
            out.append(np.zeros(shape, np.float32))
    return out


def rank_grads(model="124M", rank=0, std=1e-3):
    """Per-rank synthetic gradients: default_rng(1 + rank), N(0, std) for every tensor, in parameter order."""
    rng = np.random.default_rng(1 + rank)
    return [rng.standard_normal(shape, dtype=np.float32) * np.float32(std) for _, shape, _ in param_shapes(model)]


def flat_case(n, seed_p=0, seed_g=1, rank=0):
    """The flat-buffer configuration: p ~ N(0, 0.02) from seed_p, g ~ N(0, 1e-3) from seed_g + rank, m = v = 0."""
    p = np.random.default_rng(seed_p).standard_normal(n, dtype=np.float32) * np.float32(0.02)
    g = np.random.default_rng(seed_g + rank).standard_normal(n, dtype=np.float32) * np.float32(1e-3)
    return p, g


# Hyperparameters the benchmark configurations are quoted on.
HYPER = dict(lr=3e-4, b1=0.9, b2=0.999, eps=1e-8, wd=0.1)

"""Host-side decisions of the step kernels, checked without a GPU: which binary-op kernel a shape/stride pattern gets
(against a Python restatement of the reference's suffix_numel, core/cuda/kernels.cu:154-169) and which attention
shapes the fused kernels take."""
import ctypes as C
import itertools

import numpy as np


def suffix_numel(shape, stride):
    """core/cuda/kernels.cu:154-169: elements of an input that is the output's trailing dimensions laid out densely
    (and repeated over the leading ones), else -1."""
    dense, n, leading = 1, 1, False
    for size, st in zip(reversed(shape), reversed(stride)):
        if not leading and st == dense:
            n *= size
            dense *= size
            continue
        leading = True
        if st != 0 and size != 1:
            return -1
    return n


def plan(lib, shape, sa, sb):
    arr = lambda v: (C.c_int64 * max(1, len(v)))(*v)  # noqa: E731
    out = (C.c_int64 * 2)()
    kind = lib.slb_binary_plan(len(shape), arr(shape), arr(sa), arr(sb), out)
    return kind, out[0], out[1]


def broadcast_strides(array_shape, out_shape):
    pad = (1,) * (len(out_shape) - len(array_shape)) + tuple(array_shape)
    dense, out = 1, []
    for size in reversed(pad):
        out.append(0 if size == 1 else dense)
        dense *= size
    return list(reversed(out))


def test_training_step_shapes_take_the_wide_kernel(lib):
    out = (8, 1024, 3072)
    dense = broadcast_strides(out, out)
    assert plan(lib, out, dense, dense) == (2, 8 * 1024 * 3072, 8 * 1024 * 3072)              # residual add
    assert plan(lib, out, dense, broadcast_strides((3072,), out)) == (2, 8 * 1024 * 3072, 3072)  # bias add
    assert plan(lib, (8, 1024, 768), broadcast_strides((8, 1024, 768), (8, 1024, 768)),
                broadcast_strides((1024, 768), (8, 1024, 768))) == (2, 8 * 1024 * 768, 1024 * 768)  # positions
    assert plan(lib, (64, 64), [64, 1], [0, 0]) == (1, 4096, 1)                                # scalar: not a multiple of 4
    assert plan(lib, (7, 5), [5, 1], [0, 1]) == (1, 35, 5)
    assert plan(lib, (48, 20), [20, 1], [1, 48])[0] == 0                                       # a transposed input
    assert plan(lib, (4, 5, 6), [30, 6, 1], [6, 0, 1])[0] == 0                                 # repeats in the middle
    assert plan(lib, (1,) * 9, [0] * 9, [0] * 9)[0] == -1                                      # more than 8 dimensions
    assert plan(lib, (), [], []) == (1, 1, 1)                                                  # no dimensions: one element


def test_classification_is_the_reference_rule_on_every_small_pattern(lib):
    rng = np.random.default_rng(0)
    checked = 0
    for nd in (1, 2, 3, 4):
        for shape in itertools.product((1, 2, 4), repeat=nd):
            dense = broadcast_strides(shape, shape)
            candidates = [dense, [0] * nd]
            for _ in range(6):
                candidates.append([int(rng.choice([0, d, 1, 2, 4])) for d in dense])
            for sa, sb in itertools.product(candidates, repeat=2):
                kind, na, nb = plan(lib, shape, sa, sb)
                want_a, want_b = suffix_numel(shape, sa), suffix_numel(shape, sb)
                assert (na, nb) == (want_a, want_b), (shape, sa, sb)
                n = int(np.prod(shape))
                if want_a > 0 and want_b > 0:
                    assert kind == (2 if n % 4 == 0 and want_a % 4 == 0 and want_b % 4 == 0 else 1), (shape, sa, sb)
                else:
                    assert kind == 0, (shape, sa, sb)
                checked += 1
    assert checked > 5000


def test_fused_attention_takes_head_size_64_and_whole_tiles(lib):
    for T, hs, want in ((1024, 64, 1), (64, 64, 1), (192, 64, 1), (0, 64, 0), (32, 64, 0), (1000, 64, 0), (1024, 32, 0),
                        (1024, 128, 0), (6, 16, 0), (256, 16, 0)):
        assert lib.sl_cuda_attention_supported(T, hs) == want, (T, hs)

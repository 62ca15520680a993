"""soliton_b200: B200-native data-parallel optimizer path for Soliton (gradient mean over ranks + AdamW).

The package holds only what that path needs: the CUDA/C++ library (csrc/, built by soliton_b200.build), its ctypes
binding, and thin mirrors of the Soliton Python interfaces that call into the path (optim, distributed, tensor).
Submodules load on first use, so that `python -m soliton_b200.build` works before the library exists.
"""
import importlib

_SUBMODULES = ("arena", "build", "distributed", "optim", "tensor", "workload", "_C")


def __getattr__(name):
    if name in _SUBMODULES:
        return importlib.import_module(f"{__name__}.{name}")
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")

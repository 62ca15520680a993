"""soliton_b200: B200-native data-parallel optimizer path for Soliton (gradient mean over ranks + AdamW).

The package holds only what that path needs: the CUDA/C++ library (csrc/, built by soliton_b200.build), its ctypes
binding, and thin mirrors of the Soliton Python interfaces that call into the path (optim, distributed, tensor).
"""
from . import distributed, optim, tensor, workload  # noqa: F401
from .tensor import (empty, empty_cache, memory_stats, reset_peak_stats, set_device, set_memory_limit,  # noqa: F401
                     synchronize, tensor as from_numpy, zeros)

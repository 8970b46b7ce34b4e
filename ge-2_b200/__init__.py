"""ge2_b200: B200 (sm_100a) implementation of the per-batch graph-embedding training path
(unique-map -> fused negative-sampling decoder forward/loss/backward -> sparse Adagrad scatter -> partition swaps).

The directory name carries a hyphen; import it with ``importlib.import_module("ge-2_b200")``.  The compute path is the CUDA library ``libge2_b200.so`` built
in-tree by ``build.py``; there is no CPU or PyTorch fallback: using an op without the library raises.
"""
from . import capi  # noqa: F401
from .capi import Ge2Error, lib_path, load_library  # noqa: F401

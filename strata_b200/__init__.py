"""B200-native MoE expert block behind a C ABI (include/strata_moe.h).

The compute lives in strata_b200/libstrata_moe.so (hand-written sm_100a CUDA).  This package is
the Python binding used by the tests, the benchmark and the expert-parallel driver; it never
computes on the CPU and raises if the library or a CUDA device is missing.
"""
from .api import MoeContext, MoeLayer, StrataMoeError, library_path, load_library  # noqa: F401

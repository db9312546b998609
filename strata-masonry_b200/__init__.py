"""strata-masonry_b200: B200 (sm_100a) dense GEMM path behind a C ABI.

The package is a thin ctypes binding over ``lib/libstrata_masonry_b200.so`` plus a Python
mirror of the reference drivers' command-line contract (``drivers.py``).  There is no
CPU implementation in here: if the CUDA library has not been built, importing
``strata_masonry_b200.capi`` raises.
"""
from . import capi, gemm, sharding  # noqa: F401
from .capi import SmbError, lib  # noqa: F401

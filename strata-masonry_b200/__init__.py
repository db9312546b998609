"""strata-masonry_b200: B200 (sm_100a) dense GEMM path behind a C ABI.

The package is a thin ctypes binding over ``lib/libstrata_masonry_b200.so`` (``capi``: the
signature table, ``gemm``: plan and context classes, ``sharding``: the N column-parallel split
and the peer-mapped buffers of the fused collectives).  The drop-in executables of the reference
drivers are built from ``csrc/driver_*.cu`` into ``bin/``.  There is no CPU implementation in here: if the CUDA library has not been built, importing
``strata_masonry_b200.capi`` raises.
"""
from . import capi, gemm, sharding  # noqa: F401
from .capi import SmbError, lib  # noqa: F401

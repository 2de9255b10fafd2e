"""riemannengine_b200 — B200-native sparse-convolution hot path.

Coordinate hashing, kernel-map generation and gather-GEMM-scatter convolution
as hand-written sm_100a CUDA kernels behind a C ABI (``include/rmn_b200.h``),
with a host layer that mirrors the reference's ``SparseTensor`` /
``CoordinateManager`` / ``RiemannConvolution`` interface.
"""
from . import capi  # noqa: F401

__all__ = ["capi"]
__version__ = "0.1.0"

"""mm_rs_with_catlass_b200 — fused matmul + collective ops for B200 (sm_100a).

A Blackwell-native library with the capabilities of the Ascend "CATCOC" templates: a
symmetric-heap SHMEM layer over NVLink / NVSwitch peer memory and four fused ops
(matmul-allreduce, allgather-matmul, matmul-reduce-scatter, quantised matmul-reduce-scatter),
each a single hand-written tcgen05 / TMA kernel that communicates from inside its tile loop.
"""
from . import _native  # noqa: F401
from .tiling.config import TilingConfig  # noqa: F401

__version__ = "0.1.0"

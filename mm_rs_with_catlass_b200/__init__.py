"""mm_rs_with_catlass_b200 — fused matmul + collective ops for B200 (sm_100a).

A Blackwell-native library with the capabilities of the Ascend "CATCOC" templates: a
symmetric-heap SHMEM layer over NVLink / NVSwitch peer memory and four fused ops
(matmul-allreduce, allgather-matmul, matmul-reduce-scatter, quantised matmul-reduce-scatter),
each a single hand-written tcgen05 / TMA kernel that communicates from inside its tile loop.

Typical use (one process per GPU, ``torch.distributed`` initialised):

    import mm_rs_with_catlass_b200 as catcoc
    ctx = catcoc.init()                                   # symmetric heap over the world group
    y = catcoc.matmul_reduce_scatter(a, b)                # [M/W, N]
    y, gathered = catcoc.allgather_matmul(a_shard, b)     # [W*m, N], [W*m, K]
    ctx.finalize()
"""
from . import _native  # noqa: F401
from .tiling.config import TilingConfig  # noqa: F401
from .parallel.shmem import init, default_context, ShmemContext, ShmemError  # noqa: F401
from .ops.gemm import matmul  # noqa: F401
from .ops.fused import (matmul_allreduce, allgather_matmul, matmul_reduce_scatter,  # noqa: F401
                        quant_matmul_reduce_scatter)

from .ops.blas import (gemm, matmul_bias, matmul_add, optimized_matmul, batched_matmul,  # noqa: F401
                       grouped_matmul, grouped_quant_matmul, grouped_matmul_slice_k, group_gemm,
                       splitk_matmul, gemv)
from .ops.mx import (mxf8_matmul, mxf8_matmul_reduce_scatter, quantize_mxf8, dequantize_mxf8,  # noqa: F401
                     pack_scales)

from .ops.attention import flash_attention  # noqa: F401
from .ops.mla import mla_decode  # noqa: F401

from .ops import torch_ops  # noqa: F401  (registers torch.ops.catcoc.*)

__version__ = "0.1.0"

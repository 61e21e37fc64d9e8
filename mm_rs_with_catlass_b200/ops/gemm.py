"""Single-GPU GEMM on the library's own tcgen05 kernel.

This is the W = 1 degenerate case of every fused op (same kernel, ``MODE_LOCAL``), the
building block for unit tests and the probe used to measure the GEMM-only gap to cuBLAS.
It covers the plain kernels of the reference's GEMM template library that the fused ops
rely on: basic matmul, matmul with int32 bias and int8 matmul with per-token / per-channel
dequantisation (3rdparty/catlass/include/catlass/gemm/kernel/basic_matmul.hpp:105-137,
matmul_bias.hpp, quant_matmul.hpp).
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import _native as N
from ..tiling.config import TilingConfig
from . import _common as cm


def matmul(a: torch.Tensor, b: torch.Tensor, *, trans_a: bool = False, trans_b: bool = False,
           out: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None,
           scale_m: Optional[torch.Tensor] = None, scale_n: Optional[torch.Tensor] = None,
           bias: Optional[torch.Tensor] = None, tiling: Optional[TilingConfig] = None,
           trace: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out = A @ B`` with fp32 (int32 for int8) accumulation.

    ``a`` is stored ``[M, K]`` (``[K, M]`` with ``trans_a``), ``b`` is stored ``[K, N]``
    (``[N, K]`` with ``trans_b``). For int8 / fp8 operands ``scale_m`` (fp32 ``[M]``) and
    ``scale_n`` (fp32 ``[N]``) dequantise in the epilogue, ``bias`` (int32 ``[N]``, int8 only)
    is added to the accumulator first.
    """
    dev = cm.require_cuda(a, b, out, scale_m, scale_n, bias)
    if a.dtype != b.dtype:
        raise TypeError("A and B must share a dtype (got %s, %s)" % (a.dtype, b.dtype))
    m, n, k = cm.logical_shape(a, trans_a, b, trans_b)
    if out_dtype is None:
        if out is not None:
            out_dtype = out.dtype
        elif a.dtype == torch.int8:
            out_dtype = torch.int32 if (scale_m is None and scale_n is None) else torch.bfloat16
        elif a.dtype in (torch.float16, torch.bfloat16):
            out_dtype = a.dtype
        else:
            out_dtype = torch.bfloat16
    if out is None:
        out = torch.empty((m, n), dtype=out_dtype, device=dev)
    if out.shape != (m, n) or out.stride(-1) != 1 or out.dtype != out_dtype:
        raise ValueError("out must be a row-major [%d, %d] %s tensor" % (m, n, out_dtype))
    if a.dtype == torch.int8 and out_dtype == torch.float32 and scale_m is None and scale_n is None:
        raise ValueError("int8 GEMM without scales produces int32; pass out_dtype=torch.int32")
    if a.dtype != torch.int8 and out_dtype == torch.int32:
        raise ValueError("int32 output needs int8 operands")

    if tiling is None:
        from ..tiling.chooser import choose
        tiling = choose("matmul", m, n, k, 1, a.dtype)
    with torch.cuda.device(dev):
        oa = cm.as_operand(a, trans_a)
        ob = cm.as_operand(b, trans_b)
        args = N.OpArgs()
        args.mode = N.MODE_LOCAL
        args.in_fmt = cm.in_fmt(a.dtype)
        args.M, args.N, args.K = m, n, k
        args.trans_a, args.trans_b = int(oa.trans), int(ob.trans)
        args.a, args.lda = oa.ptr, oa.ld
        args.b, args.ldb = ob.ptr, ob.ld
        args.out, args.ldc, args.out_fmt = out.data_ptr(), out.stride(0), cm.out_fmt(out_dtype)
        args.partial_fmt = args.out_fmt
        cm.fill_tiling(args, tiling)
        args.rank, args.W = 0, 1
        for name, t, length, dt in (("scale_m", scale_m, m, torch.float32), ("scale_n", scale_n, n, torch.float32),
                                    ("bias", bias, n, torch.int32)):
            if t is not None:
                if t.dtype != dt or t.numel() != length or not t.is_contiguous():
                    raise ValueError("%s must be a contiguous %s tensor of %d elements" % (name, dt, length))
                setattr(args, name, t.data_ptr())
        args.status = cm.local_status(dev).data_ptr()
        if trace is not None:  # int64[16] device tensor: per-role cycle counters (see params.h)
            args.trace = trace.data_ptr()
        cm.launch(args, dev)
    return out

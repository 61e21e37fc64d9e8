"""``torch.ops.catcoc.*``: the single-device kernels as registered PyTorch operators.

The reference's GEMM template library ships a Torch extension whose operators take tensors and a
dtype string and allocate their own outputs
(3rdparty/catlass/examples/python_extension/src/bindings/torch_bindings.cpp:18-20,
src/wrapper/catlass_kernel_wrapper.cpp:31-290: ``basic_matmul(Tensor, Tensor, str) -> Tensor``,
``grouped_matmul(Tensor[], Tensor[], str, bool) -> Tensor[]``, ``optimized_matmul(...)``). The same
three signatures are registered here with ``torch.library`` on top of :mod:`.gemm` / :mod:`.blas`,
together with fake (meta) implementations so that the operators trace under ``torch.export`` /
``torch.compile`` graphs without running a kernel.

Importing this module registers the operators; ``mm_rs_with_catlass_b200`` does it on import.
"""
from __future__ import annotations

from typing import List

import torch

_DTYPES = {
    "float16": torch.float16, "half": torch.float16, "fp16": torch.float16,
    "bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
    "float32": torch.float32, "float": torch.float32, "fp32": torch.float32,
    "int32": torch.int32,
}


def _out_dtype(name: str) -> torch.dtype:
    try:
        return _DTYPES[name.lower()]
    except KeyError:
        raise ValueError("unknown output dtype %r (one of %s)" % (name, ", ".join(sorted(_DTYPES)))) from None


def _mn(a: torch.Tensor, b: torch.Tensor):
    if a.dim() != 2 or b.dim() != 2 or a.shape[1] != b.shape[0]:
        raise ValueError("expected A [M, K] and B [K, N], got %s and %s" % (tuple(a.shape), tuple(b.shape)))
    return a.shape[0], b.shape[1]


@torch.library.custom_op("catcoc::basic_matmul", mutates_args=())
def basic_matmul(a: torch.Tensor, b: torch.Tensor, out_dtype: str) -> torch.Tensor:
    """``A @ B``; a column-major view of either operand is read in place (stride-detected)."""
    from .gemm import matmul
    _mn(a, b)
    return matmul(a, b, out_dtype=_out_dtype(out_dtype))


@basic_matmul.register_fake
def _(a, b, out_dtype):
    m, n = _mn(a, b)
    return a.new_empty((m, n), dtype=_out_dtype(out_dtype))


@torch.library.custom_op("catcoc::optimized_matmul", mutates_args=())
def optimized_matmul(a: torch.Tensor, b: torch.Tensor, out_dtype: str) -> torch.Tensor:
    """``A @ B`` for operands of any pitch (padding prologue when TMA cannot address them)."""
    from .blas import optimized_matmul as impl
    _mn(a, b)
    return impl(a, b, out_dtype=_out_dtype(out_dtype))


@optimized_matmul.register_fake
def _(a, b, out_dtype):
    m, n = _mn(a, b)
    return a.new_empty((m, n), dtype=_out_dtype(out_dtype))


@torch.library.custom_op("catcoc::grouped_matmul", mutates_args=())
def grouped_matmul(a: List[torch.Tensor], b: List[torch.Tensor], out_dtype: str, split_k: bool) -> List[torch.Tensor]:
    """One product per list entry. With ``split_k`` false the groups share K and N and differ in
    M (``a[g]`` is ``[M_g, K]``, ``b[g]`` ``[K, N]``): the entries are stacked and run as ONE
    launch. With ``split_k`` the groups share M and N and differ in K (``a[g]`` ``[M, K_g]``,
    ``b[g]`` ``[K_g, N]``): one launch per group."""
    from . import blas
    from .gemm import matmul
    if len(a) != len(b) or not a:
        raise ValueError("grouped_matmul takes two non-empty lists of equal length")
    dt = _out_dtype(out_dtype)
    if split_k:
        return [matmul(x, y, out_dtype=dt) for x, y in zip(a, b)]
    k, n = b[0].shape
    if any(x.dim() != 2 or x.shape[1] != k for x in a) or any(tuple(y.shape) != (k, n) for y in b):
        raise ValueError("slice-M groups share K and N")
    sizes = [x.shape[0] for x in a]
    ends, acc = [], 0
    for s in sizes:
        acc += s
        ends.append(acc)
    stacked_a = torch.cat(a, dim=0)
    stacked_b = torch.stack(b, dim=0)
    umma_k = 32 // stacked_a.element_size()
    if k % umma_k:
        stacked_b = stacked_b.transpose(1, 2).contiguous()      # [G, N, K]: groups stack along N
        out = blas.grouped_matmul(stacked_a, stacked_b, ends, trans_b=True, out_dtype=dt)
    else:
        out = blas.grouped_matmul(stacked_a, stacked_b, ends, out_dtype=dt)
    return [t.clone() for t in out.split(sizes, dim=0)]


@grouped_matmul.register_fake
def _(a, b, out_dtype, split_k):
    dt = _out_dtype(out_dtype)
    return [x.new_empty((x.shape[0], y.shape[1]), dtype=dt) for x, y in zip(a, b)]

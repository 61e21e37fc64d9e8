"""The single-GPU kernel catalogue: everything the reference's GEMM template library offers
besides the plain product, on the same tcgen05 kernel.

=================================  =============================================================
reference kernel                    here
=================================  =============================================================
``KernelGemm`` (gemm.hpp)           :func:`gemm`  ``D = alpha * A @ B + beta * C`` (epilogue)
``MatmulBias`` (matmul_bias.hpp)    :func:`matmul_bias`  (fp32 bias row added in the epilogue)
``MatmulEpilogue`` (+X)             :func:`matmul_add`
``BatchedMatmul``                   :func:`batched_matmul`  (ONE launch: uniform group walk)
``GroupedMatmulSliceM``             :func:`grouped_matmul`  (ONE launch: ragged group walk, the
                                    group list stays on the device)
``GroupedMatmulSliceK``             :func:`grouped_matmul_slice_k`
``GroupedMatmulSliceMPerToken-``    :func:`grouped_quant_matmul`  (int8, per-token and per-group
``Dequant``                         per-channel scales in the epilogue)
``KernelGroupGemm``                 :func:`group_gemm`  (independent problems, one launch each)
``SplitkMatmul``                    :func:`splitk_matmul`  (K slices as groups of one launch into
                                    an fp32 workspace, then a reduction kernel)
``OptimizedMatmul`` / ``Padding-``  :func:`optimized_matmul`  (operands whose pitch TMA cannot
``Matmul``                          address are re-pitched by the pad kernel first)
``KernelGemvAiv`` / ``...Aic``      :func:`gemv`  ``z = alpha * op(A) x + beta * y``
=================================  =============================================================

File references: 3rdparty/catlass/include/catlass/gemm/kernel/{gemm,matmul_bias,matmul_epilogue,
batched_matmul,grouped_matmul_slice_m,grouped_matmul_slice_k,
grouped_matmul_slice_m_per_token_dequant,group_gemm,splitk_matmul,optimized_matmul,
padding_matmul}.hpp and 3rdparty/catlass/include/catlass/gemv/kernel/kernel_gemv_{aiv,aic}.hpp.

The *group walk* is what makes batched, grouped and split-K products one launch: the persistent
kernel's tile list is the concatenation of the groups' tile grids, and each tile carries the
offsets of its group inside the stacked operands (see ``FusedParams`` in ``params.h``).
"""
from __future__ import annotations

import ctypes as C
import math
from typing import List, Optional, Sequence, Union

import torch

from .. import _native as N
from ..tiling.config import TilingConfig
from . import _common as cm
from .gemm import matmul

GroupList = Union[torch.Tensor, Sequence[int]]


# ------------------------------------------------------------------------------------------
# affine epilogues
# ------------------------------------------------------------------------------------------
def gemm(a: torch.Tensor, b: torch.Tensor, c: Optional[torch.Tensor] = None, *, alpha: float = 1.0,
         beta: float = 0.0, trans_a: bool = False, trans_b: bool = False, out: Optional[torch.Tensor] = None,
         out_dtype: Optional[torch.dtype] = None, tiling: Optional[TilingConfig] = None) -> torch.Tensor:
    """``D = alpha * (A @ B) + beta * C``; ``out`` may be ``c`` itself (in-place update)."""
    if beta != 0.0 and c is None:
        raise ValueError("beta != 0 needs c")
    if out_dtype is None and out is None and c is not None:
        out_dtype = c.dtype
    return matmul(a, b, trans_a=trans_a, trans_b=trans_b, out=out, out_dtype=out_dtype, tiling=tiling,
                  alpha=alpha, beta=beta, c=c)


def matmul_bias(a: torch.Tensor, b: torch.Tensor, bias: torch.Tensor, *, trans_a: bool = False,
                trans_b: bool = False, out: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None,
                tiling: Optional[TilingConfig] = None) -> torch.Tensor:
    """``D = A @ B + bias[None, :]`` for floating-point operands (the bias joins in fp32, before
    the rounding to the output dtype). The int8 form with an int32 bias is ``matmul(bias=...)``."""
    if bias.dim() != 1:
        raise ValueError("bias must be a vector of N elements")
    return matmul(a, b, trans_a=trans_a, trans_b=trans_b, out=out, out_dtype=out_dtype, tiling=tiling,
                  bias_f32=bias.to(torch.float32).contiguous())


def matmul_add(a: torch.Tensor, b: torch.Tensor, x: torch.Tensor, *, trans_a: bool = False, trans_b: bool = False,
               out: Optional[torch.Tensor] = None, tiling: Optional[TilingConfig] = None) -> torch.Tensor:
    """``D = A @ B + X`` (element-wise one-source epilogue)."""
    return matmul(a, b, trans_a=trans_a, trans_b=trans_b, out=out, out_dtype=x.dtype, tiling=tiling, beta=1.0, c=x)


def optimized_matmul(a: torch.Tensor, b: torch.Tensor, **kw) -> torch.Tensor:
    """Plain product for operands of any stride: column-major views fold into the transpose
    flags, and a pitch or base address that TMA cannot address (not a multiple of 16 bytes) is
    fixed by one pass of the pad kernel before the GEMM."""
    return matmul(a, b, **kw)


# ------------------------------------------------------------------------------------------
# group walk: batched / grouped / split-K
# ------------------------------------------------------------------------------------------
def _umma_k(dtype: torch.dtype) -> int:
    return 32 // torch.empty((), dtype=dtype).element_size()


def _group_tiling(tiling: Optional[TilingConfig], rows_total: int, rows_per_group: float, n: int, k: int,
                  dtype: torch.dtype) -> TilingConfig:
    if tiling is not None:
        return tiling
    from ..tiling.chooser import heuristic
    t = heuristic("matmul", rows_total, n, k, 1, dtype)
    if t.cta_pair == 2 and (rows_per_group < 512 or rows_per_group % 256 != 0):
        t = t.with_(cta_pair=1)   # 256-row tiles would mostly be padding
    return t


def _ends_tensor(group_list: GroupList, device: torch.device) -> torch.Tensor:
    if isinstance(group_list, torch.Tensor):
        if group_list.dim() != 1:
            raise ValueError("group_list must be 1-D (cumulative row counts)")
        return group_list.to(device=device, dtype=torch.int32).contiguous()
    return torch.tensor(list(group_list), dtype=torch.int32, device=device)


def batched_matmul(a: torch.Tensor, b: torch.Tensor, *, trans_a: bool = False, trans_b: bool = False,
                   out: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None,
                   tiling: Optional[TilingConfig] = None) -> torch.Tensor:
    """``out[i] = A[i] @ B[i]`` for ``a`` stored ``[B, M, K]`` (``[B, K, M]`` with ``trans_a``) and
    ``b`` stored ``[B, K, N]`` (``[B, N, K]`` with ``trans_b``): one launch whose groups are the
    batch entries. Shapes whose group origins TMA cannot address run one launch per entry."""
    if a.dim() != 3 or b.dim() != 3 or a.shape[0] != b.shape[0]:
        raise ValueError("batched_matmul takes [B, ., .] operands with equal B")
    nb = a.shape[0]
    m, k = (a.shape[2], a.shape[1]) if trans_a else (a.shape[1], a.shape[2])
    kb, n = (b.shape[2], b.shape[1]) if trans_b else (b.shape[1], b.shape[2])
    if k != kb:
        raise ValueError("inner dimensions differ: %d vs %d" % (k, kb))
    dev = cm.require_cuda(a, b, out)
    if out_dtype is None:
        out_dtype = out.dtype if out is not None else (torch.int32 if a.dtype == torch.int8 else
                                                       a.dtype if a.dtype in (torch.float16, torch.bfloat16)
                                                       else torch.bfloat16)
    if out is None:
        out = torch.empty((nb, m, n), dtype=out_dtype, device=dev)
    if out.shape != (nb, m, n) or not out.is_contiguous():
        raise ValueError("out must be a contiguous [%d, %d, %d] tensor" % (nb, m, n))
    elt = a.element_size()
    # An operand whose entries are stacked along its K axis ([B, K, M] or [B, K, N]) must end each
    # entry on an MMA boundary; a transposed A also needs 16-byte aligned entry origins along M.
    stacked_k = trans_a or not trans_b
    walk_ok = (a.is_contiguous() and b.is_contiguous()
               and (not stacked_k or k % _umma_k(a.dtype) == 0)
               and (not trans_a or (m * elt) % 16 == 0))
    if nb == 1 or not walk_ok:
        for i in range(nb):
            matmul(a[i], b[i], trans_a=trans_a, trans_b=trans_b, out=out[i], tiling=tiling)
        return out
    group = dict(m=nb * m, n=n, k=k, num_groups=nb, group_rows=m)
    if trans_a:
        group.update(a_rows_total=m, a_k_total=nb * k, g_a_row_back=m, g_a_k=k)
    else:
        group.update(a_rows_total=nb * m, a_k_total=k)
    if trans_b:
        group.update(b_n_total=nb * n, b_k_total=k, g_b_row=n)
    else:
        group.update(b_n_total=n, b_k_total=nb * k, g_b_k=k)
    a2 = a.reshape(nb * a.shape[1], a.shape[2])
    b2 = b.reshape(nb * b.shape[1], b.shape[2])
    matmul(a2, b2, trans_a=trans_a, trans_b=trans_b, out=out.view(nb * m, n),
           tiling=_group_tiling(tiling, nb * m, m, n, k, a.dtype), _group=group)
    return out


def _grouped_launch(a, b, ends, trans_b, out, out_dtype, tiling, **epilogue):
    g = b.shape[0]
    m_total, k = a.shape
    kb, n = (b.shape[2], b.shape[1]) if trans_b else (b.shape[1], b.shape[2])
    if k != kb:
        raise ValueError("inner dimensions differ: A gives K=%d, B gives K=%d" % (k, kb))
    if ends.numel() != g:
        raise ValueError("group_list has %d entries for %d groups" % (ends.numel(), g))
    if not trans_b and k % _umma_k(a.dtype) != 0:
        raise ValueError("B stored [G, K, N] needs K %% %d == 0 (groups are stacked along K); store it [G, N, K] "
                         "and pass trans_b=True otherwise" % _umma_k(a.dtype))
    group = dict(m=m_total, n=n, k=k, num_groups=g, group_ends=ends, a_rows_total=m_total, a_k_total=k)
    if trans_b:
        group.update(b_n_total=g * n, b_k_total=k, g_b_row=n)
    else:
        group.update(b_n_total=n, b_k_total=g * k, g_b_k=k)
    if epilogue.get("scale_n") is not None or epilogue.get("bias_f32") is not None or epilogue.get("bias") is not None:
        group["g_nvec"] = n
    b2 = b.contiguous().reshape(g * b.shape[1], b.shape[2])
    a2 = a if a.is_contiguous() else a.contiguous()
    return matmul(a2, b2, trans_b=trans_b, out=out, out_dtype=out_dtype,
                  tiling=_group_tiling(tiling, m_total, m_total / max(1, g), n, k, a.dtype), _group=group, **epilogue)


def grouped_matmul(a: torch.Tensor, b: torch.Tensor, group_list: GroupList, *, trans_b: bool = False,
                   out: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None,
                   tiling: Optional[TilingConfig] = None) -> torch.Tensor:
    """Grouped product sliced along M (the MoE expert GEMM): ``a`` is ``[sum M_g, K]`` with the
    groups' rows stacked, ``b`` is ``[G, K, N]`` (``[G, N, K]`` with ``trans_b``), ``group_list``
    holds the cumulative row counts (``group_list[g]`` = one past the last row of group ``g``).
    ``out[rows of g] = a[rows of g] @ b[g]``. One launch; ``group_list`` may live on the device
    (it is read by the kernel, never by the host). Rows past ``group_list[-1]`` are left
    untouched."""
    if a.dim() != 2 or b.dim() != 3:
        raise ValueError("grouped_matmul takes a [sum M, K] and b [G, ., .]")
    dev = cm.require_cuda(a, b, out)
    return _grouped_launch(a, b, _ends_tensor(group_list, dev), trans_b, out, out_dtype, tiling)


def grouped_quant_matmul(x1: torch.Tensor, x2: torch.Tensor, scale_per_token: torch.Tensor,
                         scale_per_channel: torch.Tensor, group_list: GroupList, *, trans_b: bool = False,
                         out: Optional[torch.Tensor] = None, out_dtype: torch.dtype = torch.bfloat16,
                         tiling: Optional[TilingConfig] = None) -> torch.Tensor:
    """int8 grouped product with the dequantisation in the epilogue:
    ``out[r, :] = cast(float(x1[r] @ x2[g(r)]) * scale_per_token[r] * scale_per_channel[g(r), :])``
    with ``scale_per_token`` fp32 ``[sum M]`` and ``scale_per_channel`` fp32 ``[G, N]``."""
    if x1.dtype != torch.int8 or x2.dtype != torch.int8:
        raise TypeError("grouped_quant_matmul takes int8 operands")
    dev = cm.require_cuda(x1, x2, scale_per_token, scale_per_channel, out)
    return _grouped_launch(x1, x2, _ends_tensor(group_list, dev), trans_b, out, out_dtype, tiling,
                           scale_m=scale_per_token.contiguous(), scale_n=scale_per_channel.contiguous().view(-1))


def grouped_matmul_slice_k(a: torch.Tensor, b: torch.Tensor, group_list: Sequence[int], *,
                           out_dtype: Optional[torch.dtype] = None,
                           tiling: Optional[TilingConfig] = None) -> torch.Tensor:
    """Grouped product sliced along K (the MoE weight gradient): ``a`` is stored ``[K_total, M]``
    (tokens x features, read as its transpose), ``b`` ``[K_total, N]``, ``group_list`` the
    cumulative K counts on the host. Returns ``[G, M, N]`` with
    ``out[g] = a[k range of g].T @ b[k range of g]``; an empty group gives zeros. The K ranges are
    ragged, so each group is its own launch on views of the operands."""
    if a.dim() != 2 or b.dim() != 2 or a.shape[0] != b.shape[0]:
        raise ValueError("grouped_matmul_slice_k takes a [K_total, M] and b [K_total, N]")
    if isinstance(group_list, torch.Tensor):
        group_list = group_list.tolist()   # the ranges steer host-side views
    dev = cm.require_cuda(a, b)
    m, n = a.shape[1], b.shape[1]
    if out_dtype is None:
        out_dtype = a.dtype if a.dtype in (torch.float16, torch.bfloat16) else torch.bfloat16
    out = torch.empty((len(group_list), m, n), dtype=out_dtype, device=dev)
    begin = 0
    for g, end in enumerate(group_list):
        if end <= begin:
            out[g].zero_()
        else:
            matmul(a[begin:end], b[begin:end], trans_a=True, out=out[g], tiling=tiling)
        begin = max(begin, end)
    return out


def group_gemm(problems: Sequence[dict], *, tiling: Optional[TilingConfig] = None) -> List[torch.Tensor]:
    """Independent ``D_i = alpha_i * A_i @ B_i + beta_i * C_i`` problems of unrelated shapes, queued
    back to back on the current stream. Each problem is a dict with ``a``, ``b`` and optionally
    ``c``, ``alpha``, ``beta``, ``trans_a``, ``trans_b``, ``out``."""
    outs = []
    for pr in problems:
        outs.append(gemm(pr["a"], pr["b"], pr.get("c"), alpha=pr.get("alpha", 1.0), beta=pr.get("beta", 0.0),
                         trans_a=pr.get("trans_a", False), trans_b=pr.get("trans_b", False), out=pr.get("out"),
                         tiling=tiling))
    return outs


_NUM_SMS = 148


def pick_split_k(m: int, n: int, k: int, elt: int) -> int:
    """Number of K slices that fills the GPU: as many as keep one 128 x 128 tile per SM busy,
    each slice holding at least four pipeline stages (a stage is 256 bytes of K)."""
    stage_k = 256 // elt
    tiles = math.ceil(m / 128) * math.ceil(n / 128)
    want = max(1, _NUM_SMS // max(1, tiles))
    most = max(1, k // (4 * stage_k))
    return max(1, min(want, most, 32))


def slice_k(k: int, split_k: int, elt: int):
    """K per slice (whole pipeline stages of 256 bytes) and the number of slices that leaves."""
    stage_k = 256 // elt
    ks = math.ceil(math.ceil(k / max(1, split_k)) / stage_k) * stage_k
    return ks, math.ceil(k / ks)


def splitk_plan(m: int, n: int, k: int, elt: int):
    """``(split_k, bn)`` for a product with few output tiles: the tile width and slice count that
    fill the SMs with the fewest bytes per CTA. A CTA streams ``(128 + bn) * K / split_k`` operand
    elements whatever M is, and a CTA's intake (not HBM) bounds such a product, so wide tiles cut
    into more slices beat narrow ones: the A rows are re-read once per tile column."""
    best = None
    for bn in (256, 128):
        if n < bn and bn > 128:
            continue
        tiles = math.ceil(m / 128) * math.ceil(n / bn)
        want = max(1, _NUM_SMS // max(1, tiles))
        most = max(1, k // (4 * (256 // elt)))
        s = max(1, min(want, most, 32))
        ks, s = slice_k(k, s, elt)
        waves = math.ceil(tiles * s / _NUM_SMS)
        cost = waves * (128 + bn) * ks
        if best is None or cost < best[0]:
            best = (cost, s, bn)
    return best[1], best[2]


def splitk_partials(a: torch.Tensor, b: torch.Tensor, *, split_k: int, trans_a: bool = False, trans_b: bool = False,
                    tiling: Optional[TilingConfig] = None, part: Optional[torch.Tensor] = None,
                    _args_out: Optional[list] = None):
    """The first half of a split-K product: the K slices run as the groups of ONE launch, slice
    ``i`` writing its fp32 partial ``[M, N]`` to rows ``[i * M, (i + 1) * M)`` of the returned
    workspace. Returns ``(part, slices)``."""
    dev = cm.require_cuda(a, b, part)
    m, n, k = cm.logical_shape(a, trans_a, b, trans_b)
    elt = a.element_size()
    ks, s = slice_k(k, split_k, elt)
    if trans_a and (m * elt) % 16 != 0:
        a, trans_a = a.t().contiguous(), False   # slice origins along M must stay TMA-addressable
    if part is None:
        part = torch.empty((s * m, n), dtype=torch.float32, device=dev)
    group = dict(m=s * m, n=n, k=ks, num_groups=s, group_rows=m, a_rows_total=m, a_k_total=k, b_n_total=n,
                 b_k_total=k, g_a_row_back=m, g_a_k=ks, g_b_k=ks)
    if tiling is None:
        from ..tiling.chooser import heuristic
        tiling = heuristic("matmul", s * m, n, ks, 1, a.dtype).with_(cta_pair=1)
        if m % 128 != 0 and tiling.bn > 128:
            tiling = tiling.with_(bn=128)
    matmul(a, b, trans_a=trans_a, trans_b=trans_b, out=part, out_dtype=torch.float32, tiling=tiling, _group=group,
           _args_out=_args_out)
    return part, s


def splitk_matmul(a: torch.Tensor, b: torch.Tensor, *, split_k: Optional[int] = None, trans_a: bool = False,
                  trans_b: bool = False, out: Optional[torch.Tensor] = None,
                  out_dtype: Optional[torch.dtype] = None, alpha: float = 1.0, beta: float = 0.0,
                  c: Optional[torch.Tensor] = None, bias_f32: Optional[torch.Tensor] = None,
                  tiling: Optional[TilingConfig] = None) -> torch.Tensor:
    """``A @ B`` for shapes with few output tiles and a long K: the K range is cut into
    ``split_k`` slices that run as the groups of ONE launch, each writing an fp32 partial
    ``[M, N]`` into a workspace; a second, bandwidth-bound kernel sums the slices and applies
    ``alpha / beta / bias`` and the rounding. fp16 / bf16 / fp8 operands (floating accumulators)."""
    dev = cm.require_cuda(a, b, out, c, bias_f32)
    if a.dtype == torch.int8:
        raise TypeError("splitk_matmul takes floating-point operands (an int8 product reduces in int32)")
    m, n, k = cm.logical_shape(a, trans_a, b, trans_b)
    elt = a.element_size()
    if out_dtype is None:
        out_dtype = out.dtype if out is not None else (a.dtype if a.dtype in (torch.float16, torch.bfloat16)
                                                       else torch.bfloat16)
    if split_k is None and tiling is None:
        # tile width and slice count together: the fewest operand bytes per CTA with every SM busy
        s, bn = splitk_plan(m, n, k, elt)
        if m % 128 == 0 or bn <= 128:
            tiling = TilingConfig(bn=bn, cta_pair=1)
    else:
        s = split_k if split_k is not None else pick_split_k(m, n, k, elt)
    if slice_k(k, s, elt)[1] <= 1:
        return matmul(a, b, trans_a=trans_a, trans_b=trans_b, out=out, out_dtype=out_dtype, tiling=tiling,
                      alpha=alpha, beta=beta, c=c, bias_f32=bias_f32)
    if out is None:
        out = torch.empty((m, n), dtype=out_dtype, device=dev)
    if out.shape != (m, n) or out.stride(-1) != 1 or out.dtype not in (torch.float16, torch.bfloat16, torch.float32):
        raise ValueError("out must be a row-major floating-point [%d, %d] tensor" % (m, n))
    if c is not None and (c.shape != (m, n) or c.dtype != out.dtype or c.stride(-1) != 1):
        raise ValueError("c must match the output's shape and dtype")
    part, s = splitk_partials(a, b, split_k=s, trans_a=trans_a, trans_b=trans_b, tiling=tiling)
    with torch.cuda.device(dev):
        stream = torch.cuda.current_stream(dev).cuda_stream
        bias_ptr = None
        if bias_f32 is not None:
            if bias_f32.dtype != torch.float32 or bias_f32.numel() != n or not bias_f32.is_contiguous():
                raise ValueError("bias_f32 must be a contiguous fp32 tensor of %d elements" % n)
            bias_ptr = bias_f32.data_ptr()
        N.check(N.lib().catcoc_splitk_reduce(part.data_ptr(), s, m * n, m, n, out.data_ptr(), out.stride(0),
                                             cm.out_fmt(out.dtype), float(alpha), float(beta),
                                             c.data_ptr() if (c is not None and beta != 0.0) else None,
                                             c.stride(0) if c is not None else n, bias_ptr, C.c_void_p(stream)))
    return out


def gemv(a: torch.Tensor, x: torch.Tensor, y: Optional[torch.Tensor] = None, *, alpha: float = 1.0,
         beta: float = 0.0, trans: bool = False, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``z = alpha * op(A) @ x + beta * y`` with ``op(A) = A`` (``[M, N]`` row-major) or ``A.T``
    when ``trans``. fp16 / bf16 / fp32, fp32 accumulation. The product is HBM-bound (every
    element of A is used once), so it runs on plain SIMT kernels that stream A with 16-byte loads
    rather than on the tensor cores."""
    if a.dim() != 2 or x.dim() != 1:
        raise ValueError("gemv takes a matrix and a vector")
    dev = cm.require_cuda(a, x, y, out)
    if a.dtype not in (torch.float16, torch.bfloat16, torch.float32) or x.dtype != a.dtype:
        raise TypeError("gemv takes fp16 / bf16 / fp32 operands of one dtype")
    if a.stride(-1) != 1:
        if a.stride(0) == 1:
            a, trans = a.t(), not trans     # a column-major view is the transposed product
        else:
            a = a.contiguous()
    rows, cols = a.shape
    n_in, n_out = (rows, cols) if trans else (cols, rows)
    if x.numel() != n_in:
        raise ValueError("x must have %d elements" % n_in)
    if beta != 0.0 and (y is None or y.numel() != n_out or y.dtype != a.dtype):
        raise ValueError("beta != 0 needs y with %d elements of dtype %s" % (n_out, a.dtype))
    if out is None:
        out = torch.empty((n_out,), dtype=a.dtype, device=dev)
    if out.numel() != n_out or not out.is_contiguous() or out.dtype != a.dtype:
        raise ValueError("out must be a contiguous vector of %d elements" % n_out)
    x = x.contiguous()
    yin = y.contiguous() if (y is not None and beta != 0.0) else None
    with torch.cuda.device(dev):
        lib = N.lib()
        ws = None
        nws = lib.catcoc_gemv_workspace_floats(rows, cols, int(trans))
        if nws > 0:
            ws = torch.empty((nws,), dtype=torch.float32, device=dev)
        stream = torch.cuda.current_stream(dev).cuda_stream
        N.check(lib.catcoc_gemv(a.data_ptr(), a.stride(0), cm.out_fmt(a.dtype), rows, cols, int(trans), x.data_ptr(),
                                out.data_ptr(), yin.data_ptr() if yin is not None else None, float(alpha),
                                float(beta), ws.data_ptr() if ws is not None else None, C.c_void_p(stream)))
    return out

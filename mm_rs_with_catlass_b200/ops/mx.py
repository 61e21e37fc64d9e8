"""Block-scaled fp8 ("mxf8"): e4m3 / e5m2 values with one UE8M0 scale (a power of two) per 32
consecutive K-elements, multiplied by ``tcgen05.mma.kind::mxf8f6f4.block_scale`` with the scale
factors staged in TMEM. The reference has no such variant; it sits next to the int8 op as the
second quantised row-parallel linear.

Layouts: A is stored ``[M, K]`` and B ``[N, K]`` (both K-contiguous; a weight stored ``[K, N]``
is transposed once when it is quantised). Scales come as ``uint8 [rows, K / 32]`` (biased
exponent, value ``2 ** (s - 127)``) and are repacked by :func:`pack_scales` into the 512-byte
blocks the tensor core reads (128 rows x 4 K-blocks, row r at ``(r % 32) * 16 + (r // 32) * 4``).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .. import _native as N
from ..parallel.shmem import ShmemContext
from ..tiling.config import TilingConfig
from . import _common as cm
from . import fused as _fused

BLOCK = 32
_FP8_MAX = {"e4m3": 448.0, "e5m2": 57344.0}


def quantize_mxf8(x: torch.Tensor, fmt: str = "e4m3") -> Tuple[torch.Tensor, torch.Tensor]:
    """``x [rows, K]`` (K % 32 == 0) -> (fp8 values ``[rows, K]``, UE8M0 scales ``uint8 [rows, K/32]``).
    The scale of a block is the smallest power of two that brings its largest magnitude into the
    fp8 range."""
    rows, k = x.shape
    if k % BLOCK:
        raise ValueError("K must be a multiple of 32 for block scaling (K=%d)" % k)
    xb = x.float().reshape(rows, k // BLOCK, BLOCK)
    amax = xb.abs().amax(dim=-1)
    exp = torch.ceil(torch.log2(torch.clamp(amax, min=2.0 ** -126) / _FP8_MAX[fmt]))
    exp = torch.clamp(exp, -127, 127)
    exp = torch.where(amax > 0, exp, torch.zeros_like(exp))
    q = xb / torch.exp2(exp)[..., None]
    dt = torch.float8_e4m3fn if fmt == "e4m3" else torch.float8_e5m2
    return q.reshape(rows, k).to(dt), (exp + 127).to(torch.uint8)


def dequantize_mxf8(q: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    rows, k = q.shape
    s = torch.exp2(scales.float() - 127.0)
    return (q.float().reshape(rows, k // BLOCK, BLOCK) * s[..., None]).reshape(rows, k)


def pack_scales(scales: torch.Tensor) -> torch.Tensor:
    """``uint8 [rows, K/32]`` -> ``uint8 [ceil(rows/128), ceil(K/128), 512]`` in the tensor-core block
    layout; rows and K-blocks are padded with the neutral scale 127 (= 1.0)."""
    rows, kb = scales.shape
    rt, kt = (rows + 127) // 128, (kb + 3) // 4
    pad = torch.full((rt * 128, kt * 4), 127, dtype=torch.uint8, device=scales.device)
    pad[:rows, :kb] = scales
    # row = rt*128 + j*32 + l  ->  [rt, kt, l, j, s]
    v = pad.view(rt, 4, 32, kt, 4).permute(0, 3, 2, 1, 4).contiguous()
    return v.view(rt, kt, 512)


def _fmt_of(t: torch.Tensor) -> int:
    if t.dtype == torch.float8_e4m3fn:
        return N.IN_MXE4M3
    if t.dtype == torch.float8_e5m2:
        return N.IN_MXE5M2
    raise TypeError("block-scaled operands must be float8_e4m3fn or float8_e5m2 (got %s)" % t.dtype)


def _check(a_q, sfa_packed, b_q, sfb_packed):
    if a_q.dtype != b_q.dtype:
        raise TypeError("A and B must share an fp8 format")
    m, k = a_q.shape
    n, kb = b_q.shape
    if k != kb:
        raise ValueError("inner dimensions differ: A gives K=%d, B gives K=%d" % (k, kb))
    if k % 16:
        raise ValueError("K must be a multiple of 16")
    kt = (k + 127) // 128
    for name, sf, rows in (("sfa", sfa_packed, m), ("sfb", sfb_packed, n)):
        want = ((rows + 127) // 128, kt, 512)
        if sf.dtype != torch.uint8 or tuple(sf.shape) != want or not sf.is_contiguous():
            raise ValueError("%s must be a contiguous uint8 tensor of shape %s from pack_scales()" % (name, want))
    return m, n, k, kt


def _fill(args, a_q, sfa_packed, b_q, sfb_packed, m, n, k, kt):
    args.in_fmt = _fmt_of(a_q)
    args.M, args.N, args.K = m, n, k
    args.trans_a, args.trans_b = 0, 1
    args.a, args.lda = a_q.data_ptr(), a_q.stride(0)
    args.b, args.ldb = b_q.data_ptr(), b_q.stride(0)
    args.sfa, args.sfb, args.sf_k_blocks = sfa_packed.data_ptr(), sfb_packed.data_ptr(), kt


def mxf8_matmul(a_q: torch.Tensor, sfa_packed: torch.Tensor, b_q: torch.Tensor, sfb_packed: torch.Tensor, *,
                out_dtype: torch.dtype = torch.bfloat16, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out[M, N] = dequant(A) @ dequant(B).T`` with fp32 accumulation on one GPU."""
    dev = cm.require_cuda(a_q, b_q, sfa_packed, sfb_packed, out)
    a_q, b_q = a_q.contiguous(), b_q.contiguous()
    m, n, k, kt = _check(a_q, sfa_packed, b_q, sfb_packed)
    if out is None:
        out = torch.empty((m, n), dtype=out_dtype, device=dev)
    with torch.cuda.device(dev):
        args = N.OpArgs()
        args.mode = N.MODE_LOCAL
        _fill(args, a_q, sfa_packed, b_q, sfb_packed, m, n, k, kt)
        args.out, args.ldc, args.out_fmt = out.data_ptr(), out.stride(0), cm.out_fmt(out.dtype)
        args.partial_fmt = args.out_fmt
        args.rank, args.W = 0, 1
        args.status = cm.local_status(dev).data_ptr()
        cm.launch(args, dev)
    return out


def mxf8_matmul_reduce_scatter(a_q: torch.Tensor, sfa_packed: torch.Tensor, b_q: torch.Tensor,
                               sfb_packed: torch.Tensor, *, out_dtype: torch.dtype = torch.bfloat16,
                               out: Optional[torch.Tensor] = None, tiling: Optional[TilingConfig] = None,
                               ctx: Optional[ShmemContext] = None) -> torch.Tensor:
    """Row-parallel linear on block-scaled fp8 operands with a fused reduce-scatter.

    Per rank ``a_q [M, K_r]``, ``b_q [N, K_r]`` and their packed scales; returns this rank's rows
    ``[M/W, N]`` of ``sum_r dequant(A_r) @ dequant(B_r).T``. Partial tiles cross NVLink as
    ``out_dtype`` (fp32 with ``tiling.fp32_partials``) and are summed in fp32 on the owner."""
    dev = cm.require_cuda(a_q, b_q, sfa_packed, sfb_packed, out)
    ctx = _fused._ctx(ctx)
    if ctx.world == 1:
        return mxf8_matmul(a_q, sfa_packed, b_q, sfb_packed, out_dtype=out_dtype, out=out)
    a_q, b_q = a_q.contiguous(), b_q.contiguous()
    m, n, k, kt = _check(a_q, sfa_packed, b_q, sfb_packed)
    if m % ctx.world:
        raise ValueError("mxf8_matmul_reduce_scatter needs M %% world == 0 (M=%d, world=%d)" % (m, ctx.world))
    if out_dtype not in (torch.float16, torch.bfloat16):
        raise TypeError("out_dtype must be fp16 or bf16")
    rows = m // ctx.world
    if rows % 128:
        # a scale block covers 128 consecutive rows starting at a multiple of 128; a rank's row
        # range must start on such a boundary for its tiles to line up with the blocks
        raise ValueError("mxf8_matmul_reduce_scatter needs M / world to be a multiple of 128 (got %d)" % rows)
    if out is None:
        out = torch.empty((rows, n), dtype=out_dtype, device=dev)
    t = (tiling or TilingConfig()).with_(bn=128, cta_pair=1)
    with torch.cuda.device(dev):
        args = N.OpArgs()
        args.mode = N.MODE_RS
        _fill(args, a_q, sfa_packed, b_q, sfb_packed, m, n, k, kt)
        cm.fill_tiling(args, t)
        args.rank, args.W = ctx.rank, ctx.world
        args.epoch_ptr = ctx.launch_state.data_ptr()
        args.cta_counter = ctx.launch_state.data_ptr() + 4
        args.status = ctx.status.data_ptr()
        args.out, args.ldc, args.out_fmt = out.data_ptr(), out.stride(0), cm.out_fmt(out_dtype)
        _fused._attach_stage(ctx, args, m, n, 0, t, N.FMT_F32 if t.fp32_partials else cm.out_fmt(out_dtype))
        _fused._launched(ctx, args)
    return out

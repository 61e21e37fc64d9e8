"""Flash attention forward on the library's own tcgen05 kernel (``csrc/kernels/flash_attn.cu``).

One CTA per 256 query rows (two tiles of 128) of one (batch, head): ``S = Q K^T`` and
``O += P V`` run on the tensor cores with all four accumulators in TMEM. The softmax warps of a
tile read its scores with ``tcgen05.ld``, keep the row maximum and sum, write ``P`` back over the
scores (``tcgen05.st``) where the second product reads it as its TMEM operand, and rescale ``O``
in TMEM only when the maximum moved by more than 2^8 (lazy online softmax). While one tile is in
its softmax the tensor core runs the other tile's products. K and V stream through one TMA ring.

The reference carries the same computation as vendored template kernels for its own
accelerator (3rdparty/catlass/include/catlass/gemm/block/block_mmad_fa_qk.hpp and
block_mmad_fa_pv.hpp with the block_epilogue_fa_softmax.hpp / block_epilogue_fa_rescale_o.hpp
epilogues; the MLA decode example 3rdparty/catlass/examples/19_mla/mla_kernel.cpp is the same
recurrence with a shared latent K / V).
"""
from __future__ import annotations

import ctypes as C
import math
from typing import Optional

import torch

from .. import _native as N
from . import _common as cm


def flash_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, causal: bool = False,
                    scale: Optional[float] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``softmax(scale * q @ k^T [+ causal mask]) @ v`` per (batch, head).

    ``q`` is ``[B, Hq, Sq, D]``, ``k`` and ``v`` are ``[B, Hk, Sk, D]`` (fp16 or bf16, ``D`` 64 or
    128, ``Hq`` a multiple of ``Hk``: grouped-query heads share a key / value head). With
    ``causal`` key ``j`` is visible to query ``i`` when ``j <= i + (Sk - Sq)`` (the diagonal ends
    in the bottom-right corner, as for a decode step over a cache). Scores are accumulated in
    fp32, probabilities are rounded to the operand dtype for the second product, the output is
    rounded once at the end. Returns ``[B, Hq, Sq, D]``.
    """
    dev = cm.require_cuda(q, k, v, out)
    if q.dim() != 4 or k.dim() != 4 or v.dim() != 4:
        raise ValueError("flash_attention takes [B, H, S, D] tensors")
    if q.dtype not in (torch.float16, torch.bfloat16) or k.dtype != q.dtype or v.dtype != q.dtype:
        raise TypeError("flash_attention takes fp16 / bf16 operands of one dtype")
    b, hq, sq, d = q.shape
    if k.shape != v.shape or k.shape[0] != b or k.shape[3] != d:
        raise ValueError("k and v must be [B, Hk, Sk, D] with the batch and head dimension of q")
    hk, sk = k.shape[1], k.shape[2]
    if hq % hk:
        raise ValueError("%d query heads do not divide over %d key / value heads" % (hq, hk))
    if d not in (64, 128):
        raise ValueError("head dimension %d: 64 and 128 are built" % d)
    if causal and sk < sq:
        raise ValueError("causal attention needs Sk >= Sq")
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    if out is None:
        out = torch.empty_like(q)
    if out.shape != q.shape or out.dtype != q.dtype or not out.is_contiguous():
        raise ValueError("out must be a contiguous tensor shaped like q")
    if scale is None:
        scale = 1.0 / math.sqrt(d)
    if not scale > 0.0:
        raise ValueError("the softmax scale must be positive")
    with torch.cuda.device(dev):
        stream = torch.cuda.current_stream(dev).cuda_stream
        N.check(N.lib().catcoc_flash_attention(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), b, hq, hk, sq,
                                               sk, d, cm.out_fmt(q.dtype), int(causal), float(scale),
                                               cm.local_status(dev).data_ptr(), cm.default_timeout_ns(),
                                               C.c_void_p(stream)))
    return out


def attention_reference(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, causal: bool = False,
                        scale: Optional[float] = None) -> torch.Tensor:
    """The same function in plain fp32 PyTorch (golden for the tests, any device)."""
    b, hq, sq, d = q.shape
    hk, sk = k.shape[1], k.shape[2]
    scale = 1.0 / math.sqrt(d) if scale is None else scale
    kf = k.float().repeat_interleave(hq // hk, dim=1)
    vf = v.float().repeat_interleave(hq // hk, dim=1)
    s = torch.matmul(q.float(), kf.transpose(-1, -2)) * scale
    if causal:
        i = torch.arange(sq, device=q.device)[:, None]
        j = torch.arange(sk, device=q.device)[None, :]
        s = s.masked_fill(j > i + (sk - sq), float("-inf"))
    return torch.matmul(torch.softmax(s, dim=-1), vf)

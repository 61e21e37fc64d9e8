"""Multi-head latent attention, decode step over a paged latent cache (``csrc/kernels/mla_decode.cu``).

All query heads share one key / value stream: a 512-wide latent that is key and value at once,
plus a 64-wide rotary part that only the scores see. ``q_nope`` has already been multiplied by
the key up-projection (the "absorbed" form), so the kernel is attention with 576-wide keys and
512-wide values over a cache of 128-key pages. One CTA owns up to 128 query rows (new tokens x
heads of one sequence), one half of the output columns and one slice of the sequence; the slices
are merged by a second small kernel (flash decoding).

The reference carries the same computation as 3rdparty/catlass/examples/19_mla/mla_kernel.cpp;
argument layouts and the golden follow its gen_data.py.
"""
from __future__ import annotations

import ctypes as C
import math
from typing import Optional

import torch

from .. import _native as N
from . import _common as cm

LATENT = 512
ROPE = 64
PAGE = 128

_workspaces: dict = {}


def _pick_splits(batch: int, rows_per_item: int, max_pages: int, sms: int = 148) -> int:
    """Slices per sequence. One CTA fits an SM, so the grid runs in waves of ``sms`` CTAs and a
    slice count is judged by waves x steps per CTA (a few steps of fixed cost for the Q load, the
    pipeline fill and the epilogue included); never more slices than 128-key pages."""
    base = 2 * batch * ((rows_per_item + 127) // 128)          # CTAs with one slice
    steps = 4 * max_pages                                       # 32-key steps of the longest sequence
    best, best_cost = 1, None
    for s in range(1, int(min(max_pages, 64)) + 1):
        waves = (base * s + sms - 1) // sms
        cost = waves * ((steps + s - 1) // s + 6)
        if best_cost is None or cost < best_cost:
            best, best_cost = s, cost
    return best


def mla_decode(q_nope: torch.Tensor, q_rope: torch.Tensor, ckv_cache: torch.Tensor, krope_cache: torch.Tensor,
               block_table: torch.Tensor, kv_lens: torch.Tensor, *, q_len: int = 1, causal: bool = False,
               scale: Optional[float] = None, splits: Optional[int] = None,
               out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``softmax(scale * [q_nope, q_rope] @ [ckv, krope]^T) @ ckv`` per sequence and head.

    ``q_nope`` ``[T, H, 512]`` and ``q_rope`` ``[T, H, 64]`` hold ``q_len`` (1 to 4) new tokens for each of the
    ``B = T / q_len`` sequences; ``ckv_cache`` ``[pages, 128, 512]`` and ``krope_cache`` ``[pages, 128, 64]`` are the
    paged caches (a singleton head dimension is accepted: ``[pages, 128, 1, 512]``); ``block_table`` ``[B, max_pages]``
    (int32) names the pages of every sequence and ``kv_lens`` ``[B]`` (int32) its length including the new tokens.
    With ``causal`` new token ``t`` does not see the new tokens behind it. The cache must hold finite values in
    every row of a page that is in use (a probability of zero times a NaN is a NaN). Returns ``[T, H, 512]``.
    """
    dev = cm.require_cuda(q_nope, q_rope, ckv_cache, krope_cache, block_table, kv_lens, out)
    if ckv_cache.dim() == 4 and ckv_cache.shape[2] == 1:
        ckv_cache = ckv_cache.squeeze(2)
    if krope_cache.dim() == 4 and krope_cache.shape[2] == 1:
        krope_cache = krope_cache.squeeze(2)
    if q_nope.dim() != 3 or q_rope.dim() != 3 or q_nope.shape[2] != LATENT or q_rope.shape[2] != ROPE:
        raise ValueError("mla_decode takes q_nope [T, H, 512] and q_rope [T, H, 64]")
    if q_rope.shape[:2] != q_nope.shape[:2]:
        raise ValueError("q_nope and q_rope must agree in tokens and heads")
    if ckv_cache.dim() != 3 or tuple(ckv_cache.shape[1:]) != (PAGE, LATENT):
        raise ValueError("the latent cache must be [pages, 128, 512]")
    if krope_cache.dim() != 3 or tuple(krope_cache.shape[1:]) != (PAGE, ROPE) or krope_cache.shape[0] != ckv_cache.shape[0]:
        raise ValueError("the rotary cache must be [pages, 128, 64] with the latent cache's page count")
    dt = q_nope.dtype
    if dt not in (torch.float16, torch.bfloat16) or any(t.dtype != dt for t in (q_rope, ckv_cache, krope_cache)):
        raise TypeError("mla_decode takes fp16 / bf16 operands of one dtype")
    if block_table.dtype != torch.int32 or kv_lens.dtype != torch.int32 or block_table.dim() != 2 or kv_lens.dim() != 1:
        raise TypeError("block_table [B, max_pages] and kv_lens [B] must be int32")
    tokens, heads = q_nope.shape[0], q_nope.shape[1]
    if not 1 <= q_len <= 4 or tokens % q_len:
        raise ValueError("q_len must be 1 to 4 and divide the number of tokens")
    batch = tokens // q_len
    if block_table.shape[0] != batch or kv_lens.shape[0] != batch:
        raise ValueError("block_table and kv_lens must have one row per sequence (%d)" % batch)
    if scale is None:
        scale = 1.0 / math.sqrt(LATENT + ROPE)
    if not scale > 0.0:
        raise ValueError("the softmax scale must be positive")
    q_nope, q_rope = q_nope.contiguous(), q_rope.contiguous()
    ckv_cache, krope_cache = ckv_cache.contiguous(), krope_cache.contiguous()
    block_table, kv_lens = block_table.contiguous(), kv_lens.contiguous()
    if out is None:
        out = torch.empty_like(q_nope)
    if out.shape != q_nope.shape or out.dtype != dt or not out.is_contiguous():
        raise ValueError("out must be a contiguous tensor shaped like q_nope")
    max_pages = block_table.shape[1]
    if splits is None:
        splits = _pick_splits(batch, q_len * heads, max_pages)
    lib = N.lib()
    need = int(lib.catcoc_mla_workspace_bytes(batch, q_len, heads, int(splits)))
    ws = None
    if need:
        ws = _workspaces.get(dev.index)
        if ws is None or ws.numel() < need:
            ws = torch.empty(need, dtype=torch.uint8, device=dev)
            _workspaces[dev.index] = ws          # kept: stream order makes the reuse by the next call safe
    with torch.cuda.device(dev):
        stream = torch.cuda.current_stream(dev).cuda_stream
        N.check(lib.catcoc_mla_decode(q_nope.data_ptr(), q_rope.data_ptr(), ckv_cache.data_ptr(), krope_cache.data_ptr(),
                                      block_table.data_ptr(), kv_lens.data_ptr(), out.data_ptr(),
                                      ws.data_ptr() if ws is not None else None, batch, q_len, heads,
                                      ckv_cache.shape[0], max_pages, cm.out_fmt(dt), int(causal), float(scale), int(splits),
                                      cm.local_status(dev).data_ptr(), cm.default_timeout_ns(), C.c_void_p(stream)))
    return out


def mla_decode_reference(q_nope: torch.Tensor, q_rope: torch.Tensor, ckv_cache: torch.Tensor,
                         krope_cache: torch.Tensor, block_table: torch.Tensor, kv_lens: torch.Tensor, *,
                         q_len: int = 1, causal: bool = False, scale: Optional[float] = None) -> torch.Tensor:
    """The same function in plain fp32 PyTorch, sequence by sequence (golden for the tests, any device)."""
    if ckv_cache.dim() == 4:
        ckv_cache = ckv_cache.squeeze(2)
    if krope_cache.dim() == 4:
        krope_cache = krope_cache.squeeze(2)
    tokens, heads, _ = q_nope.shape
    batch = tokens // q_len
    scale = 1.0 / math.sqrt(LATENT + ROPE) if scale is None else scale
    out = torch.zeros(tokens, heads, LATENT, dtype=torch.float32, device=q_nope.device)
    for b in range(batch):
        n = int(kv_lens[b])
        if n <= 0:
            continue
        pages = block_table[b, :(n + PAGE - 1) // PAGE].long()
        kn = ckv_cache[pages].reshape(-1, LATENT)[:n].float()
        kr = krope_cache[pages].reshape(-1, ROPE)[:n].float()
        keys = torch.cat([kn, kr], dim=1)                                         # [n, 576]
        q = torch.cat([q_nope[b * q_len:(b + 1) * q_len], q_rope[b * q_len:(b + 1) * q_len]], dim=2).float()   # [q_len, H, 576]
        s = torch.einsum("thd,nd->thn", q, keys) * scale
        if causal:
            t = torch.arange(q_len, device=q.device)[:, None, None]
            j = torch.arange(n, device=q.device)[None, None, :]
            s = s.masked_fill(j >= n - (q_len - 1 - t), float("-inf"))
        p = torch.softmax(s, dim=-1)
        p = torch.nan_to_num(p, nan=0.0)                                          # a token that sees nothing
        out[b * q_len:(b + 1) * q_len] = torch.einsum("thn,nd->thd", p, kn)
    return out

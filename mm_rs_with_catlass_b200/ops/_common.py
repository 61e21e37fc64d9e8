"""Shared plumbing of the op layer: dtype tables, operand normalisation and native launches."""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass
from typing import Optional, Tuple

import torch

from .. import _native as N
from ..tiling.config import TilingConfig

_IN_FMT = {
    torch.float16: N.IN_F16,
    torch.bfloat16: N.IN_BF16,
    torch.int8: N.IN_S8,
}
if hasattr(torch, "float8_e4m3fn"):
    _IN_FMT[torch.float8_e4m3fn] = N.IN_E4M3
    _IN_FMT[torch.float8_e5m2] = N.IN_E5M2

_OUT_FMT = {
    torch.float16: N.FMT_F16,
    torch.bfloat16: N.FMT_BF16,
    torch.float32: N.FMT_F32,
    torch.int32: N.FMT_S32,
}


_ACTIVATIONS = {None: 0, "none": 0, "gelu": 1, "gelu_tanh": 1, "silu": 2, "relu": 3}


def act_code(name) -> int:
    """Code of an epilogue activation: ``gelu`` (tanh form), ``silu``, ``relu`` or None."""
    try:
        return _ACTIVATIONS[name]
    except KeyError:
        raise ValueError("unknown activation %r (gelu, silu, relu or None)" % (name,)) from None


def apply_activation(x: torch.Tensor, name) -> torch.Tensor:
    """The same functions in PyTorch, for the paths that cannot fuse them and for goldens."""
    code = act_code(name)
    if code == 1:
        return torch.nn.functional.gelu(x, approximate="tanh")
    if code == 2:
        return torch.nn.functional.silu(x)
    if code == 3:
        return torch.relu(x)
    return x


def in_fmt(dtype: torch.dtype) -> int:
    try:
        return _IN_FMT[dtype]
    except KeyError:
        raise TypeError("unsupported operand dtype %s (fp16, bf16, int8, fp8 e4m3/e5m2)" % dtype) from None


def out_fmt(dtype: torch.dtype) -> int:
    try:
        return _OUT_FMT[dtype]
    except KeyError:
        raise TypeError("unsupported output dtype %s (fp16, bf16, fp32, int32)" % dtype) from None


def require_cuda(*tensors: torch.Tensor) -> torch.device:
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError(
                "this op runs only on a CUDA device (sm_100a); got a %s tensor. The CPU goldens live in "
                "mm_rs_with_catlass_b200.ops.reference" % t.device)
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise RuntimeError("operands live on different devices: %s vs %s" % (dev, t.device))
    return dev


@dataclass
class Operand:
    """A matrix as the kernel sees it: storage pointer, leading dimension and whether the
    *stored* matrix is the transpose of the logical one."""
    tensor: torch.Tensor  # keeps the (possibly padded) storage alive until the launch is queued
    ptr: int
    ld: int
    trans: bool
    copied: bool = False  # the storage is a fresh padded copy of the caller's data (not reusable)


def _tma_legal(t: torch.Tensor) -> bool:
    elt = t.element_size()
    return t.stride(-1) == 1 and (t.stride(0) * elt) % 16 == 0 and t.data_ptr() % 16 == 0 and t.stride(0) >= t.shape[1]


def pad_rows(t: torch.Tensor) -> torch.Tensor:
    """Returns a copy of the 2-D row-major tensor whose row pitch is a multiple of 16 bytes,
    made by the library's own pad kernel (the analogue of the reference's padding prologue,
    3rdparty/catlass/include/catlass/gemm/kernel/padding_matmul.hpp:32-347)."""
    elt = t.element_size()
    rows, cols = t.shape
    per16 = 16 // elt
    ld = (cols + per16 - 1) // per16 * per16
    buf = torch.empty((rows, ld), dtype=t.dtype, device=t.device)
    src = t if t.stride(-1) == 1 else t.contiguous()
    stream = torch.cuda.current_stream(t.device).cuda_stream
    N.check(N.lib().catcoc_pad2d(buf.data_ptr(), ld * elt, src.data_ptr(), src.stride(0) * elt, rows, cols * elt,
                                 C.c_void_p(stream)))
    return buf


def as_operand(x: torch.Tensor, trans: bool) -> Operand:
    """Normalises a 2-D operand.

    ``x`` is the *stored* matrix ([M, K] or, with ``trans``, [K, M]; likewise for B). A stored
    matrix that is itself a column-major view (``x.stride(0) == 1``) is folded into the
    transpose flag instead of being copied, as the reference's Python wrapper does
    (3rdparty/catlass/examples/python_extension/src/wrapper/catlass_kernel_wrapper.cpp:71-85).
    """
    if x.dim() != 2:
        raise ValueError("operands must be 2-D, got shape %s" % (tuple(x.shape),))
    if x.stride(-1) != 1 and x.stride(0) == 1 and x.shape[0] > 1 and x.shape[1] > 1:
        x = x.t()
        trans = not trans
    copied = False
    if not _tma_legal(x):
        x = pad_rows(x)
        copied = True
    return Operand(x, x.data_ptr(), x.stride(0), trans, copied)


def tkey(t: Optional[torch.Tensor]):
    """Identity of a tensor as far as a launch plan is concerned: where it lives and how it is
    laid out. Two tensors with equal keys give byte-identical kernel arguments."""
    if t is None:
        return None
    return (t.data_ptr(), t.shape, t.stride(), t.dtype)


def on_device(device: torch.device) -> bool:
    return torch.cuda.current_device() == (device.index if device.index is not None else 0)


def fill_tiling(args: N.OpArgs, tiling: Optional[TilingConfig]) -> None:
    t = tiling or TilingConfig()
    args.tiling.bn = t.bn
    args.tiling.swizzle = t.swizzle
    args.tiling.num_ctas = t.num_ctas
    args.tiling.seg_dim = t.seg_dim
    args.tiling.use_multicast = 1 if t.use_multicast else 0
    args.tiling.cta_pair = t.cta_pair
    args.tiling.rounds = t.rounds
    args.tiling.pull = 0              # the fused ops switch it on once the buffers it needs are attached
    args.tiling.comm_warps = t.comm_warps
    args.tiling.push_tma = t.push_tma


def default_timeout_ns() -> int:
    """Time budget of every device-side wait (``CATCOC_TIMEOUT_MS``, default 10 s)."""
    return int(float(os.environ.get("CATCOC_TIMEOUT_MS", "10000")) * 1e6)


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def launch(args: N.OpArgs, device: torch.device, timeout_ns: Optional[int] = None) -> None:
    """Queues the kernel on the current stream of ``device`` (which must be the current device).
    The wait budget is re-read on every launch so that a cached argument block follows
    ``CATCOC_TIMEOUT_MS``."""
    args.timeout_ns = timeout_ns if timeout_ns is not None else default_timeout_ns()
    args.events, args.events_cap = _event_ring
    if _raw_stream is not None and device.index is not None:
        stream = _raw_stream(device.index)
    else:
        stream = torch.cuda.current_stream(device).cuda_stream
    code = N.lib().catcoc_fused_launch(C.byref(args), C.c_void_p(stream))
    if code < 0:
        N.check(code)
    global _launches
    _launches += 1


_launches = 0
_event_ring = (None, 0)


def set_event_ring(ptr, capacity: int) -> None:
    """Device address and record capacity of the event ring every launch from now on writes to
    (None switches it off); see utils/trace.py."""
    global _event_ring
    _event_ring = (ptr, int(capacity) if ptr else 0)


def launch_count() -> int:
    """Launches of the library's GEMM kernel queued by this process so far (fused and local)."""
    return _launches


_status_cache = {}


def local_status(device: torch.device) -> torch.Tensor:
    """Per-device status block for launches that involve no peers."""
    key = (device.type, device.index)
    st = _status_cache.get(key)
    if st is None:
        st = torch.zeros(8, dtype=torch.int32, device=device)
        _status_cache[key] = st
    return st


class StatusError(RuntimeError):
    """A kernel gave up on a wait; ``status`` holds the eight words of its status block
    (code, rank, what, expected, seen, peer, CTA, reserved)."""

    def __init__(self, message: str, status):
        super().__init__(message)
        self.status = list(status)


def raise_on_status(status: torch.Tensor, what: str) -> None:
    """Reads a status block (synchronises) and raises if a kernel reported a failed wait. The
    block is cleared, so the next launch runs again (a fused launch that finds an error latched
    returns at once)."""
    vals = status.cpu().tolist()
    if vals[0] != 0:
        status.zero_()
        raise StatusError(
            "%s failed on rank %d: %s (what=%d expected=%d seen=%d peer=%d cta=%d)"
            % (what, vals[1], N.STATUS_NAMES.get(vals[0], "code %d" % vals[0]), vals[2], vals[3], vals[4], vals[5],
               vals[6]), vals)


def logical_shape(a: torch.Tensor, trans_a: bool, b: torch.Tensor, trans_b: bool) -> Tuple[int, int, int]:
    m, k = (a.shape[1], a.shape[0]) if trans_a else (a.shape[0], a.shape[1])
    kb, n = (b.shape[1], b.shape[0]) if trans_b else (b.shape[0], b.shape[1])
    if k != kb:
        raise ValueError("inner dimensions differ: A gives K=%d, B gives K=%d" % (k, kb))
    return m, n, k

"""Single-GPU GEMM on the library's own tcgen05 kernel.

This is the W = 1 degenerate case of every fused op (same kernel, ``MODE_LOCAL``), the
building block for unit tests and the probe used to measure the GEMM-only gap to cuBLAS.
It covers the plain kernels of the reference's GEMM template library that the fused ops
rely on: basic matmul, matmul with int32 bias and int8 matmul with per-token / per-channel
dequantisation (3rdparty/catlass/include/catlass/gemm/kernel/basic_matmul.hpp:105-137,
matmul_bias.hpp, quant_matmul.hpp), and carries the affine epilogue
``alpha * A @ B + beta * C + bias`` (3rdparty/catlass/include/catlass/epilogue/block/
block_epilogue_gemm.hpp) that :mod:`.blas` builds the rest of that catalogue on.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import _native as N
from ..tiling.config import TilingConfig
from . import _common as cm


def _wants_pad_prologue(a: torch.Tensor) -> bool:
    """A 2-D operand stored row-major with K contiguous whose base or pitch is not 16-byte aligned
    (what ``_common.as_operand`` would otherwise copy into a fresh padded buffer first)."""
    elt = a.element_size()
    if a.dim() != 2 or a.stride(-1) != 1 or a.shape[0] < 1 or a.stride(0) < a.shape[1]:
        return False
    if a.data_ptr() % elt or elt > 2:
        return False
    bits = a.data_ptr() | (a.stride(0) * elt)
    if bits % 2:
        return False                       # 1-byte aligned int8 rows: narrower than the kernel's smallest load
    return bool((a.stride(0) * elt) % 16 or a.data_ptr() % 16)


class _PadState:
    """Per-device workspace of the padding prologue: the padded copy of A (two parity halves, as in
    the all-gather), its chunk stamps per geometry, and the launch counter the stamps are compared
    with. Plain device tensors: nothing here is shared with other ranks."""

    def __init__(self, device: torch.device):
        self.device = device
        self.state = torch.zeros(2, dtype=torch.int32, device=device)    # [0] launches completed, [1] CTA counter
        self.buf = None
        self.half = 0
        self.flags = {}
        self.cur = None

    def attach(self, a: torch.Tensor, m: int, k: int) -> "_PadState":
        elt = a.element_size()
        per16 = 16 // elt
        ld = (k + per16 - 1) // per16 * per16
        half = (m * ld * elt + 1023) // 1024 * 1024
        if self.buf is None or self.half < half:
            self.buf = torch.empty(2 * half, dtype=torch.uint8, device=self.device)
            self.half = half
            _plans.clear()                 # plans hold the old workspace address
        key = (m, ld, elt)
        fl = self.flags.get(key)
        if fl is None:
            words = int(N.lib().catcoc_gather_flag_words(m, ld, 1, elt))
            fl = torch.zeros(max(1, words), dtype=torch.int32, device=self.device)
            if len(self.flags) >= 64:
                self.flags.clear()
                _plans.clear()
            self.flags[key] = fl
        self.cur = (m, ld, fl)
        return self

    def fill(self, args) -> None:
        m, ld, fl = self.cur
        args.mode = N.MODE_AG
        args.rank, args.W = 0, 1
        args.ag_m, args.ag_ld, args.ag_raw = m, ld, 1
        args.gathered[0] = self.buf.data_ptr()
        args.gathered_parity_bytes = self.half
        args.gflags[0] = fl.data_ptr()
        args.epoch_ptr = self.state.data_ptr()
        args.cta_counter = self.state.data_ptr() + 4
        args.limit[N.LIM_GATHERED] = self.buf.numel()
        args.limit[N.LIM_GFLAGS] = fl.numel()


_pad_states: dict = {}


def _pad_state(device: torch.device) -> _PadState:
    key = device.index or 0
    st = _pad_states.get(key)
    if st is None:
        st = _PadState(device)
        _pad_states[key] = st
    return st


# Launch plans of :func:`matmul`: argument blocks keyed by where the operands live and how they
# are laid out. A plan holds addresses, never tensors, so it keeps no memory alive; an entry can
# only be hit again by tensors at the same addresses with the same layout, for which the block is
# exactly what a rebuild would produce. Operands that needed a padded copy are never planned.
_plans: dict = {}
_MAX_PLANS = 4096


def matmul(a: torch.Tensor, b: torch.Tensor, *, trans_a: bool = False, trans_b: bool = False,
           out: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None,
           scale_m: Optional[torch.Tensor] = None, scale_n: Optional[torch.Tensor] = None,
           bias: Optional[torch.Tensor] = None, tiling: Optional[TilingConfig] = None,
           trace: Optional[torch.Tensor] = None, alpha: float = 1.0, beta: float = 0.0,
           c: Optional[torch.Tensor] = None, bias_f32: Optional[torch.Tensor] = None,
           activation: Optional[str] = None, _group: Optional[dict] = None,
           _args_out: Optional[list] = None) -> torch.Tensor:
    """``out = alpha * (A @ B) + beta * C + bias_f32`` with fp32 (int32 for int8) accumulation.

    ``a`` is stored ``[M, K]`` (``[K, M]`` with ``trans_a``), ``b`` is stored ``[K, N]``
    (``[N, K]`` with ``trans_b``). For int8 / fp8 operands ``scale_m`` (fp32 ``[M]``) and
    ``scale_n`` (fp32 ``[N]``) dequantise in the epilogue, ``bias`` (int32 ``[N]``, int8 only)
    is added to the accumulator first. ``c`` (same dtype and shape as the output; it may be the
    output itself) and ``bias_f32`` (fp32 ``[N]``) enter after the dequantisation, in fp32,
    before the single rounding to the output dtype. ``activation`` (``"gelu"`` in its tanh form,
    ``"silu"``, ``"relu"``) is applied last, also in fp32, in the kernel's epilogue.

    ``_group`` is the group walk used by :mod:`.blas` (grouped, batched and split-K products in
    one launch): a dict with the logical ``m, n, k`` of the launch and the ``OpArgs`` group
    fields; ``a`` and ``b`` are then the stacked 2-D storages.
    """
    # Steady state: the same call on the same buffers reuses the argument block built the first
    # time (a launch plan) and goes straight to the native launch.
    key = None
    if _group is None:
        key = (a.device, cm.tkey(a), cm.tkey(b), trans_a, trans_b, cm.tkey(out), out_dtype, cm.tkey(scale_m),
               cm.tkey(scale_n), cm.tkey(bias), tiling, None if trace is None else trace.data_ptr(), alpha, beta,
               cm.tkey(c), cm.tkey(bias_f32), activation)
        plan = _plans.get(key)
        if plan is not None and cm.on_device(a.device):
            args, out_shape, plan_dtype = plan
            if out is None:
                out = torch.empty(out_shape, dtype=plan_dtype, device=a.device)
                args = N.OpArgs.from_buffer_copy(args)   # private copy: the plan itself stays immutable
                args.out = out.data_ptr()
            cm.launch(args, a.device)
            return out
    dev = cm.require_cuda(a, b, out, scale_m, scale_n, bias, c, bias_f32)
    if a.dtype != b.dtype:
        raise TypeError("A and B must share a dtype (got %s, %s)" % (a.dtype, b.dtype))
    if _group is not None:
        m, n, k = _group["m"], _group["n"], _group["k"]
    else:
        m, n, k = cm.logical_shape(a, trans_a, b, trans_b)
    n_vec = n * (_group["num_groups"] if _group is not None and _group.get("g_nvec") else 1)
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

    affine = (alpha != 1.0) or (beta != 0.0 and c is not None) or (bias_f32 is not None)
    if affine and out_dtype == torch.int32:
        raise ValueError("alpha / beta / bias_f32 need a floating-point output")
    if c is not None and beta != 0.0:
        if c.shape != (m, n) or c.dtype != out_dtype or c.stride(-1) != 1:
            raise ValueError("c must be a row-major [%d, %d] %s tensor" % (m, n, out_dtype))
    if tiling is None:
        from ..tiling.chooser import choose
        tiling = choose("matmul", m, n, k, 1, a.dtype)
    with torch.cuda.device(dev):
        # An A stored [M, K] whose base or row pitch TMA cannot take is padded INSIDE the launch: the
        # kernel's communication warps copy it row chunk by row chunk into a 16-byte-pitched workspace and
        # the TMA producer follows chunk by chunk (the one-rank form of the all-gather kernel). No extra
        # launch, no allocation per call, and the call can be planned like any other.
        pad = None
        if _group is None and not trans_a and _wants_pad_prologue(a):
            pad = _pad_state(dev).attach(a, m, k)
            oa = cm.Operand(a, a.data_ptr(), a.stride(0), False)
        else:
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
        args.limit[N.LIM_OUT] = ((out.shape[0] - 1) * out.stride(0) + out.shape[1]) * out.element_size()
        args.partial_fmt = args.out_fmt
        cm.fill_tiling(args, tiling)
        args.rank, args.W = 0, 1
        for name, t, length, dt in (("scale_m", scale_m, m, torch.float32), ("scale_n", scale_n, n_vec, torch.float32),
                                    ("bias", bias, n_vec, torch.int32), ("bias_f", bias_f32, n_vec, torch.float32)):
            if t is not None:
                if t.dtype != dt or t.numel() != length or not t.is_contiguous():
                    raise ValueError("%s must be a contiguous %s tensor of %d elements" % (name, dt, length))
                setattr(args, name, t.data_ptr())
        args.act = cm.act_code(activation)
        if args.act and out_dtype == torch.int32:
            raise ValueError("an activation needs a floating-point output")
        if affine:
            args.affine = 1
            args.alpha, args.beta = float(alpha), float(beta)
            if c is not None and beta != 0.0:
                args.c_src, args.ldc_src = c.data_ptr(), c.stride(0)
        if _group is not None:
            for key in ("num_groups", "group_rows", "a_rows_total", "a_k_total", "b_n_total", "b_k_total",
                        "g_a_row_back", "g_a_k", "g_b_row", "g_b_k", "g_nvec"):
                setattr(args, key, int(_group.get(key, 0)))
            ends = _group.get("group_ends")
            if ends is not None:
                if ends.dtype != torch.int32 or not ends.is_contiguous() or ends.numel() != args.num_groups or ends.device != dev:
                    raise ValueError("group_ends must be a contiguous int32 device tensor of num_groups elements")
                args.group_ends = ends.data_ptr()
        args.status = cm.local_status(dev).data_ptr()
        if trace is not None:  # int64[16] device tensor: per-role cycle counters (see params.h)
            args.trace = trace.data_ptr()
        if pad is not None:
            pad.fill(args)
        if _args_out is not None:
            # a caller that keeps its own plan of a group launch (ops/fused.py); None: the block points at a temporary copy
            _args_out.append(None if (oa.copied or ob.copied) else args)
        cm.launch(args, dev)
        if key is not None and not oa.copied and not ob.copied:
            if len(_plans) >= _MAX_PLANS:
                _plans.clear()
            _plans[key] = (args, tuple(out.shape), out.dtype)
    return out

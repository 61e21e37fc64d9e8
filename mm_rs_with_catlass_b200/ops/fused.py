"""The four fused matmul + collective ops.

Each call launches ONE persistent sm_100a kernel per rank (``csrc/include/catcoc/fused_gemm.cuh``):
tcgen05 tiles fed by TMA, with the collective carried out by the kernel's own epilogue /
communication warps over NVLink peer memory. No NCCL call is made here; the unfused
cuBLAS + NCCL pipeline lives in :mod:`.baseline` and is only ever the thing measured against.

Signatures keep the reference's per-rank tensor layouts
(examples/00_matmul_allreduce/matmul_allreduce.cpp:51-55,
examples/01_allgather_matmul/allgather_matmul.cpp:51-55,
examples/02_matmul_reduce_scatter/matmul_reduce_scatter.cpp:51-55,
examples/02_matmul_reduce_scatter/quant_matmul_reduce_scatter.cpp:55-60) and its transpose
switches (examples/dynamic_tiling/impl/kernel_fp16.cpp:22-86); the symmetric workspace the
reference passes as ``symmetricPtr`` is owned by the :class:`ShmemContext`.

With a world size of 1 every op degenerates to the local GEMM (plus dequantisation), through
the same kernel.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional, Tuple

import torch

from .. import _native as N
from ..parallel import shmem
from ..parallel.shmem import ShmemContext, SymmBuffer
from ..tiling.config import TilingConfig
from ..utils.log import get_logger
from . import _common as cm
from .gemm import matmul as _local_matmul

_SEG_ROWS, _SEG_COLS = 0, 1
# Smallest world size at which a tiling that leaves the choice open (pull = -1) takes the pull flavour
# (CATCOC_PULL=1 forces it, a tiling with pull=1 asks for it). In the sweeps on 2 and 4 GPUs pushing the
# partial tiles won at every M (3-15 % faster: the pushes hide behind a long K loop and the owner's last
# tiles need no further round trip), so the open choice resolves to the push flavour; the measured table
# names the flavour per shape where it was swept.
_PULL_MIN_WORLD = 9
_NVTX = os.environ.get("CATCOC_NVTX", "0") == "1"   # NVTX range around every fused launch


def _ctx(ctx: Optional[ShmemContext]) -> ShmemContext:
    return ctx if ctx is not None else shmem.default_context()


def _data_region(ctx: ShmemContext, purpose: str, half_bytes: int) -> Tuple[SymmBuffer, int]:
    """The symmetric data region of one purpose (partial-tile slabs, all-reduce output, gathered
    activation) and the distance between its two parity halves. Collective by construction:
    every rank runs the same op sequence with the same shapes, so every rank allocates at the
    same calls.

    The parity stride belongs to the BUFFER (half its size), not to the launch: consecutive
    launches of different shapes then agree on which bytes are parity 0 and which parity 1, so a
    rank that is one launch ahead never writes where a peer is still reading, and a result that
    lives in the heap is not overwritten by the next call of another shape. A shape that needs
    more than half the region gets a new, larger region; the old one goes back to the heap (the
    allocator keeps it out of circulation until no rank can still be using it)."""
    half = (int(half_bytes) + 1023) // 1024 * 1024
    buf = ctx.workspaces.get(purpose)
    if buf is None or buf.nbytes < 2 * half:
        if buf is not None:
            ctx.free(buf)
        buf = ctx.malloc(2 * half)
        ctx.workspaces[purpose] = buf
        ctx.counters["regions_grown"] = ctx.counters.get("regions_grown", 0) + 1
        _plans_of(ctx).clear()   # plans hold workspace addresses; every rank grows at the same call
    return buf, (buf.nbytes // 2) // 1024 * 1024


def _span_bytes(t: torch.Tensor) -> int:
    """Bytes from a 2-D row-major tensor's first element to one past its last."""
    return ((t.shape[0] - 1) * t.stride(0) + t.shape[1]) * t.element_size() if t.numel() else 0


def _pair(t: TilingConfig) -> int:
    return 2 if t.cta_pair == 2 else 1


# Launch plans: the argument block of a fused call, keyed by the operands' addresses and layouts
# (see ``_common.tkey``) and kept on the context. In steady state a call is a dictionary lookup,
# an output allocation and the native launch. Plans hold addresses only (no tensors); they are
# dropped whenever a workspace grows, which every rank does at the same call, so a hit on one
# rank and a rebuild on another still address the same buffers.
_MAX_PLANS = 1024


def _plans_of(ctx: ShmemContext) -> dict:
    plans = getattr(ctx, "plans", None)
    if plans is None:
        plans = {}
        ctx.plans = plans
    return plans


def _plan_put(ctx: ShmemContext, key, value) -> None:
    plans = _plans_of(ctx)
    if len(plans) >= _MAX_PLANS:
        plans.clear()
    plans[key] = value


def _plan_hit(ctx: ShmemContext, key):
    plan = _plans_of(ctx).get(key)
    if plan is not None and cm.on_device(ctx.device):
        return plan
    return None


def _with_out(args, out_ptr: int):
    """A private copy of a planned argument block with another output address."""
    args = N.OpArgs.from_buffer_copy(args)
    args.out = out_ptr
    return args


def _resolve_tiling(op: str, m: int, n: int, k: int, world: int, dtype: torch.dtype,
                    tiling: Optional[TilingConfig]) -> TilingConfig:
    if tiling is not None:
        return tiling.validate()
    from ..tiling.chooser import choose
    return choose(op, m, n, k, world, dtype)


def _seg_dim_for(op: str, m: int, n: int, world: int, elt: int, trans_b: bool, t: TilingConfig) -> int:
    """Ownership split of the all-reduce: rows while every rank still owns full 128-row tiles,
    otherwise columns (so small M does not multiply the tensor-core work by the world size).
    A column split of a B stored [K, N] needs 16-byte aligned segment origins for TMA."""
    if op != "matmul_allreduce":
        return _SEG_ROWS
    cols_ok = trans_b or (-(-n // world)) % (16 // elt) == 0
    if t.seg_dim == _SEG_COLS and cols_ok:
        return _SEG_COLS
    if t.seg_dim == _SEG_ROWS:
        return _SEG_ROWS
    return _SEG_ROWS if (m >= world * 128 or not cols_ok) else _SEG_COLS


def _base_args(ctx: ShmemContext, mode: int, a: torch.Tensor, trans_a: bool, b: torch.Tensor, trans_b: bool,
               m: int, n: int, k: int, t: TilingConfig, seg_rows: int = 0):
    """``seg_rows`` > 0: rows per rank when ownership is split by rows. An A stored [K, M] is
    read by TMA along M, so segment origins must then be 16-byte aligned; when they are not,
    A is replaced by a row-major copy."""
    oa = cm.as_operand(a, trans_a)
    if oa.trans and seg_rows and seg_rows % (16 // a.element_size()) != 0:
        oa = cm.as_operand(oa.tensor.t().contiguous(), False)
        oa.copied = True
        ctx.counters["pad_copies"] += 1
    ob = cm.as_operand(b, trans_b)
    args = N.OpArgs()
    args.mode = mode
    args.in_fmt = cm.in_fmt(a.dtype)
    args.M, args.N, args.K = m, n, k
    args.trans_a, args.trans_b = int(oa.trans), int(ob.trans)
    args.a, args.lda = oa.ptr, oa.ld
    args.b, args.ldb = ob.ptr, ob.ld
    cm.fill_tiling(args, t)
    args.rank, args.W = ctx.rank, ctx.world
    args.epoch_ptr = ctx.launch_state.data_ptr()
    args.cta_counter = ctx.launch_state.data_ptr() + 4
    args.status = ctx.status.data_ptr()
    return args, (oa, ob)


def _attach_stage(ctx: ShmemContext, args, m: int, n: int, seg_dim: int, t: TilingConfig, partial_fmt: int) -> None:
    lib = N.lib()
    bn = t.effective_bn
    stage, parity_bytes = _data_region(
        ctx, "stage", int(lib.catcoc_stage_bytes(m, n, ctx.world, seg_dim, bn, t.cta_pair, partial_fmt)) // 2)
    # one stamp array per tile geometry: word (tile, source, quarter) is only ever written by `source`
    arrive = ctx.stamps(("arrive", m, n, ctx.world, seg_dim, bn, _pair(t)),
                        int(lib.catcoc_arrive_words(m, n, ctx.world, seg_dim, bn, t.cta_pair)))
    args.partial_fmt = partial_fmt
    args.stage_parity_bytes = parity_bytes
    args.limit[N.LIM_STAGE], args.limit[N.LIM_ARRIVE] = stage.nbytes, arrive.nbytes // 4
    for p in range(ctx.world):
        args.stage[p] = stage.ptr(p)
        args.arrive[p] = arrive.ptr(p)


def _pull_possible(ctx: ShmemContext, t: TilingConfig, n: int, seg_dim: int, out: Optional[torch.Tensor]) -> bool:
    """Whether this reduce-scatter / all-reduce call takes the pull flavour: the tiling asks for it
    (or leaves the choice open), the heap has a multicast alias, and every 16-byte unit a reducer
    reads lies inside one tile row. ``CATCOC_PULL=0`` switches the automatic choice off."""
    if t.pull == 0 or t.fp32_partials or not ctx.mc_base:
        why = None if t.pull != 1 else ("fp32 partials" if t.fp32_partials else "no multicast alias")
    elif t.pull == -1 and os.environ.get("CATCOC_PULL", "1" if ctx.world >= _PULL_MIN_WORLD else "0") == "0":
        why = None
    elif n % 8 or (seg_dim == _SEG_COLS and (-(-n // ctx.world)) % 8):
        why = "N or the columns per rank are not multiples of 8"
    elif out is not None and (out.data_ptr() % 16 or (out.stride(0) * out.element_size()) % 16):
        why = "the output is not 16-byte aligned"
    else:
        return True
    if why is not None:
        ctx.note_fallback("pull -> push: " + why)
        _log.info("pull flavour not possible (%s): partial tiles are pushed to their owners", why)
    return False


def _attach_pull(ctx: ShmemContext, args, m: int, n: int, seg_dim: int, t: TilingConfig, fmt: int) -> None:
    """Buffers of the pull flavour: this rank's partial [M, N] (two parity halves) with its
    multicast alias, and the per-geometry stamp array in which every rank tells a tile's owner
    that its partial rows are in place."""
    lib = N.lib()
    part, parity_bytes = _data_region(ctx, "part", m * n * 2)
    ready = ctx.stamps(("ready", m, n, ctx.world, seg_dim, t.effective_bn, _pair(t)),
                       int(lib.catcoc_arrive_words(m, n, ctx.world, seg_dim, t.effective_bn, t.cta_pair)))
    args.partial_fmt = fmt
    args.part, args.part_mc, args.part_parity_bytes = part.ptr(), part.mc_ptr(), parity_bytes
    args.limit[N.LIM_PART], args.limit[N.LIM_ARRIVE] = part.nbytes, ready.nbytes // 4
    for p in range(ctx.world):
        args.arrive[p] = ready.ptr(p)
    args.tiling.pull = 1
    ctx.counters["pull_launch_plans"] = ctx.counters.get("pull_launch_plans", 0) + 1


_FMT_BYTES = {N.FMT_F16: 2, N.FMT_BF16: 2, N.FMT_F32: 4, N.FMT_S32: 4}
_MODE_NAMES = {N.MODE_RS: "matmul_reduce_scatter", N.MODE_AR: "matmul_allreduce", N.MODE_AG: "allgather_matmul"}
_log = get_logger("catcoc.ops")


def link_bytes_out(args) -> int:
    """Bytes one launch sends over this GPU's NVLink port (what the kernel's data path moves, from
    the argument block): partial tiles to their owners or to the switch, reduced tiles to every
    rank, the A shard to the peers."""
    W = args.W
    if W <= 1:
        return 0
    if args.mode == N.MODE_AG:
        shard = (args.M // W) * args.K * (1 if args.in_fmt >= N.IN_S8 else 2)
        return shard if (args.gathered_mc and args.tiling.use_multicast) else (W - 1) * shard
    S = args.M * args.N * _FMT_BYTES.get(args.partial_fmt, 2)
    out = S if args.tiling.pull else (W - 1) * S // W          # pull: the switch reads this rank's whole partial
    if args.mode == N.MODE_AR:
        o = args.M * args.N * _FMT_BYTES.get(args.out_fmt, 2) // W
        out += o if (args.tiling.use_multicast and args.ar_out_mc) else (W - 1) * o
    return out


def _describe(ctx: ShmemContext, args, t: TilingConfig) -> None:
    """Record of what a fused call was resolved to: kept on the context (``last_call``) and logged
    at DEBUG level (``CATCOC_LOG=DEBUG``). Runs when a launch plan is built, not on plan hits."""
    path = "local"
    if args.W > 1:
        if args.mode == N.MODE_AG:
            path = "multicast" if (args.gathered_mc and args.tiling.use_multicast) else "peer stores"
        else:
            path = "pull (in-switch sum)" if args.tiling.pull else "push (owner-side sum)"
    ctx.last_call = {"op": _MODE_NAMES.get(args.mode, "matmul"), "M": args.M, "N": args.N, "K": args.K,
                     "world": args.W, "path": path, "tiling": t, "link_bytes_out": link_bytes_out(args)}
    if _log.isEnabledFor(10):
        _log.debug("%(op)s M=%(M)d N=%(N)d K=%(K)d W=%(world)d -> %(path)s, %(link_bytes_out)d B out, %(tiling)s",
                   ctx.last_call)


def _launched(ctx: ShmemContext, args, nvtx: Optional[str] = None) -> int:
    """Launch and advance the host mirror of the epoch; returns the epoch of this launch."""
    trace = getattr(ctx, "trace", None)
    if trace is not None:   # int64[16] device tensor of per-role cycle counters (params.h)
        args.trace = trace.data_ptr()
    if _NVTX:
        torch.cuda.nvtx.range_push(_MODE_NAMES.get(args.mode, "matmul"))
        cm.launch(args, ctx.device)
        torch.cuda.nvtx.range_pop()
    else:
        cm.launch(args, ctx.device)
    ctx.epoch += 1
    ctx.counters["launches"] += 1
    ctx.counters["bytes_out"] += link_bytes_out(args)
    return ctx.epoch


def _check_pair(a: torch.Tensor, b: torch.Tensor) -> None:
    if a.dtype != b.dtype:
        raise TypeError("A and B must share a dtype (got %s, %s)" % (a.dtype, b.dtype))


# ---------------------------------------------------------------------------------------
def matmul_reduce_scatter(a: torch.Tensor, b: torch.Tensor, *, trans_a: bool = False, trans_b: bool = False,
                          out: Optional[torch.Tensor] = None, tiling: Optional[TilingConfig] = None,
                          ctx: Optional[ShmemContext] = None) -> torch.Tensor:
    """Row-parallel linear with a scattered result.

    Per rank: ``a`` ``[M, K_r]`` and ``b`` ``[K_r, N]`` (transposed storage with the flags).
    Returns rows ``[rank*M/W, (rank+1)*M/W)`` of ``sum_r A_r @ B_r`` as ``[M/W, N]``.
    Partials cross NVLink in the operand dtype (as the reference's do, and as NCCL's payload
    in the unfused pipeline is) and are summed in fp32 in a fixed rank order, so the result is
    deterministic; the owner's own partial is never rounded. ``tiling.fp32_partials`` sends fp32
    partials instead (twice the bytes, no intermediate rounding at all).
    """
    ctx = _ctx(ctx)
    key = ("rs", cm.tkey(a), cm.tkey(b), trans_a, trans_b, cm.tkey(out), tiling)
    if tiling is None:
        small = _plan_hit(ctx, ("rs_small",) + key[1:])
        if small is not None:
            if out is None:
                out = torch.empty((small[1][7], small[1][5]), dtype=a.dtype, device=ctx.device)
            return _small_allreduce_call(ctx, small, out)
    plan = _plan_hit(ctx, key)
    if plan is not None:
        args, out_shape, out_dtype = plan
        if out is None:
            out = torch.empty(out_shape, dtype=out_dtype, device=ctx.device)
            args = _with_out(args, out.data_ptr())
        _launched(ctx, args)
        return out
    dev = cm.require_cuda(a, b, out)
    _check_pair(a, b)
    m, n, k = cm.logical_shape(a, trans_a, b, trans_b)
    if ctx.world == 1:
        return _local_matmul(a, b, trans_a=trans_a, trans_b=trans_b, out=out, tiling=tiling)
    if m % ctx.world != 0:
        raise ValueError("matmul_reduce_scatter needs M %% world == 0 (M=%d, world=%d)" % (m, ctx.world))
    if a.dtype not in (torch.float16, torch.bfloat16):
        raise TypeError("matmul_reduce_scatter takes fp16 / bf16 operands; see quant_matmul_reduce_scatter")
    rows = m // ctx.world
    if out is None:
        out = torch.empty((rows, n), dtype=a.dtype, device=dev)
    if tuple(out.shape) != (rows, n) or out.stride(-1) != 1 or out.dtype != a.dtype:
        raise ValueError("out must be a row-major [%d, %d] %s tensor" % (rows, n, a.dtype))
    if tiling is None and _small_reduce_scatter_wanted(m, n, k, a.element_size(), ctx.world):
        res = _small_allreduce(ctx, a, b, trans_a, trans_b, m, n, k, out, scatter=True)
        if res is not None:
            if res[1] is not None:
                _plan_put(ctx, ("rs_small",) + key[1:], res[1])
            return res[0]
    t = _resolve_tiling("matmul_reduce_scatter", m, n, k, ctx.world, a.dtype, tiling)
    with torch.cuda.device(dev):
        args, keep = _base_args(ctx, N.MODE_RS, a, trans_a, b, trans_b, m, n, k, t, seg_rows=rows)
        args.out, args.ldc, args.out_fmt = out.data_ptr(), out.stride(0), cm.out_fmt(out.dtype)
        args.limit[N.LIM_OUT] = _span_bytes(out)
        if _pull_possible(ctx, t, n, _SEG_ROWS, out):
            _attach_pull(ctx, args, m, n, _SEG_ROWS, t, cm.out_fmt(a.dtype))
        else:
            _attach_stage(ctx, args, m, n, _SEG_ROWS, t, N.FMT_F32 if t.fp32_partials else cm.out_fmt(a.dtype))
        _describe(ctx, args, t)
        _launched(ctx, args)
        if not (keep[0].copied or keep[1].copied):
            _plan_put(ctx, key, (args, tuple(out.shape), out.dtype))
    return out


# ---------------------------------------------------------------------------------------
# Small M: split-K product + one-shot all-reduce (two launches of this library's kernels).
# measured on 2 and 4 GPUs: the two-launch path wins at M = 128 (81 vs 103 us, 70 vs 87 us) and loses at M = 256
_SMALL_AR_MAX_M = int(os.environ.get("CATCOC_SMALL_AR_MAX_M", "128"))


def _small_allreduce_wanted(m: int, n: int, k: int, elt: int) -> bool:
    """True where the fused tile loop has nothing to overlap (a single wave of tiles) and a CTA's
    intake bounds the product: few rows, a K long enough to cut, rows of whole 16-byte vectors."""
    if m > _SMALL_AR_MAX_M or n % 8 or n < 128:
        return False
    from .blas import splitk_plan
    return splitk_plan(m, n, k, elt)[0] >= 2


def _small_allreduce_tail(ctx: ShmemContext, plan, out: torch.Tensor) -> None:
    """The second launch of the few-row path (fold the planes, publish, stamp, reduce through the
    switch) and the host-side bookkeeping of the whole call."""
    _, fixed, part_base, parity_bytes, flags_off, meta = plan
    epoch = ctx.epoch + 1
    stream = torch.cuda.current_stream(ctx.device).cuda_stream
    nctx, parts_ptr, s, slice_elems, m, n, row0, rows, fmt = fixed
    code = N.lib().catcoc_splitk_allreduce(C.byref(nctx), parts_ptr, s, slice_elems, m, n, row0, rows, out.data_ptr(),
                                           out.stride(0), fmt, part_base + (epoch & 1) * parity_bytes, flags_off,
                                           1 if ctx.mc_base else 0, ctx.launch_state.data_ptr(),
                                           ctx.launch_state.data_ptr() + 4, ctx.status.data_ptr(),
                                           cm.default_timeout_ns(), C.c_void_p(stream))
    if code < 0:
        N.check(code)
    ctx.epoch = epoch
    ctx.counters["launches"] += 2
    ctx.counters["bytes_out"] += meta["bytes_out"]
    ctx.last_call = meta


def _small_allreduce_call(ctx: ShmemContext, plan, out: torch.Tensor) -> torch.Tensor:
    """Both launches of a planned few-row call: the kept argument block of the split-K product, then the tail."""
    cm.launch(plan[0], ctx.device)
    _small_allreduce_tail(ctx, plan, out)
    return out


_SMALL_RS_MAX_M = int(os.environ.get("CATCOC_SMALL_RS_MAX_M", "256"))


def _small_reduce_scatter_wanted(m: int, n: int, k: int, elt: int, world: int) -> bool:
    """The reduce-scatter takes the few-row path as the all-reduce does, and further up to
    ``_SMALL_RS_MAX_M`` rows while a rank keeps fewer than 128 of them: the fused kernel then runs
    one 128-row tile per destination that is mostly empty (8 GPUs, M = 256: 95 us fused)."""
    if _small_allreduce_wanted(m, n, k, elt):
        return True
    if _SMALL_AR_MAX_M <= 0 or m > _SMALL_RS_MAX_M or m // max(1, world) >= 128 or n % 8 or n < 128:
        return False
    from .blas import splitk_plan
    return splitk_plan(m, n, k, elt)[0] >= 2


def _small_allreduce(ctx: ShmemContext, a: torch.Tensor, b: torch.Tensor, trans_a: bool, trans_b: bool,
                     m: int, n: int, k: int, out: Optional[torch.Tensor], scatter: bool = False):
    """``sum_r A_r @ B_r`` for few rows: the GEMM kernel in its split-K form (every SM streams a
    share of B, fp32 partial planes), then ``splitk_allreduce_kernel``: fold the planes, publish
    the rounded sum in the heap, stamp every rank, and read the sum over all ranks through the
    switch (``multimem.ld_reduce``; peer loads in rank order without a multicast mapping).
    With ``scatter`` every rank reduces and keeps only its own ``m / W`` rows (reduce-scatter).
    Returns ``(out, plan)``, or None when the output cannot take 16-byte stores (the caller then
    runs the fused kernel)."""
    from .blas import splitk_plan, splitk_partials
    dev = a.device
    elt = a.element_size()
    rows = m // ctx.world if scatter else m
    row0 = ctx.rank * rows if scatter else 0
    if out is None:
        out = torch.empty((rows, n), dtype=a.dtype, device=dev)
    if out.stride(-1) != 1 or out.stride(0) % 8 or out.data_ptr() % 16:
        return None
    s, bn = splitk_plan(m, n, k, elt)
    if m % 128 and bn > 128:
        bn = 128
    lib = N.lib()
    with torch.cuda.device(dev):
        scratch = ctx.__dict__.setdefault("local_scratch", {})
        ws = scratch.get("small_ar_planes")
        if ws is None or ws.numel() < s * m * n:
            ws = torch.empty(max(s * m * n, 1 << 22), dtype=torch.float32, device=dev)
            scratch["small_ar_planes"] = ws             # local memory, reused in stream order
            _plans_of(ctx).clear()                      # plans hold the old workspace address
        buf, parity_bytes = _data_region(ctx, "small_ar", m * n * elt)
        flags = ctx.stamps(("small_ar", m, n, ctx.world), int(lib.catcoc_splitk_allreduce_flag_words(m, n, ctx.world)))
        # the first call runs the product through the op layer (checks, tensor maps) and keeps its argument block
        kept: list = []
        part, s = splitk_partials(a, b, split_k=s, trans_a=trans_a, trans_b=trans_b,
                                  tiling=TilingConfig(bn=bn, cta_pair=1), part=ws[:s * m * n].view(s * m, n), _args_out=kept)
        meta = dict(op="matmul_reduce_scatter" if scatter else "matmul_allreduce",
                    path="split-K + one-shot " + ("reduce-scatter" if scatter else "all-reduce"), split_k=s, bn=bn,
                    multicast=bool(ctx.mc_base), m=m, n=n, k=k,
                    # every peer reads this rank's copy of the rows it keeps
                    bytes_out=(ctx.world - 1) * (rows if scatter else m) * n * elt)
        copied = kept[0] is None or (trans_a and (m * elt) % 16 != 0)      # the product read a temporary copy of A
        plan = (kept[0], (ctx.native_ctx(), part.data_ptr(), s, m * n, m, n, row0, rows, cm.out_fmt(a.dtype)), buf.offset,
                parity_bytes, flags.offset, meta)
        # the product is already queued: only the second launch is left for this call
        _small_allreduce_tail(ctx, plan, out)
    return out, (None if copied else plan)


# ---------------------------------------------------------------------------------------
def matmul_allreduce(a: torch.Tensor, b: torch.Tensor, *, trans_a: bool = False, trans_b: bool = False,
                     out: Optional[torch.Tensor] = None, tiling: Optional[TilingConfig] = None,
                     ctx: Optional[ShmemContext] = None) -> torch.Tensor:
    """Row-parallel linear with the full result on every rank: ``sum_r A_r @ B_r`` as ``[M, N]``.

    Two-shot inside one kernel: partial tiles are pushed to the tile's owner, the owner folds
    them into its fp32 accumulator and writes the reduced tile into every rank's output
    (per-peer stores, or one ``multimem.st`` through NVSwitch with ``tiling.use_multicast``).

    Without ``out`` the result is a view of the symmetric heap (no extra copy); it stays valid
    until the second-next fused call on the same context. Pass ``out`` to get a private copy.
    """
    ctx = _ctx(ctx)
    key = ("ar", cm.tkey(a), cm.tkey(b), trans_a, trans_b, tiling)
    if tiling is None:
        small = _plan_hit(ctx, ("ar_small",) + key[1:])
        if small is not None:
            if out is None:
                out = torch.empty((small[1][4], small[1][5]), dtype=a.dtype, device=ctx.device)
            if out.stride(-1) == 1 and out.stride(0) % 8 == 0 and out.data_ptr() % 16 == 0 and \
                    tuple(out.shape) == (small[1][4], small[1][5]) and out.dtype == a.dtype:
                return _small_allreduce_call(ctx, small, out)
    plan = _plan_hit(ctx, key)
    if plan is not None and (out is None or (out.shape == plan[1][0].shape and out.dtype == plan[1][0].dtype)):
        args, views = plan
        view = views[_launched(ctx, args) & 1]
        if out is not None:
            out.copy_(view)
            return out
        return view
    dev = cm.require_cuda(a, b, out)
    _check_pair(a, b)
    m, n, k = cm.logical_shape(a, trans_a, b, trans_b)
    if ctx.world == 1:
        return _local_matmul(a, b, trans_a=trans_a, trans_b=trans_b, out=out, tiling=tiling)
    if a.dtype not in (torch.float16, torch.bfloat16):
        raise TypeError("matmul_allreduce takes fp16 / bf16 operands")
    if out is not None and (tuple(out.shape) != (m, n) or out.dtype != a.dtype):
        raise ValueError("out must be a [%d, %d] %s tensor" % (m, n, a.dtype))
    if tiling is None and _small_allreduce_wanted(m, n, k, a.element_size()):
        res = _small_allreduce(ctx, a, b, trans_a, trans_b, m, n, k, out)
        if res is not None:
            if res[1] is not None:
                _plan_put(ctx, ("ar_small",) + key[1:], res[1])
            return res[0]
    t = _resolve_tiling("matmul_allreduce", m, n, k, ctx.world, a.dtype, tiling)
    if t.use_multicast and not ctx.mc_base:
        t = t.with_(use_multicast=False)
    elt = a.element_size()
    seg_dim = _seg_dim_for("matmul_allreduce", m, n, ctx.world, elt, trans_b, t)
    lib = N.lib()
    with torch.cuda.device(dev):
        args, keep = _base_args(ctx, N.MODE_AR, a, trans_a, b, trans_b, m, n, k, t,
                                seg_rows=(-(-m // ctx.world)) if seg_dim == _SEG_ROWS else 0)
        args.tiling.seg_dim = seg_dim
        obuf, parity_bytes = _data_region(ctx, "ar_out", m * n * elt)
        # one word per 32-row quarter of a tile; the pull flavour stamps each of the quarter's 4 strips
        done = ctx.stamps(("done", m, n, ctx.world, seg_dim, t.effective_bn, _pair(t)),
                          4 * int(lib.catcoc_done_words(m, n, ctx.world, seg_dim, t.effective_bn, t.cta_pair)))
        args.out, args.ldc, args.out_fmt = None, n, cm.out_fmt(a.dtype)
        args.ar_out_parity_bytes = parity_bytes
        for p in range(ctx.world):
            args.ar_out[p] = obuf.ptr(p)
            args.done[p] = done.ptr(p)
        args.ar_out_mc = obuf.mc_ptr() or None
        args.done_mc = done.mc_ptr() or None
        args.limit[N.LIM_AR_OUT], args.limit[N.LIM_DONE] = obuf.nbytes, done.nbytes // 4
        if _pull_possible(ctx, t, n, seg_dim, None):
            _attach_pull(ctx, args, m, n, seg_dim, t, cm.out_fmt(a.dtype))
            args.tiling.use_multicast = 1     # the reducers broadcast through the alias
        else:
            _attach_stage(ctx, args, m, n, seg_dim, t, N.FMT_F32 if t.fp32_partials else cm.out_fmt(a.dtype))
        _describe(ctx, args, t)
        epoch = _launched(ctx, args)
        views = [obuf.tensor(a.dtype, (m, n), byte_offset=par * parity_bytes) for par in (0, 1)]
        view = views[epoch & 1]
        if not (keep[0].copied or keep[1].copied):
            _plan_put(ctx, key, (args, views))
    if out is not None:
        out.copy_(view)
        return out
    return view


# ---------------------------------------------------------------------------------------
# Few rows: gather kernel + split-K product + plane reduction (three launches of this library's kernels).
_SMALL_AG_MAX_M = int(os.environ.get("CATCOC_SMALL_AG_MAX_M", "256"))


def _small_allgather_wanted(m_total: int, n: int, k: int, elt: int, a_shard: torch.Tensor) -> bool:
    """As for the all-reduce: one wave of tiles (N_local / bn CTAs, each streaming all of the gathered A)
    leaves most SMs idle, so the product is cut along K instead and the shard travels first."""
    if m_total > _SMALL_AG_MAX_M or n % 8 or n < 128 or (k * elt) % 16:
        return False
    if a_shard.stride(-1) != 1 or (a_shard.stride(0) * elt) % 16 or a_shard.data_ptr() % 16:
        return False
    from .blas import splitk_plan
    return splitk_plan(m_total, n, k, elt)[0] >= 2


def _small_allgather_run(ctx: ShmemContext, plan: dict, a_shard: torch.Tensor, b: torch.Tensor, out: torch.Tensor):
    from .blas import splitk_partials
    lib = N.lib()
    dev = ctx.device
    epoch = ctx.epoch + 1
    par = epoch & 1
    stream = torch.cuda.current_stream(dev).cuda_stream
    code = lib.catcoc_small_allgather(C.byref(plan["nctx"]), a_shard.data_ptr(), a_shard.stride(0) * plan["elt"], plan["m"],
                                      plan["k"] * plan["elt"], plan["g_off"] + par * plan["parity_bytes"],
                                      plan["k"] * plan["elt"], plan["flags_off"], 1 if ctx.mc_base else 0,
                                      ctx.launch_state.data_ptr(), ctx.launch_state.data_ptr() + 4, ctx.status.data_ptr(),
                                      cm.default_timeout_ns(), C.c_void_p(stream))
    if code < 0:
        N.check(code)
    ctx.epoch = epoch
    gview = plan["views"][par]
    if plan["gemm"][par] is None:
        kept: list = []
        splitk_partials(gview, b, split_k=plan["s"], trans_b=plan["trans_b"], tiling=TilingConfig(bn=plan["bn"], cta_pair=1),
                        part=plan["part"], _args_out=kept)
        if plan["plannable"]:
            plan["gemm"][par] = kept[0]
    else:
        cm.launch(plan["gemm"][par], dev)
    mt, n = plan["mt"], plan["n"]
    code = lib.catcoc_splitk_reduce(plan["part"].data_ptr(), plan["s"], mt * n, mt, n, out.data_ptr(), out.stride(0),
                                    cm.out_fmt(out.dtype), 1.0, 0.0, None, n, None, C.c_void_p(stream))
    if code < 0:
        N.check(code)
    ctx.counters["launches"] += 3
    ctx.counters["bytes_out"] += plan["meta"]["bytes_out"]
    ctx.last_call = plan["meta"]
    return out, gview


def _small_allgather(ctx: ShmemContext, a_shard: torch.Tensor, b: torch.Tensor, trans_b: bool, m: int, n: int, k: int,
                     out: torch.Tensor):
    """``cat_q(A_q) @ B_r`` for few rows: ``small_allgather_kernel`` sends the shard to every rank
    (multicast stores, or a store per peer) and waits for the other shards, the GEMM kernel runs in
    its split-K form on the gathered rows, a third kernel folds the planes. Returns ``(out, gathered, plan)``."""
    from .blas import splitk_plan
    lib = N.lib()
    dev = a_shard.device
    elt = a_shard.element_size()
    W = ctx.world
    mt = W * m
    s, bn = splitk_plan(mt, n, k, elt)
    if mt % 128 and bn > 128:
        bn = 128
    with torch.cuda.device(dev):
        scratch = ctx.__dict__.setdefault("local_scratch", {})
        ws = scratch.get("small_ar_planes")
        if ws is None or ws.numel() < s * mt * n:
            ws = torch.empty(max(s * mt * n, 1 << 22), dtype=torch.float32, device=dev)
            scratch["small_ar_planes"] = ws
            _plans_of(ctx).clear()
        gbuf, parity_bytes = _data_region(ctx, "gathered_small", mt * k * elt)
        flags = ctx.stamps(("small_ag", m, k * elt, W), int(lib.catcoc_small_allgather_flag_words(m, k * elt, W)))
        ob = cm.as_operand(b, trans_b)
        plan = dict(nctx=ctx.native_ctx(), elt=elt, m=m, mt=mt, n=n, k=k, s=s, bn=bn, trans_b=trans_b, g_off=gbuf.offset,
                    parity_bytes=parity_bytes, flags_off=flags.offset, part=ws[:s * mt * n].view(s * mt, n),
                    views=[gbuf.tensor(a_shard.dtype, (mt, k), byte_offset=par * parity_bytes) for par in (0, 1)],
                    gemm=[None, None], plannable=not ob.copied,
                    meta=dict(op="allgather_matmul", path="gather kernel + split-K product", split_k=s, bn=bn,
                              multicast=bool(ctx.mc_base), m=mt, n=n, k=k,
                              bytes_out=(1 if ctx.mc_base else W - 1) * m * k * elt))
        o, g = _small_allgather_run(ctx, plan, a_shard, b, out)
    return o, g, plan


# ---------------------------------------------------------------------------------------
def allgather_matmul(a_shard: torch.Tensor, b: torch.Tensor, *, trans_b: bool = False,
                     out: Optional[torch.Tensor] = None, tiling: Optional[TilingConfig] = None,
                     activation: Optional[str] = None,
                     ctx: Optional[ShmemContext] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Column-parallel linear on a row-sharded activation.

    Per rank: ``a_shard`` ``[m, K]`` and ``b`` ``[K, N_r]`` (``[N_r, K]`` with ``trans_b``).
    Returns ``(out, gathered)``: ``out`` ``[W*m, N_r]`` with row block ``q`` equal to
    ``A_q @ B_r``, and the gathered activation ``[W*m, K]`` (a view of the symmetric heap that
    stays valid until the second-next fused call on the same context).

    Communication warps of every CTA push the local shard to the peers, nearest consumer first,
    while the tensor cores already work on the local rows; a remote row block is consumed as
    soon as its chunk stamps arrive. ``trans_a`` is not supported, as in the reference
    (examples/dynamic_tiling/impl/kernel_fp16.cpp:55-61).

    ``activation`` (``"gelu"`` in its tanh form, ``"silu"``, ``"relu"``) is applied to the product
    in the kernel's epilogue, in fp32, before the single rounding to the output dtype. The
    epilogue variant that carries it has one communication warp per CTA, which is enough when
    the shard travels by multicast stores.
    """
    ctx = _ctx(ctx)
    key = ("ag", cm.tkey(a_shard), cm.tkey(b), trans_b, cm.tkey(out), tiling, activation)
    if tiling is None and activation is None:
        small = _plan_hit(ctx, ("ag_small",) + key[1:])
        if small is not None:
            if out is None:
                out = torch.empty((small["mt"], small["n"]), dtype=a_shard.dtype, device=ctx.device)
            return _small_allgather_run(ctx, small, a_shard, b, out)
    plan = _plan_hit(ctx, key)
    if plan is not None:
        args, out_shape, out_dtype, gviews = plan
        if out is None:
            out = torch.empty(out_shape, dtype=out_dtype, device=ctx.device)
            args = _with_out(args, out.data_ptr())
        return out, gviews[_launched(ctx, args) & 1]
    dev = cm.require_cuda(a_shard, b, out)
    _check_pair(a_shard, b)
    if a_shard.dim() != 2:
        raise ValueError("a_shard must be 2-D")
    m, k = a_shard.shape
    kb, n = (b.shape[1], b.shape[0]) if trans_b else (b.shape[0], b.shape[1])
    if k != kb:
        raise ValueError("inner dimensions differ: A gives K=%d, B gives K=%d" % (k, kb))
    if ctx.world == 1:
        o = _local_matmul(a_shard, b, trans_b=trans_b, out=out, tiling=tiling, activation=activation)
        return o, a_shard
    if a_shard.dtype not in (torch.float16, torch.bfloat16):
        raise TypeError("allgather_matmul takes fp16 / bf16 operands")
    W = ctx.world
    if out is None:
        out = torch.empty((W * m, n), dtype=a_shard.dtype, device=dev)
    if tuple(out.shape) != (W * m, n) or out.stride(-1) != 1 or out.dtype != a_shard.dtype:
        raise ValueError("out must be a row-major [%d, %d] %s tensor" % (W * m, n, a_shard.dtype))
    elt = a_shard.element_size()
    if tiling is None and activation is None and _small_allgather_wanted(W * m, n, k, elt, a_shard):
        o, g, small = _small_allgather(ctx, a_shard, b, trans_b, m, n, k, out)
        if small["plannable"]:
            _plan_put(ctx, ("ag_small",) + key[1:], small)
        return o, g
    t = _resolve_tiling("allgather_matmul", W * m, n, k, W, a_shard.dtype, tiling)
    lib = N.lib()
    with torch.cuda.device(dev):
        # The gathered buffer has a dense pitch of ag_ld >= K elements (16-byte multiple); the
        # shard is copied row by row with that width, so it needs a TMA-legal pitch itself.
        per16 = 16 // elt
        ag_ld = (k + per16 - 1) // per16 * per16
        # A shard whose base or pitch TMA cannot take is not copied first: the communication warps fetch
        # it with narrower loads and the kernel reads the local rows from the gathered buffer as well
        a_src = a_shard
        raw = False
        if a_shard.stride(-1) != 1 or a_shard.stride(0) < k or a_shard.data_ptr() % elt:
            a_src = a_shard.contiguous()
            ctx.counters["pad_copies"] += 1
        if (a_src.stride(0) * elt) % 16 or a_src.data_ptr() % 16 or a_src.stride(0) < ag_ld:
            raw = True
        ob = cm.as_operand(b, trans_b)
        args = N.OpArgs()
        args.mode = N.MODE_AG
        args.in_fmt = cm.in_fmt(a_shard.dtype)
        args.M, args.N, args.K = W * m, n, k
        args.trans_a, args.trans_b = 0, int(ob.trans)
        args.a, args.lda = a_src.data_ptr(), a_src.stride(0)
        args.b, args.ldb = ob.ptr, ob.ld
        cm.fill_tiling(args, t)
        args.rank, args.W = ctx.rank, W
        args.epoch_ptr = ctx.launch_state.data_ptr()
        args.cta_counter = ctx.launch_state.data_ptr() + 4
        args.status = ctx.status.data_ptr()
        args.ag_m, args.ag_ld = m, ag_ld
        args.ag_raw = int(raw)
        args.act = cm.act_code(activation)
        gbuf, parity_bytes = _data_region(ctx, "gathered", W * m * ag_ld * elt)
        gfl = ctx.stamps(("gflags", m, ag_ld, W, elt, _pair(t)), int(lib.catcoc_gather_flag_words(m, ag_ld, W, elt)))
        args.gathered_parity_bytes = parity_bytes
        for p in range(W):
            args.gathered[p] = gbuf.ptr(p)
            args.gflags[p] = gfl.ptr(p)
        args.limit[N.LIM_GATHERED], args.limit[N.LIM_GFLAGS] = gbuf.nbytes, gfl.nbytes // 4
        args.limit[N.LIM_OUT] = _span_bytes(out)
        # shard broadcast by multicast stores (one multimem.st reaches every rank) when the heap has
        # the alias and the tiling or CATCOC_AG_MULTICAST asks for it
        want_mc = t.use_multicast if os.environ.get("CATCOC_AG_MULTICAST") is None \
            else os.environ["CATCOC_AG_MULTICAST"] == "1"
        if args.act and os.environ.get("CATCOC_AG_MULTICAST") is None:
            want_mc = True      # the epilogue variant with the activation has ONE communication warp: enough for
            #                     multicast stores (the shard leaves once), not for W - 1 peer copies
        if want_mc and ctx.mc_base:
            args.gathered_mc, args.gflags_mc = gbuf.mc_ptr(), gfl.mc_ptr()
            args.tiling.use_multicast = 1
        else:
            args.tiling.use_multicast = 0
        args.out, args.ldc, args.out_fmt = out.data_ptr(), out.stride(0), cm.out_fmt(out.dtype)
        args.partial_fmt = args.out_fmt
        _describe(ctx, args, t)
        epoch = _launched(ctx, args)
        gviews = [gbuf.tensor(a_shard.dtype, (W * m, ag_ld), byte_offset=par * parity_bytes) for par in (0, 1)]
        if ag_ld != k:
            gviews = [g[:, :k] for g in gviews]
        gathered = gviews[epoch & 1]
        if a_src is a_shard and not ob.copied:
            _plan_put(ctx, key, (args, tuple(out.shape), out.dtype, gviews))
    return out, gathered


# ---------------------------------------------------------------------------------------
def quant_matmul_reduce_scatter(x1: torch.Tensor, x2: torch.Tensor, scale_x1: torch.Tensor, scale_x2: torch.Tensor,
                                bias: Optional[torch.Tensor] = None, *, trans_a: bool = False, trans_b: bool = False,
                                out_dtype: torch.dtype = torch.bfloat16, out: Optional[torch.Tensor] = None,
                                tiling: Optional[TilingConfig] = None,
                                ctx: Optional[ShmemContext] = None) -> torch.Tensor:
    """int8 row-parallel linear with an exact int32 reduce-scatter and fused dequantisation.

    Per rank: ``x1`` int8 ``[M, K_r]``, ``x2`` int8 ``[K_r, N]``, ``scale_x1`` fp32 ``[M]``
    (per token, indexed by the global row), ``scale_x2`` fp32 ``[N]`` (per channel), optional
    ``bias`` int32 ``[N]``. Returns ``[M/W, N]``:

        cast( float( sum_q (x1_q @ x2_q + bias) )[rows of this rank] * scale_x1[rows, None] * scale_x2[None, :] )

    The bias is added on every rank, so the sum carries ``W * bias`` exactly as in the
    reference (examples/utils/gen_quant_data.py:61-72). int32 partial tiles cross NVLink
    unrounded; the sum is exact and order-free, the scales are applied once on the owner.
    """
    ctx = _ctx(ctx)
    key = ("qrs", cm.tkey(x1), cm.tkey(x2), cm.tkey(scale_x1), cm.tkey(scale_x2), cm.tkey(bias), trans_a, trans_b,
           out_dtype, cm.tkey(out), tiling)
    plan = _plan_hit(ctx, key)
    if plan is not None:
        args, out_shape, plan_dtype = plan
        if out is None:
            out = torch.empty(out_shape, dtype=plan_dtype, device=ctx.device)
            args = _with_out(args, out.data_ptr())
        _launched(ctx, args)
        return out
    dev = cm.require_cuda(x1, x2, scale_x1, scale_x2, bias, out)
    if x1.dtype != torch.int8 or x2.dtype != torch.int8:
        raise TypeError("x1 and x2 must be int8")
    if out_dtype not in (torch.float16, torch.bfloat16, torch.float32):
        raise TypeError("out_dtype must be fp16, bf16 or fp32")
    m, n, k = cm.logical_shape(x1, trans_a, x2, trans_b)
    for name, s, length, dt in (("scale_x1", scale_x1, m, torch.float32), ("scale_x2", scale_x2, n, torch.float32),
                                ("bias", bias, n, torch.int32)):
        if s is not None and (s.dtype != dt or s.numel() != length or not s.is_contiguous()):
            raise ValueError("%s must be a contiguous %s tensor of %d elements" % (name, dt, length))
    if ctx.world == 1:
        return _local_matmul(x1, x2, trans_a=trans_a, trans_b=trans_b, out=out, out_dtype=out_dtype,
                             scale_m=scale_x1, scale_n=scale_x2, bias=bias, tiling=tiling)
    if m % ctx.world != 0:
        raise ValueError("quant_matmul_reduce_scatter needs M %% world == 0 (M=%d, world=%d)" % (m, ctx.world))
    rows = m // ctx.world
    if out is None:
        out = torch.empty((rows, n), dtype=out_dtype, device=dev)
    if tuple(out.shape) != (rows, n) or out.stride(-1) != 1 or out.dtype != out_dtype:
        raise ValueError("out must be a row-major [%d, %d] %s tensor" % (rows, n, out_dtype))
    t = _resolve_tiling("quant_matmul_reduce_scatter", m, n, k, ctx.world, x1.dtype, tiling)
    with torch.cuda.device(dev):
        args, keep = _base_args(ctx, N.MODE_RS, x1, trans_a, x2, trans_b, m, n, k, t, seg_rows=rows)
        args.out, args.ldc, args.out_fmt = out.data_ptr(), out.stride(0), cm.out_fmt(out_dtype)
        args.limit[N.LIM_OUT] = _span_bytes(out)
        args.scale_m = scale_x1.data_ptr()
        args.scale_n = scale_x2.data_ptr()
        args.bias = bias.data_ptr() if bias is not None else None
        _attach_stage(ctx, args, m, n, _SEG_ROWS, t, N.FMT_S32)
        _describe(ctx, args, t)
        _launched(ctx, args)
        if not (keep[0].copied or keep[1].copied):
            _plan_put(ctx, key, (args, tuple(out.shape), out.dtype))
    return out

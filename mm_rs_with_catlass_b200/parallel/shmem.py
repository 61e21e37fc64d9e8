"""Symmetric heap and SHMEM context for the GPUs of one box.

One process per GPU. ``init()`` is collective over a ``torch.distributed`` group (any
backend: it is only used to agree on socket names and to order the bootstrap steps). Each
rank creates its slice of the heap with the CUDA VMM API, the POSIX handles travel over
abstract unix sockets, and every rank maps every slice, so a symmetric object lives at the
same offset on all ranks and a peer's copy is reachable by plain loads and stores over
NVLink. When NVLS is available (and not disabled) a multicast alias of the whole heap is
mapped too.

Host API (collective unless noted), mirroring the SHMEM calls the reference makes
(shmem_set_attr / shmem_init_attr / shmem_malloc / shmem_free / shmem_finalize,
examples/00_matmul_allreduce/matmul_allreduce.cpp:239-300):

    ctx = shmem.init(group=None, heap_bytes=2 << 30)
    buf = ctx.malloc(nbytes)              # SymmBuffer: .offset, .tensor(dtype, shape)
    ctx.free(buf)                         # returns the block (reusable two fused launches later)
    ctx.barrier()                         # device-side barrier_all on the current stream
    ctx.put(peer, dst_buf, src_tensor)    # one-sided copies (non-collective)
    ctx.finalize()

Device API: ``csrc/include/catcoc/shmem_device.cuh``.
"""
from __future__ import annotations

import atexit
import ctypes as C
import os
import secrets
import weakref
from collections import OrderedDict
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from .. import _native as N
from .allocator import HeapExhausted, SymmAllocator

DEFAULT_HEAP_BYTES = 2 << 30
_ALIGN = 256
_MAX_STAMP_REGIONS = 64


class ShmemError(RuntimeError):
    pass


class _RawCudaMemory:
    """Exposes a raw device range through ``__cuda_array_interface__`` so torch can view it."""

    def __init__(self, ptr: int, nbytes: int, owner):
        self._owner = owner  # keeps the heap alive while views exist
        self.__cuda_array_interface__ = {
            "shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3, "strides": None,
        }


@dataclass
class SymmBuffer:
    """A symmetric allocation: the same ``offset`` is valid on every rank."""
    ctx: "ShmemContext"
    offset: int
    nbytes: int

    def ptr(self, peer: Optional[int] = None) -> int:
        return self.ctx.base(self.ctx.rank if peer is None else peer) + self.offset

    def mc_ptr(self) -> int:
        return self.ctx.mc_base + self.offset if self.ctx.mc_base else 0

    def tensor(self, dtype: torch.dtype = torch.uint8, shape: Optional[Sequence[int]] = None,
               byte_offset: int = 0) -> torch.Tensor:
        """A torch view of the *local* copy."""
        raw = self.ctx._local_bytes[self.offset + byte_offset: self.offset + self.nbytes]
        t = raw.view(dtype)
        if shape is not None:
            n = 1
            for s in shape:
                n *= int(s)
            t = t[:n].view(*shape)
        return t


class ShmemContext:
    """Owns the heap, the allocator, the device barrier state and the fused-op workspaces."""

    def __init__(self, group, rank: int, world: int, device: torch.device, handle: C.c_void_p, heap_bytes: int,
                 multicast: bool):
        self.group = group
        self.rank = rank
        self.world = world
        self.device = device
        self._h = handle
        self.heap_bytes = heap_bytes
        self.multicast = multicast
        self._bases = [int(N.lib().catcoc_heap_base(handle, p) or 0) for p in range(world)]
        self.mc_base = int(N.lib().catcoc_heap_mc_base(handle) or 0) if multicast else 0
        self._local_bytes = torch.as_tensor(_RawCudaMemory(self._bases[rank], heap_bytes, self), device=device)
        # Stamps are compared with launch epochs, so no word of the heap may start out above zero.
        # init() synchronises and meets the peers after this, before anybody can write here.
        self._local_bytes.zero_()
        self._alloc = SymmAllocator(heap_bytes)
        self.epoch = 0  # host mirror of launch_state[0]: fused launches issued on this context
        self._finalized = False
        self.status = torch.zeros(8, dtype=torch.int32, device=device)
        # launch bookkeeping of the fused kernels: [0] completed launches (epoch), [1] CTA counter
        self.launch_state = torch.zeros(2, dtype=torch.int32, device=device)
        self._barrier_buf = self.malloc(4 * N.MAX_WORLD)
        self._barrier_epoch = 0
        self.workspaces: Dict[object, object] = {}   # data regions of the fused ops, by purpose
        self.stamp_regions: "OrderedDict[object, SymmBuffer]" = OrderedDict()   # stamp arrays, by geometry
        self.plans: Dict[object, object] = {}   # launch plans of the fused ops (ops/fused.py)
        # launches of fused kernels, bytes they sent over this GPU's NVLink port, padded operand copies
        self.counters: Dict[str, int] = {"launches": 0, "bytes_out": 0, "pad_copies": 0}
        self.last_call: Optional[dict] = None   # what the most recent new launch plan was resolved to
        self.fallbacks: Dict[str, int] = {}

    def note_fallback(self, reason: str) -> None:
        """Records that a call could not take the path its tiling asked for (counted per reason)."""
        self.fallbacks[reason] = self.fallbacks.get(reason, 0) + 1

    # ---- addresses -------------------------------------------------------------------
    def base(self, peer: int) -> int:
        if not 0 <= peer < self.world:
            raise ShmemError("peer %d out of range [0, %d)" % (peer, self.world))
        return self._bases[peer]

    def native_ctx(self) -> N.ShmemCtx:
        c = N.ShmemCtx()
        c.rank, c.W = self.rank, self.world
        for p in range(self.world):
            c.base[p] = self._bases[p]
        c.mc_base = self.mc_base or None
        c.barrier_off = self._barrier_buf.offset
        return c

    # ---- allocator (collective: every rank must make the same sequence of calls) ------
    def malloc(self, nbytes: int) -> SymmBuffer:
        """A block of the heap at the same offset on every rank (256-byte aligned). The contents
        are whatever the block last held; stamp arrays are zeroed by their owner (``stamps``)."""
        if nbytes <= 0:
            raise ShmemError("malloc of %d bytes" % nbytes)
        try:
            start = self._alloc.malloc(nbytes, tick=self.epoch)
        except HeapExhausted as e:
            raise ShmemError("%s; the heap has %d bytes per rank (raise heap_bytes in shmem.init or "
                             "CATCOC_HEAP_BYTES)" % (e, self.heap_bytes)) from None
        return SymmBuffer(self, start, nbytes)

    def free(self, buf: SymmBuffer) -> None:
        """Returns a block to the heap (the reference's shmem_free,
        examples/00_matmul_allreduce/matmul_allreduce.cpp:290). Collective like ``malloc``. The
        block is handed out again only after two more fused launches were issued on this
        context: peers run at most one launch apart, so by then none of them can still touch it.
        A caller that moves data with ``put`` / ``get`` outside the fused ops must make sure with a
        ``barrier()`` that no peer still uses the block."""
        try:
            self._alloc.free(buf.offset, tick=self.epoch)
        except ValueError as e:
            raise ShmemError(str(e)) from None

    def stamps(self, key, words: int) -> SymmBuffer:
        """The stamp array of one (purpose, geometry) ``key``, created on first use. Collective:
        every rank reaches the first use of a key at the same call. A new array is zeroed and the
        ranks meet at a device barrier before anybody stamps it. Arrays are kept per geometry so
        that every word has one writer and one meaning for as long as it lives; the least recently
        used ones are released when more than ``_MAX_STAMP_REGIONS`` exist."""
        buf = self.stamp_regions.get(key)
        if buf is not None:
            self.stamp_regions.move_to_end(key)
            return buf
        while len(self.stamp_regions) >= _MAX_STAMP_REGIONS:
            _, old = self.stamp_regions.popitem(last=False)
            self.free(old)
            self.plans.clear()   # plans may hold the released addresses
        buf = self.malloc(4 * max(1, int(words)))
        buf.tensor(torch.int32).zero_()
        if self.world > 1:
            self.barrier()
        self.stamp_regions[key] = buf
        return buf

    def empty(self, shape: Sequence[int], dtype: torch.dtype) -> Tuple[torch.Tensor, SymmBuffer]:
        n = 1
        for s in shape:
            n *= int(s)
        buf = self.malloc(max(1, n) * torch.empty((), dtype=dtype).element_size())
        return buf.tensor(dtype, shape), buf

    @property
    def bytes_in_use(self) -> int:
        return self._alloc.bytes_in_use

    @property
    def high_water(self) -> int:
        """Largest offset the allocator has handed out so far."""
        return self._alloc.high_water

    # ---- synchronisation ---------------------------------------------------------------
    def _stream(self) -> C.c_void_p:
        return C.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)

    def barrier(self, timeout_ms: Optional[float] = None) -> None:
        """Device-side barrier across all ranks, queued on the current stream."""
        self._barrier_epoch += 1
        nctx = self.native_ctx()
        tns = int((timeout_ms if timeout_ms is not None else float(os.environ.get("CATCOC_TIMEOUT_MS", "10000"))) * 1e6)
        N.check(N.lib().catcoc_shmem_barrier_all(C.byref(nctx), self._barrier_epoch, tns, self.status.data_ptr(),
                                                 self._stream()))

    def host_barrier(self) -> None:
        torch.cuda.synchronize(self.device)
        if self.world > 1:
            dist.barrier(group=self.group)

    def check(self, what: str = "kernel") -> None:
        """Synchronises and raises if any kernel of this context reported a failed wait."""
        from ..ops._common import raise_on_status
        raise_on_status(self.status, what)

    def reset_after_error(self) -> None:
        """Collective. Brings every rank's epoch back in step after a failed launch."""
        self.host_barrier()
        self.status.zero_()
        e = self.launch_state[:1].clone()
        if self.world > 1:
            backend = dist.get_backend(self.group)
            t = e.cpu() if backend == "gloo" else e
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.group)
            e = t.to(self.device)
        self.launch_state[0] = e[0] + 2  # skip both parities that may hold half-written data
        self.launch_state[1] = 0
        self.epoch = int(self.launch_state[0].item())
        self.host_barrier()

    # ---- one-sided data movement (non-collective) -----------------------------------------
    def put(self, peer: int, dst: SymmBuffer, src: torch.Tensor, dst_byte_offset: int = 0,
            signal: Optional[SymmBuffer] = None, signal_value: int = 1) -> None:
        """Copies ``src`` into ``dst`` on rank ``peer``; optionally adds ``signal_value`` to a
        32-bit signal word on that rank once per launched block (see ``put_blocks``)."""
        src = src.contiguous()
        nbytes = src.numel() * src.element_size()
        if dst_byte_offset + nbytes > dst.nbytes:
            raise ShmemError("put overflows the destination buffer")
        nctx = self.native_ctx()
        N.check(N.lib().catcoc_shmem_put(C.byref(nctx), peer, dst.offset + dst_byte_offset, src.data_ptr(), nbytes,
                                         signal.offset if signal is not None else -1, signal_value, self._stream()))

    @staticmethod
    def put_blocks() -> int:
        return int(N.lib().catcoc_shmem_put_blocks())

    def get(self, peer: int, dst: torch.Tensor, src: SymmBuffer, src_byte_offset: int = 0) -> None:
        if not dst.is_contiguous():
            raise ShmemError("get needs a contiguous destination")
        nbytes = dst.numel() * dst.element_size()
        nctx = self.native_ctx()
        N.check(N.lib().catcoc_shmem_get(C.byref(nctx), peer, dst.data_ptr(), src.offset + src_byte_offset, nbytes,
                                         self._stream()))

    def wait_until(self, signal: SymmBuffer, value: int, timeout_ms: float = 10000.0) -> None:
        """Queues a bounded device-side wait until the local signal word is >= value."""
        nctx = self.native_ctx()
        N.check(N.lib().catcoc_shmem_wait_until(C.byref(nctx), signal.offset, value, int(timeout_ms * 1e6),
                                                self.status.data_ptr(), self._stream()))

    def mc_broadcast(self, dst: SymmBuffer, src: torch.Tensor) -> None:
        """NVLS: one multimem.st per 16 bytes lands ``src`` in ``dst`` on every rank."""
        if not self.mc_base:
            raise ShmemError("no multicast mapping (NVLS unsupported or disabled)")
        src = src.contiguous()
        nctx = self.native_ctx()
        N.check(N.lib().catcoc_shmem_mc_broadcast(C.byref(nctx), dst.offset, src.data_ptr(),
                                                  src.numel() * src.element_size(), self._stream()))

    def mc_reduce_bf16(self, dst: torch.Tensor, src: SymmBuffer) -> None:
        """NVLS: ``dst`` = sum over ranks of the bf16 array in ``src`` (fp32 accumulate in the switch)."""
        if not self.mc_base:
            raise ShmemError("no multicast mapping (NVLS unsupported or disabled)")
        nctx = self.native_ctx()
        N.check(N.lib().catcoc_shmem_mc_reduce_bf16(C.byref(nctx), dst.data_ptr(), src.offset, dst.numel(),
                                                    self._stream()))

    # ---- teardown ----------------------------------------------------------------------
    def finalize(self, collective: bool = True) -> None:
        """Idempotent teardown. With ``collective`` (the default) all ranks first meet at a host
        barrier so that no rank unmaps memory a peer's kernel may still touch; the exit hook
        passes False because the process group may already be gone."""
        if self._finalized:
            return
        self._finalized = True
        try:
            torch.cuda.synchronize(self.device)
            if collective and self.world > 1 and dist.is_initialized():
                dist.barrier(group=self.group)
        except Exception:
            pass
        self.workspaces.clear()
        self.stamp_regions.clear()
        self.plans.clear()
        self._local_bytes = None
        N.lib().catcoc_heap_destroy(self._h)
        self._h = None
        global _default_ctx
        if _default_ctx is self:
            _default_ctx = None


_default_ctx: Optional[ShmemContext] = None


def _exchange_fds(handle, rank: int, world: int, uid: str, group, my_fd: int, timeout_ms: int) -> None:
    lib = N.lib()
    sock_name = ("catcoc-%s-%d" % (uid, rank)).encode()
    sock = N.check(lib.catcoc_fd_recv_open(sock_name))
    try:
        dist.barrier(group=group)  # every receive socket is bound
        for step in range(1, world):
            peer = (rank + step) % world
            N.check(lib.catcoc_fd_send(("catcoc-%s-%d" % (uid, peer)).encode(), my_fd, rank, timeout_ms))
        for _ in range(world - 1):
            tag = C.c_int(-1)
            fd = N.check(lib.catcoc_fd_recv(sock, timeout_ms, C.byref(tag)))
            try:
                N.check(lib.catcoc_heap_import_peer(handle, tag.value, fd))
            finally:
                lib.catcoc_fd_close(fd)
    finally:
        lib.catcoc_fd_close(sock)


def _setup_multicast(handle, rank: int, world: int, uid: str, group, timeout_ms: int) -> bool:
    """Returns True when every rank mapped the multicast alias; False leaves the heap on P2P."""
    lib = N.lib()
    sock_name = ("catcoc-mc-%s-%d" % (uid, rank)).encode()
    ok = 1
    sock = -1
    try:
        if rank != 0:
            sock = N.check(lib.catcoc_fd_recv_open(sock_name))
        dist.barrier(group=group)
        if rank == 0:
            fd = lib.catcoc_heap_mc_create(handle)
            if fd < 0:
                ok = 0
            else:
                for peer in range(1, world):
                    N.check(lib.catcoc_fd_send(("catcoc-mc-%s-%d" % (uid, peer)).encode(), fd, 0, timeout_ms))
                lib.catcoc_fd_close(fd)
                if lib.catcoc_heap_mc_join(handle, -1) < 0:
                    ok = 0
        flags: List[int] = [0] * world
        dist.all_gather_object(flags, ok if rank == 0 else 1, group=group)
        if not flags[0]:
            return False
        if rank != 0:
            tag = C.c_int(-1)
            fd = N.check(lib.catcoc_fd_recv(sock, timeout_ms, C.byref(tag)))
            try:
                if lib.catcoc_heap_mc_join(handle, fd) < 0:
                    ok = 0
            finally:
                lib.catcoc_fd_close(fd)
        dist.all_gather_object(flags, ok, group=group)  # every device added before anyone binds
        if not all(flags):
            return False
        if lib.catcoc_heap_mc_bind(handle) < 0:
            ok = 0
        dist.all_gather_object(flags, ok, group=group)
        return all(flags)
    finally:
        if sock >= 0:
            lib.catcoc_fd_close(sock)


def init(group=None, heap_bytes: Optional[int] = None, device: Optional[torch.device] = None,
         multicast: Optional[bool] = None, make_default: bool = True, bootstrap_timeout_ms: int = 60000) -> ShmemContext:
    """Collective set-up of the symmetric heap over ``group`` (default: the world group).

    ``heap_bytes`` is the per-rank heap size and must be equal on all ranks. ``multicast``
    None means "use NVLS when every GPU supports it, unless ``CATCOC_NVLS=0``".
    """
    if not torch.cuda.is_available():
        raise ShmemError("the symmetric heap needs CUDA devices")
    if dist.is_initialized():
        rank = dist.get_rank(group)
        world = dist.get_world_size(group)
    else:
        rank, world = 0, 1
    if world > N.MAX_WORLD:
        raise ShmemError("world size %d exceeds the %d GPUs of one box" % (world, N.MAX_WORLD))
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device())
    if heap_bytes is None:
        heap_bytes = int(os.environ.get("CATCOC_HEAP_BYTES", DEFAULT_HEAP_BYTES))
    lib = N.lib()

    if world > 1:
        info: List[object] = [None] * world
        dist.all_gather_object(info, (int(heap_bytes), secrets.token_hex(8)), group=group)
        sizes = {i[0] for i in info}
        if len(sizes) != 1:
            raise ShmemError("heap_bytes differs across ranks: %s" % sorted(sizes))
        uid = info[0][1]
    else:
        uid = secrets.token_hex(8)

    handle = C.c_void_p()
    N.check(lib.catcoc_heap_create(device.index or 0, rank, world, int(heap_bytes), C.byref(handle)))
    try:
        use_mc = False
        if world > 1:
            fd = N.check(lib.catcoc_heap_export_fd(handle))
            try:
                _exchange_fds(handle, rank, world, uid, group, fd, bootstrap_timeout_ms)
            finally:
                lib.catcoc_fd_close(fd)
            dist.barrier(group=group)
            want = multicast if multicast is not None else (os.environ.get("CATCOC_NVLS", "1") != "0")
            supported = [0] * world
            dist.all_gather_object(supported, int(bool(want)) & int(lib.catcoc_heap_multicast_supported(device.index or 0)),
                                   group=group)
            if all(supported):
                use_mc = _setup_multicast(handle, rank, world, uid, group, bootstrap_timeout_ms)
            dist.barrier(group=group)
        ctx = ShmemContext(group, rank, world, device, handle, int(lib.catcoc_heap_bytes(handle)), use_mc)
        torch.cuda.synchronize(device)   # the heap is zeroed ...
        if world > 1:
            dist.barrier(group=group)    # ... on every rank before any peer may write into it
    except Exception:
        lib.catcoc_heap_destroy(handle)
        raise
    if make_default:
        global _default_ctx
        _default_ctx = ctx
    _live.add(ctx)
    return ctx


def default_context() -> ShmemContext:
    """The context created by the last ``init(make_default=True)``; created on demand for a
    single-process run."""
    global _default_ctx
    if _default_ctx is None:
        if dist.is_initialized() and dist.get_world_size() > 1:
            raise ShmemError("call mm_rs_with_catlass_b200.parallel.shmem.init() on every rank first")
        _default_ctx = init()
    return _default_ctx


_live: "weakref.WeakSet[ShmemContext]" = weakref.WeakSet()


@atexit.register
def _finalize_all() -> None:
    for ctx in list(_live):
        try:
            ctx._finalized or ctx.finalize(collective=False)
        except Exception:
            pass

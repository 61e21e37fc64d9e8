"""The split-K + one-shot all-reduce kernel (csrc/kernels/small_allreduce.cu) on ONE GPU, as rank 0
of a two-rank world whose "peer" heap is the rank's own memory: the peer-load sum, the epoch
bookkeeping, and the bounded wait (a stamp that nobody writes ends the launch with an error
status instead of a hang; the context stays usable). The real two- and four-rank runs are part
of tests/multi_gpu_worker.py (modes ``ops`` and ``mixed``)."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu

ROWS, COLS, SLICES = 96, 520, 3


def _setup(device, peer_stamped):
    from mm_rs_with_catlass_b200 import _native as N
    lib = N.lib()
    words = int(lib.catcoc_splitk_allreduce_flag_words(ROWS, COLS, 2))
    part_bytes = (ROWS * COLS * 2 + 255) // 256 * 256
    heap = torch.zeros(part_bytes + 4 * words, dtype=torch.uint8, device=device)
    flags = heap[part_bytes:].view(torch.int32)
    if peer_stamped:
        flags.view(-1, 2)[:, 1] = 1            # the "peer" (source 1) has stamped every chunk for epoch 1
    ctx = N.ShmemCtx()
    ctx.rank, ctx.W = 0, 2
    ctx.base[0] = ctx.base[1] = heap.data_ptr()  # the peer's copy is this rank's own copy
    ctx.mc_base = None
    g = torch.Generator(device=device)
    g.manual_seed(3)
    parts = torch.randn(SLICES, ROWS, COLS, device=device, generator=g)
    out = torch.full((ROWS, COLS), float("nan"), dtype=torch.bfloat16, device=device)
    state = torch.zeros(2, dtype=torch.int32, device=device)     # [0] epoch, [1] CTA counter
    status = torch.zeros(8, dtype=torch.int32, device=device)
    return lib, N, ctx, heap, parts, out, state, status, part_bytes


def _launch(lib, N, ctx, parts, out, state, status, part_bytes, timeout_ns, row0=0):
    stream = torch.cuda.current_stream(out.device).cuda_stream
    return lib.catcoc_splitk_allreduce(C.byref(ctx), parts.data_ptr(), SLICES, ROWS * COLS, ROWS, COLS, row0, out.shape[0],
                                       out.data_ptr(), out.stride(0), N.FMT_BF16, 0, part_bytes, 0, state.data_ptr(),
                                       state.data_ptr() + 4, status.data_ptr(), timeout_ns, C.c_void_p(stream))


def test_sum_over_ranks_by_peer_loads_and_epoch_advance(device):
    lib, N, ctx, heap, parts, out, state, status, part_bytes = _setup(device, peer_stamped=True)
    assert _launch(lib, N, ctx, parts, out, state, status, part_bytes, 2_000_000_000) == 0, N.last_error()
    torch.cuda.synchronize(device)
    assert status.tolist()[0] == 0
    assert state.tolist() == [1, 0]                                # epoch advanced, counter back at zero
    local = parts.sum(0).to(torch.bfloat16)                        # what the rank publishes
    assert torch.equal(heap[:ROWS * COLS * 2].view(torch.bfloat16).view(ROWS, COLS), local)
    expected = (local.float() * 2).to(torch.bfloat16)              # both "ranks" hold the same copy
    assert torch.equal(out, expected)


def test_a_stamp_that_never_comes_ends_the_launch_with_a_status(device):
    lib, N, ctx, heap, parts, out, state, status, part_bytes = _setup(device, peer_stamped=False)
    assert _launch(lib, N, ctx, parts, out, state, status, part_bytes, 20_000_000) == 0, N.last_error()   # 20 ms budget
    torch.cuda.synchronize(device)                                 # returns: the wait is bounded
    st = status.tolist()
    assert st[0] == 2, st                                          # STATUS_TIMEOUT_ARRIVE
    assert st[5] == 1                                              # the source that did not arrive
    assert state.tolist()[0] == 0                                  # the epoch stays: the launch did not complete
    # a latched status makes the next launch return at once, and clearing it makes the context usable again
    assert _launch(lib, N, ctx, parts, out, state, status, part_bytes, 20_000_000) == 0
    torch.cuda.synchronize(device)
    assert state.tolist()[0] == 0
    status.zero_()
    state.zero_()
    heap[part_bytes:].view(torch.int32).view(-1, 2)[:, 1] = 1
    assert _launch(lib, N, ctx, parts, out, state, status, part_bytes, 2_000_000_000) == 0
    torch.cuda.synchronize(device)
    assert status.tolist()[0] == 0 and state.tolist()[0] == 1 and torch.isfinite(out.float()).all()


def test_argument_checks(device):
    lib, N, ctx, heap, parts, out, state, status, part_bytes = _setup(device, peer_stamped=True)
    odd = torch.empty((ROWS, 521), dtype=torch.bfloat16, device=device)
    stream = torch.cuda.current_stream(device).cuda_stream
    rc = lib.catcoc_splitk_allreduce(C.byref(ctx), parts.data_ptr(), SLICES, ROWS * 521, ROWS, 521, 0, ROWS, odd.data_ptr(),
                                     521, N.FMT_BF16, 0, part_bytes, 0, state.data_ptr(), state.data_ptr() + 4,
                                     status.data_ptr(), 0, C.c_void_p(stream))
    assert rc == N.E_ALIGNMENT                                     # rows of whole 16-byte vectors only
    assert _launch(lib, N, ctx, parts, out[:10], state, status, part_bytes, 0, row0=ROWS - 5) == N.E_BAD_ARG   # rows past the end


def test_reduce_scatter_keeps_a_row_range(device):
    lib, N, ctx, heap, parts, out, state, status, part_bytes = _setup(device, peer_stamped=True)
    row0, rows = 37, 29                                            # a range that starts and ends inside chunks
    mine = torch.full((rows, COLS), float("nan"), dtype=torch.bfloat16, device=device)
    assert _launch(lib, N, ctx, parts, mine, state, status, part_bytes, 2_000_000_000, row0=row0) == 0, N.last_error()
    torch.cuda.synchronize(device)
    assert status.tolist()[0] == 0 and state.tolist()[0] == 1
    local = parts.sum(0).to(torch.bfloat16)
    assert torch.equal(mine, (local[row0:row0 + rows].float() * 2).to(torch.bfloat16))


def _gather_setup(device, peer_stamped, m=24, cols=520):
    from mm_rs_with_catlass_b200 import _native as N
    lib = N.lib()
    row_bytes = cols * 2
    words = int(lib.catcoc_small_allgather_flag_words(m, row_bytes, 2))
    g_bytes = (2 * m * row_bytes + 255) // 256 * 256
    heap = torch.zeros(g_bytes + 4 * words, dtype=torch.uint8, device=device)
    if peer_stamped:
        heap[g_bytes:].view(torch.int32).view(-1, 2)[:, 1] = 1
    ctx = N.ShmemCtx()
    ctx.rank, ctx.W = 0, 2
    ctx.base[0] = ctx.base[1] = heap.data_ptr()
    ctx.mc_base = None
    g = torch.Generator(device=device)
    g.manual_seed(5)
    wide = torch.randn(m, cols + 24, device=device, generator=g).to(torch.bfloat16)
    shard = wide[:, :cols]                                          # a pitch wider than the row
    state = torch.zeros(2, dtype=torch.int32, device=device)
    status = torch.zeros(8, dtype=torch.int32, device=device)
    return lib, N, ctx, heap, shard, state, status, g_bytes, m, cols


def _gather(lib, N, ctx, shard, state, status, g_bytes, m, cols, timeout_ns):
    stream = torch.cuda.current_stream(shard.device).cuda_stream
    return lib.catcoc_small_allgather(C.byref(ctx), shard.data_ptr(), shard.stride(0) * 2, m, cols * 2, 0, cols * 2, g_bytes, 0,
                                      state.data_ptr(), state.data_ptr() + 4, status.data_ptr(), timeout_ns,
                                      C.c_void_p(stream))


def test_gather_kernel_places_the_shard_and_advances_the_epoch(device):
    lib, N, ctx, heap, shard, state, status, g_bytes, m, cols = _gather_setup(device, peer_stamped=True)
    assert _gather(lib, N, ctx, shard, state, status, g_bytes, m, cols, 2_000_000_000) == 0, N.last_error()
    torch.cuda.synchronize(device)
    assert status.tolist()[0] == 0 and state.tolist() == [1, 0]
    gathered = heap[:2 * m * cols * 2].view(torch.bfloat16).view(2 * m, cols)
    assert torch.equal(gathered[:m], shard)                         # rank 0's rows
    assert torch.count_nonzero(gathered[m:]) == 0                   # the peer's rows are the peer's to write


def test_gather_kernel_gives_up_on_a_shard_that_never_comes(device):
    lib, N, ctx, heap, shard, state, status, g_bytes, m, cols = _gather_setup(device, peer_stamped=False)
    assert _gather(lib, N, ctx, shard, state, status, g_bytes, m, cols, 20_000_000) == 0, N.last_error()
    torch.cuda.synchronize(device)
    st = status.tolist()
    assert st[0] == 4 and st[5] == 1, st                            # STATUS_TIMEOUT_GATHER, source 1
    assert state.tolist()[0] == 0
    bad = shard[:, 1:]                                              # rows that do not start on 16 bytes
    stream = torch.cuda.current_stream(device).cuda_stream
    rc = lib.catcoc_small_allgather(C.byref(ctx), bad.data_ptr(), bad.stride(0) * 2, m, (cols - 8) * 2, 0, cols * 2, g_bytes, 0,
                                    state.data_ptr(), state.data_ptr() + 4, status.data_ptr(), 0, C.c_void_p(stream))
    assert rc == N.E_ALIGNMENT

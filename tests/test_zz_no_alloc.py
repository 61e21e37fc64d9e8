"""The allocation-free GEMM entry point (csrc/include/catcoc/no_alloc.h), called through its
exported C symbol the way a plug-in without an allocator would call it.

Such callers get fixed buffers from their host runtime and may not call cudaMalloc; the entry
point therefore pads unaligned operands into a scratch area built into the library image
instead of allocating one. The test checks its output against the regular entry point
(``catcoc.matmul``, which allocates its padded copies) on two calls in a row that share the
scratch: the second call uses smaller, different operands, so anything the first call left
behind would show up as a wrong result. This file sorts last so that a run that stops at the
first failure has already run every other test."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _call(lib, a, b, out, m, n, k, in_fmt, out_fmt, ta, tb):
    stream = torch.cuda.current_stream(out.device).cuda_stream
    return lib.catcoc_matmul_noalloc(C.c_void_p(a.data_ptr()), a.stride(0), C.c_void_p(b.data_ptr()), b.stride(0),
                                     C.c_void_p(out.data_ptr()), out.stride(0), m, n, k, in_fmt, out_fmt, int(ta),
                                     int(tb), C.c_void_p(stream))


def _status(lib):
    words = (C.c_uint32 * 8)()
    assert lib.catcoc_matmul_noalloc_status(words) == 0
    return list(words)


def test_noalloc_entry_matches_regular_entry_on_two_calls_in_a_row(device):
    import mm_rs_with_catlass_b200 as catcoc
    from mm_rs_with_catlass_b200 import _native as N
    from mm_rs_with_catlass_b200.utils.verify import assert_close
    lib = N.lib()
    # unaligned leading dimensions (K = 1030 bf16 -> 2060-byte rows; N = 1001), so both entry
    # points have to pad; the second call is smaller and must not see the first call's data
    cases = [(513, 1001, 1030, False, False), (200, 328, 250, False, True)]
    for i, (m, n, k, ta, tb) in enumerate(cases):
        g = torch.Generator(device=device)
        g.manual_seed(100 + i)
        a = torch.randn((m, k), device=device, generator=g).to(torch.bfloat16)
        b = (torch.randn((n, k) if tb else (k, n), device=device, generator=g) * 0.05).to(torch.bfloat16)
        expected = catcoc.matmul(a, b, trans_a=ta, trans_b=tb)            # regular entry point
        out = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=device)
        torch.cuda.synchronize(device)
        before = torch.cuda.memory_allocated(device)
        free_before = torch.cuda.mem_get_info(device)[0]                   # cudaMemGetInfo: sees every allocation
        rc = _call(lib, a, b, out, m, n, k, N.IN_BF16, N.FMT_BF16, ta, tb)
        assert rc == 0, N.last_error()
        torch.cuda.synchronize(device)
        assert torch.cuda.memory_allocated(device) == before               # no torch allocation either
        if i > 0:
            # By the second call every kernel of the path is loaded (the driver may take memory when it
            # loads one): the device's free memory must not move, whoever would have allocated.
            assert torch.cuda.mem_get_info(device)[0] == free_before
        assert _status(lib)[0] == 0
        # same kernel and operands as the regular entry point (which may pick another tile shape)
        assert_close(out, expected.float(), k=k, dtype=torch.bfloat16)
        assert_close(out, (a.float() @ (b.t() if tb else b).float()), k=k, dtype=torch.bfloat16)


def test_noalloc_entry_int8_and_size_limit(device):
    import mm_rs_with_catlass_b200 as catcoc
    from mm_rs_with_catlass_b200 import _native as N
    lib = N.lib()
    a = torch.randint(-127, 128, (100, 300), device=device, dtype=torch.int32).to(torch.int8)
    b = torch.randint(-127, 128, (300, 136), device=device, dtype=torch.int32).to(torch.int8)
    out = torch.empty((100, 136), dtype=torch.int32, device=device)
    assert _call(lib, a, b, out, 100, 136, 300, N.IN_S8, N.FMT_S32, False, False) == 0, N.last_error()
    torch.cuda.synchronize(device)
    assert torch.equal(out, catcoc.matmul(a, b))
    assert torch.equal(out.double(), a.double() @ b.double())
    # beyond the built-in scratch: refused with a clear message, nothing launched
    big_a = torch.empty((4096, 2050), dtype=torch.bfloat16, device=device)
    big_b = torch.empty((2050, 64), dtype=torch.bfloat16, device=device)
    big_o = torch.empty((4096, 64), dtype=torch.bfloat16, device=device)
    rc = _call(lib, big_a, big_b, big_o, 4096, 64, 2050, N.IN_BF16, N.FMT_BF16, False, False)
    assert rc == N.E_TOO_LARGE and "scratch" in N.last_error()
    assert _call(lib, a, b, out, 0, 136, 300, N.IN_S8, N.FMT_S32, False, False) == N.E_BAD_ARG

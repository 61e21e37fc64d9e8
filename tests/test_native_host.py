"""Host-side pieces of the native library that need no GPU: error reporting, fd passing over
abstract unix sockets (the bootstrap transport), and op-layer argument checks."""
import ctypes as C
import os
import subprocess
import sys

import pytest
import torch

from mm_rs_with_catlass_b200 import _native as N

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_loads_without_a_driver_and_reports_version():
    assert N.lib().catcoc_version() >= 100


def test_fd_passing_between_processes(tmp_path):
    name = ("catcoc-test-%d" % os.getpid()).encode()
    lib = N.lib()
    sock = N.check(lib.catcoc_fd_recv_open(name))
    payload = tmp_path / "payload.txt"
    payload.write_text("hello over SCM_RIGHTS")
    child = subprocess.run([sys.executable, "-c", (
        "import sys; sys.path.insert(0, %r)\n"
        "from mm_rs_with_catlass_b200 import _native as N\n"
        "import os\n"
        "fd = os.open(%r, os.O_RDONLY)\n"
        "N.check(N.lib().catcoc_fd_send(%r, fd, 7, 5000))\n") % (REPO, str(payload), name)],
        capture_output=True, text=True, timeout=120)
    assert child.returncode == 0, child.stderr
    tag = C.c_int(-1)
    fd = N.check(lib.catcoc_fd_recv(sock, 5000, C.byref(tag)))
    assert tag.value == 7
    assert os.read(fd, 64) == b"hello over SCM_RIGHTS"
    lib.catcoc_fd_close(fd)
    lib.catcoc_fd_close(sock)


def test_fd_recv_times_out_instead_of_hanging():
    lib = N.lib()
    sock = N.check(lib.catcoc_fd_recv_open(("catcoc-test-to-%d" % os.getpid()).encode()))
    tag = C.c_int()
    assert lib.catcoc_fd_recv(sock, 50, C.byref(tag)) == N.E_IO
    assert "timed out" in N.last_error()
    lib.catcoc_fd_close(sock)


def test_fd_send_to_a_missing_peer_fails_after_its_budget():
    r, w = os.pipe()
    assert N.lib().catcoc_fd_send(b"catcoc-test-nobody-listens", r, 0, 30) == N.E_IO
    os.close(r)
    os.close(w)


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the CPU-only error path")
def test_heap_create_without_gpu_is_a_clean_error():
    h = C.c_void_p()
    rc = N.lib().catcoc_heap_create(0, 0, 1, 1 << 20, C.byref(h))
    assert rc < 0 and N.last_error()
    with pytest.raises(N.NativeError):
        N.check(rc)
    assert N.lib().catcoc_heap_create(0, 3, 2, 1 << 20, C.byref(h)) == N.E_BAD_ARG


def test_ops_refuse_cpu_tensors_loudly():
    import mm_rs_with_catlass_b200 as catcoc
    a, b = torch.randn(8, 8).bfloat16(), torch.randn(8, 8).bfloat16()
    with pytest.raises(RuntimeError, match="CUDA"):
        catcoc.matmul(a, b)
    with pytest.raises(RuntimeError, match="CUDA"):
        catcoc.matmul_reduce_scatter(a, b)


def test_bench_reference_arm_prints_unavailable():
    import json
    out = subprocess.run([sys.executable, os.path.join(REPO, "bench.py"), "--impl", "reference"], capture_output=True,
                         text=True, timeout=120)
    assert out.returncode == 0
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and "unavailable" in line


def test_data_generators_are_rank_dependent_and_seeded():
    from mm_rs_with_catlass_b200.utils.data import matmul_inputs, quant_inputs
    a0, b0 = matmul_inputs(16, 8, 32, rank=0)
    a1, _ = matmul_inputs(16, 8, 32, rank=1)
    a0b, _ = matmul_inputs(16, 8, 32, rank=0)
    assert torch.equal(a0, a0b) and not torch.equal(a0, a1)
    x1, x2, s1, s2, bias = quant_inputs(8, 16, 32, rank=0)
    y1, _, t1, _, _ = quant_inputs(8, 16, 32, rank=1)
    assert not torch.equal(x1, y1) and torch.equal(s1, t1)          # scales describe global rows
    assert s1.min() >= 0.001 and s1.max() <= 0.02 and bias.dtype == torch.int32
    d = quant_inputs(4, 8, 16, debug=True)
    assert d[0].unique().tolist() == [1] and d[4].tolist() == list(range(1, 9))


def test_tensor_files_roundtrip_and_checker_exit_code(tmp_path):
    from mm_rs_with_catlass_b200.utils import io
    g = torch.randn(16, 24)
    for dt in (torch.bfloat16, torch.float16, torch.float32, torch.int8):
        t = (g * 10).to(dt)
        io.tensor_to_file(t, str(tmp_path / "t.bin"))
        assert torch.equal(io.tensor_from_file(str(tmp_path / "t.bin"), dt, (16, 24)), t)
    io.tensor_to_file(g.to(torch.bfloat16), str(tmp_path / "out.bin"))
    io.tensor_to_file(g, str(tmp_path / "gold.bin"))
    assert io.main([str(tmp_path / "out.bin"), str(tmp_path / "gold.bin"), "bf16", "16", "24", "512"]) == 0
    bad = g.clone()
    bad[0, 0] += 5
    io.tensor_to_file(bad.to(torch.bfloat16), str(tmp_path / "out.bin"))
    assert io.main([str(tmp_path / "out.bin"), str(tmp_path / "gold.bin"), "bf16", "16", "24", "512"]) == 1


def test_shape_lists_parse():
    from mm_rs_with_catlass_b200.tiling.tune import read_shapes
    d = os.path.join(REPO, "mm_rs_with_catlass_b200", "tiling", "shapes")
    ref = read_shapes(os.path.join(d, "reference_shapes.csv"))
    assert (16384, 27392, 4096, 0, 0) in ref and (8144, 5120, 1696, 0, 1) in ref and len(ref) == 9
    assert read_shapes(os.path.join(d, "reference_shapes.csv"), start_line=1, rows=2) == ref[1:3]


def test_few_row_collectives_size_their_stamps_and_check_arguments_without_a_gpu():
    lib = N.lib()
    # one stamp word per (chunk of 2048 elements, source)
    assert lib.catcoc_splitk_allreduce_flag_words(128, 8192, 4) == (128 * 8192 // 2048) * 4
    assert lib.catcoc_splitk_allreduce_flag_words(1, 128, 8) == 8
    # one per (chunk of 256 sixteen-byte vectors, source)
    assert lib.catcoc_small_allgather_flag_words(16, 8192 * 2, 8) == (16 * 1024 // 256) * 8
    assert lib.catcoc_small_allgather_flag_words(1, 16, 2) == 2
    ctx = N.ShmemCtx()
    ctx.rank, ctx.W = 0, 2
    dummy = C.c_void_p(4096)                     # never dereferenced: every call below is refused before a launch
    words = (C.c_uint32 * 8)()
    # a world of one has nothing to reduce
    one = N.ShmemCtx()
    one.rank, one.W = 0, 1
    assert lib.catcoc_splitk_allreduce(C.byref(one), dummy, 2, 128 * 256, 128, 256, 0, 128, dummy, 256, N.FMT_BF16, 0, 0, 0,
                                       words, words, words, 0, None) == N.E_BAD_ARG
    # rows outside the matrix, rows that are not whole 16-byte vectors, an fp32 output
    assert lib.catcoc_splitk_allreduce(C.byref(ctx), dummy, 2, 128 * 256, 128, 256, 100, 64, dummy, 256, N.FMT_BF16, 0, 0, 0,
                                       words, words, words, 0, None) == N.E_BAD_ARG
    assert lib.catcoc_splitk_allreduce(C.byref(ctx), dummy, 2, 128 * 250, 128, 250, 0, 128, dummy, 250, N.FMT_BF16, 0, 0, 0,
                                       words, words, words, 0, None) == N.E_ALIGNMENT
    assert lib.catcoc_splitk_allreduce(C.byref(ctx), dummy, 2, 128 * 256, 128, 256, 0, 128, dummy, 256, N.FMT_F32, 0, 0, 0,
                                       words, words, words, 0, None) == N.E_UNSUPPORTED
    assert "fp16 / bf16" in N.last_error()
    # gather: a row length or a pitch that is not a multiple of 16 bytes
    assert lib.catcoc_small_allgather(C.byref(ctx), dummy, 1040, 8, 1030, 0, 1040, 0, 0, words, words, words, 0, None) == N.E_ALIGNMENT
    assert lib.catcoc_small_allgather(C.byref(ctx), dummy, 1032, 8, 1024, 0, 1024, 0, 0, words, words, words, 0, None) == N.E_ALIGNMENT
    assert lib.catcoc_small_allgather(C.byref(ctx), dummy, 1024, 0, 1024, 0, 1024, 0, 0, words, words, words, 0, None) == N.E_BAD_ARG


def test_attention_entry_points_refuse_bad_arguments_without_a_gpu():
    lib = N.lib()
    dummy = C.c_void_p(4096)
    words = (C.c_uint32 * 8)()
    args = lambda d, hq, hk, sq, sk, causal, scale: (dummy, dummy, dummy, dummy, 1, hq, hk, sq, sk, d, N.FMT_BF16, causal, scale,
                                                     words, 0, None)
    assert lib.catcoc_flash_attention(*args(96, 2, 2, 16, 16, 0, 0.1)) == N.E_UNSUPPORTED      # head dimension
    assert lib.catcoc_flash_attention(*args(128, 3, 2, 16, 16, 0, 0.1)) == N.E_BAD_ARG         # heads do not divide
    assert lib.catcoc_flash_attention(*args(128, 2, 2, 16, 8, 1, 0.1)) == N.E_BAD_ARG          # causal with Sk < Sq
    assert lib.catcoc_flash_attention(*args(128, 2, 2, 16, 16, 0, -0.1)) == N.E_UNSUPPORTED    # the scale must be positive
    assert lib.catcoc_mla_workspace_bytes(4, 1, 16, 1) == 0
    assert lib.catcoc_mla_workspace_bytes(4, 2, 16, 3) == 3 * (4 * 2 * 16) * (512 + 2) * 4
    mla = lambda q_len, splits, ws: lib.catcoc_mla_decode(dummy, dummy, dummy, dummy, dummy, dummy, dummy, ws, 2, q_len, 16, 8, 4,
                                                          N.FMT_BF16, 0, 0.05, splits, words, 0, None)
    assert mla(5, 1, None) == N.E_UNSUPPORTED                                                  # 1 to 4 new tokens
    assert mla(1, 3, None) == N.E_BAD_ARG                                                      # slices need the workspace
    assert mla(1, 100, dummy) == N.E_BAD_ARG

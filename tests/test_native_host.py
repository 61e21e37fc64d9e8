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

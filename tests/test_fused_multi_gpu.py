"""Fused ops on 2 / 4 / 8 GPUs of one box: launches tests/multi_gpu_worker.py with one process
per GPU and checks every case it reports. Skipped where fewer GPUs are visible."""
import json
import os
import socket
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _run(world, mode, extra_env=None, timeout=900):
    env = dict(os.environ)
    env.setdefault("CATCOC_TIMEOUT_MS", "5000")
    env.update(extra_env or {})
    for attempt in range(3):
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(world),
               "--master-addr", "127.0.0.1", "--master-port", str(_free_port()),
               os.path.join(HERE, "multi_gpu_worker.py"), mode]
        proc = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env)
        # the port found free a moment ago can be taken by the time the rendezvous binds it
        if proc.returncode == 0 or "EADDRINUSE" not in proc.stderr:
            break
    cases = []
    for line in proc.stdout.splitlines():
        if line.startswith("{"):
            try:
                cases.append(json.loads(line))
            except ValueError:
                pass
    bad = [c for c in cases if not c["ok"]]
    assert proc.returncode == 0 and not bad, "failed cases: %s\nstdout tail:\n%s\nstderr tail:\n%s" % (
        bad[:10], proc.stdout[-2000:], proc.stderr[-3000:])
    return cases


@pytest.mark.parametrize("world", [2, 4, 8])
def test_fused_ops_match_goldens(world, gpu_count):
    if gpu_count < world:
        pytest.skip("needs %d GPUs" % world)
    cases = _run(world, "ops")
    assert len(cases) > 100


@pytest.mark.parametrize("world", [2, 4, 8])
def test_mixed_geometries_back_to_back(world, gpu_count):
    """Different tile geometries and ops alternate on one context with no synchronisation in
    between; every result is checked. On three or more GPUs this is the sequence in which stamp
    words shared between geometries used to be overwritten by a lagging rank."""
    if gpu_count < world:
        pytest.skip("needs %d GPUs" % world)
    _run(world, "mixed", {"CATCOC_TIMEOUT_MS": "2000"}, timeout=600)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_benchmark_shapes_match_goldens(world, gpu_count):
    """Every fused op at the benchmark shape (M = 8192, hidden 8192, FFN 28672 / W) with the tiling the
    chooser ships, plus the pull, TMA-push, multicast and peer-store variants, against fp32 goldens."""
    if gpu_count < world:
        pytest.skip("needs %d GPUs" % world)
    cases = _run(world, "bench_shapes", {"CATCOC_TIMEOUT_MS": "3000"}, timeout=900)
    assert len(cases) >= 13


def test_fused_ops_on_plain_peer_stores_without_nvls(gpu_count):
    if gpu_count < 2:
        pytest.skip("needs 2 GPUs")
    _run(2, "ops", {"CATCOC_TEST_NVLS": "0"})


def test_fused_ops_with_partial_tiles_pushed_by_tma_store(gpu_count):
    """The opt-in push path: bulk tensor stores into the owners' slabs, stamps one tile late."""
    if gpu_count < 2:
        pytest.skip("needs 2 GPUs")
    _run(2, "ops", {"CATCOC_PUSH_TMA": "1", "CATCOC_PULL": "0"})


def test_withheld_signal_becomes_an_error_status(gpu_count):
    if gpu_count < 2:
        pytest.skip("needs 2 GPUs")
    cases = _run(2, "withhold", {"NCCL_NVLS_ENABLE": "0"}, timeout=300)
    assert {c["case"] for c in cases} >= {"withheld_signal_detected", "recovers_after_reset"}


def test_shmem_primitives_and_switch_sum_numerics(gpu_count):
    """put / get / signal / wait_until over peer memory, multicast broadcast, and how far the
    in-switch bf16 sum (multimem.ld_reduce) is from the exact sum of its terms."""
    if gpu_count < 2:
        pytest.skip("needs 2 GPUs")
    cases = _run(2, "prims", timeout=300)
    assert {c["case"] for c in cases} >= {"shmem_get_reads_the_peer", "shmem_put_signal_wait"}

"""The golden ops on CPU over gloo with 2 ranks and rank-dependent data: plumbing of the
distributed goldens, including the fp16 [256,512] x [512,256] case."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from mm_rs_with_catlass_b200.ops import reference as ref
        from mm_rs_with_catlass_b200.utils.data import matmul_inputs, quant_inputs
        from mm_rs_with_catlass_b200.utils.verify import assert_close
        M, Nn, K = 256, 256, 512
        # every rank rebuilds every rank's inputs, so the expected value needs no communication
        ins = [matmul_inputs(M, Nn, K, r, torch.float16, seed=5) for r in range(world)]
        a, b = ins[rank]
        expect = sum(x.double() @ y.double() for x, y in ins).float()
        assert_close(ref.matmul_allreduce(a, b), expect, k=K * world, dtype=torch.float16, what="allreduce")
        rows = M // world
        assert_close(ref.matmul_reduce_scatter(a, b), expect[rank * rows:(rank + 1) * rows], k=K * world,
                     dtype=torch.float16, what="reduce_scatter")
        # transposed storage gives the same result
        assert torch.equal(ref.matmul_allreduce(a.t().contiguous(), b.t().contiguous(), trans_a=True, trans_b=True),
                           ref.matmul_allreduce(a, b))
        # all-gather: row block q of the output is A_q @ B_rank
        out, gathered = ref.allgather_matmul(a, b.t().contiguous().t())
        big = torch.cat([x for x, _ in ins], 0)
        assert torch.equal(gathered, big)
        assert_close(out, big.double() @ b.double(), k=K, dtype=torch.float16, what="allgather")
        # quantised: exact integers, bias once per rank
        qs = [quant_inputs(64, 96, 128, r, seed=9) for r in range(world)]
        x1, x2, s1, s2, bias = qs[rank]
        acc = sum(u.long() @ v.long() + bb.long()[None, :] for (u, v, _, _, bb) in qs)
        exp_q = (acc.double() * s2.double()[None, :] * s1.double()[:, None])[rank * 32:(rank + 1) * 32].float()
        got = ref.quant_matmul_reduce_scatter(x1, x2, s1, s2, bias, out_dtype=torch.float32)
        assert torch.allclose(got, exp_q, rtol=1e-5, atol=1e-6)
        q.put((rank, "ok"))
    except Exception as e:  # pragma: no cover - reported to the parent
        q.put((rank, repr(e)))
    finally:
        dist.destroy_process_group()


def test_goldens_over_gloo_world2():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert sorted(results) == [(0, "ok"), (1, "ok")], results

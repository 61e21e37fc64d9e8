"""Tiling sweep: measure every feasible candidate of a shape list and record the results.

    python -m torch.distributed.run --nproc-per-node W -m mm_rs_with_catlass_b200.tiling.tune \\
        --op matmul_reduce_scatter --shapes shapes.csv --out results.csv

``shapes.csv`` uses the reference's columns ``M,K,N,Transpose A,Transpose B``
(examples/dynamic_tiling/scripts/test_shapes.csv). Every candidate gets ``--warmup`` untimed
and ``--iters`` timed launches (10 and 3 by default, the reference's WARM_UP_TIMES and
PERF_TEST_CYCLE_TIMES, examples/dynamic_tiling/include/info.h:22-23), timed with CUDA events as
the max over ranks. Rows already present in ``--out`` are skipped, so an interrupted sweep
resumes; ``--best`` writes the arg-min table that the runtime chooser loads
(the reference does this offline in examples/dynamic_tiling/utils/get_best_res.py:43-83).
"""
from __future__ import annotations

import argparse
import csv
import os
import sys
from typing import List, Tuple

import torch
import torch.distributed as dist

from . import search
from .config import TilingConfig
from .table import Row, TilingTable, dtype_name


def read_shapes(path: str, start_line: int = 0, rows: int = 0) -> List[Tuple[int, int, int, int, int]]:
    out = []
    with open(path, newline="") as fh:
        rd = csv.reader(fh)
        for i, r in enumerate(rd):
            if not r or not r[0].strip() or not r[0].strip().lstrip("-").isdigit():
                continue  # header / blank
            vals = [int(x) for x in r[:5]] + [0] * (5 - len(r[:5]))
            out.append(tuple(vals[:5]))
    if start_line or rows:
        out = out[start_line:start_line + rows if rows else None]
    return out


def measure(fn, warmup: int, iters: int, device, group=None) -> float:
    """Microseconds per launch, device-timed, max over ranks."""
    from ..utils.timing import time_steps
    return 1e3 * time_steps(fn, iters, warmup, device, group)


def make_callable(op: str, m: int, k: int, n: int, trans_a: bool, trans_b: bool, dtype: torch.dtype, ctx, device,
                  t: TilingConfig):
    from ..ops import fused
    from ..ops.gemm import matmul
    from ..utils.data import matmul_inputs, quant_inputs
    rank, world = (ctx.rank, ctx.world) if ctx is not None else (0, 1)
    if op == "quant_matmul_reduce_scatter":
        x1, x2, s1, s2, bias = quant_inputs(m, n, k, rank, device, trans_b=trans_b)
        return lambda: fused.quant_matmul_reduce_scatter(x1, x2, s1, s2, bias, trans_b=trans_b, tiling=t, ctx=ctx)
    if op == "allgather_matmul":
        a, b = matmul_inputs(m // world, n, k, rank, dtype, device, trans_b=trans_b, b_std=0.02)
        out = torch.empty((m, n), dtype=dtype, device=device)
        return lambda: fused.allgather_matmul(a, b, trans_b=trans_b, out=out, tiling=t, ctx=ctx)
    a, b = matmul_inputs(m, n, k, rank, dtype, device, trans_a=trans_a, trans_b=trans_b, b_std=0.02)
    if op == "matmul_reduce_scatter":
        out = torch.empty((m // world, n), dtype=dtype, device=device)
        return lambda: fused.matmul_reduce_scatter(a, b, trans_a=trans_a, trans_b=trans_b, out=out, tiling=t, ctx=ctx)
    if op == "matmul_allreduce":
        return lambda: fused.matmul_allreduce(a, b, trans_a=trans_a, trans_b=trans_b, tiling=t, ctx=ctx)
    out = torch.empty((m, n), dtype=dtype, device=device)
    return lambda: matmul(a, b, trans_a=trans_a, trans_b=trans_b, out=out, tiling=t)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--op", required=True, choices=search.OPS)
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp16", "int8"])
    ap.add_argument("--shapes", required=True)
    ap.add_argument("--out", required=True)
    ap.add_argument("--best", default=None)
    ap.add_argument("--warmup", type=int, default=int(os.environ.get("WARM_UP_TIMES", "10")))
    ap.add_argument("--iters", type=int, default=int(os.environ.get("PERF_TEST_CYCLE_TIMES", "3")))
    ap.add_argument("--start-line", type=int, default=0)
    ap.add_argument("--collect-rows", type=int, default=0)
    ap.add_argument("--heap-gb", type=float, default=6.0)
    ap.add_argument("--bns", default="256,128,64", help="tile widths to try")
    ap.add_argument("--pairs", default="1,2", help="1 = single CTA tiles, 2 = 2-CTA tiles")
    ap.add_argument("--swizzles", default="4,8,16")
    ap.add_argument("--rounds", default="0", help="owner rounds to try (0 = default)")
    args = ap.parse_args(argv)

    from ..parallel import shmem
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    ctx = shmem.init(heap_bytes=int(args.heap_gb * (1 << 30)))
    dtype = {"bf16": torch.bfloat16, "fp16": torch.float16, "int8": torch.int8}[args.dtype]
    op = "quant_matmul_reduce_scatter" if (args.dtype == "int8" and args.op == "matmul_reduce_scatter") else args.op

    done = TilingTable.load(args.out) if os.path.exists(args.out) else TilingTable()
    for (m, k, n, ta, tb) in read_shapes(args.shapes, args.start_line, args.collect_rows):
        prob = search.Problem(op, m, n, k, world, args.dtype, bool(ta), bool(tb), bool(ctx.mc_base), ctx.heap_bytes)
        ints = lambda txt: tuple(int(x) for x in txt.split(",") if x != "")
        for t in search.candidates(prob, ints(args.bns), ints(args.pairs), ints(args.swizzles),
                                   rounds_space=ints(args.rounds)):
            row = Row(op, m, k, n, ta, tb, dtype_name(dtype), world, t, float("nan"))
            if done.has(row):
                continue
            fn = make_callable(op, m, k, n, bool(ta), bool(tb), dtype, ctx, device, t)
            us = measure(fn, args.warmup, args.iters, device)
            ctx.check("tune %s %dx%dx%d" % (op, m, k, n))
            row = Row(op, m, k, n, ta, tb, dtype_name(dtype), world, t, us)
            done.rows.append(row)
            if rank == 0:
                TilingTable.append_row(args.out, row)
                print("%s M=%d K=%d N=%d %s -> %.1f us" % (op, m, k, n, t, us), flush=True)
    if rank == 0 and args.best:
        TilingTable.load(args.out).best().save(args.best)
    ctx.finalize()
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())

"""Tiling sweep: measure every feasible candidate of a shape list and record the results.

    python -m torch.distributed.run --nproc-per-node W -m mm_rs_with_catlass_b200.tiling.tune \\
        --op matmul_reduce_scatter --shapes shapes.csv --out results.csv
    python -m torch.distributed.run --nproc-per-node W -m mm_rs_with_catlass_b200.tiling.tune \\
        --op all --shapes tiling/shapes/llm_tp.csv --out results_wW.csv         # every op, one process
    python -m mm_rs_with_catlass_b200.tiling.tune --merge results_w2.csv results_w4.csv results_w8.csv \\
        --best mm_rs_with_catlass_b200/tiling/best_tilings.csv                  # no GPU needed

With ``--op all`` a shape row ``M,K,N`` names the un-sharded layer: the row-parallel ops
(all-reduce, reduce-scatter, int8 reduce-scatter) run ``[M, K / W] x [K / W, N]``, the all-gather
op runs the column-parallel counterpart ``[M / W, N] x [N, K / W]`` of the same layer
(the reference's sweep script runs one op per invocation, examples/dynamic_tiling/scripts/run.sh:95-123).

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
    ap.add_argument("--op", default=None, choices=search.OPS + ("all",))
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp16", "int8"])
    ap.add_argument("--shapes", default=None)
    ap.add_argument("--out", default=None)
    ap.add_argument("--merge", nargs="+", default=None, metavar="CSV",
                    help="fold result files into the arg-min table given by --best and exit (runs without a GPU)")
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
    ap.add_argument("--pulls", default="0,1", help="0 = push partial tiles, 1 = pull through the switch")
    ap.add_argument("--comm-warps", default="0", help="communication / reducer warps per CTA to try (0 = all five)")
    ap.add_argument("--max-candidates", type=int, default=0, help="per shape and op (0 = all)")
    args = ap.parse_args(argv)

    if args.merge:
        if not args.best:
            ap.error("--merge needs --best")
        rows = []
        for path in args.merge:
            rows += TilingTable.load(path).rows
        best = TilingTable(rows).best()
        best.rows.sort(key=lambda r: (r.world, r.op, r.m, r.k, r.n))
        best.save(args.best)
        print("%d measured rows -> %d best rows in %s" % (len(rows), len(best.rows), args.best))
        return 0
    if not (args.op and args.shapes and args.out):
        ap.error("--op, --shapes and --out are required for a sweep")

    from ..parallel import shmem
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    ctx = shmem.init(heap_bytes=int(args.heap_gb * (1 << 30)))
    dtypes = {"bf16": torch.bfloat16, "fp16": torch.float16, "int8": torch.int8}
    if args.op == "all":
        jobs = [("matmul_allreduce", args.dtype), ("allgather_matmul", args.dtype), ("matmul_reduce_scatter", args.dtype),
                ("quant_matmul_reduce_scatter", "int8")]
    else:
        jobs = [("quant_matmul_reduce_scatter" if (args.dtype == "int8" and args.op == "matmul_reduce_scatter")
                 else args.op, args.dtype)]
    ints = lambda txt: tuple(int(x) for x in txt.split(",") if x != "")

    done = TilingTable.load(args.out) if os.path.exists(args.out) else TilingTable()
    for (m, k_full, n_full, ta, tb) in read_shapes(args.shapes, args.start_line, args.collect_rows):
        for op, dname in jobs:
            dtype = dtypes[dname]
            m_op, k, n = m, k_full, n_full
            if args.op == "all":
                # the row names the un-sharded layer [M, K] x [K, N]
                if k_full % world or m % world:
                    continue
                k, n = (n_full, k_full // world) if op == "allgather_matmul" else (k_full // world, n_full)
                if op == "matmul_allreduce" and m > 8192:
                    continue
                if op in ("allgather_matmul", "matmul_reduce_scatter") and m < 128:
                    continue
            prob = search.Problem(op, m_op, n, k, world, dname, bool(ta), bool(tb), bool(ctx.mc_base), ctx.heap_bytes)
            cands = search.candidates(prob, ints(args.bns), ints(args.pairs), ints(args.swizzles),
                                      rounds_space=ints(args.rounds), pull_space=ints(args.pulls),
                                      comm_warps_space=ints(args.comm_warps))
            if args.max_candidates:
                cands = cands[:args.max_candidates]
            for t in cands:
                row = Row(op, m_op, k, n, ta, tb, dtype_name(dtype), world, t, float("nan"))
                if done.has(row):
                    continue
                fn = make_callable(op, m_op, k, n, bool(ta), bool(tb), dtype, ctx, device, t)
                failed = None
                try:
                    us = measure(fn, args.warmup, args.iters, device)
                    ctx.check("tune %s %dx%dx%d" % (op, m_op, k, n))
                except RuntimeError as e:
                    failed = e
                # a failed wait shows up on some ranks only: agree, re-synchronise, skip the candidate
                from ..utils.timing import max_over_ranks
                if max_over_ranks(0.0 if failed is None else 1.0, device) > 0:
                    if rank == 0:
                        print("%s M=%d K=%d N=%d %s -> FAILED (%s)" % (op, m_op, k, n, t, failed), flush=True)
                    ctx.reset_after_error()
                    continue
                row = Row(op, m_op, k, n, ta, tb, dtype_name(dtype), world, t, us)
                done.rows.append(row)
                if rank == 0:
                    TilingTable.append_row(args.out, row)
                    print("%s M=%d K=%d N=%d %s -> %.1f us" % (op, m_op, k, n, t, us), flush=True)
            torch.cuda.empty_cache()
    if rank == 0 and args.best:
        TilingTable.load(args.out).best().save(args.best)
    ctx.finalize()
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())

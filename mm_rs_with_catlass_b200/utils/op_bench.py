"""Per-op latency table at the LLM tensor-parallel shapes: fused kernel vs cuBLAS + NCCL.

    python -m torch.distributed.run --nproc-per-node W -m mm_rs_with_catlass_b200.utils.op_bench [--out table.json]

For every op and M it prints one JSON line with the fused latency, the unfused latency
(torch.matmul / torch._int_mm followed by the NCCL collective), the speed-up, the achieved
TFLOP/s per GPU and the fraction of the roofline, where the roofline time is the slower of
(FLOPs / measured GEMM peak) and (bytes that must cross NVLink / measured link bandwidth).
All times are CUDA-event times, max over ranks, 10 warm-up + 20 timed launches.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

DEFAULT_HIDDEN, DEFAULT_FFN = 8192, 28672
LINK_GBS = 770.0          # measured peer copy per direction per GPU on this pool


def peaks():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))),
                        "MEASURED_PEAKS.json")
    try:
        with open(path) as fh:
            d = json.load(fh)
        return float(d["bf16_tflops"]), "measured"
    except (OSError, KeyError, ValueError):
        return 1590.0, "fallback"


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=None)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--ms", default="128,1024,8192,16384")
    ap.add_argument("--ops", default="ar,ag,rs,q")
    ap.add_argument("--hidden", type=int, default=DEFAULT_HIDDEN, help="N of the row-parallel ops, K of the all-gather op")
    ap.add_argument("--ffn", type=int, default=DEFAULT_FFN, help="split over the ranks: K_local = ffn / W")
    ap.add_argument("--trace", action="store_true",
                    help="after timing an op, run one more launch with the kernel's cycle counters on and print "
                         "them per CTA (FusedParams::trace in csrc/include/catcoc/params.h)")
    args = ap.parse_args(argv)
    HIDDEN, FFN = args.hidden, args.ffn

    import mm_rs_with_catlass_b200 as catcoc
    from mm_rs_with_catlass_b200.ops.baseline import Baseline
    from mm_rs_with_catlass_b200.utils import timing
    from mm_rs_with_catlass_b200.utils.data import matmul_inputs, quant_inputs

    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    ctx = catcoc.init(heap_bytes=int(os.environ.get("CATCOC_HEAP_BYTES", 8 << 30)))
    base = Baseline()
    W = world
    peak_tflops, peak_src = peaks()
    rows = []

    def record(op, M, fused_fn, base_fn, flops_rank, link_bytes, peak=peak_tflops):
        t_f = timing.time_steps(fused_fn, args.iters, args.warmup, dev)
        ctx.check(op)
        t_b = timing.time_steps(base_fn, args.iters, args.warmup, dev)
        roof_ms = max(flops_rank / (peak * 1e12), link_bytes / (LINK_GBS * 1e9)) * 1e3
        row = {"op": op, "W": W, "M": M, "fused_us": 1e3 * t_f, "cublas_nccl_us": 1e3 * t_b, "speedup": t_b / t_f,
               "tflops_per_gpu": flops_rank / (t_f * 1e-3) / 1e12, "roofline_us": 1e3 * roof_ms,
               "roofline_frac": roof_ms / t_f, "peak_source": peak_src}
        if args.trace:
            from mm_rs_with_catlass_b200.utils.gemm_probe import TRACE_NAMES
            tr = torch.zeros(16, dtype=torch.int64, device=dev)
            ctx.trace = tr
            ctx.plans.clear()          # the counters' address is part of the argument block
            fused_fn()
            torch.cuda.synchronize()
            ctx.trace = None
            ctx.plans.clear()
            row["cycles_per_cta"] = {n: round(v / 148) for n, v in zip(TRACE_NAMES, tr.tolist())}
        rows.append(row)
        if rank == 0:
            print(json.dumps(row), flush=True)

    kf = FFN // W
    for M in [int(x) for x in args.ms.split(",")]:
        if "ar" in args.ops and M <= 8192:
            a, b = matmul_inputs(M, HIDDEN, kf, rank, torch.bfloat16, dev, seed=1, b_std=0.02)
            out = torch.empty((M, HIDDEN), dtype=torch.bfloat16, device=dev)
            S = M * HIDDEN * 2
            record("matmul_allreduce", M, lambda: catcoc.matmul_allreduce(a, b),
                   lambda: base.matmul_allreduce(a, b, out=out), 2.0 * M * HIDDEN * kf, 2.0 * (W - 1) / W * S)
            del a, b, out
        if M % W == 0 and M >= 1024:
            if "ag" in args.ops:
                a, b = matmul_inputs(M // W, kf, HIDDEN, rank, torch.bfloat16, dev, seed=2, b_std=0.02)
                out = torch.empty((M, kf), dtype=torch.bfloat16, device=dev)
                record("allgather_matmul", M, lambda: catcoc.allgather_matmul(a, b, out=out),
                       lambda: base.allgather_matmul(a, b, out=out), 2.0 * M * HIDDEN * kf,
                       (W - 1) / W * M * HIDDEN * 2)
                del a, b, out
            if "rs" in args.ops and W > 1:
                a, b = matmul_inputs(M, HIDDEN, kf, rank, torch.bfloat16, dev, seed=3, b_std=0.02)
                out = torch.empty((M // W, HIDDEN), dtype=torch.bfloat16, device=dev)
                record("matmul_reduce_scatter", M, lambda: catcoc.matmul_reduce_scatter(a, b, out=out),
                       lambda: base.matmul_reduce_scatter(a, b, out=out), 2.0 * M * HIDDEN * kf,
                       (W - 1) / W * M * HIDDEN * 2)
                del a, b, out
        if "q" in args.ops and M % W == 0 and W > 1:
            x1, x2, s1, s2, bias = quant_inputs(M, HIDDEN, kf, rank, dev, seed=4)
            record("quant_matmul_reduce_scatter", M,
                   lambda: catcoc.quant_matmul_reduce_scatter(x1, x2, s1, s2, bias),
                   lambda: base.quant_matmul_reduce_scatter(x1, x2, s1, s2, bias), 2.0 * M * HIDDEN * kf,
                   (W - 1) / W * M * HIDDEN * 4, peak=2.0 * peak_tflops)
            del x1, x2
        torch.cuda.empty_cache()
    if rank == 0 and args.out:
        with open(args.out, "w") as fh:
            json.dump(rows, fh, indent=1)
    ctx.finalize()
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())

"""Per-op latency table at the LLM tensor-parallel shapes: fused kernel vs cuBLAS + NCCL.

    python -m torch.distributed.run --nproc-per-node W -m mm_rs_with_catlass_b200.utils.op_bench [--out table.json]

For every op and M it prints one JSON line with the fused latency, the unfused latency
(torch.matmul / torch._int_mm followed by the NCCL collective), the speed-up, the achieved
TFLOP/s per GPU and the fraction of the roofline, where the roofline time is the slower of
(FLOPs / measured GEMM peak) and (bytes that must cross NVLink / measured link bandwidth).
All times are CUDA-event times, max over ranks, 10 warm-up + 20 timed launches.

``--variants`` times the fused op once per named variant of the chooser's tiling (A/B runs in one
process): ``default`` (the chooser's pick), ``push`` (partial tiles pushed to the owner, shard sent
peer by peer), ``pull`` (partials summed through the switch, shard sent by multicast), ``pair`` /
``single`` (2-CTA or single-CTA tiles), ``cwN`` (N communication warps), ``bnN`` (tile width),
``tma`` (pushes by TMA stores), joined with ``+`` (``pull+pair+cw3``).
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
    ap.add_argument("--ops", default="ar,ag,rs,q", help="ar, ag, rs, q (int8), mx (block-scaled fp8)")
    ap.add_argument("--variants", default="default")
    ap.add_argument("--table", default=None,
                    help="append every measured (shape, tiling, time) as a row of a tiling table CSV "
                         "(tiling/table.py); `python -m mm_rs_with_catlass_b200.tiling.tune --merge` folds such "
                         "files into the table the chooser loads")
    ap.add_argument("--hidden", type=int, default=DEFAULT_HIDDEN, help="N of the row-parallel ops, K of the all-gather op")
    ap.add_argument("--ffn", type=int, default=DEFAULT_FFN, help="split over the ranks: K_local = ffn / W")
    ap.add_argument("--shapes-csv", default=None,
                    help="rows M,K,N of un-sharded layers (the reference's shape files, e.g. "
                         "tiling/shapes/reference_shapes.csv) instead of --ms / --hidden / --ffn: the row-parallel ops "
                         "run [M, K / W] x [K / W, N], the all-gather op [M / W, N] x [N, K / W]; rows whose K or M do "
                         "not divide by the world size are skipped")
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

    from mm_rs_with_catlass_b200.tiling.chooser import choose

    def variant_tiling(op, m, n, k, dtype, variant):
        """The chooser's tiling with the overrides the variant name spells out (None = leave it to the op)."""
        if variant == "default":
            return None
        t = choose(op, m, n, k, W, dtype)
        for part in variant.split("+"):
            if part in ("push", "pull") and dtype == torch.int8:
                continue      # int32 partial tiles are always pushed
            if part == "push":
                t = t.with_(pull=0, use_multicast=(op == "matmul_allreduce" and t.use_multicast))
            elif part == "pull":
                t = t.with_(pull=1, use_multicast=True)
            elif part == "tma":
                t = t.with_(push_tma=1)
            elif part == "pair":
                t = t.with_(cta_pair=2, bn=max(128, t.effective_bn))
            elif part == "single":
                t = t.with_(cta_pair=1)
            elif part.startswith("cw"):
                t = t.with_(comm_warps=int(part[2:]))
            elif part.startswith("bn"):
                t = t.with_(bn=int(part[2:]))
            elif part.startswith("rounds"):
                t = t.with_(rounds=int(part[6:]))
            elif part.startswith("swz"):
                t = t.with_(swizzle=int(part[3:]))
            elif part != "default":
                raise SystemExit("unknown variant part %r" % part)
        return t

    variants = [v for v in args.variants.split(",") if v]
    base_cache = {}
    shape_of = {}
    layer_of = {}
    layer_now = [None]

    def record(op, M, fused_of, base_fn, flops_rank, link_bytes, peak=peak_tflops, shape=None, dtype=torch.bfloat16):
        """``fused_of(tiling)`` returns the callable of the fused op with that tiling."""
        shape_of[(op, M)] = shape
        layer_of[(op, M)] = layer_now[0]
        for variant in variants:
            tiling = variant_tiling(op, *shape, dtype, variant) if shape else None
            if tiling is None and shape and args.table:
                tiling = choose(op, *shape, W, dtype)      # record what the default resolved to
            err = None
            try:
                fused_fn = fused_of(tiling)
                t_f = timing.time_steps(fused_fn, args.iters, args.warmup, dev)
                ctx.check("%s M=%d %s" % (op, M, variant))
            except (RuntimeError, ValueError) as e:
                err = e
            # a failed wait shows up on some ranks only: agree before anybody carries on
            failed = timing.max_over_ranks(0.0 if err is None else 1.0, dev) > 0
            if failed:
                print(json.dumps({"op": op, "W": W, "M": M, "variant": variant, "rank": rank,
                                  "error": str(err)[:300] if err is not None else "failed on another rank"}), flush=True)
                ctx.reset_after_error()
                continue
            if (op, M, layer_now[0]) not in base_cache:
                base_cache[(op, M, layer_now[0])] = timing.time_steps(base_fn, args.iters, args.warmup, dev)
            t_b = base_cache[(op, M, layer_now[0])]
            one_record(op, M, variant, tiling, fused_fn, t_f, t_b, flops_rank, link_bytes, peak)

    def one_record(op, M, variant, tiling, fused_fn, t_f, t_b, flops_rank, link_bytes, peak):
        roof_ms = max(flops_rank / (peak * 1e12), link_bytes / (LINK_GBS * 1e9)) * 1e3
        row = {"op": op, "W": W, "M": M, "N": layer_now[0][0], "K_total": layer_now[0][1], "variant": variant, "fused_us": 1e3 * t_f, "cublas_nccl_us": 1e3 * t_b,
               "speedup": t_b / t_f, "tflops_per_gpu": flops_rank / (t_f * 1e-3) / 1e12, "roofline_us": 1e3 * roof_ms,
               "roofline_frac": roof_ms / t_f, "peak_source": peak_src,
               "fallbacks": dict(ctx.fallbacks)}
        if tiling is not None:
            row["tiling"] = {k: v for k, v in tiling.to_dict().items()
                             if k in ("bn", "cta_pair", "swizzle", "rounds", "pull", "use_multicast", "comm_warps", "seg_dim")}
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
            if args.table and tiling is not None and shape_of.get((op, M)) is not None:
                from mm_rs_with_catlass_b200.tiling.table import Row, TilingTable
                m_, n_, k_ = shape_of[(op, M)]
                TilingTable.append_row(args.table, Row(op, m_, k_, n_, 0, 0, "int8" if "quant" in op else "bf16", W,
                                                       tiling, 1e3 * t_f, 1e3 * t_b))

    if args.shapes_csv:
        from mm_rs_with_catlass_b200.tiling.tune import read_shapes
        layers = [(m, k, n) for (m, k, n, ta, tb) in read_shapes(args.shapes_csv)
                  if k % W == 0 and m % W == 0 and (k // W) % 8 == 0 and n % 8 == 0 and m >= 128]
    else:
        layers = [(int(x), FFN, HIDDEN) for x in args.ms.split(",")]
    for (M, FFN, HIDDEN) in layers:
        kf = FFN // W
        layer_now[0] = (HIDDEN, FFN)
        if "ar" in args.ops and (M <= 8192 or args.shapes_csv):
            a, b = matmul_inputs(M, HIDDEN, kf, rank, torch.bfloat16, dev, seed=1, b_std=0.02)
            out = torch.empty((M, HIDDEN), dtype=torch.bfloat16, device=dev)
            S = M * HIDDEN * 2
            # bytes on the busiest direction of one GPU: S with in-switch reduction + multicast, else the
            # two-shot exchange 2 (W-1)/W S
            ar_bytes = S if ctx.mc_base else 2.0 * (W - 1) / W * S
            record("matmul_allreduce", M, lambda t: (lambda: catcoc.matmul_allreduce(a, b, tiling=t)),
                   lambda: base.matmul_allreduce(a, b, out=out), 2.0 * M * HIDDEN * kf, ar_bytes,
                   shape=(M, HIDDEN, kf))
            del a, b, out
        if M % W == 0 and M >= 128:
            if "ag" in args.ops:
                a, b = matmul_inputs(M // W, kf, HIDDEN, rank, torch.bfloat16, dev, seed=2, b_std=0.02)
                out = torch.empty((M, kf), dtype=torch.bfloat16, device=dev)
                record("allgather_matmul", M, lambda t: (lambda: catcoc.allgather_matmul(a, b, out=out, tiling=t)),
                       lambda: base.allgather_matmul(a, b, out=out), 2.0 * M * HIDDEN * kf,
                       (W - 1) / W * M * HIDDEN * 2, shape=(M, kf, HIDDEN))
                del a, b, out
            if "rs" in args.ops and W > 1:
                a, b = matmul_inputs(M, HIDDEN, kf, rank, torch.bfloat16, dev, seed=3, b_std=0.02)
                out = torch.empty((M // W, HIDDEN), dtype=torch.bfloat16, device=dev)
                record("matmul_reduce_scatter", M,
                       lambda t: (lambda: catcoc.matmul_reduce_scatter(a, b, out=out, tiling=t)),
                       lambda: base.matmul_reduce_scatter(a, b, out=out), 2.0 * M * HIDDEN * kf,
                       (W - 1) / W * M * HIDDEN * 2, shape=(M, HIDDEN, kf))
                del a, b, out
        if "q" in args.ops and M % W == 0 and W > 1:
            x1, x2, s1, s2, bias = quant_inputs(M, HIDDEN, kf, rank, dev, seed=4)
            record("quant_matmul_reduce_scatter", M,
                   lambda t: (lambda: catcoc.quant_matmul_reduce_scatter(x1, x2, s1, s2, bias, tiling=t)),
                   lambda: base.quant_matmul_reduce_scatter(x1, x2, s1, s2, bias), 2.0 * M * HIDDEN * kf,
                   (W - 1) / W * M * HIDDEN * 4, peak=2.0 * peak_tflops, shape=(M, HIDDEN, kf), dtype=torch.int8)
            del x1, x2
        if "mx" in args.ops and M % (128 * W) == 0 and hasattr(torch, "float8_e4m3fn"):
            # block-scaled fp8 row-parallel linear + reduce-scatter; the unfused arm is a bf16 cuBLAS GEMM on
            # the dequantised operands (dequantised outside the timed region) + NCCL reduce-scatter
            g = torch.Generator(device=dev)
            g.manual_seed(50 + rank)
            aq, sa = catcoc.quantize_mxf8(torch.randn(M, kf, device=dev, generator=g))
            bq, sb = catcoc.quantize_mxf8(torch.randn(HIDDEN, kf, device=dev, generator=g) * 0.02)
            pa, pb = catcoc.pack_scales(sa), catcoc.pack_scales(sb)
            a16 = catcoc.dequantize_mxf8(aq, sa).to(torch.bfloat16)
            b16 = catcoc.dequantize_mxf8(bq, sb).to(torch.bfloat16).t().contiguous()
            del sa, sb
            outm = torch.empty((M // W, HIDDEN), dtype=torch.bfloat16, device=dev)
            record("mxf8_matmul_reduce_scatter", M,
                   lambda t: (lambda: catcoc.mxf8_matmul_reduce_scatter(aq, pa, bq, pb, out=outm, tiling=t)),
                   lambda: base.matmul_reduce_scatter(a16, b16, out=outm if W > 1 else None), 2.0 * M * HIDDEN * kf,
                   (W - 1) / W * M * HIDDEN * 2, peak=2.0 * peak_tflops)
            del aq, bq, pa, pb, a16, b16, outm
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

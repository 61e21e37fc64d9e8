#!/usr/bin/env python
"""Headline benchmark: the fused ops at the LLM tensor-parallel shapes, against cuBLAS + NCCL.

One "step" runs the three bf16 fused ops of a tensor-parallel block once each at M = 8192
(hidden 8192, FFN 28672, operands sharded over the N GPUs exactly as the op configs say):

    allgather_matmul       A shard [M/W, 8192]   x  B [8192, 28672/W]
    matmul_reduce_scatter  A [M, 28672/W]        x  B [28672/W, 8192]
    matmul_allreduce       A [M, 28672/W]        x  B [28672/W, 8192]

The total work is fixed as N grows (strong scaling); ``value`` is the whole-job rate
(FLOPs of the three full-size GEMMs / time of the slowest rank). The quantised
matmul_reduce_scatter is timed separately and reported under ``ops``.

In the default arm the unfused pipeline (torch.matmul + NCCL) is timed in the same process, on
the same box and clock state, in alternation with the fused kernels (A B A B), for the step,
for every op and for the end-to-end block; ``vs_baseline`` is the ratio of the two step rates.

Arms (``--impl``):
    ours       the fused kernels of this repository (default)
    baseline   the same maths as torch.matmul followed by the NCCL collective, alone
    reference  the Ascend reference itself: it cannot be built for this machine, so this arm
               prints an ``unavailable`` line

Launch: ``python bench.py`` (1 GPU) or
``python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 bench.py --gpus N``.

Whatever goes wrong, the LAST line a rank prints is one JSON object: the result, or
``{"impl": ..., "error": ..., "rank": r, "status": [8 words of the device status block]}``.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
import traceback

REPO = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, REPO)

HIDDEN, FFN, M_DEFAULT = 8192, 28672, 8192
METRIC = "fused_tp_ops_tflops"

# a device-side wait that ran out of time costs this much, once (later launches return at once)
os.environ.setdefault("CATCOC_TIMEOUT_MS", "2000")


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "baseline", "reference"])
    ap.add_argument("--m", type=int, default=M_DEFAULT)
    ap.add_argument("--no-quant", action="store_true", help="skip the int8 op in the per-op table")
    ap.add_argument("--no-e2e", action="store_true")
    return ap.parse_args()


def reference_unavailable():
    print(json.dumps({
        "impl": "reference",
        "unavailable": "the reference is Ascend C++ (bisheng/CANN + external SHMEM library) with no setup.py or "
                       "pyproject.toml: pip reports \"Neither 'setup.py' nor 'pyproject.toml' found\" and no part "
                       "of it compiles for CUDA; the measured baseline is --impl baseline (cuBLAS + NCCL)",
    }))


class _State:
    """What the error line needs, filled in as the run proceeds."""
    ctx = None
    rank = 0
    impl = "ours"
    phase = "start"


def run(args) -> int:
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    _State.rank, _State.impl = rank, args.impl
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("--gpus %d needs torch.distributed.run with --nproc-per-node %d" % (args.gpus, args.gpus))
        args.gpus = world
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        dist.init_process_group("nccl", device_id=dev)

    import mm_rs_with_catlass_b200 as catcoc
    from mm_rs_with_catlass_b200.ops.baseline import Baseline
    from mm_rs_with_catlass_b200.ops import _common as op_common
    from mm_rs_with_catlass_b200.utils import timing
    from mm_rs_with_catlass_b200.utils.data import matmul_inputs, quant_inputs
    from mm_rs_with_catlass_b200.models.tp_mlp import TPMLP, TPMLPConfig

    # Clocks and throttle reasons of this rank's GPU, sampled from here to the end of the run (every
    # region below is a timed one; on 8 GPUs the headline region alone is shorter than nvidia-smi's
    # start-up). Only samples taken under load enter the median.
    sampler = timing.ClockSampler(gpu_index=local_rank, period_ms=100).start() if rank == 0 else None
    W, M = world, args.m
    if M % max(W, 1) or FFN % W:
        raise SystemExit("M and FFN must divide by the number of GPUs")
    ours = args.impl == "ours"
    ctx = catcoc.init(heap_bytes=int(os.environ.get("CATCOC_HEAP_BYTES", 6 << 30))) if ours else None
    _State.ctx = ctx
    base = Baseline()

    def check(what):
        _State.phase = what
        if ours:
            ctx.check(what)
            if W == 1:
                from mm_rs_with_catlass_b200.ops._common import local_status, raise_on_status
                raise_on_status(local_status(dev), what)

    # ---- operands (synthetic, seeded per rank; weights random-init) ----
    kf = FFN // W
    a_rs, b_rs = matmul_inputs(M, HIDDEN, kf, rank, torch.bfloat16, dev, seed=1, b_std=0.02)      # [M, F/W] x [F/W, H]
    a_ag, b_ag = matmul_inputs(M // W, kf, HIDDEN, rank, torch.bfloat16, dev, seed=2, b_std=0.02)  # [M/W, H] x [H, F/W]
    out_rs = torch.empty((M // W, HIDDEN), dtype=torch.bfloat16, device=dev)
    out_ag = torch.empty((M, kf), dtype=torch.bfloat16, device=dev)
    out_ar = torch.empty((M, HIDDEN), dtype=torch.bfloat16, device=dev)

    fused_ops = {
        "allgather_matmul": lambda: catcoc.allgather_matmul(a_ag, b_ag, out=out_ag)[0],
        "matmul_reduce_scatter": lambda: catcoc.matmul_reduce_scatter(a_rs, b_rs, out=out_rs),
        # the all-reduce result stays in the symmetric heap (no copy)
        "matmul_allreduce": lambda: catcoc.matmul_allreduce(a_rs, b_rs, out=out_ar if W == 1 else None),
    }
    base_ops = {
        "allgather_matmul": lambda: base.allgather_matmul(a_ag, b_ag, out=out_ag)[0],
        "matmul_reduce_scatter": lambda: base.matmul_reduce_scatter(a_rs, b_rs, out=out_rs if W > 1 else None),
        "matmul_allreduce": lambda: base.matmul_allreduce(a_rs, b_rs, out=out_ar),
    }
    mine = fused_ops if ours else base_ops
    names = ["allgather_matmul", "matmul_reduce_scatter", "matmul_allreduce"]

    def step_of(table):
        fns = [table[n] for n in names]

        def step():
            for f in fns:
                f()
        return step

    step = step_of(mine)
    flops_one = 2.0 * M * HIDDEN * FFN          # whole-job FLOPs of one of the three ops
    flops_step = 3.0 * flops_one

    def launches_now():
        # launches of this repository's GEMM kernel so far (fused ops and, on one GPU, local GEMMs)
        return op_common.launch_count()

    # ---- headline: K steps, device-timed, max over ranks ----
    _State.phase = "warm-up"
    for _ in range(max(args.warmup, 3)):
        step()
    timing.sync_all(dev)
    check("warm-up")
    launches0 = launches_now() if ours else 0
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    _State.phase = "timed steps"
    t_host0 = time.perf_counter()
    start.record()
    for _ in range(args.steps):
        step()
    stop.record()
    timing.sync_all(dev)
    host_s = time.perf_counter() - t_host0
    ms_step = timing.max_over_ranks(start.elapsed_time(stop) / args.steps, dev)
    launches = (launches_now() - launches0) if ours else 0
    check("timed steps")
    value = flops_step / (ms_step * 1e-3) / 1e12

    # ---- the unfused pipeline in the same process: step and per-op table, fused and unfused
    # timed in alternation (A B A B) so that neither arm always runs on the hotter chip ----
    def t(fn, n):
        return timing.time_steps(fn, n, 3, dev)

    def abab(fn_a, fn_b, n):
        n = max(3, n // 2)
        ta, tb = [], []
        for _ in range(2):
            ta.append(t(fn_a, n))
            tb.append(t(fn_b, n))
        return sum(ta) / 2, sum(tb) / 2

    ops = {}
    base_step_ms = None
    if ours:
        _State.phase = "step, fused and unfused in alternation"
        ms_f, base_step_ms = abab(step, step_of(base_ops), args.steps)
        check("step A/B")
        ops["step"] = {"ms": ms_f, "cublas_nccl_ms": base_step_ms, "speedup_vs_cublas_nccl": base_step_ms / ms_f}
    for name in names:
        _State.phase = name
        if ours:
            ms, ms_b = abab(fused_ops[name], base_ops[name], args.steps)
            ops[name] = {"ms": ms, "tflops": flops_one / (ms * 1e-3) / 1e12, "cublas_nccl_ms": ms_b,
                         "speedup_vs_cublas_nccl": ms_b / ms}
            check(name)
        else:
            ms = t(base_ops[name], max(5, args.steps // 2))
            ops[name] = {"ms": ms, "tflops": flops_one / (ms * 1e-3) / 1e12}
    if not args.no_quant:
        _State.phase = "quant_matmul_reduce_scatter"
        x1, x2, s1, s2, bias = quant_inputs(M, HIDDEN, kf, rank, dev, seed=3)
        base_q = lambda: base.quant_matmul_reduce_scatter(x1, x2, s1, s2, bias)
        if ours:
            ms_q, ms_b = abab(lambda: catcoc.quant_matmul_reduce_scatter(x1, x2, s1, s2, bias), base_q, args.steps)
            ops["quant_matmul_reduce_scatter"] = {"ms": ms_q, "tops": flops_one / (ms_q * 1e-3) / 1e12,
                                                  "cublas_nccl_ms": ms_b, "speedup_vs_cublas_nccl": ms_b / ms_q}
            check("quant_matmul_reduce_scatter")
        else:
            ms_q = t(base_q, max(5, args.steps // 2))
            ops["quant_matmul_reduce_scatter"] = {"ms": ms_q, "tops": flops_one / (ms_q * 1e-3) / 1e12}

    # ---- end to end through the public model API: pinned host input -> device -> block -> loss -> host.
    # Every step copies its own input shard from pinned host memory (on a copy stream, one step
    # ahead of the compute, as a data loader does) and reads its own scalar result back. ----
    def end_to_end():
        _State.phase = "end to end"
        if ours:
            mlp = TPMLP(TPMLPConfig(hidden=HIDDEN, ffn=FFN), ctx, dev)
            w_up, w_down = mlp.w_up, mlp.w_down
        else:
            mlp, w_up, w_down = None, b_ag, b_rs
        x_host = [torch.randn((M // W, HIDDEN), dtype=torch.float32).to(torch.bfloat16).pin_memory() for _ in range(2)]
        x_dev = [torch.empty_like(x_host[0], device=dev) for _ in range(2)]
        loss_host = torch.zeros(2, dtype=torch.float32).pin_memory()
        copy_stream = torch.cuda.Stream(device=dev)
        ready = [torch.cuda.Event() for _ in range(2)]      # input i has landed
        consumed = [torch.cuda.Event() for _ in range(2)]   # input buffer i may be overwritten
        read = [torch.cuda.Event() for _ in range(2)]       # loss slot i holds its step's value

        def base_block(x):
            h = base.allgather_matmul(x, w_up)[0]
            return base.matmul_reduce_scatter(torch.nn.functional.gelu(h, approximate="tanh"), w_down)

        def make_e2e(block):
            state = {"i": 0, "loss": 0.0}

            def prefetch(i):
                s = i & 1
                with torch.cuda.stream(copy_stream):
                    copy_stream.wait_event(consumed[s])
                    x_dev[s].copy_(x_host[s], non_blocking=True)
                    ready[s].record(copy_stream)

            def e2e_step():
                i = state["i"]
                s = i & 1
                if i == 0:
                    prefetch(0)
                prefetch(i + 1)                       # the next step's input travels while this step computes
                cur = torch.cuda.current_stream()
                cur.wait_event(ready[s])
                y = block(x_dev[s])
                consumed[s].record(cur)
                loss_host[s:s + 1].copy_(y.float().mean().reshape(1), non_blocking=True)
                read[s].record(cur)
                if i > 0:                             # read the previous step's result: no bubble on the device
                    read[s ^ 1].synchronize()
                    state["loss"] = float(loss_host[s ^ 1])
                state["i"] = i + 1
                return state["loss"]

            def drain():
                torch.cuda.synchronize(dev)
                state["i"] = 0
                for e in consumed:
                    e.record(torch.cuda.current_stream())
            return e2e_step, drain

        def time_e2e(block, n):
            fn, drain = make_e2e(block)
            drain()
            ms = timing.time_steps(fn, n, max(args.warmup, 3), dev)
            drain()
            return ms

        flops_e2e = 2.0 * flops_one  # up + down projection
        n_e2e = max(3, args.steps // 2)
        ms_e2e, ms_e2e_base = [], []
        for _ in range(2):
            ms_e2e.append(time_e2e(mlp.forward if ours else base_block, n_e2e))
            if ours:
                ms_e2e_base.append(time_e2e(base_block, n_e2e))
        ms_e = sum(ms_e2e) / len(ms_e2e)
        e2e = {
            "value": flops_e2e / (ms_e * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms_e,
            "what": "TPMLP.forward (allgather_matmul -> gelu -> matmul_reduce_scatter); every step copies its input "
                    "shard from pinned host memory (copy stream, one step ahead) and reads its scalar loss back",
            "h2d_bytes_per_step": W * x_host[0].numel() * x_host[0].element_size(),
            "d2h_bytes_per_step": W * 4,
        }
        if ours:
            ms_b = sum(ms_e2e_base) / len(ms_e2e_base)
            e2e.update({"cublas_nccl_ms": ms_b, "cublas_nccl_value": flops_e2e / (ms_b * 1e-3) / 1e12,
                        "speedup": ms_b / ms_e})
        check("end to end")
        return e2e

    e2e = None
    if not args.no_e2e:
        try:
            e2e = end_to_end()
        except Exception as exc:   # the headline above is already measured: report it, with the failure beside it
            e2e = {"error": "%s: %s" % (type(exc).__name__, str(exc)[:400]), "phase": _State.phase}
            try:
                if ctx is not None:
                    ctx.reset_after_error()
            except Exception:
                pass

    vs = (base_step_ms / ms_step) if (ours and base_step_ms) else None
    clocks = sampler.summary() if sampler is not None else {}

    if rank == 0:
        print(json.dumps({
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": W, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": vs, "dtype": "bf16", "data": "synthetic (seeded per rank, random-init weights)",
            "impl": args.impl,
            "config": {
                "model": "tensor-parallel block ops: allgather_matmul + matmul_reduce_scatter + matmul_allreduce",
                "global_batch": M, "seq_len": M, "hidden": HIDDEN, "ffn": FFN,
                "parallelism": "tp%d" % W,
                "l2": "inputs larger than L2: each step touches > 126 MB of distinct operands and outputs",
                "timing": "CUDA events on the launching stream, barrier + synchronize on both sides, max over ranks",
                "vs_baseline": "the reference publishes no number: ratio to the cuBLAS + NCCL step timed in this "
                               "process in alternation with the fused step",
            },
            "clocks": {"sm_mhz": clocks.get("sm_mhz"), "sm_max_mhz": clocks.get("sm_max_mhz"),
                       "reasons": clocks.get("reasons", []), "samples": clocks.get("samples", 0)},
            "host_wall_s": host_s,
            "gpu_launches": launches * W,
            "ops": ops,
            "e2e": e2e,
        }))
    if ctx is not None:
        ctx.finalize()
    if world > 1:
        dist.destroy_process_group()
    return 0


def main() -> int:
    args = parse_args()
    if args.impl == "reference":
        reference_unavailable()
        return 0
    try:
        return run(args)
    except BaseException as e:   # the last stdout line must say what failed, on whichever rank
        if isinstance(e, SystemExit) and not e.code:
            return 0
        status = getattr(e, "status", None)
        try:
            if status is None and _State.ctx is not None:
                status = [int(v) for v in _State.ctx.status.cpu().tolist()]
        except Exception:
            pass
        sys.stderr.write(traceback.format_exc())
        sys.stderr.flush()
        print(json.dumps({"impl": _State.impl, "error": "%s: %s" % (type(e).__name__, e), "phase": _State.phase,
                          "rank": _State.rank, "status": status}), flush=True)
        # leave without the collective teardown: a peer may already be gone
        os._exit(1)


if __name__ == "__main__":
    sys.exit(main())

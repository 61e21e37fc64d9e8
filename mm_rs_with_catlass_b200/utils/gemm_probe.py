"""Single-GPU probe of the kernel in its local-GEMM mode: a few launches of one shape, for
profiler captures and quick timing.

    python -m mm_rs_with_catlass_b200.utils.gemm_probe M N K [--trans-b] [--pair 1|2] [--bn 256]
                                                      [--dtype bf16|fp16|int8] [--launches 3] [--time] [--trace]
                                                      [--split-k S]

``--split-k S`` runs the split-K form (K slices as the groups of one launch + the plane reduction;
``S = 0`` lets the library pick tile width and slice count). ``--time`` prints CUDA-event time and the cuBLAS time of the same shape; ``--trace`` prints the
kernel's per-role cycle counters (see ``FusedParams::trace`` in csrc/include/catcoc/params.h).
"""
from __future__ import annotations

import argparse
import json
import sys

import torch

TRACE_NAMES = ["prod_wait_empty", "prod_issue", "mma_wait_full", "mma_wait_acc", "mma_issue", "epi_wait_full",
               "epi_work", "epi_wait_peer", "cta_life", "epi_publish", "epi_own", "epi_tmem_ld", "epi_convert", "epi_flush", "epi_tiles_own", "epi_tiles_pushed"]


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("m", type=int)
    ap.add_argument("n", type=int)
    ap.add_argument("k", type=int)
    ap.add_argument("--trans-b", action="store_true")
    ap.add_argument("--pair", type=int, default=1)
    ap.add_argument("--bn", type=int, default=0)
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp16", "int8"])
    ap.add_argument("--launches", type=int, default=3)
    ap.add_argument("--time", action="store_true")
    ap.add_argument("--trace", action="store_true")
    ap.add_argument("--split-k", type=int, default=None)
    a = ap.parse_args(argv)

    from mm_rs_with_catlass_b200 import TilingConfig
    from mm_rs_with_catlass_b200.ops.gemm import matmul
    from mm_rs_with_catlass_b200.ops._common import local_status, raise_on_status
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    dt = {"bf16": torch.bfloat16, "fp16": torch.float16, "int8": torch.int8}[a.dtype]
    if dt == torch.int8:
        A = torch.randint(-127, 128, (a.m, a.k), device=dev, dtype=torch.int32).to(torch.int8)
        B = torch.randint(-127, 128, (a.n, a.k) if a.trans_b else (a.k, a.n), device=dev, dtype=torch.int32).to(torch.int8)
        out = torch.empty((a.m, a.n), dtype=torch.int32, device=dev)
    else:
        A = torch.randn(a.m, a.k, device=dev).to(dt)
        B = (torch.randn((a.n, a.k) if a.trans_b else (a.k, a.n), device=dev) * 0.02).to(dt)
        out = torch.empty((a.m, a.n), dtype=dt, device=dev)
    cfg = TilingConfig(cta_pair=a.pair, bn=a.bn)
    if a.split_k is not None and dt != torch.int8:
        from mm_rs_with_catlass_b200.ops.blas import splitk_matmul
        explicit = a.bn or a.pair != 1
        run = lambda trace=None: splitk_matmul(A, B, trans_b=a.trans_b, out=out, split_k=a.split_k or None,
                                               tiling=cfg if explicit else None)
    else:
        run = lambda trace=None: matmul(A, B, trans_b=a.trans_b, out=out, tiling=cfg, trace=trace)
    for _ in range(a.launches):
        run()
    torch.cuda.synchronize()
    res = {"m": a.m, "n": a.n, "k": a.k, "trans_b": a.trans_b, "pair": a.pair, "bn": a.bn, "dtype": a.dtype}
    if a.time:
        def timed(fn, iters=20):
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            for _ in range(iters):
                fn()
            e.record()
            torch.cuda.synchronize()
            return s.elapsed_time(e) / iters
        ms = timed(run)
        res.update(ms=ms, tflops=2.0 * a.m * a.n * a.k / ms / 1e9)
        if dt != torch.int8:
            Bm = B.t() if a.trans_b else B
            lib = lambda: torch.matmul(A, Bm, out=out)
            for _ in range(3):
                lib()
            ms_l = timed(lib)
            res.update(cublas_ms=ms_l, cublas_tflops=2.0 * a.m * a.n * a.k / ms_l / 1e9)
    if a.trace:
        tr = torch.zeros(16, dtype=torch.int64, device=dev)
        run(tr)
        torch.cuda.synchronize()
        ctas = 148
        res["cycles_per_cta"] = {n: round(v / ctas) for n, v in zip(TRACE_NAMES, tr.cpu().tolist())}
    raise_on_status(local_status(dev), "gemm_probe")
    print(json.dumps(res))
    return 0


if __name__ == "__main__":
    sys.exit(main())

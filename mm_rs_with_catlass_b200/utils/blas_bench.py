"""Times the single-GPU kernel catalogue against the library routes PyTorch takes for the same
math (cuBLAS ``matmul`` / ``addmm`` / ``bmm`` / ``mv``, a per-group loop for grouped products).

    python -m mm_rs_with_catlass_b200.utils.blas_bench [--steps 20] [--warmup 5] [--json out.json]

Every row is timed with CUDA events after warm-up with an L2 flush before each timed launch;
``ratio`` is library time / this kernel's time (above 1: this kernel is faster).
"""
from __future__ import annotations

import argparse
import json
import sys

import torch


def _rows(dev):
    import mm_rs_with_catlass_b200 as catcoc
    bf = torch.bfloat16

    def rnd(*shape, dtype=bf, scale=1.0):
        return (torch.randn(*shape, device=dev) * scale).to(dtype)

    rows = []

    # --- affine epilogue: D = alpha A B + beta C ---
    M, N, K = 8192, 8192, 4096
    a, b, c = rnd(M, K), rnd(K, N, scale=0.02), rnd(M, N)
    out = torch.empty_like(c)
    rows.append(("gemm alpha/beta %dx%dx%d" % (M, N, K), 2.0 * M * N * K,
                 lambda: catcoc.gemm(a, b, c, alpha=0.5, beta=2.0, out=out),
                 lambda: torch.addmm(c, a, b, beta=2.0, alpha=0.5, out=out)))
    bias = rnd(N, dtype=torch.float32)
    bias_bf = bias.to(bf)
    rows.append(("matmul_bias %dx%dx%d" % (M, N, K), 2.0 * M * N * K,
                 lambda: catcoc.matmul_bias(a, b, bias, out=out),
                 lambda: torch.addmm(bias_bf, a, b, out=out)))

    # --- batched ---
    B, m, n, k = 16, 1024, 1024, 1024
    ab, bb = rnd(B, m, k), rnd(B, k, n, scale=0.03)
    ob = torch.empty(B, m, n, dtype=bf, device=dev)
    rows.append(("batched %dx(%dx%dx%d)" % (B, m, n, k), 2.0 * B * m * n * k,
                 lambda: catcoc.batched_matmul(ab, bb, out=ob), lambda: torch.bmm(ab, bb, out=ob)))

    # --- grouped (MoE expert GEMM): 32 experts, ragged token counts, weights [G, N, K] ---
    G, n, k = 32, 4096, 2048
    gen = torch.Generator().manual_seed(0)
    sizes = torch.randint(64, 960, (G,), generator=gen)
    ends = sizes.cumsum(0).to(torch.int32)
    total = int(ends[-1])
    ag, wg = rnd(total, k), rnd(G, n, k, scale=0.02)
    og = torch.empty(total, n, dtype=bf, device=dev)
    ends_dev = ends.to(dev)
    bounds = [0] + ends.tolist()

    def grouped_loop():
        for g in range(G):
            torch.matmul(ag[bounds[g]:bounds[g + 1]], wg[g].t(), out=og[bounds[g]:bounds[g + 1]])

    rows.append(("grouped %d experts, %d tokens, N=%d K=%d" % (G, total, n, k), 2.0 * total * n * k,
                 lambda: catcoc.grouped_matmul(ag, wg, ends_dev, trans_b=True, out=og), grouped_loop))

    # --- split-K: few output tiles, long K ---
    for (M, N, K) in ((128, 1024, 16384), (256, 256, 32768), (128, 8192, 1024)):
        a2, b2 = rnd(M, K), rnd(K, N, scale=0.02)
        o2 = torch.empty(M, N, dtype=bf, device=dev)
        rows.append(("splitk %dx%dx%d" % (M, N, K), 2.0 * M * N * K,
                     lambda a2=a2, b2=b2, o2=o2: catcoc.splitk_matmul(a2, b2, out=o2),
                     lambda a2=a2, b2=b2, o2=o2: torch.matmul(a2, b2, out=o2)))
        rows.append(("plain  %dx%dx%d" % (M, N, K), 2.0 * M * N * K,
                     lambda a2=a2, b2=b2, o2=o2: catcoc.matmul(a2, b2, out=o2),
                     lambda a2=a2, b2=b2, o2=o2: torch.matmul(a2, b2, out=o2)))

    # --- GEMV (bytes instead of FLOPs) ---
    R, Cc = 16384, 16384
    am, xv, xr = rnd(R, Cc), rnd(Cc), rnd(R)
    yv, yr = torch.empty(R, dtype=bf, device=dev), torch.empty(Cc, dtype=bf, device=dev)
    rows.append(("gemv %dx%d" % (R, Cc), -2.0 * R * Cc,
                 lambda: catcoc.gemv(am, xv, out=yv), lambda: torch.mv(am, xv, out=yv)))
    rows.append(("gemv^T %dx%d" % (R, Cc), -2.0 * R * Cc,
                 lambda: catcoc.gemv(am, xr, trans=True, out=yr), lambda: torch.mv(am.t(), xr, out=yr)))
    return rows


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--json", default=None)
    args = ap.parse_args(argv)
    from mm_rs_with_catlass_b200.utils.timing import time_steps
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    result = []
    print("%-48s %10s %10s %7s %12s" % ("op", "ours us", "torch us", "ratio", "ours rate"))
    for name, work, ours, theirs in _rows(dev):
        t_ours = time_steps(ours, args.steps, args.warmup, dev, flush=True) * 1e3
        t_lib = time_steps(theirs, args.steps, args.warmup, dev, flush=True) * 1e3
        rate = ("%.0f TFLOP/s" % (work / t_ours * 1e-6)) if work > 0 else ("%.2f TB/s" % (-work / t_ours * 1e-6))
        print("%-48s %10.1f %10.1f %7.2f %12s" % (name, t_ours, t_lib, t_lib / t_ours, rate))
        result.append(dict(op=name, ours_us=t_ours, torch_us=t_lib, ratio=t_lib / t_ours, rate=rate))
    if args.json:
        with open(args.json, "w") as f:
            json.dump(result, f, indent=1)
    return 0


if __name__ == "__main__":
    sys.exit(main())

"""Flash attention forward: this library's tcgen05 kernel against PyTorch's fused attention
(``scaled_dot_product_attention``), CUDA-event times on one GPU, L2 flushed before every launch.

    python -m mm_rs_with_catlass_b200.utils.attn_bench [--out table.json]
    python -m mm_rs_with_catlass_b200.utils.attn_bench --shape 2,16,16,4096,128,1 --probe 3    # 3 launches of ours only (profiler runs)
"""
from __future__ import annotations

import argparse
import json
import sys

import torch


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=None)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--shape", default=None, help="B,Hq,Hk,S,D,causal: this shape only")
    ap.add_argument("--probe", type=int, default=0, help="launch this library's kernel N times and exit (no timing, no PyTorch arm)")
    args = ap.parse_args(argv)
    import mm_rs_with_catlass_b200 as catcoc
    from mm_rs_with_catlass_b200.ops import _common as cm
    from mm_rs_with_catlass_b200.utils import timing
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    rows = []
    shapes = [(4, 32, 32, 2048, 128, False), (4, 32, 32, 2048, 128, True), (2, 32, 8, 8192, 128, True),
              (1, 32, 8, 16384, 128, True), (8, 32, 32, 1024, 64, True)]
    if args.shape:
        f = [int(x) for x in args.shape.split(",")]
        shapes = [(f[0], f[1], f[2], f[3], f[4], bool(f[5]))]
    for (b, hq, hk, s, d, causal) in shapes:
        q = torch.randn(b, hq, s, d, device=dev).bfloat16()
        k = torch.randn(b, hk, s, d, device=dev).bfloat16()
        v = torch.randn(b, hk, s, d, device=dev).bfloat16()
        out = torch.empty_like(q)
        ours = lambda: catcoc.flash_attention(q, k, v, causal=causal, out=out)
        if args.probe:
            for _ in range(args.probe):
                ours()
            torch.cuda.synchronize(dev)
            cm.raise_on_status(cm.local_status(dev), "flash_attention")
            continue
        lib = lambda: torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=causal, enable_gqa=(hq != hk))
        flops = 4.0 * b * hq * s * s * d * (0.5 if causal else 1.0)
        t_o = timing.time_steps(ours, args.iters, 3, dev, flush=True)
        t_l = timing.time_steps(lib, args.iters, 3, dev, flush=True)
        row = {"B": b, "Hq": hq, "Hk": hk, "S": s, "D": d, "causal": causal, "ours_us": 1e3 * t_o,
               "sdpa_us": 1e3 * t_l, "ours_tflops": flops / (t_o * 1e-3) / 1e12, "sdpa_tflops": flops / (t_l * 1e-3) / 1e12,
               "ratio": t_l / t_o}
        rows.append(row)
        print(json.dumps(row), flush=True)
    if args.out:
        with open(args.out, "w") as fh:
            json.dump(rows, fh, indent=1)
    return 0


if __name__ == "__main__":
    sys.exit(main())

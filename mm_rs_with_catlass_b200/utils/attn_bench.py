"""Flash attention forward: this library's tcgen05 kernel against PyTorch's fused attention
(``scaled_dot_product_attention``), CUDA-event times on one GPU, L2 flushed before every launch.

    python -m mm_rs_with_catlass_b200.utils.attn_bench [--out table.json]
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
    args = ap.parse_args(argv)
    import mm_rs_with_catlass_b200 as catcoc
    from mm_rs_with_catlass_b200.utils import timing
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    rows = []
    for (b, hq, hk, s, d, causal) in [(4, 32, 32, 2048, 128, False), (4, 32, 32, 2048, 128, True),
                                      (2, 32, 8, 8192, 128, True), (1, 32, 8, 16384, 128, True),
                                      (8, 32, 32, 1024, 64, True)]:
        q = torch.randn(b, hq, s, d, device=dev).bfloat16()
        k = torch.randn(b, hk, s, d, device=dev).bfloat16()
        v = torch.randn(b, hk, s, d, device=dev).bfloat16()
        out = torch.empty_like(q)
        ours = lambda: catcoc.flash_attention(q, k, v, causal=causal, out=out)
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

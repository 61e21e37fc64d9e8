"""Latent-attention decode: this library's tcgen05 kernel against PyTorch's fused attention on
the gathered (un-paged) cache, CUDA-event times on one GPU, L2 flushed before every launch.

    python -m mm_rs_with_catlass_b200.utils.mla_bench [--out table.json]

The PyTorch arm gets the cache already gathered into a dense ``[B, 1, S, 576]`` tensor (its
gather is not timed); ``cache_gbs`` is the cache bytes of the batch divided by this kernel's time.
"""
from __future__ import annotations

import argparse
import json
import math
import sys

import torch


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=None)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--shape", default=None, help="B,H,S,q_len: this shape only")
    ap.add_argument("--splits", type=int, default=0)
    ap.add_argument("--probe", type=int, default=0, help="launch this library's kernel N times and exit")
    args = ap.parse_args(argv)
    import mm_rs_with_catlass_b200 as catcoc
    from mm_rs_with_catlass_b200.ops import _common as cm
    from mm_rs_with_catlass_b200.utils import timing
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    shapes = [(1, 16, 8192, 1), (8, 16, 4096, 1), (32, 16, 4096, 1), (128, 16, 2048, 1), (32, 128, 4096, 1),
              (128, 128, 2048, 1), (32, 16, 4096, 2)]
    if args.shape:
        shapes = [tuple(int(x) for x in args.shape.split(","))]
    rows = []
    for (b, h, s, q_len) in shapes:
        pages_per_seq = (s + 127) // 128
        num_pages = b * pages_per_seq
        q_nope = torch.randn(b * q_len, h, 512, device=dev).bfloat16()
        q_rope = torch.randn(b * q_len, h, 64, device=dev).bfloat16()
        ckv = torch.randn(num_pages, 128, 512, device=dev).bfloat16()
        krope = torch.randn(num_pages, 128, 64, device=dev).bfloat16()
        table = torch.randperm(num_pages, device=dev).reshape(b, pages_per_seq).to(torch.int32)
        lens = torch.full((b,), s, dtype=torch.int32, device=dev)
        out = torch.empty_like(q_nope)
        ours = lambda: catcoc.mla_decode(q_nope, q_rope, ckv, krope, table, lens, q_len=q_len, causal=q_len > 1,
                                         splits=args.splits or None, out=out)
        if args.probe:
            for _ in range(args.probe):
                ours()
            torch.cuda.synchronize(dev)
            cm.raise_on_status(cm.local_status(dev), "mla_decode")
            continue
        # dense arm: keys [B, 1, S, 576], values [B, 1, S, 512] (padded to 576 for the library call), queries [B, H, q_len, 576]
        keys = torch.cat([ckv[table.long()].reshape(b, s, 512), krope[table.long()].reshape(b, s, 64)], dim=2)[:, None]
        vals = torch.nn.functional.pad(keys[..., :512], (0, 64))
        qd = torch.cat([q_nope, q_rope], dim=2).reshape(b, q_len, h, 576).transpose(1, 2).contiguous()
        lib = lambda: torch.nn.functional.scaled_dot_product_attention(qd, keys, vals, is_causal=False, enable_gqa=True,
                                                                       scale=1.0 / math.sqrt(576.0))
        t_o = timing.time_steps(ours, args.iters, 3, dev, flush=True)
        try:
            t_l = timing.time_steps(lib, args.iters, 3, dev, flush=True)
        except RuntimeError:
            t_l = float("nan")
        cache_bytes = b * s * 576 * 2
        row = {"B": b, "H": h, "S": s, "q_len": q_len, "ours_us": 1e3 * t_o, "sdpa_dense_us": 1e3 * t_l,
               "cache_gbs": cache_bytes / (t_o * 1e-3) / 1e9, "tflops": 2.0 * b * q_len * h * s * (576 + 512) / (t_o * 1e-3) / 1e12,
               "ratio": t_l / t_o}
        rows.append(row)
        print(json.dumps(row), flush=True)
    cm.raise_on_status(cm.local_status(dev), "mla_decode")
    if args.out:
        with open(args.out, "w") as fh:
            json.dump(rows, fh, indent=1)
    return 0


if __name__ == "__main__":
    sys.exit(main())

"""Seeded synthetic inputs for tests, tuning and benchmarks.

The reference feeds every rank the same A and B (examples/utils/gen_data.py:33-45), which
hides rank-indexing mistakes; here every rank's data depends on its rank. The all-ones and
``arange`` debug patterns of examples/utils/gen_quant_data.py:43-52 are kept for localising
indexing errors.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch


def _gen(device, seed: int) -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return g


def matmul_inputs(m: int, n: int, k: int, rank: int = 0, dtype: torch.dtype = torch.bfloat16,
                  device="cpu", trans_a: bool = False, trans_b: bool = False, seed: int = 0,
                  a_std: float = 1.0, b_std: Optional[float] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """``A`` ~ N(0, a_std) stored [m, k] ([k, m] with trans_a) and ``B`` ~ N(0, b_std) stored
    [k, n] ([n, k] with trans_b); b_std defaults to 1/sqrt(k) so outputs stay O(1)."""
    b_std = (k ** -0.5) if b_std is None else b_std
    g = _gen(device, 1000003 * seed + 7919 * rank + 1)
    a = (torch.randn((k, m) if trans_a else (m, k), generator=g, device=device) * a_std).to(dtype)
    b = (torch.randn((n, k) if trans_b else (k, n), generator=g, device=device) * b_std).to(dtype)
    return a, b


def quant_inputs(m: int, n: int, k: int, rank: int = 0, device="cpu", trans_b: bool = False, seed: int = 0,
                 with_bias: bool = True, debug: bool = False):
    """int8 operands uniform in [-127, 127], fp32 per-token scale ~U(0.001, 0.02) (same on all
    ranks: it describes the global rows), per-channel scale ~U(0, 0.01), int32 bias.

    ``debug`` gives all-ones operands, constant scales and an ``arange`` bias."""
    g = _gen(device, 1000003 * seed + 7919 * rank + 2)
    gs = _gen(device, 1000003 * seed + 3)  # scales / bias are rank independent
    if debug:
        x1 = torch.ones((m, k), dtype=torch.int8, device=device)
        x2 = torch.ones((n, k) if trans_b else (k, n), dtype=torch.int8, device=device)
        s1 = torch.full((m,), 0.01, dtype=torch.float32, device=device)
        s2 = torch.full((n,), 0.01, dtype=torch.float32, device=device)
        bias = torch.arange(1, n + 1, dtype=torch.int32, device=device) if with_bias else None
        return x1, x2, s1, s2, bias
    x1 = torch.randint(-127, 128, (m, k), generator=g, device=device, dtype=torch.int32).to(torch.int8)
    x2 = torch.randint(-127, 128, (n, k) if trans_b else (k, n), generator=g, device=device, dtype=torch.int32).to(torch.int8)
    s1 = torch.rand(m, generator=gs, device=device) * 0.019 + 0.001
    s2 = torch.rand(n, generator=gs, device=device) * 0.01
    bias = torch.randint(-1000, 1000, (n,), generator=gs, device=device, dtype=torch.int32) if with_bias else None
    return x1, x2, s1, s2, bias

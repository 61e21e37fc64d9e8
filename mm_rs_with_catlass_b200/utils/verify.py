"""Numerical acceptance rule and tolerances.

Same rule as the reference's checker (examples/utils/verify_result.py:106-116 with the
tolerances of examples/utils/utils.py:44-52): every element must satisfy
``|out - golden| <= rtol * max(1, |golden|)`` and the mean relative bias
``sum|out - golden| / sum|golden|`` must stay under a per-dtype bound. Unlike the reference,
a failed check is an exception (and a non-zero exit code), and NaN / Inf are failures instead
of being zeroed on both sides.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch


def get_rtol(dtype: torch.dtype, k: int) -> float:
    small = k < 2048
    if dtype == torch.float16:
        return 2.0 ** -8 if small else 2.0 ** -7
    if dtype == torch.bfloat16:
        return 2.0 ** -7 if small else 2.0 ** -6
    if dtype == torch.float32:
        return 2.0 ** -11 if small else 2.0 ** -10
    raise TypeError("no tolerance defined for %s" % dtype)


def get_bias_bound(dtype: torch.dtype) -> float:
    if dtype == torch.float16:
        return 2.0 ** -10
    if dtype == torch.bfloat16:
        return 2.0 ** -7
    if dtype == torch.float32:
        return 2.0 ** -14
    raise TypeError("no bias bound defined for %s" % dtype)


@dataclass
class VerifyResult:
    ok: bool
    n_bad: int
    n_total: int
    max_abs_err: float
    mean_rel_bias: float
    rtol: float
    bias_bound: float

    def __str__(self) -> str:
        return ("%s: %d / %d elements out of tolerance (rtol %.3g), max |err| %.4g, mean relative bias %.3g "
                "(bound %.3g)" % ("PASS" if self.ok else "ERROR", self.n_bad, self.n_total, self.rtol,
                                  self.max_abs_err, self.mean_rel_bias, self.bias_bound))


def verify(out: torch.Tensor, golden: torch.Tensor, k: int, dtype: torch.dtype = None,
           magnitude: torch.Tensor = None) -> VerifyResult:
    """Compares ``out`` (any float dtype) with the fp32 ``golden``; ``k`` is the full reduction
    length (it selects the tolerance tier), ``dtype`` the precision the result was rounded to.

    ``magnitude`` (same shape as ``golden``) replaces ``|golden|`` in the tolerance. It is for
    results that are sums of terms rounded to ``dtype`` before the sum (partial tiles that cross
    the link in bf16 / fp16): the rounding error of such a sum scales with ``sum_r |term_r|``,
    which can be far above ``|sum|`` when terms cancel. The reference never meets this case
    because it feeds every rank identical data."""
    dtype = dtype or out.dtype
    rtol, bound = get_rtol(dtype, k), get_bias_bound(dtype)
    o = out.detach().float().cpu().reshape(-1)
    g = golden.detach().float().cpu().reshape(-1)
    if o.numel() != g.numel():
        raise ValueError("size mismatch: out has %d elements, golden %d" % (o.numel(), g.numel()))
    finite = torch.isfinite(o) & torch.isfinite(g)
    diff = (o - g).abs()
    scale = g.abs() if magnitude is None else torch.maximum(g.abs(), magnitude.detach().float().cpu().reshape(-1))
    tol = rtol * torch.clamp(scale, min=1.0)
    bad = (~finite) | (diff > tol)
    n_bad = int(bad.sum())
    denom = float(g[finite].abs().sum())
    bias = float(diff[finite].sum()) / denom if denom > 0 else 0.0
    max_err = float(diff[finite].max()) if bool(finite.any()) else float("inf")
    return VerifyResult(n_bad == 0 and bias <= bound, n_bad, o.numel(), max_err, bias, rtol, bound)


def assert_close(out: torch.Tensor, golden: torch.Tensor, k: int, dtype: torch.dtype = None, what: str = "",
                 magnitude: torch.Tensor = None) -> None:
    r = verify(out, golden, k, dtype, magnitude)
    if not r.ok:
        raise AssertionError("%s %s" % (what, r))

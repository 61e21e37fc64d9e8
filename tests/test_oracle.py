"""The C++ CPU oracle against PyTorch, and the acceptance rule."""
import ctypes as C

import numpy as np
import pytest
import torch

from mm_rs_with_catlass_b200 import _native as N
from mm_rs_with_catlass_b200.utils import verify as V


def ptr(t):
    return C.c_void_p(t.data_ptr())


@pytest.mark.parametrize("ta,tb", [(0, 0), (0, 1), (1, 0), (1, 1)])
def test_oracle_matmul_matches_torch(ta, tb):
    M, Nn, K = 23, 45, 68
    a = torch.randn((K, M) if ta else (M, K))
    b = torch.randn((Nn, K) if tb else (K, Nn))
    c = torch.empty(M, Nn)
    assert N.lib().catcoc_oracle_matmul_f32(ptr(a), ptr(b), ptr(c), M, Nn, K, ta, tb) == 0
    ref = (a.t() if ta else a).double() @ (b.t() if tb else b).double()
    assert torch.allclose(c.double(), ref, rtol=1e-6, atol=1e-6)


@pytest.mark.parametrize("tb", [0, 1])
def test_oracle_quant_matmul_is_exact_and_dequant_matches(tb):
    M, Nn, K = 4, 129, 128
    a = torch.randint(-127, 128, (M, K), dtype=torch.int32).to(torch.int8)
    b = torch.randint(-127, 128, (Nn, K) if tb else (K, Nn), dtype=torch.int32).to(torch.int8)
    bias = torch.randint(-1000, 1000, (Nn,), dtype=torch.int32)
    acc = torch.empty((M, Nn), dtype=torch.int32)
    assert N.lib().catcoc_oracle_quant_matmul(ptr(a), ptr(b), ptr(bias), ptr(acc), M, Nn, K, 0, tb) == 0
    ref = a.long() @ (b.t() if tb else b).long() + bias.long()[None, :]
    assert torch.equal(acc.long(), ref)
    s1, s2 = torch.rand(M) * 0.02, torch.rand(Nn) * 0.01
    out = torch.empty((M, Nn))
    assert N.lib().catcoc_oracle_dequant(ptr(acc), ptr(s1), ptr(s2), ptr(out), M, Nn) == 0
    assert torch.allclose(out, acc.float() * s2[None, :] * s1[:, None], rtol=1e-6)


def test_compare_counts_violations_and_bias():
    g = torch.tensor([1.0, 2.0, -4.0, 0.5, 100.0])
    o = g.clone()
    o[1] += 0.5
    o[4] += 0.2
    bias = C.c_double()
    bad = N.lib().catcoc_oracle_compare(ptr(o), ptr(g), 5, C.c_float(2.0 ** -7), C.byref(bias))
    assert bad == 1                                   # 0.5 > tol*2, 0.2 < tol*100
    assert abs(bias.value - 0.7 / 107.5) < 1e-6   # fp32 inputs
    nan = o.clone()
    nan[0] = float("nan")
    assert N.lib().catcoc_oracle_compare(ptr(nan), ptr(g), 5, C.c_float(1.0), C.byref(bias)) == 1


def test_tolerance_table():
    assert V.get_rtol(torch.float16, 512) == 2 ** -8 and V.get_rtol(torch.float16, 4096) == 2 ** -7
    assert V.get_rtol(torch.bfloat16, 512) == 2 ** -7 and V.get_rtol(torch.bfloat16, 4096) == 2 ** -6
    assert V.get_bias_bound(torch.float16) == 2 ** -10 and V.get_bias_bound(torch.bfloat16) == 2 ** -7


def test_verify_passes_rounded_results_and_fails_wrong_ones():
    g = torch.randn(64, 64) * 3
    assert V.verify(g.to(torch.bfloat16), g, k=512).ok
    wrong = g.clone()
    wrong[3, 5] += 1.0
    r = V.verify(wrong.to(torch.bfloat16), g, k=512)
    assert not r.ok and r.n_bad >= 1
    with pytest.raises(AssertionError):
        V.assert_close(wrong.to(torch.bfloat16), g, k=512)
    inf = g.clone()
    inf[0, 0] = float("inf")
    assert not V.verify(inf, g, k=512, dtype=torch.float32).ok

"""The kernel catalogue on the GPU against the library's own C++ CPU goldens (small shapes: the
goldens are naive loops). The larger sweeps against PyTorch are in test_blas_gpu.py."""
import ctypes as C

import pytest
import torch

import mm_rs_with_catlass_b200 as catcoc
from mm_rs_with_catlass_b200 import _native as N
from mm_rs_with_catlass_b200.utils.verify import assert_close

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
BF = torch.bfloat16


def ptr(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def f32(t):
    return t.detach().float().cpu().contiguous()


def rnd(*shape, scale=1.0, seed=0):
    g = torch.Generator().manual_seed(seed + sum(shape))
    return (torch.randn(*shape, generator=g) * scale).to(BF)


@pytest.mark.parametrize("ta,tb", [(False, False), (True, True)])
def test_gemm_affine_against_the_cpp_golden(ta, tb):
    M, Nn, K = 136, 200, 96
    a, b, c = rnd(*((K, M) if ta else (M, K))), rnd(*((Nn, K) if tb else (K, Nn)), scale=0.1), rnd(M, Nn)
    out = catcoc.gemm(a.to(DEV), b.to(DEV), c.to(DEV), alpha=0.5, beta=-1.5, trans_a=ta, trans_b=tb)
    gold = torch.empty(M, Nn)
    assert N.lib().catcoc_oracle_gemm(ptr(f32(a)), ptr(f32(b)), ptr(f32(c)), None, ptr(gold), M, Nn, K, int(ta),
                                      int(tb), 0.5, -1.5) == 0
    assert_close(out, gold, k=K, dtype=BF, what="gemm")


def test_matmul_bias_against_the_cpp_golden():
    M, Nn, K = 64, 136, 128
    a, b = rnd(M, K), rnd(K, Nn, scale=0.1)
    bias = torch.randn(Nn)
    out = catcoc.matmul_bias(a.to(DEV), b.to(DEV), bias.to(DEV))
    gold = torch.empty(M, Nn)
    assert N.lib().catcoc_oracle_gemm(ptr(f32(a)), ptr(f32(b)), None, ptr(bias), ptr(gold), M, Nn, K, 0, 0, 1.0,
                                      0.0) == 0
    assert_close(out, gold, k=K, dtype=BF, what="matmul_bias")


@pytest.mark.parametrize("trans", [False, True])
def test_gemv_against_the_cpp_golden(trans):
    rows, cols = 300, 520
    a = rnd(rows, cols, scale=0.1)
    x, y = rnd(rows if trans else cols), rnd(cols if trans else rows)
    out = catcoc.gemv(a.to(DEV), x.to(DEV), y.to(DEV), alpha=2.0, beta=0.5, trans=trans)
    gold = torch.empty(cols if trans else rows)
    assert N.lib().catcoc_oracle_gemv(ptr(f32(a)), ptr(f32(x)), ptr(f32(y)), ptr(gold), rows, cols, int(trans), 2.0,
                                      0.5) == 0
    assert_close(out, gold, k=rows if trans else cols, dtype=BF, what="gemv")


def test_batched_against_the_cpp_golden():
    B, M, Nn, K = 3, 128, 72, 64
    a, b = rnd(B, M, K), rnd(B, K, Nn, scale=0.1)
    out = catcoc.batched_matmul(a.to(DEV), b.to(DEV))
    gold = torch.empty(B, M, Nn)
    assert N.lib().catcoc_oracle_batched_matmul(ptr(f32(a)), ptr(f32(b)), ptr(gold), B, M, Nn, K, 0, 0) == 0
    assert_close(out, gold, k=K, dtype=BF, what="batched")


@pytest.mark.parametrize("tb", [False, True])
def test_grouped_against_the_cpp_golden(tb):
    G, K, Nn = 4, 64, 72
    ends = [40, 40, 170, 200]
    a = rnd(200, K)
    b = rnd(*((G, Nn, K) if tb else (G, K, Nn)), scale=0.1)
    out = catcoc.grouped_matmul(a.to(DEV), b.to(DEV), ends, trans_b=tb)
    gold = torch.zeros(200, Nn)
    e = torch.tensor(ends, dtype=torch.int32)
    assert N.lib().catcoc_oracle_grouped_matmul(ptr(f32(a)), ptr(f32(b)), ptr(e), G, ptr(gold), 200, Nn, K,
                                                int(tb)) == 0
    assert_close(out, gold, k=K, dtype=BF, what="grouped")


def test_grouped_quant_against_the_cpp_golden():
    G, K, Nn, Mt = 3, 128, 136, 150
    ends = [30, 90, 150]
    g = torch.Generator().manual_seed(5)
    x1 = torch.randint(-127, 128, (Mt, K), generator=g, dtype=torch.int32).to(torch.int8)
    x2 = torch.randint(-127, 128, (G, Nn, K), generator=g, dtype=torch.int32).to(torch.int8)
    sm, sn = torch.rand(Mt, generator=g) * 0.02, torch.rand(G, Nn, generator=g) * 0.01
    out = catcoc.grouped_quant_matmul(x1.to(DEV), x2.to(DEV), sm.to(DEV), sn.to(DEV), ends, trans_b=True,
                                      out_dtype=torch.float32)
    gold = torch.empty(Mt, Nn)
    e = torch.tensor(ends, dtype=torch.int32)
    assert N.lib().catcoc_oracle_grouped_quant_matmul(ptr(x1), ptr(x2), ptr(e), G, ptr(sm), ptr(sn), ptr(gold), Mt, Nn,
                                                      K, 1) == 0
    assert torch.allclose(out.cpu(), gold, rtol=1e-5, atol=1e-6)   # exact integer sums, fp32 scales


def test_grouped_along_k_against_the_cpp_golden():
    M, Nn, Kt = 128, 72, 160
    ends = [64, 64, 160]
    a, b = rnd(Kt, M), rnd(Kt, Nn, scale=0.1)
    out = catcoc.grouped_matmul_slice_k(a.to(DEV), b.to(DEV), ends)
    gold = torch.empty(3, M, Nn)
    e = torch.tensor(ends, dtype=torch.int32)
    assert N.lib().catcoc_oracle_grouped_matmul_slice_k(ptr(f32(a)), ptr(f32(b)), ptr(e), 3, ptr(gold), M, Nn, Kt) == 0
    assert_close(out, gold, k=96, dtype=BF, what="slice K")


def test_group_gemm_against_the_cpp_golden():
    shapes = [(64, 72, 32), (130, 8, 64), (16, 256, 48)]
    probs, As, Bs, Cs = [], [], [], []
    for i, (m, n, k) in enumerate(shapes):
        a, b, c = rnd(m, k, seed=i), rnd(k, n, scale=0.1, seed=i), rnd(m, n, seed=i)
        As.append(f32(a)); Bs.append(f32(b)); Cs.append(f32(c))
        probs.append(dict(a=a.to(DEV), b=b.to(DEV), c=c.to(DEV), alpha=1.0 + i, beta=0.5 * i))
    outs = catcoc.group_gemm(probs)
    mnk = torch.tensor(shapes, dtype=torch.int32).reshape(-1)
    alphas = torch.tensor([1.0 + i for i in range(3)])
    betas = torch.tensor([0.5 * i for i in range(3)])
    cat = lambda ts: torch.cat([t.reshape(-1) for t in ts])
    a, b, c = cat(As), cat(Bs), cat(Cs)
    gold = torch.empty_like(c)
    assert N.lib().catcoc_oracle_group_gemm(3, ptr(mnk), ptr(alphas), ptr(betas), ptr(a), ptr(b), ptr(c), ptr(gold)) == 0
    off = 0
    for (m, n, k), o in zip(shapes, outs):
        assert_close(o, gold[off:off + m * n].reshape(m, n), k=k, dtype=BF, what="group gemm %dx%dx%d" % (m, n, k))
        off += m * n

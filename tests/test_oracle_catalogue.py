"""The C++ CPU goldens of the GEMM catalogue (affine, matrix-vector, batched, grouped along M and
K, int8 grouped with dequantisation, packed independent problems) against plain PyTorch."""
import ctypes as C

import pytest
import torch

from mm_rs_with_catlass_b200 import _native as N


def ptr(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def close(a, b):
    return torch.allclose(a.double(), b.double(), rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("ta,tb", [(0, 0), (0, 1), (1, 0), (1, 1)])
@pytest.mark.parametrize("with_c,with_bias", [(True, True), (True, False), (False, True), (False, False)])
def test_gemm(ta, tb, with_c, with_bias):
    M, Nn, K = 23, 45, 68
    g = torch.Generator().manual_seed(1)
    a = torch.randn((K, M) if ta else (M, K), generator=g)
    b = torch.randn((Nn, K) if tb else (K, Nn), generator=g)
    c = torch.randn(M, Nn, generator=g) if with_c else None
    bias = torch.randn(Nn, generator=g) if with_bias else None
    out = torch.empty(M, Nn)
    assert N.lib().catcoc_oracle_gemm(ptr(a), ptr(b), ptr(c), ptr(bias), ptr(out), M, Nn, K, ta, tb, 0.5, -1.25) == 0
    ref = 0.5 * ((a.t() if ta else a).double() @ (b.t() if tb else b).double())
    if with_c:
        ref = ref - 1.25 * c.double()
    if with_bias:
        ref = ref + bias.double()[None, :]
    assert close(out, ref)


@pytest.mark.parametrize("trans", [0, 1])
def test_gemv(trans):
    rows, cols = 37, 53
    a = torch.randn(rows, cols)
    x = torch.randn(rows if trans else cols)
    y0 = torch.randn(cols if trans else rows)
    y = torch.empty_like(y0)
    assert N.lib().catcoc_oracle_gemv(ptr(a), ptr(x), ptr(y0), ptr(y), rows, cols, trans, 2.0, 0.5) == 0
    assert close(y, 2.0 * ((a.t() if trans else a).double() @ x.double()) + 0.5 * y0.double())
    assert N.lib().catcoc_oracle_gemv(ptr(a), ptr(x), None, ptr(y), rows, cols, trans, 1.0, 3.0) == 0
    assert close(y, (a.t() if trans else a).double() @ x.double())


@pytest.mark.parametrize("ta,tb", [(0, 0), (1, 1)])
def test_batched(ta, tb):
    B, M, Nn, K = 3, 9, 11, 13
    a = torch.randn((B, K, M) if ta else (B, M, K))
    b = torch.randn((B, Nn, K) if tb else (B, K, Nn))
    out = torch.empty(B, M, Nn)
    assert N.lib().catcoc_oracle_batched_matmul(ptr(a), ptr(b), ptr(out), B, M, Nn, K, ta, tb) == 0
    ref = torch.bmm((a.transpose(1, 2) if ta else a).double(), (b.transpose(1, 2) if tb else b).double())
    assert close(out, ref)


@pytest.mark.parametrize("tb", [0, 1])
def test_grouped_along_m_with_empty_and_short_lists(tb):
    G, K, Nn = 4, 16, 7
    ends = torch.tensor([5, 5, 12, 17], dtype=torch.int32)       # group 1 is empty, rows 17..19 belong to nobody
    a = torch.randn(20, K)
    b = torch.randn((G, Nn, K) if tb else (G, K, Nn))
    out = torch.full((20, Nn), 7.0)
    assert N.lib().catcoc_oracle_grouped_matmul(ptr(a), ptr(b), ptr(ends), G, ptr(out), 20, Nn, K, tb) == 0
    begin = 0
    for g in range(G):
        end = int(ends[g])
        bg = (b[g].t() if tb else b[g]).double()
        assert close(out[begin:end], a[begin:end].double() @ bg)
        begin = end
    assert (out[17:] == 7.0).all()


def test_grouped_along_k():
    G, M, Nn, Kt = 3, 6, 5, 24
    ends = torch.tensor([8, 8, 24], dtype=torch.int32)
    a = torch.randn(Kt, M)
    b = torch.randn(Kt, Nn)
    out = torch.empty(G, M, Nn)
    assert N.lib().catcoc_oracle_grouped_matmul_slice_k(ptr(a), ptr(b), ptr(ends), G, ptr(out), M, Nn, Kt) == 0
    begin = 0
    for g in range(G):
        end = int(ends[g])
        assert close(out[g], a[begin:end].t().double() @ b[begin:end].double())
        begin = end


@pytest.mark.parametrize("tb", [0, 1])
def test_grouped_quant_along_m_is_exact_before_the_scales(tb):
    G, K, Nn, Mt = 3, 64, 9, 14
    ends = torch.tensor([4, 9, 14], dtype=torch.int32)
    a = torch.randint(-127, 128, (Mt, K), dtype=torch.int32).to(torch.int8)
    b = torch.randint(-127, 128, (G, Nn, K) if tb else (G, K, Nn), dtype=torch.int32).to(torch.int8)
    sm, sn = torch.rand(Mt) * 0.02, torch.rand(G, Nn) * 0.01
    out = torch.empty(Mt, Nn)
    assert N.lib().catcoc_oracle_grouped_quant_matmul(ptr(a), ptr(b), ptr(ends), G, ptr(sm), ptr(sn), ptr(out), Mt, Nn,
                                                      K, tb) == 0
    begin = 0
    for g in range(G):
        end = int(ends[g])
        acc = a[begin:end].long() @ (b[g].t() if tb else b[g]).long()
        assert torch.equal(out[begin:end], acc.float() * sn[g][None, :] * sm[begin:end, None])
        begin = end


def test_grouped_quant_along_k_and_int32_overflow_is_reported():
    G, M, Nn, Kt = 2, 4, 3, 40
    ends = torch.tensor([16, 40], dtype=torch.int32)
    a = torch.randint(-127, 128, (Kt, M), dtype=torch.int32).to(torch.int8)
    b = torch.randint(-127, 128, (Kt, Nn), dtype=torch.int32).to(torch.int8)
    sm, sn = torch.rand(G, M), torch.rand(G, Nn)
    out = torch.empty(G, M, Nn)
    f = N.lib().catcoc_oracle_grouped_quant_matmul_slice_k
    assert f(ptr(a), ptr(b), ptr(ends), G, ptr(sm), ptr(sn), ptr(out), M, Nn, Kt) == 0
    begin = 0
    for g in range(G):
        end = int(ends[g])
        acc = a[begin:end].t().long() @ b[begin:end].long()
        assert torch.equal(out[g], acc.float() * sn[g][None, :] * sm[g][:, None])
        begin = end
    # 140 000 products of 127 * 127 exceed 2^31: the device's accumulator would wrap
    big = 140000
    a2 = torch.full((big, 1), 127, dtype=torch.int8)
    b2 = torch.full((big, 1), 127, dtype=torch.int8)
    out2 = torch.empty(1, 1, 1)
    e2 = torch.tensor([big], dtype=torch.int32)
    assert f(ptr(a2), ptr(b2), ptr(e2), 1, None, None, ptr(out2), 1, 1, big) == N.E_TOO_LARGE


def test_packed_independent_problems():
    shapes = [(3, 4, 5), (7, 2, 9), (1, 6, 1)]
    mnk = torch.tensor(shapes, dtype=torch.int32).reshape(-1)
    alphas = torch.tensor([1.0, -0.5, 2.0])
    betas = torch.tensor([0.0, 1.0, 0.25])
    As = [torch.randn(m, k) for m, n, k in shapes]
    Bs = [torch.randn(k, n) for m, n, k in shapes]
    Cs = [torch.randn(m, n) for m, n, k in shapes]
    a = torch.cat([t.reshape(-1) for t in As])
    b = torch.cat([t.reshape(-1) for t in Bs])
    c = torch.cat([t.reshape(-1) for t in Cs])
    out = torch.empty_like(c)
    assert N.lib().catcoc_oracle_group_gemm(len(shapes), ptr(mnk), ptr(alphas), ptr(betas), ptr(a), ptr(b), ptr(c),
                                            ptr(out)) == 0
    off = 0
    for i, (m, n, k) in enumerate(shapes):
        ref = alphas[i].double() * (As[i].double() @ Bs[i].double()) + betas[i].double() * Cs[i].double()
        assert close(out[off:off + m * n].reshape(m, n), ref)
        off += m * n


def test_bad_arguments_are_refused():
    out = torch.empty(4)
    assert N.lib().catcoc_oracle_gemm(None, None, None, None, ptr(out), 2, 2, 2, 0, 0, 1.0, 0.0) == N.E_BAD_ARG
    assert N.lib().catcoc_oracle_gemv(None, None, None, ptr(out), 2, 2, 0, 1.0, 0.0) == N.E_BAD_ARG
    assert N.lib().catcoc_oracle_group_gemm(1, None, None, None, None, None, None, ptr(out)) == N.E_BAD_ARG

"""The single-GPU kernel catalogue (affine epilogues, batched / grouped / split-K group walk,
GEMV) against plain fp32 PyTorch references of the same ops."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def catcoc(device):
    import mm_rs_with_catlass_b200 as c
    return c


def _sync(device, what):
    from mm_rs_with_catlass_b200.ops._common import local_status, raise_on_status
    torch.cuda.synchronize()
    raise_on_status(local_status(device), what)


def _close(out, ref, k, what=""):
    from mm_rs_with_catlass_b200.utils.verify import assert_close
    assert_close(out, ref, k=k, what=what)


def _rand(shape, dtype, device, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.rand(shape, generator=g) * 2 - 1).to(dtype).to(device)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("M,N,K,pair", [(512, 768, 320, 1), (512, 768, 320, 2), (200, 328, 136, 1), (129, 257, 65, 2)])
def test_gemm_alpha_beta(catcoc, device, dtype, M, N, K, pair):
    in_dtype = torch.bfloat16 if dtype == torch.float32 else dtype
    a, b = _rand((M, K), in_dtype, device, 1), _rand((K, N), in_dtype, device, 2)
    c = _rand((M, N), dtype, device, 3)
    out = catcoc.gemm(a, b, c, alpha=0.5, beta=-1.25, out_dtype=dtype, tiling=catcoc.TilingConfig(cta_pair=pair))
    _sync(device, "gemm alpha beta")
    _close(out, 0.5 * (a.float() @ b.float()) - 1.25 * c.float(), K)


def test_gemm_in_place_and_strided_c(catcoc, device):
    M, N, K = 384, 520, 256
    a, b = _rand((M, K), torch.bfloat16, device, 4), _rand((K, N), torch.bfloat16, device, 5)
    big = _rand((M, N + 24), torch.bfloat16, device, 6)
    c = big[:, 8:8 + N]                         # pitch N + 24, origin 16 bytes into the row
    ref = 2.0 * (a.float() @ b.float()) + 0.5 * c.float()
    out = catcoc.gemm(a, b, c, alpha=2.0, beta=0.5)
    _sync(device, "gemm strided c")
    _close(out, ref, K)
    cc = c.contiguous()
    res = catcoc.gemm(a, b, cc, alpha=2.0, beta=0.5, out=cc)     # D overwrites C
    _sync(device, "gemm in place")
    assert res.data_ptr() == cc.data_ptr()
    _close(cc, ref, K)


@pytest.mark.parametrize("tb", [False, True])
def test_matmul_bias_and_add(catcoc, device, tb):
    M, N, K = 300, 456, 264
    a = _rand((M, K), torch.float16, device, 7)
    b = _rand((N, K) if tb else (K, N), torch.float16, device, 8)
    bias = _rand((N,), torch.float16, device, 9)
    x = _rand((M, N), torch.float16, device, 10)
    ab = a.float() @ (b.t() if tb else b).float()
    out = catcoc.matmul_bias(a, b, bias, trans_b=tb)
    _sync(device, "matmul_bias")
    _close(out, ab + bias.float()[None, :], K)
    out = catcoc.matmul_add(a, b, x, trans_b=tb)
    _sync(device, "matmul_add")
    _close(out, ab + x.float(), K)


def test_fp8_dequant_with_bias_row(catcoc, device):
    if not hasattr(torch, "float8_e4m3fn"):
        pytest.skip("no fp8 dtype")
    M, N, K = 256, 384, 512
    a = _rand((M, K), torch.float32, device, 11).to(torch.float8_e4m3fn)
    b = _rand((N, K), torch.float32, device, 12).to(torch.float8_e4m3fn)
    sm = torch.rand(M, device=device) + 0.5
    sn = torch.rand(N, device=device) + 0.5
    bias = _rand((N,), torch.float32, device, 13)
    out = catcoc.matmul(a, b, trans_b=True, scale_m=sm, scale_n=sn, bias_f32=bias, alpha=0.25,
                        out_dtype=torch.bfloat16)
    _sync(device, "fp8 affine")
    ref = 0.25 * (a.float() @ b.float().t()) * sm[:, None] * sn[None, :] + bias[None, :]
    _close(out, ref, K)


@pytest.mark.parametrize("ta,tb", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("B,M,N,K", [(3, 256, 384, 128), (5, 200, 136, 96), (2, 77, 264, 80)])
def test_batched_matmul(catcoc, device, ta, tb, B, M, N, K):
    a = _rand((B, K, M) if ta else (B, M, K), torch.bfloat16, device, 14)
    b = _rand((B, N, K) if tb else (B, K, N), torch.bfloat16, device, 15)
    out = catcoc.batched_matmul(a, b, trans_a=ta, trans_b=tb)
    _sync(device, "batched")
    ref = torch.bmm((a.transpose(1, 2) if ta else a).float(), (b.transpose(1, 2) if tb else b).float())
    assert out.shape == (B, M, N)
    _close(out, ref, K)


def test_batched_matmul_pairs(catcoc, device):
    B, M, N, K = 4, 512, 512, 256
    a, b = _rand((B, M, K), torch.float16, device, 16), _rand((B, K, N), torch.float16, device, 17)
    out = catcoc.batched_matmul(a, b, tiling=catcoc.TilingConfig(cta_pair=2, bn=128))
    _sync(device, "batched pairs")
    _close(out, torch.bmm(a.float(), b.float()), K)


@pytest.mark.parametrize("tb", [False, True])
@pytest.mark.parametrize("sizes", [[128, 256, 64], [5, 0, 300, 129, 1], [0, 0, 700], [33] * 9])
@pytest.mark.parametrize("on_device", [False, True])
def test_grouped_matmul(catcoc, device, tb, sizes, on_device):
    G, N, K = len(sizes), 264, 192
    total = sum(sizes)
    ends = torch.tensor(sizes).cumsum(0)
    a = _rand((total, K), torch.bfloat16, device, 18)
    b = _rand((G, N, K) if tb else (G, K, N), torch.bfloat16, device, 19)
    gl = ends.to(device) if on_device else ends.tolist()
    out = catcoc.grouped_matmul(a, b, gl, trans_b=tb)
    _sync(device, "grouped")
    ref = torch.empty((total, N), device=device)
    begin = 0
    for g, end in enumerate(ends.tolist()):
        ref[begin:end] = a[begin:end].float() @ (b[g].t() if tb else b[g]).float()
        begin = end
    _close(out, ref, K)


def test_grouped_matmul_pair_tiles_and_short_list(catcoc, device):
    """256-row pair tiles over ragged groups, and rows past the last group stay untouched."""
    sizes, N, K = [300, 512, 40], 256, 128
    total = sum(sizes) + 100
    ends = torch.tensor(sizes).cumsum(0)
    a = _rand((total, K), torch.float16, device, 20)
    b = _rand((3, K, N), torch.float16, device, 21)
    out = torch.full((total, N), 7.0, dtype=torch.float16, device=device)
    catcoc.grouped_matmul(a, b, ends.to(device), out=out, tiling=catcoc.TilingConfig(cta_pair=2, bn=128))
    _sync(device, "grouped pairs")
    begin = 0
    for g, end in enumerate(ends.tolist()):
        _close(out[begin:end], a[begin:end].float() @ b[g].float(), K)
        begin = end
    assert bool((out[begin:] == 7.0).all())


def test_grouped_quant_matmul(catcoc, device):
    sizes, N, K = [130, 7, 0, 260], 384, 256
    G, total = len(sizes), sum(sizes)
    g = torch.Generator().manual_seed(22)
    x1 = torch.randint(-8, 8, (total, K), generator=g, dtype=torch.int8).to(device)
    x2 = torch.randint(-8, 8, (G, K, N), generator=g, dtype=torch.int8).to(device)
    st = torch.rand(total, device=device) * 0.01 + 0.001
    sc = torch.rand(G, N, device=device) + 0.5
    ends = torch.tensor(sizes).cumsum(0)
    out = catcoc.grouped_quant_matmul(x1, x2, st, sc, ends.to(device))
    _sync(device, "grouped quant")
    begin = 0
    for gi, end in enumerate(ends.tolist()):
        ref = (x1[begin:end].float() @ x2[gi].float()) * st[begin:end, None] * sc[gi][None, :]
        _close(out[begin:end], ref, K)
        begin = end


def test_grouped_matmul_slice_k_and_group_gemm(catcoc, device):
    M, N = 136, 264
    ks = [64, 0, 200, 72]
    ends = torch.tensor(ks).cumsum(0).tolist()
    a = _rand((sum(ks), M), torch.bfloat16, device, 23)
    b = _rand((sum(ks), N), torch.bfloat16, device, 24)
    out = catcoc.grouped_matmul_slice_k(a, b, ends)
    _sync(device, "slice k")
    begin = 0
    for g, end in enumerate(ends):
        _close(out[g], a[begin:end].float().t() @ b[begin:end].float(), max(1, end - begin))
        begin = end
    problems = [dict(a=_rand((64, 96), torch.float16, device, 25), b=_rand((96, 40), torch.float16, device, 26)),
                dict(a=_rand((300, 128), torch.float16, device, 27), b=_rand((128, 520), torch.float16, device, 28),
                     c=_rand((300, 520), torch.float16, device, 29), alpha=1.5, beta=0.5)]
    outs = catcoc.group_gemm(problems)
    _sync(device, "group gemm")
    _close(outs[0], problems[0]["a"].float() @ problems[0]["b"].float(), 96)
    _close(outs[1], 1.5 * (problems[1]["a"].float() @ problems[1]["b"].float()) + 0.5 * problems[1]["c"].float(), 128)


@pytest.mark.parametrize("ta,tb", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("M,N,K,S", [(128, 256, 4096, 4), (100, 136, 3000, 5), (256, 512, 1024, None), (8, 24, 2056, 3)])
def test_splitk_matmul(catcoc, device, ta, tb, M, N, K, S):
    a = _rand((K, M) if ta else (M, K), torch.bfloat16, device, 30)
    b = _rand((N, K) if tb else (K, N), torch.bfloat16, device, 31)
    c = _rand((M, N), torch.bfloat16, device, 32)
    bias = _rand((N,), torch.float32, device, 33)
    out = catcoc.splitk_matmul(a, b, split_k=S, trans_a=ta, trans_b=tb, alpha=0.5, beta=2.0, c=c, bias_f32=bias)
    _sync(device, "split-k")
    ref = 0.5 * ((a.t() if ta else a).float() @ (b.t() if tb else b).float()) + 2.0 * c.float() + bias[None, :]
    _close(out, ref, K)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("rows,cols", [(4096, 1024), (7, 5000), (1300, 77), (1, 1), (2048, 4100)])
@pytest.mark.parametrize("trans", [False, True])
def test_gemv(catcoc, device, dtype, rows, cols, trans):
    a = _rand((rows, cols), dtype, device, 34)
    n_in, n_out = (rows, cols) if trans else (cols, rows)
    x = _rand((n_in,), dtype, device, 35)
    y = _rand((n_out,), dtype, device, 36)
    out = catcoc.gemv(a, x, y, alpha=0.75, beta=-0.5, trans=trans)
    torch.cuda.synchronize()
    ref = 0.75 * ((a.t() if trans else a).float() @ x.float()) - 0.5 * y.float()
    _close(out, ref, n_in)
    out2 = catcoc.gemv(a.t(), x, trans=not trans)      # a column-major view of the same product
    torch.cuda.synchronize()
    _close(out2, (a.t() if trans else a).float() @ x.float(), n_in)

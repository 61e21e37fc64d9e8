"""Numerics of the tcgen05 kernel on one GPU against a plain fp32 PyTorch reference: every
operand layout, dtype, tile width, CTA pairing and ragged shape, plus the W = 1 path of the
fused ops and the heap primitives in a single process."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(a, b, ta, tb):
    return (a.t() if ta else a).float() @ (b.t() if tb else b).float()


@pytest.fixture(scope="module")
def catcoc(device):
    import mm_rs_with_catlass_b200 as c
    return c


def _check_status(device, what):
    from mm_rs_with_catlass_b200.ops._common import local_status, raise_on_status
    torch.cuda.synchronize()
    raise_on_status(local_status(device), what)


LAYOUTS = [(False, False), (False, True), (True, False), (True, True)]


@pytest.mark.parametrize("ta,tb", LAYOUTS)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("pair", [1, 2])
def test_layouts_and_dtypes(catcoc, device, ta, tb, dtype, pair):
    from mm_rs_with_catlass_b200.utils.data import matmul_inputs
    from mm_rs_with_catlass_b200.utils.verify import assert_close
    M, N, K = 512, 768, 320
    a, b = matmul_inputs(M, N, K, 0, dtype, device, trans_a=ta, trans_b=tb)
    out = catcoc.matmul(a, b, trans_a=ta, trans_b=tb, tiling=catcoc.TilingConfig(cta_pair=pair))
    _check_status(device, "gemm")
    assert_close(out, _ref(a, b, ta, tb), k=K, what="layout %s%s" % (ta, tb))


@pytest.mark.parametrize("M,N,K", [(23, 45, 68), (4, 128, 129), (200, 328, 136), (129, 257, 65), (1024, 5120, 6148),
                                   (1, 8, 8), (300, 8, 1000)])
@pytest.mark.parametrize("bn,pair", [(0, 1), (64, 1), (128, 2)])
def test_ragged_shapes(catcoc, device, M, N, K, bn, pair):
    """Shapes the reference records as failing or hanging (23x45x68, 4x128x129) and its
    unaligned-K all-gather shape (K = 6148) go through the pad / clip paths here."""
    from mm_rs_with_catlass_b200.utils.data import matmul_inputs
    from mm_rs_with_catlass_b200.utils.verify import assert_close
    a, b = matmul_inputs(M, N, K, 0, torch.bfloat16, device)
    out = catcoc.matmul(a, b, tiling=catcoc.TilingConfig(bn=bn, cta_pair=pair))
    _check_status(device, "ragged gemm")
    assert out.shape == (M, N)
    assert_close(out, _ref(a, b, False, False), k=K)


def test_strided_views_and_out_argument(catcoc, device):
    from mm_rs_with_catlass_b200.utils.verify import assert_close
    big = torch.randn(300, 700, device=device).bfloat16()
    a = big[:256, 100:612]                    # row pitch 700: needs the pad copy
    bt = (torch.randn(384, 512, device=device) * 0.05).bfloat16().t()   # column-major view -> folded into trans_b
    out = torch.empty(256, 384, dtype=torch.bfloat16, device=device)
    r = catcoc.matmul(a, bt, out=out)
    assert r is out
    _check_status(device, "views")
    assert_close(out, a.float() @ bt.float(), k=512)
    with pytest.raises(ValueError):
        catcoc.matmul(a, bt, out=torch.empty(8, 8, dtype=torch.bfloat16, device=device))
    with pytest.raises(TypeError):
        catcoc.matmul(a, bt.float())


@pytest.mark.parametrize("tb", [False, True])
@pytest.mark.parametrize("pair", [1, 2])
def test_int8_exact_and_dequant(catcoc, device, tb, pair):
    from mm_rs_with_catlass_b200.utils.data import quant_inputs
    M, N, K = 384, 512, 640
    x1, x2, s1, s2, bias = quant_inputs(M, N, K, 0, device, trans_b=tb)
    acc = catcoc.matmul(x1, x2, trans_b=tb, bias=bias, tiling=catcoc.TilingConfig(cta_pair=pair))
    _check_status(device, "int8")
    ref = x1.double() @ (x2.t() if tb else x2).double() + bias.double()[None, :]
    assert acc.dtype == torch.int32 and torch.equal(acc.double(), ref)
    deq = catcoc.matmul(x1, x2, trans_b=tb, bias=bias, scale_m=s1, scale_n=s2, out_dtype=torch.float32,
                        tiling=catcoc.TilingConfig(cta_pair=pair))
    _check_status(device, "int8 dequant")
    exp = (ref * s2.double()[None, :] * s1.double()[:, None]).float()
    assert torch.allclose(deq, exp, rtol=1e-5, atol=1e-6)


@pytest.mark.skipif(not hasattr(torch, "float8_e4m3fn"), reason="no fp8 dtype in this torch")
def test_fp8_operands(catcoc, device):
    M, N, K = 256, 256, 512
    a = (torch.randn(M, K, device=device) * 0.5).to(torch.float8_e4m3fn)
    b = (torch.randn(N, K, device=device) * 0.5).to(torch.float8_e4m3fn)
    out = catcoc.matmul(a, b, trans_b=True, out_dtype=torch.bfloat16)
    _check_status(device, "fp8")
    ref = a.float() @ b.float().t()
    assert torch.allclose(out.float(), ref, rtol=2e-2, atol=2e-2 * ref.abs().max().item())


@pytest.mark.skipif(not hasattr(torch, "float8_e4m3fn"), reason="no fp8 dtype in this torch")
@pytest.mark.parametrize("M,N,K", [(128, 128, 128), (256, 384, 1024), (200, 328, 160), (1, 8, 32), (513, 130, 4096)])
@pytest.mark.parametrize("fmt", ["e4m3", "e5m2"])
def test_block_scaled_fp8(catcoc, device, M, N, K, fmt):
    """mxf8: one UE8M0 scale per 32 K-elements, applied by the tensor core from TMEM. Scales are
    spread over 12 binades across rows and K-blocks, so any mix-up of rows, blocks or operands
    shows as an error of order one."""
    g = torch.Generator(device=device)
    g.manual_seed(M + N + K)
    a = torch.randn(M, K, device=device, generator=g)
    b = torch.randn(N, K, device=device, generator=g) * 0.1
    a = a * torch.exp2(torch.randint(-6, 6, (M, K // 32), device=device, generator=g).float()).repeat_interleave(32, 1)
    b = b * torch.exp2(torch.randint(-4, 4, (N, K // 32), device=device, generator=g).float()).repeat_interleave(32, 1)
    aq, sa = catcoc.quantize_mxf8(a, fmt)
    bq, sb = catcoc.quantize_mxf8(b, fmt)
    ref = catcoc.dequantize_mxf8(aq, sa) @ catcoc.dequantize_mxf8(bq, sb).t()
    out = catcoc.mxf8_matmul(aq, catcoc.pack_scales(sa), bq, catcoc.pack_scales(sb), out_dtype=torch.float32)
    _check_status(device, "mxf8")
    assert (out - ref).abs().max().item() <= 1e-4 * ref.abs().max().item()
    out16 = catcoc.mxf8_matmul(aq, catcoc.pack_scales(sa), bq, catcoc.pack_scales(sb))
    _check_status(device, "mxf8 bf16")
    assert out16.dtype == torch.bfloat16
    assert (out16.float() - ref).abs().max().item() <= 2 ** -7 * ref.abs().max().item()


def test_repeated_launches_alternating_shapes(catcoc, device):
    """Back-to-back launches on one stream with changing shapes: stale barrier / TMEM state
    from one launch must not leak into the next."""
    from mm_rs_with_catlass_b200.utils.data import matmul_inputs
    from mm_rs_with_catlass_b200.utils.verify import assert_close
    shapes = [(256, 256, 128), (130, 520, 72), (512, 256, 256)]
    data = [matmul_inputs(m, n, k, 0, torch.bfloat16, device, seed=i) for i, (m, n, k) in enumerate(shapes)]
    outs = []
    for it in range(34):
        a, b = data[it % 3]
        outs.append((it % 3, catcoc.matmul(a, b, tiling=catcoc.TilingConfig(cta_pair=1 + it % 2))))
    _check_status(device, "repeat")
    for idx, o in outs:
        a, b = data[idx]
        assert_close(o, a.float() @ b.float(), k=shapes[idx][2])


def test_world1_fused_ops_and_heap(catcoc, device):
    from mm_rs_with_catlass_b200.ops import reference
    from mm_rs_with_catlass_b200.utils.data import matmul_inputs, quant_inputs
    from mm_rs_with_catlass_b200.utils.verify import assert_close
    ctx = catcoc.init(heap_bytes=64 << 20, make_default=False)
    try:
        assert ctx.world == 1 and ctx.heap_bytes >= 64 << 20
        a, b = matmul_inputs(256, 384, 512, 0, torch.bfloat16, device)
        gold = a.float() @ b.float()
        assert_close(catcoc.matmul_reduce_scatter(a, b, ctx=ctx), gold, k=512)
        assert_close(catcoc.matmul_allreduce(a, b, ctx=ctx), gold, k=512)
        out, g = catcoc.allgather_matmul(a, b, ctx=ctx)
        assert_close(out, gold, k=512)
        assert g.data_ptr() == a.data_ptr()
        x1, x2, s1, s2, bias = quant_inputs(256, 384, 512, 0, device)
        q = catcoc.quant_matmul_reduce_scatter(x1, x2, s1, s2, bias, ctx=ctx)
        assert_close(q, reference.quant_matmul_reduce_scatter(x1, x2, s1, s2, bias, out_dtype=torch.float32), k=512,
                     dtype=torch.bfloat16)
        # heap: allocation, views, put / get to self, signal + bounded wait, barrier
        buf = ctx.malloc(1 << 16)
        sig = ctx.malloc(64)
        assert buf.offset % 256 == 0 and buf.ptr() == ctx.base(0) + buf.offset
        src = torch.arange(1 << 14, dtype=torch.int32, device=device)
        ctx.put(0, buf, src, signal=sig, signal_value=1)
        ctx.wait_until(sig, ctx.put_blocks(), timeout_ms=2000)
        ctx.barrier()
        back = torch.empty_like(src)
        ctx.get(0, back, buf)
        ctx.check("heap primitives")
        assert torch.equal(buf.tensor(torch.int32, (1 << 14,)), src) and torch.equal(back, src)
        with pytest.raises(catcoc.ShmemError):
            ctx.malloc(1 << 40)
    finally:
        ctx.finalize()
        ctx.finalize()      # idempotent


def test_bounded_wait_reports_a_status_instead_of_hanging(catcoc, device):
    """A wait on a signal nothing ever sets gives up after its budget; the kernel returns, the
    host reads an error status and the context stays usable."""
    ctx = catcoc.init(heap_bytes=16 << 20, make_default=False)
    try:
        sig = ctx.malloc(64)
        ctx.wait_until(sig, 1, timeout_ms=20)
        with pytest.raises(RuntimeError, match="timed out"):
            ctx.check("wait_until")
        # still alive: the next kernel runs normally
        a = torch.randn(128, 64, device=device).bfloat16()
        b = torch.randn(64, 128, device=device).bfloat16()
        o = catcoc.matmul(a, b)
        ctx.check("after timeout")
        assert torch.isfinite(o.float()).all()
    finally:
        ctx.finalize()


def test_flagship_block_world1(catcoc, device):
    from mm_rs_with_catlass_b200.models.tp_mlp import TPMLP, TPMLPConfig
    from mm_rs_with_catlass_b200.utils.verify import assert_close
    mlp = TPMLP(TPMLPConfig(hidden=512, ffn=1536), None, device)
    x = torch.randn(384, 512, device=device).bfloat16()
    assert_close(mlp(x), mlp.reference_forward(x).float(), k=1536)
    _check_status(device, "tpmlp")


def test_launch_plans_follow_the_data_not_the_first_call(catcoc, device):
    """A repeated call reuses its argument block (a launch plan): new contents at the same
    addresses must give new results, a new output must be written, and an operand that needs a
    padded copy is re-read on every call."""
    from mm_rs_with_catlass_b200.ops import gemm as G
    from mm_rs_with_catlass_b200.utils.verify import assert_close
    a = torch.randn(256, 192, device=device).bfloat16()
    b = torch.randn(192, 320, device=device).bfloat16()
    G._plans.clear()
    o1 = catcoc.matmul(a, b)
    n_plans = len(G._plans)
    assert n_plans == 1
    a.copy_(torch.randn(256, 192, device=device).bfloat16())
    o2 = catcoc.matmul(a, b)                       # plan hit, fresh output tensor
    assert len(G._plans) == n_plans and o2.data_ptr() != o1.data_ptr()
    _check_status(device, "plan hit")
    assert_close(o2, a.float() @ b.float(), k=192)
    out = torch.empty(256, 320, dtype=torch.bfloat16, device=device)
    assert catcoc.matmul(a, b, out=out) is out     # another key: the output is part of it
    assert catcoc.matmul(a, b, out=out) is out
    _check_status(device, "plan hit with out")
    assert_close(out, a.float() @ b.float(), k=192)
    # an A whose base TMA cannot address is padded inside the launch (from the caller's memory, on every
    # call): planned like any other operand, and still always current
    big = torch.randn(256, 200, device=device).bfloat16()
    av = big[:, 3:195]
    before = len(G._plans)
    r1 = catcoc.matmul(av, b)
    big.mul_(2.0)
    r2 = catcoc.matmul(av, b)
    _check_status(device, "padded operand")
    assert len(G._plans) == before + 1
    assert_close(r2, av.float() @ b.float(), k=192)
    assert not torch.equal(r1, r2)
    # a B that needs a padded copy still goes through the pad kernel: never planned, always current
    bbig = torch.randn(192, 330, device=device).bfloat16()
    bv = bbig[:, 5:325]
    before = len(G._plans)
    r1 = catcoc.matmul(a, bv)
    bbig.mul_(2.0)
    r2 = catcoc.matmul(a, bv)
    _check_status(device, "padded B")
    assert len(G._plans) == before
    assert_close(r2, a.float() @ bv.float(), k=192)
    assert not torch.equal(r1, r2)


@pytest.mark.parametrize("act", ["gelu", "silu", "relu"])
@pytest.mark.parametrize("pair", [1, 2])
def test_activation_in_the_epilogue(catcoc, act, pair):
    """The activation runs on the fp32 accumulator, before the single rounding to the output dtype."""
    from mm_rs_with_catlass_b200.ops._common import apply_activation
    from mm_rs_with_catlass_b200.utils.verify import assert_close
    dev = torch.device("cuda:0")
    a = torch.randn(384, 256, device=dev).to(torch.bfloat16)
    b = (torch.randn(256, 328, device=dev) * 0.2).to(torch.bfloat16)
    out = catcoc.matmul(a, b, activation=act, tiling=catcoc.TilingConfig(bn=128, cta_pair=pair))
    gold = apply_activation(a.float() @ b.float(), act)
    assert_close(out, gold, k=256, dtype=torch.bfloat16, what="matmul + " + act)
    with pytest.raises(ValueError):
        catcoc.matmul(a, b, activation="tanh")


def test_unaligned_a_is_padded_inside_the_launch(catcoc):
    """An A whose row pitch (or base) is not a multiple of 16 bytes is padded by the kernel's own
    communication warps while the product already runs: no padded copy is made beforehand, the
    call is planned, and repeated calls (alternating workspace halves) stay correct."""
    from mm_rs_with_catlass_b200.ops import gemm as G
    from mm_rs_with_catlass_b200.utils.verify import assert_close
    dev = torch.device("cuda:0")
    for (m, n, k, off) in [(300, 256, 6148 // 4, 0), (513, 136, 250, 0), (129, 64, 72, 1), (64, 512, 1030, 3)]:
        storage = torch.randn(m * k + 8, device=dev).to(torch.bfloat16)
        a = storage[off:off + m * k].view(m, k)          # `off` elements into the storage: 2-byte aligned base
        b = (torch.randn(k, n, device=dev) * 0.1).to(torch.bfloat16)
        assert G._wants_pad_prologue(a)
        plans_before = len(G._plans)
        for rep in range(3):
            out = catcoc.matmul(a, b)
            assert_close(out, a.float() @ b.float(), k=k, dtype=torch.bfloat16, what="pad prologue %dx%dx%d" % (m, n, k))
        assert len(G._plans) == plans_before + 1          # planned once, hit afterwards
    _check_status(dev, "pad prologue")
    # with scales (int8) the same path feeds the quantised epilogue
    x1 = torch.randint(-127, 128, (200, 300), device=dev, dtype=torch.int32).to(torch.int8)   # 300-byte rows
    x2 = torch.randint(-127, 128, (300, 256), device=dev, dtype=torch.int32).to(torch.int8)
    assert G._wants_pad_prologue(x1)
    out = catcoc.matmul(x1, x2)
    assert torch.equal(out.cpu().long(), x1.cpu().long() @ x2.cpu().long())
    _check_status(dev, "pad prologue int8")

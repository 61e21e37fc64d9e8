"""Flash attention forward (tcgen05 QK^T and PV with P read from TMEM, two query tiles per CTA,
online softmax with a lazily moved reference maximum and the accumulator rescaled in TMEM)
against a plain fp32 PyTorch reference: head dimensions, dtypes, ragged sequence lengths, causal
masks with and without a cache offset, grouped-query heads, score ranges that do and do not
move the reference maximum."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _run(b, hq, hk, sq, sk, d, dtype, causal, seed=0, key_gain=None):
    import mm_rs_with_catlass_b200 as catcoc
    from mm_rs_with_catlass_b200.ops.attention import attention_reference
    from mm_rs_with_catlass_b200.ops._common import local_status, raise_on_status
    dev = torch.device("cuda:0")
    g = torch.Generator(device=dev)
    g.manual_seed(seed)
    q = torch.randn(b, hq, sq, d, device=dev, generator=g).to(dtype)
    k = torch.randn(b, hk, sk, d, device=dev, generator=g).to(dtype)
    v = torch.randn(b, hk, sk, d, device=dev, generator=g).to(dtype)
    if key_gain is not None:
        # keys grow (or shrink) along the sequence: the row maxima of later blocks sit far above (below) the earlier ones
        ramp = torch.linspace(key_gain[0], key_gain[1], sk, device=dev)[None, None, :, None]
        k = (k.float() * ramp).to(dtype)
    out = catcoc.flash_attention(q, k, v, causal=causal)
    torch.cuda.synchronize()
    raise_on_status(local_status(dev), "flash_attention")
    gold = attention_reference(q, k, v, causal=causal)
    err = (out.float() - gold).abs().max().item()
    # probabilities are rounded to the operand dtype before the second product
    tol = 2.5e-2 if dtype == torch.bfloat16 else 4e-3
    assert torch.isfinite(out.float()).all()
    assert err < tol, "max |err| %.4g (tolerance %.3g)" % (err, tol)


@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("causal", [False, True])
def test_aligned_sequences(d, dtype, causal):
    _run(2, 4, 4, 256, 256, d, dtype, causal)


@pytest.mark.parametrize("sq,sk", [(1, 1), (1, 300), (77, 77), (128, 129), (200, 456), (384, 1000)])
@pytest.mark.parametrize("causal", [False, True])
def test_ragged_lengths_and_cache_offsets(sq, sk, causal):
    _run(1, 2, 2, sq, sk, 128, torch.bfloat16, causal, seed=sq + sk)


def test_grouped_query_heads_share_key_value_heads():
    _run(2, 8, 2, 192, 320, 128, torch.bfloat16, True, seed=5)
    _run(1, 6, 3, 130, 130, 64, torch.float16, False, seed=6)


@pytest.mark.parametrize("sq,sk", [(256, 256), (257, 257), (500, 500), (700, 1300), (1024, 1024)])
@pytest.mark.parametrize("causal", [False, True])
def test_several_ctas_and_a_ragged_second_tile(sq, sk, causal):
    _run(2, 3, 3, sq, sk, 128, torch.bfloat16, causal, seed=sq)
    _run(1, 2, 1, sq, sk, 64, torch.float16, causal, seed=sq + 1)


@pytest.mark.parametrize("gain", [(0.2, 6.0), (6.0, 0.2), (1.0, 1.0)])
@pytest.mark.parametrize("causal", [False, True])
def test_reference_maximum_moves_or_stays(gain, causal):
    # growing keys force a rescale of O in almost every block, shrinking keys none after the first
    _run(1, 2, 2, 384, 1536, 128, torch.bfloat16, causal, seed=11, key_gain=gain)
    _run(1, 2, 2, 384, 1536, 64, torch.float16, causal, seed=12, key_gain=gain)


def test_long_sequence_many_blocks():
    _run(1, 2, 1, 512, 4096, 128, torch.bfloat16, True, seed=9)


def test_argument_checks():
    import mm_rs_with_catlass_b200 as catcoc
    dev = torch.device("cuda:0")
    q = torch.randn(1, 2, 16, 96, device=dev).bfloat16()
    with pytest.raises(ValueError):
        catcoc.flash_attention(q, q, q)                       # head dimension 96
    q = torch.randn(1, 3, 16, 64, device=dev).bfloat16()
    k = torch.randn(1, 2, 16, 64, device=dev).bfloat16()
    with pytest.raises(ValueError):
        catcoc.flash_attention(q, k, k)                       # 3 query heads over 2 key / value heads
    with pytest.raises(ValueError):
        catcoc.flash_attention(q[:, :2], k[:, :, :8], k[:, :, :8], causal=True)   # causal with Sk < Sq
    with pytest.raises(ValueError):
        catcoc.flash_attention(k, k, k, scale=-1.0)           # the kernel takes the row maximum before scaling

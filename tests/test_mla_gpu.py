"""Multi-head latent attention decode (paged latent cache, 576-wide keys, 512-wide values, P read
from TMEM, flash-decoding slices) against a plain fp32 PyTorch reference built the way the
reference's data generator builds its golden (3rdparty/catlass/examples/19_mla/gen_data.py)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(batch, q_len, heads, kv_lens, dtype, causal=False, splits=None, seed=0, shuffle_pages=True):
    import mm_rs_with_catlass_b200 as catcoc
    from mm_rs_with_catlass_b200.ops.mla import mla_decode_reference
    from mm_rs_with_catlass_b200.ops._common import local_status, raise_on_status
    dev = torch.device("cuda:0")
    g = torch.Generator(device=dev)
    g.manual_seed(seed)
    max_pages = max(1, (max(kv_lens) + 127) // 128)
    num_pages = batch * max_pages + 3
    u = lambda *shape: (torch.rand(*shape, device=dev, generator=g) * 2 - 1).to(dtype)
    q_nope, q_rope = u(batch * q_len, heads, 512), u(batch * q_len, heads, 64)
    ckv, krope = u(num_pages, 128, 512), u(num_pages, 128, 64)
    perm = torch.randperm(num_pages, device=dev, generator=g) if shuffle_pages else torch.arange(num_pages, device=dev)
    table = perm[:batch * max_pages].reshape(batch, max_pages).to(torch.int32)
    lens = torch.tensor(kv_lens, dtype=torch.int32, device=dev)
    out = catcoc.mla_decode(q_nope, q_rope, ckv, krope, table, lens, q_len=q_len, causal=causal, splits=splits)
    torch.cuda.synchronize()
    raise_on_status(local_status(dev), "mla_decode")
    gold = mla_decode_reference(q_nope, q_rope, ckv, krope, table, lens, q_len=q_len, causal=causal)
    assert torch.isfinite(out.float()).all()
    err = (out.float() - gold).abs().max().item()
    tol = 1.5e-2 if dtype == torch.bfloat16 else 3e-3
    assert err < tol, "max |err| %.4g (tolerance %.3g)" % (err, tol)


@pytest.mark.parametrize("heads", [16, 32, 64, 128])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_head_counts_one_slice(heads, dtype):
    _case(2, 1, heads, [128, 300], dtype, splits=1, seed=heads)


@pytest.mark.parametrize("kv_lens", [[1], [31, 32, 33], [127, 128, 129], [1000, 17, 513], [4096, 2050]])
@pytest.mark.parametrize("splits", [1, 3, None])
def test_ragged_lengths_and_slices(kv_lens, splits):
    _case(len(kv_lens), 1, 16, kv_lens, torch.bfloat16, splits=splits, seed=sum(kv_lens))
    _case(len(kv_lens), 1, 128, kv_lens, torch.float16, splits=splits, seed=sum(kv_lens) + 1)


@pytest.mark.parametrize("q_len", [2, 3, 4])
@pytest.mark.parametrize("causal", [False, True])
def test_several_new_tokens_with_and_without_mask(q_len, causal):
    _case(2, q_len, 16, [260, 75], torch.bfloat16, causal=causal, seed=q_len)        # 32 to 64 rows: the 64-row form
    _case(2, q_len, 128, [260, 75], torch.bfloat16, causal=causal, splits=2, seed=q_len + 10)   # several 128-row chunks


def test_the_reference_example_shape():
    # batch 1, one new token, 128 keys, 16 heads, 16 pages of 128: the command line of the reference's README
    _case(1, 1, 16, [128], torch.float16, splits=1, seed=1, shuffle_pages=False)


def test_argument_checks():
    import mm_rs_with_catlass_b200 as catcoc
    dev = torch.device("cuda:0")
    qn = torch.zeros(2, 16, 512, device=dev, dtype=torch.bfloat16)
    qr = torch.zeros(2, 16, 64, device=dev, dtype=torch.bfloat16)
    ckv = torch.zeros(4, 128, 512, device=dev, dtype=torch.bfloat16)
    kr = torch.zeros(4, 128, 64, device=dev, dtype=torch.bfloat16)
    table = torch.zeros(2, 2, device=dev, dtype=torch.int32)
    lens = torch.tensor([5, 5], device=dev, dtype=torch.int32)
    with pytest.raises(ValueError):
        catcoc.mla_decode(qn, qr, ckv[:, :64], kr, table, lens)               # pages of 64 keys
    with pytest.raises(TypeError):
        catcoc.mla_decode(qn, qr, ckv, kr, table.long(), lens)                # int64 block table
    with pytest.raises(ValueError):
        catcoc.mla_decode(qn, qr, ckv, kr, table, lens, q_len=5)
    with pytest.raises(ValueError):
        catcoc.mla_decode(qn, qr, ckv, kr, table[:1], lens)                   # one table row for two sequences

"""Host-side pieces of the latent-attention decode op: the PyTorch golden against a dense
computation without pages, and the choice of slices per sequence."""
import math

import torch

from mm_rs_with_catlass_b200.ops.mla import mla_decode_reference, _pick_splits


def test_golden_matches_a_dense_computation_without_pages():
    torch.manual_seed(0)
    batch, q_len, heads, pages_per_seq = 2, 2, 3, 2
    lens = [130, 77]
    num_pages = batch * pages_per_seq
    q_nope, q_rope = torch.randn(batch * q_len, heads, 512), torch.randn(batch * q_len, heads, 64)
    ckv, krope = torch.randn(num_pages, 128, 512), torch.randn(num_pages, 128, 64)
    table = torch.tensor([[3, 1], [0, 2]], dtype=torch.int32)
    for causal in (False, True):
        got = mla_decode_reference(q_nope, q_rope, ckv, krope, table, torch.tensor(lens, dtype=torch.int32), q_len=q_len,
                                   causal=causal)
        for b in range(batch):
            keys = torch.cat([torch.cat([ckv[p], krope[p]], dim=1) for p in table[b].tolist()], dim=0)[:lens[b]]
            for t in range(q_len):
                n_vis = lens[b] - (q_len - 1 - t) if causal else lens[b]
                for h in range(heads):
                    q = torch.cat([q_nope[b * q_len + t, h], q_rope[b * q_len + t, h]])
                    s = (keys[:n_vis] @ q) / math.sqrt(576.0)
                    want = torch.softmax(s, dim=0) @ keys[:n_vis, :512]
                    assert torch.allclose(got[b * q_len + t, h], want, atol=1e-4, rtol=1e-4)


def test_golden_accepts_a_singleton_head_dimension_and_empty_sequences():
    q_nope, q_rope = torch.randn(2, 4, 512), torch.randn(2, 4, 64)
    ckv, krope = torch.randn(2, 128, 1, 512), torch.randn(2, 128, 1, 64)
    table = torch.tensor([[0], [1]], dtype=torch.int32)
    out = mla_decode_reference(q_nope, q_rope, ckv, krope, table, torch.tensor([0, 5], dtype=torch.int32))
    assert torch.count_nonzero(out[0]) == 0 and torch.isfinite(out).all() and torch.count_nonzero(out[1]) > 0


def test_slices_fill_whole_waves_without_exceeding_the_pages():
    assert _pick_splits(batch=1, rows_per_item=16, max_pages=1) == 1          # a 128-key sequence cannot be cut
    assert _pick_splits(batch=1, rows_per_item=16, max_pages=64) == 64        # one sequence: as many slices as allowed
    assert _pick_splits(batch=256, rows_per_item=128, max_pages=32) <= 2      # several waves already
    s = _pick_splits(batch=32, rows_per_item=16, max_pages=32)                # 64 CTAs per slice count
    assert s == 2 and 64 * s <= 148                                           # one full wave beats 2.2 waves of 5 slices
    for batch, rows, pages in [(8, 128, 32), (3, 64, 17), (128, 16, 16)]:
        s = _pick_splits(batch, rows, pages)
        assert 1 <= s <= pages

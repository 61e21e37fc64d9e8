"""Host-side rules of the kernel catalogue that need no GPU: split-K sizing, argument checks and
the refusal of CPU tensors."""
import pytest
import torch

from mm_rs_with_catlass_b200.ops import blas


def test_pick_split_k_fills_the_machine_without_starving_a_slice():
    assert blas.pick_split_k(8192, 8192, 8192, 2) == 1            # plenty of tiles already
    s = blas.pick_split_k(128, 1024, 16384, 2)
    assert 4 <= s <= 32 and 16384 // s >= 4 * 128                 # every slice keeps >= 4 pipeline stages
    assert blas.pick_split_k(128, 8192, 1024, 2) <= 2             # K too short to cut further
    assert blas.pick_split_k(256, 256, 32768, 1) >= 8             # 8-bit operands: 256-element stages


def test_argument_checks_come_before_any_launch():
    a = torch.randn(4, 8)
    with pytest.raises(ValueError, match="beta"):
        blas.gemm(a, a.t(), None, beta=1.0)
    with pytest.raises(ValueError, match="vector"):
        blas.matmul_bias(a, a.t(), torch.zeros(2, 2))
    with pytest.raises(ValueError, match="equal B"):
        blas.batched_matmul(torch.zeros(2, 4, 8), torch.zeros(3, 8, 4))
    with pytest.raises(ValueError, match="inner dimensions"):
        blas.batched_matmul(torch.zeros(2, 4, 8), torch.zeros(2, 6, 4))
    with pytest.raises(ValueError, match="grouped_matmul takes"):
        blas.grouped_matmul(torch.zeros(2, 4, 8), torch.zeros(3, 8, 4), [1, 2, 3])
    with pytest.raises(TypeError, match="int8"):
        blas.grouped_quant_matmul(a, torch.zeros(1, 8, 4), torch.ones(4), torch.ones(1, 4), [4])
    with pytest.raises(ValueError, match="matrix and a vector"):
        blas.gemv(torch.zeros(4), torch.zeros(4))


def test_cpu_tensors_are_refused():
    a, b = torch.randn(8, 8).half(), torch.randn(8, 8).half()
    for call in (lambda: blas.gemm(a, b), lambda: blas.batched_matmul(a[None], b[None]),
                 lambda: blas.grouped_matmul(a, b[None], [8]), lambda: blas.splitk_matmul(a, b, split_k=2),
                 lambda: blas.gemv(a, a[0])):
        with pytest.raises(RuntimeError, match="CUDA"):
            call()


def test_slices_are_whole_pipeline_stages_and_cover_k():
    for k, s, elt in [(14336, 4, 2), (7168, 16, 2), (1000, 3, 2), (8192, 5, 1), (96, 8, 2)]:
        ks, n = blas.slice_k(k, s, elt)
        assert ks % (256 // elt) == 0                  # a slice is a whole number of 256-byte K stages
        assert (n - 1) * ks < k <= n * ks and n <= s   # the slices cover K, the last one may be short


def test_splitk_plan_prefers_wide_tiles_cut_into_more_slices():
    # 128 x 8192 x 14336: 32 tiles of 256 columns x 4 slices stream (128 + 256) * 3584 elements per CTA,
    # 64 tiles of 128 columns x 2 slices (128 + 128) * 7168: the wide tiles win
    assert blas.splitk_plan(128, 8192, 14336, 2) == (4, 256)
    s, bn = blas.splitk_plan(128, 8192, 7168, 2)
    assert bn == 256 and s == 4
    # nothing to cut: a short K, or tiles enough for every SM
    assert blas.splitk_plan(128, 8192, 256, 2)[0] == 1
    assert blas.splitk_plan(4096, 8192, 8192, 2)[0] == 1
    # a narrow output cannot take 256-column tiles
    assert blas.splitk_plan(64, 128, 32768, 2)[1] == 128


def test_small_allreduce_is_chosen_for_few_rows_and_a_long_k_only():
    from mm_rs_with_catlass_b200.ops import fused
    assert fused._small_allreduce_wanted(128, 8192, 14336, 2)
    assert fused._small_allreduce_wanted(1, 128, 8192, 2)
    assert not fused._small_allreduce_wanted(fused._SMALL_AR_MAX_M + 1, 8192, 14336, 2)
    assert not fused._small_allreduce_wanted(128, 8192, 256, 2)        # K too short to cut
    assert not fused._small_allreduce_wanted(128, 8190, 14336, 2)      # rows of whole 16-byte vectors only
    assert not fused._small_allreduce_wanted(128, 64, 14336, 2)        # narrower than one tile


def test_reduce_scatter_takes_the_few_row_path_while_a_rank_keeps_less_than_a_tile():
    from mm_rs_with_catlass_b200.ops import fused
    assert fused._small_reduce_scatter_wanted(128, 8192, 14336, 2, 2)       # as the all-reduce
    assert fused._small_reduce_scatter_wanted(256, 8192, 3584, 2, 8)        # 32 rows per rank
    assert fused._small_reduce_scatter_wanted(256, 8192, 7168, 2, 4)        # 64 rows per rank
    assert not fused._small_reduce_scatter_wanted(256, 8192, 14336, 2, 2)   # a full 128-row tile per rank: fused kernel
    assert not fused._small_reduce_scatter_wanted(512, 8192, 3584, 2, 8)    # enough tiles for every SM: nothing to cut

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

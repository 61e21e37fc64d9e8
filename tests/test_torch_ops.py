"""``torch.ops.catcoc.*`` registration: schemas, fake (meta) implementations on CPU, and the real
kernels on a GPU."""
import pytest
import torch

import mm_rs_with_catlass_b200  # noqa: F401  (registers the operators)


def test_operators_are_registered_with_the_reference_signatures():
    for name in ("basic_matmul", "optimized_matmul", "grouped_matmul"):
        assert hasattr(torch.ops.catcoc, name)
    schema = str(torch.ops.catcoc.basic_matmul.default._schema)
    assert "Tensor a" in schema and "str out_dtype" in schema and "-> Tensor" in schema
    schema = str(torch.ops.catcoc.grouped_matmul.default._schema)
    assert "Tensor[] a" in schema and "bool split_k" in schema and "-> Tensor[]" in schema


def test_fake_implementations_give_shapes_and_dtypes_without_a_gpu():
    a = torch.empty(48, 32, device="meta", dtype=torch.float16)
    b = torch.empty(32, 20, device="meta", dtype=torch.float16)
    o = torch.ops.catcoc.basic_matmul(a, b, "float32")
    assert o.shape == (48, 20) and o.dtype == torch.float32 and o.device.type == "meta"
    o = torch.ops.catcoc.optimized_matmul(a, b, "bf16")
    assert o.shape == (48, 20) and o.dtype == torch.bfloat16
    outs = torch.ops.catcoc.grouped_matmul([a, a[:7]], [b, b], "float16", False)
    assert [tuple(t.shape) for t in outs] == [(48, 20), (7, 20)]
    with pytest.raises(ValueError):
        torch.ops.catcoc.basic_matmul(a, b, "complex64")


def test_cpu_tensors_are_refused_with_a_pointer_to_the_goldens():
    a, b = torch.randn(8, 8).half(), torch.randn(8, 8).half()
    with pytest.raises(RuntimeError, match="CUDA"):
        torch.ops.catcoc.basic_matmul(a, b, "float16")


@pytest.mark.gpu
def test_operators_run_the_kernels(device):
    from mm_rs_with_catlass_b200.utils.verify import assert_close
    a = torch.randn(200, 136, device=device).half()
    b = torch.randn(136, 264, device=device).half()
    assert_close(torch.ops.catcoc.basic_matmul(a, b, "float16"), a.float() @ b.float(), k=136)
    assert_close(torch.ops.catcoc.optimized_matmul(a.t().contiguous().t(), b, "float32"), a.float() @ b.float(), k=136)
    xs = [torch.randn(m, 96, device=device).bfloat16() for m in (130, 5, 64)]
    ws = [torch.randn(96, 72, device=device).bfloat16() for _ in xs]
    outs = torch.ops.catcoc.grouped_matmul(xs, ws, "bfloat16", False)
    for o, x, w in zip(outs, xs, ws):
        assert_close(o, x.float() @ w.float(), k=96)
    xs = [torch.randn(40, k, device=device).bfloat16() for k in (64, 136)]
    ws = [torch.randn(x.shape[1], 48, device=device).bfloat16() for x in xs]
    outs = torch.ops.catcoc.grouped_matmul(xs, ws, "float32", True)
    for o, x, w in zip(outs, xs, ws):
        assert_close(o, x.float() @ w.float(), k=x.shape[1])

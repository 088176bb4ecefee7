"""Host-side mirror of the reference interface: names, argument meaning, error behaviour.
No GPU is needed: every check below fails before a kernel would be launched."""
import inspect

import pytest
import torch

import hf_kernels_helion_b200 as pkg
from hf_kernels_helion_b200 import runtime, tp
from hf_kernels_helion_b200._ops import _OPS_NAME

FP8 = torch.float8_e4m3fn


def _args(M=4, N=128, K=256):
    return (torch.zeros(M, K).to(FP8), torch.zeros(N, K).to(FP8), torch.ones(M, K // 128), torch.ones(N // 128, K // 128))


def test_public_names_and_signature_match_the_reference():
    # torch-ext/finegrained_fp8_helion/__init__.py:7-8 and :17
    assert "w8a8_block_fp8_matmul" in pkg.__all__
    sig = inspect.signature(pkg.w8a8_block_fp8_matmul)
    assert list(sig.parameters) == ["A", "B", "As", "Bs", "block_size", "output_dtype"]
    assert sig.parameters["output_dtype"].default is torch.float32


def test_op_namespace_and_schema_match_the_reference():
    # build/torch-cuda/_ops.py:21-25 and torch-ext/finegrained_fp8_helion/op.py:8-11
    assert _OPS_NAME == "_finegrained_fp8_helion_cuda_b0d7177"
    op = getattr(torch.ops, _OPS_NAME).w8a8_block_fp8_matmul
    schema = str(op.default._schema)
    assert "Tensor A, Tensor B, Tensor As, Tensor Bs, SymInt block_n, SymInt block_k" in schema or \
           "Tensor A, Tensor B, Tensor As, Tensor Bs, int block_n, int block_k" in schema
    assert schema.rstrip().endswith("-> Tensor")


def test_fake_impl_shapes_and_dtypes():
    A, B, As, Bs = [t.to("meta") for t in _args(5, 256, 384)]
    ns = getattr(torch.ops, _OPS_NAME)
    assert ns.w8a8_block_fp8_matmul(A, B, As, Bs, 128, 128).shape == (5, 256)
    assert ns.w8a8_block_fp8_matmul(A, B, As, Bs, 128, 128).dtype == torch.float32   # op.py:16 of the reference
    assert ns.w8a8_block_fp8_matmul_out(A, B, As, Bs, 128, 128, 0).dtype == torch.bfloat16
    q, s = ns.fp8_act_quant(torch.empty(5, 384, dtype=torch.bfloat16, device="meta"), 128)
    assert q.shape == (5, 384) and q.dtype == FP8 and s.shape == (5, 3) and s.dtype == torch.float32


def test_argument_validation():
    A, B, As, Bs = _args()
    with pytest.raises(ValueError, match="block_size"):
        runtime.gemm(A, B, As, Bs, 64, 128, torch.bfloat16)
    with pytest.raises(ValueError, match="output dtype"):
        runtime.gemm(A, B, As, Bs, 128, 128, torch.float16)
    with pytest.raises(ValueError, match="float8_e4m3fn"):
        runtime.gemm(A.float(), B, As, Bs, 128, 128, torch.bfloat16)
    with pytest.raises(ValueError, match="float32"):
        runtime.gemm(A, B, As.double(), Bs, 128, 128, torch.bfloat16)
    with pytest.raises(ValueError, match="As must be"):
        runtime.gemm(A, B, As[:, :1], Bs, 128, 128, torch.bfloat16)
    with pytest.raises(ValueError, match="Bs must be"):
        runtime.gemm(A, B, As, torch.ones(128, 2), 128, 128, torch.bfloat16)   # legacy per-row scales are rejected
    with pytest.raises(ValueError, match="K="):
        runtime.gemm(A, B[:, :128], As, Bs, 128, 128, torch.bfloat16)
    with pytest.raises(ValueError, match="2-D"):
        runtime.gemm(A[0], B, As, Bs, 128, 128, torch.bfloat16)
    with pytest.raises(ValueError, match="unknown variant"):
        runtime.resolve_variant("fastest")


def test_no_cpu_fallback():
    A, B, As, Bs = _args()
    with pytest.raises(RuntimeError, match="no CPU implementation"):
        pkg.w8a8_block_fp8_matmul(A, B, As, Bs, [128, 128], torch.bfloat16)
    with pytest.raises(RuntimeError, match="no CPU implementation"):
        pkg.fp8_act_quant(torch.zeros(4, 128, dtype=torch.bfloat16))
    with pytest.raises(ValueError, match="bfloat16"):
        pkg.fp8_act_quant(torch.zeros(4, 128))
    with pytest.raises(ValueError, match="multiple of 8"):
        pkg.fp8_act_quant(torch.zeros(4, 100, dtype=torch.bfloat16))


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from hf_kernels_helion_b200 import _lib

    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", tmp_path / "libb200fp8.so")
    with pytest.raises(RuntimeError, match="no non-CUDA fallback"):
        _lib.load()


def test_product_code_never_imports_the_oracle():
    import pathlib

    root = pathlib.Path(pkg.__file__).parent
    for f in list(root.rglob("*.py")) + list(root.rglob("*.cu")) + list(root.rglob("*.cuh")):
        assert "oracle" not in f.read_text(), f"{f} mentions the oracle"


def test_shard_bounds():
    assert tp.shard_bounds(18432, 8, 3) == (6912, 9216)
    assert tp.shard_bounds(18432, 1, 0) == (0, 18432)
    with pytest.raises(ValueError):
        tp.shard_bounds(18432 + 128, 8, 0)
    B = torch.arange(512 * 4).reshape(512, 4)
    Bs = torch.arange(4 * 1).reshape(4, 1)
    b, bs = tp.shard_weight(B, Bs, 2, 1)
    assert torch.equal(b, B[256:]) and torch.equal(bs, Bs[2:])

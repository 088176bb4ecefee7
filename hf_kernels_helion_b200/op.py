"""torch custom ops of the package.

``w8a8_block_fp8_matmul`` keeps the reference's schema and fp32 result
(finegrained-fp8-helion/finegrained-fp8-helion/torch-ext/finegrained_fp8_helion/op.py:8-16).
``w8a8_block_fp8_matmul_out`` adds an output-dtype code so that bf16 results are
written by the GEMM epilogue instead of a second cast pass; ``fp8_act_quant`` is the
per-token-group quantiser the reference lacks.
"""
from __future__ import annotations

import torch

from . import runtime
from ._ops import add_op_namespace_prefix

_DTYPES = {0: torch.bfloat16, 1: torch.float32}


@torch.library.custom_op(add_op_namespace_prefix("w8a8_block_fp8_matmul"), mutates_args=())
def w8a8_block_fp8_matmul(A: torch.Tensor, B: torch.Tensor, As: torch.Tensor, Bs: torch.Tensor,
                          block_n: int, block_k: int) -> torch.Tensor:
    return runtime.gemm(A, B, As, Bs, block_n, block_k, torch.float32)


@w8a8_block_fp8_matmul.register_fake
def _(A, B, As, Bs, block_n, block_k):
    return A.new_empty((A.shape[0], B.shape[0]), dtype=torch.float32)


@torch.library.custom_op(add_op_namespace_prefix("w8a8_block_fp8_matmul_out"), mutates_args=())
def w8a8_block_fp8_matmul_out(A: torch.Tensor, B: torch.Tensor, As: torch.Tensor, Bs: torch.Tensor,
                              block_n: int, block_k: int, out_dtype: int) -> torch.Tensor:
    return runtime.gemm(A, B, As, Bs, block_n, block_k, _DTYPES[out_dtype])


@w8a8_block_fp8_matmul_out.register_fake
def _(A, B, As, Bs, block_n, block_k, out_dtype):
    return A.new_empty((A.shape[0], B.shape[0]), dtype=_DTYPES[out_dtype])


@torch.library.custom_op(add_op_namespace_prefix("fp8_act_quant"), mutates_args=())
def fp8_act_quant(x: torch.Tensor, group: int) -> tuple[torch.Tensor, torch.Tensor]:
    return runtime.quant_act(x, group)


@fp8_act_quant.register_fake
def _(x, group):
    return (x.new_empty(x.shape, dtype=torch.float8_e4m3fn),
            x.new_empty((x.shape[0], -(-x.shape[1] // group)), dtype=torch.float32))

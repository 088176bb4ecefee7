"""Second drop-in served by the same CUDA path: deep-gemm-helion's blockwise FP8 GEMM.

Mirrors ``deep_gemm_helion.gemm_fp8_fp8_bf16_nt(A, B, As, Bs, block_size=128)``
(deep-gemm-helion/deep-gemm-helion/torch-ext/deep_gemm_helion/__init__.py:6-8) and its torch op
``_deep_gemm_helion_cuda_b3690f6::gemm_fp8_fp8_bf16_nt(A, B, As, Bs, block_k) -> bf16 [M, N]``
(torch-ext/deep_gemm_helion/op.py:7-16).  Operands: A [M, K] and B [N, K] float8_e4m3fn,
As [M, K/128] and Bs [N, K/128] fp32 - one B scale per ROW of B, unlike
w8a8_block_fp8_matmul's one per 128 x 128 block.  Only block_size 128 exists here.
"""
from __future__ import annotations

import hashlib

import torch

from . import runtime

_KERNEL_NAME = "deep_gemm_helion"
OPS_NAME = f"_{_KERNEL_NAME}_cuda_{hashlib.sha1(_KERNEL_NAME.encode()).hexdigest()[:7]}"


@torch.library.custom_op(f"{OPS_NAME}::gemm_fp8_fp8_bf16_nt", mutates_args=())
def _gemm_fp8_fp8_bf16_nt(A: torch.Tensor, B: torch.Tensor, As: torch.Tensor, Bs: torch.Tensor,
                          block_k: int) -> torch.Tensor:
    return runtime.gemm_rowscale(A, B, As, Bs, block_k, torch.bfloat16)


@_gemm_fp8_fp8_bf16_nt.register_fake
def _(A, B, As, Bs, block_k):
    return A.new_empty((A.shape[0], B.shape[0]), dtype=torch.bfloat16)


def gemm_fp8_fp8_bf16_nt(A, B, As, Bs, block_size=128):
    """DeepGEMM-style blockwise fp8 GEMM (NT layout): (A*As) @ (B*Bs)^T -> bf16."""
    return getattr(torch.ops, OPS_NAME).gemm_fp8_fp8_bf16_nt(A, B, As, Bs, int(block_size))


__all__ = ["gemm_fp8_fp8_bf16_nt"]

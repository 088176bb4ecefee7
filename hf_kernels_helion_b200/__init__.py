"""B200-native (sm_100a) block-FP8 matmul and activation quantiser.

Public surface mirrors the reference package ``finegrained_fp8_helion``
(finegrained-fp8-helion/finegrained-fp8-helion/torch-ext/finegrained_fp8_helion/__init__.py:7-17):
``w8a8_block_fp8_matmul(A, B, As, Bs, block_size, output_dtype=torch.float32)``.
Additions that the reference does not have are ``fp8_act_quant``, ``fp8_weight_quant``,
``fp8_linear`` and the tensor-parallel helpers in ``hf_kernels_helion_b200.tp``.
"""
from __future__ import annotations

import torch

from . import runtime
from ._ops import ops
from .op import fp8_act_quant as _q
from .op import w8a8_block_fp8_matmul as _m
from .op import w8a8_block_fp8_matmul_out as _mo
from .runtime import check_device_status

_OUT_CODE = {torch.bfloat16: 0, torch.float32: 1}


def w8a8_block_fp8_matmul(A: torch.Tensor, B: torch.Tensor, As: torch.Tensor, Bs: torch.Tensor,
                          block_size, output_dtype=torch.float32) -> torch.Tensor:
    """C = A @ B.T with block scales.  A: [M, K] float8_e4m3fn, B: [N, K] float8_e4m3fn,
    As: [M, K // bk] fp32, Bs: [N // bn, K // bk] fp32, block_size = [block_n, block_k]
    (only [128, 128]).  Returns [M, N] in output_dtype; fp32 accumulation.  bf16 and fp32
    results are written by the kernel itself, other dtypes by a cast of the fp32 result.

    The reference's own harness (finegrained-fp8-helion/bench.py:25-28) still calls this function
    in an older form, `w8a8_block_fp8_matmul(A, B, sA, sB, 128)`: an int block size and one B scale
    per ROW of B, sB [N, K // 128].  That form is accepted too and runs the row-scaled kernel."""
    if isinstance(block_size, int):
        res = runtime.gemm_rowscale(A, B, As, Bs, block_size,
                                    output_dtype if output_dtype in _OUT_CODE else torch.float32)
        return res if res.dtype == output_dtype else res.to(output_dtype)
    block_n, block_k = int(block_size[0]), int(block_size[1])
    code = _OUT_CODE.get(output_dtype)
    if code is None:
        return ops.w8a8_block_fp8_matmul(A, B, As, Bs, block_n, block_k).to(output_dtype)
    if code == 1:
        return ops.w8a8_block_fp8_matmul(A, B, As, Bs, block_n, block_k)
    return ops.w8a8_block_fp8_matmul_out(A, B, As, Bs, block_n, block_k, code)


def fp8_act_quant(x: torch.Tensor, block_size: int = 128):
    """Per-token-group quantiser: x [M, K] bf16 -> (q [M, K] float8_e4m3fn, s [M, K // 128] fp32)
    with s = group amax / 448 and q = e4m3(x / s).  No counterpart in the reference."""
    return ops.fp8_act_quant(x, int(block_size))


def fp8_weight_quant(w: torch.Tensor, block_size: int = 128):
    """128x128-block quantiser: w [N, K] bf16 -> (q [N, K] float8_e4m3fn, s [N // 128, K // 128] fp32)."""
    return runtime.quant_weight(w, int(block_size))


def fp8_linear(x: torch.Tensor, weight: torch.Tensor, weight_scale: torch.Tensor,
               output_dtype=torch.bfloat16) -> torch.Tensor:
    """Quantise bf16 activations per 1x128 group and multiply by a block-FP8 weight [N, K].
    For decode-sized inputs (at most 256 rows, K a multiple of 128, bf16 / fp32 result) this is
    ONE library call (b200fp8_linear: the quantiser writes straight into the GEMM kernel's input
    layout; measured 2 us faster at M <= 64, N = 28672); larger inputs run the quantiser and the
    matmul as two calls, which is faster there (1148 vs 1242 us at 8192 x 18432 x 7168).
    Same values either way."""
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    if (x2.shape[0] <= 256 and x2.shape[1] % 128 == 0 and x2.dtype == torch.bfloat16
            and output_dtype in (torch.bfloat16, torch.float32)):
        y = runtime.linear(x2, weight, weight_scale, output_dtype)
    else:
        q, s = fp8_act_quant(x2)
        y = w8a8_block_fp8_matmul(q, weight, s, weight_scale, [128, 128], output_dtype)
    return y.reshape(*lead, weight.shape[0])


__all__ = ["w8a8_block_fp8_matmul", "fp8_act_quant", "fp8_weight_quant", "fp8_linear", "check_device_status"]

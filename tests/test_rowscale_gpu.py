"""Row-scaled B (deep-gemm-helion's operand layout) on the GPU: b200fp8_gemm_rowscale and the
drop-in `gemm_fp8_fp8_bf16_nt` against the reference-generated fixtures and the CPU oracle."""
from pathlib import Path

import numpy as np
import pytest
import torch

from hf_kernels_helion_b200 import deep_gemm, runtime
from oracle import fp8_oracle as oracle

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden"


@pytest.mark.parametrize("name", ["rowscale_96x256x384", "rowscale_130x128x256", "rowscale_1x384x512"])
def test_golden_vectors_from_reference_source(device, name):
    g = np.load(GOLDEN / f"{name}.npz")
    A = torch.from_numpy(g["A"]).view(torch.float8_e4m3fn)
    B = torch.from_numpy(g["B"]).view(torch.float8_e4m3fn)
    As, Bs = torch.from_numpy(g["As"]), torch.from_numpy(g["Bs"])
    out = deep_gemm.gemm_fp8_fp8_bf16_nt(A.to(device), B.to(device), As.to(device), Bs.to(device), 128)
    assert out.dtype == torch.bfloat16 and tuple(out.shape) == (A.shape[0], B.shape[0])
    ref32 = oracle.gemm_rowscale_blockwise(A, B, As, Bs)
    assert oracle.bf16_ulp_error(out.cpu(), ref32) <= 1
    # the reference kernel's own bf16 output differs from ours by at most one rounding step
    want = torch.from_numpy(g["out_kernel_bf16_bits"]).view(torch.bfloat16)
    assert oracle.bf16_ulp_error(want, out.float().cpu()) <= 1.01
    runtime.check_device_status()


@pytest.mark.parametrize("M,N,K", [(1, 128, 128), (16, 384, 512), (130, 200, 320), (512, 512, 2048), (257, 1100, 1152),
                                   (2048, 2048, 4096), (64, 512, 8192), (200, 384, 16384), (300, 40000, 256)])
def test_rowscale_vs_oracle(device, M, N, K):
    """Ragged M, N (not a multiple of 128) and K (last K block short); fp32 and bf16 results. K <= 8192 keeps the
    B scales of a tile in shared memory (64 K blocks exactly at K = 8192), K = 16384 is beyond that table and
    reads them from global memory; N = 40000 gives every CTA more than one tile, so the table is recycled."""
    A, B, As, Bs = oracle.make_rowscale_inputs(M, N, K, M + N + K)
    ref = oracle.gemm_rowscale_dequant(A, B, As, Bs)
    d = [t.to(device) for t in (A, B, As, Bs)]
    out32 = runtime.gemm_rowscale(*d, 128, torch.float32)
    assert oracle.max_err_over_rms(out32.cpu(), ref) <= 1e-4           # tolerance of the fp32 path; measured ~3e-6
    out16 = runtime.gemm_rowscale(*d, 128, torch.bfloat16)
    assert oracle.bf16_ulp_error(out16.cpu(), ref) <= 1
    runtime.check_device_status()


def test_rowscale_equals_block_scaled_kernel_on_block_constant_scales(device):
    """When the 128 rows of every block share one scale, the row-scaled entry must agree with
    w8a8_block_fp8_matmul's kernel (same products, same accumulation order per K block)."""
    M, N, K = 384, 512, 1024
    A, B, As, Bsb = oracle.make_quantised_inputs(M, N, K, 3)
    Bs_row = Bsb.repeat_interleave(128, dim=0)[:N].contiguous()
    d = [t.to(device) for t in (A, B, As)]
    a = runtime.gemm_rowscale(*d, Bs_row.to(device), 128, torch.float32)
    b = runtime.gemm(*d, Bsb.to(device), 128, 128, torch.float32, variant="tile128")
    assert oracle.max_err_over_rms(a.cpu(), b.cpu()) <= 1e-6


def test_rowscale_argument_errors(device):
    A, B, As, Bs = [t.to(device) for t in oracle.make_rowscale_inputs(16, 128, 256, 0)]
    with pytest.raises(ValueError):
        deep_gemm.gemm_fp8_fp8_bf16_nt(A, B, As, Bs, 64)
    with pytest.raises(ValueError):
        deep_gemm.gemm_fp8_fp8_bf16_nt(A, B, As, Bs[:64], 128)
    with pytest.raises(RuntimeError):
        deep_gemm.gemm_fp8_fp8_bf16_nt(A.cpu(), B.cpu(), As.cpu(), Bs.cpu(), 128)


def test_legacy_call_form_of_the_reference_harness(device):
    """finegrained-fp8-helion/bench.py:25-28 calls w8a8_block_fp8_matmul(A, B, sA, sB, 128) with
    per-row B scales; the result must be that of the row-scaled kernel (fp32 by default)."""
    import hf_kernels_helion_b200 as pkg

    A, B, As, Bs = oracle.make_rowscale_inputs(200, 256, 512, 5)
    d = [t.to(device) for t in (A, B, As, Bs)]
    out = pkg.w8a8_block_fp8_matmul(*d, 128)
    assert out.dtype == torch.float32
    assert oracle.max_err_over_rms(out.cpu(), oracle.gemm_rowscale_dequant(A, B, As, Bs)) <= 1e-4
    out16 = pkg.w8a8_block_fp8_matmul(*d, 128, torch.bfloat16)
    assert torch.equal(out16, deep_gemm.gemm_fp8_fp8_bf16_nt(*d, 128))

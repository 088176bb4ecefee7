"""b200fp8_gemm_decode_static: the decode GEMM for callers that cannot allocate device memory
(a serving process that gave all of HBM to its own pool, a latency-critical loop that cannot
take cudaMalloc's device-wide synchronisation).  Its workspace is a fixed array inside the
library, so it must give exactly what the workspace-taking entry point gives.

Collected last on purpose (file name): a run that stops at the first failure has then already
run every other test.  Passes alone in a fresh process and after the rest of the suite.
"""
import pytest
import torch

from oracle import fp8_oracle as oracle

pytestmark = pytest.mark.gpu

FP32_TOL = 1e-4          # same bound as tests/test_gemm_gpu.py


def _call_static(lib, A, B, As, Bs, out, status):
    M, K = A.shape
    N = B.shape[0]
    return lib.b200fp8_gemm_decode_static(
        A.data_ptr(), B.data_ptr(), As.data_ptr(), Bs.data_ptr(), out.data_ptr(), M, N, K,
        A.stride(0), B.stride(0), As.stride(0), Bs.stride(0), out.stride(0),
        1 if out.dtype == torch.float32 else 0, status.data_ptr(), torch.cuda.current_stream().cuda_stream)


def _call_workspace(lib, A, B, As, Bs, out, status):
    M, K = A.shape
    N = B.shape[0]
    nbytes = lib.b200fp8_gemm_workspace_bytes(M, N, K, 3)
    ws = torch.empty(max(nbytes, 256), dtype=torch.uint8, device=A.device)
    st = lib.b200fp8_gemm(A.data_ptr(), B.data_ptr(), As.data_ptr(), Bs.data_ptr(), out.data_ptr(), M, N, K,
                          A.stride(0), B.stride(0), As.stride(0), Bs.stride(0), out.stride(0),
                          1 if out.dtype == torch.float32 else 0, 3, ws.data_ptr(), ws.numel(), status.data_ptr(),
                          torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    return st


def test_static_scratch_entry_matches_workspace_entry(device, lib):
    status = torch.zeros(1, dtype=torch.int32, device=device)
    # two calls in a row with different shapes and contents: the second must not see the first one's scratch
    for (M, N, K, seed, dtype) in [(16, 3072, 2048, 1, torch.float32), (5, 28672, 1024, 2, torch.bfloat16)]:
        A, B, As, Bs = [t.to(device) for t in oracle.make_quantised_inputs(M, N, K, seed)]
        want = torch.empty(M, N, dtype=dtype, device=device)
        got = torch.full((M, N), float("nan"), dtype=dtype, device=device)
        assert _call_workspace(lib, A, B, As, Bs, want, status) == 0
        assert _call_static(lib, A, B, As, Bs, got, status) == 0
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        assert torch.equal(got, want)                      # same kernels, same reduction order: bit-identical
        ref = oracle.gemm_dequant(A.cpu(), B.cpu(), As.cpu(), Bs.cpu())
        if dtype == torch.float32:
            assert oracle.max_err_over_rms(got.cpu(), ref) <= FP32_TOL
        else:
            assert oracle.bf16_ulp_error(got.cpu(), ref) <= 1


def test_static_scratch_entry_rejects_what_does_not_fit(device, lib):
    status = torch.zeros(1, dtype=torch.int32, device=device)
    A, B, As, Bs = [t.to(device) for t in oracle.make_quantised_inputs(64, 256, 256, 3)]
    out = torch.empty(64, 256, dtype=torch.bfloat16, device=device)
    need = lib.b200fp8_gemm_workspace_bytes(64, 256, 256, 3)
    if need > (4 << 20):
        assert _call_static(lib, A, B, As, Bs, out, status) == 10          # B200FP8_ERR_TOO_LARGE
    big = [t.to(device) for t in oracle.make_quantised_inputs(64, 28672, 256, 4)]
    out = torch.empty(64, 28672, dtype=torch.bfloat16, device=device)
    assert lib.b200fp8_gemm_workspace_bytes(64, 28672, 256, 3) > (4 << 20)
    assert _call_static(lib, *big, out, status) == 10
    assert "capacity" in lib.b200fp8_strerror(10).decode()
    assert _call_static(lib, A[:0], B, As[:0], Bs, out[:0, :256], status) == 0   # empty problem is a no-op

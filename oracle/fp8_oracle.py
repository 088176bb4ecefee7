"""CPU oracle for the finegrained-fp8 hot path.  TEST INFRASTRUCTURE ONLY.

This file restates, on the CPU with plain torch / numpy, the arithmetic of the
reference package ``finegrained-fp8-helion`` (AmesingFlank/hf_kernels_helion).
Only ``tests/``, ``__graft_entry__.smoke()`` and ``bench.py`` may import it - ``bench.py`` in two
places: the ``cpu_baseline`` / ``--impl reference`` legs (where it is the timed CPU baseline) and the
parity check after the timed regions (where it checks sampled rows of the GPU result); the
product package never does.

What each function follows (paths are relative to the reference repository):

* ``gemm_blockwise``   finegrained-fp8-helion/finegrained-fp8-helion/torch-ext/finegrained_fp8_helion/fp8.py:24-38
                       (tile loop, ``As[m, k // bk]`` / ``Bs[n // bn, k // bk]`` indexing, fp32
                       accumulation, ``dot * sa[:, None] * sb`` order)
* ``gemm_dequant``     finegrained-fp8-helion/bench.py:11-14 (``ref``: dequantise, then one fp32 matmul),
                       with the B scale expanded per 128x128 block instead of per row because the
                       package API takes ``Bs [N // bn, K // bk]`` (torch-ext/finegrained_fp8_helion/__init__.py:9-11)
* ``w8a8_block_fp8_matmul``  torch-ext/finegrained_fp8_helion/__init__.py:7-14 (block_size unpacking and the
                       final ``.to(output_dtype)``)
* ``quant_act`` / ``quant_weight``  have NO counterpart in the reference; they restate the
                       benchmark configuration text: fp32 ``scale = amax / 448`` per 1x128 group
                       (activations) or 128x128 block (weights), then a round-to-nearest-even cast of
                       ``x / scale`` to float8_e4m3fn.  One documented deviation from the literal
                       formula: an all-zero group yields ``scale = 0, q = 0`` (the literal ``0 / 0`` is a
                       NaN whose sign bit differs between x86 and CUDA).

Pinning.  The GEMM functions are pinned by tests/golden (outputs of the reference's own source
executed in this repository's build container, see tests/golden/make_golden.py).  The quantisers
are pinned only by an independent bit-level e4m3 encoder (``e4m3_encode_rne`` below) because the
reference contains no quantiser: for them, parity with the reference is UNPINNED.
"""
from __future__ import annotations

import numpy as np
import torch

E4M3_MAX = 448.0
GROUP = 128


# --------------------------------------------------------------------------- generators

def make_inputs(M: int, N: int, K: int, seed: int = 0):
    """bf16 activations ~N(0,1) and weights ~N(0,0.02) of the benchmark configurations
    (A first, then W, from one torch CPU generator)."""
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    a = torch.randn(M, K, generator=g, dtype=torch.float32).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g, dtype=torch.float32) * 0.02).to(torch.bfloat16)
    return a, w


def make_quantised_inputs(M: int, N: int, K: int, seed: int = 0):
    a, w = make_inputs(M, N, K, seed)
    A, As = quant_act(a)
    B, Bs = quant_weight(w)
    return A, B, As, Bs


# --------------------------------------------------------------------------- quantisers

def _ceil_div(a: int, b: int) -> int:
    return -(-a // b)


def quant_act(x: torch.Tensor, group: int = GROUP):
    """x [M, K] bf16/fp32 -> (q [M, K] float8_e4m3fn, s [M, ceil(K/group)] fp32)."""
    assert x.dim() == 2
    M, K = x.shape
    G = _ceil_div(K, group)
    xf = x.to(torch.float32)
    pad = G * group - K
    if pad:
        xf = torch.nn.functional.pad(xf, (0, pad))
    xg = xf.view(M, G, group)
    amax = xg.abs().amax(dim=2)
    scale = amax / E4M3_MAX
    safe = torch.where(scale == 0, torch.ones_like(scale), scale)
    y = xg / safe.unsqueeze(2)
    y = torch.where((scale == 0).unsqueeze(2), torch.zeros_like(y), y)
    q = y.view(M, G * group)[:, :K].contiguous().to(torch.float8_e4m3fn)
    return q, scale.contiguous()


def quant_weight(w: torch.Tensor, block: int = GROUP):
    """w [N, K] -> (q [N, K] float8_e4m3fn, s [ceil(N/block), ceil(K/block)] fp32)."""
    assert w.dim() == 2
    N, K = w.shape
    NB, KB = _ceil_div(N, block), _ceil_div(K, block)
    wf = w.to(torch.float32)
    wf = torch.nn.functional.pad(wf, (0, KB * block - K, 0, NB * block - N))
    wb = wf.view(NB, block, KB, block)
    amax = wb.abs().amax(dim=(1, 3))
    scale = amax / E4M3_MAX
    safe = torch.where(scale == 0, torch.ones_like(scale), scale)
    y = wb / safe[:, None, :, None]
    y = torch.where((scale == 0)[:, None, :, None], torch.zeros_like(y), y)
    q = y.reshape(NB * block, KB * block)[:N, :K].contiguous().to(torch.float8_e4m3fn)
    return q, scale.contiguous()


def e4m3_encode_rne(v: np.ndarray) -> np.ndarray:
    """Independent bit-level float32 -> float8_e4m3fn encoder (round-to-nearest-even,
    no infinities, NaN = 0x7F/0xFF, finite values beyond the last rounding boundary of
    448 saturate to 448).  Written from the format definition: 1 sign, 4 exponent bits
    (bias 7), 3 mantissa bits, subnormals with exponent field 0 (step 2^-9)."""
    v = np.asarray(v, dtype=np.float32)
    bits = v.view(np.uint32)
    sign = ((bits >> 24) & 0x80).astype(np.uint8)
    a = np.abs(v).astype(np.float64)
    out = np.zeros(v.shape, dtype=np.uint8)
    nan = np.isnan(v)
    # spacing of representable values around |v|: 2^(e-3) for normal binades, 2^-9 below 2^-6
    with np.errstate(divide="ignore"):
        e = np.floor(np.log2(np.where(a > 0, a, 1.0)))
    e = np.clip(e, -6, 8)
    step = np.exp2(e - 3)
    k = a / step
    kr = np.rint(k)  # numpy rint is round-half-to-even
    val = kr * step
    val = np.minimum(val, E4M3_MAX)
    # encode val (exactly representable now)
    with np.errstate(divide="ignore"):
        e2 = np.floor(np.log2(np.where(val > 0, val, 1.0)))
    normal = val >= 2.0 ** -6
    mant_n = np.rint(val / np.exp2(e2 - 3)).astype(np.int64) - 8
    exp_n = (e2 + 7).astype(np.int64)
    code_n = (exp_n << 3) | mant_n
    code_s = np.rint(val / 2.0 ** -9).astype(np.int64)
    code = np.where(normal, code_n, code_s).astype(np.uint8)
    out = sign | code
    out = np.where(nan, np.uint8(0x7F) | sign, out).astype(np.uint8)
    return out


def e4m3_decode(b: np.ndarray) -> np.ndarray:
    """float8_e4m3fn byte -> float32, from the format definition."""
    b = np.asarray(b, dtype=np.uint8).astype(np.int64)
    s = np.where(b & 0x80, -1.0, 1.0)
    e = (b >> 3) & 0xF
    m = b & 0x7
    normal = s * np.exp2(e - 7.0) * (1.0 + m / 8.0)
    sub = s * (m / 8.0) * 2.0 ** -6
    v = np.where(e == 0, sub, normal)
    v = np.where((e == 15) & (m == 7), np.nan, v)
    return v.astype(np.float32)


# --------------------------------------------------------------------------- GEMM

def gemm_blockwise(A, B, As, Bs, block_n: int = 128, block_k: int = 128, tile_m: int = 256) -> torch.Tensor:
    """fp32 [M, N]; blockwise accumulation, one fp32 dot per (M tile, N block, K block)."""
    M, K = A.shape
    N = B.shape[0]
    Af = A.to(torch.float32)
    Bf = B.to(torch.float32)
    out = torch.empty(M, N, dtype=torch.float32)
    for m0 in range(0, M, tile_m):
        m1 = min(m0 + tile_m, M)
        for n0 in range(0, N, block_n):
            n1 = min(n0 + block_n, N)
            nb = n0 // block_n
            acc = torch.zeros(m1 - m0, n1 - n0, dtype=torch.float32)
            for k0 in range(0, K, block_k):
                k1 = min(k0 + block_k, K)
                kb = k0 // block_k
                sa = As[m0:m1, kb]
                sb = Bs[nb, kb]
                acc = acc + (Af[m0:m1, k0:k1] @ Bf[n0:n1, k0:k1].T) * sa[:, None] * sb
            out[m0:m1, n0:n1] = acc
    return out


def gemm_dequant(A, B, As, Bs, block_n: int = 128, block_k: int = 128) -> torch.Tensor:
    """fp32 [M, N]; dequantise both operands, then one fp32 matmul."""
    M, K = A.shape
    N = B.shape[0]
    saf = As.repeat_interleave(block_k, dim=1)[:, :K]
    sbf = Bs.repeat_interleave(block_n, dim=0)[:N].repeat_interleave(block_k, dim=1)[:, :K]
    return (A.to(torch.float32) * saf) @ (B.to(torch.float32) * sbf).T


def gemm_rowscale_blockwise(A, B, As, Bs_row, block_k: int = 128, tile: int = 128) -> torch.Tensor:
    """fp32 [M, N] with one B scale per ROW of B: the loop of deep-gemm-helion's kernel
    (deep-gemm-helion/deep-gemm-helion/torch-ext/deep_gemm_helion/fp8.py:19-28):
    acc += dot(a, b^T) * sA[tm, kb][:, None] * sB[tn, kb][None, :] per K block, multiplication
    order as written there. The kernel stores bf16 (fp8.py:29); the cast is left to the caller."""
    M, K = A.shape
    N = B.shape[0]
    Af = A.to(torch.float32)
    Bf = B.to(torch.float32)
    out = torch.empty(M, N, dtype=torch.float32)
    for m0 in range(0, M, tile):
        m1 = min(m0 + tile, M)
        for n0 in range(0, N, tile):
            n1 = min(n0 + tile, N)
            acc = torch.zeros(m1 - m0, n1 - n0, dtype=torch.float32)
            for k0 in range(0, K, block_k):
                k1 = min(k0 + block_k, K)
                kb = k0 // block_k
                acc = acc + (Af[m0:m1, k0:k1] @ Bf[n0:n1, k0:k1].T) * As[m0:m1, kb][:, None] * Bs_row[n0:n1, kb][None, :]
            out[m0:m1, n0:n1] = acc
    return out


def gemm_rowscale_dequant(A, B, As, Bs_row, block_k: int = 128) -> torch.Tensor:
    """fp32 [M, N]; dequantise with per-row scales on both sides, then one fp32 matmul
    (deep-gemm-helion/bench.py:11-14 `ref`, before its bf16 cast)."""
    K = A.shape[1]
    saf = As.repeat_interleave(block_k, dim=1)[:, :K]
    sbf = Bs_row.repeat_interleave(block_k, dim=1)[:, :K]
    return (A.to(torch.float32) * saf) @ (B.to(torch.float32) * sbf).T


def make_rowscale_inputs(M: int, N: int, K: int, seed: int = 0):
    """Operands with the distribution of deep-gemm-helion/bench.py:24-27: e4m3(randn * 0.3),
    scales U[0.5, 1), one per row and K block on both sides; generated on the CPU."""
    g = torch.Generator().manual_seed(seed)
    kb = _ceil_div(K, GROUP)
    A = (torch.randn(M, K, generator=g) * 0.3).to(torch.float8_e4m3fn)
    B = (torch.randn(N, K, generator=g) * 0.3).to(torch.float8_e4m3fn)
    As = torch.rand(M, kb, generator=g) * 0.5 + 0.5
    Bs = torch.rand(N, kb, generator=g) * 0.5 + 0.5
    return A, B, As, Bs


def w8a8_block_fp8_matmul(A, B, As, Bs, block_size, output_dtype=torch.float32) -> torch.Tensor:
    block_n, block_k = int(block_size[0]), int(block_size[1])
    return gemm_blockwise(A, B, As, Bs, block_n, block_k).to(output_dtype)


# --------------------------------------------------------------------------- error metrics

def max_err_over_rms(out: torch.Tensor, ref: torch.Tensor) -> float:
    ref = ref.to(torch.float64)
    rms = ref.pow(2).mean().sqrt().item()
    if rms == 0:
        return float((out.to(torch.float64) - ref).abs().max().item())
    return float((out.to(torch.float64) - ref).abs().max().item() / rms)


def bf16_ulp_error(out_bf16: torch.Tensor, ref_fp32: torch.Tensor, noise: float = 2e-5) -> float:
    """Largest |out - ref| measured in bf16 units in the last place OF THE REFERENCE VALUE,
    after allowing `noise * rms(ref)` of absolute slack for fp32 summation-order
    differences (they dominate for elements that cancel to nearly zero, where one bf16 ulp
    is far below the fp32 noise of the sum).  A correctly rounded bf16 output gives <= 0.5;
    "within one bf16 ulp" means <= 1."""
    ref = ref_fp32.to(torch.float64)
    out = out_bf16.to(torch.float64)
    rms = ref.pow(2).mean().sqrt().item()
    mag = ref.abs().clamp_min(1e-300)
    ulp = torch.exp2(torch.floor(torch.log2(mag)) - 7.0)
    err = ((out - ref).abs() - noise * rms).clamp_min(0.0) / ulp
    return float(err.max().item())


def bf16_ulp_distance(out_bf16: torch.Tensor, ref_fp32: torch.Tensor) -> torch.Tensor:
    """Distance, in bf16 units in the last place, between a bf16 tensor and bf16(ref)."""
    a = out_bf16.contiguous().view(torch.int16).to(torch.int32)
    b = ref_fp32.to(torch.bfloat16).contiguous().view(torch.int16).to(torch.int32)

    def ordered(v):  # map sign-magnitude bit patterns to a monotone integer line
        return torch.where(v < 0, -(v & 0x7FFF), v)

    return (ordered(a) - ordered(b)).abs()

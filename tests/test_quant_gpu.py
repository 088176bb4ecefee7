"""Quantiser kernels on the GPU against the CPU oracle: fp8 bytes and fp32 scales bit-exact."""
import pytest
import torch

import hf_kernels_helion_b200 as pkg
from hf_kernels_helion_b200 import runtime
from oracle import fp8_oracle as oracle

pytestmark = pytest.mark.gpu


def _assert_bit_exact(q, s, q_ref, s_ref):
    assert q.dtype == torch.float8_e4m3fn and s.dtype == torch.float32
    assert torch.equal(q.cpu().view(torch.uint8), q_ref.view(torch.uint8))
    assert torch.equal(s.cpu().view(torch.int32), s_ref.view(torch.int32))


@pytest.mark.parametrize("M,K", [(1, 128), (3, 256), (16, 8192), (130, 384), (512, 2048), (7, 200), (5, 8),
                                 (1000, 1032), (4096, 8192)])
def test_act_quant_bit_exact(device, M, K):
    g = torch.Generator().manual_seed(M * 131 + K)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    q_ref, s_ref = oracle.quant_act(x)
    q, s = pkg.fp8_act_quant(x.to(device))
    _assert_bit_exact(q, s, q_ref, s_ref)


def test_act_quant_value_ranges(device):
    """Wide dynamic range inside and across groups: subnormal e4m3 results, tiny and huge
    amax, all-zero groups, negative zero."""
    g = torch.Generator().manual_seed(3)
    x = torch.randn(64, 1024, generator=g)
    x[:, :128] *= 1e-30
    x[:, 128:256] *= 1e30
    x[:, 256:384] *= torch.logspace(-6, 0, 128)       # most elements land in the e4m3 subnormal range
    x[:, 384:512] = 0
    x[0, 384] = -0.0
    x[:, 512:640] = torch.where(torch.rand(64, 128, generator=g) < 0.9, torch.zeros(()), x[:, 512:640])
    x = x.to(torch.bfloat16)
    q_ref, s_ref = oracle.quant_act(x)
    q, s = pkg.fp8_act_quant(x.to(device))
    _assert_bit_exact(q, s, q_ref, s_ref)
    assert not torch.isnan(q.float()).any()


def _assert_same_with_nans(q, s, q_ref, s_ref):
    """Bytes and scales as the checker's, where a NaN byte may differ in its sign bit (the sign of an
    inf / inf or x / NaN quotient is the platform's choice) and a NaN scale in its payload."""
    qb, qr = q.cpu().view(torch.uint8), q_ref.view(torch.uint8)
    nan_b, nan_r = (qb & 0x7F) == 0x7F, (qr & 0x7F) == 0x7F
    assert torch.equal(nan_b, nan_r)
    assert torch.equal(qb[~nan_b], qr[~nan_r])
    sc, sr = s.cpu(), s_ref
    assert torch.equal(torch.isnan(sc), torch.isnan(sr))
    keep = ~torch.isnan(sr)
    assert torch.equal(sc[keep].view(torch.int32), sr[keep].view(torch.int32))


@pytest.mark.parametrize("K", [512, 200])        # the contiguous kernel and the strided / ragged one
def test_act_quant_nan_and_inf_groups(device, K):
    """A NaN anywhere in a group reaches the group's scale (scale NaN, every byte of the group NaN);
    an Inf makes the scale infinite: finite elements become zero, infinite ones NaN. Other groups of
    the same row are untouched."""
    g = torch.Generator().manual_seed(11)
    x = torch.randn(8, K, generator=g)
    x[0, 5] = float("nan")
    x[1, 130] = float("nan")
    x[1, 131] = float("inf")
    x[2, 0] = float("inf")
    x[3, 127] = float("-inf")
    x[3, 3] = float("inf")
    x[4, K - 1] = float("nan")
    x = x.to(torch.bfloat16)
    q_ref, s_ref = oracle.quant_act(x)
    assert torch.isnan(s_ref[0, 0]) and torch.isinf(s_ref[2, 0])           # the checker propagates them
    q, s = pkg.fp8_act_quant(x.to(device))
    _assert_same_with_nans(q, s, q_ref, s_ref)
    assert (q.cpu().view(torch.uint8)[0, :128] & 0x7F).eq(0x7F).all()        # whole group NaN
    assert not torch.isnan(s.cpu()[0, 1:]).any()


def test_weight_quant_nan_block(device):
    g = torch.Generator().manual_seed(12)
    w = (torch.randn(256, 384, generator=g) * 0.02)
    w[130, 7] = float("nan")
    w[5, 300] = float("inf")
    w = w.to(torch.bfloat16)
    q_ref, s_ref = oracle.quant_weight(w)
    q, s = pkg.fp8_weight_quant(w.to(device))
    _assert_same_with_nans(q, s, q_ref, s_ref)


def test_act_quant_every_bf16_value(device):
    """All 65536 bf16 bit patterns that are finite, paired with several group maxima."""
    bits = torch.arange(0, 65536, dtype=torch.int32).to(torch.int16)
    vals = bits.view(torch.bfloat16)
    finite = torch.isfinite(vals.float())
    vals = vals[finite]
    n = vals.numel() // 127 * 127
    body = vals[:n].view(-1, 127)
    for top in (1.0, 3.0, 448.0, 1e-3, 2.0 ** 100):
        x = torch.cat([body, torch.full((body.shape[0], 1), top, dtype=torch.bfloat16)], dim=1).contiguous()
        q_ref, s_ref = oracle.quant_act(x)
        q, s = pkg.fp8_act_quant(x.to(device))
        _assert_bit_exact(q, s, q_ref, s_ref)


def _bf16_from(exp, mant):
    """bf16 values 2^exp * (1 + mant / 128) for integer tensors exp (unbiased) and mant (0..127)."""
    bits = ((exp + 127) << 7) | mant
    return bits.to(torch.int16).view(torch.bfloat16)


def test_act_quant_all_mantissa_pairs(device):
    """The kernel divides through a reciprocal and one remainder correction. Whether that equals
    the IEEE division depends only on the mantissas of x and of the group maximum, so every
    (x mantissa, amax mantissa) pair is run, both signs, at quotient exponents down to the
    e4m3 flush range, and at group maxima from below the reciprocal path's lower limit to the
    largest bf16 value."""
    mant = torch.arange(128, dtype=torch.int32)
    for amax_exp in (-70, -52, -51, -30, -3, 0, 7, 60, 127):
        rel = torch.arange(0, -21, -1, dtype=torch.int32)                    # x exponent relative to amax
        x_exp = (amax_exp + rel).clamp(min=-126)
        xs = _bf16_from(x_exp[:, None].expand(-1, 128), mant[None, :].expand(21, -1)).reshape(-1)   # 2688 values
        xs = torch.cat([xs, -xs])
        rows = []
        for am in range(128):
            top = _bf16_from(torch.tensor([amax_exp], dtype=torch.int32), torch.tensor([am], dtype=torch.int32))
            body = xs[xs.float().abs() <= top.float()]
            pad = (-body.numel()) % 127
            body = torch.cat([body, torch.zeros(pad, dtype=torch.bfloat16)]).view(-1, 127)
            rows.append(torch.cat([body, top.expand(body.shape[0], 1)], dim=1))
        x = torch.cat(rows, dim=0).contiguous()
        q_ref, s_ref = oracle.quant_act(x)
        q, s = pkg.fp8_act_quant(x.to(device))
        _assert_bit_exact(q, s, q_ref, s_ref)


def test_act_quant_scale_of_every_amax(device):
    """scale = amax / 448 for every positive finite bf16 amax, subnormal ones included."""
    bits = torch.arange(1, 0x7F80, dtype=torch.int32).to(torch.int16)
    amax = bits.view(torch.bfloat16)
    x = torch.zeros(amax.numel(), 128, dtype=torch.bfloat16)
    x[:, 5] = amax
    x[:, 77] = -amax
    q_ref, s_ref = oracle.quant_act(x)
    q, s = pkg.fp8_act_quant(x.to(device))
    _assert_bit_exact(q, s, q_ref, s_ref)


def test_act_quant_views_and_sentinels(device):
    """Row-strided input view; output written through the C ABI into a sentinel-filled
    buffer must leave every byte outside [M, K] untouched."""
    from hf_kernels_helion_b200 import _lib

    M, K, LD = 37, 384, 512
    g = torch.Generator().manual_seed(11)
    big = torch.randn(M + 2, LD, generator=g).to(torch.bfloat16).to(device)
    x = big[1:M + 1, 64:64 + K]                       # stride(0) = 512, offset 64 elements = 128 bytes
    q_ref, s_ref = oracle.quant_act(x.cpu())
    q, s = pkg.fp8_act_quant(x)
    _assert_bit_exact(q, s, q_ref, s_ref)

    qbuf = torch.full((M + 2, LD), 0x5A, dtype=torch.uint8, device=device)
    sbuf = torch.full((M + 2, 8), 42.0, dtype=torch.float32, device=device)
    qv, sv = qbuf[1:M + 1, 64:64 + K], sbuf[1:M + 1, 2:5]
    st = _lib.load().b200fp8_quant_act(x.data_ptr(), qv.data_ptr(), sv.data_ptr(), M, K, LD, LD, 8,
                                       torch.cuda.current_stream().cuda_stream)
    assert st == 0
    torch.cuda.synchronize()
    assert torch.equal(qv.cpu(), q_ref.view(torch.uint8))
    assert torch.equal(sv.cpu(), s_ref)
    mask = torch.ones_like(qbuf, dtype=torch.bool)
    mask[1:M + 1, 64:64 + K] = False
    assert bool((qbuf[mask] == 0x5A).all())
    smask = torch.ones_like(sbuf, dtype=torch.bool)
    smask[1:M + 1, 2:5] = False
    assert bool((sbuf[smask] == 42.0).all())


@pytest.mark.parametrize("N,K", [(128, 128), (256, 384), (130, 200), (512, 2048), (2048, 4096)])
def test_weight_quant_bit_exact(device, N, K):
    g = torch.Generator().manual_seed(N * 17 + K)
    w = (torch.randn(N, K, generator=g) * 0.02).to(torch.bfloat16)
    q_ref, s_ref = oracle.quant_weight(w)
    q, s = pkg.fp8_weight_quant(w.to(device))
    _assert_bit_exact(q, s, q_ref, s_ref)


def test_quant_feeds_gemm_layout(device):
    """The scales come out in exactly the As layout the matmul takes."""
    a, w = oracle.make_inputs(64, 256, 512, 4)
    q, s = pkg.fp8_act_quant(a.to(device))
    wq, ws = pkg.fp8_weight_quant(w.to(device))
    out = pkg.w8a8_block_fp8_matmul(q, wq, s, ws, [128, 128], torch.float32)
    ref = oracle.gemm_blockwise(*oracle.make_quantised_inputs(64, 256, 512, 4))
    runtime.check_device_status()
    assert oracle.max_err_over_rms(out.cpu(), ref) < 1e-4
    y = pkg.fp8_linear(a.to(device).view(4, 16, 512), wq, ws)
    assert y.shape == (4, 16, 256) and y.dtype == torch.bfloat16

"""The CPU oracle against the golden vectors produced from the reference's own source
(tests/golden/make_golden.py) and against an independent bit-level e4m3 codec."""
import hashlib
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import fp8_oracle as oracle

GOLDEN = Path(__file__).resolve().parent / "golden"
SMALL = ["small_96x256x384", "small_130x128x256", "small_1x384x512"]


def _load_small(name):
    z = np.load(GOLDEN / f"{name}.npz")
    A = torch.from_numpy(z["A"]).view(torch.float8_e4m3fn)
    B = torch.from_numpy(z["B"]).view(torch.float8_e4m3fn)
    return z, A, B, torch.from_numpy(z["As"]), torch.from_numpy(z["Bs"])


@pytest.mark.parametrize("name", SMALL)
def test_blockwise_oracle_matches_reference_kernel_source(name):
    z, A, B, As, Bs = _load_small(name)
    ref = torch.from_numpy(z["out_kernel_fp32"])
    out = oracle.gemm_blockwise(A, B, As, Bs)
    # same statements, possibly a different M tile: fp32 matmul blocking may differ in the last bits
    assert oracle.max_err_over_rms(out, ref) < 1e-5
    assert out.shape == ref.shape


@pytest.mark.parametrize("name", SMALL)
def test_dequant_oracle_matches_reference_bench_ref(name):
    z, A, B, As, Bs = _load_small(name)
    ref_bits = torch.from_numpy(z["out_bench_bf16_bits"])
    out = oracle.gemm_dequant(A, B, As, Bs).to(torch.bfloat16)
    ulp = oracle.bf16_ulp_distance(out, ref_bits.view(torch.bfloat16).float())
    assert int(ulp.max()) <= 1
    assert float((ulp > 0).float().mean()) < 1e-3


@pytest.mark.parametrize("name", SMALL)
def test_golden_inputs_are_the_seeded_generator(name):
    z, A, B, As, Bs = _load_small(name)
    A2, B2, As2, Bs2 = oracle.make_quantised_inputs(int(z["M"]), int(z["N"]), int(z["K"]), int(z["seed"]))
    assert torch.equal(A.view(torch.uint8), A2.view(torch.uint8))
    assert torch.equal(B.view(torch.uint8), B2.view(torch.uint8))
    assert torch.equal(As, As2) and torch.equal(Bs, Bs2)


def _sha(t):
    return hashlib.sha256(t.contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()


def test_config1_against_reference_outputs():
    """BASELINE configuration 1: M = N = 512, K = 2048, seed 0 (the reference's CPU-runnable case)."""
    z = np.load(GOLDEN / "config1_512x512x2048.npz")
    A, B, As, Bs = oracle.make_quantised_inputs(512, 512, 2048, 0)
    assert _sha(A) == str(z["sha_A"]) and _sha(B) == str(z["sha_B"])
    assert _sha(As) == str(z["sha_As"]) and _sha(Bs) == str(z["sha_Bs"])
    rs, cs = int(z["row_step"]), int(z["col_step"])
    out_b = oracle.gemm_blockwise(A, B, As, Bs)
    out_d = oracle.gemm_dequant(A, B, As, Bs)
    ref = torch.from_numpy(z["out_kernel_fp32"])
    assert oracle.max_err_over_rms(out_b[::rs, ::cs], ref) < 1e-5
    assert oracle.max_err_over_rms(out_d[::rs, ::cs], ref) < 1e-5      # the two formulations agree in fp32
    assert abs(out_b.double().sum().item() - float(z["out_kernel_sum"])) <= 1e-6 * float(z["out_kernel_abs_sum"])
    ref_bits = torch.from_numpy(z["out_bench_bf16_bits"]).view(torch.bfloat16)
    ulp = oracle.bf16_ulp_distance(out_d[::rs, ::cs].to(torch.bfloat16).contiguous(), ref_bits.float())
    assert int(ulp.max()) <= 1


def test_wrapper_semantics():
    A, B, As, Bs = oracle.make_quantised_inputs(64, 128, 256, 5)
    o32 = oracle.w8a8_block_fp8_matmul(A, B, As, Bs, [128, 128])
    assert o32.dtype == torch.float32                   # reference default output dtype
    o16 = oracle.w8a8_block_fp8_matmul(A, B, As, Bs, [128, 128], torch.bfloat16)
    assert torch.equal(o16, o32.to(torch.bfloat16))     # plain cast of the fp32 result


# ------------------------------------------------------------------ e4m3 codec and quantisers

def test_e4m3_decode_matches_torch_for_all_bytes():
    b = np.arange(256, dtype=np.uint8)
    mine = oracle.e4m3_decode(b)
    theirs = torch.from_numpy(b).view(torch.float8_e4m3fn).float().numpy()
    assert np.array_equal(np.isnan(mine), np.isnan(theirs))
    ok = ~np.isnan(mine)
    assert np.array_equal(mine[ok], theirs[ok])


def test_e4m3_encode_matches_torch_cast():
    g = torch.Generator().manual_seed(0)
    v = torch.cat([
        torch.randn(200000, generator=g) * 100,
        torch.randn(100000, generator=g) * 0.01,
        torch.randn(100000, generator=g) * 1e-3,
        torch.linspace(-448.0, 448.0, 100001),
        torch.from_numpy(oracle.e4m3_decode(np.arange(0, 127, dtype=np.uint8))),          # exact values
        torch.from_numpy((oracle.e4m3_decode(np.arange(0, 126, dtype=np.uint8)) +
                          oracle.e4m3_decode(np.arange(1, 127, dtype=np.uint8))) / 2),    # exact ties
        torch.tensor([0.0, -0.0, 2.0 ** -10, 2.0 ** -9, 2.0 ** -11, 463.9, 448.00003]),
    ]).float()
    v = v[v.abs() < 464]    # beyond this torch's cast yields NaN while a saturating cast yields 448; never reached
    mine = oracle.e4m3_encode_rne(v.numpy())
    theirs = v.to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    assert np.array_equal(mine, theirs)


@pytest.mark.parametrize("M,K", [(4, 128), (33, 384), (7, 200)])
def test_quant_act_against_literal_formula(M, K):
    g = torch.Generator().manual_seed(M * K)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    q, s = oracle.quant_act(x)
    assert q.shape == (M, K) and s.shape == (M, -(-K // 128))
    xf = x.float().numpy()
    for kg in range(s.shape[1]):
        blk = xf[:, kg * 128:(kg + 1) * 128]
        amax = np.abs(blk).max(axis=1).astype(np.float32)
        scale = (amax / np.float32(448.0)).astype(np.float32)
        assert np.array_equal(scale, s[:, kg].numpy())
        y = (blk / scale[:, None]).astype(np.float32)
        assert np.array_equal(oracle.e4m3_encode_rne(y), q[:, kg * 128:(kg + 1) * 128].view(torch.uint8).numpy())
    # the largest element of every group maps to +-448
    deq = q.float().abs().numpy()
    for kg in range(s.shape[1]):
        assert np.all(deq[:, kg * 128:(kg + 1) * 128].max(axis=1) == 448.0)


def test_quant_zero_group_is_zero_not_nan():
    x = torch.zeros(2, 256, dtype=torch.bfloat16)
    x[1, 130] = 3.0
    q, s = oracle.quant_act(x)
    assert not torch.isnan(q.float()).any()
    assert s[0, 0] == 0 and s[0, 1] == 0 and s[1, 0] == 0 and s[1, 1] == 3.0 / 448
    assert q.float()[1, 130] == 448


def test_quant_weight_blocks():
    g = torch.Generator().manual_seed(9)
    w = (torch.randn(200, 300, generator=g) * 0.02).to(torch.bfloat16)
    q, s = oracle.quant_weight(w)
    assert q.shape == (200, 300) and s.shape == (2, 3)
    wf = w.float()
    for nb in range(2):
        for kb in range(3):
            blk = wf[nb * 128:(nb + 1) * 128, kb * 128:(kb + 1) * 128]
            assert s[nb, kb] == blk.abs().max() / 448
            assert torch.equal((blk / s[nb, kb]).to(torch.float8_e4m3fn).view(torch.uint8),
                               q[nb * 128:(nb + 1) * 128, kb * 128:(kb + 1) * 128].view(torch.uint8))


ROWSCALE = ["rowscale_96x256x384", "rowscale_130x128x256", "rowscale_1x384x512"]


@pytest.mark.parametrize("name", ROWSCALE)
def test_rowscale_oracles_match_reference_deep_gemm_source(name):
    """Row-scaled B (deep-gemm-helion): the blockwise restatement against the reference kernel's
    own output, the dequantise-then-matmul one against the reference harness's `ref`; both
    fixtures were produced by running the reference's source files (tests/golden/make_golden.py)."""
    g = np.load(GOLDEN / f"{name}.npz")
    A = torch.from_numpy(g["A"]).view(torch.float8_e4m3fn)
    B = torch.from_numpy(g["B"]).view(torch.float8_e4m3fn)
    As, Bs = torch.from_numpy(g["As"]), torch.from_numpy(g["Bs"])
    M, N, K, seed = int(g["M"]), int(g["N"]), int(g["K"]), int(g["seed"])
    A2, B2, As2, Bs2 = oracle.make_rowscale_inputs(M, N, K, seed)
    assert torch.equal(A.view(torch.uint8), A2.view(torch.uint8)) and torch.equal(B.view(torch.uint8), B2.view(torch.uint8))
    assert torch.equal(As, As2) and torch.equal(Bs, Bs2) and tuple(Bs.shape) == (N, K // 128)
    want_kernel = torch.from_numpy(g["out_kernel_bf16_bits"]).view(torch.bfloat16)
    want_bench = torch.from_numpy(g["out_bench_bf16_bits"]).view(torch.bfloat16)
    assert torch.equal(oracle.gemm_rowscale_blockwise(A, B, As, Bs).to(torch.bfloat16), want_kernel)
    assert torch.equal(oracle.gemm_rowscale_dequant(A, B, As, Bs).to(torch.bfloat16), want_bench)

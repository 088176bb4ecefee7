"""The C-ABI shared library: loads without a GPU, exports what include/b200fp8.h declares,
and rejects bad arguments before touching a device."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "b200fp8.h"


def declared_functions():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(b200fp8_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    names = declared_functions()
    for must in ["b200fp8_quant_act", "b200fp8_quant_weight", "b200fp8_gemm", "b200fp8_gemm_workspace_bytes",
                 "b200fp8_strerror", "b200fp8_version"]:
        assert must in names


def test_every_declared_symbol_is_exported(lib):
    for name in declared_functions():
        assert hasattr(lib, name), f"{name} is declared in include/b200fp8.h but not exported"


def test_python_binding_covers_the_header(lib):
    from hf_kernels_helion_b200 import _lib

    assert sorted(_lib.SIGNATURES) == declared_functions()


def test_version_and_strerror(lib):
    assert lib.b200fp8_version() >= 100
    seen = set()
    for code in range(0, 11):
        msg = lib.b200fp8_strerror(code).decode()
        assert msg and msg != "unknown status"
        seen.add(msg)
    assert len(seen) == 11
    assert lib.b200fp8_strerror(999).decode() == "unknown status"


def test_argument_errors_need_no_device(lib):
    null = None
    # negative sizes
    assert lib.b200fp8_gemm(null, null, null, null, null, -1, 1, 1, 1, 1, 1, 1, 1, 0, 0, null, 0, null, null) == 2
    assert lib.b200fp8_quant_act(null, null, null, -1, 128, 128, 128, 1, null) == 2
    assert lib.b200fp8_quant_weight(null, null, null, 128, -1, 128, 128, 1, null) == 2
    # unknown dtype / variant
    assert lib.b200fp8_gemm(null, null, null, null, null, 1, 1, 1, 1, 1, 1, 1, 1, 7, 0, null, 0, null, null) == 4
    assert lib.b200fp8_gemm(null, null, null, null, null, 1, 1, 1, 1, 1, 1, 1, 1, 0, 9, null, 0, null, null) == 5
    # empty problems are no-ops
    assert lib.b200fp8_gemm(null, null, null, null, null, 0, 5, 128, 128, 128, 1, 1, 5, 0, 0, null, 0, null, null) == 0
    assert lib.b200fp8_quant_act(null, null, null, 0, 128, 128, 128, 1, null) == 0
    # NULL / misaligned / short leading dimension for the quantiser
    assert lib.b200fp8_quant_act(null, null, null, 4, 128, 128, 128, 1, null) == 1
    buf = ctypes.create_string_buffer(4096)
    p = ctypes.addressof(buf)
    p16 = (p + 15) & ~15
    assert lib.b200fp8_quant_act(p16, p16, p16, 4, 100, 128, 128, 1, null) == 3      # K % 8
    assert lib.b200fp8_quant_act(p16 + 2, p16, p16, 4, 128, 128, 128, 1, null) == 3  # x not 16-byte aligned
    assert lib.b200fp8_quant_act(p16, p16, p16, 4, 128, 64, 128, 1, null) == 2       # ldx < K
    # output NULL / ldc too small
    assert lib.b200fp8_gemm(p16, p16, p16, p16, null, 4, 4, 128, 128, 128, 1, 1, 4, 0, 0, null, 0, null, null) == 1
    assert lib.b200fp8_gemm(p16, p16, p16, p16, p16, 4, 4, 128, 128, 128, 1, 1, 2, 0, 0, null, 0, null, null) == 2


def test_argument_errors_of_the_newer_entry_points(lib):
    null = None
    buf = ctypes.create_string_buffer(4096)
    p16 = (ctypes.addressof(buf) + 15) & ~15
    # fused quantise-and-multiply: K must be a multiple of 128, x must be there
    assert lib.b200fp8_linear(null, p16, p16, p16, 4, 128, 128, 128, 128, 1, 128, 0, 0, null, 0, null, null) == 1
    assert lib.b200fp8_linear_workspace_bytes(-1, 1, 1, 0) == -2
    assert lib.b200fp8_linear_workspace_bytes(16, 28672, 8192, 3) == -5            # no stream-K form of it
    assert lib.b200fp8_linear_workspace_bytes(16, 28672, 8192, 2) == 64 * 128 * 4 + 16 * 8192
    # row-scaled B: same checks as the block-scaled GEMM
    assert lib.b200fp8_gemm_rowscale(null, null, null, null, null, -1, 1, 1, 1, 1, 1, 1, 1, 0, null, 0, null, null) == 2
    assert lib.b200fp8_gemm_rowscale(null, null, null, null, null, 1, 1, 1, 1, 1, 1, 1, 1, 7, null, 0, null, null) == 4
    assert lib.b200fp8_gemm_rowscale_workspace_bytes(256, 512, 1024) == 8 * 256 * 4 + 8 * 512 * 4
    # peer barrier: group size and rank are checked before anything is launched
    arr = (ctypes.c_void_p * 8)(*([p16] * 8))
    assert lib.b200fp8_peer_barrier(null, 2, 0, 1, null, null) == 1
    assert lib.b200fp8_peer_barrier(arr, 0, 0, 1, null, null) == 2
    assert lib.b200fp8_peer_barrier(arr, 9, 0, 1, null, null) == 2
    assert lib.b200fp8_peer_barrier(arr, 2, 2, 1, null, null) == 2


def test_workspace_and_variant_queries(lib):
    AUTO, T128, T256, SK = 0, 1, 2, 3
    ast = 64 * 4096 * 4                                       # K-block-major copy of As: [K/128][M] fp32
    assert lib.b200fp8_gemm_workspace_bytes(4096, 4096, 8192, T128) == ast
    assert lib.b200fp8_gemm_workspace_bytes(4096, 4096, 8192, T256) == ast
    # 512 tiles on 148 SMs: 444 whole tiles + 68 tail tiles cut into 2 K ranges each (fp32 partial tiles)
    assert lib.b200fp8_gemm_workspace_bytes(4096, 4096, 8192, 4) == ast + 68 * 2 * 128 * 256 * 4
    assert lib.b200fp8_gemm_workspace_bytes(4096, 4096, 8192, AUTO) in (ast, ast + 68 * 2 * 128 * 256 * 4)
    # CTA-pair forms: the plain ones need the scale copy only; the split-K one adds two partial tiles per K range
    # (34 tail tiles x 2 ranges x 2 CTAs on a device with 74 pairs; nothing where the device reports no pairs)
    assert lib.b200fp8_gemm_workspace_bytes(4096, 4096, 8192, 5) == ast
    assert lib.b200fp8_gemm_workspace_bytes(4096, 4096, 8192, 6) == ast
    assert lib.b200fp8_gemm_workspace_bytes(4096, 4096, 8192, 7) in (ast, ast + 34 * 2 * 2 * 128 * 256 * 4)
    assert lib.b200fp8_gemm_workspace_bytes(4096, 4096, 8192, 8) == -5
    assert lib.b200fp8_gemm_workspace_bytes(300, 512, 200, T128) == 2 * 384 * 4   # M padded to 128, K blocks rounded up
    assert lib.b200fp8_gemm_workspace_bytes(4096, 4096, 8192, SK) == -5     # M > 256 cannot use stream-K
    assert lib.b200fp8_gemm_workspace_bytes(16, 28672, 8192, 42) == -5
    assert lib.b200fp8_gemm_workspace_bytes(-1, 1, 1, AUTO) == -2
    w1 = lib.b200fp8_gemm_workspace_bytes(1, 28672, 8192, SK)
    w16 = lib.b200fp8_gemm_workspace_bytes(16, 28672, 8192, SK)
    w256 = lib.b200fp8_gemm_workspace_bytes(256, 28672, 8192, SK)
    assert 0 < w1 == w16 < w256
    grid = lib.b200fp8_streamk_grid(16, 28672, 8192)
    assert w16 == 64 * 16 * 4 + 2 * grid * 16 * 128 * 4      # AsT [K/128][16] + two partial slots per CTA
    TSK = 4
    assert lib.b200fp8_gemm_pick_variant(1, 28672, 8192) == T256     # decode shapes: plain tile kernel measured fastest
    assert lib.b200fp8_gemm_pick_variant(256, 28672, 8192) == T256
    assert lib.b200fp8_gemm_pick_variant(16, 128, 512) == T128
    # 112 tiles on 148 SMs: the tail cannot be split in two, the variant degenerates to plain tiles
    # (K-block-major scales + the 16-row copy of A that M <= 16 goes through)
    assert lib.b200fp8_gemm_workspace_bytes(16, 28672, 8192, TSK) == 64 * 128 * 4 + 16 * 8192
    assert lib.b200fp8_gemm_workspace_bytes(17, 28672, 8192, TSK) == 64 * 128 * 4
    assert lib.b200fp8_gemm_pick_variant(4096, 4096, 8192) in (T128, T256, 4, 5, 6, 7)   # 5 to 7: CTA pairs where the device can run clusters of two


@pytest.mark.parametrize("tiles,num_kb,grid", [(224, 64, 148), (8, 8, 148), (3, 5, 4), (1, 1, 1), (7, 3, 5),
                                               (224, 56, 132), (17, 64, 148), (1, 64, 64)])
def test_streamk_partition_covers_every_unit_once(lib, tiles, num_kb, grid):
    """Host model of the stream-K split: contiguous ranges, each unit owned once, the
    owner function inverts the range function, and the slot rule the fix-up kernel uses
    (first segment of a CTA -> slot 2c, a later one -> slot 2c + 1) names every partial
    piece of every split tile exactly once."""
    total = tiles * num_kb
    grid = min(grid, total)
    first = [lib.b200fp8_streamk_first_unit(c, total, grid) for c in range(grid + 1)]
    assert first[0] == 0 and first[-1] == total
    sizes = [first[c + 1] - first[c] for c in range(grid)]
    assert min(sizes) >= 1 and max(sizes) - min(sizes) <= 1
    for c in range(grid):
        for u in (first[c], first[c + 1] - 1):
            assert lib.b200fp8_streamk_owner(u, total, grid) == c
    # pieces written by the main kernel: (tile, cta) -> slot
    written = {}
    for c in range(grid):
        u0, u1 = first[c], first[c + 1]
        t_first = u0 // num_kb
        for t in range(u0 // num_kb, (u1 - 1) // num_kb + 1):
            kb0 = max(u0, t * num_kb) - t * num_kb
            kb1 = min(u1, (t + 1) * num_kb) - t * num_kb
            if kb0 == 0 and kb1 == num_kb:
                continue                                 # full tile: written straight to C
            slot = 2 * c + (0 if t == t_first else 1)
            assert slot not in written.values()
            written[(t, c)] = slot
    # pieces the fix-up kernel reads
    read = {}
    for t in range(tiles):
        c_first = lib.b200fp8_streamk_owner(t * num_kb, total, grid)
        c_last = lib.b200fp8_streamk_owner(t * num_kb + num_kb - 1, total, grid)
        if c_first == c_last:
            continue
        for c in range(c_first, c_last + 1):
            first_tile_of_c = first[c] // num_kb
            read[(t, c)] = 2 * c + (0 if first_tile_of_c == t else 1)
    assert read == written


@pytest.mark.gpu
def test_peer_barrier_wait_runs_out_cleanly(lib, device):
    """A bounded device-side wait that really runs out, without a fault or a hang: the barrier kernel
    is told there are two GPUs, both flag arrays are this GPU's own, and nobody ever publishes the
    second slot. After `limit_clocks` (about a millisecond) the kernel records
    B200FP8_DEV_WAIT_TIMEOUT in the status word and returns; the host raises; the device stays usable."""
    import time

    import torch

    from hf_kernels_helion_b200 import _lib, runtime
    from oracle import fp8_oracle as oracle

    runtime.check_device_status(device)                       # start clean
    flags = torch.zeros(8, dtype=torch.int32, device=device)
    arr = (ctypes.c_void_p * 2)(flags.data_ptr(), flags.data_ptr())
    word = runtime.status_word(device)
    stream = torch.cuda.current_stream(device).cuda_stream
    t0 = time.perf_counter()
    with torch.cuda.device(device):
        st = lib.b200fp8_peer_barrier_limited(arr, 2, 0, 1, 2_000_000, word.data_ptr(), stream)
    assert st == 0
    torch.cuda.synchronize(device)
    assert time.perf_counter() - t0 < 1.0                      # 2e6 clocks is about a millisecond
    assert int(word.item()) == 1                               # B200FP8_DEV_WAIT_TIMEOUT
    assert int(flags[0].item()) == 1 and int(flags[1].item()) == 0    # own epoch published, peer slot untouched
    with pytest.raises(RuntimeError, match="device status 1"):
        runtime.check_device_status(device)
    runtime.check_device_status(device)                       # the check cleared the word
    # a barrier whose peers have all published returns at once and leaves the word clean
    flags[1] = 2
    with torch.cuda.device(device):
        assert lib.b200fp8_peer_barrier_limited(arr, 2, 0, 2, 2_000_000, word.data_ptr(), stream) == 0
    runtime.check_device_status(device)
    # argument errors
    assert lib.b200fp8_peer_barrier_limited(arr, 2, 0, 1, 0, word.data_ptr(), stream) == 2
    assert lib.b200fp8_peer_barrier_limited(None, 2, 0, 1, 1000, word.data_ptr(), stream) == 1
    # and the device still computes
    A, B, As, Bs = oracle.make_quantised_inputs(130, 256, 256, 5)
    out = runtime.gemm(A.to(device), B.to(device), As.to(device), Bs.to(device), 128, 128, torch.float32)
    runtime.check_device_status(device)
    assert oracle.max_err_over_rms(out.cpu(), oracle.gemm_dequant(A, B, As, Bs)) <= 1e-4

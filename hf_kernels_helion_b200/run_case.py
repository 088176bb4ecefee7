"""Run one shape of the hot path a few times and print its device time.

    python -m hf_kernels_helion_b200.run_case <variant|quant|rowscale> M N K [launches]

`variant` is a name from `_lib.VARIANT_NAMES` ("auto", "tile128", "tile256", "streamk", "tile256_sk", "pair256",
"pair256_split", "pair256_split_sk") and runs `b200fp8_gemm` on random e4m3 operands with scales in [0.5, 1); "rowscale" runs
`b200fp8_gemm_rowscale` (one B scale per row of B); "quant" runs the per-token-group activation quantiser on a
random bf16 [M, K] matrix (N is ignored). The launches are back to back on one stream, so the
command is small enough to be wrapped by a profiler capture of a single kernel; the time printed is the mean
over the launches after the first, measured with CUDA events.
"""
import sys

import torch

import hf_kernels_helion_b200 as pkg
from hf_kernels_helion_b200 import _lib, runtime


def main(argv):
    if len(argv) < 5:
        print(__doc__)
        return 2
    variant, M, N, K = argv[1], int(argv[2]), int(argv[3]), int(argv[4])
    launches = int(argv[5]) if len(argv) > 5 else 4
    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    if variant == "quant":
        x = torch.randn(M, K, device=dev).to(torch.bfloat16)
        run = lambda: pkg.fp8_act_quant(x)
        work, unit = M * K * (2 + 1) + 4 * M * (K // 128), "GB/s"
    elif variant == "rowscale":
        A = (torch.randn(M, K, device=dev) * 0.3).to(torch.float8_e4m3fn)
        B = (torch.randn(N, K, device=dev) * 0.3).to(torch.float8_e4m3fn)
        As = torch.rand(M, K // 128, device=dev) * 0.5 + 0.5
        Bs = torch.rand(N, K // 128, device=dev) * 0.5 + 0.5
        run = lambda: runtime.gemm_rowscale(A, B, As, Bs, 128, torch.bfloat16)
        work, unit = 2 * M * N * K, "TFLOP/s"
    else:
        if variant not in _lib.VARIANT_NAMES:
            raise SystemExit(f"unknown variant {variant!r}; one of {sorted(_lib.VARIANT_NAMES)}, 'rowscale' or 'quant'")
        A = (torch.randn(M, K, device=dev) * 0.3).to(torch.float8_e4m3fn)
        B = (torch.randn(N, K, device=dev) * 0.3).to(torch.float8_e4m3fn)
        As = torch.rand(M, K // 128, device=dev) * 0.5 + 0.5
        Bs = torch.rand((N + 127) // 128, K // 128, device=dev) * 0.5 + 0.5
        run = lambda: runtime.gemm(A, B, As, Bs, 128, 128, torch.bfloat16, variant=variant)
        work, unit = 2 * M * N * K, "TFLOP/s"
    run()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(max(launches - 1, 1)):
        run()
    stop.record()
    torch.cuda.synchronize()
    pkg.check_device_status()
    ms = start.elapsed_time(stop) / max(launches - 1, 1)
    rate = work / (ms * 1e-3) / (1e9 if unit == "GB/s" else 1e12)
    print(f"{variant} M={M} N={N} K={K}: {ms * 1e3:.1f} us per launch, {rate:.1f} {unit} "
          f"(host-launched, includes launch gaps)")
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv))

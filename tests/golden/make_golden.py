"""Generate tests/golden/*.npz from the REFERENCE's own source files.

Run once, in a container that has the reference checkout (default
``~/reference``, override with ``REFERENCE_ROOT``):

    python tests/golden/make_golden.py

Two pieces of reference code are executed, unmodified, on the CPU:

1. ``finegrained-fp8-helion/bench.py`` function ``ref`` (lines 11-14): the file cannot
   be imported as a module (it imports the ``kernels`` package and a hard-coded path at
   the top), so the function definition is taken out of the parsed file with ``ast``
   and compiled by itself.  It expects per-row B scales ``[N, K // bk]``; the block
   scales ``Bs [N // 128, K // 128]`` are expanded with ``repeat_interleave(128, 0)``
   first, which is the same matrix of per-element scales.

2. ``finegrained-fp8-helion/finegrained-fp8-helion/torch-ext/finegrained_fp8_helion/fp8.py``
   (the Helion kernel, lines 19-39).  Helion is not installed, so the module is loaded
   with a ~60-line eager stand-in for the four DSL entry points the kernel uses
   (``helion.aot_kernel``, ``hl.tile``, ``hl.zeros``, ``hl.dot``): tiles become Python
   slices and the kernel body then runs as ordinary torch on the CPU, statement by
   statement as written.  The M tile size, which the kernel leaves to the autotuner
   (``block_size=[None, block_n]``), is taken from the shipped sm_100 heuristic
   ``_helion_aot_fp8_cuda_sm100.py``.

3. ``deep-gemm-helion/deep-gemm-helion/torch-ext/deep_gemm_helion/fp8.py`` (the second
   block-FP8 kernel, one B scale per row of B; lines 13-29) under the same stand-in, and
   ``deep-gemm-helion/bench.py`` function ``ref`` (lines 11-14) taken out with ``ast``;
   ``python tests/golden/make_golden.py deep-gemm`` writes only these fixtures.

The inputs are the seeded synthetic tensors of oracle/fp8_oracle.py; each fixture
stores the inputs' bytes (small cases) or their SHA-256 (the 512x512x2048
configuration) next to the outputs so a drift of the generator is told apart from a
drift of the arithmetic.
"""
from __future__ import annotations

import ast
import hashlib
import importlib.util
import os
import sys
import types
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))
from oracle import fp8_oracle as oracle  # noqa: E402

REF = Path(os.environ.get("REFERENCE_ROOT", str(Path.home() / "reference")))
FP8_DIR = REF / "finegrained-fp8-helion" / "finegrained-fp8-helion" / "torch-ext" / "finegrained_fp8_helion"


# --------------------------------------------------------------------------- (1) bench.py:ref

def load_bench_ref():
    src = (REF / "finegrained-fp8-helion" / "bench.py").read_text()
    tree = ast.parse(src)
    fn = next(n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name == "ref")
    mod = ast.Module(body=[fn], type_ignores=[])
    ns = {"torch": torch}
    exec(compile(mod, "reference:finegrained-fp8-helion/bench.py", "exec"), ns)
    return ns["ref"]


# --------------------------------------------------------------------------- (2) eager stand-in for helion

class _Tile:
    def __init__(self, begin, end):
        self.begin, self.end = begin, end

    def __len__(self):
        return self.end - self.begin


def _conv(idx):
    if isinstance(idx, tuple):
        return tuple(_conv(i) for i in idx)
    if isinstance(idx, _Tile):
        return slice(idx.begin, idx.end)
    return idx


class _TileTensor(torch.Tensor):
    """torch.Tensor that accepts _Tile objects as indices."""

    @classmethod
    def __torch_function__(cls, func, types_, args=(), kwargs=None):
        with torch._C.DisableTorchFunctionSubclass():
            return func(*args, **(kwargs or {}))

    def __getitem__(self, idx):
        return self.as_subclass(torch.Tensor)[_conv(idx)]

    def __setitem__(self, idx, value):
        self.as_subclass(torch.Tensor)[_conv(idx)] = value


class _TorchProxy:
    """Forwards to torch, except that empty() returns a tile-indexable tensor."""

    def __getattr__(self, name):
        return getattr(torch, name)

    @staticmethod
    def empty(*a, **k):
        return torch.empty(*a, **k).as_subclass(_TileTensor)


def _make_helion_stub(m_tile_for):
    helion = types.ModuleType("helion")
    hl = types.ModuleType("helion.language")
    state = {"m_tile": 128}

    def tile(sizes, block_size=None):
        if isinstance(sizes, (list, tuple)):
            bs = [None] * len(sizes) if block_size is None else list(block_size)
            bs = [state["m_tile"] if b is None else int(b) for b in bs]
            M, N = int(sizes[0]), int(sizes[1])
            for m0 in range(0, M, bs[0]):
                for n0 in range(0, N, bs[1]):
                    yield _Tile(m0, min(m0 + bs[0], M)), _Tile(n0, min(n0 + bs[1], N))
        else:
            b = int(block_size)
            for k0 in range(0, int(sizes), b):
                yield _Tile(k0, min(k0 + b, int(sizes)))

    def zeros(shape, dtype=torch.float32):
        return torch.zeros([len(s) if isinstance(s, _Tile) else int(s) for s in shape], dtype=dtype)

    def dot(a, b):
        return a @ b

    def aot_kernel(**_kw):
        def deco(fn):
            def run(*args):
                state["m_tile"] = m_tile_for(*args)
                wrapped = [a.as_subclass(_TileTensor) if isinstance(a, torch.Tensor) else a for a in args]
                g = fn.__globals__
                saved = g["torch"]
                g["torch"] = _TorchProxy()
                try:
                    return fn(*wrapped).as_subclass(torch.Tensor)
                finally:
                    g["torch"] = saved
            return run
        return deco

    hl.tile, hl.zeros, hl.dot, hl.constexpr = tile, zeros, dot, int
    helion.aot_kernel, helion.kernel, helion.language = aot_kernel, aot_kernel, hl
    return helion, hl


def load_reference_kernel():
    spec = importlib.util.spec_from_file_location("_ref_heur", FP8_DIR / "_helion_aot_fp8_cuda_sm100.py")
    heur = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(heur)

    def m_tile_for(*args):
        return int(heur.autotune__w8a8_block_fp8_matmul(*args)["block_sizes"][0])

    helion, hl = _make_helion_stub(m_tile_for)
    sys.modules["helion"], sys.modules["helion.language"] = helion, hl
    try:
        spec = importlib.util.spec_from_file_location("_ref_fp8", FP8_DIR / "fp8.py")
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
    finally:
        del sys.modules["helion"], sys.modules["helion.language"]
    return mod._w8a8_block_fp8_matmul


# --------------------------------------------------------------------------- (3) deep-gemm-helion

DG_DIR = REF / "deep-gemm-helion" / "deep-gemm-helion" / "torch-ext" / "deep_gemm_helion"


def load_deep_gemm_kernel():
    """deep_gemm_helion/fp8.py:13-29 under the same eager stand-in. Its tiles over [M, N] are left
    entirely to the autotuner (`hl.tile([M, N])`); 128 x 128 is used."""
    helion, hl = _make_helion_stub(lambda *args: 128)
    sys.modules["helion"], sys.modules["helion.language"] = helion, hl
    try:
        spec = importlib.util.spec_from_file_location("_ref_dg_fp8", DG_DIR / "fp8.py")
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
    finally:
        del sys.modules["helion"], sys.modules["helion.language"]
    return mod._fp8_blockwise_gemm


def load_deep_gemm_bench_ref():
    src = (REF / "deep-gemm-helion" / "bench.py").read_text()
    tree = ast.parse(src)
    fn = next(n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name == "ref")
    ns = {"torch": torch}
    exec(compile(ast.Module(body=[fn], type_ignores=[]), "reference:deep-gemm-helion/bench.py", "exec"), ns)
    return ns["ref"]


def make_deep_gemm_fixtures():
    kernel, bench_ref = load_deep_gemm_kernel(), load_deep_gemm_bench_ref()
    for name, (M, N, K, seed) in {"rowscale_96x256x384": (96, 256, 384, 11), "rowscale_130x128x256": (130, 128, 256, 12),
                                  "rowscale_1x384x512": (1, 384, 512, 13)}.items():
        A, B, As, Bs = oracle.make_rowscale_inputs(M, N, K, seed)
        out_kernel = kernel(A, B, As, Bs, 128)              # bf16, as the op returns it
        out_bench = bench_ref(A, B, As, Bs, 128)            # bf16
        np.savez_compressed(HERE / f"{name}.npz", M=M, N=N, K=K, seed=seed,
                            A=A.view(torch.uint8).numpy(), B=B.view(torch.uint8).numpy(),
                            As=As.numpy(), Bs=Bs.numpy(),
                            out_kernel_bf16_bits=out_kernel.view(torch.int16).numpy(),
                            out_bench_bf16_bits=out_bench.view(torch.int16).numpy())
        print(name, "kernel-vs-bench max/rms", oracle.max_err_over_rms(out_kernel.float(), out_bench.float()))


# --------------------------------------------------------------------------- fixtures

def sha(t: torch.Tensor) -> str:
    return hashlib.sha256(t.contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()


def main():
    bench_ref = load_bench_ref()
    kernel = load_reference_kernel()

    # small cases: inputs stored in full (ragged M; N, K multiples of 128 as the reference's scale shapes imply)
    for name, (M, N, K, seed) in {"small_96x256x384": (96, 256, 384, 1), "small_130x128x256": (130, 128, 256, 2),
                                  "small_1x384x512": (1, 384, 512, 3)}.items():
        A, B, As, Bs = oracle.make_quantised_inputs(M, N, K, seed)
        out_kernel = kernel(A, B, As, Bs, 128, 128)                        # fp32, as the op returns it
        out_bench = bench_ref(A, B, As, Bs.repeat_interleave(128, dim=0)[:N], 128)  # bf16
        np.savez_compressed(HERE / f"{name}.npz", M=M, N=N, K=K, seed=seed,
                            A=A.view(torch.uint8).numpy(), B=B.view(torch.uint8).numpy(),
                            As=As.numpy(), Bs=Bs.numpy(),
                            out_kernel_fp32=out_kernel.numpy(),
                            out_bench_bf16_bits=out_bench.view(torch.int16).numpy())
        print(name, "kernel-vs-bench max/rms", oracle.max_err_over_rms(out_kernel, out_bench.float()))

    # configuration 1 of the benchmark (512 x 512 x 2048, seed 0): inputs by hash, outputs subsampled
    M, N, K = 512, 512, 2048
    A, B, As, Bs = oracle.make_quantised_inputs(M, N, K, 0)
    out_kernel = kernel(A, B, As, Bs, 128, 128)
    out_bench = bench_ref(A, B, As, Bs.repeat_interleave(128, dim=0)[:N], 128)
    np.savez_compressed(HERE / "config1_512x512x2048.npz", M=M, N=N, K=K, seed=0,
                        sha_A=sha(A), sha_B=sha(B), sha_As=sha(As), sha_Bs=sha(Bs),
                        row_step=7, col_step=5,
                        out_kernel_fp32=out_kernel[::7, ::5].contiguous().numpy(),
                        out_bench_bf16_bits=out_bench[::7, ::5].contiguous().view(torch.int16).numpy(),
                        out_kernel_sum=np.float64(out_kernel.double().sum().item()),
                        out_kernel_abs_sum=np.float64(out_kernel.double().abs().sum().item()))
    print("config1 kernel-vs-bench max/rms", oracle.max_err_over_rms(out_kernel, out_bench.float()))


if __name__ == "__main__":
    if sys.argv[1:] == ["deep-gemm"]:
        make_deep_gemm_fixtures()
    else:
        main()
        make_deep_gemm_fixtures()

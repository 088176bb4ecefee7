"""Write the package as a `kernels`-style loadable tree:

    python -m hf_kernels_helion_b200.make_tree OUT_DIR

produces the layout the reference ships for `finegrained-fp8-helion`
(finegrained-fp8-helion/finegrained-fp8-helion/build/torch-cuda/: the package's modules flat in one
directory, `metadata.json`, and a sub-directory named like the kernel whose `__init__.py` loads the
flat `__init__.py` by path) so that `PYTHONPATH=OUT_DIR/torch-cuda` makes
`import finegrained_fp8_helion` resolve to this implementation:

    OUT_DIR/torch-cuda/__init__.py _ops.py op.py runtime.py _lib.py tp.py libb200fp8.so metadata.json
    OUT_DIR/torch-cuda/finegrained_fp8_helion/__init__.py
    OUT_DIR/benchmarks/benchmark.py        setup / benchmark_* / verify_* for kernels.benchmark

`metadata.json` keeps the reference's name, id and backend and has an empty `python-depends`
(the reference's is ["helion"], build.toml:9). The tree is binary: it carries the built
`libb200fp8.so`, not the CUDA sources.
"""
from __future__ import annotations

import json
import shutil
import sys
from pathlib import Path

from . import build as _build

KERNEL_NAME = "finegrained_fp8_helion"
MODULES = ["__init__.py", "_ops.py", "op.py", "runtime.py", "_lib.py", "tp.py"]

SHIM = '''"""Loads the flat package one directory up under a private module name and re-exports it."""
import importlib.util
import sys
from pathlib import Path

_init = Path(__file__).resolve().parent.parent / "__init__.py"
_name = "_b200fp8_tree_%x" % (hash(str(_init)) & 0xFFFFFFFFFFFF)
_spec = importlib.util.spec_from_file_location(_name, _init, submodule_search_locations=[str(_init.parent)])
_mod = importlib.util.module_from_spec(_spec)
sys.modules[_name] = _mod
_spec.loader.exec_module(_mod)
globals().update({k: v for k, v in vars(_mod).items() if not k.startswith("__")})
__all__ = list(getattr(_mod, "__all__", []))
'''

BENCHMARK = '''"""Benchmark cases for the `kernels` benchmark runner: one class, three workloads.
Each `benchmark_<name>` runs the op, `verify_<name>` returns the fp32 dequantise-then-matmul result
the runner compares `self.out` with."""
import torch

try:
    from kernels.benchmark import Benchmark
except ImportError:                      # runner absent: a stand-in with the two attributes used here
    class Benchmark:
        def __init__(self, kernel=None, device="cuda"):
            self.kernel, self.device = kernel, torch.device(device)


def _inputs(M, N, K, device):
    g = torch.Generator(device="cpu").manual_seed(0)
    a = (torch.randn(M, K, generator=g) * 0.3).to(torch.float8_e4m3fn).to(device)
    b = (torch.randn(N, K, generator=g) * 0.3).to(torch.float8_e4m3fn).to(device)
    sa = (torch.rand(M, K // 128, generator=g) * 0.5 + 0.5).to(device)
    sb = (torch.rand(N // 128, K // 128, generator=g) * 0.5 + 0.5).to(device)
    return a, b, sa, sb


def _reference(a, b, sa, sb):
    af = a.float() * sa.repeat_interleave(128, 1)
    bf = b.float() * sb.repeat_interleave(128, 0).repeat_interleave(128, 1)
    return (af @ bf.T).to(torch.bfloat16)


class FinegrainedFp8HelionBenchmark(Benchmark):
    seed = 0

    def _setup(self, M, N, K):
        self.a, self.b, self.sa, self.sb = _inputs(M, N, K, self.device)
        self.out = torch.empty(M, N, dtype=torch.bfloat16, device=self.device)

    def _run(self):
        self.out = self.kernel.w8a8_block_fp8_matmul(self.a, self.b, self.sa, self.sb, [128, 128], torch.bfloat16)

    def setup(self):
        self._setup(2048, 2048, 4096)

    def benchmark_base(self):
        self._run()

    def verify_base(self) -> torch.Tensor:
        return _reference(self.a, self.b, self.sa, self.sb)

    def setup_large(self):
        self._setup(4096, 4096, 8192)

    def benchmark_large(self):
        self._run()

    def verify_large(self) -> torch.Tensor:
        return _reference(self.a, self.b, self.sa, self.sb)

    def setup_decode(self):
        self._setup(16, 28672, 8192)

    def benchmark_decode(self):
        self._run()

    def verify_decode(self) -> torch.Tensor:
        return _reference(self.a, self.b, self.sa, self.sb)
'''


def make_tree(out_dir: Path) -> Path:
    lib = _build.build()
    pkg = Path(__file__).resolve().parent
    root = out_dir / "torch-cuda"
    (root / KERNEL_NAME).mkdir(parents=True, exist_ok=True)
    (out_dir / "benchmarks").mkdir(parents=True, exist_ok=True)
    for name in MODULES:
        shutil.copy2(pkg / name, root / name)
    shutil.copy2(lib, root / lib.name)
    meta = {
        "name": "finegrained-fp8-helion",
        "id": "_finegrained_fp8_helion_cuda_b0d7177",
        "version": 1,
        "license": "Apache-2.0",
        "python-depends": [],
        "backend": {"type": "cuda", "archs": ["10.0a"]},
    }
    (root / "metadata.json").write_text(json.dumps(meta, indent=2) + "\n")
    (root / KERNEL_NAME / "__init__.py").write_text(SHIM)
    (out_dir / "benchmarks" / "benchmark.py").write_text(BENCHMARK)
    return root


if __name__ == "__main__":
    if len(sys.argv) != 2:
        print(__doc__)
        sys.exit(2)
    print(make_tree(Path(sys.argv[1])))

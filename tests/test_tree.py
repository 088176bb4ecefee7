"""The `kernels`-style loadable tree written by hf_kernels_helion_b200.make_tree: same layout as the
reference's build/torch-cuda, importable as `finegrained_fp8_helion` with PYTHONPATH alone.
Each check runs in a child process: the tree registers the same torch op namespace as the package."""
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest

REPO = Path(__file__).resolve().parent.parent


def _make(tmp_path):
    from hf_kernels_helion_b200 import make_tree
    return make_tree.make_tree(tmp_path / "result")


def _run(root, code, timeout=300):
    env = dict(os.environ, PYTHONPATH=str(root))
    return subprocess.run([sys.executable, "-c", code], cwd=str(root.parent), env=env, capture_output=True, text=True,
                          timeout=timeout)


def test_tree_layout_and_import(tmp_path):
    root = _make(tmp_path)
    names = {p.name for p in root.iterdir()}
    assert {"__init__.py", "_ops.py", "op.py", "metadata.json", "libb200fp8.so", "finegrained_fp8_helion"} <= names
    meta = json.loads((root / "metadata.json").read_text())
    assert meta["id"] == "_finegrained_fp8_helion_cuda_b0d7177" and meta["python-depends"] == []
    assert (root.parent / "benchmarks" / "benchmark.py").exists()
    res = _run(root, "import finegrained_fp8_helion as k, torch, inspect\n"
                     "assert 'w8a8_block_fp8_matmul' in k.__all__\n"
                     "sig = inspect.signature(k.w8a8_block_fp8_matmul)\n"
                     "assert list(sig.parameters)[:5] == ['A', 'B', 'As', 'Bs', 'block_size']\n"
                     "assert sig.parameters['output_dtype'].default is torch.float32\n"
                     "op = torch.ops._finegrained_fp8_helion_cuda_b0d7177.w8a8_block_fp8_matmul\n"
                     "assert 'hf_kernels_helion_b200' not in __import__('sys').modules\n"
                     "print('ok')")
    assert res.returncode == 0 and "ok" in res.stdout, res.stderr


@pytest.mark.gpu
def test_tree_runs_on_gpu(tmp_path):
    root = _make(tmp_path)
    code = f"""
import sys, torch
sys.path.insert(0, {str(REPO)!r})
import finegrained_fp8_helion as k
from oracle import fp8_oracle as oracle
A, B, As, Bs = oracle.make_quantised_inputs(256, 512, 1024, 0)
out = k.w8a8_block_fp8_matmul(A.cuda(), B.cuda(), As.cuda(), Bs.cuda(), [128, 128], torch.bfloat16)
ref = oracle.gemm_dequant(A, B, As, Bs)
assert oracle.bf16_ulp_error(out.cpu(), ref) <= 1
sys.path.insert(0, {str(root.parent / 'benchmarks')!r})
import benchmark
b = benchmark.FinegrainedFp8HelionBenchmark(kernel=k, device='cuda')
b.setup(); b.benchmark_base(); torch.cuda.synchronize()
want = b.verify_base()
err = (b.out.float() - want.float()).abs().max().item() / want.float().pow(2).mean().sqrt().item()
assert err < 2e-2, err
k.check_device_status()
print('ok')
"""
    res = _run(root, code)
    assert res.returncode == 0 and "ok" in res.stdout, res.stdout + res.stderr

"""The reference arm of bench.py runs on the CPU: its JSON line must carry the keys of the
benchmark contract (the GPU arm prints the same keys plus roofline / clocks / extra_shapes)."""
import json
import os
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def test_reference_arm_prints_one_contract_line():
    env = dict(os.environ)
    env.pop("RANK", None)
    res = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "1"],
                         cwd=str(ROOT), env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr
    lines = [l for l in res.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    for key in ("impl", "metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better",
                "scaling", "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e", "gpu_launches"):
        assert key in d, key
    assert d["impl"] == "reference" and d["unit"] == "TFLOP/s" and d["value"] > 0 and d["gpu_launches"] == 0
    assert d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["cores"] >= 1
    assert d["e2e"]["h2d_bytes_per_step"] == 0 and d["e2e"]["d2h_bytes_per_step"] == 0
    assert "workload" in d["config"] and "model" not in d["config"]


def test_reference_arm_is_silent_on_other_ranks():
    env = dict(os.environ, RANK="1", WORLD_SIZE="2")
    res = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "1",
                          "--warmup", "1"], cwd=str(ROOT), env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0 and res.stdout.strip() == ""


def test_bench_inputs_are_the_oracle_generator(monkeypatch):
    """The GPU arm draws its inputs on the CPU from seed 0, activations first, then the weight - the
    sequence of oracle.make_inputs - so that its parity check compares like with like."""
    import importlib
    import sys as _sys

    import torch

    _sys.path.insert(0, str(ROOT))
    bench = importlib.import_module("bench")
    from oracle import fp8_oracle as oracle

    monkeypatch.setattr(bench, "M", 48)
    monkeypatch.setattr(bench, "K", 256)
    monkeypatch.setattr(bench, "N", 384)
    (a0, a1), w = bench.make_inputs_cpu()
    a_ref, w_ref = oracle.make_inputs(48, 384, 256, seed=0)
    assert torch.equal(a0, a_ref) and torch.equal(w, w_ref)
    assert a1.shape == a0.shape and not torch.equal(a1, a0)


def test_clock_sampler_window():
    import importlib
    import sys as _sys

    _sys.path.insert(0, str(ROOT))
    bench = importlib.import_module("bench")
    s = bench.ClockSampler(0)
    row = lambda mhz, cap: ["0", str(mhz), "1965", "900.0", "0x4", "Not Active", "Not Active", "Not Active", cap]  # noqa: E731
    s.rows = [(10.0, row(1500, "Active")), (10.5, row(1600, "Active")), (11.0, row(1900, "Not Active")), (20.0, ["bad"])]
    w = s.window(9.9, 10.6)
    assert w["sm_mhz"] == 1550.0 and w["samples"] == 2 and w["reasons"] == ["sw_power_cap"] and w["sm_max_mhz"] == 1965.0
    assert s.window(10.9, 11.1)["reasons"] == []
    assert s.window(30.0, 31.0) is None

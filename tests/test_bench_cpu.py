"""bench.py on a machine without a GPU: its own arm refuses to run (there is no CPU path to fall back to), and the
reference arm -- the CPU restatement timed on the host cores -- prints the contract's line."""
import json
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


def _run(*args, timeout=600):
    env = {k: v for k, v in os.environ.items() if k not in ("RANK", "WORLD_SIZE", "LOCAL_RANK")}
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True, timeout=timeout,
                          cwd=ROOT, env=env)


def test_own_arm_needs_a_gpu_and_says_so():
    import torch
    if torch.cuda.is_available():
        import pytest
        pytest.skip("a CUDA device is present")
    out = _run("--steps", "1", "--warmup", "1")
    assert out.returncode != 0
    assert "no CPU path" in out.stderr
    assert '"value"' not in out.stdout          # nothing that could be read as a measurement


def test_reference_arm_prints_the_contract_line():
    out = _run("--impl", "reference", "--steps", "2", "--warmup", "1")
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [ln for ln in out.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["metric"] == "fp64_equiv_tflops" and d["unit"] == "TFLOP/s"
    assert d["n_gpus"] == 1 and d["steps"] == 2 and d["warmup"] == 1 and d["higher_is_better"] is True
    assert d["value"] > 0 and d["ms_per_step"] > 0
    assert d["e2e"] == {"value": d["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    cb = d["cpu_baseline"]
    assert cb["kind"] == "port" and cb["value"] == d["value"] and cb["cores"] >= 1 and "block" in cb["sample"]
    assert d["config"]["n"] == 8192 and d["config"]["moduli"] == 16 and "workload" in d["config"]
    assert d["extrapolated"] is True and d["rows_timed"] >= 1 and d["cols_timed"] >= 1


def test_arguments_keep_the_contract_defaults():
    sys.path.insert(0, ROOT)
    import importlib
    bench = importlib.import_module("bench")
    src = open(os.path.join(ROOT, "bench.py")).read()
    for flag in ("--gpus", "--steps", "--warmup", "--impl", "--rows", "--strong", "--strong-size", "--e2e-steps"):
        assert f'"{flag}"' in src, flag
    cfg = bench.workload_config(8192, 16, 8)
    assert cfg["M_total"] == 8192 * 8 and cfg["parallelism"] == "row-block x8" and "model" not in cfg

"""The benchmark program's command-line contract as far as it can be checked without a device (CPU)."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(*args):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True, timeout=300,
                          env=dict(os.environ, PYTHONPATH=ROOT, CUDA_VISIBLE_DEVICES=""))


def test_reference_arm_without_a_device_prints_one_unavailable_line_and_exits_zero():
    r = _run("--impl", "reference", "--gpus", "1", "--steps", "1", "--warmup", "1")
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [l for l in r.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and isinstance(d["unavailable"], str) and "\n" not in d["unavailable"]


def test_help_lists_the_contract_flags_and_defaults_are_small():
    r = _run("--help")
    assert r.returncode == 0
    for flag in ("--gpus", "--steps", "--warmup", "--impl"):
        assert flag in r.stdout
    src = open(os.path.join(ROOT, "bench.py")).read()
    for key in ('"metric"', '"value"', '"unit"', '"n_gpus"', '"ms_per_step"', '"higher_is_better"', '"scaling"', '"vs_baseline"', '"dtype"',
                '"data"', '"config"', '"e2e"', '"gpu_launches"', '"clocks"', "h2d_bytes_per_step", "d2h_bytes_per_step"):
        assert key in src, key                                                # every key of the one-line result is produced somewhere


def test_a_result_line_parses_into_schema_rows():
    from scirust_b200.utils.bench_schema import from_bench_line
    line = json.dumps({"metric": "train_tokens_per_s", "value": 600000.0, "unit": "tok/s", "n_gpus": 1, "steps": 10, "warmup": 3,
                       "ms_per_step": 27.3, "higher_is_better": True, "scaling": "weak", "vs_baseline": 150.0, "dtype": "bf16",
                       "data": "synthetic", "config": {"model": "sciagent-12l", "global_batch": 8, "seq_len": 2048, "parallelism": "dp1"},
                       "e2e": {"value": 590000.0, "unit": "tok/s", "h2d_bytes_per_step": 131072, "d2h_bytes_per_step": 4}, "gpu_launches": 400})
    rows = from_bench_line(line)
    assert [r.value for r in rows] == [600000.0, 590000.0, 27.3] and rows[1].method.endswith(":e2e") and rows[0].dataset == "synthetic:B8xS2048"

"""The CPU arm of bench.py (`--impl reference`: the reference's CPU implementation of the forward timed on a bounded
sample) prints one JSON line with the keys the benchmark contract names, in both of its forms: the reference's own
golden when its files have been fetched (oracle/fetch_reference.py), the restatement otherwise.  Runs a tiny sample
so that it finishes in seconds."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


import pytest

HAVE_REF = os.path.isfile(os.path.join(ROOT, "baseline", "_ref", "hstu_v2", "backend", "pytorch_native_backend.py"))


@pytest.mark.parametrize("kind", ["reference", "port"])
def test_reference_arm_prints_the_contract_line(kind):
    if kind == "reference" and not HAVE_REF:
        pytest.skip("the reference's files have not been fetched into baseline/_ref")
    env = dict(os.environ)
    if kind == "port":
        env["HSTU_NO_REFERENCE_FILES"] = "1"
    proc = subprocess.run(
        [sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--workload", "cfg2", "--max-batch", "8",
         "--steps", "1", "--warmup", "0"],
        cwd=ROOT, env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=300)
    assert proc.returncode == 0, proc.stderr[-2000:]
    line = json.loads(proc.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference"
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e"):
        assert key in line, key
    assert line["metric"] == "hstu_jagged_fwd_causal_tflops" and line["unit"] == "TFLOP/s"
    assert line["value"] > 0 and line["cpu_baseline"]["kind"] == kind and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["e2e"]["value"] == line["value"]
    assert "workload" in line["config"] and "model" not in line["config"]


def test_non_zero_ranks_of_the_reference_arm_stay_silent():
    env = dict(os.environ, RANK="1", LOCAL_RANK="1", WORLD_SIZE="2")
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2"],
                          cwd=ROOT, env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=120)
    assert proc.returncode == 0 and proc.stdout.strip() == ""

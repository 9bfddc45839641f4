"""CPU: the benchmark's command line as the driver uses it.

`bench.py --impl reference` runs anywhere (it times the CPU formulation of the step on the host cores) and
must print ONE JSON line with the keys of the repository arm plus `impl`; the repository arm itself must
not quietly fall back to the CPU when no GPU is present.
"""

import json
import pathlib
import subprocess
import sys

import pytest
import torch

ROOT = pathlib.Path(__file__).resolve().parents[1]


def _run(*flags):
    return subprocess.run([sys.executable, str(ROOT / "bench.py"), *flags], capture_output=True, text=True, cwd=ROOT,
                          timeout=600)


def test_reference_arm_prints_one_json_line_with_the_contract_keys():
    r = _run("--impl", "reference", "--steps", "1", "--warmup", "1")
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [ln for ln in r.stdout.splitlines() if ln.strip()]
    assert len(lines) == 1
    line = json.loads(lines[0])
    assert line["impl"] == "reference" and line["n_gpus"] == 1 and line["higher_is_better"] is True
    for key in ("metric", "value", "unit", "steps", "warmup", "ms_per_step", "scaling", "vs_baseline", "dtype", "data",
                "config", "cpu_baseline", "e2e"):
        assert key in line, key
    assert line["value"] > 0 and line["unit"] == "GB/s" and "workload" in line["config"]
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["cpu_baseline"]["value"] == pytest.approx(line["value"])
    e2e = line["e2e"]
    assert e2e["value"] == pytest.approx(line["value"]) and e2e["unit"] == line["unit"]
    assert e2e["h2d_bytes_per_step"] == 0 and e2e["d2h_bytes_per_step"] == 0


@pytest.mark.skipif(torch.cuda.is_available(), reason="needs a machine without a GPU")
def test_repository_arm_fails_loudly_without_a_gpu():
    r = _run("--steps", "1", "--warmup", "1", "--headline-only", "--no-cpu-baseline")
    assert r.returncode != 0
    assert not r.stdout.strip()   # no result line from a CPU fallback

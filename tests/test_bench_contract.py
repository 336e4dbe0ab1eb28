"""The reference arm of bench.py on the host cores (no GPU): one JSON line
with the keys the bench contract names, measured by the reference's own CPU
build, and nothing for the ranks other than rank 0."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "oracle", "_ref", "libiris_ref_blas.so")


def run_reference_arm(env_extra, *flags):
    env = dict(os.environ, **env_extra)
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1",
                          "--warmup", "0"] + list(flags), capture_output=True, text=True, env=env, timeout=600, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    return [l for l in out.stdout.splitlines() if l.startswith("{")]


@pytest.mark.skipif(not os.path.exists(REF), reason="the reference's CPU build (oracle/_ref) is not here")
def test_reference_arm_prints_one_line_with_the_contract_keys():
    lines = run_reference_arm({})
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["n_gpus"] == 1 and d["steps"] == 1 and d["higher_is_better"] is True
    assert d["unit"] == "TFLOP/s" and d["value"] > 0 and d["ms_per_step"] > 0 and d["vs_baseline"] is None
    assert d["config"]["workload"] == "klein4b-1024" and d["config"]["tokens"] == 4608 and d["config"]["heads"] == 24
    cpu = d["cpu_baseline"]
    assert cpu["kind"] == "reference" and cpu["cores"] >= 1 and cpu["value"] == d["value"] and cpu["sample"]
    assert d["e2e"] == {"value": d["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert d["gpu_launches"] == 0


def test_reference_arm_is_silent_on_the_other_ranks():
    assert run_reference_arm({"RANK": "1", "WORLD_SIZE": "2", "LOCAL_RANK": "1"}, "--gpus", "2") == []

"""bench.py's command line without a GPU: the reference arm runs (it is the reference's own CPU code, or the
restatement, on a bounded sample), the own arm refuses to run instead of falling back to the CPU."""
import json
import os
import subprocess
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(*args, timeout=300):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True,
                          timeout=timeout, cwd=ROOT)


def test_reference_arm_prints_one_json_line_with_the_contract_keys():
    r = _run("--impl", "reference", "--steps", "1", "--warmup", "0", "--cpu-sample-div", "2048")
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [ln for ln in r.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["metric"] == "gcn_train_epoch_ms" and d["unit"] == "ms"
    assert d["higher_is_better"] is False and d["n_gpus"] == 1 and d["vs_baseline"] is None
    assert d["value"] > 0 and d["ms_per_step"] == d["value"]
    assert d["config"]["workload"].startswith("rmat_products") and "model" not in d["config"]
    cb = d["cpu_baseline"]
    assert cb["kind"] in ("reference", "port") and cb["cores"] >= 1 and cb["value"] == d["value"] and cb["sample"]
    assert d["e2e"] == {"value": d["value"], "unit": "ms", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert d["gpu_launches"] == 0
    # the arm runs without the package's CUDA library in the process
    assert all("graphcuda_b200" not in so for so in d["shared_objects_of_this_repo_loaded"])
    # the value is an extrapolation and says so: both measured points and the growth exponent are in the line
    assert cb["extrapolated"] is True and cb["measured"]["ms_per_step"] > 0 and cb["second_point"]["ms_per_step"] > 0
    assert 0.5 < cb["growth_exponent"] < 2.0


def test_own_arm_needs_a_gpu_and_says_so():
    if torch.cuda.is_available():
        return  # covered by the GPU runs
    r = _run("--steps", "1", "--warmup", "0", "--no-aux", "--no-cpu-baseline")
    assert r.returncode != 0
    assert "no CPU path" in (r.stderr + r.stdout)

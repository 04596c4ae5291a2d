"""The CPU-runnable part of bench.py's contract: the reference arm prints ONE JSON line with the agreed keys, on one
process and under torchrun (rank 0 alone works and prints; the other ranks exit 0 without output)."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
KEYS = {"impl", "metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
        "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e"}


def _check(out: str, n_gpus: int):
    lines = [l for l in out.splitlines() if l.strip()]
    assert len(lines) == 1, out
    d = json.loads(lines[0])
    assert KEYS <= set(d) and d["impl"] == "reference" and d["n_gpus"] == n_gpus and d["vs_baseline"] is None
    assert d["value"] > 0 and d["unit"] == "TFLOP/s" and d["higher_is_better"] is True
    assert d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["cores"] >= 1 and d["cpu_baseline"]["value"] == d["value"]
    assert d["e2e"] == {"value": d["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert "workload" in d["config"] and "model" not in d["config"]
    return d


def test_reference_arm_single_process():
    r = subprocess.run([sys.executable, "bench.py", "--impl", "reference", "--steps", "1", "--warmup", "1"], cwd=ROOT,
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert _check(r.stdout, 1)["scaling"] == "weak"


def test_reference_arm_under_torchrun_uses_all_cores_on_rank0():
    env = dict(os.environ, OMP_NUM_THREADS="1")  # what torchrun exports to its workers
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
                        "127.0.0.1", "--master-port", "29541", "bench.py", "--impl", "reference", "--gpus", "2", "--steps", "1",
                        "--warmup", "1"], cwd=ROOT, capture_output=True, text=True, timeout=900, env=env)
    assert r.returncode == 0, r.stderr[-2000:]
    d = _check(r.stdout, 2)
    assert d["scaling"] == "strong" and d["cpu_baseline"]["cores"] == len(os.sched_getaffinity(0))

"""The CPU arm of bench.py runs without a GPU: its JSON line carries the keys the benchmark contract names."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _line(*argv, env=None):
    e = dict(os.environ)
    e.update(env or {})
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py")] + list(argv), capture_output=True, text=True,
                       timeout=600, env=e)
    assert r.returncode == 0, r.stderr[-2000:]
    return r.stdout.strip().splitlines()


def test_reference_arm_line():
    out = _line("--impl", "reference", "--workload", "cfg1", "--steps", "2", "--warmup", "1")
    assert len(out) == 1
    d = json.loads(out[0])
    for key in ("impl", "metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better",
                "scaling", "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e"):
        assert key in d, key
    assert d["impl"] == "reference" and d["unit"] == "GFLOP/s" and d["value"] > 0 and d["n_gpus"] == 1
    assert d["config"]["workload"] == "cfg1" and d["dtype"] == "f64" and d["vs_baseline"] is None
    assert d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["cores"] >= 1
    assert d["e2e"]["value"] == d["value"] and d["e2e"]["h2d_bytes_per_step"] == 0


def test_reference_arm_under_a_launcher_uses_all_cores_and_only_rank_0_prints():
    # torchrun exports OMP_NUM_THREADS=1; the CPU arm must not fall back to one thread because of it
    out = _line("--impl", "reference", "--workload", "cfg1", "--steps", "1", "--warmup", "0", "--gpus", "2",
                env={"OMP_NUM_THREADS": "1", "RANK": "0", "WORLD_SIZE": "2"})
    d = json.loads(out[0])
    assert d["cpu_baseline"]["cores"] == len(os.sched_getaffinity(0)) and d["n_gpus"] == 2
    out = _line("--impl", "reference", "--workload", "cfg1", "--steps", "1", "--warmup", "0", "--gpus", "2",
                env={"RANK": "1", "WORLD_SIZE": "2"})
    assert out == []

"""The benchmark's reference arm runs on CPU and prints the agreed JSON line."""
import json
import os
import subprocess
import sys

from tests.conftest import ROOT


def test_reference_arm_json_line():
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference",
                        "--rows", "200000", "--batch", "4096", "--steps", "3", "--warmup", "1"],
                       capture_output=True, text=True, timeout=300, cwd=ROOT)
    assert p.returncode == 0, p.stderr
    lines = [l for l in p.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["unit"] == "GB/s" and d["higher_is_better"] is True
    assert d["steps"] == 3 and d["warmup"] == 1 and d["value"] > 0
    assert d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["cores"] >= 1
    assert d["e2e"]["h2d_bytes_per_step"] == 0 and d["e2e"]["d2h_bytes_per_step"] == 0
    assert "workload" in d["config"]


def test_reference_arm_other_ranks_stay_silent():
    env = dict(os.environ, RANK="1", WORLD_SIZE="2", LOCAL_RANK="1")
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference",
                        "--rows", "100000", "--batch", "1024", "--steps", "1", "--warmup", "0"],
                       capture_output=True, text=True, timeout=120, cwd=ROOT, env=env)
    assert p.returncode == 0 and p.stdout.strip() == ""


def test_reference_gpu_arm_reports_unavailable_without_a_gpu():
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference-gpu",
                        "--rows", "20000", "--batch", "512", "--steps", "2", "--warmup", "1"],
                       capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    line = json.loads(p.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference-gpu" and "unavailable" in line


def test_reference_arm_ignores_the_launchers_thread_limit_and_times_every_ranks_batch():
    """torch.distributed.run exports OMP_NUM_THREADS=1; the CPU arm must still use every core
    it may run on, and with --gpus N time N batches per step (the whole job's keys)."""
    env = dict(os.environ, OMP_NUM_THREADS="1", RANK="0", WORLD_SIZE="4", LOCAL_RANK="0")
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference",
                        "--gpus", "4", "--rows", "200000", "--batch", "4096", "--steps", "2",
                        "--warmup", "1"],
                       capture_output=True, text=True, timeout=300, cwd=ROOT, env=env)
    assert p.returncode == 0, p.stderr
    d = json.loads([l for l in p.stdout.splitlines() if l.startswith("{")][0])
    cores = len(os.sched_getaffinity(0))
    assert d["cores"] == cores and d["cpu_baseline"]["cores"] == cores
    assert d["batches_per_step"] == 4 and d["n_gpus"] == 4
    # value counts all four batches of a step
    assert abs(d["value"] - 4 * 4096 * 512 / (d["ms_per_step"] * 1e-3) / 1e9) < 1e-6 * d["value"] + 1e-9
    one = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference",
                          "--rows", "200000", "--batch", "4096", "--steps", "2", "--warmup", "1",
                          "--cpu-threads", "2"], capture_output=True, text=True, timeout=300, cwd=ROOT)
    d1 = json.loads([l for l in one.stdout.splitlines() if l.startswith("{")][0])
    assert d1["cores"] == 2 and d1["batches_per_step"] == 1
    assert d1["config"] == {**d["config"]}

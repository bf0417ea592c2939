"""What bench.py promises without a GPU: more than one GPU is refused with one line and exit code 2,
the reference arm says why it is unavailable, and the plain CPU baseline runs."""
import json
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def run(*args):
    return subprocess.run([sys.executable, str(ROOT / "bench.py"), *args], cwd=ROOT, text=True, capture_output=True, timeout=600)


def test_more_than_one_gpu_is_refused_with_one_line():
    p = run("--gpus", "2", "--steps", "2", "--warmup", "1")
    assert p.returncode == 2
    assert len(p.stdout.strip().splitlines()) == 1 and "one GPU" in p.stdout


def test_reference_arm_says_why_it_is_unavailable():
    p = run("--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "1")
    assert p.returncode == 0
    rec = json.loads(p.stdout.strip().splitlines()[-1])
    assert rec["impl"] == "reference" and isinstance(rec["unavailable"], str) and "\n" not in rec["unavailable"]


def test_cpu_baseline_times_the_plain_implementation():
    p = run("--cpu-baseline")
    assert p.returncode == 0, p.stderr[-2000:]
    rec = json.loads(p.stdout.strip().splitlines()[-1])
    assert rec["impl"] == "plain-cpu" and set(rec["points"]) == {"tiny_A", "tiny_B"}
    assert all(v["prompt_tok_s"] > 0 and v["decode_tok_s"] > 0 for v in rec["points"].values())

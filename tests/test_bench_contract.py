"""The parts of bench.py's contract that need no GPU: more than one GPU is refused with one line
and exit code 2; the reference arm answers with one JSON line and exit code 0."""

from __future__ import annotations

import json
import subprocess
import sys
from pathlib import Path

BENCH = Path(__file__).resolve().parent.parent / "bench.py"


def run(*args: str) -> subprocess.CompletedProcess:
    return subprocess.run([sys.executable, str(BENCH), *args], capture_output=True, text=True, timeout=120)


def test_more_than_one_gpu_is_refused_in_one_line() -> None:
    for n in ("2", "4", "8"):
        p = run("--gpus", n, "--steps", "2", "--warmup", "1")
        assert p.returncode == 2
        lines = [ln for ln in (p.stdout + p.stderr).splitlines() if ln.strip()]
        assert len(lines) == 1 and "one GPU" in lines[0]


def test_reference_arm_prints_one_json_line() -> None:
    p = run("--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "1")
    assert p.returncode == 0
    lines = [ln for ln in p.stdout.splitlines() if ln.strip()]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference"
    assert ("unavailable" in d and isinstance(d["unavailable"], str) and "\n" not in d["unavailable"]) or "value" in d

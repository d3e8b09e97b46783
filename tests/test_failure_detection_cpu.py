"""Failure detection with failures made on the host, as gloo ranks on the CPU: a rank that goes silent is named by the
others from the heartbeat store and they carry on without it; a collective one rank never joins ends with an error
after the group's time limit."""

import os
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


def run(mode: str, world: int, port: int) -> str:
    env = dict(os.environ, PYTHONPATH=f"{ROOT}:{os.environ.get('PYTHONPATH', '')}", OMP_NUM_THREADS="1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), str(ROOT / "tests" / "failure_worker_cpu.py"), mode]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=180)
    assert r.returncode == 0, (r.stdout + r.stderr)[-3000:]
    return r.stdout


def test_a_silent_rank_is_named_and_the_others_continue():
    out = run("silent_rank", 3, 29731)
    assert "[rank 0] LOST 2" in out and "[rank 1] LOST 2" in out
    assert "[rank 0] RECOVERED 3" in out and "[rank 1] RECOVERED 3" in out


def test_a_collective_nobody_joins_ends_with_an_error():
    out = run("absent_rank", 2, 29741)
    assert "[rank 0] TIMED_OUT" in out and "NO_ERROR" not in out and "[rank 1] RELEASED" in out

"""Tensor-parallel Pi0.5 plan on 2 / 4 / 8 GPUs against the single-rank eager model (child processes)."""

import os
import signal
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]


@pytest.mark.parametrize("shard_expert", [False, True])
@pytest.mark.parametrize("world", [2, 4, 8])
def test_tp_plan_matches_single_rank(world, shard_expert):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    # PHYAI_PI05_TP_SCATTER_ROWS: the test geometry has 80-160 prefix rows; groups of four and more take the
    # reduce-scatter / all-gather prefix with it
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PHYAI_PEER_GUARD="1", PYTHONPATH=f"{ROOT}:{os.environ.get('PYTHONPATH', '')}",
               PI05_TP_SHARD_EXPERT="1" if shard_expert else "0", PHYAI_PI05_TP_SCATTER_ROWS="64")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr",
           "127.0.0.1", "--master-port", str(29650 + world + (20 if shard_expert else 0)), str(ROOT / "tests" / "pi05_tp_worker.py")]
    proc = subprocess.Popen(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, start_new_session=True)
    try:
        out, err = proc.communicate(timeout=420)
    except subprocess.TimeoutExpired:
        os.killpg(proc.pid, signal.SIGKILL)
        out, err = proc.communicate()
        pytest.fail("tensor-parallel worker did not finish within 420 s: " + (out + err)[-3000:])
    assert proc.returncode == 0 and "PI05_TP_OK" in out, (out + err)[-4000:]

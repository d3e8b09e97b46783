"""Peer-memory collectives on real GPUs: bounded waits on one GPU, the fused kernels on two or more."""

import os
import signal
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]


def test_bounded_wait_reports_instead_of_hanging():
    from phyai_b200 import ops

    ops.kernel_status()
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    ops.ext().flag_wait_probe(flag, 1, 0.05)   # nothing ever sets the flag: the wait must give up
    torch.cuda.synchronize()
    assert ops.kernel_status() == 4            # kStatusTimeoutPeer
    flag.fill_(3)
    ops.ext().flag_wait_probe(flag, 1, 0.05)
    torch.cuda.synchronize()
    assert ops.kernel_status() == 0
    assert torch.ones(4, device="cuda").sum().item() == 4   # the context is still usable


@pytest.mark.parametrize("world", [2, 4, 8])
def test_peer_collectives(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PHYAI_PEER_GUARD="1", PYTHONPATH=f"{ROOT}:{os.environ.get('PYTHONPATH', '')}")
    port = 29600 + world
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr",
           "127.0.0.1", "--master-port", str(port), str(ROOT / "tests" / "peer_worker.py")]
    # own process group: if the ranks ever stall, the whole tree (launcher + workers) is ended, not just the launcher,
    # and the pipes close so that the failure is reported at once
    proc = subprocess.Popen(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, start_new_session=True)
    try:
        out, err = proc.communicate(timeout=420)
    except subprocess.TimeoutExpired:
        os.killpg(proc.pid, signal.SIGKILL)
        out, err = proc.communicate()
        pytest.fail("peer worker did not finish within 420 s: " + (out + err)[-3000:])
    tail = (out + err)[-4000:]
    assert proc.returncode == 0 and "PEER_OK" in out, tail

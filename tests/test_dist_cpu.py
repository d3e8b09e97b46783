"""Multi-process checks on CPU (gloo, two ranks): collectives, tensor-parallel Cosmos3, CFG-parallel guidance."""

import os
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


@pytest.mark.parametrize("mode,port", [("collectives", 29711), ("cosmos3_tp", 29712), ("cosmos3_cfg", 29713), ("pi05_tp", 29714), ("pi05_dp", 29715), ("pi0_dp", 29716), ("vae_tiles", 29717), ("seq_parallel", 29718), ("cosmos3_wn_engine", 29719),
                                       ("cosmos3_policy_wn_engine", 29720)])
def test_two_ranks(mode, port, world=2):
    env = dict(os.environ, PYTHONPATH=f"{ROOT}:{os.environ.get('PYTHONPATH', '')}", OMP_NUM_THREADS="2")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), str(ROOT / "tests" / "dist_worker_cpu.py"), mode]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "DIST_OK" in r.stdout, (r.stdout + r.stderr)[-4000:]


@pytest.mark.parametrize("mode,port", [("cosmos3_wn_engine", 29723), ("cosmos3_policy_wn_engine", 29724)])
def test_four_ranks_two_guidance_branches_of_two_tensor_parallel_ranks(mode, port):
    test_two_ranks(mode, port, world=4)


@pytest.mark.parametrize("mode,port", [("pi05_tp", 29725), ("cosmos3_tp", 29726), ("collectives", 29727), ("seq_parallel", 29728)])
def test_four_ranks(mode, port):
    """The tensor-parallel paths at four ranks: more ranks than KV heads (replicated heads), cameras that do not divide
    over the ranks, four-way collectives and token shards."""
    test_two_ranks(mode, port, world=4)

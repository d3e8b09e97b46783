"""CudaIpcBuffer across two processes on one GPU: the creator fills the buffer, a child maps the handle, checks the
contents and writes an answer the creator reads back. No kernel waits on another process: the hand-over is the child's exit."""

import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]

CHILD = r"""
import sys, torch
sys.path.insert(0, sys.argv[1])
from phyai_b200.runtime.ipc_buffer import CudaIpcBuffer, CudaIpcHandle
torch.cuda.set_device(0)
buf = CudaIpcBuffer.attach(CudaIpcHandle.from_json(sys.argv[2]))
assert not buf.is_creator
t = buf.tensor((1024,), torch.float32)
assert torch.equal(t[:512].cpu(), torch.arange(512, dtype=torch.float32)), "creator's data not visible"
t[512:] = t[:512] * 2
torch.cuda.synchronize()
buf.close()
print("CHILD_OK")
"""


def test_cuda_ipc_buffer_is_shared_between_processes():
    from phyai_b200.runtime.ipc_buffer import CudaIpcBuffer

    with CudaIpcBuffer.create(4096, 0) as buf:
        assert buf.is_creator and buf.nbytes == 4096
        t = buf.tensor((1024,), torch.float32)
        t.zero_()
        t[:512] = torch.arange(512, dtype=torch.float32, device="cuda")
        torch.cuda.synchronize()
        r = subprocess.run([sys.executable, "-c", CHILD, str(ROOT), buf.handle.to_json()], capture_output=True, text=True, timeout=300)
        assert r.returncode == 0 and "CHILD_OK" in r.stdout, (r.stdout + r.stderr)[-2000:]
        torch.cuda.synchronize()
        assert torch.equal(t[512:].cpu(), torch.arange(512, dtype=torch.float32) * 2)
        with pytest.raises(ValueError):
            buf.tensor((2048,), torch.float32)

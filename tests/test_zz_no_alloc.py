"""The allocation-free C entry point (csrc/noalloc.h), called through its exported symbol with raw device pointers."""

import ctypes
import importlib

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    mod = importlib.import_module("phyai_b200._C")
    lib = ctypes.CDLL(mod.__file__)
    fn = lib.pb_noalloc_add_rmsnorm
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_float, ctypes.c_void_p]
    return fn


@pytest.mark.parametrize("rows,cols", [(50, 1024), (968, 2048), (7, 5120), (3, 8)])
def test_matches_the_torch_facing_op_twice_in_a_row(rows, cols):
    from phyai_b200 import ops

    fn = _lib()
    g = torch.Generator(device="cuda").manual_seed(rows * 131 + cols)
    x = torch.randn(rows, cols, device="cuda", generator=g).bfloat16()
    w = (torch.randn(cols, device="cuda", generator=g) * 0.2 + 1.0).bfloat16()
    stream = torch.cuda.current_stream().cuda_stream
    for call in range(2):       # the second call reuses the scratch the first one dirtied
        r = torch.randn(rows, cols, device="cuda", generator=g).bfloat16()
        r_new, r_old = r.clone(), r.clone()
        y_new = torch.empty_like(x)
        before = torch.cuda.memory_allocated()
        rc = fn(x.data_ptr(), r_new.data_ptr(), w.data_ptr(), y_new.data_ptr(), rows, cols, 1e-6, stream)
        assert rc == 0 and torch.cuda.memory_allocated() == before
        y_old = ops.norm(x, "rms", weight=w, residual=r_old, eps=1e-6)
        torch.cuda.synchronize()
        assert torch.equal(r_new, r_old), call                                  # the bf16 residual sum is exact either way
        scale = y_old.float().abs().max().item()
        assert (y_new.float() - y_old.float()).abs().max().item() <= 1e-2 * scale, call
    assert ops.kernel_status() == 0


def test_rejects_what_it_cannot_do():
    fn = _lib()
    t = torch.zeros(16, 64, device="cuda", dtype=torch.bfloat16)
    w = torch.ones(64, device="cuda", dtype=torch.bfloat16)
    assert fn(t.data_ptr(), t.data_ptr(), w.data_ptr(), t.data_ptr(), 16385, 64, 1e-6, None) == 1      # more rows than the scratch holds
    assert fn(t.data_ptr(), t.data_ptr(), w.data_ptr(), t.data_ptr(), 16, 60, 1e-6, None) == 1          # cols not a multiple of 8
    assert fn(t.data_ptr() + 2, t.data_ptr(), w.data_ptr(), t.data_ptr(), 8, 64, 1e-6, None) == 1        # misaligned
    torch.cuda.synchronize()
    assert torch.ones(4, device="cuda").sum().item() == 4

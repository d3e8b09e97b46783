"""The ctypes NCCL binding against a stand-in library (host pointers, one rank): signatures, error path, version."""

import subprocess
import textwrap

import pytest
import torch

FAKE = textwrap.dedent(r"""
    #include <cstring>
    #include <cstddef>
    extern "C" {
    typedef struct { char internal[128]; } ncclUniqueId;
    static const int esz[] = {1, 1, 4, 4, 8, 8, 2, 4, 8, 2};
    static int calls = 0;
    const char* ncclGetErrorString(int r) { return r == 0 ? "no error" : "fake failure"; }
    int ncclGetVersion(int* v) { *v = 22809; return 0; }
    int ncclGetUniqueId(ncclUniqueId* id) { std::memset(id->internal, 7, 128); return 0; }
    int ncclCommInitRank(void** comm, int n, ncclUniqueId id, int rank) { if (id.internal[5] != 7 || rank >= n) return 5; *comm = (void*)0x1234; return 0; }
    int ncclAllReduce(const void* s, void* r, size_t c, int dt, int op, void* comm, void* st) { if (comm != (void*)0x1234) return 4; ++calls; std::memmove(r, s, c * esz[dt]); return 0; }
    int ncclAllGather(const void* s, void* r, size_t c, int dt, void* comm, void* st) { ++calls; std::memmove(r, s, c * esz[dt]); return 0; }
    int ncclReduceScatter(const void* s, void* r, size_t c, int dt, int op, void* comm, void* st) { ++calls; std::memmove(r, s, c * esz[dt]); return 0; }
    int ncclBroadcast(const void* s, void* r, size_t c, int dt, int root, void* comm, void* st) { ++calls; std::memmove(r, s, c * esz[dt]); return 0; }
    int ncclSend(const void* s, size_t c, int dt, int peer, void* comm, void* st) { return peer == 99 ? 3 : 0; }
    int ncclRecv(void* r, size_t c, int dt, int peer, void* comm, void* st) { return 0; }
    int ncclGroupStart() { return 0; }
    int ncclGroupEnd() { return 0; }
    int ncclCommDestroy(void* comm) { return 0; }
    int fake_calls() { return calls; }
    }
""")


@pytest.fixture(scope="module")
def fake_lib(tmp_path_factory):
    d = tmp_path_factory.mktemp("fakenccl")
    (d / "fake.cpp").write_text(FAKE)
    so = d / "libfakenccl.so"
    subprocess.run(["g++", "-shared", "-fPIC", "-O1", str(d / "fake.cpp"), "-o", str(so)], check=True)
    return str(so)


def test_binding_calls_and_errors(fake_lib):
    from phyai_b200.parallel.backends.nccl_binding import NcclError, NcclLibrary

    lib = NcclLibrary(fake_lib)
    assert lib.version() == (2, 28, 9)
    uid = lib.unique_id()
    assert bytes(uid.internal) == b"\x07" * 128
    comm = lib.comm_init_rank(1, uid, 0)
    with pytest.raises(NcclError, match="fake failure"):
        lib.comm_init_rank(1, uid, 3)
    x = torch.arange(6, dtype=torch.bfloat16)
    y = torch.zeros_like(x)
    lib.all_reduce(x.data_ptr(), y.data_ptr(), x.numel(), x.dtype, "sum", comm, 0)
    assert torch.equal(x, y)
    z = torch.zeros(6, dtype=torch.float32)
    src = torch.arange(6.0)
    lib.all_gather(src.data_ptr(), z.data_ptr(), 6, torch.float32, comm, 0)
    assert z.tolist() == [0, 1, 2, 3, 4, 5]
    lib.group_start()
    lib.send(x.data_ptr(), 6, x.dtype, 0, comm, 0)
    lib.recv(y.data_ptr(), 6, y.dtype, 0, comm, 0)
    lib.group_end()
    with pytest.raises(NcclError):
        lib.send(x.data_ptr(), 6, x.dtype, 99, comm, 0)
    assert lib.lib.fake_calls() == 2
    lib.comm_destroy(comm)
    with pytest.raises(NcclError):
        NcclLibrary("/nonexistent/libnccl.so")


def test_library_discovery_prefers_override(monkeypatch, fake_lib):
    from phyai_b200.parallel.backends import nccl_binding as nb

    monkeypatch.setenv("PHYAI_NCCL_SO_PATH", fake_lib)
    assert nb.find_library() == fake_lib
    monkeypatch.delenv("PHYAI_NCCL_SO_PATH")
    assert "nccl" in nb.find_library()

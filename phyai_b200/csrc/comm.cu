// Symmetric (IPC-shared) device buffers for the peer-memory kernels.
//
// Each rank cudaMalloc's one slab and exports it with cudaIpcGetMemHandle; the
// handles travel over the host process group and every peer maps them with
// cudaIpcOpenMemHandle. The reference's only peer-memory primitive is the unused
// CudaIpcBuffer (phyai/src/phyai/runtime/ipc_buffer.py:252-556); here the same idea
// is the substrate of the fused compute + collective kernels.
#include "comm.cuh"

#include <pybind11/pybind11.h>

#include <string>

#include "gemm.cuh"
#include "ptx.cuh"

namespace py = pybind11;

namespace {

void throw_on(cudaError_t e, const char* what) {
  if (e != cudaSuccess) {
    cudaGetLastError();
    throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
  }
}

// Returns (device pointer as int, 64-byte IPC handle).
py::tuple ipc_alloc(size_t bytes) {
  void* p = nullptr;
  throw_on(cudaMalloc(&p, bytes), "cudaMalloc");
  throw_on(cudaMemset(p, 0, bytes), "cudaMemset");
  cudaIpcMemHandle_t h;
  throw_on(cudaIpcGetMemHandle(&h, p), "cudaIpcGetMemHandle");
  return py::make_tuple(reinterpret_cast<uintptr_t>(p),
                        py::bytes(reinterpret_cast<const char*>(&h), sizeof(h)));
}
uintptr_t ipc_open(const py::bytes& handle) {
  std::string s = handle;
  if (s.size() != sizeof(cudaIpcMemHandle_t)) throw std::runtime_error("bad IPC handle size");
  cudaIpcMemHandle_t h;
  memcpy(&h, s.data(), sizeof(h));
  void* p = nullptr;
  throw_on(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle");
  return reinterpret_cast<uintptr_t>(p);
}
void ipc_close(uintptr_t p) {
  throw_on(cudaIpcCloseMemHandle(reinterpret_cast<void*>(p)), "cudaIpcCloseMemHandle");
}
void ipc_free(uintptr_t p) { throw_on(cudaFree(reinterpret_cast<void*>(p)), "cudaFree"); }

}  // namespace

void register_comm(py::module_& m) {
  m.def("ipc_alloc", &ipc_alloc);
  m.def("ipc_open", &ipc_open);
  m.def("ipc_close", &ipc_close);
  m.def("ipc_free", &ipc_free);
}

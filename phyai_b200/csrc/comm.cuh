// Peer-memory communication layer (comm.cu): IPC-shared symmetric buffers and the
// kernels that move data between GPUs with plain peer loads / stores.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace pb {

constexpr int kMaxRanks = 8;

// Pointers of one symmetric allocation as seen from this process: entry r is rank
// r's copy (entry `rank` is the local one).
struct PeerPtrs {
  void* p[kMaxRanks];
};

}  // namespace pb

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

// Where a GEMM epilogue in push mode sends its tiles: slots[parity][rank] of every
// rank's symmetric slab, then one arrival per CTA on every rank's channel counter.
// world == 0 means "not pushing" (the kernel stores to its ordinary output).
// rows_per_rank > 0 turns the broadcast into a scatter: row m goes only to rank
// m / rows_per_rank (the reduce-scatter half of a two-step all-reduce).
// wait_channel >= 0 makes the kernel wait, before it loads its activations, until that
// channel has seen wait_expect arrivals (the activations were written by peers), and
// close the channel's call when its last CTA is done.
struct PushParams {
  PeerPtrs data;            // slab base of every rank (bf16 elements are addressed from here)
  PeerPtrs sig;             // channel signal array of every rank
  const void* local_sig;    // this rank's channel signal array (parity is read from it)
  long long slots_off;      // element offset of the slot area inside the slab
  long long slot_stride;    // elements between consecutive source ranks' slots
  int ld;                   // row stride of a slot, elements
  int world, rank, channel;
  int rows_per_rank;
  int wait_channel;
  unsigned int wait_expect;
};

}  // namespace pb

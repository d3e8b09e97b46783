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

// What the consumer of a pushed product does with it: h = residual + (sum of the ranks' slots + bias) * gate,
// y = norm(h). Used by the stand-alone reduce kernel and by the tail of a push-mode GEMM (see PushParams::tail).
struct ReduceNormArgs {
  const __nv_bfloat16* slots;   // local: [world][M][ld] partials of this call's parity
  long long slot_stride;        // elements between consecutive ranks' slots
  int world, M, N, ld;
  __nv_bfloat16* residual;      // [M, ldr] in/out: h = residual + sum * gate; may be null
  int ldr;
  const __nv_bfloat16* col_gate;  // [N] or null
  const __nv_bfloat16* bias;      // [N] or null (added once)
  __nv_bfloat16* h_out;         // where h goes when residual is null (may be null)
  int ldh;
  __nv_bfloat16* y;             // [M, ldy] normalised output (null: no norm)
  int ldy;
  int norm_mode;                // NormMode from ops.cuh; -1 = none
  const __nv_bfloat16* weight;  // rms / gemma weight
  const __nv_bfloat16* mod;     // AdaRMS row (scale | shift | gate), shared by all rows
  float eps;
  int row0, nrows;              // rows this rank reduces ([0, M) unless the producer scattered)
  int slot_row0;                // global row stored at slot row 0 (row0 when scattered, else 0)
  // all-gather of the normalised rows: y_world > 0 stores each y row at element offset
  // y_off + row * ldy of EVERY rank's slab instead of `y`, then signals y_channel
  PeerPtrs y_dst;
  long long y_off;
  int y_world, y_channel;
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
  // tail != 0 (push mode on few rows, every CTA of the grid resident at once): after its arrival each CTA
  // waits for tail_expect arrivals on the channel and reduces its share of the rows (`red`), so the product,
  // the all-reduce, the residual and the norm are one launch and one peer round trip
  int tail;
  unsigned int tail_expect;
  ReduceNormArgs red;
};

}  // namespace pb

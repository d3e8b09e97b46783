// A C entry point that performs no allocation of any kind (device or host).
//
// This function has no counterpart in the reference project. It exists for callers that cannot
// tolerate an allocation on the launch path: code running inside CUDA stream capture (where
// cudaMalloc is illegal), a real-time control loop that must not take the allocator's lock, or a
// host language binding (C, Rust, a robot middleware node) that owns all buffers itself and only
// wants to hand over raw device pointers. Everything else in this library is reached through
// PyTorch, whose ops may allocate workspaces and outputs.
//
//   h = x + residual            (rounded to bf16, written back into `residual`)
//   y = h * rsqrt(mean(h^2) + eps) * weight
//
// i.e. the residual-add + RMSNorm that sits between every pair of linear layers, computed in two
// launches with each row spread over several thread blocks: phase 1 adds and accumulates the row
// sums of squares with fp32 atomics, phase 2 normalises. The sums travel through a scratch array
// that lives in the library image itself (a file-scope `static __device__` array), not in memory
// obtained at run time.
//
// Limits: rows <= PB_NOALLOC_MAX_ROWS (the scratch holds one float per row), cols a multiple of 8
// and <= 65536, all pointers 16-byte aligned device pointers to contiguous bf16 ([rows, cols] for
// x, residual, y; [cols] for weight). A call outside these limits launches nothing and returns
// PB_NOALLOC_BAD_SHAPE with a message on stderr.
//
// The first call on a device looks up the scratch array's address (cudaGetSymbolAddress) and
// caches it in a fixed table; make that first call before starting a stream capture. The scratch
// is cleared on `stream` at the start of every call (cudaMemsetAsync of rows * 4 bytes), so calls
// on one stream may follow each other freely; two calls that overlap in time on DIFFERENT streams
// of the same device share the scratch and race: serialise them.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define PB_NOALLOC_MAX_ROWS 16384
#define PB_NOALLOC_OK 0
#define PB_NOALLOC_BAD_SHAPE 1   /* rows / cols / alignment outside the documented limits */
#define PB_NOALLOC_SETUP_FAILED 2 /* the scratch symbol could not be resolved on this device */
#define PB_NOALLOC_LAUNCH_FAILED 3

// `stream` is a cudaStream_t passed as an opaque pointer (0 = the default stream).
int pb_noalloc_add_rmsnorm(const void* x, void* residual, const void* weight, void* y, int rows, int cols, float eps,
                           void* stream);

#ifdef __cplusplus
}
#endif

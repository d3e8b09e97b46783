// Residual-add + RMSNorm through a C ABI that allocates nothing (see noalloc.h for the contract).
//
// The row statistics cross from the first kernel to the second through global memory, the same
// scheme the GEMM epilogue uses for its fused-norm path (sum of squares accumulated with fp32
// atomics, consumer normalises); here the accumulators are a static array inside this image.
#include "noalloc.h"

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

namespace {

static __device__ __align__(256) float g_row_sumsq[PB_NOALLOC_MAX_ROWS];

constexpr int kMaxDevices = 64;
float* g_scratch_ptr[kMaxDevices] = {nullptr};   // fixed table: no container, no heap

constexpr int kThreads = 256;
constexpr int kColsPerBlock = kThreads * 8;      // one 16-byte vector per thread

// h = x + r (bf16), written back to r; partial sum of squares of the rounded values -> sumsq[row]
__global__ void add_sumsq_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ r, float* __restrict__ sumsq,
                                 int cols) {
  __shared__ float red[kThreads / 32];
  const int row = blockIdx.x, c = (blockIdx.y * kThreads + threadIdx.x) * 8;
  float ss = 0.f;
  if (c < cols) {
    const size_t off = size_t(row) * cols + c;
    const uint4 a = *reinterpret_cast<const uint4*>(x + off);
    const uint4 b = *reinterpret_cast<const uint4*>(r + off);
    const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&a);
    const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&b);
    uint4 o;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      o2[i] = __floats2bfloat162_rn(__bfloat162float(a2[i].x) + __bfloat162float(b2[i].x),
                                    __bfloat162float(a2[i].y) + __bfloat162float(b2[i].y));
      const float h0 = __bfloat162float(o2[i].x), h1 = __bfloat162float(o2[i].y);
      ss += h0 * h0 + h1 * h1;
    }
    *reinterpret_cast<uint4*>(r + off) = o;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < kThreads / 32 ? red[threadIdx.x] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (threadIdx.x == 0) atomicAdd(sumsq + row, t);
  }
}

__global__ void apply_norm_kernel(const __nv_bfloat16* __restrict__ h, const __nv_bfloat16* __restrict__ w,
                                  const float* __restrict__ sumsq, __nv_bfloat16* __restrict__ y, int cols, float eps) {
  const int row = blockIdx.x, c = (blockIdx.y * kThreads + threadIdx.x) * 8;
  if (c >= cols) return;
  const float rstd = rsqrtf(sumsq[row] / float(cols) + eps);
  const size_t off = size_t(row) * cols + c;
  const uint4 a = *reinterpret_cast<const uint4*>(h + off);
  const uint4 g = *reinterpret_cast<const uint4*>(w + c);
  const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&a);
  const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&g);
  uint4 o;
  __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
  for (int i = 0; i < 4; ++i)
    o2[i] = __floats2bfloat162_rn(__bfloat162float(a2[i].x) * rstd * __bfloat162float(g2[i].x),
                                  __bfloat162float(a2[i].y) * rstd * __bfloat162float(g2[i].y));
  *reinterpret_cast<uint4*>(y + off) = o;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace

extern "C" __attribute__((visibility("default")))
int pb_noalloc_add_rmsnorm(const void* x, void* residual, const void* weight, void* y, int rows, int cols, float eps,
                           void* stream) {
  if (rows <= 0 || rows > PB_NOALLOC_MAX_ROWS || cols <= 0 || cols % 8 || cols > 65536 || !x || !residual || !weight || !y ||
      !aligned16(x) || !aligned16(residual) || !aligned16(weight) || !aligned16(y)) {
    fprintf(stderr, "pb_noalloc_add_rmsnorm: unsupported call (rows=%d, limit %d; cols=%d, multiple of 8 up to 65536; "
                    "pointers must be non-null and 16-byte aligned)\n", rows, PB_NOALLOC_MAX_ROWS, cols);
    return PB_NOALLOC_BAD_SHAPE;
  }
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return PB_NOALLOC_SETUP_FAILED;
  if (g_scratch_ptr[dev] == nullptr) {
    // once per device; do this before stream capture begins
    float* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_row_sumsq);
    if (e != cudaSuccess || p == nullptr) {
      fprintf(stderr, "pb_noalloc_add_rmsnorm: cudaGetSymbolAddress failed: %s\n", cudaGetErrorString(e));
      cudaGetLastError();
      return PB_NOALLOC_SETUP_FAILED;
    }
    g_scratch_ptr[dev] = p;
  }
  float* sumsq = g_scratch_ptr[dev];
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // the accumulators must start at zero for this call's rows
  if (cudaMemsetAsync(sumsq, 0, size_t(rows) * sizeof(float), st) != cudaSuccess) { cudaGetLastError(); return PB_NOALLOC_LAUNCH_FAILED; }
  const dim3 grid(rows, (cols + kColsPerBlock - 1) / kColsPerBlock);
  add_sumsq_kernel<<<grid, kThreads, 0, st>>>(static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(residual), sumsq, cols);
  apply_norm_kernel<<<grid, kThreads, 0, st>>>(static_cast<const __nv_bfloat16*>(residual), static_cast<const __nv_bfloat16*>(weight),
                                               sumsq, static_cast<__nv_bfloat16*>(y), cols, eps);
  if (cudaGetLastError() != cudaSuccess) return PB_NOALLOC_LAUNCH_FAILED;
  return PB_NOALLOC_OK;
}

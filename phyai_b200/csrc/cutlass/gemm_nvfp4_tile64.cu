// NVFP4 block-scaled GEMM, 128 x 64 x 256 tiles, one CTA per tile, no cluster (every TMA load is a plain per-CTA load).
#include "gemm_nvfp4_tile.cuh"

namespace nvfp4 {
int run_tile64(const void* A, const void* SFA, const void* B, const void* SFB, void* D, int M, int N, int K, float alpha,
                void* workspace, size_t workspace_bytes, cudaStream_t stream) {
  return run_gemm<GemmOf<Shape<_128, _64, _256>, Shape<_1, _1, _1>>>(A, SFA, B, SFB, D, M, N, K, alpha, workspace, workspace_bytes, stream);
}
}  // namespace nvfp4

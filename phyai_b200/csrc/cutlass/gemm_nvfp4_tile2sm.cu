// NVFP4 block-scaled GEMM, 256 x 256 x 256 tiles on CTA pairs (cta_group::2): two SMs share one accumulator tile and
// each loads half of the B operand. Operands are this GPU's own memory (single-GPU linears only).
#include "gemm_nvfp4_tile.cuh"

namespace nvfp4 {
int run_tile2sm(const void* A, const void* SFA, const void* B, const void* SFB, void* D, int M, int N, int K, float alpha,
                void* workspace, size_t workspace_bytes, cudaStream_t stream) {
  return run_gemm<GemmOf<Shape<_256, _256, _256>, Shape<_2, _1, _1>>>(A, SFA, B, SFB, D, M, N, K, alpha, workspace, workspace_bytes, stream);
}
}  // namespace nvfp4

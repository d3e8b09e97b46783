// Block-scaled fp8 GEMM (e4m3, 1 x 128 / 128 x 128 fp32 scales): 256 x 128 tiles on CTA pairs. Operands are this GPU's own memory.
#include "gemm_fp8_blockwise_tile.cuh"

namespace fp8bw {
int run_2sm128(const void* A, const float* SFA, const void* B, const float* SFB, const void* C, void* D, int M, int N, int K,
              void* workspace, size_t workspace_bytes, cudaStream_t stream) {
  return run_gemm<GemmOf<Shape<_256,_128,_128>, Shape<_2,_1,_1>, cutlass::gemm::KernelTmaWarpSpecializedBlockwise2SmSm100>>(A, SFA, B, SFB, C, D, M, N, K, workspace, workspace_bytes, stream);
}
}  // namespace fp8bw

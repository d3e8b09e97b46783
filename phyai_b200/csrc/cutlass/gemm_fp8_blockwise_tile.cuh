// CUTLASS sm100 collective for e4m3 operands with software block scales (fp32, one per 1 x 128 block of the activation
// and per 128 x 128 block of the weight, both K-major: the layouts block-fp8 checkpoints and this package's quantiser
// produce), parametrised by tile, cluster and schedule; each instance compiles in its own translation unit.
#pragma once
#include <cuda_runtime.h>

#include "cute/tensor.hpp"
#include "cutlass/cutlass.h"
#include "cutlass/detail/blockwise_scale_layout.hpp"
#include "cutlass/epilogue/collective/collective_builder.hpp"
#include "cutlass/epilogue/thread/linear_combination.h"
#include "cutlass/gemm/collective/collective_builder.hpp"
#include "cutlass/gemm/device/gemm_universal_adapter.h"
#include "cutlass/gemm/dispatch_policy.hpp"
#include "cutlass/gemm/kernel/gemm_universal.hpp"
#include "cutlass/util/packed_stride.hpp"

namespace fp8bw {

using namespace cute;

using Element8 = cutlass::float_e4m3_t;
using ElementD = cutlass::bfloat16_t;
using Acc = float;
using ScaleConfig = cutlass::detail::Sm100BlockwiseScaleConfig<1, 128, 128, UMMA::Major::K, UMMA::Major::K>;
using LayoutSFA = decltype(ScaleConfig::deduce_layoutSFA());
using LayoutSFB = decltype(ScaleConfig::deduce_layoutSFB());

template <class Tile, class Cluster, class Schedule>
struct GemmOf {
  using Epilogue = typename cutlass::epilogue::collective::CollectiveBuilder<
      cutlass::arch::Sm100, cutlass::arch::OpClassTensorOp, Tile, Cluster, cutlass::epilogue::collective::EpilogueTileAuto, Acc, Acc,
      ElementD, cutlass::layout::RowMajor, 8, ElementD, cutlass::layout::RowMajor, 8,
      cutlass::epilogue::collective::EpilogueScheduleAuto>::CollectiveOp;
  using Mainloop = typename cutlass::gemm::collective::CollectiveBuilder<
      cutlass::arch::Sm100, cutlass::arch::OpClassTensorOp, Element8, cute::tuple<cutlass::layout::RowMajor, LayoutSFA>, 16, Element8,
      cute::tuple<cutlass::layout::ColumnMajor, LayoutSFB>, 16, Acc, Tile, Cluster,
      cutlass::gemm::collective::StageCountAutoCarveout<static_cast<int>(sizeof(typename Epilogue::SharedStorage))>, Schedule>::CollectiveOp;
  using Kernel = cutlass::gemm::kernel::GemmUniversal<Shape<int, int, int, int>, Mainloop, Epilogue, void>;
  using Gemm = cutlass::gemm::device::GemmUniversalAdapter<Kernel>;
};

// D = A . SFA @ (B . SFB)^T [+ C]; C (bf16 [M, N], may alias D) is added when given.
template <class G>
int run_gemm(const void* A, const float* SFA, const void* B, const float* SFB, const void* C, void* D, int M, int N, int K,
             void* workspace, size_t workspace_bytes, cudaStream_t stream) {
  using Gemm = typename G::Gemm;
  auto sA = cutlass::make_cute_packed_stride(typename Gemm::GemmKernel::StrideA{}, make_shape(M, K, 1));
  auto sB = cutlass::make_cute_packed_stride(typename Gemm::GemmKernel::StrideB{}, make_shape(N, K, 1));
  auto sC = cutlass::make_cute_packed_stride(typename Gemm::GemmKernel::StrideC{}, make_shape(M, N, 1));
  auto sD = cutlass::make_cute_packed_stride(typename Gemm::GemmKernel::StrideD{}, make_shape(M, N, 1));
  auto lA = ScaleConfig::tile_atom_to_shape_SFA(make_shape(M, N, K, 1));
  auto lB = ScaleConfig::tile_atom_to_shape_SFB(make_shape(M, N, K, 1));
  typename Gemm::Arguments args{cutlass::gemm::GemmUniversalMode::kGemm,
                                {M, N, K, 1},
                                {reinterpret_cast<const Element8*>(A), sA, reinterpret_cast<const Element8*>(B), sB, SFA, lA, SFB, lB},
                                {{1.f, C ? 1.f : 0.f}, reinterpret_cast<const ElementD*>(C), sC, reinterpret_cast<ElementD*>(D), sD}};
  Gemm gemm;
  if (gemm.can_implement(args) != cutlass::Status::kSuccess) return 1;
  if (Gemm::get_workspace_size(args) > workspace_bytes) return 2;
  if (gemm.initialize(args, workspace, stream) != cutlass::Status::kSuccess) return 3;
  if (gemm.run(stream) != cutlass::Status::kSuccess) return 4;
  return 0;
}

}  // namespace fp8bw

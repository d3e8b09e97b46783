// CUTLASS sm100 block-scaled collective for NVFP4 operands, parametrised by the tile shape; each tile shape is
// instantiated in its own translation unit (gemm_nvfp4_tile*.cu) so that they compile side by side.
#pragma once
#include <cuda_runtime.h>

#include "cute/tensor.hpp"
#include "cutlass/cutlass.h"
#include "cutlass/detail/sm100_blockscaled_layout.hpp"
#include "cutlass/epilogue/collective/collective_builder.hpp"
#include "cutlass/epilogue/thread/linear_combination.h"
#include "cutlass/gemm/collective/collective_builder.hpp"
#include "cutlass/gemm/device/gemm_universal_adapter.h"
#include "cutlass/gemm/dispatch_policy.hpp"
#include "cutlass/gemm/kernel/gemm_universal.hpp"
#include "cutlass/util/packed_stride.hpp"

namespace nvfp4 {

using namespace cute;

using ElementAB = cutlass::nv_float4_t<cutlass::float_e2m1_t>;
using ElementD = cutlass::bfloat16_t;
using Acc = float;
constexpr int kAlignAB = 32;                                        // elements: 16 bytes of packed e2m1
constexpr int kAlignD = 128 / cutlass::sizeof_bits<ElementD>::value;

template <class TileShape, class Cluster>
struct GemmOf {
  using Epilogue = typename cutlass::epilogue::collective::CollectiveBuilder<
      cutlass::arch::Sm100, cutlass::arch::OpClassBlockScaledTensorOp, TileShape, Cluster,
      cutlass::epilogue::collective::EpilogueTileAuto, Acc, Acc, ElementD, cutlass::layout::RowMajor, kAlignD, ElementD,
      cutlass::layout::RowMajor, kAlignD, cutlass::epilogue::collective::EpilogueScheduleAuto>::CollectiveOp;
  using Mainloop = typename cutlass::gemm::collective::CollectiveBuilder<
      cutlass::arch::Sm100, cutlass::arch::OpClassBlockScaledTensorOp, ElementAB, cutlass::layout::RowMajor, kAlignAB, ElementAB,
      cutlass::layout::ColumnMajor, kAlignAB, Acc, TileShape, Cluster,
      cutlass::gemm::collective::StageCountAutoCarveout<static_cast<int>(sizeof(typename Epilogue::SharedStorage))>,
      cutlass::gemm::collective::KernelScheduleAuto>::CollectiveOp;
  using Kernel = cutlass::gemm::kernel::GemmUniversal<Shape<int, int, int, int>, Mainloop, Epilogue, void>;
  using Gemm = cutlass::gemm::device::GemmUniversalAdapter<Kernel>;
};

template <class G>
int run_gemm(const void* A, const void* SFA, const void* B, const void* SFB, void* D, int M, int N, int K, float alpha,
             void* workspace, size_t workspace_bytes, cudaStream_t stream) {
  using Gemm = typename G::Gemm;
  using Cfg = typename Gemm::GemmKernel::CollectiveMainloop::Sm1xxBlkScaledConfig;
  using StrideA = typename Gemm::GemmKernel::StrideA;
  using StrideB = typename Gemm::GemmKernel::StrideB;
  using StrideC = typename Gemm::GemmKernel::StrideC;
  using StrideD = typename Gemm::GemmKernel::StrideD;
  auto sA = cutlass::make_cute_packed_stride(StrideA{}, make_shape(M, K, 1));
  auto sB = cutlass::make_cute_packed_stride(StrideB{}, make_shape(N, K, 1));
  auto sC = cutlass::make_cute_packed_stride(StrideC{}, make_shape(M, N, 1));
  auto sD = cutlass::make_cute_packed_stride(StrideD{}, make_shape(M, N, 1));
  auto lA = Cfg::tile_atom_to_shape_SFA(make_shape(M, N, K, 1));
  auto lB = Cfg::tile_atom_to_shape_SFB(make_shape(M, N, K, 1));
  typename Gemm::Arguments args{
      cutlass::gemm::GemmUniversalMode::kGemm,
      {M, N, K, 1},
      {reinterpret_cast<const typename ElementAB::DataType*>(A), sA, reinterpret_cast<const typename ElementAB::DataType*>(B), sB,
       reinterpret_cast<const typename ElementAB::ScaleFactorType*>(SFA), lA,
       reinterpret_cast<const typename ElementAB::ScaleFactorType*>(SFB), lB},
      {{alpha, 0.f}, nullptr, sC, reinterpret_cast<ElementD*>(D), sD}};
  Gemm gemm;
  if (gemm.can_implement(args) != cutlass::Status::kSuccess) return 1;
  if (Gemm::get_workspace_size(args) > workspace_bytes) return 2;
  if (gemm.initialize(args, workspace, stream) != cutlass::Status::kSuccess) return 3;
  if (gemm.run(stream) != cutlass::Status::kSuccess) return 4;
  return 0;
}

}  // namespace nvfp4

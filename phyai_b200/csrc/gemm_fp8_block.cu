// Block-scaled fp8 GEMM for sm_100a: e4m3 operands with fp32 scales per 1x128 activation block
// and per 128x128 weight block (the layout of block-quantised checkpoints).
//
// The tensor core cannot apply these scales itself, so every 128-deep K block is multiplied into
// a FRESH tensor-memory accumulator (tcgen05.mma kind::f8f6f4, four K = 32 instructions) and four
// "promotion" warps fold it into fp32 registers with the block's scale:
//
//     acc[i][c] += a_scale[row][kb] * w_scale[nblock][kb] * partial_kb[i][c]
//
// Two accumulator buffers in tensor memory let the MMAs of block kb + 1 run while block kb is
// promoted. For skinny problems the operands are swapped (weights fill the 128-row operand, the
// activation rows become the MMA N), which moves the per-row activation scale from "one per
// thread" to "one per column": those BN x KB factors are staged in shared memory once.
// Roles: warp 0 TMA producer, warp 1 MMA issuer, then PW promotion warps (4, or 8 for the 256-wide tile
// of large problems: two warps per tensor-memory lane quadrant, each folding half of the columns, so the
// promotion of a block (128 columns per thread) takes less time than its MMAs); afterwards all threads run
// the shared epilogue (bias / activation / gated activation / gate / residual).
//
// Capability parity: phyai/src/phyai/layers/linear/backends/flashinfer.py:132-172
// (gemm_fp8_nt_groupwise) and the dequantise + matmul fallback in backends/torch.py:139-176.
#include <cstring>

#include "gemm.cuh"
#include "gemm_epilogue.cuh"
#include "launch.cuh"
#include "ptx.cuh"

namespace pb {

namespace {
constexpr int kBStagesMax = 6;
constexpr int kP = 128;         // rows of the 128-row operand
constexpr int kRowB = 128;      // bytes of one operand row per K block (128 e4m3)
}  // namespace

template <int BN, bool SWAP, int PW>
__global__ void __launch_bounds__(64 + 32 * PW)
gemm_fp8_block_kernel(const __grid_constant__ CUtensorMap tmP, const __grid_constant__ CUtensorMap tmQ, EpiParams ep,
                      const float* __restrict__ a_scale, const float* __restrict__ w_scale, int total_kb, int stages,
                      int* status) {
  constexpr int P_BYTES = kP * kRowB, Q_BYTES = BN * kRowB, STAGE_BYTES = P_BYTES + Q_BYTES;
  constexpr int TM = SWAP ? BN : kP, TN = SWAP ? kP : BN, LDS = TN + 4;
  constexpr int TCOLS = 2 * BN < 32 ? 32 : 2 * BN;
  constexpr int NTHREADS = 64 + 32 * PW;
  constexpr int CW = BN / (PW / 4);            // accumulator columns one promotion thread owns

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ __align__(8) uint64_t full_bar[kBStagesMax], empty_bar[kBStagesMax], tfull[2], tempty[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ volatile int err_s;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int p_tile = blockIdx.x, q_tile = blockIdx.y;
  float* colscale = reinterpret_cast<float*>(smem + stages * STAGE_BYTES);   // SWAP: [total_kb][BN] activation scales

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&tfull[b], 1); mbar_init(&tempty[b], PW); }
    err_s = 0;
    mbar_fence_init();
    prefetch_tmap(&tmP);
    prefetch_tmap(&tmQ);
  }
  if (warp == 1) { tmem_alloc(&tmem_base_s, TCOLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_s;
  pdl_launch_dependents();
  pdl_wait();

  if constexpr (SWAP) {
    // activation rows of this tile are the MMA N: stage their per-K-block scales (0 past M)
    const int m0 = q_tile * BN;
    for (int i = threadIdx.x; i < total_kb * BN; i += NTHREADS) {
      const int kb = i / BN, c = i % BN;
      colscale[i] = (m0 + c < ep.M) ? a_scale[size_t(m0 + c) * total_kb + kb] : 0.f;
    }
  }
  __syncthreads();

  if (warp == 0) {
    const int p_row = p_tile * kP, q_row = q_tile * BN;
    for (int kb = 0; kb < total_kb && !err_s; ++kb) {
      const int s = kb % stages;
      if (kb >= stages && !mbar_wait(&empty_bar[s], uint32_t((kb / stages) & 1) ^ 1)) { err_s = kStatusTimeoutEmpty; break; }
      if (lane == 0) {
        uint8_t* sp = smem + s * STAGE_BYTES;
        mbar_expect_tx(&full_bar[s], STAGE_BYTES);
        tma_load_2d(sp, &tmP, &full_bar[s], kb * 128, p_row);
        tma_load_2d(sp + P_BYTES, &tmQ, &full_bar[s], kb * 128, q_row);
      }
      __syncwarp();
    }
  } else if (warp == 1) {
    const uint32_t idesc = make_idesc_e4m3(kP, BN);
    for (int kb = 0; kb < total_kb && !err_s; ++kb) {
      const int s = kb % stages, buf = kb & 1;
      if (!mbar_wait(&full_bar[s], uint32_t((kb / stages) & 1))) { err_s = kStatusTimeoutFull; break; }
      if (kb >= 2 && !mbar_wait(&tempty[buf], uint32_t(((kb >> 1) & 1) ^ 1))) { err_s = kStatusTimeoutAcc; break; }
      tc_fence_after();
      if (lane == 0) {
        const uint32_t pa = smem_u32(smem + s * STAGE_BYTES);
        const uint64_t dp = make_smem_desc_sw128(pa), dq = make_smem_desc_sw128(pa + P_BYTES);
#pragma unroll
        for (int k = 0; k < 4; ++k) umma_f8f6f4(tmem + buf * BN, dp + 2 * k, dq + 2 * k, idesc, k != 0);
        umma_commit(&empty_bar[s]);
        umma_commit(&tfull[buf]);
      }
      __syncwarp();
    }
  } else {
    // ---------------------------------------------------------------- promotion
    const int quad = warp & 3, i = quad * 32 + lane;        // row of the P operand = tensor-memory lane
    const int cb = ((warp - 2) >> 2) * CW;                  // first accumulator column of this thread
    float acc[CW];
#pragma unroll
    for (int c = 0; c < CW; ++c) acc[c] = 0.f;
    const int p_global = p_tile * kP + i;
    // the P operand's own scale: activation row (1 x 128 blocks) or weight block row (128 x 128)
    const float* my_scale = SWAP ? w_scale + size_t(p_tile) * total_kb
                                 : a_scale + size_t(min(p_global, ep.M - 1)) * total_kb;
    const float* w_blk = SWAP ? nullptr : w_scale + size_t((q_tile * BN + cb) / 128) * total_kb;
    bool ok = true;
    for (int kb = 0; kb < total_kb && !err_s; ++kb) {
      const int buf = kb & 1;
      if (!mbar_wait(&tfull[buf], uint32_t((kb >> 1) & 1))) { err_s = kStatusTimeoutAcc; ok = false; break; }
      tc_fence_after();
      const float f = SWAP ? my_scale[kb] : my_scale[kb] * w_blk[kb];
      constexpr int CH = CW >= 32 ? 32 : 16;
#pragma unroll
      for (int c = 0; c < CW; c += CH) {
        uint32_t r[CH];
        const uint32_t taddr = tmem + (uint32_t(quad * 32) << 16) + uint32_t(buf * BN + cb + c);
        if constexpr (CH == 32) tmem_ld_32x32(taddr, r); else tmem_ld_32x16(taddr, r);
        tmem_ld_wait();
        if constexpr (SWAP) {
          const float* cs = colscale + kb * BN + cb + c;
#pragma unroll
          for (int j = 0; j < CH; ++j) acc[c + j] = fmaf(f * cs[j], __uint_as_float(r[j]), acc[c + j]);
        } else {
#pragma unroll
          for (int j = 0; j < CH; ++j) acc[c + j] = fmaf(f, __uint_as_float(r[j]), acc[c + j]);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[buf]);
    }
    // accumulators -> staging tile in output orientation (the operand stages are idle by now:
    // the last tfull completion covers every MMA, hence every operand read)
    if (ok && !err_s) {
      float* stg = reinterpret_cast<float*>(smem);
      if constexpr (!SWAP) {
#pragma unroll
        for (int c = 0; c < CW; c += 4)
          *reinterpret_cast<float4*>(stg + i * LDS + cb + c) = make_float4(acc[c], acc[c + 1], acc[c + 2], acc[c + 3]);
      } else {
#pragma unroll
        for (int c = 0; c < CW; ++c) stg[(cb + c) * LDS + i] = acc[c];
      }
    }
  }

  __syncthreads();
  const int err = err_s;
  if (err == 0) {
    const int m0 = SWAP ? q_tile * BN : p_tile * kP;
    const int n0 = SWAP ? p_tile * kP : q_tile * BN;
    epilogue_pass<TN>(ep, reinterpret_cast<const float*>(smem), smem_u32(smem), LDS, m0, n0, 0, TM, 1, warp, lane, NTHREADS / 32);
  } else if (threadIdx.x == 0) {
    if (status) atomicCAS(status, 0, err);
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);   // let copies in flight land
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, TCOLS);
}

template <int BN, bool SWAP, int PW = 4>
static cudaError_t launch_block(const CUtensorMap& tmP, const CUtensorMap& tmQ, const EpiParams& ep, const float* a_scale,
                                const float* w_scale, dim3 grid, int total_kb, int stages, size_t smem, cudaStream_t st) {
  auto kern = gemm_fp8_block_kernel<BN, SWAP, PW>;
  static bool attr_done = false;
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return e;
    attr_done = true;
  }
  return launch_kernel(kern, grid, dim3(64 + 32 * PW), smem, st, 1, tmP, tmQ, ep, a_scale, w_scale, total_kb, stages,
                       kernel_status_ptr());
}

cudaError_t gemm_fp8_block_launch(const GemmArgs& a, cudaStream_t stream) {
  if (a.M <= 0 || a.N <= 0 || a.K <= 0 || a.K % 128 || a.N % 8 || !a.a_scale || !a.w_scale) return cudaErrorInvalidValue;
  if ((reinterpret_cast<uintptr_t>(a.x) & 15) || (reinterpret_cast<uintptr_t>(a.w) & 15) || a.ldx % 16 || a.ldw % 16 ||
      (reinterpret_cast<uintptr_t>(a.out) & 15) || a.ldo % 4 || (reinterpret_cast<uintptr_t>(a.bias) & 7) ||
      (reinterpret_cast<uintptr_t>(a.col_gate) & 7) || (reinterpret_cast<uintptr_t>(a.residual) & 7) || (a.residual && a.ldr % 4))
    return cudaErrorInvalidValue;
  const bool swap = a.M <= 64;
  // large problems: 256-wide tiles with eight promotion warps (MMA-bound); otherwise 128-wide with four
  const bool wide = !swap && a.M > 256 && a.N >= 512 && a.N % 128 == 0;
  const int bn = swap ? (a.M <= 16 ? 16 : (a.M <= 32 ? 32 : 64)) : (wide ? 256 : 128);
  const int total_kb = a.K / 128;
  const int p_rows = swap ? a.N : a.M, q_rows = swap ? a.M : a.N;
  const int p_tiles = (p_rows + kP - 1) / kP, q_tiles = (q_rows + bn - 1) / bn;
  const int stage_bytes = kP * kRowB + bn * kRowB;
  const int tm = swap ? bn : kP, tn = swap ? kP : bn;
  const size_t staging = size_t(tm) * (tn + 4) * 4;
  const size_t scales = swap ? size_t(total_kb) * bn * 4 : 0;
  int stages = kBStagesMax;
  while (stages > 2 && size_t(stages) * stage_bytes + scales > 180 * 1024) --stages;
  if (stages > total_kb) stages = total_kb < 2 ? 2 : total_kb;
  size_t smem = size_t(stages) * stage_bytes + scales;
  if (smem < staging) smem = staging;
  smem += 1024;
  if (smem > 200 * 1024) return cudaErrorInvalidValue;

  CUtensorMap tmP, tmQ;
  if (!make_tmap_2d(&tmP, swap ? a.w : a.x, p_rows, a.K, swap ? a.ldw : a.ldx, kP, 1)) return cudaErrorInvalidValue;
  if (!make_tmap_2d(&tmQ, swap ? a.x : a.w, q_rows, a.K, swap ? a.ldx : a.ldw, bn, 1)) return cudaErrorInvalidValue;
  EpiParams ep;
  memset(&ep, 0, sizeof(ep));
  ep.out = a.out; ep.ldo = a.ldo; ep.M = a.M; ep.N = a.N;
  ep.bias = a.bias; ep.residual = a.residual; ep.ldr = a.ldr; ep.res_mod = a.res_mod; ep.col_gate = a.col_gate;
  ep.act = a.act; ep.glu = a.glu; ep.out_fp32 = a.out_fp32;
  dim3 grid(p_tiles, q_tiles, 1);
  if (swap) {
    switch (bn) {
      case 16: return launch_block<16, true>(tmP, tmQ, ep, a.a_scale, a.w_scale, grid, total_kb, stages, smem, stream);
      case 32: return launch_block<32, true>(tmP, tmQ, ep, a.a_scale, a.w_scale, grid, total_kb, stages, smem, stream);
      default: return launch_block<64, true>(tmP, tmQ, ep, a.a_scale, a.w_scale, grid, total_kb, stages, smem, stream);
    }
  }
  if (wide) return launch_block<256, false, 8>(tmP, tmQ, ep, a.a_scale, a.w_scale, grid, total_kb, stages, smem, stream);
  return launch_block<128, false>(tmP, tmQ, ep, a.a_scale, a.w_scale, grid, total_kb, stages, smem, stream);
}

}  // namespace pb

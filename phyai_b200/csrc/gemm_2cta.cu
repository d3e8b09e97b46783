// Persistent tcgen05 GEMM on CTA pairs (cta_group::2), bf16, 256 x 256 output tiles.
//
// Two CTAs on neighbouring SMs form a cluster and work on one 256 x 256 tile. Each CTA loads 128 rows
// of the activations and 128 rows (output columns) of the weights per 64-deep K block; one thread of
// the pair's first CTA issues tcgen05.mma.cta_group::2 instructions of shape 256 x 256 x 16 that read
// the activation rows of each CTA from that CTA's shared memory and the weight rows from both. Each
// CTA therefore stages 32 KB per K block for 128 x 256 outputs instead of 48 KB (a 6-stage ring fits
// where the single-CTA kernel has 4), and the shared-memory bandwidth per multiply halves. The
// accumulator of a CTA (its 128 rows x 256 columns, fp32) lives in its own tensor memory, double
// buffered, so the next tile is multiplied while the 4 epilogue warps of each CTA drain the last one.
//
//   warp 0      TMA producer (both CTAs); transaction bytes of both land on the first CTA's barrier
//   warp 1      first CTA: issues every MMA, then signals "stage free" / "accumulator ready" to the
//               barriers of both CTAs with one tcgen05.commit; second CTA: tensor-memory bookkeeping
//   warps 2-5   epilogue, one thread per accumulator row (gemm_row_epilogue.cuh); "accumulator
//               drained" arrives on the first CTA's barrier from both CTAs
//
// Tile order, operands, epilogue semantics and results are those of gemm_persist_kernel. Every wait
// is bounded; on a timeout the CTA records a status, lets copies in flight land, meets its partner at
// the cluster barrier and frees its tensor memory.
#include <cstdlib>
#include <cstring>

#include "comm_device.cuh"
#include "gemm.cuh"
#include "gemm_epilogue.cuh"
#include "gemm_row_epilogue.cuh"
#include "launch.cuh"
#include "ptx.cuh"

namespace pb {

namespace {
constexpr int kCThreads = 192;
constexpr int kCStages = 6;
constexpr int kCM = 256, kCN = 256, kCBK = 64;   // tile of the CTA pair
constexpr int kCRows = 128;                       // activation rows and weight rows one CTA stages
constexpr int kCStageBytes = 2 * kCRows * 128;    // 32 KB
constexpr uint16_t kPairMask = 3;                 // both CTAs of the cluster

// tcgen05 instructions of one kernel must all name the same CTA group: the pair forms of the helpers.
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_f16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                              uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n" ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Every MMA this thread issued so far arrives, on retirement, on the barrier at this shared-memory
// offset in each CTA of `mask`.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar, uint16_t mask) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
                   smem_u32(bar)),
               "h"(mask)
               : "memory");
}
// Tiled load into this CTA's shared memory whose completion bytes go to a barrier of the pair's
// first CTA (`bar_cluster_addr` is a shared::cluster address).
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* m, uint32_t bar_cluster_addr, int x,
                                                 int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];" ::"r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr) : "memory");
}
}  // namespace

template <int ACT, bool GLU>
__global__ void __launch_bounds__(kCThreads, 1)
gemm_2cta_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW, EpiParams ep,
                 int p_tiles, int q_tiles, int total_kb, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ __align__(8) uint64_t full_bar[kCStages], empty_bar[kCStages], tfull[2], tempty[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ volatile int err_s;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rank = int(cluster_ctarank());          // 0: the CTA that issues the MMAs
  const int n_tiles = p_tiles * q_tiles;
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;   // clusters are (2, 1, 1): a pair is two neighbours in x

  if (threadIdx.x == 0) {
    for (int s = 0; s < kCStages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&tfull[b], 1); mbar_init(&tempty[b], 8); }   // 4 epilogue warps x 2 CTAs
    err_s = 0;
    mbar_fence_init();
    prefetch_tmap(&tmX);
    prefetch_tmap(&tmW);
  }
  if (warp == 1) { tmem_alloc_pair(&tmem_base_s, 512); tmem_relinquish_pair(); }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();            // the partner's barriers exist before anything signals them
  tc_fence_after();
  const uint32_t tmem = tmem_base_s;
  pdl_launch_dependents();
  pdl_wait();
  if (ep.zero && blockIdx.x == 0) {
    for (int i = threadIdx.x; i < ep.zero_n; i += kCThreads) ep.zero[i] = 0.f;   // predecessors are complete, successors wait
  }

  if (warp == 0) {
    // ------------------------------------------------------------------ producer (both CTAs)
    int it = 0;
    for (int t = pair; t < n_tiles && !err_s; t += n_pairs) {
      int p, q;
      grouped_tile_coords(t, p_tiles, q_tiles, p, q);
      for (int kb = 0; kb < total_kb; ++kb, ++it) {
        const int s = it % kCStages;
        if (it >= kCStages && !mbar_wait(&empty_bar[s], uint32_t((it / kCStages) & 1) ^ 1)) { err_s = kStatusTimeoutEmpty; break; }
        if (lane == 0) {
          uint8_t* sp = smem + s * kCStageBytes;
          if (rank == 0) mbar_expect_tx(&full_bar[s], 2 * kCStageBytes);   // this CTA's bytes and the partner's
          const uint32_t bar = map_to_cta(smem_u32(&full_bar[s]), 0);
          tma_load_2d_pair(sp, &tmX, bar, kb * kCBK, p * kCM + rank * kCRows);
          tma_load_2d_pair(sp + kCRows * 128, &tmW, bar, kb * kCBK, q * kCN + rank * kCRows);
        }
        __syncwarp();
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (first CTA only)
    if (rank == 0) {
      const uint32_t idesc = make_idesc_f16(kCM, kCN, 1);
      int it = 0, ti = 0;
      for (int t = pair; t < n_tiles && !err_s; t += n_pairs, ++ti) {
        const int buf = ti & 1;
        if (ti >= 2 && !mbar_wait(&tempty[buf], uint32_t(((ti >> 1) & 1) ^ 1))) { err_s = kStatusTimeoutAcc; break; }
        tc_fence_after();
        bool ok = true;
        for (int kb = 0; kb < total_kb; ++kb, ++it) {
          const int s = it % kCStages;
          if (!mbar_wait(&full_bar[s], uint32_t((it / kCStages) & 1))) { err_s = kStatusTimeoutFull; ok = false; break; }
          tc_fence_after();
          if (lane == 0) {
            const uint32_t pa = smem_u32(smem + s * kCStageBytes);
            const uint64_t dx = make_smem_desc_sw128(pa), dw = make_smem_desc_sw128(pa + kCRows * 128);
#pragma unroll
            for (int k = 0; k < 4; ++k) umma_f16_pair(tmem + buf * kCN, dx + 2 * k, dw + 2 * k, idesc, (kb | k) != 0);
            umma_commit_pair(&empty_bar[s], kPairMask);
          }
          __syncwarp();
        }
        if (!ok) break;
        if (lane == 0) umma_commit_pair(&tfull[buf], kPairMask);
        __syncwarp();
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (one thread per row)
    const int quad = warp & 3, row_in_tile = quad * 32 + lane;
    const uint32_t lane_base = tmem + (uint32_t(quad * 32) << 16);
    int ti = 0;
    for (int t = pair; t < n_tiles && !err_s; t += n_pairs, ++ti) {
      int p, q;
      grouped_tile_coords(t, p_tiles, q_tiles, p, q);
      const int buf = ti & 1;
      if (!mbar_wait(&tfull[buf], uint32_t((ti >> 1) & 1))) { err_s = kStatusTimeoutAcc; break; }
      tc_fence_after();
      row_epilogue_tile<ACT, GLU>(ep, lane_base + uint32_t(buf * kCN), kCN, p * kCM + rank * kCRows + row_in_tile, q * kCN);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&tempty[buf]), 0));
    }
  }

  tc_fence_before();
  __syncthreads();
  if (err_s && threadIdx.x == 0) {
    if (status) atomicCAS(status, 0, int(err_s));
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);   // let copies in flight land
  }
  __syncthreads();
  cluster_sync_all();            // the partner may still be reading this CTA's operands or signalling its barriers
  if (warp == 1) tmem_dealloc_pair(tmem, 512);
}

static unsigned long long g_2cta_launches = 0;

template <int ACT, bool GLU>
static cudaError_t launch_2cta(const CUtensorMap& tx, const CUtensorMap& tw, const EpiParams& ep, int p_tiles, int q_tiles,
                               int total_kb, int clusters, cudaStream_t st) {
  const size_t smem = size_t(kCStages) * kCStageBytes + 1024;
  auto kern = gemm_2cta_kernel<ACT, GLU>;
  static bool attr_done = false;
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    if (e != cudaSuccess) return e;
    attr_done = true;
  }
  // the CTA pair of cta_group::2 is a cluster of two along x
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * clusters);
  cfg.blockDim = dim3(kCThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attrs[2];
  int na = 0;
  attrs[na].id = cudaLaunchAttributeClusterDimension;
  attrs[na].val.clusterDim.x = 2;
  attrs[na].val.clusterDim.y = 1;
  attrs[na].val.clusterDim.z = 1;
  ++na;
  if (pdl_enabled()) {
    attrs[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  cfg.attrs = attrs;
  cfg.numAttrs = na;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, kern, tx, tw, ep, p_tiles, q_tiles, total_kb, kernel_status_ptr());
  if (e == cudaSuccess) { bump_launch_counter(1); ++g_2cta_launches; }
  return e;
}

static int sm_count() {
  int sms = 148, dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return sms > 0 ? sms : 148;
}

static int g_2cta_mode = -1;   // -1: PHYAI_GEMM_2CTA decides, 0 / 1: set by the program
void set_gemm_2cta(int mode) { g_2cta_mode = mode; }
unsigned long long gemm_2cta_launches() { return g_2cta_launches; }

bool gemm_2cta_eligible(const GemmArgs& a) {
  // PHYAI_GEMM_2CTA=1 (or set_gemm_2cta(1)) routes every large plain bf16 problem to the CTA-pair kernel, 0 none.
  // Unset: the shapes where it measured ahead of the persistent kernel inside a CUDA graph, i.e. very wide outputs
  // (968 x 2048 -> 32768: 117.5 -> 111.4 us; 7040 x 5120 -> 27648: 1758 -> 1636 us) and long-K products of many rows
  // (7040 x 13824 -> 5120: 818 -> 783 us); it was level or behind elsewhere (7040 x 5120 -> 7168: 417 -> 423 us).
  static const int env_mode = [] { const char* e = getenv("PHYAI_GEMM_2CTA"); return !e || !e[0] ? -1 : (e[0] == '1' ? 1 : 0); }();
  const int mode = g_2cta_mode < 0 ? env_mode : g_2cta_mode;
  if (mode == 0 || a.push) return false;
  if (mode < 0 && !(a.N >= 16384 || (a.K >= 8192 && a.N >= 4096 && a.M >= 4096))) return false;
  if (((a.M + kCM - 1) / kCM) * ((a.N + kCN - 1) / kCN) < sm_count() / 2) return false;
  return a.M >= 512 && a.N >= 2048 && a.K >= 256 && !a.fp8 && !a.out_fp32 && !a.rope &&
         !a.a_scale && !a.w_scale && !a.trace && a.force_bn == 0 && a.force_swap == -1 && a.force_splits == 0 &&
         (reinterpret_cast<uintptr_t>(a.bias) & 15) == 0 && (reinterpret_cast<uintptr_t>(a.col_gate) & 15) == 0 &&
         (reinterpret_cast<uintptr_t>(a.residual) & 15) == 0 && (!a.residual || a.ldr % 8 == 0) && a.ldo % 8 == 0;
}

cudaError_t gemm_2cta_launch(const GemmArgs& a, cudaStream_t stream) {
  CUtensorMap tx, tw;
  if (!make_tmap_2d(&tx, a.x, a.M, a.K, a.ldx, kCRows, 2) || !make_tmap_2d(&tw, a.w, a.N, a.K, a.ldw, kCRows, 2))
    return cudaErrorInvalidValue;
  EpiParams ep;
  memset(&ep, 0, sizeof(ep));
  ep.out = a.out; ep.ldo = a.ldo; ep.M = a.M; ep.N = a.N; ep.bias = a.bias; ep.residual = a.residual; ep.ldr = a.ldr;
  ep.res_mod = a.res_mod; ep.col_gate = a.col_gate; ep.act = a.act; ep.glu = a.glu;
  ep.row_scale = a.row_scale; ep.sumsq = a.sumsq; ep.zero = a.zero; ep.zero_n = a.zero_n;
  ep.rs_inv_dim = a.row_rms_dim > 0 ? 1.f / float(a.row_rms_dim) : 0.f; ep.rs_eps = a.row_rms_eps;
  const int p_tiles = (a.M + kCM - 1) / kCM, q_tiles = (a.N + kCN - 1) / kCN, total_kb = (a.K + kCBK - 1) / kCBK;
  const int pairs = sm_count() / 2;
  const int clusters = p_tiles * q_tiles < pairs ? p_tiles * q_tiles : pairs;
#define PB_C(A, G) launch_2cta<A, G>(tx, tw, ep, p_tiles, q_tiles, total_kb, clusters, stream)
  if (a.glu) {
    switch (a.act) { case 1: return PB_C(1, true); case 2: return PB_C(2, true); case 3: return PB_C(3, true); default: return PB_C(0, true); }
  }
  switch (a.act) { case 1: return PB_C(1, false); case 2: return PB_C(2, false); case 3: return PB_C(3, false); default: return PB_C(0, false); }
#undef PB_C
}

}  // namespace pb

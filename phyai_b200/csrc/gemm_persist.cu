// Persistent tcgen05 GEMM for large problems (M >= 512, N >= 2048), bf16, 128 x 256 tiles.
//
// gemm.cu launches one CTA per output tile: its tensor core sits idle while the tile's
// accumulator is drained, converted and stored, and again while the next CTA on that SM sets up.
// Here one CTA per SM walks a list of tiles and the roles never stop:
//
//   warp 0      TMA producer: operands of tile after tile into a 4-stage shared-memory ring
//   warp 1      issues every tcgen05.mma; accumulators alternate between two 256-column halves
//               of tensor memory, so tile i + 1 is multiplied while tile i is drained
//   warps 2-5   epilogue: one thread per accumulator row reads 32 columns at a time out of
//               tensor memory, applies bias / activation / gated activation / gate / residual
//               and stores the row segment straight to global memory (no staging tile: shared
//               memory belongs to the operand ring)
//
// Tiles are taken in the grouped order (8 column tiles per group) so the tiles in flight across
// the chip form a compact block of the output and both operands are re-read from L2.
// Same operands, epilogue semantics and result as gemm_kernel; the launcher in gemm.cu routes a
// call here when the shape qualifies and nothing exotic (fp8, fp32 output, the rotating QKV epilogue)
// is requested. Every wait is bounded.
#include <cstdlib>
#include <cstring>
#include <type_traits>

#include "comm_device.cuh"
#include "gemm.cuh"
#include "gemm_epilogue.cuh"
#include "gemm_row_epilogue.cuh"
#include "launch.cuh"
#include "ptx.cuh"

namespace pb {

namespace {
constexpr int kPThreads = 192;
constexpr int kPStages = 4;
constexpr int kPM = 128, kPN = 256, kPBK = 64;
constexpr int kPStageBytes = (kPM + kPN) * 128;   // 48 KB
}  // namespace

// COMM: the variant that talks to peer GPUs. `push.world > 0`: the bare bf16 product goes to the slots of
// every rank (or, with rows_per_rank, of the row's owner) and the CTA signals the channel once, after its
// last tile. `push.wait_channel >= 0`: the activations are being written by peers; the producer waits for
// their arrivals before its first load and the kernel closes the channel's call at the end.
struct NoCommP { int wait_channel, world; };
template <int ACT, bool GLU, bool COMM>
__global__ void __launch_bounds__(kPThreads, 1)
gemm_persist_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW, EpiParams ep,
                    const __grid_constant__ std::conditional_t<COMM, PushParams, NoCommP> push,
                    int p_tiles, int q_tiles, int total_kb, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ __align__(8) uint64_t full_bar[kPStages], empty_bar[kPStages], tfull[2], tempty[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ volatile int err_s;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_tiles = p_tiles * q_tiles;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kPStages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&tfull[b], 1); mbar_init(&tempty[b], 4); }
    err_s = 0;
    mbar_fence_init();
    prefetch_tmap(&tmX);
    prefetch_tmap(&tmW);
  }
  if (warp == 1) { tmem_alloc(&tmem_base_s, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_s;
  pdl_launch_dependents();
  pdl_wait();
  if (ep.zero && blockIdx.x == 0) {
    for (int i = threadIdx.x; i < ep.zero_n; i += kPThreads) ep.zero[i] = 0.f;   // predecessors are complete, successors wait
  }

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    if constexpr (COMM) if (push.wait_channel >= 0) {
      if (lane == 0) {
        const ChannelSig* ws = reinterpret_cast<const ChannelSig*>(push.local_sig) + push.wait_channel;
        const int wp = int(ld_relaxed_sys(&ws->epoch) & 1u);
        if (!wait_counter_ge(&ws->arrive[wp], push.wait_expect)) err_s = kStatusTimeoutPeer;
        asm volatile("fence.proxy.async;" ::: "memory");   // peers' stores before this CTA's TMA reads
      }
      __syncwarp();
    }
    int it = 0;
    for (int t = blockIdx.x; t < n_tiles && !err_s; t += gridDim.x) {
      int p, q;
      grouped_tile_coords(t, p_tiles, q_tiles, p, q);
      for (int kb = 0; kb < total_kb; ++kb, ++it) {
        const int s = it % kPStages;
        if (it >= kPStages && !mbar_wait(&empty_bar[s], uint32_t((it / kPStages) & 1) ^ 1)) { err_s = kStatusTimeoutEmpty; break; }
        if (lane == 0) {
          uint8_t* sp = smem + s * kPStageBytes;
          mbar_expect_tx(&full_bar[s], kPStageBytes);
          tma_load_2d(sp, &tmX, &full_bar[s], kb * kPBK, p * kPM);
          tma_load_2d(sp + kPM * 128, &tmW, &full_bar[s], kb * kPBK, q * kPN);
        }
        __syncwarp();
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    const uint32_t idesc = make_idesc_f16(kPM, kPN, 1);
    int it = 0, ti = 0;
    for (int t = blockIdx.x; t < n_tiles && !err_s; t += gridDim.x, ++ti) {
      const int buf = ti & 1;
      if (ti >= 2 && !mbar_wait(&tempty[buf], uint32_t(((ti >> 1) & 1) ^ 1))) { err_s = kStatusTimeoutAcc; break; }
      tc_fence_after();
      bool ok = true;
      for (int kb = 0; kb < total_kb; ++kb, ++it) {
        const int s = it % kPStages;
        if (!mbar_wait(&full_bar[s], uint32_t((it / kPStages) & 1))) { err_s = kStatusTimeoutFull; ok = false; break; }
        tc_fence_after();
        if (lane == 0) {
          const uint32_t pa = smem_u32(smem + s * kPStageBytes);
          const uint64_t dx = make_smem_desc_sw128(pa), dw = make_smem_desc_sw128(pa + kPM * 128);
#pragma unroll
          for (int k = 0; k < 4; ++k) umma_f16(tmem + buf * kPN, dx + 2 * k, dw + 2 * k, idesc, (kb | k) != 0);
          umma_commit(&empty_bar[s]);
        }
        __syncwarp();
      }
      if (!ok) break;
      if (lane == 0) umma_commit(&tfull[buf]);
      __syncwarp();
    }
  } else {
    // ------------------------------------------------------------------ epilogue (one thread per row)
    const int quad = warp & 3, row_in_tile = quad * 32 + lane;
    const uint32_t lane_base = tmem + (uint32_t(quad * 32) << 16);
    int ti = 0;
    int push_parity = 0;
    if constexpr (COMM) if (push.world > 0)
      push_parity = int(ld_relaxed_sys(&(reinterpret_cast<const ChannelSig*>(push.local_sig) + push.channel)->epoch) & 1u);
    for (int t = blockIdx.x; t < n_tiles && !err_s; t += gridDim.x, ++ti) {
      int p, q;
      grouped_tile_coords(t, p_tiles, q_tiles, p, q);
      const int buf = ti & 1;
      if (!mbar_wait(&tfull[buf], uint32_t((ti >> 1) & 1))) { err_s = kStatusTimeoutAcc; break; }
      tc_fence_after();
      const int m = p * kPM + row_in_tile, n0 = q * kPN;
      const bool live = m < ep.M;
      const __nv_bfloat16* res_row = (ep.residual && live) ? ep.residual + size_t(ep.res_mod > 0 ? (m % ep.res_mod) : m) * ep.ldr : nullptr;
      __nv_bfloat16* out_row = reinterpret_cast<__nv_bfloat16*>(ep.out) + size_t(live ? m : 0) * ep.ldo;
      float rscale = 1.f, ss = 0.f;
      if (ep.row_scale && live) {
        rscale = ep.row_scale[m];
        if (ep.rs_inv_dim > 0.f) rscale = rsqrtf(rscale * ep.rs_inv_dim + ep.rs_eps);
      }
#pragma unroll 1
      for (int c = 0; c < kPN; c += 32) {
        uint32_t r[32];
        tmem_ld_32x32(lane_base + uint32_t(buf * kPN + c), r);
        tmem_ld_wait();
        if (!live) continue;
#pragma unroll
        for (int g = 0; g < 4; ++g) {            // 8 accumulator columns per group
          const int n = n0 + c + 8 * g;
          if (n >= ep.N) continue;
          float x[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) x[j] = __uint_as_float(r[8 * g + j]);
          if constexpr (COMM) if (push.world > 0) {
            uint4 o;
            __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
            for (int j = 0; j < 4; ++j) o2[j] = __floats2bfloat162_rn(x[2 * j], x[2 * j + 1]);
            const size_t slot = size_t(push.slots_off) + (size_t(push_parity) * push.world + push.rank) * size_t(push.slot_stride);
            if (push.rows_per_rank > 0) {
              const int dst = m / push.rows_per_rank;
              *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(push.data.p[dst]) + slot +
                                        size_t(m - dst * push.rows_per_rank) * push.ld + n) = o;
            } else {
              for (int dst = 0; dst < push.world; ++dst)
                *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(push.data.p[dst]) + slot + size_t(m) * push.ld + n) = o;
            }
            continue;
          }
          ss += row_epilogue_8<ACT, GLU>(ep, x, n, res_row, out_row, rscale);
        }
      }
      if (ep.sumsq && live) atomicAdd(ep.sumsq + m, ss);   // one add per row and tile
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[buf]);
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
  if (warp == 1) tmem_dealloc(tmem, 512);
  if constexpr (COMM) {
    if (push.world > 0 && threadIdx.x == 0 && !err_s) {
      const int parity = int(ld_relaxed_sys(&(reinterpret_cast<const ChannelSig*>(push.local_sig) + push.channel)->epoch) & 1u);
      channel_signal_all(push.sig, push.channel, parity, push.world);   // every store of this CTA is behind the barrier above
    }
    if (push.wait_channel >= 0) {
      ChannelSig* ws = const_cast<ChannelSig*>(reinterpret_cast<const ChannelSig*>(push.local_sig)) + push.wait_channel;
      const int wp = int(ld_relaxed_sys(&ws->epoch) & 1u);   // unchanged until every CTA took its ticket
      channel_finish(ws, wp, gridDim.x);
    }
  }
}

template <int ACT, bool GLU>
static cudaError_t launch_persist(const CUtensorMap& tx, const CUtensorMap& tw, const EpiParams& ep, const PushParams* push,
                                  int p_tiles, int q_tiles, int total_kb, int ctas, cudaStream_t st) {
  const size_t smem = size_t(kPStages) * kPStageBytes + 1024;
  if (push) {
    auto kern = gemm_persist_kernel<ACT, GLU, true>;
    static bool attr_done = false;
    if (!attr_done) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
      if (e != cudaSuccess) return e;
      attr_done = true;
    }
    return launch_kernel(kern, dim3(ctas), dim3(kPThreads), smem, st, 1, tx, tw, ep, *push, p_tiles, q_tiles, total_kb, kernel_status_ptr());
  }
  auto kern = gemm_persist_kernel<ACT, GLU, false>;
  static bool attr_done = false;
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    if (e != cudaSuccess) return e;
    attr_done = true;
  }
  NoCommP none{-1, 0};
  return launch_kernel(kern, dim3(ctas), dim3(kPThreads), smem, st, 1, tx, tw, ep, none, p_tiles, q_tiles, total_kb, kernel_status_ptr());
}

bool gemm_persist_eligible(const GemmArgs& a) {
  static const bool off = [] { const char* e = getenv("PHYAI_GEMM_PERSIST"); return e && e[0] == '0'; }();
  if (off) return false;
  int sms = 148;
  {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  }
  // fewer tiles than SMs: the one-tile-per-CTA kernel splits K over a cluster and fills the chip better
  if (((a.M + kPM - 1) / kPM) * ((a.N + kPN - 1) / kPN) < sms) return false;
  if (a.push && (a.push->world > 0 || a.push->wait_channel >= 0)) {
    // peer variants of this kernel: PHYAI_GEMM_PERSIST_COMM=0 keeps them on the one-tile-per-CTA kernel
    static const bool comm_on = [] { const char* e = getenv("PHYAI_GEMM_PERSIST_COMM"); return !(e && e[0] == '0'); }();
    if (!comm_on) return false;
    // Push / scatter from here are row-per-thread 16-byte stores: fine when half of the rows stay local (2 ranks:
    // 233.0 -> 213.9 ms per Cosmos3 step), but at 4 ranks three quarters of them cross NVLink in 64-byte pieces and the
    // step got slower (77.4 -> 83.8 ms on 8 GPUs), so larger groups keep the one-tile kernel, whose push epilogue
    // writes 256 contiguous bytes per warp. The wait mode only reads local memory and stays here.
    static const int push_max_world = [] { const char* e = getenv("PHYAI_GEMM_PERSIST_PUSH_WORLD"); return e ? atoi(e) : 2; }();
    if (a.push->world > push_max_world) return false;
  }
  if (a.push && a.push->world > 0 && (a.push->ld % 8 || a.push->slots_off % 8 || a.push->slot_stride % 8)) return false;
  return a.M >= 512 && a.N >= 2048 && a.K >= 256 && !a.fp8 && !a.out_fp32 && !a.rope && !a.a_scale && !(a.push && (a.row_scale || a.sumsq)) &&
         !a.w_scale && !a.trace && a.force_bn == 0 && a.force_swap == -1 && a.force_splits == 0 &&
         (reinterpret_cast<uintptr_t>(a.bias) & 15) == 0 && (reinterpret_cast<uintptr_t>(a.col_gate) & 15) == 0 &&
         (reinterpret_cast<uintptr_t>(a.residual) & 15) == 0 && (!a.residual || a.ldr % 8 == 0) && a.ldo % 8 == 0;
}

cudaError_t gemm_persist_launch(const GemmArgs& a, cudaStream_t stream, int* n_ctas) {
  CUtensorMap tx, tw;
  if (!make_tmap_2d(&tx, a.x, a.M, a.K, a.ldx, kPM, 2) || !make_tmap_2d(&tw, a.w, a.N, a.K, a.ldw, kPN, 2)) return cudaErrorInvalidValue;
  EpiParams ep;
  memset(&ep, 0, sizeof(ep));
  ep.out = a.out; ep.ldo = a.ldo; ep.M = a.M; ep.N = a.N; ep.bias = a.bias; ep.residual = a.residual; ep.ldr = a.ldr;
  ep.res_mod = a.res_mod; ep.col_gate = a.col_gate; ep.act = a.act; ep.glu = a.glu;
  ep.row_scale = a.row_scale; ep.sumsq = a.sumsq; ep.zero = a.zero; ep.zero_n = a.zero_n;
  ep.rs_inv_dim = a.row_rms_dim > 0 ? 1.f / float(a.row_rms_dim) : 0.f; ep.rs_eps = a.row_rms_eps;
  const int p_tiles = (a.M + kPM - 1) / kPM, q_tiles = (a.N + kPN - 1) / kPN, total_kb = (a.K + kPBK - 1) / kPBK;
  int sms = 148;
  {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 148;
  }
  const int ctas = p_tiles * q_tiles < sms ? p_tiles * q_tiles : sms;
  if (n_ctas) *n_ctas = ctas;
  PushParams pp;
  const PushParams* push = nullptr;
  if (a.push) {
    pp = *a.push;
    if (pp.world == 0 && pp.wait_channel < 0) pp.wait_channel = -1;
    push = &pp;
  }
#define PB_P(A, G) launch_persist<A, G>(tx, tw, ep, push, p_tiles, q_tiles, total_kb, ctas, stream)
  if (a.glu) {
    switch (a.act) { case 1: return PB_P(1, true); case 2: return PB_P(2, true); case 3: return PB_P(3, true); default: return PB_P(0, true); }
  }
  switch (a.act) { case 1: return PB_P(1, false); case 2: return PB_P(2, false); case 3: return PB_P(3, false); default: return PB_P(0, false); }
#undef PB_P
}

}  // namespace pb

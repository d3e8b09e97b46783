// tcgen05 GEMM for sm_100a: out = epilogue(X[M,K] @ W[N,K]^T).
//
// One CTA computes a 128 x BN accumulator tile that lives in tensor memory. The
// 128-row operand ("P") and the BN-row operand ("Q") are both K-major and arrive
// through TMA (128-byte swizzle, one copy per CTA) into a ring of shared-memory
// stages; one thread issues tcgen05.mma and frees stages with tcgen05.commit.
// For skinny problems (M <= 256, the action-expert regime) the operands are
// swapped so the weight rows fill the 128-wide MMA M dimension and the few
// activation rows become the MMA N dimension; the K loop is then split over a
// thread-block cluster (1,1,S) and the S partial tiles are summed through
// distributed shared memory, each CTA finishing 1/S of the rows.
//
// Warp roles (192 threads): warp 0 = TMA producer, warp 1 = MMA issuer and TMEM
// owner, warps 2..5 = TMEM -> shared staging (one 32-lane quadrant each). After
// staging, all threads run the reduce + epilogue + store pass over the tile in
// output orientation, so global accesses are coalesced along N in both modes.
//
// Capability parity: this replaces the library GEMMs behind the reference's
// linear kernels (phyai/src/phyai/layers/linear/backends/flashinfer.py:110-126,
// phyai/src/phyai/layers/linear/backends/torch.py:98-176) and fuses what the
// reference runs as separate kernels after them (bias, activation, gated
// activation, gated residual, residual add).
#include "gemm.cuh"

#include <atomic>
#include <cstdlib>
#include <cstring>
#include <type_traits>
#include <mutex>
#include <unordered_map>
#include <vector>

#include "comm_device.cuh"
#include "gemm_epilogue.cuh"
#include "launch.cuh"
#include "ptx.cuh"

namespace pb {

// ------------------------------------------------------------- shared globals
__device__ int g_kernel_status = 0;
static std::atomic<uint64_t> g_launches{0};

int* kernel_status_ptr() {
  static thread_local int* ptrs[64] = {nullptr};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return nullptr;
  if (!ptrs[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_kernel_status) != cudaSuccess) return nullptr;
    ptrs[dev] = static_cast<int*>(p);
  }
  return ptrs[dev];
}
int read_and_clear_kernel_status() {
  int* p = kernel_status_ptr();
  if (!p) return -1;
  int v = 0;
  cudaMemcpy(&v, p, sizeof(int), cudaMemcpyDeviceToHost);
  if (v != 0) cudaMemset(p, 0, sizeof(int));
  return v;
}
uint64_t launch_counter() { return g_launches.load(); }
void reset_launch_counter() { g_launches.store(0); }
void bump_launch_counter(unsigned long long n) { g_launches.fetch_add(n); }
static std::atomic<bool> g_pdl{false};
bool pdl_enabled() { return g_pdl.load(); }
void set_pdl_enabled(bool on) { g_pdl.store(on); }

constexpr int kThreads = 192;
constexpr int kMaxStages = 8;
constexpr int kTileP = 128;        // rows of the 128-row operand = UMMA M
constexpr int kRowBytes = 128;     // one swizzle-128B row: 64 bf16 or 128 e4m3

// COMM selects the variant that talks to peer GPUs (push / scatter epilogue, wait before the
// activation loads). The plain variant does not even carry the parameter block, which keeps
// the launch descriptor of the thousands of ordinary GEMMs in a captured step small.
struct NoComm { int wait_channel, world; };
// Largest grid whose CTAs are taken to be resident at once (148 SMs, one CTA each; clusters of up to eight
// fragment over the GPCs, hence the margin).
constexpr int kTailMaxCtas = 128;
template <int BN, bool SWAP, bool FP8, bool COMM>
__global__ void __launch_bounds__(kThreads)
gemm_kernel(const __grid_constant__ CUtensorMap tmP, const __grid_constant__ CUtensorMap tmQ,
            EpiParams ep, const __grid_constant__ std::conditional_t<COMM, PushParams, NoComm> push,
            int total_kb, int kb_per_split, int stages, int* status, unsigned long long* trace) {
  constexpr int BK = FP8 ? 128 : 64;                 // elements per k-block
  constexpr int P_BYTES = kTileP * kRowBytes;        // 16 KB
  constexpr int Q_BYTES = BN * kRowBytes;
  constexpr int STAGE_BYTES = P_BYTES + Q_BYTES;
  constexpr int TMEM_COLS = BN < 32 ? 32 : (BN == 192 ? 256 : BN);   // allocations are powers of two
  constexpr int TM = SWAP ? BN : kTileP;             // tile rows in output orientation
  constexpr int TN = SWAP ? kTileP : BN;             // tile cols in output orientation
  constexpr int LDS = TN + 4;                        // staging row stride (floats)

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  __shared__ __align__(8) uint64_t full_bar[kMaxStages];
  __shared__ __align__(8) uint64_t empty_bar[kMaxStages];
  __shared__ __align__(8) uint64_t acc_bar;
  __shared__ uint32_t tmem_base_s;
  __shared__ int err_s;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // optional phase timestamps (ns): 8 slots per CTA, written by one thread of the phase
  unsigned long long* tr = trace ? trace + 32 * (blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z))
                                 : nullptr;
  if (tr && threadIdx.x == 0) tr[0] = globaltimer_ns();
  // Tile order: the hardware hands out blockIdx.x fastest. Walking all P tiles of one Q tile
  // before the next Q tile makes every wave of CTAs re-read the whole P operand; instead the
  // linear block index sweeps groups of kGroupQ Q-tiles with P-tiles inside, so the ~148 tiles
  // in flight form a compact block of the output and both operands are reused out of L2.
  constexpr int kGroupQ = 8;
  int p_tile, q_tile;
  {
    const int P = gridDim.x, Q = gridDim.y;
    const int lin = blockIdx.x + P * blockIdx.y;
    const int g = lin / (kGroupQ * P);
    const int q0 = g * kGroupQ;
    const int gq = min(kGroupQ, Q - q0);
    const int r = lin - g * kGroupQ * P;
    q_tile = q0 + r % gq;
    p_tile = r / gq;
  }
  const int split = blockIdx.z;
  const int nsplit = gridDim.z;
  const int kb0 = split * kb_per_split;
  const int nkb = min(kb_per_split, total_kb - kb0);

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(&acc_bar, 1);
    err_s = 0;
    mbar_fence_init();
    prefetch_tmap(&tmP);
    prefetch_tmap(&tmQ);
  }
  if (warp == 1) {
    tmem_alloc(&tmem_base_s, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_s;

  pdl_launch_dependents();
  if (warp != 0) pdl_wait();  // everything but the weight prefetch below depends on earlier kernels
  if (tr && threadIdx.x == 0) tr[1] = globaltimer_ns();

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    // Weights never depend on a predecessor kernel: their first tiles are requested
    // before the dependency wait, the activation tiles of the same stages right after it.
    const CUtensorMap* tmW = SWAP ? &tmP : &tmQ;
    const CUtensorMap* tmX = SWAP ? &tmQ : &tmP;
    const int w_row = SWAP ? p_tile * kTileP : q_tile * BN;
    const int x_row = SWAP ? q_tile * BN : p_tile * kTileP;
    constexpr int W_OFF = SWAP ? 0 : P_BYTES, X_OFF = SWAP ? P_BYTES : 0;
    const int pre = min(nkb, stages);
    if (lane == 0) {
      for (int kb = 0; kb < pre; ++kb) {
        mbar_expect_tx(&full_bar[kb], STAGE_BYTES);
        tma_load_2d(smem + kb * STAGE_BYTES + W_OFF, tmW, &full_bar[kb], (kb0 + kb) * BK, w_row);
      }
    }
    pdl_wait();
    if constexpr (COMM) if (push.wait_channel >= 0) {
      // the activations were stored by peer GPUs: wait for their arrivals, then order the
      // TMA (async proxy) reads after the acquire
      if (lane == 0) {
        const ChannelSig* ws = reinterpret_cast<const ChannelSig*>(push.local_sig) + push.wait_channel;
        const int wp = int(ld_relaxed_sys(&ws->epoch) & 1u);
        if (!wait_counter_ge(&ws->arrive[wp], push.wait_expect)) err_s = kStatusTimeoutPeer;
        asm volatile("fence.proxy.async;" ::: "memory");
      }
      __syncwarp();
    }
    if (lane == 0) {
      for (int kb = 0; kb < pre; ++kb)
        tma_load_2d(smem + kb * STAGE_BYTES + X_OFF, tmX, &full_bar[kb], (kb0 + kb) * BK, x_row);
    }
    __syncwarp();
    for (int kb = pre; kb < nkb; ++kb) {
      const int s = kb % stages;
      const uint32_t ph = (kb / stages) & 1;
      if (!mbar_wait(&empty_bar[s], ph ^ 1)) {
        if (lane == 0) { err_s = kStatusTimeoutEmpty; }
        break;
      }
      if (lane == 0) {
        uint8_t* sp = smem + s * STAGE_BYTES;
        mbar_expect_tx(&full_bar[s], STAGE_BYTES);
        tma_load_2d(sp + W_OFF, tmW, &full_bar[s], (kb0 + kb) * BK, w_row);
        tma_load_2d(sp + X_OFF, tmX, &full_bar[s], (kb0 + kb) * BK, x_row);
      }
      __syncwarp();
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    const uint32_t idesc = FP8 ? make_idesc_e4m3(kTileP, BN) : make_idesc_f16(kTileP, BN, 1);
    bool ok = true;
    for (int kb = 0; kb < nkb; ++kb) {
      const int s = kb % stages;
      const uint32_t ph = (kb / stages) & 1;
      if (!mbar_wait(&full_bar[s], ph)) {
        if (lane == 0) { err_s = kStatusTimeoutFull; }
        ok = false;
        break;
      }
      tc_fence_after();
      if (lane == 0) {
        const uint32_t pa = smem_u32(smem + s * STAGE_BYTES);
        const uint64_t dp = make_smem_desc_sw128(pa);
        const uint64_t dq = make_smem_desc_sw128(pa + P_BYTES);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          // 32 bytes of K per instruction: +2 in the descriptor's 16-byte address units
          umma_f16_or_f8<FP8>(tmem_base, dp + 2 * k, dq + 2 * k, idesc, (kb | k) != 0);
        }
        umma_commit(&empty_bar[s]);
      }
      __syncwarp();
    }
    if (lane == 0 && ok) umma_commit(&acc_bar);
    if (tr && lane == 0) tr[2] = globaltimer_ns();
    __syncwarp();
  } else {
    // ----------------------------------------- TMEM -> shared staging (4 warps)
    const int quad = warp & 3;
    float* stg = reinterpret_cast<float*>(smem);
    if (!mbar_wait(&acc_bar, 0)) {
      if (lane == 0) { err_s = kStatusTimeoutAcc; }
    } else {
      tc_fence_after();
      if (tr && threadIdx.x == 64) tr[3] = globaltimer_ns();
      const int i = quad * 32 + lane;  // row of the P operand inside the tile
      constexpr int CH = BN >= 32 ? 32 : 16;
#pragma unroll 1
      for (int c = 0; c < BN; c += CH) {
        uint32_t r[CH];
        const uint32_t taddr = tmem_base + (uint32_t(quad * 32) << 16) + uint32_t(c);
        if constexpr (CH == 32) tmem_ld_32x32(taddr, r); else tmem_ld_32x16(taddr, r);
        tmem_ld_wait();
        if constexpr (!SWAP) {
          float4* dst = reinterpret_cast<float4*>(stg + i * LDS + c);
#pragma unroll
          for (int t = 0; t < CH / 4; ++t)
            dst[t] = make_float4(__uint_as_float(r[4 * t]), __uint_as_float(r[4 * t + 1]),
                                 __uint_as_float(r[4 * t + 2]), __uint_as_float(r[4 * t + 3]));
        } else {
#pragma unroll
          for (int j = 0; j < CH; ++j) stg[(c + j) * LDS + i] = __uint_as_float(r[j]);
        }
      }
      tc_fence_before();
    }
  }

  __syncthreads();
  if (nsplit > 1) cluster_sync_all();
  if (tr && threadIdx.x == 0) tr[4] = globaltimer_ns();
  const int err = err_s;

  if (ep.zero && blockIdx.x + blockIdx.y + blockIdx.z == 0) {
    // predecessors have completed (every thread is past its dependency wait), successors still wait on this grid
    for (int i = threadIdx.x; i < ep.zero_n; i += kThreads) ep.zero[i] = 0.f;
  }
  if (err == 0) {
    // ------------------------- reduce over the cluster + epilogue + store
    const int m0 = SWAP ? q_tile * BN : p_tile * kTileP;
    const int n0 = SWAP ? p_tile * kTileP : q_tile * BN;
    const int rows_per_cta = TM / nsplit;
    bool pushed = false;
    if constexpr (COMM) if (push.world > 0) {
      pushed = true;
      const ChannelSig* ls = reinterpret_cast<const ChannelSig*>(push.local_sig) + push.channel;
      const int parity = int(ld_relaxed_sys(&ls->epoch) & 1u);
      epilogue_push<TN>(push, parity, ep.M, ep.N, smem_u32(smem), reinterpret_cast<const float*>(smem), LDS,
                        m0, n0, split * rows_per_cta, rows_per_cta, nsplit, warp, lane, kThreads / 32);
      __syncthreads();
      if (threadIdx.x == 0) channel_signal_all(push.sig, push.channel, parity, push.world);
      if (push.tail) {
        // consumer half in the same launch: all CTAs of the grid are resident, so waiting here for every
        // rank's tiles (this rank's other CTAs included) cannot starve a CTA that has not pushed yet
        __shared__ float tail_red[32];
        __shared__ int tail_ok;
        ChannelSig* lsm = const_cast<ChannelSig*>(ls);
        if (threadIdx.x == 0) {
          const bool ok = wait_counter_ge(&ls->arrive[parity], push.tail_expect);
          tail_ok = ok ? 1 : 0;
          if (!ok && status) atomicCAS(status, 0, kStatusTimeoutPeer);
        }
        __syncthreads();
        const int n_cta = gridDim.x * gridDim.y * gridDim.z;
        if (tail_ok) {
          ReduceNormArgs b = push.red;
          b.slots = push.red.slots + size_t(parity) * b.world * b.slot_stride;
          const int lin = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
          for (int row = lin; row < b.M; row += n_cta) {
            reduce_norm_row(b, row, tail_red);
            __syncthreads();
          }
        }
        channel_finish(lsm, parity, unsigned(n_cta));
      }
    }
    if (!pushed) {
      epilogue_pass<TN>(ep, reinterpret_cast<const float*>(smem), smem_u32(smem), LDS, m0, n0,
                        split * rows_per_cta, rows_per_cta, nsplit, warp, lane, kThreads / 32);
    }
  } else if (threadIdx.x == 0) {
    if (status) atomicCAS(status, 0, err);
    // let copies that are still in flight land before the block goes away
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) { __nanosleep(1000); }
  }

  if (tr && threadIdx.x == 0) tr[5] = globaltimer_ns();
  if (nsplit > 1) cluster_sync_all();  // peers may still be reading this CTA's staging tile
  if (tr && threadIdx.x == 0) tr[6] = globaltimer_ns();
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
  if constexpr (COMM) if (push.wait_channel >= 0) {
    ChannelSig* ws = const_cast<ChannelSig*>(reinterpret_cast<const ChannelSig*>(push.local_sig)) + push.wait_channel;
    const int wp = int(ld_relaxed_sys(&ws->epoch) & 1u);  // unchanged until every CTA took its ticket
    channel_finish(ws, wp, gridDim.x * gridDim.y * gridDim.z);
  }
}

// ------------------------------------------------------------ host: TMA maps
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

struct TmapKey {
  const void* ptr;
  uint64_t rows, cols, ld;
  uint32_t box_rows, elem;
  bool operator==(const TmapKey& o) const {
    return ptr == o.ptr && rows == o.rows && cols == o.cols && ld == o.ld &&
           box_rows == o.box_rows && elem == o.elem;
  }
};
struct TmapKeyHash {
  size_t operator()(const TmapKey& k) const {
    size_t h = reinterpret_cast<size_t>(k.ptr);
    auto mix = [&h](uint64_t v) { h ^= v + 0x9e3779b97f4a7c15ull + (h << 6) + (h >> 2); };
    mix(k.rows); mix(k.cols); mix(k.ld); mix(k.box_rows); mix(k.elem);
    return h;
  }
};

// 2-D K-major operand [rows, cols] with row stride ld (elements), box = 128 bytes x box_rows.
bool make_tmap_2d(CUtensorMap* out, const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld,
                  uint32_t box_rows, uint32_t elem_bytes) {
  static std::mutex mu;
  static std::unordered_map<TmapKey, CUtensorMap, TmapKeyHash> cache;
  TmapKey key{ptr, rows, cols, ld, box_rows, elem_bytes};
  {
    std::lock_guard<std::mutex> g(mu);
    auto it = cache.find(key);
    if (it != cache.end()) { *out = it->second; return true; }
  }
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) return false;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * elem_bytes};
  cuuint32_t box[2] = {uint32_t(kRowBytes / elem_bytes), box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                           : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  CUresult r = enc(out, dt, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return false;
  std::lock_guard<std::mutex> g(mu);
  if (cache.size() > 65536) cache.clear();
  cache.emplace(key, *out);
  return true;
}

// 3-D bf16 view (d, head, row): extents {D, H, R}, byte strides {head_stride, row_stride};
// box = 64 elements x box_h heads x box_r rows, 128-byte swizzle, zero fill outside.
bool make_tmap_3d_bf16(CUtensorMap* out, const void* ptr, uint64_t D, uint64_t H, uint64_t R,
                       uint64_t head_stride_elems, uint64_t row_stride_elems, uint32_t box_h,
                       uint32_t box_r) {
  struct K3 { const void* p; uint64_t d, h, r, hs, rs; uint32_t bh, br; };
  static std::mutex mu;
  static std::vector<std::pair<K3, CUtensorMap>> cache;
  {
    std::lock_guard<std::mutex> g(mu);
    for (auto& e : cache) {
      const K3& k = e.first;
      if (k.p == ptr && k.d == D && k.h == H && k.r == R && k.hs == head_stride_elems &&
          k.rs == row_stride_elems && k.bh == box_h && k.br == box_r) { *out = e.second; return true; }
    }
  }
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) return false;
  cuuint64_t dims[3] = {D, H, R};
  cuuint64_t strides[2] = {head_stride_elems * 2, row_stride_elems * 2};
  cuuint32_t box[3] = {64, box_h, box_r};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides,
                   box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return false;
  std::lock_guard<std::mutex> g(mu);
  if (cache.size() > 4096) cache.clear();
  cache.push_back({K3{ptr, D, H, R, head_stride_elems, row_stride_elems, box_h, box_r}, *out});
  return true;
}

// ---------------------------------------------------------------- host: launch
template <int BN, bool SWAP, bool FP8>
static cudaError_t launch_inst(const CUtensorMap& tmP, const CUtensorMap& tmQ, const EpiParams& ep,
                               const PushParams& push, dim3 grid, int total_kb, int kbps, int stages, size_t smem,
                               cudaStream_t stream, unsigned long long* trace) {
  if (push.world > 0 || push.wait_channel >= 0) {
    auto kern = gemm_kernel<BN, SWAP, FP8, true>;
    static bool attr_done = false;
    if (!attr_done) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
      if (e != cudaSuccess) return e;
      attr_done = true;
    }
    return launch_kernel(kern, grid, dim3(kThreads), smem, stream, int(grid.z), tmP, tmQ, ep, push, total_kb,
                         kbps, stages, kernel_status_ptr(), trace);
  }
  auto kern = gemm_kernel<BN, SWAP, FP8, false>;
  static bool attr_done = false;
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return e;
    attr_done = true;
  }
  NoComm none{-1, 0};
  return launch_kernel(kern, grid, dim3(kThreads), smem, stream, int(grid.z), tmP, tmQ, ep, none, total_kb,
                       kbps, stages, kernel_status_ptr(), trace);
}

template <bool SWAP, bool FP8>
static cudaError_t launch_bn(int bn, const CUtensorMap& tmP, const CUtensorMap& tmQ,
                             const EpiParams& ep, const PushParams& push, dim3 grid, int total_kb,
                             int kbps, int stages, size_t smem, cudaStream_t st,
                             unsigned long long* tr) {
  switch (bn) {
    case 16: return launch_inst<16, SWAP, FP8>(tmP, tmQ, ep, push, grid, total_kb, kbps, stages, smem, st, tr);
    case 32: return launch_inst<32, SWAP, FP8>(tmP, tmQ, ep, push, grid, total_kb, kbps, stages, smem, st, tr);
    case 64: return launch_inst<64, SWAP, FP8>(tmP, tmQ, ep, push, grid, total_kb, kbps, stages, smem, st, tr);
    case 128: return launch_inst<128, SWAP, FP8>(tmP, tmQ, ep, push, grid, total_kb, kbps, stages, smem, st, tr);
    case 192:
      if constexpr (!SWAP && !FP8) return launch_inst<192, SWAP, FP8>(tmP, tmQ, ep, push, grid, total_kb, kbps, stages, smem, st, tr);
      else return cudaErrorInvalidValue;
    case 256: return launch_inst<256, SWAP, FP8>(tmP, tmQ, ep, push, grid, total_kb, kbps, stages, smem, st, tr);
    default: return cudaErrorInvalidValue;
  }
}

static int num_sms() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

cudaError_t gemm_launch(const GemmArgs& a, cudaStream_t stream, int* n_ctas) {
  const int eb = a.fp8 ? 1 : 2;
  const int BK = a.fp8 ? 128 : 64;
  if (a.M <= 0 || a.N <= 0 || a.K <= 0) return cudaErrorInvalidValue;
  if (a.tail_done) *a.tail_done = 0;
  // TMA: 16-byte aligned base and row strides; vector epilogue: N multiple of 8.
  if ((reinterpret_cast<uintptr_t>(a.x) & 15) || (reinterpret_cast<uintptr_t>(a.w) & 15) ||
      (size_t(a.ldx) * eb) % 16 || (size_t(a.ldw) * eb) % 16 || (a.N % 8) ||
      (reinterpret_cast<uintptr_t>(a.out) & 15) || (a.ldo % 4))
    return cudaErrorInvalidValue;
  // the epilogue reads bias / gate / residual as 8-byte vectors, scales as 16-byte vectors
  if ((reinterpret_cast<uintptr_t>(a.bias) & 7) || (reinterpret_cast<uintptr_t>(a.col_gate) & 7) ||
      (reinterpret_cast<uintptr_t>(a.residual) & 7) || (a.residual && (a.ldr % 4)) ||
      (reinterpret_cast<uintptr_t>(a.w_scale) & 15))
    return cudaErrorInvalidValue;
  if (a.block_scaled) return cudaErrorInvalidValue;  // handled by gemm_fp8_block_launch
  if (!a.out2 && gemm_2cta_eligible(a)) {
    const cudaError_t e = gemm_2cta_launch(a, stream);
    if (e != cudaErrorInvalidClusterSize) return e;
    cudaGetLastError();   // pairs cannot be scheduled in this context (e.g. an SM partition): use one CTA per tile set
    set_gemm_2cta(0);
  }
  if (!a.out2 && gemm_persist_eligible(a)) {
    if (a.push && (a.push->world < 0 || a.push->world > kMaxRanks ||
                   (a.push->world > 0 && (a.glu || a.act || a.bias || a.residual || a.col_gate)) ||
                   (a.push->world > 0 && a.push->rows_per_rank > 0 &&
                    (a.M + a.push->rows_per_rank - 1) / a.push->rows_per_rank > a.push->world)))
      return cudaErrorInvalidValue;
    return gemm_persist_launch(a, stream, n_ctas);
  }

  // K split over a cluster when the tiles alone leave more than half of the SMs idle. Tiles of up to 128 columns keep
  // their stages under 100 KB, so two CTAs fit on an SM: there one more doubling is taken while every CTA still gets
  // four K blocks (50 x 1024 -> 8192: 9.8 -> 8.2 us with 256 CTAs instead of 128).
  const auto pick_splits = [](int ctas, int total_kb, int bn) {
    int splits = 1;
    if (ctas * 2 <= num_sms()) {
      splits = 8;
      while (splits > 1 && (ctas * splits > num_sms() || total_kb / splits < 2)) splits >>= 1;
    }
    int kbps = (total_kb + splits - 1) / splits;
    while (splits > 1 && (total_kb + kbps - 1) / kbps != splits) {
      splits >>= 1;
      kbps = (total_kb + splits - 1) / splits;
    }
    if (bn <= 128 && splits < 8 && ctas * 2 <= num_sms() && ctas * splits * 2 <= 2 * num_sms() && total_kb / (splits * 2) >= 4 &&
        total_kb % (splits * 2) == 0)
      splits *= 2;
    return splits;
  };
  int mid_splits = 0;      // > 0: K split chosen together with the tile width for mid-size problems
  bool swap = a.M <= 256;
  if (a.force_swap == 0) swap = false;
  if (a.force_swap == 1) swap = true;
  int bn;
  if (swap) {
    bn = 16;
    while (bn < a.M && bn < 256) bn <<= 1;
  } else {
    bn = a.N >= 2048 && a.M >= 512 ? 256 : 128;
    if (a.N <= 64) bn = 64;
    if (a.N <= 32) bn = 32;
    if (a.M >= 512 && a.N >= 512 && !a.fp8 && a.force_bn == 0 && a.force_splits == 0) {
      // Mid-size problems are a wave or two of tiles: pick the tile width (128 / 192 / 256) whose
      // waves x K blocks per CTA x cycles per K block is smallest, i.e. the one that wastes the fewest
      // SM-cycles on a partial last wave (768 x 3456: 84 tiles of 256 or 162 of 128 cost about the same,
      // 108 of 192 a sixth less). Cycles per K block: the slower of the MMAs (2 cycles per column) and the
      // operand ingest ((128 + width) x 128 bytes at about 96 bytes per cycle), so narrow tiles pay for
      // their lower arithmetic intensity.
      const int p_t = (a.M + kTileP - 1) / kTileP, kb = (a.K + BK - 1) / BK;
      if (p_t <= 8 && a.K < 8192 && !a.push) {
        // Up to about a thousand rows with a short or medium K (vision tower, prefix QKV / o-proj): measured sweep of
        // tile width x K split inside a CUDA graph. 128-wide tiles win throughout: their stages fit twice on an SM, so
        // up to 2 x 148 CTAs are resident at once, and where the tiles alone leave that under-filled K is split over a
        // cluster until they fill it (768 x 1152 -> 1152: 20.3 -> 10.1 us; 768 x 4304 -> 1152: 29.6 -> 16.7 us;
        // 968 x 2048 -> 2048: 17.1 -> 14.1 us; the wide shapes gain 1.5-2 us from the narrower tile alone). Every split
        // keeps at least eight K blocks. Products that leave through the peer epilogue keep the wave model below: on
        // tensor-parallel shards (K of 512-4096 per rank, one arrival per CTA and rank) the extra CTAs cost more than
        // they hide (a four-GPU request went from 15.9 to 16.3 ms with them).
        bn = 128;
        const int tiles = p_t * ((a.N + 127) / 128);
        int sp = 1;
        while (sp < 8 && tiles * sp * 2 <= 2 * num_sms() && kb / (sp * 2) >= 8) sp *= 2;
        mid_splits = sp;
      } else {
        long best = -1;
        for (int cand : {256, 192, 128}) {
          const int ctas_c = p_t * ((a.N + cand - 1) / cand);
          const int sp = pick_splits(ctas_c, kb, cand);
          const int waves = (ctas_c * sp + num_sms() - 1) / num_sms();
          const int per_kb = cand == 256 ? 512 : cand == 192 ? 427 : 341;
          const long cost = long(waves) * ((kb + sp - 1) / sp + (sp > 1 ? 3 : 1)) * per_kb;   // + fixed per-CTA work (cluster reduce when split)
          if (best < 0 || cost < best) { best = cost; bn = cand; }
        }
      }
    }
  }
  if (a.force_bn) bn = a.force_bn;
  if (a.glu && !swap && bn < 16) return cudaErrorInvalidValue;

  const int p_rows = swap ? a.N : a.M, q_rows = swap ? a.M : a.N;
  const int p_tiles = (p_rows + kTileP - 1) / kTileP;
  const int q_tiles = (q_rows + bn - 1) / bn;
  const int total_kb = (a.K + BK - 1) / BK;
  const int ctas = p_tiles * q_tiles;

  int splits = a.force_splits > 0 ? a.force_splits : (mid_splits > 0 && !a.force_bn ? mid_splits : pick_splits(ctas, total_kb, bn));
  int kbps = (total_kb + splits - 1) / splits;
  while (splits > 1 && (total_kb + kbps - 1) / kbps != splits) {
    splits >>= 1;
    kbps = (total_kb + splits - 1) / splits;
  }
  const int tm = swap ? bn : kTileP;
  if (tm % splits) return cudaErrorInvalidValue;

  const int stage_bytes = kTileP * kRowBytes + bn * kRowBytes;
  const int tn = swap ? kTileP : bn;
  const size_t staging = size_t(tm) * (tn + 4) * 4;
  int stages = kMaxStages;
  const size_t budget = (ctas * splits > num_sms() && bn <= 128) ? 100 * 1024 : 196 * 1024;
  while (stages > 2 && size_t(stages) * stage_bytes > budget) --stages;
  if (stages > kbps) stages = kbps < 2 ? 2 : kbps;
  size_t smem = size_t(stages) * stage_bytes;
  if (smem < staging) smem = staging;
  smem += 1024;  // alignment slack
  if (smem > 200 * 1024) return cudaErrorInvalidValue;

  CUtensorMap tmP, tmQ;
  const void* p_ptr = swap ? a.w : a.x;
  const void* q_ptr = swap ? a.x : a.w;
  const int p_ld = swap ? a.ldw : a.ldx, q_ld = swap ? a.ldx : a.ldw;
  if (!make_tmap_2d(&tmP, p_ptr, p_rows, a.K, p_ld, kTileP, eb)) return cudaErrorInvalidValue;
  if (!make_tmap_2d(&tmQ, q_ptr, q_rows, a.K, q_ld, bn, eb)) return cudaErrorInvalidValue;

  EpiParams ep;
  ep.out = a.out; ep.ldo = a.ldo; ep.M = a.M; ep.N = a.N;
  ep.bias = a.bias; ep.residual = a.residual; ep.ldr = a.ldr; ep.res_mod = a.res_mod;
  ep.col_gate = a.col_gate; ep.row_scale = a.row_scale; ep.sumsq = a.sumsq;
  ep.a_scale = a.a_scale; ep.w_scale = a.w_scale;
  ep.act = a.act; ep.glu = a.glu; ep.out_fp32 = a.out_fp32;
  ep.rs_inv_dim = a.row_rms_dim > 0 ? 1.f / float(a.row_rms_dim) : 0.f; ep.rs_eps = a.row_rms_eps;
  ep.rope = a.rope; ep.zero = a.zero; ep.zero_n = a.zero_n;
  ep.out2 = a.out2; ep.col_scale2 = a.col_scale2; ep.ldo2 = a.ldo2;
  if (a.out2 && (a.glu || a.out_fp32 || a.rope || a.push || !a.col_scale2 || (a.ldo2 % 4) ||
                 (reinterpret_cast<uintptr_t>(a.out2) & 7) || (reinterpret_cast<uintptr_t>(a.col_scale2) & 7)))
    return cudaErrorInvalidValue;
#ifdef PHYAI_DEBUG
  ep.status = kernel_status_ptr();
#endif
  if (a.rope && (a.glu || a.act || a.residual || a.col_gate || a.sumsq || a.fp8 || a.out_fp32)) return cudaErrorInvalidValue;

  PushParams push;
  memset(&push, 0, sizeof(push));
  push.wait_channel = -1;
  if (a.push) {
    // the consumer adds bias / residual / norm; a push-mode product is the bare partial sum
    if (a.push->world < 0 || a.push->world > kMaxRanks ||
        (a.push->world > 0 && (a.glu || a.act || a.bias || a.residual || a.col_gate || a.row_scale ||
                               a.sumsq || a.fp8 || (a.push->ld % 4))))
      return cudaErrorInvalidValue;
    if (a.push->world > 0 && a.push->rows_per_rank > 0 &&
        (a.M + a.push->rows_per_rank - 1) / a.push->rows_per_rank > a.push->world)
      return cudaErrorInvalidValue;
    push = *a.push;
  }
  dim3 grid(p_tiles, q_tiles, splits);
  if (n_ctas) *n_ctas = p_tiles * q_tiles * splits;
  if (push.tail) {
    // the tail waits on this grid's own CTAs: only when all of them (clusters included) are resident together
    if (p_tiles * q_tiles * splits > kTailMaxCtas || push.world <= 0 || push.rows_per_rank > 0) push.tail = 0;
    else push.tail_expect = unsigned(p_tiles * q_tiles * splits) * unsigned(push.world);
  }
  if (a.tail_done) *a.tail_done = push.tail;
  if (swap) {
    return a.fp8 ? launch_bn<true, true>(bn, tmP, tmQ, ep, push, grid, total_kb, kbps, stages, smem, stream, a.trace)
                 : launch_bn<true, false>(bn, tmP, tmQ, ep, push, grid, total_kb, kbps, stages, smem, stream, a.trace);
  }
  return a.fp8 ? launch_bn<false, true>(bn, tmP, tmQ, ep, push, grid, total_kb, kbps, stages, smem, stream, a.trace)
               : launch_bn<false, false>(bn, tmP, tmQ, ep, push, grid, total_kb, kbps, stages, smem, stream, a.trace);
}

}  // namespace pb

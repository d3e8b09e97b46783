// Memory-bound kernels for sm_100a: every one is a single pass over its rows with
// 16-byte vector accesses and fp32 arithmetic. They cover what the reference runs
// through Triton / FlashInfer / ATen:
//   norms            phyai-kernel/phyai_kernel/triton/{rms_norm,layer_norm,ada_rms_norm}.py
//   RoPE + KV write  phyai/src/phyai/layers/rotary_embedding.py:520-578,
//                    phyai/src/phyai/cache/kv_cache_pool.py:139-182 (two index_put_)
//   masked embedding phyai-kernel/phyai_kernel/triton/masked_embedding.py:35-77
//   gated act        phyai/src/phyai/layers/mlp/dense_mlp.py:87-108
//   Euler / CFG      phyai/src/phyai/models/pi05/model_runner_pi05.py:735-737,
//                    phyai/src/phyai/models/cosmos3/scheduler_wn_cosmos3.py:228
#include "ops.cuh"

#include <cuda_fp8.h>

#include <cstdlib>

#include "gemm.cuh"
#include "launch.cuh"
#include "ptx.cuh"

#define PB_LAUNCH(kern, grid, block, stream, ...)                                           \
  do {                                                                                    \
    cudaError_t e__ = launch_kernel(kern, dim3(grid), dim3(block), 0, stream, 1, __VA_ARGS__); \
    if (e__ != cudaSuccess) return e__;                                                   \
  } while (0)

namespace pb {

namespace {

// Eight bf16 values moved as one 16-byte word (a plain aggregate of four 32-bit words, so copies are single
// 128-bit loads / stores). Widening to fp32 is a shift / mask of the bit pattern on the integer pipe: the
// conversion instruction shares the 16-per-clock special-function pipe, which a profile of the many-row norm
// showed as its busiest unit (140 % of sustained peak) while DRAM sat at 42 %.
struct alignas(16) BF8 {
  uint32_t u[4];
};

__device__ __forceinline__ void unpack8(const BF8& b, float (&f)[8]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(b.u[i] << 16);
    f[2 * i + 1] = __uint_as_float(b.u[i] & 0xffff0000u);
  }
}
__device__ __forceinline__ BF8 pack8(const float (&f)[8]) {
  BF8 b;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    b.u[i] = *reinterpret_cast<const uint32_t*>(&h);
  }
  return b;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// Block-wide sum; red must hold 32 floats. Every thread gets the result.
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  const int nw = (blockDim.x + 31) >> 5;
  float t = lane < nw ? red[lane] : 0.f;
  return warp_sum(t);
}
__device__ __forceinline__ float block_max(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  const int nw = (blockDim.x + 31) >> 5;
  float t = lane < nw ? red[lane] : -INFINITY;
  return warp_max(t);
}

}  // namespace

// ---------------------------------------------------------------------- norms
template <int MODE>
__global__ void norm_kernel(NormArgs a) {
  __shared__ float red[32];
  const int row = blockIdx.x;
  const int nv = a.D >> 3;
  pdl_launch_dependents();
  pdl_wait();
  const BF8* xr = reinterpret_cast<const BF8*>(a.x + size_t(row) * a.ldx);
  BF8* rr = a.residual ? reinterpret_cast<BF8*>(a.residual + size_t(row) * a.ldr) : nullptr;
  BF8* yr = reinterpret_cast<BF8*>(a.y + size_t(row) * a.ldy);

  // pass 1: (optional residual add, written back) + moments
  float s1 = 0.f, s2 = 0.f;
  for (int v = threadIdx.x; v < nv; v += blockDim.x) {
    float f[8];
    unpack8(xr[v], f);
    if (rr) {
      float g[8];
      unpack8(rr[v], g);
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] += g[i];
      BF8 h = pack8(f);
      rr[v] = h;
      unpack8(h, f);  // the norm sees the rounded sum, as a separate add kernel would produce
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) { s1 += f[i]; s2 += f[i] * f[i]; }
  }
  float mean = 0.f, rstd;
  if (MODE == kNormLayer) {
    s1 = block_sum(s1, red);
    s2 = block_sum(s2, red);
    mean = s1 / a.D;
    const float var = fmaxf(s2 / a.D - mean * mean, 0.f);
    rstd = rsqrtf(var + a.eps);
  } else {
    if (a.sumsq && !rr) s2 = a.sumsq[row]; else s2 = block_sum(s2, red);
    rstd = rsqrtf(s2 / a.D + a.eps);
  }
  const BF8* src = rr ? rr : xr;
  const BF8* wv = a.weight ? reinterpret_cast<const BF8*>(a.weight) : nullptr;
  const BF8* bv = a.bias ? reinterpret_cast<const BF8*>(a.bias) : nullptr;
  const BF8* mv = nullptr;
  if (MODE == kNormAdaRms) mv = reinterpret_cast<const BF8*>(a.mod + size_t(row / a.group) * 3 * a.D);

  float amax = 0.f;
  for (int v = threadIdx.x; v < nv; v += blockDim.x) {
    float f[8], o[8];
    unpack8(src[v], f);
    if (MODE == kNormLayer) {
      float w[8], b[8];
      unpack8(wv[v], w);
      unpack8(bv[v], b);
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = (f[i] - mean) * rstd * w[i] + b[i];
    } else if (MODE == kNormAdaRms) {
      float sc[8], sh[8];
      unpack8(mv[v], sc);
      unpack8(mv[nv + v], sh);
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = f[i] * rstd * (1.f + sc[i]) + sh[i];
    } else if (MODE == kNormRmsNoWeight) {
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = f[i] * rstd;
    } else {
      float w[8];
      unpack8(wv[v], w);
#pragma unroll
      for (int i = 0; i < 8; ++i)
        o[i] = f[i] * rstd * (MODE == kNormGemmaRms ? 1.f + w[i] : w[i]);
    }
    const BF8 packed = pack8(o);
    if (a.y) yr[v] = packed;
    if (a.y8) {
      float q8[8];
      unpack8(packed, q8);  // the fp8 copy quantises the rounded bf16 values
#pragma unroll
      for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(q8[i]));
    }
  }
  if (a.y8) {
    // second sweep for the fp8 copy: per-row scale, or one scale per 128 columns
    if (a.y8_block == 0) {
      amax = block_max(amax, red);
      const float sc = fmaxf(amax, 1e-12f) / 448.f;
      if (threadIdx.x == 0) a.y8_scale[row] = sc;
      const float inv = 1.f / sc;
      for (int v = threadIdx.x; v < nv; v += blockDim.x) {
        float o[8];
        unpack8(yr[v], o);
        uint8_t q[8];
#pragma unroll
        for (int i = 0; i < 8; ++i)
          q[i] = __nv_cvt_float_to_fp8(o[i] * inv, __NV_SATFINITE, __NV_E4M3);
        *reinterpret_cast<uint2*>(a.y8 + size_t(row) * a.D + v * 8) =
            *reinterpret_cast<uint2*>(q);
      }
    } else {
      // 16 consecutive threads own one 128-column block
      __syncthreads();
      const int nb = a.D >> 7;
      for (int v0 = 0; v0 < nv; v0 += blockDim.x) {
        const int v = v0 + threadIdx.x;
        float o[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        if (v < nv) unpack8(yr[v], o);
        float m = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) m = fmaxf(m, fabsf(o[i]));
#pragma unroll
        for (int off = 8; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
        const float sc = fmaxf(m, 1e-12f) / 448.f;
        if (v < nv) {
          if ((v & 15) == 0) a.y8_scale[size_t(row) * nb + (v >> 4)] = sc;
          const float inv = 1.f / sc;
          uint8_t q[8];
#pragma unroll
          for (int i = 0; i < 8; ++i)
            q[i] = __nv_cvt_float_to_fp8(o[i] * inv, __NV_SATFINITE, __NV_E4M3);
          *reinterpret_cast<uint2*>(a.y8 + size_t(row) * a.D + v * 8) =
              *reinterpret_cast<uint2*>(q);
        }
      }
    }
  }
}

// Many-row variant: one WARP per row, eight rows per CTA, no shared memory and no block barrier.
// The block-per-row kernel above is shaped for a handful of rows (latency); with thousands of
// rows its barrier and shared-memory reduction dominate, while here a warp streams its row with
// 512-byte coalesced accesses, reduces with shuffles and re-reads the row (an L1 / L2 hit) for
// the second pass. RMS family only (no LayerNorm moments, no fp8 copy, no precomputed sums).
template <int MODE>
__global__ void norm_rows_kernel(NormArgs a) {
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  pdl_launch_dependents();
  pdl_wait();
  if (row >= a.rows) return;
  const int nv = a.D >> 3;
  const BF8* xr = reinterpret_cast<const BF8*>(a.x + size_t(row) * a.ldx);
  BF8* rr = a.residual ? reinterpret_cast<BF8*>(a.residual + size_t(row) * a.ldr) : nullptr;
  BF8* yr = reinterpret_cast<BF8*>(a.y + size_t(row) * a.ldy);
  float s2 = 0.f;
  for (int v = lane; v < nv; v += 32) {
    float f[8];
    unpack8(xr[v], f);
    if (rr) {
      float g[8];
      unpack8(rr[v], g);
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] += g[i];
      const BF8 h = pack8(f);
      rr[v] = h;
      unpack8(h, f);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) s2 += f[i] * f[i];
  }
  s2 = warp_sum(s2);
  const float rstd = rsqrtf(s2 / a.D + a.eps);
  const BF8* src = rr ? rr : xr;
  const BF8* wv = a.weight ? reinterpret_cast<const BF8*>(a.weight) : nullptr;
  const BF8* mv = MODE == kNormAdaRms ? reinterpret_cast<const BF8*>(a.mod + size_t(row / a.group) * 3 * a.D) : nullptr;
  for (int v = lane; v < nv; v += 32) {
    float f[8], o[8];
    unpack8(src[v], f);
    if (MODE == kNormAdaRms) {
      float sc[8], sh[8];
      unpack8(mv[v], sc);
      unpack8(mv[nv + v], sh);
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = f[i] * rstd * (1.f + sc[i]) + sh[i];
    } else if (MODE == kNormRmsNoWeight) {
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = f[i] * rstd;
    } else {
      float w[8];
      unpack8(wv[v], w);
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = f[i] * rstd * (MODE == kNormGemmaRms ? 1.f + w[i] : w[i]);
    }
    yr[v] = pack8(o);
  }
}

// Register-resident variant of the above for rows of at most 256 * NVL elements. Warps are persistent and
// walk the rows with a grid stride; a lane issues all of its 16-byte loads of the NEXT row (NVL independent
// loads) before it reduces, scales and stores the current one from registers, so every warp has a full row
// of loads in flight at all times: one read and one write per element, and the memory queue stays full
// without relying on occupancy.
template <int MODE, int NVL>
__global__ void __launch_bounds__(256) norm_rows_reg_kernel(NormArgs a) {
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  const int stride = gridDim.x * wpb;
  int row = blockIdx.x * wpb + (threadIdx.x >> 5);
  pdl_launch_dependents();
  pdl_wait();
  if (row >= a.rows) return;
  const int nv = a.D >> 3;
  const BF8* wv = a.weight ? reinterpret_cast<const BF8*>(a.weight) : nullptr;
  BF8 nx[NVL];
  {
    const BF8* xr = reinterpret_cast<const BF8*>(a.x + size_t(row) * a.ldx);
#pragma unroll
    for (int j = 0; j < NVL; ++j) {
      const int v = lane + 32 * j;
      if (v < nv) nx[j] = xr[v];
    }
  }
  for (; row < a.rows; row += stride) {
    BF8 xv[NVL];
#pragma unroll
    for (int j = 0; j < NVL; ++j) xv[j] = nx[j];
    const int next = row + stride;
    if (next < a.rows) {
      const BF8* xr = reinterpret_cast<const BF8*>(a.x + size_t(next) * a.ldx);
#pragma unroll
      for (int j = 0; j < NVL; ++j) {
        const int v = lane + 32 * j;
        if (v < nv) nx[j] = xr[v];
      }
    }
    BF8* yr = reinterpret_cast<BF8*>(a.y + size_t(row) * a.ldy);
    if (a.residual) {
      BF8* rr = reinterpret_cast<BF8*>(a.residual + size_t(row) * a.ldr);
#pragma unroll
      for (int j = 0; j < NVL; ++j) {
        const int v = lane + 32 * j;
        if (v < nv) {
          float f[8], g[8];
          unpack8(xv[j], f);
          unpack8(rr[v], g);
#pragma unroll
          for (int i = 0; i < 8; ++i) f[i] += g[i];
          xv[j] = pack8(f);        // the norm sees the rounded sum, as a separate add kernel would produce
          rr[v] = xv[j];
        }
      }
    }
    float s2 = 0.f;
#pragma unroll
    for (int j = 0; j < NVL; ++j) {
      if (lane + 32 * j < nv) {
        float f[8];
        unpack8(xv[j], f);
#pragma unroll
        for (int i = 0; i < 8; ++i) s2 += f[i] * f[i];
      }
    }
    s2 = warp_sum(s2);
    const float rstd = rsqrtf(s2 / a.D + a.eps);
    const BF8* mv = MODE == kNormAdaRms ? reinterpret_cast<const BF8*>(a.mod + size_t(row / a.group) * 3 * a.D) : nullptr;
#pragma unroll
    for (int j = 0; j < NVL; ++j) {
      const int v = lane + 32 * j;
      if (v < nv) {
        float f[8], o[8];
        unpack8(xv[j], f);
        if (MODE == kNormAdaRms) {
          float sc[8], sh[8];
          unpack8(mv[v], sc);
          unpack8(mv[nv + v], sh);
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] = f[i] * rstd * (1.f + sc[i]) + sh[i];
        } else if (MODE == kNormRmsNoWeight) {
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] = f[i] * rstd;
        } else {
          float w[8];
          unpack8(wv[v], w);
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] = f[i] * rstd * (MODE == kNormGemmaRms ? 1.f + w[i] : w[i]);
        }
        yr[v] = pack8(o);
      }
    }
  }
}

// Streaming variant for tens of thousands of rows: persistent CTAs, a dedicated warp moves groups of
// eight rows global -> shared memory with bulk asynchronous copies (one instruction per group when the
// rows are contiguous) into a ring of stages, so the copy engine keeps the DRAM queue full with no
// per-thread load instructions outstanding. Eight consumer warps take one row each: the row goes from
// shared memory into registers, the stage is handed back at once, and the warp reduces, scales and
// stores from registers. No residual input (that variant stays on norm_rows_reg_kernel).
constexpr int kNormTmaRows = 8;
template <int MODE, int NVL>
__global__ void __launch_bounds__(288) norm_rows_tma_kernel(NormArgs a, int stages, int* status) {
  extern __shared__ uint8_t nsm_raw[];
  uint8_t* sm = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(nsm_raw) + 127) & ~uintptr_t(127));
  __shared__ __align__(8) uint64_t full_bar[4], empty_bar[4];
  __shared__ volatile int err_s;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row_bytes = a.D * 2, stage_bytes = kNormTmaRows * row_bytes;
  const int n_groups = (a.rows + kNormTmaRows - 1) / kNormTmaRows;
  const bool contiguous = a.ldx == a.D;
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], kNormTmaRows); }
    err_s = 0;
    mbar_fence_init();
  }
  __syncthreads();
  pdl_launch_dependents();
  pdl_wait();
  if (warp == kNormTmaRows) {
    // ------------------------------------------------------------------ copy warp
    if (lane == 0) {
      int it = 0;
      for (int g = blockIdx.x; g < n_groups && !err_s; g += gridDim.x, ++it) {
        const int s = it % stages;
        if (it >= stages && !mbar_wait(&empty_bar[s], uint32_t((it / stages) & 1) ^ 1)) { err_s = kStatusTimeoutEmpty; break; }
        const int r0 = g * kNormTmaRows, nr = min(kNormTmaRows, a.rows - r0);
        mbar_expect_tx(&full_bar[s], uint32_t(nr * row_bytes));
        uint8_t* dst = sm + size_t(s) * stage_bytes;
        if (contiguous) {
          bulk_load(dst, a.x + size_t(r0) * a.ldx, uint32_t(nr * row_bytes), &full_bar[s]);
        } else {
          for (int r = 0; r < nr; ++r) bulk_load(dst + r * row_bytes, a.x + size_t(r0 + r) * a.ldx, uint32_t(row_bytes), &full_bar[s]);
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ one row per warp and group
    const int nv = a.D >> 3;
    const BF8* wv = a.weight ? reinterpret_cast<const BF8*>(a.weight) : nullptr;
    int it = 0;
    for (int g = blockIdx.x; g < n_groups && !err_s; g += gridDim.x, ++it) {
      const int s = it % stages;
      if (!mbar_wait(&full_bar[s], uint32_t((it / stages) & 1))) { err_s = kStatusTimeoutFull; break; }
      const int row = g * kNormTmaRows + warp;
      const bool live = row < a.rows;
      BF8 xv[NVL];
      if (live) {
        const BF8* xs = reinterpret_cast<const BF8*>(sm + size_t(s) * stage_bytes + size_t(warp) * row_bytes);
#pragma unroll
        for (int j = 0; j < NVL; ++j) {
          const int v = lane + 32 * j;
          if (v < nv) xv[j] = xs[v];
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty_bar[s]);     // the row is in registers: the stage can be refilled
      if (!live) continue;
      float s2 = 0.f;
#pragma unroll
      for (int j = 0; j < NVL; ++j) {
        if (lane + 32 * j < nv) {
          float f[8];
          unpack8(xv[j], f);
#pragma unroll
          for (int i = 0; i < 8; ++i) s2 += f[i] * f[i];
        }
      }
      s2 = warp_sum(s2);
      const float rstd = rsqrtf(s2 / a.D + a.eps);
      const BF8* mv = MODE == kNormAdaRms ? reinterpret_cast<const BF8*>(a.mod + size_t(row / a.group) * 3 * a.D) : nullptr;
      BF8* yr = reinterpret_cast<BF8*>(a.y + size_t(row) * a.ldy);
#pragma unroll
      for (int j = 0; j < NVL; ++j) {
        const int v = lane + 32 * j;
        if (v < nv) {
          float f[8], o[8];
          unpack8(xv[j], f);
          if (MODE == kNormAdaRms) {
            float sc[8], sh[8];
            unpack8(mv[v], sc);
            unpack8(mv[nv + v], sh);
#pragma unroll
            for (int i = 0; i < 8; ++i) o[i] = f[i] * rstd * (1.f + sc[i]) + sh[i];
          } else if (MODE == kNormRmsNoWeight) {
#pragma unroll
            for (int i = 0; i < 8; ++i) o[i] = f[i] * rstd;
          } else {
            float w[8];
            unpack8(wv[v], w);
#pragma unroll
            for (int i = 0; i < 8; ++i) o[i] = f[i] * rstd * (MODE == kNormGemmaRms ? 1.f + w[i] : w[i]);
          }
          yr[v] = pack8(o);
        }
      }
    }
  }
  __syncthreads();
  if (err_s && threadIdx.x == 0) {
    if (status) atomicCAS(status, 0, int(err_s));
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);   // let copies in flight land
  }
}

template <int MODE, int NVL>
static cudaError_t launch_norm_tma(const NormArgs& a, cudaStream_t s) {
  const int stage_bytes = kNormTmaRows * a.D * 2;
  int stages = (200 * 1024) / stage_bytes;
  if (stages > 4) stages = 4;
  const size_t smem = size_t(stages) * stage_bytes + 128;
  auto kern = norm_rows_tma_kernel<MODE, NVL>;
  static bool attr_done = false;
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 201 * 1024);
    if (e != cudaSuccess) return e;
    attr_done = true;
  }
  int sms = 148, dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int n_groups = (a.rows + kNormTmaRows - 1) / kNormTmaRows;
  const int grid = n_groups < sms ? n_groups : sms;
  return launch_kernel(kern, dim3(grid), dim3(288), smem, s, 1, a, stages, kernel_status_ptr());
}

template <int MODE>
static cudaError_t launch_norm_rows(const NormArgs& a, cudaStream_t s) {
  // the bulk-copy variant measured slower than the register-resident one (0.33 vs 0.30 ms at 65536 x 4096): opt-in
  static const bool tma_on = [] { const char* e = getenv("PHYAI_NORM_TMA"); return e && e[0] == '1'; }();
  if (tma_on && !a.residual && a.rows >= 4096 && a.D >= 1024 && a.D <= 6144 && (reinterpret_cast<uintptr_t>(a.x) & 15) == 0) {
    if (a.D <= 2048) return launch_norm_tma<MODE, 8>(a, s);
    if (a.D <= 4096) return launch_norm_tma<MODE, 16>(a, s);
    return launch_norm_tma<MODE, 24>(a, s);
  }
  const int grid = (a.rows + 7) / 8;
  int sms = 148, dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  // persistent warps: as many CTAs as fit at once (registers bound it), each warp strides over the rows
  if (a.D <= 2048) PB_LAUNCH((norm_rows_reg_kernel<MODE, 8>), min(grid, sms * 2), 256, s, a);
  else if (a.D <= 4096) PB_LAUNCH((norm_rows_reg_kernel<MODE, 16>), min(grid, sms), 256, s, a);
  else if (a.D <= 6144) PB_LAUNCH((norm_rows_reg_kernel<MODE, 24>), min(grid, sms), 256, s, a);
  else PB_LAUNCH(norm_rows_kernel<MODE>, grid, 256, s, a);
  return cudaGetLastError();
}

cudaError_t norm_launch(const NormArgs& a, cudaStream_t s) {
  if (a.rows <= 0) return cudaSuccess;
  if (a.D % 8 || a.ldx % 8 || a.ldy % 8 || (a.residual && a.ldr % 8)) return cudaErrorInvalidValue;
  if (a.y8 && a.y8_block && (a.D % 128)) return cudaErrorInvalidValue;
  if (a.y8 && !a.y) return cudaErrorInvalidValue;
  if (a.rows >= 1024 && a.mode != kNormLayer && !a.y8 && !a.sumsq && a.y && a.D <= 16384) {
    switch (a.mode) {
      case kNormRms: return launch_norm_rows<kNormRms>(a, s);
      case kNormGemmaRms: return launch_norm_rows<kNormGemmaRms>(a, s);
      case kNormAdaRms: return launch_norm_rows<kNormAdaRms>(a, s);
      case kNormRmsNoWeight: return launch_norm_rows<kNormRmsNoWeight>(a, s);
      default: return cudaErrorInvalidValue;
    }
  }
  int threads = ((a.D / 8) + 31) / 32 * 32;
  if (threads > 1024) threads = 1024;
  if (threads < 32) threads = 32;
  switch (a.mode) {
    case kNormRms: PB_LAUNCH(norm_kernel<kNormRms>, a.rows, threads, s, a); break;
    case kNormGemmaRms: PB_LAUNCH(norm_kernel<kNormGemmaRms>, a.rows, threads, s, a); break;
    case kNormLayer: PB_LAUNCH(norm_kernel<kNormLayer>, a.rows, threads, s, a); break;
    case kNormAdaRms: PB_LAUNCH(norm_kernel<kNormAdaRms>, a.rows, threads, s, a); break;
    case kNormRmsNoWeight: PB_LAUNCH(norm_kernel<kNormRmsNoWeight>, a.rows, threads, s, a); break;
    default: return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

// ---------------------------------------------------------- RoPE + KV scatter
// One warp per (token, head). Heads [0,Hq) are queries (normed, rotated, written to
// q_out), [Hq,Hq+Hkv) keys (normed, rotated, scattered to k_pool), the rest values.
__global__ void rope_kv_kernel(RopeKvArgs a) {
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  const long long wid = (long long)blockIdx.x * warps_per_block + (threadIdx.x >> 5);
  const int H = a.Hq + 2 * a.Hkv;
  pdl_launch_dependents();
  pdl_wait();
  if (a.zero) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < a.zero_n; i += (long long)gridDim.x * blockDim.x)
      a.zero[i] = 0.f;
  }
  if (wid >= (long long)a.M * H) return;
  const int tok = int(wid / H), h = int(wid % H);
  const int D = a.D, half_rot = (a.rot_dim > 0 ? a.rot_dim : D) >> 1;
  const __nv_bfloat16* src = a.qkv + size_t(tok) * a.ld + size_t(h) * D;
  const bool is_q = h < a.Hq, is_k = !is_q && h < a.Hq + a.Hkv;
  __nv_bfloat16* dst;
  if (is_q) {
    dst = a.q_out + size_t(tok) * a.ldq + size_t(h) * D;
  } else {
    const long long slot = a.slots ? a.slots[tok] : a.slot_base + tok;
    __nv_bfloat16* pool = is_k ? a.k_pool : a.v_pool;
    if (pool == nullptr) return;
    const int hk = is_k ? h - a.Hq : h - a.Hq - a.Hkv;
    dst = pool + size_t(slot) * a.pool_row_stride + size_t(hk) * D;
  }
  if (!is_q && !is_k) {
    for (int i = lane * 8; i < D; i += 256)
      *reinterpret_cast<uint4*>(dst + i) = *reinterpret_cast<const uint4*>(src + i);
    return;
  }
  const __nv_bfloat16* nw = is_q ? a.q_norm_w : a.k_norm_w;
  float rstd = 1.f;
  if (nw) {
    float ss = 0.f;
    for (int i = lane; i < D; i += 32) {
      const float v = bf2f(src[i]);
      ss += v * v;
    }
    ss = warp_sum(ss);
    rstd = rsqrtf(ss / D + a.norm_eps);
  }
  const float* cs = nullptr;
  if (a.cos_sin) cs = a.cos_sin + size_t(a.pos ? a.pos[tok] : tok) * (2 * half_rot);
  for (int i = lane; i < (D >> 1); i += 32) {
    // pair (i, i + half_rot) inside the rotated span; dims past rot_dim pass through
    if (i < half_rot) {
      float x1 = bf2f(src[i]), x2 = bf2f(src[i + half_rot]);
      if (nw) {
        // norm output is rounded to bf16 before the rotation, as separate kernels would
        x1 = bf2f(__float2bfloat16(x1 * rstd * bf2f(nw[i])));
        x2 = bf2f(__float2bfloat16(x2 * rstd * bf2f(nw[i + half_rot])));
      }
      float c = 1.f, s = 0.f;
      if (cs) { c = cs[i]; s = cs[half_rot + i]; }
      dst[i] = __float2bfloat16(x1 * c - x2 * s);
      dst[i + half_rot] = __float2bfloat16(x2 * c + x1 * s);
    }
  }
  for (int i = 2 * half_rot + lane; i < D; i += 32) {
    float x = bf2f(src[i]);
    if (nw) x = x * rstd * bf2f(nw[i]);
    dst[i] = __float2bfloat16(x);
  }
}

cudaError_t rope_kv_launch(const RopeKvArgs& a, cudaStream_t s) {
  if (a.M <= 0) return cudaSuccess;
  if (a.D % 8 || a.ld % 8) return cudaErrorInvalidValue;
  const long long warps = (long long)a.M * (a.Hq + 2 * a.Hkv);
  const int wpb = 8;
  PB_LAUNCH(rope_kv_kernel, unsigned((warps + wpb - 1) / wpb), wpb * 32, s, a);
  return cudaGetLastError();
}

// ------------------------------------------------------------------ embedding
__global__ void embedding_kernel(const long long* ids, int n, const __nv_bfloat16* table, int D,
                                 long long lo, long long hi, float scale, __nv_bfloat16* out,
                                 int ldo, const int* dst_rows) {
  const int m = blockIdx.x;
  pdl_launch_dependents();
  pdl_wait();
  const long long id = ids[m];
  const bool in = id >= lo && id < hi;
  const int row = dst_rows ? dst_rows[m] : m;
  if (row < 0) return;
  BF8* o = reinterpret_cast<BF8*>(out + size_t(row) * ldo);
  const BF8* t = reinterpret_cast<const BF8*>(table + size_t(in ? id - lo : 0) * D);
  for (int v = threadIdx.x; v < (D >> 3); v += blockDim.x) {
    float f[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (in) {
      unpack8(t[v], f);
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] *= scale;
    }
    o[v] = pack8(f);
  }
}
cudaError_t embedding_launch(const long long* ids, int n, const __nv_bfloat16* table, int D,
                             long long lo, long long hi, float scale, __nv_bfloat16* out, int ldo,
                             const int* dst_rows, cudaStream_t s) {
  if (n <= 0) return cudaSuccess;
  if (D % 8 || ldo % 8) return cudaErrorInvalidValue;
  PB_LAUNCH(embedding_kernel, n, 128, s, ids, n, table, D, lo, hi, scale, out, ldo, dst_rows);
  return cudaGetLastError();
}

// --------------------------------------------------------------------- im2col
__global__ void im2col_kernel(const __nv_bfloat16* pix, int C, int H, int W, int p,
                              __nv_bfloat16* out, int kpad) {
  const int gw = W / p, gh = H / p;
  const int patch = blockIdx.x;             // over n_img * gh * gw
  const int img = patch / (gh * gw), rem = patch % (gh * gw);
  const int py0 = (rem / gw) * p, px0 = (rem % gw) * p;
  const int kreal = C * p * p;
  pdl_launch_dependents();
  pdl_wait();
  for (int k = threadIdx.x; k < kpad; k += blockDim.x) {
    __nv_bfloat16 v = __float2bfloat16(0.f);
    if (k < kreal) {
      const int c = k / (p * p), r = k % (p * p);
      const int y = py0 + r / p, x = px0 + r % p;
      v = pix[((size_t(img) * C + c) * H + y) * W + x];
    }
    out[size_t(patch) * kpad + k] = v;
  }
}
cudaError_t im2col_launch(const __nv_bfloat16* pix, int n_img, int C, int H, int W, int p,
                          __nv_bfloat16* out, int kpad, cudaStream_t s) {
  if (H % p || W % p || kpad < C * p * p) return cudaErrorInvalidValue;
  PB_LAUNCH(im2col_kernel, n_img * (H / p) * (W / p), 256, s, pix, C, H, W, p, out, kpad);
  return cudaGetLastError();
}

// ------------------------------------------------------------------ gated act
__device__ __forceinline__ float act_f(float v, int act) {
  switch (act) {
    case kActGeluTanh: return gelu_tanh_f(v);
    case kActSilu: return silu_f(v);
    case kActGeluErf: return gelu_erf_f(v);
    default: return v;
  }
}
__global__ void gated_act_kernel(const __nv_bfloat16* x, __nv_bfloat16* y, int M, int I, int act,
                                 int interleaved) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  pdl_launch_dependents();
  pdl_wait();
  if (idx >= (long long)M * I) return;
  const int m = int(idx / I), j = int(idx % I);
  const __nv_bfloat16* r = x + size_t(m) * 2 * I;
  const float g = bf2f(interleaved ? r[2 * j] : r[j]);
  const float u = bf2f(interleaved ? r[2 * j + 1] : r[I + j]);
  y[size_t(m) * I + j] = __float2bfloat16(act_f(g, act) * u);
}
cudaError_t gated_act_launch(const __nv_bfloat16* x, __nv_bfloat16* y, int M, int I, int act,
                             int interleaved, cudaStream_t s) {
  const long long n = (long long)M * I;
  if (n <= 0) return cudaSuccess;
  PB_LAUNCH(gated_act_kernel, unsigned((n + 255) / 256), 256, s, x, y, M, I, act, interleaved);
  return cudaGetLastError();
}

__global__ void unary_kernel(const __nv_bfloat16* x, __nv_bfloat16* y, long long n, int act) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  pdl_launch_dependents();
  pdl_wait();
  if (i < n) y[i] = __float2bfloat16(act_f(bf2f(x[i]), act));
}
cudaError_t unary_launch(const __nv_bfloat16* x, __nv_bfloat16* y, long long n, int act,
                         cudaStream_t s) {
  if (n <= 0) return cudaSuccess;
  PB_LAUNCH(unary_kernel, unsigned((n + 255) / 256), 256, s, x, y, n, act);
  return cudaGetLastError();
}

// ------------------------------------------------------------ sampler updates
__global__ void axpy_kernel(void* x, int x_fp32, const __nv_bfloat16* v, float dt, long long n) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  pdl_launch_dependents();
  pdl_wait();
  if (i >= n) return;
  if (x_fp32) {
    float* xf = reinterpret_cast<float*>(x);
    xf[i] += dt * bf2f(v[i]);
  } else {
    __nv_bfloat16* xb = reinterpret_cast<__nv_bfloat16*>(x);
    xb[i] = __float2bfloat16(bf2f(xb[i]) + dt * bf2f(v[i]));
  }
}
cudaError_t axpy_launch(void* x, int x_fp32, const __nv_bfloat16* v, float dt, long long n,
                        cudaStream_t s) {
  if (n <= 0) return cudaSuccess;
  PB_LAUNCH(axpy_kernel, unsigned((n + 255) / 256), 256, s, x, x_fp32, v, dt, n);
  return cudaGetLastError();
}

__global__ void cfg_combine_kernel(const __nv_bfloat16* c, const __nv_bfloat16* u, float g,
                                   __nv_bfloat16* out, float* x, float dt, long long n) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  pdl_launch_dependents();
  pdl_wait();
  if (i >= n) return;
  const float vc = bf2f(c[i]), vu = bf2f(u[i]);
  const float v = vu + g * (vc - vu);
  if (out) out[i] = __float2bfloat16(v);
  if (x) x[i] += dt * v;
}
cudaError_t cfg_combine_launch(const __nv_bfloat16* cond, const __nv_bfloat16* uncond, float g,
                               __nv_bfloat16* out, float* x_fp32, float dt, long long n,
                               cudaStream_t s) {
  if (n <= 0) return cudaSuccess;
  PB_LAUNCH(cfg_combine_kernel, unsigned((n + 255) / 256), 256, s, cond, uncond, g, out, x_fp32, dt, n);
  return cudaGetLastError();
}

// ------------------------------------------------------------ small / odd linears
// y = x @ w^T + bias for the shapes the tensor-core GEMM does not take (fp32 or fp16 operands, K or N not a
// multiple of 8): one warp per output column and group of four rows, fp32 accumulation, lanes stride K.
// These are the tiny projections around a model (timestep embedders, action heads), not its hot path.
template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return bf2f(v); }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16(v); }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half(v); }

template <typename TX, typename TW>
__global__ void linear_simt_kernel(const TX* x, const TW* w, const TW* bias, TX* y, int M, int N, int K, int ldx, int ldw, int ldy) {
  constexpr int R = 4;
  const int warps = blockDim.x >> 5, lane = threadIdx.x & 31;
  const int n = blockIdx.x * warps + (threadIdx.x >> 5);
  const int m0 = blockIdx.y * R;
  pdl_launch_dependents();
  pdl_wait();
  if (n >= N) return;
  float acc[R] = {0.f, 0.f, 0.f, 0.f};
  const TW* wr = w + size_t(n) * ldw;
  for (int k = lane; k < K; k += 32) {
    const float wv = to_f32<TW>(wr[k]);
#pragma unroll
    for (int r = 0; r < R; ++r)
      if (m0 + r < M) acc[r] += wv * to_f32<TX>(x[size_t(m0 + r) * ldx + k]);
  }
#pragma unroll
  for (int r = 0; r < R; ++r) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc[r] += __shfl_xor_sync(0xffffffffu, acc[r], o);
  }
  if (lane == 0) {
    const float b = bias ? to_f32<TW>(bias[n]) : 0.f;
#pragma unroll
    for (int r = 0; r < R; ++r)
      if (m0 + r < M) y[size_t(m0 + r) * ldy + n] = from_f32<TX>(acc[r] + b);
  }
}

template <typename TX, typename TW>
static cudaError_t linear_simt_typed(const void* x, const void* w, const void* bias, void* y, int M, int N, int K, int ldx,
                                     int ldw, int ldy, cudaStream_t s) {
  const int warps = 8;
  dim3 grid((N + warps - 1) / warps, (M + 3) / 4);
  PB_LAUNCH((linear_simt_kernel<TX, TW>), grid, warps * 32, s, reinterpret_cast<const TX*>(x), reinterpret_cast<const TW*>(w),
            reinterpret_cast<const TW*>(bias), reinterpret_cast<TX*>(y), M, N, K, ldx, ldw, ldy);
  return cudaGetLastError();
}

// dtype codes: 0 = fp32, 1 = bf16, 2 = fp16 (bias has the weight's type, y has x's type)
cudaError_t linear_simt_launch(const void* x, int x_type, const void* w, int w_type, const void* bias, void* y, int M, int N,
                               int K, int ldx, int ldw, int ldy, cudaStream_t s) {
  if (M <= 0 || N <= 0 || K <= 0) return cudaSuccess;
#define PB_LS(TX, TW) return linear_simt_typed<TX, TW>(x, w, bias, y, M, N, K, ldx, ldw, ldy, s)
  switch (x_type * 3 + w_type) {
    case 0: PB_LS(float, float);
    case 1: PB_LS(float, __nv_bfloat16);
    case 2: PB_LS(float, __half);
    case 3: PB_LS(__nv_bfloat16, float);
    case 4: PB_LS(__nv_bfloat16, __nv_bfloat16);
    case 5: PB_LS(__nv_bfloat16, __half);
    case 6: PB_LS(__half, float);
    case 7: PB_LS(__half, __nv_bfloat16);
    case 8: PB_LS(__half, __half);
  }
#undef PB_LS
  return cudaErrorInvalidValue;
}

// ------------------------------------------------------------ per-domain linear
// y[b, t, :] = x[b, t, :] @ W[domain[b]] + bias[domain[b]] with W stored [domains][in][out] (the checkpoint layout of
// the embodiment-specific action projections): one thread per output column and four rows, the domain read on the
// device so the caller never synchronises. A few MFLOP per call; CUDA cores.
__global__ void domain_linear_kernel(const __nv_bfloat16* x, const __nv_bfloat16* w, const __nv_bfloat16* bias,
                                     const long long* domain, __nv_bfloat16* y, int T, int K, int N) {
  constexpr int R = 4;
  const int n = blockIdx.x * blockDim.x + threadIdx.x;
  const int b = blockIdx.z, t0 = blockIdx.y * R;
  pdl_launch_dependents();
  pdl_wait();
  if (n >= N) return;
  const long long d = domain[b];
  const __nv_bfloat16* wd = w + size_t(d) * K * N + n;
  const __nv_bfloat16* xb = x + (size_t(b) * T + t0) * K;
  float acc[R] = {0.f, 0.f, 0.f, 0.f};
  for (int k = 0; k < K; ++k) {
    const float wv = bf2f(wd[size_t(k) * N]);
#pragma unroll
    for (int r = 0; r < R; ++r)
      if (t0 + r < T) acc[r] += wv * bf2f(xb[size_t(r) * K + k]);
  }
  const float bv = bf2f(bias[size_t(d) * N + n]);
#pragma unroll
  for (int r = 0; r < R; ++r)
    if (t0 + r < T) y[(size_t(b) * T + t0 + r) * N + n] = __float2bfloat16(acc[r] + bv);
}
cudaError_t domain_linear_launch(const __nv_bfloat16* x, const __nv_bfloat16* w, const __nv_bfloat16* bias, const long long* domain,
                                 __nv_bfloat16* y, int B, int T, int K, int N, cudaStream_t s) {
  if (B <= 0 || T <= 0 || N <= 0) return cudaSuccess;
  const int threads = N >= 256 ? 256 : ((N + 31) / 32 * 32);
  dim3 grid((N + threads - 1) / threads, (T + 3) / 4, B);
  PB_LAUNCH(domain_linear_kernel, grid, threads, s, x, w, bias, domain, y, T, K, N);
  return cudaGetLastError();
}

// ------------------------------------------------------------ UniPC sampler step
// One multistep update of a flow-matching latent, element by element, with everything the host loop used to
// issue as separate tensor ops: guidance combine, x0 prediction, corrector, predictor, history rotation and the
// re-imposition of clean (conditioning) frames. The tensor is viewed as [B][C][T][inner]; `keep` flags (b, t)
// pairs whose elements are overwritten with `cond` after the update; columns >= `live_inner` of the innermost
// dimension carry no signal (padding of an action vector) and get a zero velocity.
__global__ void unipc_step_kernel(UniPCStepArgs a) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  pdl_launch_dependents();
  pdl_wait();
  if (i >= a.n) return;
  float v = bf2f(a.v[i]);
  if (a.v_uncond) {
    const float vu = bf2f(a.v_uncond[i]);
    v = vu + a.g * (v - vu);
  }
  const long long col = i % a.inner;
  if (col >= a.live_inner) v = 0.f;
  const float x = bf2f(a.x[i]);
  const float m_t = x - a.sigma * v;
  const float m1 = a.m1[i];
  float xs = x;
  if (a.has_corr) {
    xs = a.c_x * a.x_last[i] + a.c_0 * m1 + a.c_t * m_t;
    if (a.c_1 != 0.f) xs += a.c_1 * a.m2[i];
    xs = bf2f(__float2bfloat16(xs));          // the corrected sample is what a bf16 model input would have seen
  }
  float out = a.p_x * xs + a.p_0 * m_t;
  if (a.p_1 != 0.f) out += a.p_1 * m1;
  a.x_last[i] = xs;
  a.m2[i] = m1;
  a.m1[i] = m_t;
  __nv_bfloat16 o = __float2bfloat16(out);
  if (a.keep) {
    const long long frame = (i / a.inner) % a.T;
    const long long b = i / (a.inner * a.T * a.C);
    if (a.keep[b * a.T + frame]) o = a.cond[i];
  }
  a.x[i] = o;
}
cudaError_t unipc_step_launch(const UniPCStepArgs& a, cudaStream_t s) {
  if (a.n <= 0) return cudaSuccess;
  PB_LAUNCH(unipc_step_kernel, unsigned((a.n + 255) / 256), 256, s, a);
  return cudaGetLastError();
}

// --------------------------------------------------------------- row scatter
__global__ void scatter_rows_kernel(const __nv_bfloat16* src, int D, int lds, __nv_bfloat16* dst,
                                    int ldd, const int* rows) {
  const int i = blockIdx.x;
  pdl_launch_dependents();
  pdl_wait();
  const int r = rows ? rows[i] : i;
  if (r < 0) return;
  const uint4* s4 = reinterpret_cast<const uint4*>(src + size_t(i) * lds);
  uint4* d4 = reinterpret_cast<uint4*>(dst + size_t(r) * ldd);
  for (int v = threadIdx.x; v < (D >> 3); v += blockDim.x) d4[v] = s4[v];
}
cudaError_t scatter_rows_launch(const __nv_bfloat16* src, int n, int D, int lds,
                                __nv_bfloat16* dst, int ldd, const int* rows, cudaStream_t s) {
  if (n <= 0) return cudaSuccess;
  if (D % 8 || lds % 8 || ldd % 8) return cudaErrorInvalidValue;
  PB_LAUNCH(scatter_rows_kernel, n, 128, s, src, D, lds, dst, ldd, rows);
  return cudaGetLastError();
}

// ------------------------------------------------------------------ fp8 quant
__global__ void quant_fp8_kernel(const __nv_bfloat16* x, int D, int ldx, uint8_t* y, float* scale,
                                 int block) {
  __shared__ float red[32];
  const int row = blockIdx.x;
  const int nv = D >> 3;
  pdl_launch_dependents();
  pdl_wait();
  const BF8* xr = reinterpret_cast<const BF8*>(x + size_t(row) * ldx);
  if (block == 0) {
    float amax = 0.f;
    for (int v = threadIdx.x; v < nv; v += blockDim.x) {
      float f[8];
      unpack8(xr[v], f);
#pragma unroll
      for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(f[i]));
    }
    amax = block_max(amax, red);
    const float sc = fmaxf(amax, 1e-12f) / 448.f;
    if (threadIdx.x == 0) scale[row] = sc;
    const float inv = 1.f / sc;
    for (int v = threadIdx.x; v < nv; v += blockDim.x) {
      float f[8];
      unpack8(xr[v], f);
      uint8_t q[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) q[i] = __nv_cvt_float_to_fp8(f[i] * inv, __NV_SATFINITE, __NV_E4M3);
      *reinterpret_cast<uint2*>(y + size_t(row) * D + v * 8) = *reinterpret_cast<uint2*>(q);
    }
  } else {
    const int nb = D >> 7;
    for (int v0 = 0; v0 < nv; v0 += blockDim.x) {
      const int v = v0 + threadIdx.x;
      float f[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      if (v < nv) unpack8(xr[v], f);
      float m = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) m = fmaxf(m, fabsf(f[i]));
#pragma unroll
      for (int off = 8; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
      const float sc = fmaxf(m, 1e-12f) / 448.f;
      if (v < nv) {
        if ((v & 15) == 0) scale[size_t(row) * nb + (v >> 4)] = sc;
        const float inv = 1.f / sc;
        uint8_t q[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) q[i] = __nv_cvt_float_to_fp8(f[i] * inv, __NV_SATFINITE, __NV_E4M3);
        *reinterpret_cast<uint2*>(y + size_t(row) * D + v * 8) = *reinterpret_cast<uint2*>(q);
      }
    }
  }
}
cudaError_t quant_fp8_launch(const __nv_bfloat16* x, int rows, int D, int ldx, uint8_t* y,
                             float* scale, int block, cudaStream_t s) {
  if (rows <= 0) return cudaSuccess;
  if (D % 8 || ldx % 8 || (block && D % 128)) return cudaErrorInvalidValue;
  int threads = ((D / 8) + 31) / 32 * 32;
  if (threads > 1024) threads = 1024;
  PB_LAUNCH(quant_fp8_kernel, rows, threads, s, x, D, ldx, y, scale, block);
  return cudaGetLastError();
}


// ---------------------------------------------------------------------- snake
// y[b, c, t] = x + sin^2(alpha[c] x) / (beta[c] + 1e-9), x of shape [B, C, T] (T contiguous). One pass,
// fp32 math; the reference composes it from five elementwise ATen kernels on an fp32 copy
// (phyai/src/phyai/layers/activation.py:40-67).
template <typename T>
__global__ void snake_kernel(const T* x, T* y, const float* alpha, const float* beta, int C, long long Tn, long long total) {
  pdl_launch_dependents();
  pdl_wait();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int c = int((i / Tn) % C);
    const float a = alpha[c], ib = 1.f / (beta[c] + 1e-9f);
    float v;
    if constexpr (sizeof(T) == 2) v = bf2f(reinterpret_cast<const __nv_bfloat16*>(x)[i]);
    else v = reinterpret_cast<const float*>(x)[i];
    const float sn = sinf(a * v);
    const float o = v + sn * sn * ib;
    if constexpr (sizeof(T) == 2) reinterpret_cast<__nv_bfloat16*>(y)[i] = __float2bfloat16(o);
    else reinterpret_cast<float*>(y)[i] = o;
  }
}
cudaError_t snake_launch(const void* x, void* y, int is_bf16, const float* alpha, const float* beta, int C, long long T,
                         long long total, cudaStream_t s) {
  if (total <= 0) return cudaSuccess;
  if (C <= 0 || T <= 0) return cudaErrorInvalidValue;
  const int threads = 256;
  long long blocks = (total + threads - 1) / threads;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (is_bf16) PB_LAUNCH(snake_kernel<__nv_bfloat16>, unsigned(blocks), threads, s, reinterpret_cast<const __nv_bfloat16*>(x),
                         reinterpret_cast<__nv_bfloat16*>(y), alpha, beta, C, T, total);
  else PB_LAUNCH(snake_kernel<float>, unsigned(blocks), threads, s, reinterpret_cast<const float*>(x),
                 reinterpret_cast<float*>(y), alpha, beta, C, T, total);
  return cudaGetLastError();
}

}  // namespace pb

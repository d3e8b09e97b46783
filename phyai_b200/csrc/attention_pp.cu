// Pipelined tcgen05 flash attention for long dense sequences (sm_100a).
//
// attention_tc.cu walks one 128-row query tile through load -> S -> softmax -> PV one step
// after the other, which is right for the short, latency-bound calls of the action expert
// but leaves the tensor core idle during every softmax. This kernel is the throughput
// variant for the diffusion / prefill regime (thousands of query rows, head_dim <= 128,
// dense q, contiguous K/V):
//
//   * a CTA owns TWO query tiles of 128 rows of one head; while the 128 softmax threads of
//     tile 0 work on S0 the tensor core computes S1, then O0 += P0 V while tile 1 is in
//     softmax, and so on (ping-pong);
//   * warp roles: warps 0-3 softmax of tile 0, warps 4-7 softmax of tile 1, warp 8 issues
//     every tcgen05.mma, warp 9 drives TMA (Q once, K and V through two-stage rings);
//   * P never touches shared memory: the softmax threads write it as packed bf16 into the
//     tensor-memory columns of their S tile and the PV product reads its A operand from
//     there; the next S of that tile is issued behind the PV that reads it (the tensor pipe
//     executes one thread's instructions in order);
//   * the running maximum is only raised when it would grow by more than 2^8, so the
//     read-modify-write of O in tensor memory almost never happens after the first chunks.
//
// Tensor memory (512 columns): S0 [0,128) S1 [128,256) O0 [256,384) O1 [384,512).
// Every wait is bounded; a timeout records a status, all roles drain and the CTA exits.
//
// Capability parity: the reference runs its diffusion attention through FlashInfer
// (phyai/src/phyai/layers/attention/backends/flashinfer_diffusion.py) and the prefix
// attention through FlashInfer prefill (.../flashinfer_ar.py).
#include <cstdlib>

#include "attention.cuh"
#include "gemm.cuh"
#include "launch.cuh"
#include "ptx.cuh"

#include <cstring>

namespace pb {

namespace {

constexpr int kT = 128;                 // rows per query tile, KV entries per chunk
constexpr int kPPThreads = 320;
constexpr int kBlk = 128 * 128;         // bytes of one [128 rows x 128 B] swizzled block
constexpr float kRaise = 8.0f;          // raise the running max only beyond this (log2 units)

// 2^x on the FMA pipe (round-to-nearest split x = n + f with the 1.5 * 2^23 trick, a cubic for 2^f on
// [-0.5, 0.5] with relative error below 6e-4, well under bf16 rounding of P, and n added to the exponent
// field). The special-function unit delivers 16 exponentials per clock and SM, which for a 128-wide head
// costs as many cycles as the two matrix products of the tile, so a kernel variant can route one or two of
// every four probabilities through here (template parameter NP); it is off by default because it measured slower.
__device__ __forceinline__ float exp2_fma(float x) {
  x = fmaxf(x, -125.f);
  const float t = x + 12582912.f;
  const float f = x - (t - 12582912.f);
  float p = fmaf(f, 0.0555041f, 0.2402265f);
  p = fmaf(p, f, 0.6931472f);
  p = fmaf(p, f, 1.0f);
  return __int_as_float(__float_as_int(p) + (__float_as_int(t) << 23));
}

// Packed fp32 pairs (one 64-bit register): sm_100 issues fma / add on both halves with one instruction, which
// halves the scale-subtract and row-sum instructions of the softmax; the three-input max halves the max pass.
// The softmax warps are issue-bound (two warps per scheduler next to 128 scores per thread and chunk).
__device__ __forceinline__ uint64_t pack2(float a, float b) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& a, float& b) { asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v)); }
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

}  // namespace

// DB: head dim padded to 64 * DB, DB in {1, 2}. NP: how many of every four probabilities take exp2_fma (0..2).
template <int DB, int NP>
__global__ void __launch_bounds__(kPPThreads, 1)
attn_pp_kernel(AttnParams p, int* status, const __grid_constant__ CUtensorMap tmQ,
               const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV) {
  constexpr int DP = 64 * DB;
  constexpr int TILE_BYTES = DB * kBlk;   // one 128 x DP bf16 operand tile
  constexpr int O_COL = 256;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sQ = smem_u32(smem);                 // 2 tiles
  const uint32_t sK = sQ + 2 * TILE_BYTES;            // 2 stages
  const uint32_t sV = sK + 2 * TILE_BYTES;            // 2 stages
  __shared__ __align__(8) uint64_t bar_q, bar_done, bar_kf[2], bar_ke[2], bar_vf[2], bar_ve[2], bar_s[2], bar_p[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ volatile int err_s;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int b = blockIdx.z, head = blockIdx.y, kvh = head / p.group;
  const int q_len = p.q_len[b], kv_len = p.kv_len[b], q_start = p.q_start[b], kv_base = p.kv_indptr[b];
  const int row0 = blockIdx.x * 2 * kT;   // first query token of this CTA within the sequence
  const bool live = row0 < q_len;

  if (tid == 0) {
    mbar_init(&bar_q, 1);
    mbar_init(&bar_done, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bar_kf[i], 1); mbar_init(&bar_ke[i], 1);
      mbar_init(&bar_vf[i], 1); mbar_init(&bar_ve[i], 1);
      mbar_init(&bar_s[i], 1);  mbar_init(&bar_p[i], kT);
    }
    err_s = 0;
    mbar_fence_init();
    prefetch_tmap(&tmQ); prefetch_tmap(&tmK); prefetch_tmap(&tmV);
  }
  if (warp == 8) {
    tmem_alloc(&tmem_base_s, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_s;
  pdl_launch_dependents();
  pdl_wait();

  int n_chunks = 0;
  const int causal_off = kv_len - q_len;
  if (live) {
    n_chunks = (kv_len + kT - 1) / kT;
    if (p.causal) {
      const int last_tok = min(q_len - 1, row0 + 2 * kT - 1);
      n_chunks = min(n_chunks, max(0, (last_tok + causal_off + 1 + kT - 1) / kT));
    }
  }

  if (warp == 9) {
    // ------------------------------------------------------------------ TMA producer
    if (n_chunks > 0) {
      if (lane == 0) {
        mbar_expect_tx(&bar_q, 2 * TILE_BYTES);
        for (int t = 0; t < 2; ++t)
          for (int blk = 0; blk < DB; ++blk)
            tma_load_3d(sQ + t * TILE_BYTES + blk * kBlk, &tmQ, &bar_q, blk * 64, head, q_start + row0 + t * kT);
      }
      for (int j = 0; j < n_chunks && !err_s; ++j) {
        const int s = j & 1;
        const uint32_t ph = uint32_t((j >> 1) & 1);
        if (j >= 2) {
          if (!mbar_wait(&bar_ke[s], ph ^ 1)) { err_s = kStatusTimeoutEmpty; break; }
        }
        if (lane == 0) {
          mbar_expect_tx(&bar_kf[s], TILE_BYTES);
          for (int blk = 0; blk < DB; ++blk)
            tma_load_3d(sK + s * TILE_BYTES + blk * kBlk, &tmK, &bar_kf[s], blk * 64, kvh, kv_base + j * kT);
        }
        if (j >= 2) {
          if (!mbar_wait(&bar_ve[s], ph ^ 1)) { err_s = kStatusTimeoutEmpty; break; }
        }
        if (lane == 0) {
          mbar_expect_tx(&bar_vf[s], TILE_BYTES);
          for (int blk = 0; blk < DB; ++blk)
            tma_load_3d(sV + s * TILE_BYTES + blk * kBlk, &tmV, &bar_vf[s], blk * 64, kvh, kv_base + j * kT);
        }
        __syncwarp();
      }
    }
  } else if (warp == 8) {
    // ------------------------------------------------------------------ MMA issuer
    if (n_chunks > 0) {
      const uint32_t idesc_s = make_idesc_f16(kT, kT, 1);
      const uint32_t idesc_o = make_idesc_f16_bmn(kT, DP, 1);
      auto issue_s = [&](int t, int stage) {   // S_t = Q_t K^T
        if (lane == 0) {
#pragma unroll
          for (int kk = 0; kk < DP / 16; ++kk) {
            const uint64_t dq = make_smem_desc_sw128(sQ + t * TILE_BYTES + (kk >> 2) * kBlk) + 2 * (kk & 3);
            const uint64_t dk = make_smem_desc_sw128(sK + stage * TILE_BYTES + (kk >> 2) * kBlk) + 2 * (kk & 3);
            umma_f16(tmem + t * kT, dq, dk, idesc_s, kk != 0);
          }
          umma_commit(&bar_s[t]);
        }
        __syncwarp();
      };
      auto issue_pv = [&](int t, int stage, bool acc) {   // O_t += P_t V, P read from tensor memory
        if (lane == 0) {
#pragma unroll
          for (int kk = 0; kk < kT / 16; ++kk) {
            const uint64_t dv = make_smem_desc_sw128_mn(sV + stage * TILE_BYTES + kk * 2048, kBlk, 1024);
            umma_f16_ts(tmem + O_COL + t * kT, tmem + t * kT + kk * 8, dv, idesc_o, (acc || kk != 0) ? 1u : 0u);
          }
        }
        __syncwarp();
      };
      bool ok = mbar_wait(&bar_q, 0) && mbar_wait(&bar_kf[0], 0);
      if (!ok) err_s = kStatusTimeoutFull;
      if (ok) {
        tc_fence_after();
        issue_s(0, 0);
        issue_s(1, 0);
        if (lane == 0) umma_commit(&bar_ke[0]);
        __syncwarp();
      }
      for (int j = 0; j < n_chunks && ok && !err_s; ++j) {
        const int s = j & 1, sn = (j + 1) & 1;
        const uint32_t ph = uint32_t((j >> 1) & 1), phn = uint32_t(((j + 1) >> 1) & 1), pj = uint32_t(j & 1);
        const bool has_next = j + 1 < n_chunks;
        ok = mbar_wait(&bar_vf[s], ph) && (!has_next || mbar_wait(&bar_kf[sn], phn));
        if (!ok) { err_s = kStatusTimeoutFull; break; }
        ok = mbar_wait(&bar_p[0], pj);
        if (!ok) { err_s = kStatusTimeoutAcc; break; }
        tc_fence_after();
        issue_pv(0, s, j > 0);
        if (has_next) issue_s(0, sn);
        ok = mbar_wait(&bar_p[1], pj);
        if (!ok) { err_s = kStatusTimeoutAcc; break; }
        tc_fence_after();
        issue_pv(1, s, j > 0);
        if (lane == 0) umma_commit(&bar_ve[s]);
        __syncwarp();
        if (has_next) {
          issue_s(1, sn);
          if (lane == 0) umma_commit(&bar_ke[sn]);
          __syncwarp();
        }
      }
      if (lane == 0) umma_commit(&bar_done);
      __syncwarp();
    }
  } else {
    // ------------------------------------------------------------------ softmax of tile t
    const int t = warp >> 2;                 // 0 or 1
    const int r = tid & (kT - 1);            // row inside the tile = tensor-memory lane
    const int tok = row0 + t * kT + r;       // query token inside the sequence
    const uint32_t lane_addr = tmem + (uint32_t((warp & 3) * 32) << 16);
    const uint32_t s_addr = lane_addr + t * kT, o_addr = lane_addr + O_COL + t * kT;
    const float scale_log2 = p.sm_scale * 1.4426950408889634f;
    float m_ref = -INFINITY, l_run = 0.f;    // m_ref: the maximum P and O are currently expressed against
    int jlim_row = kv_len;
    if (p.causal) jlim_row = min(kv_len, tok + causal_off + 1);
    bool ok = true;
    for (int j = 0; j < n_chunks && !err_s; ++j) {
      if (!mbar_wait(&bar_s[t], uint32_t(j & 1))) { err_s = kStatusTimeoutAcc; ok = false; break; }
      tc_fence_after();
      uint32_t sv[kT];
#pragma unroll
      for (int c = 0; c < kT; c += 32) tmem_ld_32x32(s_addr + c, *reinterpret_cast<uint32_t(*)[32]>(&sv[c]));
      tmem_ld_wait();
      const int lim = jlim_row - j * kT;     // columns [0, lim) of this chunk are visible to the row
      float mx = -INFINITY;
      if (lim >= kT) {
#pragma unroll
        for (int c = 0; c < kT; c += 2) mx = max3(mx, __uint_as_float(sv[c]), __uint_as_float(sv[c + 1]));
      } else {
#pragma unroll
        for (int c = 0; c < kT; ++c) mx = fmaxf(mx, c < lim ? __uint_as_float(sv[c]) : -INFINITY);
      }
      mx *= scale_log2;
      // raise the reference maximum only when it matters; stale-by-<=8 maxima keep P <= 2^8
      float corr = 1.f;
      const bool raise = mx > m_ref + kRaise || (m_ref == -INFINITY && mx > -INFINITY);
      if (raise) {
        corr = m_ref == -INFINITY ? 0.f : exp2f(m_ref - mx);
        m_ref = mx;
      }
      const float m_use = m_ref == -INFINITY ? 0.f : m_ref;
      float sum = 0.f;
      uint32_t pk[kT / 2];
      if (NP == 0 && lim >= kT) {
        const uint64_t sc2 = pack2(scale_log2, scale_log2), nm2 = pack2(-m_use, -m_use);
        uint64_t sum2 = pack2(0.f, 0.f);
#pragma unroll
        for (int c = 0; c < kT; c += 2) {
          float x0, x1;
          unpack2(fma2(pack2(__uint_as_float(sv[c]), __uint_as_float(sv[c + 1])), sc2, nm2), x0, x1);
          const float p0 = exp2f(x0), p1 = exp2f(x1);
          sum2 = add2(sum2, pack2(p0, p1));
          const __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
          pk[c >> 1] = *reinterpret_cast<const uint32_t*>(&h);
        }
        float s0, s1;
        unpack2(sum2, s0, s1);
        sum = s0 + s1;
      } else if (lim >= kT) {
#pragma unroll
        for (int c = 0; c < kT; c += 4) {
          const float p0 = exp2f(__uint_as_float(sv[c]) * scale_log2 - m_use);
          const float x1 = __uint_as_float(sv[c + 1]) * scale_log2 - m_use, x3 = __uint_as_float(sv[c + 3]) * scale_log2 - m_use;
          const float p1 = NP >= 2 ? exp2_fma(x1) : exp2f(x1);
          const float p2 = exp2f(__uint_as_float(sv[c + 2]) * scale_log2 - m_use);
          const float p3 = NP >= 1 ? exp2_fma(x3) : exp2f(x3);
          sum += (p0 + p1) + (p2 + p3);
          const __nv_bfloat162 h0 = __floats2bfloat162_rn(p0, p1), h1 = __floats2bfloat162_rn(p2, p3);
          pk[c >> 1] = *reinterpret_cast<const uint32_t*>(&h0);
          pk[(c >> 1) + 1] = *reinterpret_cast<const uint32_t*>(&h1);
        }
      } else {
#pragma unroll
        for (int c = 0; c < kT; c += 2) {
          const float p0 = c < lim ? exp2f(__uint_as_float(sv[c]) * scale_log2 - m_use) : 0.f;
          const float p1 = c + 1 < lim ? exp2f(__uint_as_float(sv[c + 1]) * scale_log2 - m_use) : 0.f;
          sum += p0 + p1;
          const __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
          pk[c >> 1] = *reinterpret_cast<const uint32_t*>(&h);
        }
      }
      l_run = l_run * corr + sum;
      // O_t is quiescent here: S_t(j) complete implies every earlier PV of this tile retired
      if (__any_sync(0xffffffffu, j > 0 && corr != 1.f)) {
#pragma unroll 1
        for (int c = 0; c < DP; c += 32) {
          uint32_t o[32];
          tmem_ld_32x32(o_addr + c, o);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * corr);
          tmem_st_32x32(o_addr + c, o);
        }
      }
      tmem_st_32x32(s_addr, *reinterpret_cast<const uint32_t(*)[32]>(&pk[0]));
      tmem_st_32x32(s_addr + 32, *reinterpret_cast<const uint32_t(*)[32]>(&pk[32]));
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&bar_p[t]);
    }
    // ---------------- write-out: O_t / l straight from tensor memory
    if (n_chunks > 0 && ok && !err_s) {
      if (!mbar_wait(&bar_done, 0)) {
        err_s = kStatusTimeoutAcc;
      } else {
        tc_fence_after();
        const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
        const bool live_row = tok < q_len;
        __nv_bfloat16* dst = p.out + size_t(q_start + (live_row ? tok : 0)) * p.o_tok_stride + size_t(head) * p.o_head_stride;
#pragma unroll 1
        for (int c = 0; c < DP; c += 32) {
          uint32_t o[32];
          tmem_ld_32x32(o_addr + c, o);
          tmem_ld_wait();
          if (live_row) {
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
              if (c + 8 * q4 < p.head_dim) {
                uint4 w;
                __nv_bfloat162* w2 = reinterpret_cast<__nv_bfloat162*>(&w);
#pragma unroll
                for (int e = 0; e < 4; ++e)
                  w2[e] = __floats2bfloat162_rn(__uint_as_float(o[8 * q4 + 2 * e]) * inv, __uint_as_float(o[8 * q4 + 2 * e + 1]) * inv);
                *reinterpret_cast<uint4*>(dst + c + 8 * q4) = w;
              }
            }
          }
        }
      }
    } else if (live && n_chunks == 0 && tok < q_len) {
      // nothing visible to this CTA's rows: the result is zero
      __nv_bfloat16* dst = p.out + size_t(q_start + tok) * p.o_tok_stride + size_t(head) * p.o_head_stride;
      for (int c = 0; c < p.head_dim; c += 8) *reinterpret_cast<uint4*>(dst + c) = make_uint4(0, 0, 0, 0);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (err_s) {
    if (tid == 0) {
      if (status) atomicCAS(status, 0, int(err_s));
      // let copies that are still in flight land before the block goes away
      const uint64_t t0 = globaltimer_ns();
      while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
    }
    __syncthreads();
  }
  if (warp == 8) tmem_dealloc(tmem, 512);
}

template <int DB, int NP>
static cudaError_t attn_pp_launch_db(const AttnParams& p, cudaStream_t stream) {
  auto kern = attn_pp_kernel<DB, NP>;
  const size_t smem = size_t(6 * DB) * kBlk + 1024;
  static bool attr_done = false;
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    if (e != cudaSuccess) return e;
    attr_done = true;
  }
  CUtensorMap tq, tk, tv;
  const int Hq = p.num_kv_heads * p.group;
  if (!make_tmap_3d_bf16(&tq, p.q, p.head_dim, Hq, p.q_rows, p.q_head_stride, p.q_tok_stride, 1, kT) ||
      !make_tmap_3d_bf16(&tk, p.k, p.head_dim, p.num_kv_heads, p.kv_rows, p.kv_head_stride, p.kv_row_stride, 1, kT) ||
      !make_tmap_3d_bf16(&tv, p.v, p.head_dim, p.num_kv_heads, p.kv_rows, p.kv_head_stride, p.kv_row_stride, 1, kT))
    return cudaErrorInvalidValue;
  return launch_kernel(kern, dim3((p.max_q_len + 2 * kT - 1) / (2 * kT), Hq, p.batch), dim3(kPPThreads), smem, stream, 1,
                       p, kernel_status_ptr(), tq, tk, tv);
}

bool attn_pp_supported(const AttnParams& p) {
  const auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
  return !p.kv_indices && p.splits == 1 && p.head_dim <= 128 && p.head_dim % 8 == 0 && p.q_rows > 0 && p.kv_rows > 0 &&
         al16(p.q) && al16(p.k) && al16(p.v) && al16(p.out) &&
         (p.q_tok_stride | p.q_head_stride | p.kv_row_stride | p.kv_head_stride | p.o_tok_stride | p.o_head_stride) % 8 == 0;
}

cudaError_t attn_pp_launch(const AttnParams& p, cudaStream_t stream) {
  if (!attn_pp_supported(p) || p.batch <= 0 || p.max_q_len <= 0 || p.group <= 0) return cudaErrorInvalidValue;
  // PHYAI_ATTN_POLY = 0 / 1 / 2: how many of every four exponentials go to the FMA pipe. Measured on one box at the
  // Cosmos3 shape: 0.98 / 1.03 / 1.10 ms, i.e. the FMA pipe, not the special-function unit, is the busier one here: default 0.
  static const int np = [] { const char* e = getenv("PHYAI_ATTN_POLY"); return e && e[0] >= '0' && e[0] <= '2' ? e[0] - '0' : 0; }();
  if (p.head_dim <= 64) return np == 0 ? attn_pp_launch_db<1, 0>(p, stream) : np == 2 ? attn_pp_launch_db<1, 2>(p, stream) : attn_pp_launch_db<1, 1>(p, stream);
  return np == 0 ? attn_pp_launch_db<2, 0>(p, stream) : np == 2 ? attn_pp_launch_db<2, 2>(p, stream) : attn_pp_launch_db<2, 1>(p, stream);
}

}  // namespace pb

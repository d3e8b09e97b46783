// tcgen05 flash attention for sm_100a: S = Q K^T and O += P V run on the 5th-generation
// tensor cores with both accumulators in tensor memory.
//
// A CTA owns 128 query rows (token x head-in-group pairs, so the heads of a GQA/MQA
// group share one pass over K/V) and walks KV in chunks of 128 entries:
//
//   load K chunk -> S(128x128) = Q K^T  [tcgen05.mma, K-major operands]
//   softmax warps read S from TMEM (one thread per row), keep running (max, sum),
//   write P as bf16 into shared memory in the operand layout, rescale O in TMEM
//   when the running max moved
//   load V chunk -> O(128xD) += P V     [tcgen05.mma, V is the MN-major B operand]
//
// The KV range can be split over a thread-block cluster (1,1,S); the S partial
// (max, sum, O) triples are merged through distributed shared memory and each CTA
// writes 128/S rows of the result. Q/K/V rows are gathered with cp.async straight
// into the 128-byte-swizzled layout the tensor core reads, so paged pools (page
// size 1, arbitrary row indices) cost nothing extra.
//
// Same interface and semantics as attn_kernel in attention.cu (see attention.cuh).
#include "attention.cuh"
#include "gemm.cuh"
#include "launch.cuh"
#include "ptx.cuh"

#include <cstring>

namespace pb {

namespace {

constexpr int kTQ = 128;         // query rows per CTA = UMMA M
constexpr int kTK = 128;         // KV entries per chunk = UMMA N of S, K of PV
constexpr int kTcThreads = 256;  // warps 0-3: softmax, warp 4: MMA issue + TMEM, all 8: loads / merge
constexpr int kBlkBytes = 128 * 128;  // one [128 rows x 128 B] swizzled block

__device__ __forceinline__ void cp16(uint32_t dst, const void* src, bool valid) {
  const int sz = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(sz)
               : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

// Byte offset of the 16-byte chunk holding elements [8c, 8c+8) of row r in a tile stored as
// 64-element column blocks of [128 rows x 128 B] with the 128-byte swizzle.
__device__ __forceinline__ uint32_t sw_off(int r, int c) {
  return uint32_t(c >> 3) * kBlkBytes + uint32_t(r) * 128u + uint32_t(((c & 7) ^ (r & 7)) << 4);
}

}  // namespace

// EXTRA: the instantiation that also applies a sliding window (`p.window`) and / or a logit soft cap (`p.soft_cap`);
// the plain one carries neither the compares nor the tanh.
template <int DB, bool EXTRA = false>  // head dim padded to 64 * DB
__global__ void __launch_bounds__(kTcThreads)
attn_tc_kernel(AttnParams p, int* status, const __grid_constant__ CUtensorMap tmQ,
               const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
               int use_tma) {
  constexpr int DP = 64 * DB;
  constexpr int CH = DP / 8;                  // 16-byte chunks per Q/K/V row
  constexpr int Q_BYTES = DB * kBlkBytes;     // also K and V chunk bytes
  constexpr int TMEM_COLS = DP > 128 ? 512 : 256;
  constexpr int O_COL = 128;                  // S at columns [0,128), O at [128, 128+DP)
  constexpr int LDO = DP + 4;                 // fp32 staging row stride

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  const uint32_t sQ = smem_u32(smem), sK = sQ + Q_BYTES, sV = sK + Q_BYTES, sP = sV + Q_BYTES;
  __shared__ __align__(8) uint64_t bar_s, bar_o, bar_k, bar_v;
  __shared__ uint32_t tmem_base_s;
  __shared__ int err_s;
  __shared__ float m_s[kTQ], l_s[kTQ];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  unsigned long long* tr = p.trace ? p.trace + 16 * (blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z)) : nullptr;
#define PB_STAMP(i) do { if (tr && tid == 0) tr[i] = globaltimer_ns(); } while (0)
  PB_STAMP(0);
  const int nsplit = p.splits;
  const int b = blockIdx.z / nsplit, split = blockIdx.z % nsplit;
  const int kvh = blockIdx.y, G = p.group;
  const int q_len = p.q_len[b], kv_len = p.kv_len[b], q_start = p.q_start[b], kv_base = p.kv_indptr[b];
  const int rows_total = q_len * G, row0 = blockIdx.x * kTQ;
  const bool cta_live = row0 < rows_total;   // same for every CTA of the cluster

  if (tid == 0) {
    mbar_init(&bar_s, 1);
    mbar_init(&bar_o, 1);
    mbar_init(&bar_k, 1);
    mbar_init(&bar_v, 1);
    err_s = 0;
    mbar_fence_init();
  }
  if (warp == 4) {
    tmem_alloc(&tmem_base_s, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_s;
  pdl_launch_dependents();
  pdl_wait();
  PB_STAMP(1);

  float m_run = -INFINITY, l_run = 0.f;       // softmax threads: tid = row in tile
  const int my_tok = (row0 + tid) / G;
  int n_done = 0;

  if (cta_live) {
    int n_chunks = (kv_len + kTK - 1) / kTK;
    const int causal_off = kv_len - q_len;
    if (p.causal) {
      const int last_tok = min(q_len - 1, (row0 + kTQ - 1) / G);
      n_chunks = min(n_chunks, max(0, (last_tok + causal_off + 1 + kTK - 1) / kTK));
    }
    const int cps = (n_chunks + nsplit - 1) / nsplit;
    const int c_begin = split * cps, c_end = min(n_chunks, c_begin + cps);

    auto load_rows = [&](uint32_t dst, const __nv_bfloat16* base, int chunk, bool is_q) {
      for (int i = tid; i < 128 * CH; i += kTcThreads) {
        const int r = i / CH, c = i % CH;
        bool ok = c * 8 < p.head_dim;
        const __nv_bfloat16* src = base;
        if (is_q) {
          const int row = row0 + r;
          ok = ok && row < rows_total;
          if (ok) src = base + size_t(q_start + row / G) * p.q_tok_stride +
                        size_t(kvh * G + row % G) * p.q_head_stride + c * 8;
        } else {
          const int j = chunk * kTK + r;
          ok = ok && j < kv_len;
          if (ok) {
            const size_t rowi = p.kv_indices ? size_t(p.kv_indices[kv_base + j]) : size_t(kv_base + j);
            src = base + rowi * p.kv_row_stride + size_t(kvh) * p.kv_head_stride + c * 8;
          }
        }
        cp16(dst + sw_off(r, c), src, ok);
      }
      cp_commit();
    };

    // TMA path (dense q, contiguous KV): one thread issues DB box loads per operand; the
    // boxes are (64 d) x (G heads) x (128/G tokens) for Q and (64 d) x 1 x 128 rows for K/V,
    // columns past head_dim and rows past the tensor are zero-filled by the hardware.
    auto tma_q_k = [&](int chunk, bool with_q) {
      if (tid == 0) {
        mbar_expect_tx(&bar_k, uint32_t((with_q ? 2 : 1) * Q_BYTES));
        for (int blk = 0; blk < DB; ++blk) {
          if (with_q) tma_load_3d(sQ + blk * kBlkBytes, &tmQ, &bar_k, blk * 64, kvh * G, q_start + row0 / G);
          tma_load_3d(sK + blk * kBlkBytes, &tmK, &bar_k, blk * 64, kvh, kv_base + chunk * kTK);
        }
      }
    };
    auto tma_v = [&](int chunk) {
      if (tid == 0) {
        mbar_expect_tx(&bar_v, uint32_t(Q_BYTES));
        for (int blk = 0; blk < DB; ++blk)
          tma_load_3d(sV + blk * kBlkBytes, &tmV, &bar_v, blk * 64, kvh, kv_base + chunk * kTK);
      }
    };
    if (c_begin < c_end) {
      if (use_tma) {
        tma_q_k(c_begin, true);
        tma_v(c_begin);
      } else {
        load_rows(sQ, p.q, 0, true);
        load_rows(sK, p.k, c_begin, false);
        load_rows(sV, p.v, c_begin, false);
      }
    }
    const float scale_log2 = p.sm_scale * 1.4426950408889634f;
    const uint32_t idesc_s = make_idesc_f16(kTQ, kTK, 1);
    const uint32_t idesc_o = make_idesc_f16_bmn(kTQ, DP, 1);
    const uint32_t lane_addr = tmem + (uint32_t((warp & 3) * 32) << 16);

    for (int ch = c_begin; ch < c_end; ++ch) {
      const uint32_t ph = uint32_t(n_done & 1);
      // ---- operands of this chunk are in shared memory
      if (use_tma) {
        if (warp == 4) {
          if (!mbar_wait(&bar_k, ph)) err_s = kStatusTimeoutFull;
          if (!mbar_wait(&bar_v, ph)) err_s = kStatusTimeoutFull;
        }
      } else {
        cp_wait_all();
        fence_proxy_async_smem();
      }
      __syncthreads();
      if (ch == c_begin) PB_STAMP(2);
      if (err_s) break;
      // ---- S = Q K^T
      if (warp == 4) {
        tc_fence_after();
        if (lane == 0) {
#pragma unroll
          for (int kk = 0; kk < DP / 16; ++kk) {
            const uint64_t dq = make_smem_desc_sw128(sQ + (kk >> 2) * kBlkBytes) + 2 * (kk & 3);
            const uint64_t dk = make_smem_desc_sw128(sK + (kk >> 2) * kBlkBytes) + 2 * (kk & 3);
            umma_f16(tmem, dq, dk, idesc_s, kk != 0);
          }
          umma_commit(&bar_s);
        }
        __syncwarp();
      }
      // ---- softmax over the chunk (warps 0-3, one row per thread)
      if (warp < 4) {
        if (!mbar_wait(&bar_s, ph)) err_s = kStatusTimeoutAcc;
        tc_fence_after();
        const int jbase = ch * kTK;
        int jlim = kv_len;                                 // first masked kv index for this row
        if (p.causal) jlim = min(jlim, my_tok + causal_off + 1);
        int jlo = 0;                                       // first visible kv index (sliding window)
        if constexpr (EXTRA) {
          if (p.window > 0) jlo = max(0, my_tok + causal_off - p.window + 1);
        }
        // score in the log2 domain; with a soft cap: cap * tanh(score / cap) first
        const float cap = EXTRA ? p.soft_cap : 0.f, inv_cap = cap > 0.f ? 1.f / cap : 0.f;
        auto score = [&](uint32_t raw) {
          if constexpr (EXTRA) {
            if (cap > 0.f) return cap * tanhf(__uint_as_float(raw) * p.sm_scale * inv_cap) * 1.4426950408889634f;
          }
          return __uint_as_float(raw) * scale_log2;
        };
        auto seen = [&](int j) { return EXTRA ? (j < jlim && j >= jlo) : j < jlim; };
        float mx = -INFINITY;
#pragma unroll 1
        for (int c = 0; c < kTK; c += 32) {
          uint32_t r[32];
          tmem_ld_32x32(lane_addr + c, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (seen(jbase + c + j)) mx = fmaxf(mx, score(r[j]));
        }
        const float m_new = fmaxf(m_run, mx);
        const float m_use = m_new == -INFINITY ? 0.f : m_new;
        const float corr = exp2f(m_run - m_use);
        float sum = 0.f;
#pragma unroll 1
        for (int c = 0; c < kTK; c += 32) {
          uint32_t r[32];
          tmem_ld_32x32(lane_addr + c, r);
          tmem_ld_wait();
#pragma unroll
          for (int q8 = 0; q8 < 4; ++q8) {
            uint32_t pk[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int j0 = c + q8 * 8 + 2 * e;
              const float p0 = seen(jbase + j0) ? exp2f(score(r[q8 * 8 + 2 * e]) - m_use) : 0.f;
              const float p1 = seen(jbase + j0 + 1) ? exp2f(score(r[q8 * 8 + 2 * e + 1]) - m_use) : 0.f;
              sum += p0 + p1;
              __nv_bfloat162 pb2 = __floats2bfloat162_rn(p0, p1);
              pk[e] = *reinterpret_cast<uint32_t*>(&pb2);
            }
            const uint32_t dst = sP + sw_off(tid, (c >> 3) + q8);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(pk[0]), "r"(pk[1]),
                         "r"(pk[2]), "r"(pk[3]) : "memory");
          }
        }
        l_run = l_run * corr + sum;
        // ---- O was accumulated against the old max: rescale it in tensor memory
        // (tcgen05.ld / st are warp-collective: the decision must be warp-uniform)
        if (__any_sync(0xffffffffu, n_done > 0 && corr != 1.f)) {
#pragma unroll 1
          for (int c = 0; c < DP; c += 32) {
            uint32_t r[32];
            tmem_ld_32x32(lane_addr + O_COL + c, r);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) * corr);
            tmem_st_32x32(lane_addr + O_COL + c, r);
          }
          tmem_st_wait();
        }
        m_run = m_new;
        fence_proxy_async_smem();   // P writes -> visible to the tensor core
        tc_fence_before();
      }
      __syncthreads();
      if (ch == c_begin) PB_STAMP(3);
      if (err_s) break;
      // K is free: start fetching the next chunk's K while P V runs
      if (ch + 1 < c_end) {
        if (use_tma) tma_q_k(ch + 1, false); else load_rows(sK, p.k, ch + 1, false);
      }
      // ---- O += P V
      if (warp == 4) {
        tc_fence_after();
        if (lane == 0) {
#pragma unroll
          for (int kk = 0; kk < kTK / 16; ++kk) {
            const uint64_t dp = make_smem_desc_sw128(sP + (kk >> 2) * kBlkBytes) + 2 * (kk & 3);
            const uint64_t dv = make_smem_desc_sw128_mn(sV + kk * 2048, kBlkBytes, 1024);
            umma_f16(tmem + O_COL, dp, dv, idesc_o, (n_done > 0 || kk != 0) ? 1u : 0u);
          }
          umma_commit(&bar_o);
        }
        __syncwarp();
      }
      if (!mbar_wait(&bar_o, ph)) err_s = kStatusTimeoutAcc;   // P, V (and S) are free again
      tc_fence_after();
      __syncthreads();
      if (ch == c_begin) PB_STAMP(4);
      if (err_s) break;
      if (ch + 1 < c_end) {
        if (use_tma) tma_v(ch + 1); else load_rows(sV, p.v, ch + 1, false);
      }
      ++n_done;
    }
    cp_wait_all();
  }
  __syncthreads();
  PB_STAMP(5);
  const int err = err_s;

  // ---------------- write-out
  const uint32_t so_addr = smem_u32(smem), m_addr = smem_u32(m_s), l_addr = smem_u32(l_s);
  if (nsplit == 1) {
    // No split: the thread that owns a row normalises it straight out of tensor memory.
    if (cta_live && !err && warp < 4) {
      const int row = row0 + tid;
      const bool live_row = row < rows_total;
      const uint32_t lane_addr = tmem + (uint32_t((warp & 3) * 32) << 16);
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      __nv_bfloat16* dst = p.out;
      if (live_row) dst += size_t(q_start + row / G) * p.o_tok_stride + size_t(kvh * G + row % G) * p.o_head_stride;
#pragma unroll 1
      for (int c = 0; c < DP; c += 32) {
        uint32_t r[32];
        if (n_done > 0) {
          tc_fence_after();
          tmem_ld_32x32(lane_addr + O_COL + c, r);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = 0u;
        }
        if (live_row) {
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            if (c + 8 * t < p.head_dim) {
              uint4 o;
              __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
              for (int e = 0; e < 4; ++e)
                o2[e] = __floats2bfloat162_rn(__uint_as_float(r[8 * t + 2 * e]) * inv,
                                              __uint_as_float(r[8 * t + 2 * e + 1]) * inv);
              *reinterpret_cast<uint4*>(dst + c + 8 * t) = o;
            }
          }
        }
      }
      tc_fence_before();
    }
    PB_STAMP(8);
  } else {
    // Split KV: stage this CTA's partial (O, m, l) in its own shared memory, then every CTA
    // finishes 128/S rows by pulling the S partial rows through distributed shared memory.
    // One warp per row, lanes along the columns (coalesced remote reads, all S of them in
    // flight together), row-invariant work (weights, output pointer) done once per row.
    float* so = reinterpret_cast<float*>(smem);
    if (cta_live && !err && warp < 4) {
      const uint32_t lane_addr = tmem + (uint32_t((warp & 3) * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < DP; c += 32) {
        uint32_t r[32];
        if (n_done > 0) {
          tc_fence_after();
          tmem_ld_32x32(lane_addr + O_COL + c, r);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = 0u;
        }
        float4* dst = reinterpret_cast<float4*>(so + tid * LDO + c);
#pragma unroll
        for (int t = 0; t < 8; ++t)
          dst[t] = make_float4(__uint_as_float(r[4 * t]), __uint_as_float(r[4 * t + 1]),
                               __uint_as_float(r[4 * t + 2]), __uint_as_float(r[4 * t + 3]));
      }
      m_s[tid] = m_run;
      l_s[tid] = l_run;
      tc_fence_before();
    }
    __syncthreads();
    PB_STAMP(7);
    cluster_sync_all();
    PB_STAMP(8);
    if (cta_live && !err) {
      const int rpc = kTQ / nsplit;
      for (int lr = warp; lr < rpc; lr += kTcThreads / 32) {
        const int r = split * rpc + lr;
        const int row = row0 + r;
        if (row >= rows_total) continue;
        float mv[8], wv[8];
        float mmax = -INFINITY, lsum = 0.f;
#pragma unroll
        for (int s2 = 0; s2 < 8; ++s2)
          if (s2 < nsplit) { mv[s2] = ld_dsmem_f1(map_to_cta(m_addr + r * 4, s2)); mmax = fmaxf(mmax, mv[s2]); }
#pragma unroll
        for (int s2 = 0; s2 < 8; ++s2) {
          wv[s2] = 0.f;
          if (s2 < nsplit && mmax != -INFINITY) {
            wv[s2] = exp2f(mv[s2] - mmax);
            lsum += ld_dsmem_f1(map_to_cta(l_addr + r * 4, s2)) * wv[s2];
          }
        }
        const float inv = lsum > 0.f ? 1.f / lsum : 0.f;
        __nv_bfloat16* dst = p.out + size_t(q_start + row / G) * p.o_tok_stride +
                             size_t(kvh * G + row % G) * p.o_head_stride;
#pragma unroll
        for (int c = lane * 4; c < DP; c += 128) {
          if (c >= p.head_dim) continue;
          float4 ov[8];
#pragma unroll
          for (int s2 = 0; s2 < 8; ++s2)
            if (s2 < nsplit) ov[s2] = ld_dsmem_f4(map_to_cta(so_addr + uint32_t(r * LDO + c) * 4u, s2));
          float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
          for (int s2 = 0; s2 < 8; ++s2)
            if (s2 < nsplit) {
              acc.x += ov[s2].x * wv[s2]; acc.y += ov[s2].y * wv[s2];
              acc.z += ov[s2].z * wv[s2]; acc.w += ov[s2].w * wv[s2];
            }
          const __nv_bfloat162 o01 = __floats2bfloat162_rn(acc.x * inv, acc.y * inv);
          const __nv_bfloat162 o23 = __floats2bfloat162_rn(acc.z * inv, acc.w * inv);
          uint2 raw;
          raw.x = *reinterpret_cast<const uint32_t*>(&o01);
          raw.y = *reinterpret_cast<const uint32_t*>(&o23);
          *reinterpret_cast<uint2*>(dst + c) = raw;
        }
      }
    }
  }
  PB_STAMP(9);
  if (err && tid == 0 && status) atomicCAS(status, 0, err);
  if (nsplit > 1) cluster_sync_all();  // peers may still be reading this CTA's partial rows
  tc_fence_before();
  __syncthreads();
  if (warp == 4) tmem_dealloc(tmem, TMEM_COLS);
}

template <int DB, bool EXTRA>
static cudaError_t attn_tc_launch_db(const AttnParams& p, cudaStream_t stream) {
  auto kern = attn_tc_kernel<DB, EXTRA>;
  const size_t smem = size_t(3 * DB + 2) * kBlkBytes + 1024;
  static bool attr_done = false;
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    if (e != cudaSuccess) return e;
    attr_done = true;
  }
  // TMA needs dense, 16-byte aligned operands and a group size that tiles 128 rows
  CUtensorMap tq, tk, tv;
  memset(&tq, 0, sizeof(tq)); memset(&tk, 0, sizeof(tk)); memset(&tv, 0, sizeof(tv));
  int use_tma = 0;
  const auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
  if (!p.kv_indices && p.q_rows > 0 && p.kv_rows > 0 && (kTQ % p.group) == 0 && al16(p.q) && al16(p.k) &&
      al16(p.v)) {
    const int Hq = p.num_kv_heads * p.group;
    use_tma = make_tmap_3d_bf16(&tq, p.q, p.head_dim, Hq, p.q_rows, p.q_head_stride, p.q_tok_stride,
                                p.group, kTQ / p.group) &&
              make_tmap_3d_bf16(&tk, p.k, p.head_dim, p.num_kv_heads, p.kv_rows, p.kv_head_stride,
                                p.kv_row_stride, 1, kTK) &&
              make_tmap_3d_bf16(&tv, p.v, p.head_dim, p.num_kv_heads, p.kv_rows, p.kv_head_stride,
                                p.kv_row_stride, 1, kTK);
  }
  const int max_rows = p.max_q_len * p.group;
  return launch_kernel(kern, dim3((max_rows + kTQ - 1) / kTQ, p.num_kv_heads, p.batch * p.splits),
                       dim3(kTcThreads), smem, stream, p.splits, p, kernel_status_ptr(), tq, tk, tv, use_tma);
}

cudaError_t attn_tc_launch(const AttnParams& p, cudaStream_t stream) {
  if (p.head_dim % 8 || p.head_dim > 256 || p.head_dim <= 0) return cudaErrorInvalidValue;
  if (p.splits != 1 && p.splits != 2 && p.splits != 4 && p.splits != 8) return cudaErrorInvalidValue;
  if (p.batch <= 0 || p.max_q_len <= 0 || p.group <= 0) return cudaErrorInvalidValue;
  if ((p.q_tok_stride | p.q_head_stride | p.kv_row_stride | p.kv_head_stride | p.o_tok_stride |
       p.o_head_stride) % 8)
    return cudaErrorInvalidValue;
  if (p.window > 0 || p.soft_cap > 0.f) {
    if (p.head_dim <= 64) return attn_tc_launch_db<1, true>(p, stream);
    if (p.head_dim <= 128) return attn_tc_launch_db<2, true>(p, stream);
    return attn_tc_launch_db<4, true>(p, stream);
  }
  if (p.head_dim <= 64) return attn_tc_launch_db<1, false>(p, stream);
  if (p.head_dim <= 128) return attn_tc_launch_db<2, false>(p, stream);
  return attn_tc_launch_db<4, false>(p, stream);
}

}  // namespace pb

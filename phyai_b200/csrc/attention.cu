// Ragged / paged flash attention for sm_100a (bf16 in, fp32 softmax + accumulate).
//
// One kernel covers every attention shape of the served models:
//   * SigLIP vision blocks: dense, non-causal, head_dim 72 (zero-padded to 128);
//   * Gemma prefix self-attention over the paged KV pool (page size 1), 8 query
//     heads sharing 1 KV head: the heads of a group are folded into the query
//     tile rows, so K/V tiles are fetched once per group instead of once per head;
//   * action-expert joint attention: 50 query tokens against prefix + suffix
//     slots; the KV range is split over a thread-block cluster (1,1,S) and the S
//     partial (max, sum, O) triples are merged through distributed shared memory;
//   * Cosmos3 UND (causal) and GEN (non-causal over [text | gen] KV) attention.
//
// Sequence b reads q rows [q_start[b], q_start[b]+q_len[b]) and KV entries
// kv_indptr[b] + [0, kv_len[b]); an entry is a row of the K/V pools, either
// directly (kv_indices == null) or through kv_indices (paged, page size 1).
//
// Capability parity: phyai/src/phyai/layers/attention/ar/backends/flashinfer.py:68-177,
// phyai/src/phyai/layers/attention/diffusion/backends/flashinfer.py:78-193,
// phyai/src/phyai/layers/attention/attention/backends/{flashinfer,sdpa}.py.
#include "attention.cuh"

#include "gemm.cuh"
#include "launch.cuh"
#include "ptx.cuh"

namespace pb {

namespace {

constexpr int kBM = 64;   // query rows per CTA (16 per warp)
constexpr int kBN = 64;   // KV entries per tile
constexpr int kAttnThreads = 128;

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  const int sz = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(sz)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                        uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                          uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Byte offset of 16-byte chunk `chunk` of row `row` in a [rows][DP] bf16 tile whose
// chunks are XOR-swizzled by the row so ldmatrix reads hit distinct banks.
template <int DP>
__device__ __forceinline__ uint32_t tile_off(int row, int chunk) {
  return uint32_t(row) * (DP * 2) + uint32_t((chunk ^ (row & 7)) << 4);
}

}  // namespace

template <int DP>
__global__ void __launch_bounds__(kAttnThreads)
attn_kernel(AttnParams p) {
  constexpr int CHUNKS = DP / 8;          // 16-byte chunks per row
  constexpr int TILE_BYTES = kBN * DP * 2;
  constexpr int KSTEPS = DP / 16;
  constexpr int ONB = DP / 8;             // output n-blocks of 8 columns
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) &
                                             ~uintptr_t(127));
  // layout: Q | K0 | K1 | V0 | V1 ; after the loop K0.. is reused as fp32 O staging.
  const uint32_t sQ = smem_u32(smem);
  const uint32_t sK = sQ + kBM * DP * 2;
  const uint32_t sV = sK + 2 * TILE_BYTES;
  __shared__ float m_s[kBM];
  __shared__ float l_s[kBM];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int nsplit = p.splits;
  const int b = blockIdx.z / nsplit;
  const int split = blockIdx.z % nsplit;
  const int kvh = blockIdx.y;
  const int G = p.group;
  const int q_len = p.q_len[b], kv_len = p.kv_len[b];
  const int q_start = p.q_start[b];
  const int kv_base = p.kv_indptr[b];
  const int rows_total = q_len * G;      // (token, head-in-group) pairs
  const int row0 = blockIdx.x * kBM;
  const bool cta_live = row0 < rows_total;   // uniform across the cluster (same x, b)

  pdl_launch_dependents();
  pdl_wait();

  float o_acc[ONB][4];
#pragma unroll
  for (int i = 0; i < ONB; ++i) { o_acc[i][0] = o_acc[i][1] = o_acc[i][2] = o_acc[i][3] = 0.f; }
  float m_run[2] = {-INFINITY, -INFINITY};
  float l_run[2] = {0.f, 0.f};

  if (cta_live) {
    // ---- KV tile range of this split
    int n_tiles = (kv_len + kBN - 1) / kBN;
    const int causal_off = kv_len - q_len;
    if (p.causal) {
      const int last_tok = min(q_len - 1, (row0 + kBM - 1) / G);
      const int lim = last_tok + causal_off + 1;  // exclusive kv bound for this q tile
      n_tiles = min(n_tiles, max(0, (lim + kBN - 1) / kBN));
    }
    const int tps = (n_tiles + nsplit - 1) / nsplit;
    const int t_begin = split * tps;
    const int t_end = min(n_tiles, t_begin + tps);

    // ---- load Q tile (rows beyond rows_total are zero)
    for (int c = tid; c < kBM * CHUNKS; c += kAttnThreads) {
      const int r = c / CHUNKS, ch = c % CHUNKS;
      const int row = row0 + r;
      const bool ok = row < rows_total && ch * 8 < p.head_dim;
      const int tok = ok ? row / G : 0, hg = ok ? row % G : 0;
      const __nv_bfloat16* src = p.q + size_t(q_start + tok) * p.q_tok_stride +
                                 size_t(kvh * G + hg) * p.q_head_stride + ch * 8;
      cp_async16(sQ + tile_off<DP>(r, ch), src, ok);
    }
    cp_async_commit();

    auto load_kv = [&](int t, int stage) {
      for (int c = tid; c < kBN * CHUNKS; c += kAttnThreads) {
        const int r = c / CHUNKS, ch = c % CHUNKS;
        const int j = t * kBN + r;
        const bool ok = j < kv_len && ch * 8 < p.head_dim;
        size_t rowi = 0;
        if (ok) rowi = p.kv_indices ? size_t(p.kv_indices[kv_base + j]) : size_t(kv_base + j);
        const size_t off = rowi * p.kv_row_stride + size_t(kvh) * p.kv_head_stride + ch * 8;
        cp_async16(sK + stage * TILE_BYTES + tile_off<DP>(r, ch), p.k + off, ok);
        cp_async16(sV + stage * TILE_BYTES + tile_off<DP>(r, ch), p.v + off, ok);
      }
      cp_async_commit();
    };

    if (t_begin < t_end) load_kv(t_begin, 0);
    const float scale_log2 = p.sm_scale * 1.4426950408889634f;
    const int g4 = lane >> 2, t4 = lane & 3;
    // rows of this thread inside the CTA tile
    const int r_lo = warp * 16 + g4, r_hi = r_lo + 8;
    const int tok_lo = (row0 + r_lo) / G, tok_hi = (row0 + r_hi) / G;

    for (int t = t_begin; t < t_end; ++t) {
      const int stage = (t - t_begin) & 1;
      if (t + 1 < t_end) {
        load_kv(t + 1, stage ^ 1);
        cp_async_wait<1>();
      } else {
        cp_async_wait<0>();
      }
      __syncthreads();

      // ---- S = Q K^T for this warp's 16 rows x 64 kv
      float s[kBN / 8][4];
#pragma unroll
      for (int i = 0; i < kBN / 8; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f; }
      const uint32_t kb = sK + stage * TILE_BYTES;
#pragma unroll
      for (int ks = 0; ks < KSTEPS; ++ks) {
        uint32_t a0, a1, a2, a3;
        {
          const int r = warp * 16 + (lane & 15);
          const int ch = ks * 2 + (lane >> 4);
          ldsm_x4(sQ + tile_off<DP>(r, ch), a0, a1, a2, a3);
        }
#pragma unroll
        for (int nb = 0; nb < kBN / 16; ++nb) {
          // two n-blocks (16 kv rows) x 16 d: matrices (n0-7,d0-7),(n0-7,d8-15),(n8-15,d0-7),(n8-15,d8-15)
          uint32_t b0, b1, b2, b3;
          const int r = nb * 16 + (lane & 7) + ((lane >> 4) << 3);
          const int ch = ks * 2 + ((lane >> 3) & 1);
          ldsm_x4(kb + tile_off<DP>(r, ch), b0, b1, b2, b3);
          mma_bf16(s[2 * nb], a0, a1, a2, a3, b0, b1);
          mma_bf16(s[2 * nb + 1], a0, a1, a2, a3, b2, b3);
        }
      }

      // ---- mask + online softmax (log2 domain)
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int i = 0; i < kBN / 8; ++i) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int j = t * kBN + i * 8 + t4 * 2 + (e & 1);
          const int tok = (e < 2) ? tok_lo : tok_hi;
          bool ok = j < kv_len;
          if (p.causal) ok = ok && (j <= tok + causal_off);
          const float v = ok ? s[i][e] * scale_log2 : -INFINITY;
          s[i][e] = v;
          mx[e >> 1] = fmaxf(mx[e >> 1], v);
        }
      }
      float corr[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
        const float m_new = fmaxf(m_run[h], mx[h]);
        const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
        corr[h] = exp2f(m_run[h] - m_use);   // m_run = -inf -> 0
        m_run[h] = m_new;
        mx[h] = m_use;
        l_run[h] *= corr[h];
      }
      float rs[2] = {0.f, 0.f};
#pragma unroll
      for (int i = 0; i < kBN / 8; ++i) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float pv = exp2f(s[i][e] - mx[e >> 1]);
          s[i][e] = pv;
          rs[e >> 1] += pv;
        }
      }
      l_run[0] += rs[0];
      l_run[1] += rs[1];
#pragma unroll
      for (int i = 0; i < ONB; ++i) {
        o_acc[i][0] *= corr[0]; o_acc[i][1] *= corr[0];
        o_acc[i][2] *= corr[1]; o_acc[i][3] *= corr[1];
      }

      // ---- O += P V
      const uint32_t vb = sV + stage * TILE_BYTES;
#pragma unroll
      for (int kk = 0; kk < kBN / 16; ++kk) {
        const uint32_t a0 = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
        const uint32_t a1 = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
        const uint32_t a2 = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
        const uint32_t a3 = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
        for (int nb = 0; nb < ONB / 2; ++nb) {
          // V rows kk*16..+15 (k), d columns nb*16..+15 (n); transposed 8x8 loads:
          // matrices (k0-7,n0-7),(k8-15,n0-7),(k0-7,n8-15),(k8-15,n8-15)
          uint32_t b0, b1, b2, b3;
          const int r = kk * 16 + (lane & 15);
          const int ch = nb * 2 + (lane >> 4);
          ldsm_x4_t(vb + tile_off<DP>(r, ch), b0, b1, b2, b3);
          mma_bf16(o_acc[2 * nb], a0, a1, a2, a3, b0, b1);
          mma_bf16(o_acc[2 * nb + 1], a0, a1, a2, a3, b2, b3);
        }
      }
      __syncthreads();  // tile buffers are rewritten by the next prefetch
    }
    cp_async_wait<0>();
    // row sums live split over the 4 lanes of a quad
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
      l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
    }
    __syncthreads();

    // ---- stage partial (O, m, l) in shared memory (fp32, row stride DP + 4)
    float* so = reinterpret_cast<float*>(smem + kBM * DP * 2);
    constexpr int LDO = DP + 4;
#pragma unroll
    for (int i = 0; i < ONB; ++i) {
      const int c = i * 8 + t4 * 2;
      *reinterpret_cast<float2*>(so + r_lo * LDO + c) = make_float2(o_acc[i][0], o_acc[i][1]);
      *reinterpret_cast<float2*>(so + r_hi * LDO + c) = make_float2(o_acc[i][2], o_acc[i][3]);
    }
    if (t4 == 0) {
      m_s[r_lo] = m_run[0]; l_s[r_lo] = l_run[0];
      m_s[r_hi] = m_run[1]; l_s[r_hi] = l_run[1];
    }
  }
  __syncthreads();
  if (nsplit > 1) cluster_sync_all();

  if (cta_live) {
    // ---- merge the splits: this CTA finishes rows [split*rpc, (split+1)*rpc)
    constexpr int LDO = DP + 4;
    const int rpc = kBM / nsplit;
    const uint32_t so_addr = sQ + kBM * DP * 2;
    const uint32_t m_addr = smem_u32(m_s), l_addr = smem_u32(l_s);
    constexpr int G4 = DP / 4;
    for (int g = tid; g < rpc * G4; g += kAttnThreads) {
      const int r = split * rpc + g / G4;
      const int c = (g % G4) * 4;
      const int row = row0 + r;
      if (row >= rows_total || c >= p.head_dim) continue;
      float mmax = -INFINITY;
      for (int s2 = 0; s2 < nsplit; ++s2) {
        const float mv = nsplit == 1 ? m_s[r] : ld_dsmem_f1(map_to_cta(m_addr + r * 4, s2));
        mmax = fmaxf(mmax, mv);
      }
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      float lsum = 0.f;
      if (mmax != -INFINITY) {
        for (int s2 = 0; s2 < nsplit; ++s2) {
          float mv, lv;
          float4 ov;
          if (nsplit == 1) {
            mv = m_s[r]; lv = l_s[r];
            ov = *reinterpret_cast<const float4*>(
                reinterpret_cast<const float*>(smem + kBM * DP * 2) + r * LDO + c);
          } else {
            mv = ld_dsmem_f1(map_to_cta(m_addr + r * 4, s2));
            lv = ld_dsmem_f1(map_to_cta(l_addr + r * 4, s2));
            ov = ld_dsmem_f4(map_to_cta(so_addr + uint32_t(r * LDO + c) * 4u, s2));
          }
          const float w = exp2f(mv - mmax);
          lsum += lv * w;
          acc.x += ov.x * w; acc.y += ov.y * w; acc.z += ov.z * w; acc.w += ov.w * w;
        }
      }
      const float inv = lsum > 0.f ? 1.f / lsum : 0.f;
      const int tok = row / G, hg = row % G;
      __nv_bfloat16* dst = p.out + size_t(q_start + tok) * p.o_tok_stride +
                           size_t(kvh * G + hg) * p.o_head_stride + c;
      __nv_bfloat162 o01 = __floats2bfloat162_rn(acc.x * inv, acc.y * inv);
      __nv_bfloat162 o23 = __floats2bfloat162_rn(acc.z * inv, acc.w * inv);
      uint2 raw;
      raw.x = *reinterpret_cast<uint32_t*>(&o01);
      raw.y = *reinterpret_cast<uint32_t*>(&o23);
      *reinterpret_cast<uint2*>(dst) = raw;
    }
  }
  if (nsplit > 1) cluster_sync_all();
}

template <int DP>
static cudaError_t attn_launch_dp(const AttnParams& p, cudaStream_t stream) {
  auto kern = attn_kernel<DP>;
  const size_t smem = size_t(kBM) * DP * 2 + 4 * size_t(kBN) * DP * 2 + 128;
  static bool attr_done = false;
  if (!attr_done) {
    cudaError_t e =
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    if (e != cudaSuccess) return e;
    attr_done = true;
  }
  const int max_rows = p.max_q_len * p.group;
  return launch_kernel(kern, dim3((max_rows + kBM - 1) / kBM, p.num_kv_heads, p.batch * p.splits),
                       dim3(kAttnThreads), smem, stream, p.splits, p);
}

cudaError_t attn_launch(const AttnParams& p, cudaStream_t stream) {
  if (p.head_dim % 8 || p.head_dim > 256 || p.head_dim <= 0) return cudaErrorInvalidValue;
  if (p.splits != 1 && p.splits != 2 && p.splits != 4 && p.splits != 8) return cudaErrorInvalidValue;
  if (p.batch <= 0 || p.max_q_len <= 0 || p.group <= 0) return cudaErrorInvalidValue;
  if ((p.q_tok_stride | p.q_head_stride | p.kv_row_stride | p.kv_head_stride | p.o_tok_stride |
       p.o_head_stride) % 8)
    return cudaErrorInvalidValue;
  if (p.head_dim <= 128) return attn_launch_dp<128>(p, stream);
  return attn_launch_dp<256>(p, stream);
}

}  // namespace pb

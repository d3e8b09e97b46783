// Reduce + epilogue + store pass of the tcgen05 GEMM (included by gemm.cu).
//
// The accumulator tile sits in shared memory in output orientation: TM rows of TN
// fp32 values with row stride LDS. One warp owns a row at a time, a lane owns four
// consecutive columns, so every global access of a warp is one contiguous segment
// and all row-invariant work (row scale, residual row pointer, output row pointer)
// is hoisted out of the column loop. With a split-K cluster the S partial tiles are
// summed through distributed shared memory (all S loads are issued before the first
// add, so their latencies overlap).
#pragma once
#include "comm.cuh"
#include "gemm.cuh"
#include "ptx.cuh"

namespace pb {

struct EpiParams {
  void* out;
  int ldo, M, N;
  const __nv_bfloat16* bias;
  const __nv_bfloat16* residual;
  int ldr, res_mod;
  const __nv_bfloat16* col_gate;
  const float* row_scale;
  float* sumsq;
  const float* a_scale;
  const float* w_scale;
  int act, glu, out_fp32;
  float rs_inv_dim = 0.f, rs_eps = 0.f;   // > 0: row_scale holds a sum of squares, scale = rsqrt(ss * inv_dim + eps)
  const RopeEpi* rope = nullptr;          // non-null: rotate + scatter instead of storing to `out`
  float* zero = nullptr;                  // optional fp32 scratch cleared by the first CTA (sum-of-squares
  int zero_n = 0;                         // accumulators that a later launch adds into)
  int* status = nullptr;                  // debug build: where a failed index check is recorded
  // second output of a plain (non-gated) bf16 store: out2[m, n] = bf16(stored value * (1 + col_scale2[n])), the input
  // of a norm whose column factor is applied here and whose per-row factor the consuming GEMM applies (row_rms)
  __nv_bfloat16* out2 = nullptr;
  const __nv_bfloat16* col_scale2 = nullptr;
  int ldo2 = 0;
};

__device__ __forceinline__ float epi_act(float v, int act) {
  switch (act) {
    case 1: return gelu_tanh_f(v);
    case 2: return silu_f(v);
    case 3: return gelu_erf_f(v);
    default: return v;
  }
}
__device__ __forceinline__ void ld_bf16x4(const __nv_bfloat16* p, float (&f)[4]) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  f[0] = __uint_as_float(raw.x << 16); f[1] = __uint_as_float(raw.x & 0xffff0000u);
  f[2] = __uint_as_float(raw.y << 16); f[3] = __uint_as_float(raw.y & 0xffff0000u);
}

template <int ACT>
__device__ __forceinline__ float epi_act_c(float v) {
  if constexpr (ACT == 1) return gelu_tanh_f(v);
  else if constexpr (ACT == 2) return silu_f(v);
  else if constexpr (ACT == 3) return gelu_erf_f(v);
  else return v;
}

// ACT, GLU and AUX are compile-time: a run-time switch inside the element loop gets
// if-converted (every element then pays for every activation), and with one or two
// warps per scheduler every uniform branch is a pipeline bubble. AUX = false is the
// plain "convert and store" path with no optional operand at all.
//
// Loop order: a lane owns 4 consecutive columns (column-invariant operands are read
// once), and walks the rows of its warp four at a time with all accumulator loads
// issued before the first use, so their latencies overlap.
template <int TN, int ACT, bool GLU, bool AUX>
__device__ __forceinline__ void epilogue_pass_t(const EpiParams& ep, const float* stg,
                                              uint32_t stg_addr, int lds, int m0, int n0, int r0,
                                              int rows, int nsplit, int warp, int lane,
                                              int nwarps) {
  constexpr int U = 4;
  const int row_end = min(r0 + rows, ep.M - m0);
#pragma unroll
  for (int c = lane * 4; c < TN; c += 128) {
    const int n = n0 + c;
    if (n >= ep.N) continue;
    float bias4[4] = {0.f, 0.f, 0.f, 0.f}, gate4[4] = {1.f, 1.f, 1.f, 1.f}, ws4[4] = {1.f, 1.f, 1.f, 1.f};
    float cs4[4] = {0.f, 0.f, 0.f, 0.f};
    if constexpr (AUX) {
      if (ep.bias) ld_bf16x4(ep.bias + n, bias4);
      if constexpr (!GLU) {
        if (ep.out2) ld_bf16x4(ep.col_scale2 + n, cs4);
      }
      if (ep.w_scale) {
        const float4 w = *reinterpret_cast<const float4*>(ep.w_scale + n);
        ws4[0] = w.x; ws4[1] = w.y; ws4[2] = w.z; ws4[3] = w.w;
      }
      if (ep.col_gate) {
        if constexpr (GLU) {
          const __nv_bfloat162 g = *reinterpret_cast<const __nv_bfloat162*>(ep.col_gate + (n >> 1));
          gate4[0] = bf2f(g.x); gate4[1] = bf2f(g.y);
        } else {
          ld_bf16x4(ep.col_gate + n, gate4);
        }
      }
    }
    for (int row = r0 + warp; row < row_end; row += nwarps * U) {
      float v[U][4];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int rr = row + u * nwarps;
        v[u][0] = v[u][1] = v[u][2] = v[u][3] = 0.f;
        if (rr < row_end) {
          if (nsplit == 1) {
            const float4 a = *reinterpret_cast<const float4*>(stg + rr * lds + c);
            v[u][0] = a.x; v[u][1] = a.y; v[u][2] = a.z; v[u][3] = a.w;
          } else {
            const uint32_t off = stg_addr + uint32_t(rr * lds + c) * 4u;
            float4 part[8];
#pragma unroll
            for (int r = 0; r < 8; ++r)
              if (r < nsplit) part[r] = ld_dsmem_f4(map_to_cta(off, r));
#pragma unroll
            for (int r = 0; r < 8; ++r)
              if (r < nsplit) { v[u][0] += part[r].x; v[u][1] += part[r].y; v[u][2] += part[r].z; v[u][3] += part[r].w; }
          }
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int rr = row + u * nwarps;
        if (rr >= row_end) continue;
        const int m = m0 + rr;
        if (!PB_DEBUG_CHECK(m >= 0 && m < ep.M && n >= 0 && n < ep.N && ep.ldo >= (GLU ? ep.N / 2 : ep.N), ep.status)) continue;
        float* x = v[u];
        const __nv_bfloat16* res_row = nullptr;
        if constexpr (AUX) {
          float rscale = 1.f;
          if (ep.row_scale) {
            rscale = ep.row_scale[m];
            if (ep.rs_inv_dim > 0.f) rscale = rsqrtf(rscale * ep.rs_inv_dim + ep.rs_eps);
          }
          if (ep.a_scale) rscale *= ep.a_scale[m];
#pragma unroll
          for (int t = 0; t < 4; ++t) x[t] = x[t] * (rscale * ws4[t]) + bias4[t];
          if (ep.residual) res_row = ep.residual + size_t(ep.res_mod > 0 ? (m % ep.res_mod) : m) * ep.ldr;
        }
        float ss = 0.f;
        if constexpr (GLU) {
          float y0 = epi_act_c<ACT>(x[0]) * x[1], y1 = epi_act_c<ACT>(x[2]) * x[3];
          const int no = n >> 1;
          if constexpr (AUX) {
            y0 *= gate4[0]; y1 *= gate4[1];
            if (res_row) {
              const __nv_bfloat162 r2 = *reinterpret_cast<const __nv_bfloat162*>(res_row + no);
              y0 += bf2f(r2.x); y1 += bf2f(r2.y);
            }
          }
          if (AUX && ep.out_fp32) {
            *reinterpret_cast<float2*>(reinterpret_cast<float*>(ep.out) + size_t(m) * ep.ldo + no) = make_float2(y0, y1);
            ss = y0 * y0 + y1 * y1;
          } else {
            const __nv_bfloat162 o = __floats2bfloat162_rn(y0, y1);
            *reinterpret_cast<__nv_bfloat162*>(reinterpret_cast<__nv_bfloat16*>(ep.out) + size_t(m) * ep.ldo + no) = o;
            const float q0 = bf2f(o.x), q1 = bf2f(o.y);
            ss = q0 * q0 + q1 * q1;
          }
        } else {
          if constexpr (ACT != 0) {
#pragma unroll
            for (int t = 0; t < 4; ++t) x[t] = epi_act_c<ACT>(x[t]);
          }
          if constexpr (AUX) {
#pragma unroll
            for (int t = 0; t < 4; ++t) x[t] *= gate4[t];
            if (res_row) {
              float r4[4];
              ld_bf16x4(res_row + n, r4);
#pragma unroll
              for (int t = 0; t < 4; ++t) x[t] += r4[t];
            }
          }
          if (AUX && ep.out_fp32) {
            *reinterpret_cast<float4*>(reinterpret_cast<float*>(ep.out) + size_t(m) * ep.ldo + n) = make_float4(x[0], x[1], x[2], x[3]);
            ss = x[0] * x[0] + x[1] * x[1] + x[2] * x[2] + x[3] * x[3];
          } else {
            const __nv_bfloat162 o01 = __floats2bfloat162_rn(x[0], x[1]);
            const __nv_bfloat162 o23 = __floats2bfloat162_rn(x[2], x[3]);
            uint2 raw;
            raw.x = *reinterpret_cast<const uint32_t*>(&o01);
            raw.y = *reinterpret_cast<const uint32_t*>(&o23);
            *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(ep.out) + size_t(m) * ep.ldo + n) = raw;
            if constexpr (AUX) {
              // a norm consuming the sum of squares sees the rounded values
              const float q0 = bf2f(o01.x), q1 = bf2f(o01.y);
              const float q2 = bf2f(o23.x), q3 = bf2f(o23.y);
              ss = q0 * q0 + q1 * q1 + q2 * q2 + q3 * q3;
              if (ep.out2) {
                const __nv_bfloat162 s01 = __floats2bfloat162_rn(q0 * (1.f + cs4[0]), q1 * (1.f + cs4[1]));
                const __nv_bfloat162 s23 = __floats2bfloat162_rn(q2 * (1.f + cs4[2]), q3 * (1.f + cs4[3]));
                uint2 raw2;
                raw2.x = *reinterpret_cast<const uint32_t*>(&s01);
                raw2.y = *reinterpret_cast<const uint32_t*>(&s23);
                *reinterpret_cast<uint2*>(ep.out2 + size_t(m) * ep.ldo2 + n) = raw2;
              }
            }
          }
        }
        if constexpr (AUX) {
          if (ep.sumsq) {
            // lanes past the N edge skipped the column block: reduce over the active ones only
            const unsigned mask = __activemask();
            for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(mask, ss, o);
            if (lane == 0) atomicAdd(ep.sumsq + m, ss);
          }
        }
      }
    }
  }
}

// Push-mode store pass: the (cluster-reduced) accumulator rows of this CTA, rounded to
// bf16, go to slots[parity][rank] of every rank over NVLink with plain 8-byte stores (a
// warp writes 256 contiguous bytes of one row per destination). The caller signals the
// channel once every thread of the CTA is past this function.
template <int TN>
__device__ __forceinline__ void epilogue_push(const PushParams& pp, int parity, int M, int N,
                                              uint32_t stg_addr, const float* stg, int lds, int m0,
                                              int n0, int r0, int rows, int nsplit, int warp,
                                              int lane, int nwarps) {
  const int row_end = min(r0 + rows, M - m0);
  const size_t slot = size_t(pp.slots_off) + (size_t(parity) * pp.world + pp.rank) * size_t(pp.slot_stride);
#pragma unroll
  for (int c = lane * 4; c < TN; c += 128) {
    const int n = n0 + c;
    if (n >= N) continue;
    for (int rr = r0 + warp; rr < row_end; rr += nwarps) {
      float v0 = 0.f, v1 = 0.f, v2 = 0.f, v3 = 0.f;
      if (nsplit == 1) {
        const float4 a = *reinterpret_cast<const float4*>(stg + rr * lds + c);
        v0 = a.x; v1 = a.y; v2 = a.z; v3 = a.w;
      } else {
        const uint32_t off = stg_addr + uint32_t(rr * lds + c) * 4u;
        float4 part[8];
#pragma unroll
        for (int r = 0; r < 8; ++r)
          if (r < nsplit) part[r] = ld_dsmem_f4(map_to_cta(off, r));
#pragma unroll
        for (int r = 0; r < 8; ++r)
          if (r < nsplit) { v0 += part[r].x; v1 += part[r].y; v2 += part[r].z; v3 += part[r].w; }
      }
      const __nv_bfloat162 o01 = __floats2bfloat162_rn(v0, v1), o23 = __floats2bfloat162_rn(v2, v3);
      uint2 raw;
      raw.x = *reinterpret_cast<const uint32_t*>(&o01);
      raw.y = *reinterpret_cast<const uint32_t*>(&o23);
      const size_t off = slot + size_t(m0 + rr) * pp.ld + n;
      if (pp.rows_per_rank > 0) {
        // scattered: the owner's slot holds only its own rows, counted from its first row
        const int r = (m0 + rr) / pp.rows_per_rank;
        const size_t offs = slot + size_t(m0 + rr - r * pp.rows_per_rank) * pp.ld + n;
        *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(pp.data.p[r]) + offs) = raw;
      } else {
        for (int r = 0; r < pp.world; ++r)
          *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(pp.data.p[r]) + off) = raw;
      }
    }
  }
}

// Fused-QKV store pass (see RopeEpi): row scale and bias as in the generic pass, then q / k pairs
// are rotated in fp32 and written to their two half-head positions, v columns are copied.
template <int TN>
__device__ __forceinline__ void epilogue_rope(const EpiParams& ep, const float* stg, uint32_t stg_addr,
                                              int lds, int m0, int n0, int r0, int rows, int nsplit,
                                              int warp, int lane, int nwarps) {
  const RopeEpi rp = *ep.rope;
  const int row_end = min(r0 + rows, ep.M - m0);
  const int half = rp.D >> 1;
#pragma unroll
  for (int c = lane * 4; c < TN; c += 128) {
    const int n = n0 + c;
    if (n >= ep.N) continue;
    float bias4[4] = {0.f, 0.f, 0.f, 0.f};
    if (ep.bias) ld_bf16x4(ep.bias + n, bias4);
    const int head = n / rp.D, within = n - head * rp.D;
    const bool is_q = head < rp.Hq, is_k = !is_q && head < rp.Hq + rp.Hkv;
    const int i0 = within >> 1;                       // dims i0, i0 + 1 and their partners i0 + half, i0 + 1 + half
    for (int rr = r0 + warp; rr < row_end; rr += nwarps) {
      float x[4] = {0.f, 0.f, 0.f, 0.f};
      if (nsplit == 1) {
        const float4 a = *reinterpret_cast<const float4*>(stg + rr * lds + c);
        x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w;
      } else {
        const uint32_t off = stg_addr + uint32_t(rr * lds + c) * 4u;
        float4 part[8];
#pragma unroll
        for (int r = 0; r < 8; ++r)
          if (r < nsplit) part[r] = ld_dsmem_f4(map_to_cta(off, r));
#pragma unroll
        for (int r = 0; r < 8; ++r)
          if (r < nsplit) { x[0] += part[r].x; x[1] += part[r].y; x[2] += part[r].z; x[3] += part[r].w; }
      }
      const int m = m0 + rr;
      if (!PB_DEBUG_CHECK(m >= 0 && m < ep.M && rp.slots[m] >= 0 && rp.pos[m] >= 0, ep.status)) continue;
      float rscale = 1.f;
      if (ep.row_scale) {
        rscale = ep.row_scale[m];
        if (ep.rs_inv_dim > 0.f) rscale = rsqrtf(rscale * ep.rs_inv_dim + ep.rs_eps);
      }
#pragma unroll
      for (int t = 0; t < 4; ++t) x[t] = x[t] * rscale + bias4[t];
      if (!is_q && !is_k) {
        __nv_bfloat16* dst = rp.v_pool + size_t(rp.slots[m]) * rp.pool_stride + size_t(head - rp.Hq - rp.Hkv) * rp.D + within;
        const __nv_bfloat162 o01 = __floats2bfloat162_rn(x[0], x[1]), o23 = __floats2bfloat162_rn(x[2], x[3]);
        uint2 raw;
        raw.x = *reinterpret_cast<const uint32_t*>(&o01);
        raw.y = *reinterpret_cast<const uint32_t*>(&o23);
        *reinterpret_cast<uint2*>(dst) = raw;
        continue;
      }
      const float* cs = rp.cos_sin + size_t(rp.pos[m]) * rp.D;
      const float2 cc = *reinterpret_cast<const float2*>(cs + i0), sn = *reinterpret_cast<const float2*>(cs + half + i0);
      // the projection is rounded to bf16 before the rotation, as the separate kernels would see it
      const float a0 = bf2f(__float2bfloat16(x[0])), b0 = bf2f(__float2bfloat16(x[1]));
      const float a1 = bf2f(__float2bfloat16(x[2])), b1 = bf2f(__float2bfloat16(x[3]));
      __nv_bfloat16* dst = is_q ? rp.q_out + size_t(m) * rp.ldq + size_t(head) * rp.D
                                : rp.k_pool + size_t(rp.slots[m]) * rp.pool_stride + size_t(head - rp.Hq) * rp.D;
      *reinterpret_cast<__nv_bfloat162*>(dst + i0) = __floats2bfloat162_rn(a0 * cc.x - b0 * sn.x, a1 * cc.y - b1 * sn.y);
      *reinterpret_cast<__nv_bfloat162*>(dst + half + i0) = __floats2bfloat162_rn(b0 * cc.x + a0 * sn.x, b1 * cc.y + a1 * sn.y);
    }
  }
}

template <int TN>
__device__ __forceinline__ void epilogue_pass(const EpiParams& ep, const float* stg,
                                              uint32_t stg_addr, int lds, int m0, int n0, int r0,
                                              int rows, int nsplit, int warp, int lane,
                                              int nwarps) {
#define PB_EPI(A, G)                                                                              \
  do {                                                                                            \
    if (aux) epilogue_pass_t<TN, A, G, true>(ep, stg, stg_addr, lds, m0, n0, r0, rows, nsplit, warp, lane, nwarps); \
    else epilogue_pass_t<TN, A, G, false>(ep, stg, stg_addr, lds, m0, n0, r0, rows, nsplit, warp, lane, nwarps);    \
  } while (0)
  if (ep.rope) {
    epilogue_rope<TN>(ep, stg, stg_addr, lds, m0, n0, r0, rows, nsplit, warp, lane, nwarps);
    return;
  }
  const bool aux = ep.bias || ep.residual || ep.col_gate || ep.row_scale || ep.sumsq || ep.a_scale ||
                   ep.w_scale || ep.out_fp32 || ep.out2;
  if (ep.glu) {
    switch (ep.act) {
      case 1: PB_EPI(1, true); break;
      case 2: PB_EPI(2, true); break;
      case 3: PB_EPI(3, true); break;
      default: PB_EPI(0, true); break;
    }
  } else {
    switch (ep.act) {
      case 1: PB_EPI(1, false); break;
      case 2: PB_EPI(2, false); break;
      case 3: PB_EPI(3, false); break;
      default: PB_EPI(0, false); break;
    }
  }
#undef PB_EPI
}

}  // namespace pb

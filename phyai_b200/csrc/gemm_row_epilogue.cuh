// Row-per-thread GEMM epilogue straight out of tensor memory, shared by the persistent kernels
// (gemm_persist.cu, gemm_2cta.cu): thread t of an epilogue warp owns accumulator row (lane base + t),
// reads 32 fp32 columns at a time, applies bias / activation / gated activation / column gate /
// residual and stores bf16 row segments to global memory. No shared-memory staging: shared memory
// belongs to the operand ring.
#pragma once
#include "gemm_epilogue.cuh"
#include "ptx.cuh"

namespace pb {

constexpr int kGroupQ = 8;   // column tiles per group of the grouped tile order

// Grouped order: tiles walk down the rows of a band of kGroupQ column tiles before moving to the next
// band, so the tiles in flight across the chip form a compact block and both operands re-hit in L2.
__device__ __forceinline__ void grouped_tile_coords(int t, int P, int Q, int& p, int& q) {
  const int g = t / (kGroupQ * P);
  const int q0 = g * kGroupQ;
  const int gq = min(kGroupQ, Q - q0);
  const int r = t - g * kGroupQ * P;
  q = q0 + r % gq;
  p = r / gq;
}

__device__ __forceinline__ void unpack_bf16x8(const uint4& raw, float (&f)[8]) {
  // bf16 -> fp32 is a shift / mask of the bit pattern (integer pipe; the conversion instruction is a 16-per-clock unit)
  const uint32_t* u = reinterpret_cast<const uint32_t*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) { f[2 * i] = __uint_as_float(u[i] << 16); f[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u); }
}

// Eight consecutive accumulator columns [n, n + 8) of row m (x holds them); n < ep.N, n % 8 == 0.
// `rscale` multiplies the accumulator before the bias; the return value is the sum of squares of the
// stored (rounded) values.
template <int ACT, bool GLU>
__device__ __forceinline__ float row_epilogue_8(const EpiParams& ep, float (&x)[8], int n, const __nv_bfloat16* res_row,
                                                __nv_bfloat16* out_row, float rscale = 1.f) {
#pragma unroll
  for (int j = 0; j < 8; ++j) x[j] *= rscale;
  if (ep.bias) {
    float b[8];
    unpack_bf16x8(*reinterpret_cast<const uint4*>(ep.bias + n), b);
#pragma unroll
    for (int j = 0; j < 8; ++j) x[j] += b[j];
  }
  if constexpr (GLU) {
    float y[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) y[j] = epi_act_c<ACT>(x[2 * j]) * x[2 * j + 1];
    const int no = n >> 1;
    if (ep.col_gate) {
      const uint2 gr = *reinterpret_cast<const uint2*>(ep.col_gate + no);
      const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gr);
      y[0] *= bf2f(g2[0].x); y[1] *= bf2f(g2[0].y);
      y[2] *= bf2f(g2[1].x); y[3] *= bf2f(g2[1].y);
    }
    if (res_row) {
      const uint2 rr = *reinterpret_cast<const uint2*>(res_row + no);
      const __nv_bfloat162* r2 = reinterpret_cast<const __nv_bfloat162*>(&rr);
      y[0] += bf2f(r2[0].x); y[1] += bf2f(r2[0].y);
      y[2] += bf2f(r2[1].x); y[3] += bf2f(r2[1].y);
    }
    const __nv_bfloat162 o0 = __floats2bfloat162_rn(y[0], y[1]), o1 = __floats2bfloat162_rn(y[2], y[3]);
    uint2 o;
    o.x = *reinterpret_cast<const uint32_t*>(&o0);
    o.y = *reinterpret_cast<const uint32_t*>(&o1);
    *reinterpret_cast<uint2*>(out_row + no) = o;
    const float q0 = bf2f(o0.x), q1 = bf2f(o0.y), q2 = bf2f(o1.x), q3 = bf2f(o1.y);
    return q0 * q0 + q1 * q1 + q2 * q2 + q3 * q3;
  } else {
    if constexpr (ACT != 0) {
#pragma unroll
      for (int j = 0; j < 8; ++j) x[j] = epi_act_c<ACT>(x[j]);
    }
    if (ep.col_gate) {
      float gt[8];
      unpack_bf16x8(*reinterpret_cast<const uint4*>(ep.col_gate + n), gt);
#pragma unroll
      for (int j = 0; j < 8; ++j) x[j] *= gt[j];
    }
    if (res_row) {
      float rs[8];
      unpack_bf16x8(*reinterpret_cast<const uint4*>(res_row + n), rs);
#pragma unroll
      for (int j = 0; j < 8; ++j) x[j] += rs[j];
    }
    uint4 o;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) o2[j] = __floats2bfloat162_rn(x[2 * j], x[2 * j + 1]);
    *reinterpret_cast<uint4*>(out_row + n) = o;
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float q0 = bf2f(o2[j].x), q1 = bf2f(o2[j].y);
      ss += q0 * q0 + q1 * q1;
    }
    return ss;
  }
}

// One accumulator row of `width` columns starting at tensor-memory address `taddr` (lane already
// selected) -> global row m, output columns from n0. Every thread of the warp must call this (the
// tensor-memory loads are warp-collective); rows past M only drain.
template <int ACT, bool GLU>
__device__ __forceinline__ void row_epilogue_tile(const EpiParams& ep, uint32_t taddr, int width, int m, int n0) {
  const bool live = m < ep.M;
  const __nv_bfloat16* res_row = (ep.residual && live) ? ep.residual + size_t(ep.res_mod > 0 ? (m % ep.res_mod) : m) * ep.ldr : nullptr;
  __nv_bfloat16* out_row = reinterpret_cast<__nv_bfloat16*>(ep.out) + size_t(live ? m : 0) * ep.ldo;
  float rscale = 1.f, ss = 0.f;
  if (ep.row_scale && live) {
    rscale = ep.row_scale[m];
    if (ep.rs_inv_dim > 0.f) rscale = rsqrtf(rscale * ep.rs_inv_dim + ep.rs_eps);
  }
#pragma unroll 1
  for (int c = 0; c < width; c += 32) {
    uint32_t r[32];
    tmem_ld_32x32(taddr + uint32_t(c), r);
    tmem_ld_wait();
    if (!live) continue;
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      const int n = n0 + c + 8 * g;
      if (n >= ep.N) continue;
      float x[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) x[j] = __uint_as_float(r[8 * g + j]);
      ss += row_epilogue_8<ACT, GLU>(ep, x, n, res_row, out_row, rscale);
    }
  }
  if (ep.sumsq && live) atomicAdd(ep.sumsq + m, ss);   // one add per row and tile
}

}  // namespace pb

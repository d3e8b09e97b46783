// Host-visible declarations for the tcgen05 GEMM family (see gemm.cu).
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "comm.cuh"

namespace pb {

enum GemmAct : int { kActNone = 0, kActGeluTanh = 1, kActSilu = 2, kActGeluErf = 3 };

// out[M, N'] = epilogue( X[M, K] @ W[N, K]^T ), bf16 (or e4m3) operands, fp32 accumulate.
//
// Epilogue, in this order, on the fp32 accumulator acc[m, n]:
//   acc *= row_scale[m]                 (row_scale != null; e.g. a fused RMS 1/rms; with row_rms_dim > 0
//                                        row_scale[m] is a sum of squares and the factor is
//                                        rsqrt(row_scale[m] / row_rms_dim + row_rms_eps))
//   acc *= a_scale[m] * w_scale[n]      (per-row / per-channel dequant scales, fp8 only)
//   acc += bias[n]                      (bias != null)
//   acc  = act(acc)                     (act != none, glu == 0)
//   glu: y[m, n/2] = act(acc[m, 2j]) * acc[m, 2j+1]   (weight rows interleaved gate/up)
//   acc *= col_gate[n]                  (col_gate != null; row-broadcast gate vector)
//   acc *= row_gate... (unused)
//   acc += residual[m % res_mod, n]     (residual != null)
//   sumsq[m] += sum_n acc^2             (sumsq != null; fp32 atomics; feeds a fused RMSNorm)
//   store bf16 (or fp32 when out_fp32)
// Destination of a fused-QKV projection whose epilogue rotates q / k and scatters k / v to the KV
// pool (lives in device memory; the kernel gets a pointer). The weight rows of every q and k head
// are permuted so that output column 2i of a head is dimension i and column 2i + 1 is dimension
// i + D/2: a rotation pair sits in adjacent accumulator columns. v heads keep their order.
struct RopeEpi {
  __nv_bfloat16* q_out;        // [M, Hq * D], row stride ldq
  __nv_bfloat16* k_pool;       // [slots, Hkv * D], row stride pool_stride
  __nv_bfloat16* v_pool;
  const float* cos_sin;        // [positions, D]: cos(D/2) | sin(D/2)
  const int* pos;              // [M] table row per token
  const long long* slots;      // [M] pool row per token
  long long pool_stride;
  int ldq, Hq, Hkv, D;
};

struct GemmArgs {
  const void* x = nullptr;   // [M, K], row stride ldx elements
  const void* w = nullptr;   // [N, K], row stride ldw elements
  void* out = nullptr;       // [M, N or N/2], row stride ldo elements
  int M = 0, N = 0, K = 0;
  int ldx = 0, ldw = 0, ldo = 0;
  const __nv_bfloat16* bias = nullptr;      // [N]
  const __nv_bfloat16* residual = nullptr;  // [res_rows, ldr]
  int ldr = 0;
  int res_mod = 0;                          // 0: residual row = m
  const __nv_bfloat16* col_gate = nullptr;  // [N]
  const float* row_scale = nullptr;         // [M]
  const RopeEpi* rope = nullptr;     // device pointer: rotate q / k and scatter k / v instead of storing `out`
  float* zero = nullptr;                    // fp32 scratch this launch clears (not the one it accumulates into)
  int zero_n = 0;
  int row_rms_dim = 0;                      // > 0: row_scale is the sum of squares of a row of that width
  float row_rms_eps = 0.f;
  float* sumsq = nullptr;                   // [M]
  __nv_bfloat16* out2 = nullptr;            // [M, ldo2] second bf16 output: stored value * (1 + col_scale2[n]) (one-tile kernel, no glu)
  const __nv_bfloat16* col_scale2 = nullptr;  // [N]
  int ldo2 = 0;
  int act = kActNone;
  int glu = 0;
  int out_fp32 = 0;
  int fp8 = 0;                              // operands are e4m3, K counted in elements
  const float* a_scale = nullptr;           // fp8: [M] or [M, K/128] (block)
  const float* w_scale = nullptr;           // fp8: [N] or [N/128, K/128] (block)
  int block_scaled = 0;                     // fp8: 128x128 weight blocks, 1x128 act blocks
  int force_bn = 0, force_swap = -1, force_splits = 0;  // tuning overrides (0/-1 = auto)
  unsigned long long* trace = nullptr;  // optional: 8 globaltimer stamps per CTA (debugging)
  // Push mode (row-parallel linear fused with its all-reduce): the raw bf16 product goes to
  // every rank's slots instead of `out`; bias/act/residual belong to the consumer kernel.
  const PushParams* push = nullptr;
  // receives 1 when the launch also ran the consumer half (push->tail asked for it and the grid allowed it)
  int* tail_done = nullptr;
};

// Launches on `stream`. Returns cudaSuccess or the launch error; argument
// problems (alignment, unsupported shape) return cudaErrorInvalidValue.
// `n_ctas`, when given, receives the number of CTAs launched (what a push-mode consumer
// multiplies by the world size to know how many arrivals to expect).
cudaError_t gemm_launch(const GemmArgs& a, cudaStream_t stream, int* n_ctas = nullptr);

// 2-D K-major operand map: [rows, cols] with row stride ld (elements), box = 128 bytes x box_rows,
// 128-byte swizzle (elem_bytes 2 = bf16, 1 = 8-bit).
bool make_tmap_2d(CUtensorMap* out, const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld,
                  uint32_t box_rows, uint32_t elem_bytes);

// Block-scaled fp8 GEMM (gemm_fp8_block.cu): e4m3 operands, fp32 scales per 1x128 activation block
// (a_scale [M, K/128]) and per 128x128 weight block (w_scale [ceil(N/128), K/128]); epilogue fields
// of GemmArgs as for gemm_launch (bias, act, glu, col_gate, residual, out_fp32).
cudaError_t gemm_fp8_block_launch(const GemmArgs& a, cudaStream_t stream);

// Persistent variant for large bf16 problems (gemm_persist.cu); gemm_launch routes eligible calls to it.
bool gemm_persist_eligible(const GemmArgs& a);
cudaError_t gemm_persist_launch(const GemmArgs& a, cudaStream_t stream, int* n_ctas = nullptr);

// CTA-pair variant (gemm_2cta.cu): 256 x 256 tiles on two SMs with tcgen05.mma.cta_group::2.
bool gemm_2cta_eligible(const GemmArgs& a);
cudaError_t gemm_2cta_launch(const GemmArgs& a, cudaStream_t stream);
void set_gemm_2cta(int mode);   // 1 on, 0 off, -1 follow the PHYAI_GEMM_2CTA variable
unsigned long long gemm_2cta_launches();

// 3-D bf16 tensor map (d, head, row) for the attention kernels (see gemm.cu).
bool make_tmap_3d_bf16(CUtensorMap* out, const void* ptr, uint64_t D, uint64_t H, uint64_t R,
                       uint64_t head_stride_elems, uint64_t row_stride_elems, uint32_t box_h,
                       uint32_t box_r);

// Device-global status word shared by the kernels of this library (0 = ok).
int* kernel_status_ptr();
int read_and_clear_kernel_status();

// How many kernels of this library were launched since the last reset.
uint64_t launch_counter();
void reset_launch_counter();
void bump_launch_counter(unsigned long long n = 1);

}  // namespace pb

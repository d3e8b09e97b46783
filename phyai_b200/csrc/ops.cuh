// Host-visible declarations for the memory-bound kernels (ops.cu): norms, RoPE +
// KV scatter, embedding, patch extraction, gated activations, sampler updates,
// fp8 activation quantisation.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace pb {

enum NormMode : int { kNormRms = 0, kNormGemmaRms = 1, kNormLayer = 2, kNormAdaRms = 3, kNormRmsNoWeight = 4 };

struct NormArgs {
  const __nv_bfloat16* x = nullptr;     // [rows, D] row stride ldx
  __nv_bfloat16* y = nullptr;           // [rows, D] row stride ldy
  const __nv_bfloat16* weight = nullptr;  // [D] (rms / layer gamma)
  const __nv_bfloat16* bias = nullptr;    // [D] (layer beta)
  const __nv_bfloat16* mod = nullptr;     // AdaRMS: [rows/group, 3D] = scale | shift | gate
  __nv_bfloat16* residual = nullptr;    // optional, in place: residual += x; y = norm(residual)
  const float* sumsq = nullptr;         // optional: precomputed sum of squares per row
  int rows = 0, D = 0, ldx = 0, ldy = 0, ldr = 0;
  int group = 1;                        // AdaRMS: rows sharing one modulation row
  int mode = kNormRms;
  float eps = 1e-6f;
  // optional fp8 output: y8 = e4m3(y / s) with s per row (block = 0) or per 128 columns
  uint8_t* y8 = nullptr;
  float* y8_scale = nullptr;
  int y8_block = 0;
};
cudaError_t norm_launch(const NormArgs& a, cudaStream_t s);

struct RopeKvArgs {
  const __nv_bfloat16* qkv = nullptr;   // [M, ld]: q heads | k heads | v heads, each D wide
  int M = 0, ld = 0, Hq = 0, Hkv = 0, D = 0;
  const int* pos = nullptr;             // [M] row of cos_sin per token (null: row = token)
  const float* cos_sin = nullptr;       // [rows, D]: cos(D/2) | sin(D/2); null = no rotation
  int rot_dim = 0;                      // rotate the first rot_dim dims (0 = D)
  const __nv_bfloat16* q_norm_w = nullptr;  // optional per-head RMSNorm weights [D]
  const __nv_bfloat16* k_norm_w = nullptr;
  float norm_eps = 1e-6f;
  __nv_bfloat16* q_out = nullptr;       // [M, Hq*D], row stride ldq
  int ldq = 0;
  __nv_bfloat16* k_pool = nullptr;      // [slots, Hkv, D]
  __nv_bfloat16* v_pool = nullptr;
  long long pool_row_stride = 0;
  const long long* slots = nullptr;     // [M] pool row per token (null: row = slot_base + token)
  long long slot_base = 0;
  float* zero = nullptr;                // optional fp32 scratch cleared by this launch (e.g. the sum-of-squares
  int zero_n = 0;                       // accumulators a later GEMM epilogue adds into)
};
cudaError_t rope_kv_launch(const RopeKvArgs& a, cudaStream_t s);

// out[dst_row(m), :] = (lo <= id < hi) ? table[id - lo, :] * scale : 0
cudaError_t embedding_launch(const long long* ids, int n_ids, const __nv_bfloat16* table, int D,
                             long long lo, long long hi, float scale, __nv_bfloat16* out, int ldo,
                             const int* dst_rows, cudaStream_t s);

// pixels [n_img, C, H, W] -> patches [n_img * (H/p) * (W/p), kpad], k = (c, py, px), zero tail
cudaError_t im2col_launch(const __nv_bfloat16* pix, int n_img, int C, int H, int W, int p,
                          __nv_bfloat16* out, int kpad, cudaStream_t s);

// y[m, j] = act(x[m, j]) * x[m, I + j]   (x: [M, 2I], split halves; interleaved = pairs)
cudaError_t gated_act_launch(const __nv_bfloat16* x, __nv_bfloat16* y, int M, int I, int act,
                             int interleaved, cudaStream_t s);

// x += dt * v (elementwise; x fp32 or bf16, v bf16)
// Gated DeltaNet decode step (gdn.cu): q, k [B, H, Dk], v [B, H, Dv], g, beta [B, H] (all fp32 or all bf16),
// state_pool fp32 [slots, H, Dk, Dv] updated in place at rows state_indices[B]; out [B, H, Dv].
cudaError_t gdn_decode_launch(const void* q, const void* k, const void* v, const void* g, const void* beta, int in_bf16,
                              float* state_pool, const long long* state_indices, void* out, int out_bf16, int B, int H,
                              int Dk, int Dv, float scale, int l2norm, cudaStream_t stream);

// Snake activation over [B, C, T] (alpha, beta fp32 [C], already exponentiated).
cudaError_t snake_launch(const void* x, void* y, int is_bf16, const float* alpha, const float* beta, int C, long long T,
                         long long total, cudaStream_t s);

cudaError_t axpy_launch(void* x, int x_fp32, const __nv_bfloat16* v, float dt, long long n,
                        cudaStream_t s);

// out = uncond + g * (cond - uncond); optional fused Euler step x += dt * out
cudaError_t cfg_combine_launch(const __nv_bfloat16* cond, const __nv_bfloat16* uncond, float g,
                               __nv_bfloat16* out, float* x_fp32, float dt, long long n,
                               cudaStream_t s);

// y = x @ w^T + bias on CUDA cores for operands the tensor-core GEMM does not take (dtype codes 0 fp32, 1 bf16, 2 fp16).
cudaError_t linear_simt_launch(const void* x, int x_type, const void* w, int w_type, const void* bias, void* y, int M, int N,
                               int K, int ldx, int ldw, int ldy, cudaStream_t s);

// y[b, t, :] = x[b, t, :] @ W[domain[b]] + bias[domain[b]]; W is [domains][K][N], bias [domains][N], all bf16.
cudaError_t domain_linear_launch(const __nv_bfloat16* x, const __nv_bfloat16* w, const __nv_bfloat16* bias, const long long* domain,
                                 __nv_bfloat16* y, int B, int T, int K, int N, cudaStream_t s);

// One UniPC (order <= 2, flow prediction) update of a latent viewed as [B][C][T][inner]:
//   v = v_uncond + g (v - v_uncond)        when v_uncond is given
//   m_t = x - sigma v;  x_s = c_x x_last + c_0 m1 + c_1 m2 + c_t m_t (has_corr) else x
//   x <- p_x x_s + p_0 m_t + p_1 m1;  x_last <- x_s;  m2 <- m1;  m1 <- m_t
//   x[b, :, t, :] <- cond[b, :, t, :] where keep[b, t]
struct UniPCStepArgs {
  const __nv_bfloat16* v;
  const __nv_bfloat16* v_uncond;   // null: v is already guided
  float g;
  __nv_bfloat16* x;                // sample, in and out
  float* x_last;                   // state (fp32, same numel)
  float* m1;                       // x0 prediction of the previous step
  float* m2;                       // ... of the step before
  float sigma;
  int has_corr;
  float c_x, c_0, c_1, c_t, p_x, p_0, p_1;
  const unsigned char* keep;       // [B, T] or null
  const __nv_bfloat16* cond;       // same shape as x (read where keep is set)
  long long n, inner, T, C, live_inner;
};
cudaError_t unipc_step_launch(const UniPCStepArgs& a, cudaStream_t s);

// dst[rows[i], :] = src[i, :]   (row scatter of 16-byte aligned rows)
cudaError_t scatter_rows_launch(const __nv_bfloat16* src, int n, int D, int lds,
                                __nv_bfloat16* dst, int ldd, const int* rows, cudaStream_t s);

// e4m3 quantisation: per row (block = 0) or per 1 x 128 block; scale = amax / 448
cudaError_t quant_fp8_launch(const __nv_bfloat16* x, int rows, int D, int ldx, uint8_t* y,
                             float* scale, int block, cudaStream_t s);

// gelu / silu / snake elementwise
cudaError_t unary_launch(const __nv_bfloat16* x, __nv_bfloat16* y, long long n, int act,
                         cudaStream_t s);

}  // namespace pb

// Host-visible declarations of the persistent action-expert kernel (expert_stack.cu).
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace pb {

// One launch runs Euler steps [step_begin, step_end) of a flow-matching action expert (Gemma-style
// blocks on M <= 64 action rows that attend into a prefix K/V range of one KV head) with one CTA per
// SM. Every vector below is fp32 and indexed [step][layer][...] unless noted.
struct ExpertStackParams {
  int M = 0, H = 0, I = 0, Hq = 0, D = 0, A = 0;   // rows, hidden, MLP width, q heads, head dim, action dim
  int n_layers = 0, step_begin = 0, step_end = 0;
  int att_splits = 0;                              // KV splits per head (Hq * att_splits <= grid)
  float eps = 1e-6f, dt = 0.f, sm_scale = 1.f;
  // [n_layers * 4 + 1] tensor maps in device memory: per layer qkv / o / gate_up / down weights
  // (box 64 x 128), then the attention-output buffer `attn` (box 64 x 64)
  const CUtensorMap* tmaps = nullptr;
  const float* in_scale = nullptr;     // [.., H]   factor on the rows entering the QKV projection (1 + scale)
  const float* post_scale = nullptr;   // [.., H]   same for the gate/up projection
  const float* gate_in = nullptr;      // [.., H]   gate on the attention branch before the residual add
  const float* gate_post = nullptr;    // [.., H]   gate on the MLP branch
  const float* qkv_bias = nullptr;     // [.., (Hq + 2) * D]   shift @ Wqkv^T
  const float* gu_bias = nullptr;      // [.., 2 * I]          shift @ Wgu^T (gate / up interleaved)
  const float* fin_scale = nullptr;    // [step][H]
  const float* out_bias = nullptr;     // [step][A]  shift @ Wout^T + b_out
  const __nv_bfloat16* w_in = nullptr;   // [H, A]
  const __nv_bfloat16* b_in = nullptr;   // [H]
  const __nv_bfloat16* w_out = nullptr;  // [A, H]
  const __nv_bfloat16* k_pool = nullptr; // [layers, slots, D] (one KV head)
  const __nv_bfloat16* v_pool = nullptr;
  long long pool_layer_stride = 0, pool_row_stride = 0;   // elements
  const int* kv_ptr = nullptr;         // device: first pool row of the KV range
  const int* kv_len = nullptr;         // device: rows of the range including the M action rows at its end
  const int* pos = nullptr;            // [M] rotary table row per action row
  const float* cos_sin = nullptr;      // [positions, D]: cos(D/2) | sin(D/2)
  const __nv_bfloat16* x0 = nullptr;   // [M, A] state at step_begin
  __nv_bfloat16* out = nullptr;        // [M, A] state after step_end - 1
  // scratch, all rows padded to 64
  float* x_t = nullptr;                // [64, A]
  float* h = nullptr;                  // [64, H]
  float* acc_qkv = nullptr;            // [64, (Hq + 2) * D]
  float* acc_gu = nullptr;             // [64, 2 * I]
  float* ss = nullptr;                 // [2][64] sums of squares of the rows of h
  __nv_bfloat16* attn = nullptr;       // [64, Hq * D]
  float* part_o = nullptr;             // [Hq][att_splits][64][D]
  float* part_ml = nullptr;            // [Hq][att_splits][64][2]
  unsigned* barrier = nullptr;         // grid barrier word, cleared before every launch
  int* status = nullptr;
  unsigned long long* trace = nullptr; // optional: 64 globaltimer stamps per CTA
  int debug = 0;                       // bit 0: plain stores instead of reductions (timing experiments; wrong results)
};

// Bytes of fp32 / bf16 scratch the kernel needs for a geometry (see the struct): the caller allocates.
cudaError_t expert_stack_launch(const ExpertStackParams& p, cudaStream_t stream);
// How many CTAs a launch on the current device uses (0: the kernel cannot be made resident).
int expert_stack_grid();

}  // namespace pb

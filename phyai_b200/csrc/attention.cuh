// Host-visible declarations for the ragged / paged flash-attention kernel (attention.cu).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace pb {

struct AttnParams {
  const __nv_bfloat16* q = nullptr;   // [tokens, Hq, D] via (q_tok_stride, q_head_stride)
  const __nv_bfloat16* k = nullptr;   // [rows, Hkv, D] via (kv_row_stride, kv_head_stride)
  const __nv_bfloat16* v = nullptr;
  __nv_bfloat16* out = nullptr;       // [tokens, Hq, D] via (o_tok_stride, o_head_stride)
  const int* q_start = nullptr;       // [batch] first q token of each sequence
  const int* q_len = nullptr;         // [batch]
  const int* kv_indptr = nullptr;     // [batch] first KV entry of each sequence
  const int* kv_len = nullptr;        // [batch]
  const int* kv_indices = nullptr;    // optional: KV entry -> pool row (page size 1)
  long long q_tok_stride = 0, q_head_stride = 0;
  long long kv_row_stride = 0, kv_head_stride = 0;
  long long o_tok_stride = 0, o_head_stride = 0;
  int batch = 0, num_kv_heads = 0, group = 1, head_dim = 0;
  int max_q_len = 0;                  // grid sizing: max over the batch of q_len
  int causal = 0;                     // q token i sees kv j <= i + (kv_len - q_len)
  int splits = 1;                     // KV split over a cluster (1, 2, 4 or 8)
  float sm_scale = 1.0f;
  int window = 0;                     // > 0: q token i sees only the last `window` kv entries up to its own position (tcgen05 latency kernel)
  float soft_cap = 0.f;               // > 0: scores become cap * tanh(score / cap) before the softmax (same kernel)
  unsigned long long* trace = nullptr;  // optional: 16 globaltimer stamps per CTA (debugging)
  long long q_rows = 0, kv_rows = 0;  // extents of the q and k/v tensors (rows), for TMA maps
};

cudaError_t attn_launch(const AttnParams& p, cudaStream_t stream);     // mma.sync path
cudaError_t attn_tc_launch(const AttnParams& p, cudaStream_t stream);  // tcgen05 path
// tcgen05 two-tile pipelined path: dense q, contiguous K/V, head_dim <= 128, no KV split
cudaError_t attn_pp_launch(const AttnParams& p, cudaStream_t stream);
bool attn_pp_supported(const AttnParams& p);

}  // namespace pb

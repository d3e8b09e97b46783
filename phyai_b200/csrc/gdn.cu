// Gated DeltaNet, one decode step per sequence against a pool of recurrent states.
//
//   S <- exp(g) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q        (S is Dk x Dv, fp32)
//
// One CTA per (sequence, head); a thread owns value columns, so every pass over the state reads
// and writes rows of Dv consecutive floats (coalesced), and the state makes exactly one round trip:
// pass 1 reads S and forms S^T k, pass 2 re-reads it (L1 / L2 hit), applies decay and the rank-1
// update, writes it back and forms S^T q on the way. q and k are L2-normalised in shared memory first.
//
// Counterpart of the reference's recurrent decode path
// (phyai/src/phyai/layers/attention/gdn/backends/flashinfer.py:161-208, backends/fla.py:180-239).
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "launch.cuh"
#include "ops.cuh"
#include "ptx.cuh"

namespace pb {

namespace {

__device__ __forceinline__ float ld_any(const void* p, size_t i, int is_bf16) {
  return is_bf16 ? bf2f(reinterpret_cast<const __nv_bfloat16*>(p)[i]) : reinterpret_cast<const float*>(p)[i];
}

__global__ void __launch_bounds__(128)
gdn_decode_kernel(const void* q, const void* k, const void* v, const void* g, const void* beta, int in_bf16,
                  float* state_pool, const long long* state_indices, void* out, int out_bf16, int H, int Dk, int Dv,
                  float scale, int l2norm) {
  __shared__ float qs[256], ks[256], red[8];
  const int h = blockIdx.x, b = blockIdx.y, tid = threadIdx.x;
  pdl_launch_dependents();
  pdl_wait();
  const size_t tok = size_t(b) * H + h;
  float sq = 0.f, sk = 0.f;
  for (int i = tid; i < Dk; i += blockDim.x) {
    const float a = ld_any(q, tok * Dk + i, in_bf16), c = ld_any(k, tok * Dk + i, in_bf16);
    qs[i] = a; ks[i] = c;
    sq += a * a; sk += c * c;
  }
  for (int o = 16; o > 0; o >>= 1) { sq += __shfl_xor_sync(0xffffffffu, sq, o); sk += __shfl_xor_sync(0xffffffffu, sk, o); }
  if ((tid & 31) == 0) { red[tid >> 5] = sq; red[4 + (tid >> 5)] = sk; }
  __syncthreads();
  const float nq = red[0] + red[1] + red[2] + red[3], nk = red[4] + red[5] + red[6] + red[7];
  // F.normalize: x / max(||x||, 1e-12)
  const float rq = (l2norm ? 1.f / fmaxf(sqrtf(nq), 1e-12f) : 1.f) * scale, rk = l2norm ? 1.f / fmaxf(sqrtf(nk), 1e-12f) : 1.f;
  const float eg = __expf(ld_any(g, tok, in_bf16)), bt = ld_any(beta, tok, in_bf16);
  float* S = state_pool + (size_t(state_indices[b]) * H + h) * size_t(Dk) * Dv;
  for (int col = tid; col < Dv; col += blockDim.x) {
    float pred = 0.f;
    for (int i = 0; i < Dk; ++i) pred += S[size_t(i) * Dv + col] * ks[i];
    pred *= eg * rk;                                             // (exp(g) S)^T k_hat
    const float u = (ld_any(v, tok * Dv + col, in_bf16) - pred) * bt;
    float o = 0.f;
    for (int i = 0; i < Dk; ++i) {
      const float s = S[size_t(i) * Dv + col] * eg + ks[i] * rk * u;
      S[size_t(i) * Dv + col] = s;
      o += s * qs[i];
    }
    o *= rq;
    if (out_bf16) reinterpret_cast<__nv_bfloat16*>(out)[tok * Dv + col] = __float2bfloat16(o);
    else reinterpret_cast<float*>(out)[tok * Dv + col] = o;
  }
}

}  // namespace

cudaError_t gdn_decode_launch(const void* q, const void* k, const void* v, const void* g, const void* beta, int in_bf16,
                              float* state_pool, const long long* state_indices, void* out, int out_bf16, int B, int H,
                              int Dk, int Dv, float scale, int l2norm, cudaStream_t stream) {
  if (B <= 0 || H <= 0 || Dk <= 0 || Dk > 256 || Dv <= 0) return cudaErrorInvalidValue;
  return launch_kernel(gdn_decode_kernel, dim3(H, B), dim3(128), 0, stream, 1, q, k, v, g, beta, in_bf16, state_pool,
                       state_indices, out, out_bf16, H, Dk, Dv, scale, l2norm);
}

}  // namespace pb

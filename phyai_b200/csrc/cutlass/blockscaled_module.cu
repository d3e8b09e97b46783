// Module ``phyai_b200._blockscaled``: NVFP4 linear on the block-scaled tensor-core path of sm_100a. The GEMM is a CUTLASS
// sm100 collective instantiated in this directory (one translation unit per tile shape), with this repository's kernels
// around it. (The blockwise fp8 collective of the same library was measured here too: at 128 x 128 and 256 x 128-pair
// tiles it ran level with csrc/gemm_fp8_block.cu on every shape, so block-scaled fp8 stays on the in-tree kernel.)
//
//   y[M, N] = alpha * (x4 . sfx) @ (w4 . sfw)^T        x4, w4: e2m1 packed two per byte (K-major),
//                                                      sfx, sfw: one ue4m3 scale per 16 elements of K
//
// The GEMM is the CUTLASS sm100 block-scaled collective (tcgen05.mma kind::mxf4nvf4 with the scale factors
// staged into tensor memory, TMA operand loads, no cluster: loads are per CTA) instantiated for three one-CTA tile
// shapes and one CTA-pair shape; the kernels around it are this file's own: activation quantisation (bf16 rows -> e2m1 + ue4m3
// scales written directly in the 128 x 4 interleaved scale layout the MMA reads), the re-layout of a
// checkpoint's row-major weight scales into that layout, and the bias add.
//
// Scale layout (checked against the collective's own layout function on the host): scale (row r, block kb)
// of a matrix with KB = ceil(K / 64) * 4 padded scale columns lives at byte
//   ((r / 128) * (KB / 4) + kb / 4) * 512 + (r % 32) * 16 + ((r % 128) / 32) * 4 + kb % 4.
//
// What the reference calls for this: FlashInfer mm_fp4 + nvfp4_quantize with the 128x4 layout
// (phyai/src/phyai/layers/linear/backends/flashinfer.py:163-200, phyai/src/phyai/layers/quant/nvfp4.py:180-225).
#include <ATen/cuda/CUDAContext.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <torch/extension.h>

namespace nvfp4 {

int run_tile64(const void*, const void*, const void*, const void*, void*, int, int, int, float, void*, size_t, cudaStream_t);
int run_tile128(const void*, const void*, const void*, const void*, void*, int, int, int, float, void*, size_t, cudaStream_t);
int run_tile256(const void*, const void*, const void*, const void*, void*, int, int, int, float, void*, size_t, cudaStream_t);
int run_tile2sm(const void*, const void*, const void*, const void*, void*, int, int, int, float, void*, size_t, cudaStream_t);

// ------------------------------------------------------------------ own kernels
__host__ __device__ inline size_t sf_offset(int row, int kb, int kb_padded) {
  return (size_t(row >> 7) * (kb_padded >> 2) + (kb >> 2)) * 512 + size_t(row & 31) * 16 + ((row & 127) >> 5) * 4 + (kb & 3);
}

__device__ __forceinline__ float bf2f(__nv_bfloat16 v) { return __bfloat162float(v); }

// ue4m3 byte of a non-negative float (round to nearest, saturating) and its value back
__device__ __forceinline__ uint8_t f2e4m3(float v) {
  unsigned short r;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(0.f), "f"(v));
  return uint8_t(r & 0xff);
}
__device__ __forceinline__ float e4m32f(uint8_t b) {
  const int e = (b >> 3) & 0xf, m = b & 7;
  return e == 0 ? float(m) * 0.001953125f : __int_as_float(((e + 120) << 23) | (m << 20));
}
// two floats -> one byte of e2m1 (first argument in the low nibble)
__device__ __forceinline__ uint8_t f2e2m1x2(float lo, float hi) {
  unsigned short r;
  asm("{ .reg .b8 t; cvt.rn.satfinite.e2m1x2.f32 t, %1, %2; cvt.u16.u8 %0, t; }" : "=h"(r) : "f"(hi), "f"(lo));
  return uint8_t(r);
}

// One thread per 16-element block: amax -> ue4m3 scale (relative to the tensor's global scale) -> e2m1 codes.
__global__ void quant_act_kernel(const __nv_bfloat16* x, int M, int K, int ldx, float inv_global, uint8_t* q, uint8_t* sf, int kb_padded) {
  const int nkb = K >> 4;
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)M * nkb) return;
  const int row = int(i / nkb), kb = int(i - (long long)row * nkb);
  const uint4* src = reinterpret_cast<const uint4*>(x + size_t(row) * ldx + kb * 16);
  const uint4 a = src[0], b = src[1];
  float v[16];
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&a);
  const __nv_bfloat162* r = reinterpret_cast<const __nv_bfloat162*>(&b);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    v[2 * j] = bf2f(p[j].x); v[2 * j + 1] = bf2f(p[j].y);
    v[8 + 2 * j] = bf2f(r[j].x); v[8 + 2 * j + 1] = bf2f(r[j].y);
  }
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < 16; ++j) amax = fmaxf(amax, fabsf(v[j]));
  const uint8_t sb = f2e4m3(amax * (1.f / 6.f) * inv_global);
  const float s = e4m32f(sb);
  const float inv = s > 0.f ? inv_global / s : 0.f;      // x / (s * global)
  uint32_t w[2] = {0u, 0u};
#pragma unroll
  for (int j = 0; j < 8; ++j) w[j >> 2] |= uint32_t(f2e2m1x2(v[2 * j] * inv, v[2 * j + 1] * inv)) << (8 * (j & 3));
  *reinterpret_cast<uint2*>(q + (size_t(row) * K >> 1) + kb * 8) = make_uint2(w[0], w[1]);
  sf[sf_offset(row, kb, kb_padded)] = sb;
}

// row-major [rows, nkb] scales -> the interleaved layout (padding bytes of `dst` are zero and stay so)
__global__ void swizzle_sf_kernel(const uint8_t* src, int rows, int nkb, uint8_t* dst, int kb_padded) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)rows * nkb) return;
  const int row = int(i / nkb), kb = int(i - (long long)row * nkb);
  dst[sf_offset(row, kb, kb_padded)] = src[i];
}

__global__ void add_bias_kernel(__nv_bfloat16* y, const __nv_bfloat16* bias, long long total, int N) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  y[i] = __float2bfloat16(bf2f(y[i]) + bf2f(bias[i % N]));
}

// ------------------------------------------------------------------ bindings
using torch::Tensor;
static cudaStream_t cur() { return at::cuda::getCurrentCUDAStream().stream(); }
static int64_t padded_kb(int64_t K) { return (K + 63) / 64 * 4; }
static int64_t sf_bytes(int64_t rows, int64_t K) { return (rows + 127) / 128 * 128 * padded_kb(K); }

int64_t scale_bytes(int64_t rows, int64_t K) { return sf_bytes(rows, K); }

void quantize_act(const Tensor& x, double global_scale, Tensor& q, Tensor& sf) {
  TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.scalar_type() == at::kBFloat16 && x.stride(1) == 1, "quantize_act: bf16 [M, K]");
  const int64_t M = x.size(0), K = x.size(1);
  TORCH_CHECK(K % 32 == 0 && x.stride(0) % 8 == 0 && (reinterpret_cast<uintptr_t>(x.data_ptr()) & 15) == 0, "quantize_act: K % 32, 16-byte rows");
  TORCH_CHECK(q.is_contiguous() && q.scalar_type() == at::kByte && q.numel() == M * K / 2, "quantize_act: q is uint8 [M, K/2]");
  TORCH_CHECK(sf.is_contiguous() && sf.element_size() == 1 && sf.numel() >= sf_bytes(M, K), "quantize_act: scale buffer too small");
  TORCH_CHECK(global_scale > 0, "quantize_act: global scale must be positive");
  const long long n = M * (K / 16);
  if (n == 0) return;
  quant_act_kernel<<<unsigned((n + 255) / 256), 256, 0, cur()>>>(reinterpret_cast<const __nv_bfloat16*>(x.data_ptr()), int(M), int(K),
                                                                int(x.stride(0)), float(1.0 / global_scale),
                                                                reinterpret_cast<uint8_t*>(q.data_ptr()),
                                                                reinterpret_cast<uint8_t*>(sf.data_ptr()), int(padded_kb(K)));
  TORCH_CHECK(cudaGetLastError() == cudaSuccess, "quant_act_kernel launch failed");
}

Tensor swizzle_scales(const Tensor& sf_linear, int64_t K) {
  TORCH_CHECK(sf_linear.is_cuda() && sf_linear.dim() == 2 && sf_linear.is_contiguous() && sf_linear.element_size() == 1 &&
              sf_linear.size(1) == K / 16, "swizzle_scales: one-byte scales [rows, K/16]");
  const int64_t rows = sf_linear.size(0);
  Tensor out = torch::zeros({sf_bytes(rows, K)}, sf_linear.options().dtype(at::kByte));
  const long long n = rows * (K / 16);
  if (n)
    swizzle_sf_kernel<<<unsigned((n + 255) / 256), 256, 0, cur()>>>(reinterpret_cast<const uint8_t*>(sf_linear.data_ptr()), int(rows),
                                                                   int(K / 16), reinterpret_cast<uint8_t*>(out.data_ptr()), int(padded_kb(K)));
  TORCH_CHECK(cudaGetLastError() == cudaSuccess, "swizzle_sf_kernel launch failed");
  return out;
}

// x4 [M, K/2], w4 [N, K/2] packed e2m1; sfx / sfw in the interleaved layout; out bf16 [M, N]. tile: 0 auto, 64 / 128 / 256 (one CTA per tile), 512 (256 x 256 on a CTA pair).
void gemm(const Tensor& x4, const Tensor& sfx, const Tensor& w4, const Tensor& sfw, Tensor& out, double alpha,
          const c10::optional<Tensor>& bias, Tensor& workspace, int64_t tile) {
  TORCH_CHECK(x4.is_cuda() && w4.is_cuda() && x4.is_contiguous() && w4.is_contiguous() && x4.scalar_type() == at::kByte &&
              w4.scalar_type() == at::kByte && x4.dim() == 2 && w4.dim() == 2 && x4.size(1) == w4.size(1), "nvfp4 gemm: packed operands");
  const int M = int(x4.size(0)), N = int(w4.size(0)), K = int(x4.size(1) * 2);
  TORCH_CHECK(K % 32 == 0 && N % 8 == 0, "nvfp4 gemm: K % 32 and N % 8");
  TORCH_CHECK(out.is_contiguous() && out.scalar_type() == at::kBFloat16 && out.size(0) == M && out.size(1) == N, "nvfp4 gemm: out bf16 [M, N]");
  TORCH_CHECK(sfx.numel() >= sf_bytes(M, K) && sfw.numel() >= sf_bytes(N, K) && sfx.element_size() == 1 && sfw.element_size() == 1,
              "nvfp4 gemm: scale buffers");
  TORCH_CHECK(workspace.is_cuda() && workspace.is_contiguous(), "nvfp4 gemm: workspace");
  if (M == 0) return;
  if (tile == 0) {
    // fill the 148 SMs: the widest tile that still gives about a wave of CTAs
    const long m_t = (M + 127) / 128;
    tile = m_t * ((N + 255) / 256) >= 120 ? 256 : (m_t * ((N + 127) / 128) >= 100 ? 128 : 64);
    // several waves of 256-wide tiles: CTA pairs halve the B traffic per SM
    if (tile == 256 && ((M + 255) / 256) * ((N + 255) / 256) >= 148) tile = 512;
  }
  const void *A = x4.data_ptr(), *B = w4.data_ptr(), *SA = sfx.data_ptr(), *SB = sfw.data_ptr();
  void* ws = workspace.data_ptr();
  const size_t wsb = size_t(workspace.numel()) * workspace.element_size();
  int rc;
  if (tile == 512) rc = run_tile2sm(A, SA, B, SB, out.data_ptr(), M, N, K, float(alpha), ws, wsb, cur());
  else if (tile == 256) rc = run_tile256(A, SA, B, SB, out.data_ptr(), M, N, K, float(alpha), ws, wsb, cur());
  else if (tile == 128) rc = run_tile128(A, SA, B, SB, out.data_ptr(), M, N, K, float(alpha), ws, wsb, cur());
  else rc = run_tile64(A, SA, B, SB, out.data_ptr(), M, N, K, float(alpha), ws, wsb, cur());
  TORCH_CHECK(rc == 0, "nvfp4 gemm: stage ", rc, " failed (1 shape not supported, 2 workspace, 3 initialise, 4 launch)");
  if (bias.has_value() && bias->defined()) {
    TORCH_CHECK(bias->scalar_type() == at::kBFloat16 && bias->is_contiguous() && bias->numel() == N, "nvfp4 gemm: bias bf16 [N]");
    const long long total = (long long)M * N;
    add_bias_kernel<<<unsigned((total + 255) / 256), 256, 0, cur()>>>(reinterpret_cast<__nv_bfloat16*>(out.data_ptr()),
                                                                     reinterpret_cast<const __nv_bfloat16*>(bias->data_ptr()), total, N);
  }
}

}  // namespace nvfp4

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {

  m.def("scale_bytes", &nvfp4::scale_bytes);
  m.def("quantize_act", &nvfp4::quantize_act);
  m.def("swizzle_scales", &nvfp4::swizzle_scales);
  m.def("gemm", &nvfp4::gemm);
}

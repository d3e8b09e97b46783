// Python bindings: torch tensors in, raw pointers + the current CUDA stream out.
// No allocation happens here; callers own every buffer (so the calls are safe to
// capture in a CUDA graph).
#include <ATen/cuda/CUDAContext.h>
#include <torch/extension.h>

#include <cstring>

#include "attention.cuh"
#include "comm.cuh"
#include "expert_stack.cuh"
#include "gemm.cuh"
#include "launch.cuh"
#include "ops.cuh"

namespace {

using at::Tensor;
using OptT = c10::optional<Tensor>;

inline cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

inline void check(cudaError_t e, const char* what) {
  if (e != cudaSuccess) {
    // a launch error leaves a sticky "last error"; clear it so later calls report their own
    cudaGetLastError();
    TORCH_CHECK(false, what, ": ", cudaGetErrorString(e));
  }
}
inline const __nv_bfloat16* bf(const OptT& t) {
  if (!t.has_value() || !t->defined()) return nullptr;
  TORCH_CHECK(t->is_cuda() && t->scalar_type() == at::kBFloat16, "expected a CUDA bf16 tensor");
  return reinterpret_cast<const __nv_bfloat16*>(t->data_ptr());
}
inline const __nv_bfloat16* bf(const Tensor& t) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kBFloat16, "expected a CUDA bf16 tensor");
  return reinterpret_cast<const __nv_bfloat16*>(t.data_ptr());
}
inline __nv_bfloat16* bfm(const Tensor& t) { return const_cast<__nv_bfloat16*>(bf(t)); }
inline const float* f32(const OptT& t) {
  if (!t.has_value() || !t->defined()) return nullptr;
  TORCH_CHECK(t->is_cuda() && t->scalar_type() == at::kFloat, "expected a CUDA fp32 tensor");
  return reinterpret_cast<const float*>(t->data_ptr());
}
inline const int* i32(const OptT& t) {
  if (!t.has_value() || !t->defined()) return nullptr;
  TORCH_CHECK(t->is_cuda() && t->scalar_type() == at::kInt, "expected a CUDA int32 tensor");
  return reinterpret_cast<const int*>(t->data_ptr());
}
inline const long long* i64(const OptT& t) {
  if (!t.has_value() || !t->defined()) return nullptr;
  TORCH_CHECK(t->is_cuda() && t->scalar_type() == at::kLong, "expected a CUDA int64 tensor");
  return reinterpret_cast<const long long*>(t->data_ptr());
}

void gemm(const Tensor& x, const Tensor& w, Tensor& out, const OptT& bias, const OptT& residual,
          int64_t res_mod, const OptT& col_gate, const OptT& row_scale, const OptT& sumsq,
          int64_t act, bool glu, const OptT& a_scale, const OptT& w_scale, int64_t force_bn,
          int64_t force_swap, int64_t force_splits, const OptT& trace, int64_t wait_sig_ptr,
          int64_t wait_channel, int64_t wait_expect, int64_t row_rms_dim, double row_rms_eps,
          const OptT& rope, const OptT& zero, const OptT& out2, const OptT& col_scale2) {
  TORCH_CHECK(x.dim() == 2 && w.dim() == 2 && out.dim() == 2, "gemm: 2-D tensors expected");
  TORCH_CHECK(x.stride(1) == 1 && w.stride(1) == 1 && out.stride(1) == 1, "gemm: rows must be contiguous");
  TORCH_CHECK(x.size(1) == w.size(1), "gemm: K mismatch");
  const bool fp8 = x.scalar_type() == at::kFloat8_e4m3fn;
  TORCH_CHECK(fp8 || x.scalar_type() == at::kBFloat16, "gemm: x must be bf16 or float8_e4m3fn");
  TORCH_CHECK(w.scalar_type() == x.scalar_type(), "gemm: x and w dtypes differ");
  pb::GemmArgs a;
  a.x = x.data_ptr(); a.w = w.data_ptr(); a.out = out.data_ptr();
  a.M = int(x.size(0)); a.N = int(w.size(0)); a.K = int(x.size(1));
  a.ldx = int(x.stride(0)); a.ldw = int(w.stride(0)); a.ldo = int(out.stride(0));
  TORCH_CHECK(out.size(0) == a.M && out.size(1) == (glu ? a.N / 2 : a.N), "gemm: out shape");
  TORCH_CHECK(out.scalar_type() == at::kBFloat16 || out.scalar_type() == at::kFloat, "gemm: out dtype");
  a.out_fp32 = out.scalar_type() == at::kFloat;
  a.bias = bf(bias);
  if (residual.has_value() && residual->defined()) {
    TORCH_CHECK(residual->dim() == 2 && residual->stride(1) == 1, "gemm: residual layout");
    a.residual = bf(residual);
    a.ldr = int(residual->stride(0));
    a.res_mod = int(res_mod);
  }
  a.col_gate = bf(col_gate);
  a.row_scale = f32(row_scale);
  a.row_rms_dim = int(row_rms_dim); a.row_rms_eps = float(row_rms_eps);
  if (rope.has_value() && rope->defined()) {
    TORCH_CHECK(rope->is_cuda() && rope->scalar_type() == at::kByte && rope->is_contiguous() &&
                rope->numel() == int64_t(sizeof(pb::RopeEpi)), "gemm: rope must come from rope_epilogue_desc");
    TORCH_CHECK(a.N % 4 == 0, "gemm: rope epilogue needs N % 4 == 0");
    a.rope = reinterpret_cast<const pb::RopeEpi*>(rope->data_ptr());
  }
  if (zero.has_value() && zero->defined()) {
    TORCH_CHECK(zero->is_contiguous(), "gemm: zero must be contiguous");
    a.zero = const_cast<float*>(f32(zero)); a.zero_n = int(zero->numel());
  }
  a.sumsq = const_cast<float*>(f32(sumsq));
  if (out2.has_value() && out2->defined()) {
    TORCH_CHECK(out2->dim() == 2 && out2->stride(1) == 1 && out2->scalar_type() == at::kBFloat16 && out2->size(0) == out.size(0) &&
                out2->size(1) == out.size(1), "gemm: out2 must be bf16 of out's shape");
    TORCH_CHECK(col_scale2.has_value() && col_scale2->defined() && col_scale2->is_contiguous() && col_scale2->numel() == out.size(1),
                "gemm: out2 needs col_scale2 [N]");
    a.out2 = bfm(*out2); a.ldo2 = int(out2->stride(0)); a.col_scale2 = bf(col_scale2);
  }
  a.act = int(act); a.glu = glu ? 1 : 0; a.fp8 = fp8 ? 1 : 0;
  a.a_scale = f32(a_scale); a.w_scale = f32(w_scale);
  TORCH_CHECK(!fp8 || (a.a_scale && a.w_scale), "gemm: fp8 needs a_scale [M] and w_scale [N]");
  a.force_bn = int(force_bn); a.force_swap = int(force_swap); a.force_splits = int(force_splits);
  if (trace.has_value() && trace->defined()) {
    TORCH_CHECK(trace->is_cuda() && trace->scalar_type() == at::kLong && trace->is_contiguous(), "gemm: trace must be a CUDA int64 tensor");
    a.trace = reinterpret_cast<unsigned long long*>(trace->data_ptr());
  }
  pb::PushParams pp;
  if (wait_channel >= 0) {
    // x was written by peer GPUs: the kernel waits for wait_expect arrivals on the channel first
    memset(&pp, 0, sizeof(pp));
    pp.local_sig = reinterpret_cast<const void*>(static_cast<uintptr_t>(wait_sig_ptr));
    pp.wait_channel = int(wait_channel);
    pp.wait_expect = unsigned(wait_expect);
    a.push = &pp;
  }
  check(pb::gemm_launch(a, cur_stream()), "gemm_launch");
}

void gemm_fp8_block(const Tensor& x, const Tensor& w, Tensor& out, const Tensor& a_scale, const Tensor& w_scale,
                    const OptT& bias, const OptT& residual, const OptT& col_gate, int64_t act, bool glu) {
  TORCH_CHECK(x.dim() == 2 && w.dim() == 2 && out.dim() == 2, "gemm_fp8_block: 2-D tensors expected");
  TORCH_CHECK(x.scalar_type() == at::kFloat8_e4m3fn && w.scalar_type() == at::kFloat8_e4m3fn, "gemm_fp8_block: e4m3 operands");
  TORCH_CHECK(x.stride(1) == 1 && w.stride(1) == 1 && out.stride(1) == 1 && x.size(1) == w.size(1), "gemm_fp8_block: layout");
  pb::GemmArgs a;
  a.x = x.data_ptr(); a.w = w.data_ptr(); a.out = out.data_ptr();
  a.M = int(x.size(0)); a.N = int(w.size(0)); a.K = int(x.size(1));
  a.ldx = int(x.stride(0)); a.ldw = int(w.stride(0)); a.ldo = int(out.stride(0));
  const int64_t kb = a.K / 128;
  TORCH_CHECK(a.K % 128 == 0, "gemm_fp8_block: K must be a multiple of 128");
  TORCH_CHECK(a_scale.is_contiguous() && a_scale.numel() == int64_t(a.M) * kb, "gemm_fp8_block: a_scale must be [M, K/128]");
  TORCH_CHECK(w_scale.is_contiguous() && w_scale.numel() == int64_t((a.N + 127) / 128) * kb, "gemm_fp8_block: w_scale must be [ceil(N/128), K/128]");
  TORCH_CHECK(out.size(0) == a.M && out.size(1) == (glu ? a.N / 2 : a.N), "gemm_fp8_block: out shape");
  a.out_fp32 = out.scalar_type() == at::kFloat;
  a.a_scale = f32(OptT(a_scale)); a.w_scale = f32(OptT(w_scale));
  a.bias = bf(bias); a.col_gate = bf(col_gate);
  if (residual.has_value() && residual->defined()) { a.residual = bf(residual); a.ldr = int(residual->stride(0)); }
  a.act = int(act); a.glu = glu ? 1 : 0; a.fp8 = 1; a.block_scaled = 1;
  check(pb::gemm_fp8_block_launch(a, cur_stream()), "gemm_fp8_block_launch");
}

void attention(const Tensor& q, const Tensor& k, const Tensor& v, Tensor& out,
               const Tensor& q_start, const Tensor& q_len, const Tensor& kv_indptr,
               const Tensor& kv_len, const OptT& kv_indices, int64_t max_q_len, bool causal,
               int64_t splits, double sm_scale, int64_t impl, const OptT& trace, int64_t window, double soft_cap) {
  // q/out: [tokens, Hq, D]; k/v: [rows, Hkv, D]; innermost dim contiguous
  TORCH_CHECK(q.dim() == 3 && k.dim() == 3 && v.dim() == 3 && out.dim() == 3, "attention: 3-D tensors");
  TORCH_CHECK(q.stride(2) == 1 && k.stride(2) == 1 && v.stride(2) == 1 && out.stride(2) == 1,
              "attention: head_dim must be contiguous");
  TORCH_CHECK(k.stride(0) == v.stride(0) && k.stride(1) == v.stride(1), "attention: k/v strides differ");
  pb::AttnParams p;
  p.q = bf(q); p.k = bf(k); p.v = bf(v); p.out = bfm(out);
  p.q_start = i32(q_start); p.q_len = i32(q_len); p.kv_indptr = i32(kv_indptr); p.kv_len = i32(kv_len);
  p.kv_indices = i32(kv_indices);
  p.q_tok_stride = q.stride(0); p.q_head_stride = q.stride(1);
  p.kv_row_stride = k.stride(0); p.kv_head_stride = k.stride(1);
  p.o_tok_stride = out.stride(0); p.o_head_stride = out.stride(1);
  p.batch = int(q_len.numel());
  p.num_kv_heads = int(k.size(1));
  TORCH_CHECK(q.size(1) % k.size(1) == 0, "attention: Hq must be a multiple of Hkv");
  p.group = int(q.size(1) / k.size(1));
  p.head_dim = int(q.size(2));
  p.max_q_len = int(max_q_len);
  p.causal = causal ? 1 : 0;
  p.splits = int(splits);
  p.sm_scale = float(sm_scale);
  p.window = int(window); p.soft_cap = float(soft_cap);
  TORCH_CHECK((window <= 0 && soft_cap <= 0) || impl == 1, "attention: sliding window / soft cap are served by the tcgen05 latency kernel (impl 1)");
  p.q_rows = q.size(0); p.kv_rows = k.size(0);
  if (trace.has_value() && trace->defined()) p.trace = reinterpret_cast<unsigned long long*>(trace->data_ptr());
  // impl: 0 = mma.sync, 1 = tcgen05 (latency variant), 2 = tcgen05 pipelined (throughput variant)
  if (impl == 2) check(pb::attn_pp_launch(p, cur_stream()), "attn_pp_launch");
  else if (impl == 1) check(pb::attn_tc_launch(p, cur_stream()), "attn_tc_launch");
  else check(pb::attn_launch(p, cur_stream()), "attn_launch");
}

void norm(const Tensor& x, const OptT& y, int64_t mode, const OptT& weight, const OptT& bias,
          const OptT& mod, int64_t group, const OptT& residual, const OptT& sumsq, double eps,
          const OptT& y8, const OptT& y8_scale, int64_t y8_block) {
  TORCH_CHECK(x.dim() == 2 && x.stride(1) == 1, "norm: x must be 2-D with contiguous rows");
  pb::NormArgs a;
  a.x = bf(x); a.rows = int(x.size(0)); a.D = int(x.size(1)); a.ldx = int(x.stride(0));
  if (y.has_value() && y->defined()) {
    TORCH_CHECK(y->dim() == 2 && y->stride(1) == 1 && y->size(0) == x.size(0) && y->size(1) == x.size(1), "norm: y shape");
    a.y = bfm(*y); a.ldy = int(y->stride(0));
  }
  a.weight = bf(weight); a.bias = bf(bias); a.mod = bf(mod);
  a.group = int(group); a.mode = int(mode); a.eps = float(eps);
  if (residual.has_value() && residual->defined()) {
    a.residual = bfm(*residual); a.ldr = int(residual->stride(0));
  }
  a.sumsq = f32(sumsq);
  if (y8.has_value() && y8->defined()) {
    TORCH_CHECK(y8->is_contiguous(), "norm: y8 must be contiguous");
    a.y8 = reinterpret_cast<uint8_t*>(y8->data_ptr());
    a.y8_scale = const_cast<float*>(f32(y8_scale));
    a.y8_block = int(y8_block);
  }
  if (a.mode == pb::kNormLayer) TORCH_CHECK(a.weight && a.bias, "layernorm needs weight and bias");
  if (a.mode == pb::kNormRms || a.mode == pb::kNormGemmaRms) TORCH_CHECK(a.weight, "rmsnorm needs weight");
  if (a.mode == pb::kNormAdaRms) TORCH_CHECK(a.mod && a.group > 0, "adarmsnorm needs modulation");
  check(pb::norm_launch(a, cur_stream()), "norm_launch");
}

// Device-resident descriptor for the GEMM's rotate-and-scatter epilogue (see pb::RopeEpi). The caller
// keeps the returned tensor and every tensor named here alive for as long as launches use it.
Tensor rope_epilogue_desc(const Tensor& q_out, const Tensor& k_pool, const Tensor& v_pool, const Tensor& cos_sin,
                          const Tensor& pos, const Tensor& slots, int64_t Hq, int64_t Hkv, int64_t D) {
  TORCH_CHECK(q_out.dim() == 2 && q_out.stride(1) == 1 && q_out.size(1) == Hq * D, "rope_epilogue_desc: q_out layout");
  TORCH_CHECK(k_pool.stride(0) == v_pool.stride(0) && k_pool.stride(0) >= Hkv * D, "rope_epilogue_desc: pools");
  TORCH_CHECK(D % 8 == 0 && cos_sin.size(-1) == D && cos_sin.is_contiguous(), "rope_epilogue_desc: cos_sin must be [positions, D]");
  pb::RopeEpi r;
  memset(&r, 0, sizeof(r));
  r.q_out = bfm(q_out);
  r.k_pool = bfm(k_pool);
  r.v_pool = bfm(v_pool);
  r.cos_sin = f32(cos_sin);
  r.pos = i32(pos);
  r.slots = i64(slots);
  TORCH_CHECK(r.pos && r.slots, "rope_epilogue_desc: pos (int32) and slots (int64) are required");
  r.pool_stride = k_pool.stride(0);
  r.ldq = int(q_out.stride(0)); r.Hq = int(Hq); r.Hkv = int(Hkv); r.D = int(D);
  Tensor host = at::empty({int64_t(sizeof(r))}, at::TensorOptions().dtype(at::kByte));
  memcpy(host.data_ptr(), &r, sizeof(r));
  return host.to(q_out.device());
}

void rope_kv(const Tensor& qkv, int64_t Hq, int64_t Hkv, int64_t D, const OptT& pos,
             const OptT& cos_sin, int64_t rot_dim, const OptT& q_norm_w, const OptT& k_norm_w,
             double norm_eps, Tensor& q_out, const OptT& k_pool, const OptT& v_pool,
             const OptT& slots, int64_t slot_base, const OptT& zero) {
  TORCH_CHECK(qkv.dim() == 2 && qkv.stride(1) == 1, "rope_kv: qkv layout");
  TORCH_CHECK(qkv.size(1) == (Hq + 2 * Hkv) * D, "rope_kv: qkv width");
  pb::RopeKvArgs a;
  a.qkv = bf(qkv); a.M = int(qkv.size(0)); a.ld = int(qkv.stride(0));
  a.Hq = int(Hq); a.Hkv = int(Hkv); a.D = int(D);
  a.pos = i32(pos); a.cos_sin = f32(cos_sin); a.rot_dim = int(rot_dim);
  a.q_norm_w = bf(q_norm_w); a.k_norm_w = bf(k_norm_w); a.norm_eps = float(norm_eps);
  TORCH_CHECK(q_out.dim() == 2 && q_out.stride(1) == 1, "rope_kv: q_out layout");
  a.q_out = bfm(q_out); a.ldq = int(q_out.stride(0));
  if (k_pool.has_value() && k_pool->defined()) {
    TORCH_CHECK(v_pool.has_value() && k_pool->stride(0) == v_pool->stride(0), "rope_kv: pools");
    a.k_pool = bfm(*k_pool); a.v_pool = bfm(*v_pool);
    a.pool_row_stride = k_pool->stride(0);
  }
  a.slots = i64(slots); a.slot_base = slot_base;
  if (zero.has_value() && zero->defined()) {
    TORCH_CHECK(zero->is_contiguous(), "rope_kv: zero must be contiguous");
    a.zero = const_cast<float*>(f32(zero)); a.zero_n = int(zero->numel());
  }
  check(pb::rope_kv_launch(a, cur_stream()), "rope_kv_launch");
}

void embedding(const Tensor& ids, const Tensor& table, int64_t lo, int64_t hi, double scale,
               Tensor& out, const OptT& dst_rows) {
  TORCH_CHECK(ids.is_contiguous() && table.is_contiguous() && out.stride(-1) == 1, "embedding: layout");
  check(pb::embedding_launch(i64(OptT(ids)), int(ids.numel()), bf(table), int(table.size(1)), lo,
                             hi, float(scale), bfm(out), int(out.stride(0)), i32(dst_rows),
                             cur_stream()),
        "embedding_launch");
}

void im2col(const Tensor& pix, int64_t patch, Tensor& out) {
  TORCH_CHECK(pix.dim() == 4 && pix.is_contiguous() && out.is_contiguous(), "im2col: layout");
  check(pb::im2col_launch(bf(pix), int(pix.size(0)), int(pix.size(1)), int(pix.size(2)),
                          int(pix.size(3)), int(patch), bfm(out), int(out.size(1)), cur_stream()),
        "im2col_launch");
}

void gated_act(const Tensor& x, Tensor& y, int64_t act, bool interleaved) {
  TORCH_CHECK(x.is_contiguous() && y.is_contiguous() && x.size(-1) == 2 * y.size(-1), "gated_act: layout");
  const int I = int(y.size(-1));
  check(pb::gated_act_launch(bf(x), bfm(y), int(y.numel() / I), I, int(act), interleaved ? 1 : 0,
                             cur_stream()),
        "gated_act_launch");
}

void unary(const Tensor& x, Tensor& y, int64_t act) {
  TORCH_CHECK(x.is_contiguous() && y.is_contiguous() && x.numel() == y.numel(), "unary: layout");
  check(pb::unary_launch(bf(x), bfm(y), x.numel(), int(act), cur_stream()), "unary_launch");
}

void axpy(Tensor& x, const Tensor& v, double dt) {
  TORCH_CHECK(x.is_contiguous() && v.is_contiguous() && x.numel() == v.numel(), "axpy: layout");
  TORCH_CHECK(x.scalar_type() == at::kFloat || x.scalar_type() == at::kBFloat16, "axpy: x dtype");
  check(pb::axpy_launch(x.data_ptr(), x.scalar_type() == at::kFloat, bf(v), float(dt), x.numel(),
                        cur_stream()),
        "axpy_launch");
}

Tensor gdn_decode(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& g, const Tensor& beta,
                  Tensor& state_pool, const Tensor& state_indices, double scale, bool l2norm) {
  TORCH_CHECK(q.dim() == 3 && k.sizes() == q.sizes() && v.dim() == 3 && v.size(0) == q.size(0) && v.size(1) == q.size(1),
              "gdn_decode: q, k [B, H, Dk], v [B, H, Dv]");
  const auto dt = q.scalar_type();
  TORCH_CHECK((dt == at::kBFloat16 || dt == at::kFloat) && k.scalar_type() == dt && v.scalar_type() == dt &&
              g.scalar_type() == dt && beta.scalar_type() == dt, "gdn_decode: inputs must all be fp32 or all bf16");
  TORCH_CHECK(q.is_cuda() && q.is_contiguous() && k.is_contiguous() && v.is_contiguous() && g.is_contiguous() &&
              beta.is_contiguous(), "gdn_decode: contiguous CUDA inputs");
  const int B = int(q.size(0)), H = int(q.size(1)), Dk = int(q.size(2)), Dv = int(v.size(2));
  TORCH_CHECK(g.numel() == int64_t(B) * H && beta.numel() == int64_t(B) * H, "gdn_decode: g, beta [B, H]");
  TORCH_CHECK(state_pool.is_cuda() && state_pool.scalar_type() == at::kFloat && state_pool.is_contiguous() &&
              state_pool.dim() == 4 && state_pool.size(1) == H && state_pool.size(2) == Dk && state_pool.size(3) == Dv,
              "gdn_decode: state_pool must be fp32 [slots, H, Dk, Dv]");
  TORCH_CHECK(state_indices.is_cuda() && state_indices.scalar_type() == at::kLong && state_indices.numel() == B,
              "gdn_decode: state_indices int64 [B]");
  Tensor out = at::empty_like(v);
  check(pb::gdn_decode_launch(q.data_ptr(), k.data_ptr(), v.data_ptr(), g.data_ptr(), beta.data_ptr(), dt == at::kBFloat16,
                              reinterpret_cast<float*>(state_pool.data_ptr()), i64(OptT(state_indices)), out.data_ptr(),
                              dt == at::kBFloat16, B, H, Dk, Dv, float(scale), l2norm ? 1 : 0, cur_stream()),
        "gdn_decode_launch");
  return out;
}

Tensor snake(const Tensor& x, const Tensor& alpha, const Tensor& beta) {
  TORCH_CHECK(x.is_cuda() && x.dim() == 3 && x.is_contiguous(), "snake: x must be a contiguous CUDA [B, C, T] tensor");
  TORCH_CHECK(x.scalar_type() == at::kBFloat16 || x.scalar_type() == at::kFloat, "snake: bf16 or fp32");
  TORCH_CHECK(alpha.numel() == x.size(1) && beta.numel() == x.size(1) && alpha.is_contiguous() && beta.is_contiguous(),
              "snake: alpha, beta [C]");
  Tensor out = at::empty_like(x);
  check(pb::snake_launch(x.data_ptr(), out.data_ptr(), x.scalar_type() == at::kBFloat16, f32(OptT(alpha)), f32(OptT(beta)),
                         int(x.size(1)), x.size(2), x.numel(), cur_stream()), "snake_launch");
  return out;
}

void cfg_combine(const Tensor& cond, const Tensor& uncond, double g, const OptT& out,
                 const OptT& x_fp32, double dt) {
  TORCH_CHECK(cond.is_contiguous() && uncond.is_contiguous() && cond.numel() == uncond.numel(), "cfg_combine: layout");
  __nv_bfloat16* o = (out.has_value() && out->defined()) ? bfm(*out) : nullptr;
  check(pb::cfg_combine_launch(bf(cond), bf(uncond), float(g), o,
                               const_cast<float*>(f32(x_fp32)), float(dt), cond.numel(),
                               cur_stream()),
        "cfg_combine_launch");
}

Tensor domain_linear(const Tensor& x, const Tensor& w, const Tensor& bias, const Tensor& domain) {
  TORCH_CHECK(x.is_cuda() && x.dim() == 3 && x.is_contiguous() && x.scalar_type() == at::kBFloat16, "domain_linear: x bf16 [B, T, K]");
  const int64_t B = x.size(0), T = x.size(1), K = x.size(2);
  TORCH_CHECK(w.is_contiguous() && w.scalar_type() == at::kBFloat16 && w.dim() == 2 && w.size(1) % K == 0, "domain_linear: w bf16 [domains, K * N]");
  const int64_t N = w.size(1) / K;
  TORCH_CHECK(bias.is_contiguous() && bias.scalar_type() == at::kBFloat16 && bias.dim() == 2 && bias.size(0) == w.size(0) && bias.size(1) == N,
              "domain_linear: bias bf16 [domains, N]");
  TORCH_CHECK(domain.is_cuda() && domain.is_contiguous() && domain.scalar_type() == at::kLong && domain.numel() == B, "domain_linear: domain int64 [B]");
  Tensor y = at::empty({B, T, N}, x.options());
  check(pb::domain_linear_launch(bf(x), bf(w), bf(bias), i64(OptT(domain)), bfm(y), int(B), int(T), int(K), int(N), cur_stream()),
        "domain_linear_launch");
  return y;
}

Tensor linear_simt(const Tensor& x, const Tensor& w, const OptT& bias) {
  auto code = [](const Tensor& t) {
    switch (t.scalar_type()) {
      case at::kFloat: return 0;
      case at::kBFloat16: return 1;
      case at::kHalf: return 2;
      default: TORCH_CHECK(false, "linear_simt: fp32 / bf16 / fp16 only"); return -1;
    }
  };
  TORCH_CHECK(x.is_cuda() && w.is_cuda() && x.dim() == 2 && w.dim() == 2 && x.stride(1) == 1 && w.stride(1) == 1 &&
              x.size(1) == w.size(1), "linear_simt: x [M, K], w [N, K], unit inner strides");
  const void* b = nullptr;
  if (bias.has_value() && bias->defined()) {
    TORCH_CHECK(bias->is_contiguous() && bias->numel() == w.size(0) && bias->scalar_type() == w.scalar_type(), "linear_simt: bias [N] of the weight's dtype");
    b = bias->data_ptr();
  }
  Tensor y = at::empty({x.size(0), w.size(0)}, x.options());
  check(pb::linear_simt_launch(x.data_ptr(), code(x), w.data_ptr(), code(w), b, y.data_ptr(), int(x.size(0)), int(w.size(0)),
                               int(x.size(1)), int(x.stride(0)), int(w.stride(0)), int(y.stride(0)), cur_stream()), "linear_simt_launch");
  return y;
}

void unipc_step(const Tensor& v, const OptT& v_uncond, double g, Tensor& x, Tensor& x_last, Tensor& m1, Tensor& m2,
                double sigma, bool has_corr, std::vector<double> corr, std::vector<double> pred, const OptT& keep,
                const OptT& cond, int64_t C, int64_t T, int64_t inner, int64_t live_inner) {
  TORCH_CHECK(v.is_cuda() && v.is_contiguous() && x.is_contiguous() && v.numel() == x.numel(), "unipc_step: v / x layout");
  TORCH_CHECK(v.scalar_type() == at::kBFloat16 && x.scalar_type() == at::kBFloat16, "unipc_step: bf16 velocity and sample");
  for (const Tensor* t : {&x_last, &m1, &m2})
    TORCH_CHECK(t->is_contiguous() && t->scalar_type() == at::kFloat && t->numel() == x.numel(), "unipc_step: fp32 state of the sample's size");
  TORCH_CHECK(corr.size() == 4 && pred.size() == 3, "unipc_step: corr (c_x, c_0, c_1, c_t), pred (p_x, p_0, p_1)");
  TORCH_CHECK(C > 0 && T > 0 && inner > 0 && x.numel() % (C * T * inner) == 0, "unipc_step: [B, C, T, inner] view");
  pb::UniPCStepArgs a;
  a.v = bf(v); a.v_uncond = nullptr; a.g = float(g);
  if (v_uncond.has_value() && v_uncond->defined()) {
    TORCH_CHECK(v_uncond->is_contiguous() && v_uncond->scalar_type() == at::kBFloat16 && v_uncond->numel() == v.numel(), "unipc_step: v_uncond");
    a.v_uncond = bf(*v_uncond);
  }
  a.x = bfm(x); a.x_last = reinterpret_cast<float*>(x_last.data_ptr());
  a.m1 = reinterpret_cast<float*>(m1.data_ptr()); a.m2 = reinterpret_cast<float*>(m2.data_ptr());
  a.sigma = float(sigma); a.has_corr = has_corr ? 1 : 0;
  a.c_x = float(corr[0]); a.c_0 = float(corr[1]); a.c_1 = float(corr[2]); a.c_t = float(corr[3]);
  a.p_x = float(pred[0]); a.p_0 = float(pred[1]); a.p_1 = float(pred[2]);
  a.keep = nullptr; a.cond = nullptr;
  if (keep.has_value() && keep->defined()) {
    TORCH_CHECK(cond.has_value() && cond->defined() && cond->is_contiguous() && cond->scalar_type() == at::kBFloat16 &&
                cond->numel() == x.numel(), "unipc_step: cond must match the sample");
    TORCH_CHECK(keep->is_contiguous() && keep->element_size() == 1 && keep->numel() == x.numel() / (C * inner), "unipc_step: keep is [B, T] bytes");
    a.keep = reinterpret_cast<const unsigned char*>(keep->data_ptr());
    a.cond = bf(*cond);
  }
  a.n = x.numel(); a.inner = inner; a.T = T; a.C = C; a.live_inner = live_inner > 0 ? live_inner : inner;
  check(pb::unipc_step_launch(a, cur_stream()), "unipc_step_launch");
}

void scatter_rows(const Tensor& src, Tensor& dst, const OptT& rows) {
  TORCH_CHECK(src.dim() == 2 && dst.dim() == 2 && src.stride(1) == 1 && dst.stride(1) == 1, "scatter_rows: layout");
  check(pb::scatter_rows_launch(bf(src), int(src.size(0)), int(src.size(1)), int(src.stride(0)),
                                bfm(dst), int(dst.stride(0)), i32(rows), cur_stream()),
        "scatter_rows_launch");
}

void quant_fp8(const Tensor& x, Tensor& y, Tensor& scale, int64_t block) {
  TORCH_CHECK(x.dim() == 2 && x.stride(1) == 1 && y.is_contiguous(), "quant_fp8: layout");
  check(pb::quant_fp8_launch(bf(x), int(x.size(0)), int(x.size(1)), int(x.stride(0)),
                             reinterpret_cast<uint8_t*>(y.data_ptr()),
                             const_cast<float*>(f32(OptT(scale))), int(block), cur_stream()),
        "quant_fp8_launch");
}

// Tensor maps of the persistent action-expert kernel: per layer (qkv, o, gate_up, down) weight maps with
// 64 x 128 boxes, then the attention-output buffer with a 64 x 64 box; returned as a device byte tensor
// that the caller keeps alive together with the tensors named here.
Tensor expert_stack_tmaps(const std::vector<Tensor>& weights, const Tensor& attn) {
  TORCH_CHECK(!weights.empty() && weights.size() % 4 == 0, "expert_stack_tmaps: four weights per layer");
  const size_t n = weights.size() + 1;
  Tensor host = at::empty({int64_t(n * sizeof(CUtensorMap))}, at::TensorOptions().dtype(at::kByte));
  CUtensorMap* maps = reinterpret_cast<CUtensorMap*>(host.data_ptr());
  for (size_t i = 0; i < weights.size(); ++i) {
    const Tensor& w = weights[i];
    TORCH_CHECK(w.is_cuda() && w.scalar_type() == at::kBFloat16 && w.dim() == 2 && w.stride(1) == 1 &&
                w.size(0) % 128 == 0 && w.size(1) % 64 == 0, "expert_stack_tmaps: weight ", i, " must be bf16 [128a, 64b]");
    TORCH_CHECK(pb::make_tmap_2d(&maps[i], w.data_ptr(), uint64_t(w.size(0)), uint64_t(w.size(1)), uint64_t(w.stride(0)), 128, 2),
                "expert_stack_tmaps: cuTensorMapEncodeTiled failed");
  }
  TORCH_CHECK(attn.is_cuda() && attn.scalar_type() == at::kBFloat16 && attn.dim() == 2 && attn.size(0) == 64 &&
              attn.is_contiguous(), "expert_stack_tmaps: attn must be bf16 [64, Hq * D]");
  TORCH_CHECK(pb::make_tmap_2d(&maps[n - 1], attn.data_ptr(), 64, uint64_t(attn.size(1)), uint64_t(attn.stride(0)), 64, 2),
              "expert_stack_tmaps: cuTensorMapEncodeTiled failed");
  // cudaMalloc'ed storage is 256-byte aligned, which covers the 64-byte alignment a tensor map needs
  return host.to(attn.device());
}

int64_t expert_stack_grid() { return pb::expert_stack_grid(); }

void expert_stack_run(const Tensor& tmaps, int64_t M, int64_t H, int64_t I, int64_t Hq, int64_t D, int64_t A,
                      int64_t n_layers, int64_t step_begin, int64_t step_end, int64_t att_splits, double eps,
                      double dt, double sm_scale, const Tensor& in_scale, const Tensor& post_scale,
                      const Tensor& gate_in, const Tensor& gate_post, const Tensor& qkv_bias, const Tensor& gu_bias,
                      const Tensor& fin_scale, const Tensor& out_bias, const Tensor& w_in, const Tensor& b_in,
                      const Tensor& w_out, const Tensor& k_pool, const Tensor& v_pool, const Tensor& kv_ptr,
                      const Tensor& kv_len, const Tensor& pos, const Tensor& cos_sin, const Tensor& x0, Tensor& out,
                      Tensor& scratch_f32, Tensor& attn, Tensor& barrier, const OptT& trace, int64_t debug) {
  pb::ExpertStackParams p;
  p.M = int(M); p.H = int(H); p.I = int(I); p.Hq = int(Hq); p.D = int(D); p.A = int(A);
  p.n_layers = int(n_layers); p.step_begin = int(step_begin); p.step_end = int(step_end);
  p.att_splits = int(att_splits);
  p.eps = float(eps); p.dt = float(dt); p.sm_scale = float(sm_scale);
  TORCH_CHECK(tmaps.is_cuda() && tmaps.scalar_type() == at::kByte && tmaps.is_contiguous() &&
              tmaps.numel() == int64_t((n_layers * 4 + 1) * sizeof(CUtensorMap)), "expert_stack_run: tmaps");
  p.tmaps = reinterpret_cast<const CUtensorMap*>(tmaps.data_ptr());
  const int64_t SL = step_end * n_layers, Nqkv = (Hq + 2) * D;
  const auto vec = [](const Tensor& t, int64_t min_numel, const char* name) {
    TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kFloat && t.is_contiguous() && t.numel() >= min_numel,
                "expert_stack_run: ", name, " must be a contiguous CUDA fp32 tensor of at least ", min_numel, " elements");
    return reinterpret_cast<const float*>(t.data_ptr());
  };
  p.in_scale = vec(in_scale, SL * H, "in_scale"); p.post_scale = vec(post_scale, SL * H, "post_scale");
  p.gate_in = vec(gate_in, SL * H, "gate_in"); p.gate_post = vec(gate_post, SL * H, "gate_post");
  p.qkv_bias = vec(qkv_bias, SL * Nqkv, "qkv_bias"); p.gu_bias = vec(gu_bias, SL * 2 * I, "gu_bias");
  p.fin_scale = vec(fin_scale, step_end * H, "fin_scale"); p.out_bias = vec(out_bias, step_end * A, "out_bias");
  TORCH_CHECK(w_in.is_contiguous() && w_in.numel() == H * A && b_in.numel() == H && w_out.is_contiguous() &&
              w_out.numel() == A * H, "expert_stack_run: input / output projection shapes");
  p.w_in = bf(w_in); p.b_in = bf(b_in); p.w_out = bf(w_out);
  TORCH_CHECK(k_pool.dim() == 4 && k_pool.size(2) == 1 && k_pool.size(3) == D && k_pool.stride(3) == 1 &&
              k_pool.size(0) >= n_layers && k_pool.strides() == v_pool.strides(), "expert_stack_run: pools must be [layers, slots, 1, D]");
  p.k_pool = bf(k_pool); p.v_pool = bf(v_pool);
  p.pool_layer_stride = k_pool.stride(0); p.pool_row_stride = k_pool.stride(1);
  TORCH_CHECK(p.pool_row_stride % 8 == 0 && p.pool_layer_stride % 8 == 0, "expert_stack_run: pool strides");
  p.kv_ptr = i32(OptT(kv_ptr)); p.kv_len = i32(OptT(kv_len)); p.pos = i32(OptT(pos));
  TORCH_CHECK(pos.numel() >= M && cos_sin.is_contiguous() && cos_sin.size(-1) == D, "expert_stack_run: pos / cos_sin");
  p.cos_sin = f32(OptT(cos_sin));
  TORCH_CHECK(x0.is_contiguous() && x0.numel() >= M * A && out.is_contiguous() && out.numel() >= M * A, "expert_stack_run: x0 / out");
  p.x0 = bf(x0); p.out = bfm(out);
  // fp32 scratch: x_t | h | acc_qkv | acc_gu | ss | part_o | part_ml, every block 64 rows
  const int64_t need = 64 * (A + H + Nqkv + 2 * I + 2) + Hq * att_splits * 64 * (D + 2);
  TORCH_CHECK(scratch_f32.is_cuda() && scratch_f32.scalar_type() == at::kFloat && scratch_f32.is_contiguous() &&
              scratch_f32.numel() >= need, "expert_stack_run: scratch_f32 needs ", need, " floats");
  float* s = reinterpret_cast<float*>(scratch_f32.data_ptr());
  p.x_t = s; s += 64 * A;
  p.h = s; s += 64 * H;
  p.acc_qkv = s; s += 64 * Nqkv;
  p.acc_gu = s; s += 64 * 2 * I;
  p.ss = s; s += 128;
  p.part_o = s; s += Hq * att_splits * 64 * D;
  p.part_ml = s;
  TORCH_CHECK(attn.is_cuda() && attn.scalar_type() == at::kBFloat16 && attn.is_contiguous() && attn.numel() == 64 * Hq * D,
              "expert_stack_run: attn must be bf16 [64, Hq * D]");
  p.attn = bfm(attn);
  TORCH_CHECK(barrier.is_cuda() && barrier.scalar_type() == at::kInt && barrier.numel() >= 1, "expert_stack_run: barrier");
  p.barrier = reinterpret_cast<unsigned*>(barrier.data_ptr());
  p.status = pb::kernel_status_ptr();
  if (trace.has_value() && trace->defined()) {
    TORCH_CHECK(trace->is_cuda() && trace->scalar_type() == at::kLong && trace->is_contiguous() &&
                trace->numel() >= 64 * pb::expert_stack_grid(), "expert_stack_run: trace needs 64 int64 per CTA");
    p.trace = reinterpret_cast<unsigned long long*>(trace->data_ptr());
  }
  p.debug = int(debug);
  check(pb::expert_stack_launch(p, cur_stream()), "expert_stack_launch");
}

}  // namespace

void register_comm(pybind11::module_& m);

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  namespace py = pybind11;
  m.def("gemm", &gemm, py::arg("x"), py::arg("w"), py::arg("out"), py::arg("bias") = py::none(),
        py::arg("residual") = py::none(), py::arg("res_mod") = 0, py::arg("col_gate") = py::none(),
        py::arg("row_scale") = py::none(), py::arg("sumsq") = py::none(), py::arg("act") = 0,
        py::arg("glu") = false, py::arg("a_scale") = py::none(), py::arg("w_scale") = py::none(),
        py::arg("force_bn") = 0, py::arg("force_swap") = -1, py::arg("force_splits") = 0,
        py::arg("trace") = py::none(), py::arg("wait_sig_ptr") = 0, py::arg("wait_channel") = -1,
        py::arg("wait_expect") = 0, py::arg("row_rms_dim") = 0, py::arg("row_rms_eps") = 0.0,
        py::arg("rope") = py::none(), py::arg("zero") = py::none(), py::arg("out2") = py::none(),
        py::arg("col_scale2") = py::none());
  m.def("rope_epilogue_desc", &rope_epilogue_desc, py::arg("q_out"), py::arg("k_pool"), py::arg("v_pool"),
        py::arg("cos_sin"), py::arg("pos"), py::arg("slots"), py::arg("Hq"), py::arg("Hkv"), py::arg("D"));
  m.def("gemm_fp8_block", &gemm_fp8_block, py::arg("x"), py::arg("w"), py::arg("out"), py::arg("a_scale"), py::arg("w_scale"),
        py::arg("bias") = py::none(), py::arg("residual") = py::none(), py::arg("col_gate") = py::none(), py::arg("act") = 0,
        py::arg("glu") = false);
  m.def("attention", &attention, py::arg("q"), py::arg("k"), py::arg("v"), py::arg("out"),
        py::arg("q_start"), py::arg("q_len"), py::arg("kv_indptr"), py::arg("kv_len"),
        py::arg("kv_indices") = py::none(), py::arg("max_q_len"), py::arg("causal") = false,
        py::arg("splits") = 1, py::arg("sm_scale") = 1.0, py::arg("impl") = 1, py::arg("trace") = py::none(),
        py::arg("window") = 0, py::arg("soft_cap") = 0.0);
  m.def("norm", &norm, py::arg("x"), py::arg("y"), py::arg("mode"), py::arg("weight") = py::none(),
        py::arg("bias") = py::none(), py::arg("mod") = py::none(), py::arg("group") = 1,
        py::arg("residual") = py::none(), py::arg("sumsq") = py::none(), py::arg("eps") = 1e-6,
        py::arg("y8") = py::none(), py::arg("y8_scale") = py::none(), py::arg("y8_block") = 0);
  m.def("rope_kv", &rope_kv, py::arg("qkv"), py::arg("Hq"), py::arg("Hkv"), py::arg("D"),
        py::arg("pos") = py::none(), py::arg("cos_sin") = py::none(), py::arg("rot_dim") = 0,
        py::arg("q_norm_w") = py::none(), py::arg("k_norm_w") = py::none(),
        py::arg("norm_eps") = 1e-6, py::arg("q_out"), py::arg("k_pool") = py::none(),
        py::arg("v_pool") = py::none(), py::arg("slots") = py::none(), py::arg("slot_base") = 0,
        py::arg("zero") = py::none());
  m.def("embedding", &embedding, py::arg("ids"), py::arg("table"), py::arg("lo"), py::arg("hi"),
        py::arg("scale"), py::arg("out"), py::arg("dst_rows") = py::none());
  m.def("im2col", &im2col);
  m.def("gated_act", &gated_act);
  m.def("unary", &unary);
  m.def("axpy", &axpy);
  m.def("cfg_combine", &cfg_combine, py::arg("cond"), py::arg("uncond"), py::arg("g"),
        py::arg("out") = py::none(), py::arg("x_fp32") = py::none(), py::arg("dt") = 0.0);
  m.def("scatter_rows", &scatter_rows, py::arg("src"), py::arg("dst"), py::arg("rows") = py::none());
  m.def("quant_fp8", &quant_fp8);
  m.def("snake", &snake);
  m.def("unipc_step", &unipc_step);
  m.def("linear_simt", &linear_simt);
  m.def("domain_linear", &domain_linear);
  m.def("gdn_decode", &gdn_decode, py::arg("q"), py::arg("k"), py::arg("v"), py::arg("g"), py::arg("beta"),
        py::arg("state_pool"), py::arg("state_indices"), py::arg("scale"), py::arg("l2norm") = true);
  m.def("kernel_status", [] { return pb::read_and_clear_kernel_status(); });
  m.def("launch_counter", [] { return pb::launch_counter(); });
  m.def("reset_launch_counter", [] { pb::reset_launch_counter(); });
  m.def("set_pdl", [](bool on) { pb::set_pdl_enabled(on); });
  m.def("set_gemm_2cta", [](int64_t mode) { pb::set_gemm_2cta(int(mode)); });
  m.def("gemm_2cta_launches", []() { return int64_t(pb::gemm_2cta_launches()); });
  m.def("pdl_enabled", [] { return pb::pdl_enabled(); });
  m.def("expert_stack_tmaps", &expert_stack_tmaps);
  m.def("expert_stack_grid", &expert_stack_grid);
  m.def("expert_stack_run", &expert_stack_run, py::arg("tmaps"), py::arg("M"), py::arg("H"), py::arg("I"), py::arg("Hq"),
        py::arg("D"), py::arg("A"), py::arg("n_layers"), py::arg("step_begin"), py::arg("step_end"), py::arg("att_splits"),
        py::arg("eps"), py::arg("dt"), py::arg("sm_scale"), py::arg("in_scale"), py::arg("post_scale"), py::arg("gate_in"),
        py::arg("gate_post"), py::arg("qkv_bias"), py::arg("gu_bias"), py::arg("fin_scale"), py::arg("out_bias"),
        py::arg("w_in"), py::arg("b_in"), py::arg("w_out"), py::arg("k_pool"), py::arg("v_pool"), py::arg("kv_ptr"),
        py::arg("kv_len"), py::arg("pos"), py::arg("cos_sin"), py::arg("x0"), py::arg("out"), py::arg("scratch_f32"),
        py::arg("attn"), py::arg("barrier"), py::arg("trace") = py::none(), py::arg("debug") = 0);
  register_comm(m);
}

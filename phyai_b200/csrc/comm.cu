// Peer-memory communication kernels and the symmetric (IPC-shared) buffers under them.
//
// Each rank cudaMalloc's one slab and exports it with cudaIpcGetMemHandle; the handles
// travel over the host process group and every peer maps them with
// cudaIpcOpenMemHandle. All inter-GPU traffic in the kernels below is plain ld/st to
// those peer pointers over NVLink (no TMA from peer memory).
//
//   reduce_norm      consumer half of the fused row-parallel linear: waits for the
//                    partial tiles every rank's GEMM epilogue pushed into the local
//                    slots, sums them, adds the (gated) residual and applies
//                    RMSNorm / Gemma RMSNorm / AdaRMSNorm in the same pass
//   push_partial     stand-alone producer (used when the GEMM ran unfused, and by tests)
//   cfg_exchange     CFG-parallel combine: each branch writes its velocity into the
//                    partner's buffer, waits for the partner's, applies
//                    uncond + g (cond - uncond) and optionally the Euler update
//   gather_consume   consumer half of the row all-gather (shards are pushed, like partials)
//   flag_wait_probe  a bounded wait on a flag nobody sets (failure-detection tests)
//
// The reference has no peer-memory code path; its nearest primitive is the unused
// CudaIpcBuffer (phyai/src/phyai/runtime/ipc_buffer.py:252-556) and its collectives are
// NCCL calls (phyai/src/phyai/layers/linear/layers.py:628-630,
// phyai/src/phyai/models/cosmos3/scheduler_wn_cosmos3.py:227-228).
#include "comm.cuh"

#include <ATen/cuda/CUDAContext.h>
#include <torch/extension.h>

#include <cstdlib>
#include <cstring>
#include <string>

#include "comm_device.cuh"
#include "gemm.cuh"
#include "launch.cuh"

#define PB_LAUNCH(kern, grid, block, stream, ...) \
  throw_on(pb::launch_kernel(kern, dim3(grid), dim3(block), 0, stream, 1, __VA_ARGS__), #kern)

namespace py = pybind11;

namespace pb {

// ------------------------------------------------------------------ kernels
__global__ void reduce_norm_kernel(ReduceNormArgs a, ChannelSig* local_sig, int channel,
                                   unsigned int expect_per_call, PeerPtrs sig_peers, int* status) {
  __shared__ float red[32];
  __shared__ int ok_s;
  ChannelSig* sig = local_sig + channel;
  pdl_launch_dependents();
  pdl_wait();
  const unsigned int e = ld_relaxed_sys(&sig->epoch);
  const int parity = int(e & 1u);
  if (threadIdx.x == 0) {
    const bool ok = wait_counter_ge(&sig->arrive[parity], expect_per_call);
    ok_s = ok ? 1 : 0;
    if (!ok && status) atomicCAS(status, 0, kStatusTimeoutPeer);
  }
  __syncthreads();
  if (ok_s) {
    ReduceNormArgs b = a;
    b.slots = a.slots + size_t(parity) * a.world * a.slot_stride;
    for (int row = a.row0 + blockIdx.x; row < a.row0 + a.nrows; row += gridDim.x) {
      reduce_norm_row(b, row, red);
      __syncthreads();
    }
  }
  if (a.y_world > 0) {
    // the gathered rows of this CTA are on their way: one arrival per CTA on every rank
    __syncthreads();
    if (threadIdx.x == 0) {
      const unsigned int ye = ld_relaxed_sys(&(local_sig + a.y_channel)->epoch);
      channel_signal_all(sig_peers, a.y_channel, int(ye & 1u), a.y_world);
    }
  }
  channel_finish(sig, parity, gridDim.x);
}

// Copies this rank's partial [M, N] (row stride ldx) into slots[parity][rank] of every peer.
__global__ void push_partial_kernel(const __nv_bfloat16* x, int M, int N, int ldx, PeerPtrs data,
                                    long long slots_off, long long slot_stride, int ld, int world,
                                    int rank, PeerPtrs sig, ChannelSig* local_sig, int channel) {
  pdl_launch_dependents();
  pdl_wait();
  const unsigned int e = ld_relaxed_sys(&(local_sig + channel)->epoch);
  const int parity = int(e & 1u);
  const int nv = N >> 3;
  const long long total = (long long)M * nv;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int row = int(i / nv), v = int(i % nv);
    const uint4 val = *reinterpret_cast<const uint4*>(x + size_t(row) * ldx + v * 8);
    for (int r = 0; r < world; ++r) {
      __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(data.p[r]) + slots_off +
                           (size_t(parity) * world + rank) * slot_stride + size_t(row) * ld + v * 8;
      *reinterpret_cast<uint4*>(dst) = val;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) channel_signal_all(sig, channel, parity, world);
}

// CFG pair exchange. `mine` is this branch's prediction (n bf16). Both ranks of the pair
// end with the combined velocity; x (fp32, optional) receives the Euler step.
__global__ void cfg_exchange_kernel(const __nv_bfloat16* mine, long long n, PeerPtrs data,
                                    long long buf_off, int my_pos, int partner_pos, int is_cond,
                                    float g, __nv_bfloat16* out, float* x, float dt, PeerPtrs sig,
                                    ChannelSig* local_sig, int channel, int* status) {
  __shared__ int ok_s;
  ChannelSig* ls = local_sig + channel;
  pdl_launch_dependents();
  pdl_wait();
  const unsigned int e = ld_relaxed_sys(&ls->epoch);
  const int parity = int(e & 1u);
  const long long nv = n >> 3;
  // push my prediction into the partner's inbox for this parity
  __nv_bfloat16* inbox_remote =
      reinterpret_cast<__nv_bfloat16*>(data.p[partner_pos]) + buf_off + size_t(parity) * n;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nv;
       i += (long long)gridDim.x * blockDim.x)
    reinterpret_cast<uint4*>(inbox_remote)[i] = reinterpret_cast<const uint4*>(mine)[i];
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    ChannelSig* ps = reinterpret_cast<ChannelSig*>(sig.p[partner_pos]) + channel;
    red_release_sys_add(&ps->arrive[parity], 1u);
    const bool ok = wait_counter_ge(&ls->arrive[parity], gridDim.x);
    ok_s = ok ? 1 : 0;
    if (!ok && status) atomicCAS(status, 0, kStatusTimeoutPeer);
  }
  __syncthreads();
  if (ok_s) {
    const __nv_bfloat16* theirs =
        reinterpret_cast<const __nv_bfloat16*>(data.p[my_pos]) + buf_off + size_t(parity) * n;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nv;
         i += (long long)gridDim.x * blockDim.x) {
      const uint4 a = reinterpret_cast<const uint4*>(mine)[i];
      const uint4 b = reinterpret_cast<const uint4*>(theirs)[i];
      const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&a);
      const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&b);
      uint4 o;
      __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float m0 = bf2f(a2[k].x), m1 = bf2f(a2[k].y);
        const float t0 = bf2f(b2[k].x), t1 = bf2f(b2[k].y);
        const float c0 = is_cond ? m0 : t0, c1 = is_cond ? m1 : t1;
        const float u0 = is_cond ? t0 : m0, u1 = is_cond ? t1 : m1;
        const float v0 = u0 + g * (c0 - u0), v1 = u1 + g * (c1 - u1);
        o2[k] = __floats2bfloat162_rn(v0, v1);
        if (x) {
          x[i * 8 + 2 * k] += dt * v0;
          x[i * 8 + 2 * k + 1] += dt * v1;
        }
      }
      if (out) reinterpret_cast<uint4*>(out)[i] = o;
    }
  }
  channel_finish(ls, parity, gridDim.x);
}

// Consumer half of the row all-gather: every rank pushed its shard into
// slots[parity][rank] of every peer (push_partial); wait for all of them, then copy the
// gathered [world * rows, N] matrix out of the slots into `out` (local to local).
__global__ void gather_consume_kernel(const __nv_bfloat16* slots, long long slot_stride, int rows,
                                      int N, int ld, int world, __nv_bfloat16* out, int ldo,
                                      ChannelSig* local_sig, int channel, unsigned int expect,
                                      int* status) {
  __shared__ int ok_s;
  ChannelSig* ls = local_sig + channel;
  pdl_launch_dependents();
  pdl_wait();
  const unsigned int e = ld_relaxed_sys(&ls->epoch);
  const int parity = int(e & 1u);
  if (threadIdx.x == 0) {
    const bool ok = wait_counter_ge(&ls->arrive[parity], expect);
    ok_s = ok ? 1 : 0;
    if (!ok && status) atomicCAS(status, 0, kStatusTimeoutPeer);
  }
  __syncthreads();
  if (ok_s) {
    const int nv = N >> 3;
    const long long total = (long long)world * rows * nv;
    const __nv_bfloat16* base = slots + size_t(parity) * world * slot_stride;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
      const int v = int(i % nv);
      const long long rr = i / nv;
      const int row = int(rr % rows), r = int(rr / rows);
      if (out)
        *reinterpret_cast<uint4*>(out + (size_t(r) * rows + row) * ldo + v * 8) =
            *reinterpret_cast<const uint4*>(base + size_t(r) * slot_stride + size_t(row) * ld + v * 8);
    }
  }
  channel_finish(ls, parity, gridDim.x);
}

__global__ void flag_wait_probe_kernel(const unsigned int* flag, unsigned int want,
                                       unsigned long long timeout_ns, int* status) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    if (!wait_counter_ge(flag, want, timeout_ns) && status) atomicCAS(status, 0, kStatusTimeoutPeer);
  }
}

}  // namespace pb

// ------------------------------------------------------------------ bindings
namespace {

using at::Tensor;
using OptT = c10::optional<Tensor>;

void throw_on(cudaError_t e, const char* what) {
  if (e != cudaSuccess) {
    cudaGetLastError();
    throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
  }
}
inline cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }
inline const __nv_bfloat16* bfp(const OptT& t) {
  if (!t.has_value() || !t->defined()) return nullptr;
  TORCH_CHECK(t->is_cuda() && t->scalar_type() == at::kBFloat16, "expected a CUDA bf16 tensor");
  return reinterpret_cast<const __nv_bfloat16*>(t->data_ptr());
}

// (uint8 tensor over a fresh cudaMalloc slab, 64-byte IPC handle). The slab is zeroed.
py::tuple ipc_alloc(int64_t bytes) {
  void* p = nullptr;
  throw_on(cudaMalloc(&p, size_t(bytes)), "cudaMalloc");
  throw_on(cudaMemset(p, 0, size_t(bytes)), "cudaMemset");
  throw_on(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
  cudaIpcMemHandle_t h;
  throw_on(cudaIpcGetMemHandle(&h, p), "cudaIpcGetMemHandle");
  int dev = 0;
  cudaGetDevice(&dev);
  Tensor t = at::from_blob(p, {bytes}, at::TensorOptions().dtype(at::kByte).device(at::kCUDA, dev));
  return py::make_tuple(t, py::bytes(reinterpret_cast<const char*>(&h), sizeof(h)),
                        reinterpret_cast<uintptr_t>(p));
}
uintptr_t ipc_open(const py::bytes& handle) {
  std::string s = handle;
  if (s.size() != sizeof(cudaIpcMemHandle_t)) throw std::runtime_error("bad IPC handle size");
  cudaIpcMemHandle_t h;
  memcpy(&h, s.data(), sizeof(h));
  void* p = nullptr;
  throw_on(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle");
  return reinterpret_cast<uintptr_t>(p);
}
void ipc_close(uintptr_t p) { throw_on(cudaIpcCloseMemHandle(reinterpret_cast<void*>(p)), "cudaIpcCloseMemHandle"); }
void ipc_free(uintptr_t p) { throw_on(cudaFree(reinterpret_cast<void*>(p)), "cudaFree"); }

pb::PeerPtrs to_ptrs(const std::vector<uintptr_t>& v, int64_t byte_off = 0) {
  pb::PeerPtrs p;
  TORCH_CHECK(v.size() <= pb::kMaxRanks, "at most ", pb::kMaxRanks, " ranks per peer group");
  for (int i = 0; i < pb::kMaxRanks; ++i)
    p.p[i] = i < int(v.size()) ? reinterpret_cast<void*>(v[i] + byte_off) : nullptr;
  return p;
}

// Sums the world partials pushed for this channel, adds residual (* gate), norms.
// With rows_per_rank > 0 only this rank's rows are reduced (the producer scattered them) and
// residual / h_out / y are indexed by global row. With y_gather_off >= 0 the normalised rows
// go to that element offset of every rank's slab and y_channel is signalled; the return
// value is then the number of arrivals a consumer of the gathered matrix waits for.
static pb::ReduceNormArgs make_reduce_args(const std::vector<uintptr_t>& data_ptrs, int64_t rank, int64_t slots_off_elems,
                                           int64_t slot_stride, int64_t M, int64_t N, int64_t ld, const OptT& residual,
                                           const OptT& col_gate, const OptT& bias, const OptT& h_out, const OptT& y,
                                           int64_t norm_mode, const OptT& weight, const OptT& mod, double eps,
                                           int64_t rows_per_rank, int64_t y_gather_off, int64_t y_ld, int64_t y_channel) {
  pb::ReduceNormArgs a;
  const int world = int(data_ptrs.size());
  a.slots = reinterpret_cast<const __nv_bfloat16*>(data_ptrs[rank]) + slots_off_elems;
  a.slot_stride = slot_stride; a.world = world; a.M = int(M); a.N = int(N); a.ld = int(ld);
  TORCH_CHECK(N % 8 == 0 && ld % 8 == 0, "reduce_norm: N and ld must be multiples of 8");
  a.residual = nullptr; a.ldr = 0;
  if (residual.has_value() && residual->defined()) {
    a.residual = const_cast<__nv_bfloat16*>(bfp(residual)); a.ldr = int(residual->stride(0));
  }
  a.col_gate = bfp(col_gate); a.bias = bfp(bias);
  a.h_out = nullptr; a.ldh = 0;
  if (h_out.has_value() && h_out->defined()) { a.h_out = const_cast<__nv_bfloat16*>(bfp(h_out)); a.ldh = int(h_out->stride(0)); }
  a.y = nullptr; a.ldy = 0;
  if (y.has_value() && y->defined()) { a.y = const_cast<__nv_bfloat16*>(bfp(y)); a.ldy = int(y->stride(0)); }
  a.norm_mode = int(norm_mode); a.weight = bfp(weight); a.mod = bfp(mod); a.eps = float(eps);
  a.row0 = 0; a.nrows = int(M); a.slot_row0 = 0;
  if (rows_per_rank > 0) {
    a.row0 = int(rank * rows_per_rank);
    a.slot_row0 = a.row0;
    a.nrows = int(std::max<int64_t>(0, std::min<int64_t>(rows_per_rank, M - a.row0)));
  }
  a.y_world = 0; a.y_off = 0; a.y_channel = 0;
  a.y_dst = to_ptrs(data_ptrs);
  if (y_gather_off >= 0) {
    TORCH_CHECK(y_ld % 8 == 0 && y_gather_off % 8 == 0, "reduce_norm: gathered rows must be 16-byte aligned");
    a.y_world = world; a.y_off = y_gather_off; a.ldy = int(y_ld); a.y_channel = int(y_channel);
  }
  return a;
}

static int64_t launch_reduce(const pb::ReduceNormArgs& a, const std::vector<uintptr_t>& data_ptrs, int64_t rank,
                             int64_t sig_off_bytes, int64_t channel, int64_t expect, int64_t max_ctas) {
  auto* sig = reinterpret_cast<pb::ChannelSig*>(data_ptrs[rank] + sig_off_bytes);
  int threads = int(((a.N / 8) + 31) / 32 * 32);
  threads = threads > 512 ? 512 : (threads < 64 ? 64 : threads);
  int grid = int(a.nrows < max_ctas ? a.nrows : max_ctas);
  if (grid < 1) grid = 1;
  PB_LAUNCH(pb::reduce_norm_kernel, grid, threads, cur_stream(), a, sig, int(channel), unsigned(expect),
            to_ptrs(data_ptrs, sig_off_bytes), pb::kernel_status_ptr());
  throw_on(cudaGetLastError(), "reduce_norm_kernel");
  return int64_t(grid) * int64_t(data_ptrs.size());
}

int64_t reduce_norm(const std::vector<uintptr_t>& data_ptrs, int64_t rank, int64_t slots_off_elems,
                 int64_t slot_stride, int64_t M, int64_t N, int64_t ld, int64_t sig_off_bytes,
                 int64_t channel, int64_t expect, const OptT& residual, const OptT& col_gate,
                 const OptT& bias, const OptT& h_out, const OptT& y, int64_t norm_mode,
                 const OptT& weight, const OptT& mod, double eps, int64_t max_ctas,
                 int64_t rows_per_rank, int64_t y_gather_off, int64_t y_ld, int64_t y_channel) {
  const pb::ReduceNormArgs a = make_reduce_args(data_ptrs, rank, slots_off_elems, slot_stride, M, N, ld, residual, col_gate,
                                                bias, h_out, y, norm_mode, weight, mod, eps, rows_per_rank, y_gather_off,
                                                y_ld, y_channel);
  return launch_reduce(a, data_ptrs, rank, sig_off_bytes, channel, expect, max_ctas);
}

int64_t push_partial(const Tensor& x, const std::vector<uintptr_t>& data_ptrs, int64_t rank,
                     int64_t slots_off_elems, int64_t slot_stride, int64_t ld, int64_t sig_off_bytes,
                     int64_t channel) {
  TORCH_CHECK(x.dim() == 2 && x.stride(1) == 1 && x.size(1) % 8 == 0, "push_partial: layout");
  const int world = int(data_ptrs.size());
  const long long total = x.size(0) * (x.size(1) / 8);
  int grid = int((total + 255) / 256);
  grid = grid > 64 ? 64 : (grid < 1 ? 1 : grid);
  auto* sig = reinterpret_cast<pb::ChannelSig*>(data_ptrs[rank] + sig_off_bytes);
  PB_LAUNCH(pb::push_partial_kernel, grid, 256, cur_stream(), 
      bfp(OptT(x)), int(x.size(0)), int(x.size(1)), int(x.stride(0)), to_ptrs(data_ptrs), slots_off_elems,
      slot_stride, int(ld), world, int(rank), to_ptrs(data_ptrs, sig_off_bytes), sig, int(channel));
  throw_on(cudaGetLastError(), "push_partial_kernel");
  return int64_t(grid) * world;  // arrivals each rank will see per call
}

// Row-parallel product pushed straight from the GEMM epilogue into every rank's slots.
// Returns the number of arrivals each rank's consumer must wait for on this call.
int64_t gemm_push(const Tensor& x, const Tensor& w, const std::vector<uintptr_t>& data_ptrs, int64_t rank,
                  int64_t slots_off_elems, int64_t slot_stride, int64_t ld, int64_t sig_off_bytes,
                  int64_t channel, int64_t rows_per_rank, int64_t force_bn, int64_t force_swap,
                  int64_t force_splits) {
  TORCH_CHECK(x.dim() == 2 && w.dim() == 2 && x.stride(1) == 1 && w.stride(1) == 1, "gemm_push: layout");
  TORCH_CHECK(x.scalar_type() == at::kBFloat16 && w.scalar_type() == at::kBFloat16, "gemm_push: bf16 operands");
  TORCH_CHECK(x.size(1) == w.size(1), "gemm_push: K mismatch");
  pb::PushParams pp;
  memset(&pp, 0, sizeof(pp));
  pp.data = to_ptrs(data_ptrs);
  pp.sig = to_ptrs(data_ptrs, sig_off_bytes);
  pp.local_sig = reinterpret_cast<const void*>(data_ptrs[rank] + sig_off_bytes);
  pp.slots_off = slots_off_elems; pp.slot_stride = slot_stride; pp.ld = int(ld);
  pp.world = int(data_ptrs.size()); pp.rank = int(rank); pp.channel = int(channel);
  pp.rows_per_rank = int(rows_per_rank); pp.wait_channel = -1; pp.wait_expect = 0;
  pb::GemmArgs a;
  a.x = x.data_ptr(); a.w = w.data_ptr(); a.out = nullptr;
  a.M = int(x.size(0)); a.N = int(w.size(0)); a.K = int(x.size(1));
  a.ldx = int(x.stride(0)); a.ldw = int(w.stride(0)); a.ldo = int(ld);
  TORCH_CHECK((rows_per_rank > 0 ? rows_per_rank : int64_t(a.M)) * ld <= slot_stride && a.N <= ld,
              "gemm_push: product does not fit a slot");
  TORCH_CHECK(rows_per_rank == 0 || rows_per_rank * pp.world >= a.M, "gemm_push: rows_per_rank too small");
  a.force_bn = int(force_bn); a.force_swap = int(force_swap); a.force_splits = int(force_splits);
  a.push = &pp;
  int ctas = 0;
  throw_on(pb::gemm_launch(a, cur_stream(), &ctas), "gemm_launch (push)");
  return int64_t(ctas) * pp.world;
}

// Row-parallel linear + all-reduce + residual (* gate) + norm over the peer group. On few rows the GEMM's own CTAs
// do the consumer half after their arrival (one launch); otherwise the product is pushed and the reduce kernel
// follows. Returns 1 when it was a single launch.
int64_t linear_reduce(const Tensor& x, const Tensor& w, const std::vector<uintptr_t>& data_ptrs, int64_t rank,
                      int64_t slots_off_elems, int64_t slot_stride, int64_t ld, int64_t sig_off_bytes, int64_t channel,
                      const OptT& residual, const OptT& col_gate, const OptT& bias, const OptT& h_out, const OptT& y,
                      int64_t norm_mode, const OptT& weight, const OptT& mod, double eps, int64_t max_ctas, bool allow_tail) {
  TORCH_CHECK(x.dim() == 2 && w.dim() == 2 && x.stride(1) == 1 && w.stride(1) == 1, "linear_reduce: layout");
  TORCH_CHECK(x.scalar_type() == at::kBFloat16 && w.scalar_type() == at::kBFloat16, "linear_reduce: bf16 operands");
  TORCH_CHECK(x.size(1) == w.size(1), "linear_reduce: K mismatch");
  const int64_t M = x.size(0), N = w.size(0);
  pb::PushParams pp;
  memset(&pp, 0, sizeof(pp));
  pp.data = to_ptrs(data_ptrs);
  pp.sig = to_ptrs(data_ptrs, sig_off_bytes);
  pp.local_sig = reinterpret_cast<const void*>(data_ptrs[rank] + sig_off_bytes);
  pp.slots_off = slots_off_elems; pp.slot_stride = slot_stride; pp.ld = int(ld);
  pp.world = int(data_ptrs.size()); pp.rank = int(rank); pp.channel = int(channel);
  pp.rows_per_rank = 0; pp.wait_channel = -1; pp.wait_expect = 0;
  pp.red = make_reduce_args(data_ptrs, rank, slots_off_elems, slot_stride, M, N, ld, residual, col_gate, bias, h_out, y,
                            norm_mode, weight, mod, eps, 0, -1, 0, 0);
  static const bool tail_env = [] { const char* e = getenv("PHYAI_COMM_FUSED_TAIL"); return !e || atoi(e) != 0; }();
  pp.tail = (allow_tail && tail_env && M <= 256) ? 1 : 0;
  pb::GemmArgs a;
  a.x = x.data_ptr(); a.w = w.data_ptr(); a.out = nullptr;
  a.M = int(M); a.N = int(N); a.K = int(x.size(1));
  a.ldx = int(x.stride(0)); a.ldw = int(w.stride(0)); a.ldo = int(ld);
  TORCH_CHECK(M * ld <= slot_stride && N <= ld, "linear_reduce: product does not fit a slot");
  a.push = &pp;
  int ctas = 0, tail_done = 0;
  a.tail_done = &tail_done;
  throw_on(pb::gemm_launch(a, cur_stream(), &ctas), "gemm_launch (linear_reduce)");
  if (tail_done) return 1;
  launch_reduce(pp.red, data_ptrs, rank, sig_off_bytes, channel, int64_t(ctas) * pp.world, max_ctas);
  return 0;
}

void cfg_exchange(const Tensor& mine, const std::vector<uintptr_t>& data_ptrs, int64_t my_pos,
                  int64_t partner_pos, int64_t buf_off_elems, bool is_cond, double g, const OptT& out,
                  const OptT& x_fp32, double dt, int64_t sig_off_bytes, int64_t channel) {
  TORCH_CHECK(mine.is_contiguous() && mine.numel() % 8 == 0, "cfg_exchange: numel must be a multiple of 8");
  const long long n = mine.numel();
  int grid = int((n / 8 + 255) / 256);
  grid = grid > 128 ? 128 : (grid < 1 ? 1 : grid);  // all CTAs must be co-resident: they wait on the partner
  auto* sig = reinterpret_cast<pb::ChannelSig*>(data_ptrs[my_pos] + sig_off_bytes);
  float* xp = nullptr;
  if (x_fp32.has_value() && x_fp32->defined()) {
    TORCH_CHECK(x_fp32->scalar_type() == at::kFloat && x_fp32->numel() == n, "cfg_exchange: x_fp32");
    xp = reinterpret_cast<float*>(x_fp32->data_ptr());
  }
  __nv_bfloat16* op = (out.has_value() && out->defined()) ? const_cast<__nv_bfloat16*>(bfp(out)) : nullptr;
  PB_LAUNCH(pb::cfg_exchange_kernel, grid, 256, cur_stream(), 
      bfp(OptT(mine)), n, to_ptrs(data_ptrs), buf_off_elems, int(my_pos), int(partner_pos), is_cond ? 1 : 0,
      float(g), op, xp, float(dt), to_ptrs(data_ptrs, sig_off_bytes), sig, int(channel), pb::kernel_status_ptr());
  throw_on(cudaGetLastError(), "cfg_exchange_kernel");
}

void gather_consume(const std::vector<uintptr_t>& data_ptrs, int64_t rank, int64_t slots_off_elems,
                    int64_t slot_stride, int64_t rows, int64_t N, int64_t ld, const OptT& out,
                    int64_t sig_off_bytes, int64_t channel, int64_t expect) {
  const bool copy = out.has_value() && out->defined();
  TORCH_CHECK(N % 8 == 0 && (!copy || (out->dim() == 2 && out->stride(1) == 1)), "gather_consume: layout");
  const int world = int(data_ptrs.size());
  const long long total = (long long)world * rows * (N / 8);
  int grid = int((total + 255) / 256);
  grid = grid > 128 ? 128 : (grid < 1 ? 1 : grid);
  if (!copy) grid = 1;  // wait only: the gathered rows are read in place by the next kernel
  auto* sig = reinterpret_cast<pb::ChannelSig*>(data_ptrs[rank] + sig_off_bytes);
  PB_LAUNCH(pb::gather_consume_kernel, grid, 256, cur_stream(), 
      reinterpret_cast<const __nv_bfloat16*>(data_ptrs[rank]) + slots_off_elems, slot_stride, int(rows), int(N),
      int(ld), world, copy ? const_cast<__nv_bfloat16*>(bfp(out)) : nullptr, copy ? int(out->stride(0)) : 0, sig, int(channel),
      unsigned(expect), pb::kernel_status_ptr());
  throw_on(cudaGetLastError(), "gather_consume_kernel");
}

void flag_wait_probe(const Tensor& flag, int64_t want, double timeout_s) {
  TORCH_CHECK(flag.is_cuda() && flag.scalar_type() == at::kInt, "flag_wait_probe: int32 CUDA tensor");
  PB_LAUNCH(pb::flag_wait_probe_kernel, 1, 32, cur_stream(), 
      reinterpret_cast<const unsigned int*>(flag.data_ptr()), unsigned(want),
      (unsigned long long)(timeout_s * 1e9), pb::kernel_status_ptr());
  throw_on(cudaGetLastError(), "flag_wait_probe_kernel");
}

}  // namespace

void register_comm(py::module_& m) {
  m.def("ipc_alloc", &ipc_alloc);
  m.def("ipc_open", &ipc_open);
  m.def("ipc_close", &ipc_close);
  m.def("ipc_free", &ipc_free);
  m.def("reduce_norm", &reduce_norm);
  m.def("push_partial", &push_partial);
  m.def("gemm_push", &gemm_push);
  m.def("linear_reduce", &linear_reduce);
  m.def("cfg_exchange", &cfg_exchange);
  m.def("gather_consume", &gather_consume);
  m.def("flag_wait_probe", &flag_wait_probe);
  m.attr("CHANNEL_SIG_BYTES") = int(sizeof(pb::ChannelSig));
}

// Device-side pieces of the peer-memory protocol shared by comm.cu and gemm.cu.
//
// A "channel" is one call site of a fused collective (e.g. the o-proj of layer 7).
// Every rank keeps the channel's signal words in its own symmetric memory:
//
//   arrive[2]  how many producer CTAs (over all ranks) have finished pushing into
//              this rank's slots for the call of parity 0 / 1
//   epoch      number of completed calls on this channel (parity = epoch & 1)
//   done       ticket counter used to find the last consumer CTA of a call
//
// Call e (parity p): producers on every rank store their partial tiles into
// slots[p][src_rank] of EVERY rank (plain st.global to peer pointers), fence at
// system scope and add 1 to the destination's arrive[p] (red.release.sys). Consumers
// spin (bounded) on their local arrive[p] until it equals producers x ranks, then read
// only local memory. The last consumer CTA zeroes arrive[p] and bumps epoch. Slots and
// counters of parity p are reused by call e+2; a peer can reach call e+2 only after it
// consumed this rank's pushes of call e+1, which this rank issues after finishing call
// e, so double buffering is enough and no trailing barrier is needed.
//
// Every wait is bounded (about one second); on expiry the kernel records
// kStatusTimeoutPeer and returns normally, so a missing peer never hangs the GPU.
#pragma once
#include "comm.cuh"
#include "ptx.cuh"

namespace pb {

struct ChannelSig {
  unsigned int arrive[2];
  unsigned int epoch;
  unsigned int done;
  unsigned int pad[4];
};

__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned int ld_relaxed_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_sys_add(unsigned int* p, unsigned int v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Spin until *p >= want (acquire, system scope). False after ~timeout_ns.
__device__ __forceinline__ bool wait_counter_ge(const unsigned int* p, unsigned int want,
                                                uint64_t timeout_ns = 1000000000ull) {
  if (ld_acquire_sys(p) >= want) return true;
  const uint64_t t0 = globaltimer_ns();
  unsigned int spins = 0;
  while (ld_acquire_sys(p) < want) {
    if ((++spins & 0xff) == 0) {
      if (globaltimer_ns() - t0 > timeout_ns) return false;
      __nanosleep(64);
    }
  }
  return true;
}

// Called by one thread of a producer CTA after the CTA's pushes are complete
// (the caller has executed __syncthreads() after the last store).
__device__ __forceinline__ void channel_signal_all(const PeerPtrs& sig, int channel, int parity,
                                                   int world) {
  __threadfence_system();
  for (int r = 0; r < world; ++r) {
    ChannelSig* s = reinterpret_cast<ChannelSig*>(sig.p[r]) + channel;
    red_release_sys_add(&s->arrive[parity], 1u);
  }
}


// One CTA reduces row `row`: h = residual + (sum_r slot_r + bias) * gate, y = norm(h).
// `red` is 32 floats of shared memory. N must be a multiple of 8.
__device__ __forceinline__ void reduce_norm_row(const ReduceNormArgs& a, int row, float* red) {
  const int nv = a.N >> 3;
  float ss = 0.f;
  __nv_bfloat16* hrow = a.residual ? a.residual + size_t(row) * a.ldr
                                   : (a.h_out ? a.h_out + size_t(row) * a.ldh : nullptr);
  for (int v = threadIdx.x; v < nv; v += blockDim.x) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int r = 0; r < a.world; ++r) {
      const uint4 raw = *reinterpret_cast<const uint4*>(a.slots + size_t(r) * a.slot_stride +
                                                        size_t(row - a.slot_row0) * a.ld + v * 8);
      const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        acc[2 * i] += bf2f(b2[i].x);
        acc[2 * i + 1] += bf2f(b2[i].y);
      }
    }
    if (a.bias) {
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += bf2f(a.bias[v * 8 + i]);
    }
    if (a.col_gate) {
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] *= bf2f(a.col_gate[v * 8 + i]);
    }
    if (a.residual) {
      const uint4 raw = *reinterpret_cast<const uint4*>(a.residual + size_t(row) * a.ldr + v * 8);
      const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        acc[2 * i] += bf2f(b2[i].x);
        acc[2 * i + 1] += bf2f(b2[i].y);
      }
    }
    uint4 out;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      o2[i] = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
      const float x0 = bf2f(o2[i].x), x1 = bf2f(o2[i].y);
      ss += x0 * x0 + x1 * x1;
    }
    if (hrow) *reinterpret_cast<uint4*>(hrow + v * 8) = out;
  }
  if ((a.y == nullptr && a.y_world == 0) || hrow == nullptr) return;
  // block-wide sum of squares
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  __syncthreads();
  if (lane == 0) red[warp] = ss;
  __syncthreads();
  const int nw = (blockDim.x + 31) >> 5;
  float t = lane < nw ? red[lane] : 0.f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  const float rstd = a.norm_mode < 0 ? 1.f : rsqrtf(t / a.N + a.eps);
  __syncthreads();  // h row written by this CTA is re-read below
  for (int v = threadIdx.x; v < nv; v += blockDim.x) {
    const uint4 raw = *reinterpret_cast<const uint4*>(hrow + v * 8);
    const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
    uint4 out;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float x0 = bf2f(b2[i].x) * rstd, x1 = bf2f(b2[i].y) * rstd;
      const int c = v * 8 + 2 * i;
      if (a.norm_mode == 3) {  // AdaRMS: (1 + scale) and shift from the modulation row
        x0 = x0 * (1.f + bf2f(a.mod[c])) + bf2f(a.mod[a.N + c]);
        x1 = x1 * (1.f + bf2f(a.mod[c + 1])) + bf2f(a.mod[a.N + c + 1]);
      } else if (a.norm_mode == 1) {  // Gemma (1 + w)
        x0 *= 1.f + bf2f(a.weight[c]);
        x1 *= 1.f + bf2f(a.weight[c + 1]);
      } else if (a.norm_mode == 0) {
        x0 *= bf2f(a.weight[c]);
        x1 *= bf2f(a.weight[c + 1]);
      }
      o2[i] = __floats2bfloat162_rn(x0, x1);
    }
    if (a.y_world > 0) {
      const size_t off = size_t(a.y_off) + size_t(row) * a.ldy + v * 8;
      for (int r = 0; r < a.y_world; ++r)
        *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(a.y_dst.p[r]) + off) = out;
    } else {
      *reinterpret_cast<uint4*>(a.y + size_t(row) * a.ldy + v * 8) = out;
    }
  }
}

// End-of-call bookkeeping by the consumers of a channel: the last CTA to get here
// clears the parity's arrival counter and publishes the next epoch.
__device__ __forceinline__ void channel_finish(ChannelSig* local, int parity, unsigned int n_ctas) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned int t = atomicAdd(&local->done, 1u);
    if (t == n_ctas - 1) {
      local->arrive[parity] = 0;
      local->done = 0;
      __threadfence_system();
      st_release_sys(&local->epoch, ld_relaxed_sys(&local->epoch) + 1u);
    }
  }
}

}  // namespace pb

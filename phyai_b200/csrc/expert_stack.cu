// Persistent action-expert kernel for sm_100a: every Euler step of the flow-matching expert
// (input projection, n_layers Gemma blocks, final norm + output projection + state update) in
// ONE cooperative launch, one CTA per SM.
//
// The expert works on a few dozen action rows, so a block's five GEMMs and its attention are
// dependency-bound, not bandwidth-bound: as separate launches they cost ~10 us each while their
// weights stream in ~1 us. Here the launch boundaries become grid barriers and the weights never
// wait for them:
//
//   * warp 0 (producer) walks the static (step, layer, projection, tile) schedule of its CTA and
//     streams 128 x 64 weight tiles by TMA into a 7-slot shared-memory ring, running ahead of the
//     compute across phases and barriers, bounded only by free slots;
//   * warp 1 (one thread) issues tcgen05.mma: weight tile = 128-row A operand, the (<= 64) action
//     rows = N, accumulators in tensor memory;
//   * warps 2-9 (workers) build the activation operand of each phase in shared memory straight
//     from the fp32 results of the previous phase ("epilogue on load": AdaRMS scale, row 1/rms,
//     bias, rotary embedding, GeGLU all happen here), drain the accumulators with fp32 reductions
//     into L2-resident buffers (split-K over CTAs needs no second pass; the residual add is the
//     reduction itself), and run the grid barrier.
//
// Work split: every projection is cut into (128-row weight tile, 64-wide K block) pairs, n-major,
// and CTA c takes pairs [c T / G, (c + 1) T / G): all SMs stream weights in every phase. The
// attention phase runs (head, KV split) units: S = Q K^T and O = P V on the tensor cores for up
// to 64 keys, partial (max, sum, O) to L2, merged by the next phase.
//
// Every wait is bounded (about one second): a wait that runs out raises a grid-wide abort bit in
// the barrier word, every role drains, tensor memory is freed, the status word says why.
//
// Replaces the per-block launch sequence of the reference's action-expert loop
// (phyai/src/phyai/models/pi05/model_runner_pi05.py:689-738, modeling_pi05.py:801-835).
#include "expert_stack.cuh"

#include <cstring>

#include "gemm.cuh"
#include "ptx.cuh"

namespace pb {

namespace {

constexpr int kThreads = 320;          // warp 0 producer, warp 1 MMA, warps 2..9 workers
constexpr int kWorkers = 256;
constexpr int kRing = 7;               // weight tiles in flight per CTA
constexpr int kSlotBytes = 128 * 128;  // 128 weight rows x 64 bf16
constexpr int kActBlk = 64 * 128;      // 64 action rows x 64 bf16
constexpr int kMaxPairs = 8;
constexpr int kRegionA = 104 * 1024;   // activation blocks (8 x 8 KB) or attention tiles (P 8 | Q 32 | K 32 | V 32)
constexpr int kSmemBytes = 1024 + kRing * kSlotBytes + kRegionA;
constexpr uint32_t kAbortBit = 0x80000000u;
constexpr int kTmemCols = 512;
constexpr int kSCol = 192, kOCol = 256;   // accumulators of the projections at [0, 192), S at [192, 256), O at [256, 512)
constexpr int kRows = 64;              // padded action rows
constexpr int kD = 256;                // head dim
constexpr int kKeys = 64;              // keys per attention unit

__device__ __forceinline__ unsigned ld_relaxed_gpu(const unsigned* p) {
  unsigned v;
  asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_gpu_add(unsigned* p, unsigned v) {
  asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void worker_sync() { asm volatile("bar.sync 1, 256;" ::: "memory"); }
__device__ __forceinline__ void cp16(uint32_t dst, const void* src, bool valid) {
  const int sz = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(sz) : "memory");
}
__device__ __forceinline__ void st_shared_v2(uint32_t dst, uint32_t a, uint32_t b) {
  asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(dst), "r"(a), "r"(b) : "memory");
}
__device__ __forceinline__ void st_shared_v4(uint32_t dst, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ void red_add_v4(float* dst, float4 v) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&v);
}
__device__ __forceinline__ float round_bf16(float x) { return bf2f(__float2bfloat16(x)); }

// Byte offset of element (row r, column c) in a K-major tile stored as 64-column blocks of
// [64 rows x 128 B] with the 128-byte swizzle (c a multiple of 4: the 8-byte group that holds it).
__device__ __forceinline__ uint32_t sw64(int r, int c) {
  return uint32_t(c >> 6) * uint32_t(kActBlk) + uint32_t(r) * 128u + uint32_t((((c & 63) >> 3) ^ (r & 7)) << 4) +
         uint32_t(c & 7) * 2u;
}

// Bounded mbarrier wait that also gives up when the CTA is aborting.
__device__ __forceinline__ bool es_wait(uint64_t* bar, uint32_t parity, volatile int* abort_s) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = globaltimer_ns();
  uint32_t spins = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++spins & 0xff) == 0) {
      if (*abort_s) return false;
      if (globaltimer_ns() - t0 > 1000000000ull) return false;
    }
  }
  return true;
}

struct Geo { int n_tiles, kbs; };
__device__ __forceinline__ Geo gemm_geo(const ExpertStackParams& p, int g) {
  switch (g) {
    case 0: return {(p.Hq + 2) * p.D / 128, p.H / 64};
    case 1: return {p.H / 128, p.Hq * p.D / 64};
    case 2: return {2 * p.I / 128, p.H / 64};
    default: return {p.H / 128, p.I / 64};
  }
}
__device__ __forceinline__ void pair_range(const Geo& g, int cta, int G, int& p0, int& p1) {
  const int total = g.n_tiles * g.kbs;
  p0 = int((long long)total * cta / G);
  p1 = int((long long)total * (cta + 1) / G);
}


// ------------------------------------------------------------------ worker routines
// The loaders below are separate functions on purpose: inlined into the kernel they share its register
// budget (168 per thread at 320 threads), a batch of loads gets spilled as it is issued, and a spilled load
// has to arrive before the spill can store it: the batch degenerates into one L2 round trip per load.
// As functions of their own each has room to keep a whole batch in flight.
struct WCtx {
  const ExpertStackParams* p;
  int cta, G, wtid, lane, M, H, Nqkv, N2I;
  uint32_t sA;           // shared-memory address of the phase-private region
  float inv_H;
};

// Thread mapping of the two activation loaders: a worker owns one 4-column group (c4 = wtid & 15) of rows
// r0, r0 + 16, r0 + 32, r0 + 48 (r0 = wtid >> 4) in every K block of the CTA, so the index arithmetic is a few
// adds per element (no division by run-time values: eight warps per SM leave ~1000 instructions per
// microsecond per warp, and a software division costs a hundred cycles of dependent latency).

// activation operand = rows of h times a per-column factor (bf16, swizzled K-major blocks, one per pair);
// optionally the row sums of squares of the K blocks of weight tile 0 (each K block exactly once per grid)
__device__ __noinline__ void es_load_h(const WCtx& c, int kbs, int p0, int p1, const float* scale, float* ss) {
  constexpr int UP = 4;                       // pairs per batch of loads
  const ExpertStackParams& p = *c.p;
  const int c4 = c.wtid & 15, r0 = c.wtid >> 4, np = p1 - p0;
  int kb = p0 % kbs, nt = p0 / kbs;
  const float* hrow[4];
  uint32_t soff[4];
  bool ok[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int m = r0 + 16 * j;
    ok[j] = m < c.M;
    hrow[j] = p.h + size_t(ok[j] ? m : 0) * c.H + c4 * 4;
    soff[j] = c.sA + sw64(m, c4 * 4);
  }
  for (int pr = 0; pr < np; pr += UP) {
    float4 hv[UP][4], sc[UP];
    bool t0[UP];
#pragma unroll
    for (int b = 0; b < UP; ++b) {
      t0[b] = false;
      if (pr + b < np) {
        const int k = kb * 64;
        t0[b] = nt == 0;
        sc[b] = __ldg(reinterpret_cast<const float4*>(scale + k + c4 * 4));
#pragma unroll
        for (int j = 0; j < 4; ++j)
          hv[b][j] = ok[j] ? __ldcg(reinterpret_cast<const float4*>(hrow[j] + k)) : make_float4(0.f, 0.f, 0.f, 0.f);
        if (++kb == kbs) { kb = 0; ++nt; }
      }
    }
#pragma unroll
    for (int b = 0; b < UP; ++b) {
      if (pr + b < np) {
        const uint32_t blk = uint32_t(pr + b) * kActBlk;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float4 h4 = hv[b][j];
          if (ok[j]) st_shared_v2(blk + soff[j], pack_bf16(h4.x * sc[b].x, h4.y * sc[b].y), pack_bf16(h4.z * sc[b].z, h4.w * sc[b].w));
          if (ss != nullptr && t0[b]) {                    // uniform over the CTA: the shuffles see full warps
            float sq = h4.x * h4.x + h4.y * h4.y + h4.z * h4.z + h4.w * h4.w;
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
            if (c4 == 0 && ok[j]) atomicAdd(ss + r0 + 16 * j, sq);
          }
        }
      }
    }
  }
}

// activation operand of the down projection: GeGLU of the gate / up sums (row 1/rms and bias applied on the way)
__device__ __noinline__ void es_load_glu(const WCtx& c, int kbs, int p0, int p1, const float* bias, const float* ss) {
  constexpr int UP = 2;
  const ExpertStackParams& p = *c.p;
  const int c4 = c.wtid & 15, r0 = c.wtid >> 4, np = p1 - p0;
  int kb = p0 % kbs;
  const float* grow[4];
  uint32_t soff[4];
  float rms[4];
  bool ok[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int m = r0 + 16 * j;
    ok[j] = m < c.M;
    grow[j] = p.acc_gu + size_t(ok[j] ? m : 0) * c.N2I + c4 * 8;
    soff[j] = c.sA + sw64(m, c4 * 4);
    rms[j] = ok[j] ? __ldcg(ss + m) : 1.f;
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) rms[j] = rsqrtf(rms[j] * c.inv_H + p.eps);
  for (int pr = 0; pr < np; pr += UP) {
    float4 a0[UP][4], a1[UP][4], b0[UP], b1[UP];
#pragma unroll
    for (int b = 0; b < UP; ++b) {
      if (pr + b < np) {
        const int k2 = kb * 128;                           // gate / up interleaved: two values per intermediate column
        b0[b] = __ldg(reinterpret_cast<const float4*>(bias + k2 + c4 * 8));
        b1[b] = __ldg(reinterpret_cast<const float4*>(bias + k2 + c4 * 8 + 4));
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if (ok[j]) {
            a0[b][j] = __ldcg(reinterpret_cast<const float4*>(grow[j] + k2));
            a1[b][j] = __ldcg(reinterpret_cast<const float4*>(grow[j] + k2 + 4));
          }
        }
        if (++kb == kbs) kb = 0;
      }
    }
#pragma unroll
    for (int b = 0; b < UP; ++b) {
      if (pr + b < np) {
        const uint32_t blk = uint32_t(pr + b) * kActBlk;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if (ok[j]) {
            const float r = rms[j];
            const float4 x0 = a0[b][j], x1 = a1[b][j];
            const float y0 = gelu_tanh_f(x0.x * r + b0[b].x) * (x0.y * r + b0[b].y);
            const float y1 = gelu_tanh_f(x0.z * r + b0[b].z) * (x0.w * r + b0[b].w);
            const float y2 = gelu_tanh_f(x1.x * r + b1[b].x) * (x1.y * r + b1[b].y);
            const float y3 = gelu_tanh_f(x1.z * r + b1[b].z) * (x1.w * r + b1[b].w);
            st_shared_v2(blk + soff[j], pack_bf16(y0, y1), pack_bf16(y2, y3));
          }
        }
      }
    }
  }
}

// one q or k head row group of the fused projection: 1/rms, bias, rounding to bf16, rotation; 4 + 4 values
__device__ __forceinline__ void rope_store(float4 a, float4 b, float4 ba, float4 bb, float4 c, float4 s, float rms,
                                           uint32_t tile, int r, int d0) {
  const float xa[4] = {round_bf16(a.x * rms + ba.x), round_bf16(a.y * rms + ba.y), round_bf16(a.z * rms + ba.z), round_bf16(a.w * rms + ba.w)};
  const float xb[4] = {round_bf16(b.x * rms + bb.x), round_bf16(b.y * rms + bb.y), round_bf16(b.z * rms + bb.z), round_bf16(b.w * rms + bb.w)};
  const float cc[4] = {c.x, c.y, c.z, c.w}, sn[4] = {s.x, s.y, s.z, s.w};
  float lo[4], hi[4];
#pragma unroll
  for (int t = 0; t < 4; ++t) { lo[t] = xa[t] * cc[t] - xb[t] * sn[t]; hi[t] = xb[t] * cc[t] + xa[t] * sn[t]; }
  st_shared_v2(tile + sw64(r, d0), pack_bf16(lo[0], lo[1]), pack_bf16(lo[2], lo[3]));
  st_shared_v2(tile + sw64(r, 128 + d0), pack_bf16(hi[0], hi[1]), pack_bf16(hi[2], hi[3]));
}

struct AttUnit { int head, split, p0, np, q0, nq, kv_ptr; };   // pool rows [p0, p0 + np), action rows [q0, q0 + nq)

// Q / K / V tiles of one attention unit: pool rows by cp.async (zero fill past the unit's rows), q rows of the
// head and the unit's share of the freshly projected rows from the fp32 sums. A worker owns one 4-wide
// dimension group d0 (and its rotation partner d0 + 128) of rows r0, r0 + 8, ...: biases are read once.
__device__ __noinline__ void es_load_att(const WCtx& c, const AttUnit& u, int layer, const float* bias) {
  const ExpertStackParams& p = *c.p;
  const uint32_t sQ = c.sA + 8192, sK = sQ + 32768, sV = sK + 32768;
  const int kn = u.np + u.nq;
  const int cg = c.wtid & 31, r0 = c.wtid >> 5, d0 = cg * 4;
  const __nv_bfloat16* kpl = p.k_pool + size_t(layer) * p.pool_layer_stride + cg * 8;
  const __nv_bfloat16* vpl = p.v_pool + size_t(layer) * p.pool_layer_stride + cg * 8;
  {
    // thread (cg, r0): 16-byte chunk cg of rows r0, r0 + 8, ..., r0 + 56
    const uint32_t cbase = uint32_t(cg >> 3) * kActBlk;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int r = r0 + 8 * j;
      const bool in_pool = r < u.np;
      if (in_pool || r >= kn) {
        const size_t row = size_t(in_pool ? u.kv_ptr + u.p0 + r : 0) * p.pool_row_stride;
        const uint32_t off = cbase + uint32_t(r) * 128u + uint32_t(((cg & 7) ^ (r & 7)) << 4);
        cp16(sK + off, kpl + row, in_pool);
        cp16(sV + off, vpl + row, in_pool);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  }
  {
    const float* src0 = p.acc_qkv + u.head * kD + d0;
    const float* bs = bias + u.head * kD + d0;
    const float4 ba = __ldg(reinterpret_cast<const float4*>(bs)), bb = __ldg(reinterpret_cast<const float4*>(bs + 128));
#pragma unroll 1
    for (int jb = 0; jb < 8; jb += 4) {
      float4 a[4], b[4], cc[4], sn[4];
      float ssv[4];
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const int m = r0 + 8 * (jb + t);
        if (m < c.M) {
          const float* cs = p.cos_sin + size_t(__ldg(p.pos + m)) * kD + d0;
          ssv[t] = __ldcg(p.ss + m);
          a[t] = __ldcg(reinterpret_cast<const float4*>(src0 + size_t(m) * c.Nqkv));
          b[t] = __ldcg(reinterpret_cast<const float4*>(src0 + size_t(m) * c.Nqkv + 128));
          cc[t] = __ldg(reinterpret_cast<const float4*>(cs));
          sn[t] = __ldg(reinterpret_cast<const float4*>(cs + 128));
        }
      }
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const int m = r0 + 8 * (jb + t);
        if (m < c.M) rope_store(a[t], b[t], ba, bb, cc[t], sn[t], rsqrtf(ssv[t] * c.inv_H + p.eps), sQ, m, d0);
      }
    }
  }
  if (r0 < u.nq) {                                           // nq <= 8 (ceil(M / S)): one row per thread
    const int m = u.q0 + r0, r = u.np + r0;
    const float* src = p.acc_qkv + size_t(m) * c.Nqkv + p.Hq * kD + d0;
    const float* bs = bias + p.Hq * kD + d0;
    const float* cs = p.cos_sin + size_t(__ldg(p.pos + m)) * kD + d0;
    const float ssv = __ldcg(p.ss + m);
    const float4 a = __ldcg(reinterpret_cast<const float4*>(src)), b = __ldcg(reinterpret_cast<const float4*>(src + 128));
    const float4 v0 = __ldcg(reinterpret_cast<const float4*>(src + kD)), v1 = __ldcg(reinterpret_cast<const float4*>(src + kD + 128));
    const float4 ba = __ldg(reinterpret_cast<const float4*>(bs)), bb = __ldg(reinterpret_cast<const float4*>(bs + 128));
    const float4 b0 = __ldg(reinterpret_cast<const float4*>(bs + kD)), b1 = __ldg(reinterpret_cast<const float4*>(bs + kD + 128));
    const float4 cc = __ldg(reinterpret_cast<const float4*>(cs)), sn = __ldg(reinterpret_cast<const float4*>(cs + 128));
    const float rms = rsqrtf(ssv * c.inv_H + p.eps);
    rope_store(a, b, ba, bb, cc, sn, rms, sK, r, d0);
    st_shared_v2(sV + sw64(r, d0), pack_bf16(v0.x * rms + b0.x, v0.y * rms + b0.y), pack_bf16(v0.z * rms + b0.z, v0.w * rms + b0.w));
    st_shared_v2(sV + sw64(r, 128 + d0), pack_bf16(v1.x * rms + b1.x, v1.y * rms + b1.y), pack_bf16(v1.z * rms + b1.z, v1.w * rms + b1.w));
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
}

// Merge the KV splits of every (row, head): all partial slots hold finite numbers (zeros until a unit first
// wrote them), so the loads of all splits go out together and a weight of zero removes the slots of empty units.
__device__ __noinline__ void es_merge(const WCtx& c, int S, int QW) {
  constexpr int kMaxS = 18;
  const ExpertStackParams& p = *c.p;
  const int total = c.M * p.Hq * 64;
  for (int i = c.cta * kWorkers + c.wtid; i < total; i += c.G * kWorkers) {
    const int m = i / (p.Hq * 64), rem = i - m * (p.Hq * 64), hh = rem >> 6, d4 = rem & 63;
    const float* ml = p.part_ml + (size_t(hh) * S * kRows + m) * 2;
    const float* po = p.part_o + (size_t(hh) * S * kRows + m) * kD + d4 * 4;
    float2 mlv[kMaxS];
    float4 ov[kMaxS];
#pragma unroll
    for (int s2 = 0; s2 < kMaxS; ++s2) {
      mlv[s2] = make_float2(-INFINITY, 0.f);
      ov[s2] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (s2 < S) {
        mlv[s2] = __ldcg(reinterpret_cast<const float2*>(ml + size_t(s2) * kRows * 2));
        ov[s2] = __ldcg(reinterpret_cast<const float4*>(po + size_t(s2) * kRows * kD));
      }
    }
    float mmax = -INFINITY;
#pragma unroll
    for (int s2 = 0; s2 < kMaxS; ++s2) mmax = fmaxf(mmax, mlv[s2].y > 0.f ? mlv[s2].x : -INFINITY);
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    float lsum = 0.f;
#pragma unroll
    for (int s2 = 0; s2 < kMaxS; ++s2) {
      const float w = mlv[s2].y > 0.f ? exp2f(mlv[s2].x - mmax) : 0.f;
      lsum += w * mlv[s2].y;
      acc.x += w * ov[s2].x; acc.y += w * ov[s2].y; acc.z += w * ov[s2].z; acc.w += w * ov[s2].w;
    }
    const float inv = lsum > 0.f ? 1.f / lsum : 0.f;
    uint2 raw;
    raw.x = pack_bf16(acc.x * inv, acc.y * inv);
    raw.y = pack_bf16(acc.z * inv, acc.w * inv);
    *reinterpret_cast<uint2*>(p.attn + size_t(m) * QW + hh * kD + d4 * 4) = raw;
  }
}

// Second half of a projection's drain: the staged tiles (shared memory, [tile][64][132] fp32) go to L2 as
// 16-byte reductions, 512 contiguous bytes per warp, starting at a row that differs from CTA to CTA.
constexpr int kLds = 132;
__device__ __noinline__ void es_reduce_out(const WCtx& c, const float* stg, int nt0, int na, float* out, int ldo,
                                           const float* gate) {
  const ExpertStackParams& p = *c.p;
  const int n4 = c.wtid & 31, r0 = c.wtid >> 5;           // a warp covers one row of a tile, 8 rows in flight per CTA
  const int rot = (c.cta * 3) % c.M;
  for (int a = 0; a < na; ++a) {
    const int n = (nt0 + a) * 128 + n4 * 4;
    float4 g = make_float4(1.f, 1.f, 1.f, 1.f);
    if (gate) g = __ldg(reinterpret_cast<const float4*>(gate + n));
    const float* src = stg + a * kRows * kLds + n4 * 4;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int mi = r0 + 8 * j;
      if (mi < c.M) {
        int m = mi + rot;
        if (m >= c.M) m -= c.M;
        float4 v = *reinterpret_cast<const float4*>(src + m * kLds);
        v.x *= g.x; v.y *= g.y; v.z *= g.z; v.w *= g.w;
        if (p.debug & 1) *reinterpret_cast<float4*>(out + size_t(m) * ldo + n) = v;   // timing experiment: no reductions
        else red_add_v4(out + size_t(m) * ldo + n, v);
      }
    }
  }
}

}  // namespace

__global__ void __launch_bounds__(kThreads, 1)
expert_stack_kernel(const __grid_constant__ ExpertStackParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* ring = smem;
  uint8_t* regA = smem + kRing * kSlotBytes;
  __shared__ __align__(8) uint64_t full_bar[kRing];
  __shared__ __align__(8) uint64_t empty_bar[kRing];
  __shared__ __align__(8) uint64_t act_ready, acc_bar, s_bar, p_ready;
  __shared__ uint32_t tmem_base_s;
  __shared__ volatile int abort_s;
  __shared__ int go_s;      // the workers' common decision after a grid barrier (written by one thread between two worker barriers)

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int cta = blockIdx.x, G = gridDim.x;
  const int M = p.M, H = p.H, Nqkv = (p.Hq + 2) * p.D, N2I = 2 * p.I, QW = p.Hq * p.D;
  const int S = p.att_splits;

  if (tid == 0) {
    for (int s = 0; s < kRing; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(&act_ready, kWorkers);
    mbar_init(&acc_bar, 1);
    mbar_init(&s_bar, 1);
    mbar_init(&p_ready, 64);
    abort_s = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(&tmem_base_s, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_s;

  // raise the abort: this CTA drains, the barrier word tells every other CTA
  auto fail = [&](int code) {
    if (abort_s == 0) abort_s = code;
    atomicOr(p.barrier, kAbortBit);
    if (p.status) atomicCAS(p.status, 0, code);
  };

  // attention unit of this CTA (the KV range is read from device memory: it changes per request)
  const int kv_len = p.kv_len[0], kv_ptr = p.kv_ptr[0];
  const int Lp = kv_len - M;                                   // rows that live in the pool
  // Split s takes pool rows [s kp, (s+1) kp) and action rows [s kq, (s+1) kq): the rows the projection just
  // produced are spread over all units instead of landing on the last one (softmax does not care about order).
  const int kp = (max(Lp, 0) + S - 1) / S, kq = (M + S - 1) / S;
  const bool att_unit = cta < p.Hq * S;
  const int att_head = cta / S, att_split = cta % S;
  const int att_p0 = att_split * kp, att_np = att_unit ? max(0, min(kp, Lp - att_p0)) : 0;   // pool rows of the unit
  const int att_q0 = att_split * kq, att_nq = att_unit ? max(0, min(kq, M - att_q0)) : 0;    // action rows of the unit
  const int att_kn = att_np + att_nq;
  const bool att_live = att_unit && att_kn > 0;
  if (tid == 0 && (kp + kq > kKeys || kq > 8 || Lp < 0)) fail(kStatusBadArg);
  __syncthreads();

  if (warp == 0) {
    // ================================================================ weight producer
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = abort_s == 0;
      for (int step = p.step_begin; step < p.step_end && ok; ++step) {
        for (int layer = 0; layer < p.n_layers && ok; ++layer) {
          for (int g = 0; g < 4 && ok; ++g) {
            const Geo geo = gemm_geo(p, g);
            int p0, p1;
            pair_range(geo, cta, G, p0, p1);
            const CUtensorMap* tm = p.tmaps + layer * 4 + g;
            for (int pr = p0; pr < p1; ++pr, ++it) {
              const int slot = int(it % kRing);
              const uint32_t par = (it / kRing) & 1u;
              if (!es_wait(&empty_bar[slot], par ^ 1u, &abort_s)) {
                fail(kStatusTimeoutEmpty);
                ok = false;
                break;
              }
              mbar_expect_tx(&full_bar[slot], kSlotBytes);
              tma_load_2d(ring + slot * kSlotBytes, tm, &full_bar[slot], (pr % geo.kbs) * 64, (pr / geo.kbs) * 128);
            }
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ================================================================ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = make_idesc_f16(128, kRows, 1);
      const uint32_t idesc_s = make_idesc_f16(128, kKeys, 1);
      const uint32_t idesc_o = make_idesc_f16_bmn(128, kD, 1);
      const uint32_t sA = smem_u32(regA);
      const uint32_t sP = sA, sQ = sA + 8192, sK = sQ + 32768, sV = sK + 32768;
      uint32_t it = 0, act_par = 0, p_par = 0;
      bool ok = true;
      auto gemm_phase = [&](int g) {
        const Geo geo = gemm_geo(p, g);
        int p0, p1;
        pair_range(geo, cta, G, p0, p1);
        if (!es_wait(&act_ready, act_par, &abort_s)) { fail(kStatusTimeoutFull); ok = false; return; }
        act_par ^= 1u;
        tc_fence_after();
        const int nt0 = p0 / geo.kbs;
        for (int pr = p0; pr < p1; ++pr, ++it) {
          const int slot = int(it % kRing);
          const uint32_t par = (it / kRing) & 1u;
          if (!es_wait(&full_bar[slot], par, &abort_s)) { fail(kStatusTimeoutFull); ok = false; return; }
          tc_fence_after();
          const int kb = pr % geo.kbs, acc = pr / geo.kbs - nt0;
          const uint64_t da = make_smem_desc_sw128(smem_u32(ring + slot * kSlotBytes));
          const uint64_t db = make_smem_desc_sw128(sA + uint32_t(pr - p0) * kActBlk);
          const bool first = pr == p0 || kb == 0;
#pragma unroll
          for (int k = 0; k < 4; ++k) umma_f16(tmem + uint32_t(acc * kRows), da + 2 * k, db + 2 * k, idesc, (first && k == 0) ? 0u : 1u);
          umma_commit(&empty_bar[slot]);
        }
        if (p1 > p0) umma_commit(&acc_bar);
      };
      for (int step = p.step_begin; step < p.step_end && ok; ++step) {
        for (int layer = 0; layer < p.n_layers && ok; ++layer) {
          gemm_phase(0);
          if (!ok) break;
          if (att_live) {
            if (!es_wait(&act_ready, act_par, &abort_s)) { fail(kStatusTimeoutFull); ok = false; break; }
            act_par ^= 1u;
            tc_fence_after();
#pragma unroll
            for (int kk = 0; kk < kD / 16; ++kk) {
              const uint64_t dq = make_smem_desc_sw128(sQ + (kk >> 2) * kActBlk) + 2 * (kk & 3);
              const uint64_t dk = make_smem_desc_sw128(sK + (kk >> 2) * kActBlk) + 2 * (kk & 3);
              umma_f16(tmem + kSCol, dq, dk, idesc_s, kk != 0);
            }
            umma_commit(&s_bar);
            if (!es_wait(&p_ready, p_par, &abort_s)) { fail(kStatusTimeoutAcc); ok = false; break; }
            p_par ^= 1u;
            tc_fence_after();
#pragma unroll
            for (int kk = 0; kk < kKeys / 16; ++kk) {
              const uint64_t dp = make_smem_desc_sw128(sP) + 2 * kk;
              const uint64_t dv = make_smem_desc_sw128_mn(sV + kk * 2048, kActBlk, 1024);
              umma_f16(tmem + kOCol, dp, dv, idesc_o, kk != 0);
            }
            umma_commit(&acc_bar);
          }
          gemm_phase(1);
          if (!ok) break;
          gemm_phase(2);
          if (!ok) break;
          gemm_phase(3);
        }
      }
    }
    __syncwarp();
  } else {
    // ================================================================ workers
    const int wtid = tid - 64;                 // 0..255
    const int quad = warp & 3;                 // TMEM lane quadrant this warp may read
    const int half = (warp - 2) >> 2;          // which half of the columns it takes
    const uint32_t lane_base = tmem + (uint32_t(quad * 32) << 16);
    const uint32_t sA = smem_u32(regA);
    const uint32_t sP = sA, sQ = sA + 8192, sK = sQ + 32768, sV = sK + 32768;
    const float inv_H = 1.f / float(H);
    const WCtx wc{&p, cta, G, wtid, lane, M, H, Nqkv, N2I, sA, inv_H};
    const AttUnit au{att_head, att_split, att_p0, att_np, att_q0, att_nq, kv_ptr};
    uint32_t epoch = 0, acc_par = 0, s_par = 0;
    unsigned long long* tr = p.trace ? p.trace + 64 * cta : nullptr;
    int tr_i = 0;
    bool tracing = false;
#define ES_STAMP() do { if (tr && tracing && wtid == 64 && tr_i < 64) tr[tr_i++] = globaltimer_ns(); } while (0)

    auto grid_sync = [&]() -> bool {
      __threadfence();
      worker_sync();
      if (wtid == 0) {
        ++epoch;
        const unsigned target = epoch * unsigned(G);
        if (abort_s == 0) {
          red_release_gpu_add(p.barrier, 1u);
          const uint64_t t0 = globaltimer_ns();
          uint32_t spins = 0;
          for (;;) {
            const unsigned v = ld_relaxed_gpu(p.barrier);
            if (v & kAbortBit) { if (abort_s == 0) abort_s = kStatusTimeoutPeer; break; }
            if (v >= target) break;
            if ((++spins & 63) == 0 && globaltimer_ns() - t0 > 1000000000ull) { fail(kStatusTimeoutPeer); break; }
          }
        }
        go_s = abort_s == 0 ? 1 : 0;
        __threadfence();
      }
      worker_sync();
      return go_s != 0;
    };
    auto zero_rows = [&](float* base, int width) {
      // rows [0, M) of a [64, width] fp32 buffer (contiguous), spread over every worker of the grid
      const int total = (M * width) >> 2;
      float4* b4 = reinterpret_cast<float4*>(base);
      for (int i = cta * kWorkers + wtid; i < total; i += G * kWorkers) b4[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    };
    auto arrive_act = [&]() {
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(&act_ready);
    };
    // drain the accumulators of a projection phase: out[m, n] += gate[n] * acc (fp32 reductions in L2)
    // Drain the accumulators of a projection phase: out[m, n] += gate[n] * acc with fp32 reductions in L2.
    // The tiles go through shared memory (the activation blocks are dead once the accumulator barrier fired)
    // so that a thread owns four consecutive columns: one 16-byte reduction instead of four, a warp covers
    // 512 contiguous bytes, and the row order can start anywhere: CTAs that share a weight tile add into the
    // same rows, and each starts at another row so that they do not queue up on one address.
    auto drain = [&](const Geo& geo, int p0, int p1, float* out, int ldo, const float* gate) {
      const bool any = p1 > p0;
      const int nt0 = any ? p0 / geo.kbs : 0, na = any ? (p1 - 1) / geo.kbs - nt0 + 1 : 0;
      float* stg = reinterpret_cast<float*>(regA);
      if (any) {
        if (!es_wait(&acc_bar, acc_par, &abort_s)) fail(kStatusTimeoutAcc);
        tc_fence_after();
        for (int a = 0; a < na; ++a) {
          uint32_t r[32];
          tmem_ld_32x32(lane_base + uint32_t(a * kRows + half * 32), r);
          tmem_ld_wait();
          float* dst = stg + (a * kRows + half * 32) * kLds + quad * 32 + lane;
#pragma unroll
          for (int j = 0; j < 32; ++j) dst[j * kLds] = __uint_as_float(r[j]);
        }
        tc_fence_before();
        acc_par ^= 1u;
      }
      worker_sync();
      if (any) es_reduce_out(wc, stg, nt0, na, out, ldo, gate);
    };
    for (int step = p.step_begin; step < p.step_end; ++step) {
      const bool first_step = step == p.step_begin;
      // ------------------------------------------------ input projection (and the first clearing)
      if (first_step) {
        zero_rows(p.acc_qkv, Nqkv);
        zero_rows(p.acc_gu, N2I);
        if (cta == 0 && wtid < 2 * kRows) p.ss[wtid] = 0.f;
      }
      {
        const int per_row = H >> 2, total = M * per_row, A = p.A;
        for (int i = cta * kWorkers + wtid; i < total; i += G * kWorkers) {
          const int m = i / per_row, n = (i - m * per_row) * 4;
          float acc[4];
#pragma unroll
          for (int t = 0; t < 4; ++t) acc[t] = bf2f(p.b_in[n + t]);
          for (int j = 0; j < A; j += 4) {
            float x[4];
            if (first_step) {
              const uint2 raw = *reinterpret_cast<const uint2*>(p.x0 + size_t(m) * A + j);
              x[0] = __uint_as_float(raw.x << 16); x[1] = __uint_as_float(raw.x & 0xffff0000u);
              x[2] = __uint_as_float(raw.y << 16); x[3] = __uint_as_float(raw.y & 0xffff0000u);
            } else {
              const float4 xv = __ldcg(reinterpret_cast<const float4*>(p.x_t + size_t(m) * A + j));
              x[0] = round_bf16(xv.x); x[1] = round_bf16(xv.y); x[2] = round_bf16(xv.z); x[3] = round_bf16(xv.w);
            }
#pragma unroll
            for (int t = 0; t < 4; ++t) {
              const uint2 wr = __ldg(reinterpret_cast<const uint2*>(p.w_in + size_t(n + t) * A + j));
              acc[t] += x[0] * __uint_as_float(wr.x << 16) + x[1] * __uint_as_float(wr.x & 0xffff0000u) +
                        x[2] * __uint_as_float(wr.y << 16) + x[3] * __uint_as_float(wr.y & 0xffff0000u);
            }
          }
          *reinterpret_cast<float4*>(p.h + size_t(m) * H + n) = make_float4(acc[0], acc[1], acc[2], acc[3]);
        }
      }
      if (!grid_sync()) goto done;

      for (int layer = 0; layer < p.n_layers; ++layer) {
        const size_t sl = size_t(step) * p.n_layers + layer;
        tracing = first_step && layer == 1;
        ES_STAMP();
        // ---------------------------------------------------------------- QKV projection
        {
          const Geo geo = gemm_geo(p, 0);
          int p0, p1;
          pair_range(geo, cta, G, p0, p1);
          es_load_h(wc, geo.kbs, p0, p1, p.in_scale + sl * H, p.ss);
          arrive_act();
          ES_STAMP();
          if (!(first_step && layer == 0)) {
            zero_rows(p.acc_gu, N2I);                       // consumed by the previous down projection
            if (cta == 0 && wtid < kRows) p.ss[kRows + wtid] = 0.f;
          }
          drain(geo, p0, p1, p.acc_qkv, Nqkv, nullptr);
          ES_STAMP();
        }
        if (!grid_sync()) goto done;
        ES_STAMP();
        // ---------------------------------------------------------------- attention units
        if (att_live) {
          const float* bias = p.qkv_bias + sl * Nqkv;
          es_load_att(wc, au, layer, bias);
          arrive_act();
          ES_STAMP();
          // softmax of the unit: one thread per query row (rows live in lane quadrants 0 and 1)
          if (quad < 2 && half == 0) {
            const int row = quad * 32 + lane;
            if (!es_wait(&s_bar, s_par, &abort_s)) fail(kStatusTimeoutAcc);
            tc_fence_after();
            uint32_t r0[32], r1[32];
            tmem_ld_32x32(lane_base + kSCol, r0);
            tmem_ld_32x32(lane_base + kSCol + 32, r1);
            tmem_ld_wait();
            const float sl2 = p.sm_scale * 1.4426950408889634f;
            float mx = -INFINITY;
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              if (j < att_kn) mx = fmaxf(mx, __uint_as_float(r0[j]) * sl2);
              if (32 + j < att_kn) mx = fmaxf(mx, __uint_as_float(r1[j]) * sl2);
            }
            float sum = 0.f;
#pragma unroll
            for (int c = 0; c < 8; ++c) {
              uint32_t pk[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const int j = c * 8 + 2 * e;
                const float s0 = __uint_as_float(j < 32 ? r0[j & 31] : r1[j & 31]);
                const float s1 = __uint_as_float(j + 1 < 32 ? r0[(j + 1) & 31] : r1[(j + 1) & 31]);
                const float p0f = j < att_kn ? exp2f(s0 * sl2 - mx) : 0.f;
                const float p1f = j + 1 < att_kn ? exp2f(s1 * sl2 - mx) : 0.f;
                sum += p0f + p1f;
                pk[e] = pack_bf16(p0f, p1f);
              }
              st_shared_v4(sP + uint32_t(row) * 128u + uint32_t((c ^ (row & 7)) << 4), pk[0], pk[1], pk[2], pk[3]);
            }
            if (row < M)
              *reinterpret_cast<float2*>(p.part_ml + (size_t(att_head * S + att_split) * kRows + row) * 2) = make_float2(mx, sum);
            fence_proxy_async_smem();
            tc_fence_before();
            mbar_arrive(&p_ready);
          }
          s_par ^= 1u;
          ES_STAMP();
          // partial O rows to L2
          if (quad < 2) {
            const int row = quad * 32 + lane;
            if (!es_wait(&acc_bar, acc_par, &abort_s)) fail(kStatusTimeoutAcc);
            tc_fence_after();
            float* dst = p.part_o + (size_t(att_head * S + att_split) * kRows + row) * kD + half * 128;
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
              uint32_t r[32];
              tmem_ld_32x32(lane_base + kOCol + half * 128 + c * 32, r);
              tmem_ld_wait();
              if (row < M) {
#pragma unroll
                for (int t = 0; t < 8; ++t)
                  *reinterpret_cast<float4*>(dst + c * 32 + 4 * t) = make_float4(__uint_as_float(r[4 * t]), __uint_as_float(r[4 * t + 1]),
                                                                                 __uint_as_float(r[4 * t + 2]), __uint_as_float(r[4 * t + 3]));
              }
            }
            tc_fence_before();
          }
          acc_par ^= 1u;
        } else if (att_unit) {
          // a unit without rows: an empty partial
          if (wtid < M) *reinterpret_cast<float2*>(p.part_ml + (size_t(att_head * S + att_split) * kRows + wtid) * 2) = make_float2(-INFINITY, 0.f);
        }
        ES_STAMP();
        if (!grid_sync()) goto done;
        ES_STAMP();
        // ---------------------------------------------------------------- merge the splits
        {
          es_merge(wc, S, QW);
          zero_rows(p.acc_qkv, Nqkv);                        // consumed by the attention units
          if (cta == 0 && wtid < kRows) p.ss[wtid] = 0.f;
        }
        if (!grid_sync()) goto done;
        ES_STAMP();
        // ---------------------------------------------------------------- output projection of the attention
        {
          const Geo geo = gemm_geo(p, 1);
          int p0, p1;
          pair_range(geo, cta, G, p0, p1);
          if (wtid == 0) {
            // attn was written by other CTAs with ordinary stores: order the TMA reads behind the barrier's acquire
            asm volatile("fence.proxy.async;" ::: "memory");
            mbar_expect_tx(&act_ready, uint32_t(p1 - p0) * kActBlk);
            const CUtensorMap* tm = p.tmaps + p.n_layers * 4;
            for (int pr = p0; pr < p1; ++pr) tma_load_2d(regA + (pr - p0) * kActBlk, tm, &act_ready, (pr % geo.kbs) * 64, 0);
          } else {
            mbar_arrive(&act_ready);
          }
          ES_STAMP();
          drain(geo, p0, p1, p.h, H, p.gate_in + sl * H);
          ES_STAMP();
        }
        if (!grid_sync()) goto done;
        ES_STAMP();
        // ---------------------------------------------------------------- gate / up projection
        {
          const Geo geo = gemm_geo(p, 2);
          int p0, p1;
          pair_range(geo, cta, G, p0, p1);
          es_load_h(wc, geo.kbs, p0, p1, p.post_scale + sl * H, p.ss + kRows);
          arrive_act();
          ES_STAMP();
          drain(geo, p0, p1, p.acc_gu, N2I, nullptr);
          ES_STAMP();
        }
        if (!grid_sync()) goto done;
        ES_STAMP();
        // ---------------------------------------------------------------- down projection (GeGLU on load)
        {
          const Geo geo = gemm_geo(p, 3);
          int p0, p1;
          pair_range(geo, cta, G, p0, p1);
          const float* bias = p.gu_bias + sl * N2I;
          es_load_glu(wc, geo.kbs, p0, p1, bias, p.ss + kRows);
          arrive_act();
          ES_STAMP();
          drain(geo, p0, p1, p.h, H, p.gate_post + sl * H);
          ES_STAMP();
        }
        if (!grid_sync()) goto done;
      }
      tracing = false;

      // ------------------------------------------------ final norm + output projection + Euler update
      {
        const int A = p.A, total = M * A;
        const int gw = cta * (kWorkers / 32) + (warp - 2), nw = G * (kWorkers / 32);
        const float* fs = p.fin_scale + size_t(step) * H;
        for (int i = gw; i < total; i += nw) {
          const int m = i / A, j = i - m * A;
          float acc = 0.f, sq = 0.f;
          for (int k = lane * 4; k < H; k += 128) {
            const float4 hv = __ldcg(reinterpret_cast<const float4*>(p.h + size_t(m) * H + k));
            const float4 sc = __ldg(reinterpret_cast<const float4*>(fs + k));
            const uint2 wr = __ldg(reinterpret_cast<const uint2*>(p.w_out + size_t(j) * H + k));
            acc += hv.x * sc.x * __uint_as_float(wr.x << 16) + hv.y * sc.y * __uint_as_float(wr.x & 0xffff0000u) +
                   hv.z * sc.z * __uint_as_float(wr.y << 16) + hv.w * sc.w * __uint_as_float(wr.y & 0xffff0000u);
            sq += hv.x * hv.x + hv.y * hv.y + hv.z * hv.z + hv.w * hv.w;
          }
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) {
            acc += __shfl_xor_sync(0xffffffffu, acc, o);
            sq += __shfl_xor_sync(0xffffffffu, sq, o);
          }
          if (lane == 0) {
            const float v = acc * rsqrtf(sq * inv_H + p.eps) + __ldg(p.out_bias + size_t(step) * A + j);
            const float xp = first_step ? bf2f(p.x0[i]) : __ldcg(p.x_t + i);
            const float xn = xp + p.dt * v;
            p.x_t[i] = xn;
            if (step + 1 == p.step_end) p.out[i] = __float2bfloat16(xn);
          }
        }
      }
      if (step + 1 < p.step_end && !grid_sync()) goto done;
    }
  done:;
#undef ES_STAMP
  }

  if (abort_s != 0 && tid == 0) {
    // weight tiles of this CTA may still be in flight: let them land before the block goes away
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, kTmemCols);
}

// ----------------------------------------------------------------------- host
int expert_stack_grid() {
  static int cached[64];
  static bool have[64] = {false};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
  if (have[dev]) return cached[dev];
  int sms = 0, per_sm = 0;
  if (cudaFuncSetAttribute(expert_stack_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, expert_stack_kernel, kThreads, kSmemBytes) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  cached[dev] = per_sm > 0 ? sms : 0;
  have[dev] = true;
  return cached[dev];
}

cudaError_t expert_stack_launch(const ExpertStackParams& p, cudaStream_t stream) {
  const int G = expert_stack_grid();
  if (G <= 0) return cudaErrorInvalidConfiguration;
  // geometry the kernel is written for
  if (p.M <= 0 || p.M > kRows || p.D != kD || p.A <= 0 || p.A % 4 || p.H % 128 || p.I % 64 ||
      ((p.Hq + 2) * p.D) % 128 || (2 * p.I) % 128 || p.n_layers <= 0 || p.step_end <= p.step_begin || p.step_begin < 0)
    return cudaErrorInvalidValue;
  if (p.att_splits <= 0 || p.Hq * p.att_splits > G || (p.M + p.att_splits - 1) / p.att_splits > 8) return cudaErrorInvalidValue;
  const int nt[4] = {(p.Hq + 2) * p.D / 128, p.H / 128, 2 * p.I / 128, p.H / 128};
  const int kb[4] = {p.H / 64, p.Hq * p.D / 64, p.H / 64, p.I / 64};
  for (int g = 0; g < 4; ++g) {
    const long long total = (long long)nt[g] * kb[g];
    for (int c = 0; c < G; ++c) {
      const int p0 = int(total * c / G), p1 = int(total * (c + 1) / G);
      if (p1 - p0 > kMaxPairs) return cudaErrorInvalidValue;                                  // activation blocks per CTA
      if (p1 > p0 && (p1 - 1) / kb[g] - p0 / kb[g] + 1 > 3) return cudaErrorInvalidValue;     // accumulators per CTA
    }
  }
  if (!p.tmaps || !p.barrier || !p.h || !p.acc_qkv || !p.acc_gu || !p.ss || !p.attn || !p.part_o || !p.part_ml ||
      !p.x_t || !p.x0 || !p.out || !p.kv_ptr || !p.kv_len || !p.pos || !p.cos_sin)
    return cudaErrorInvalidValue;
  cudaError_t e = cudaMemsetAsync(p.barrier, 0, sizeof(unsigned), stream);
  if (e != cudaSuccess) return e;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(G);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  bump_launch_counter(1);
  return cudaLaunchKernelEx(&cfg, expert_stack_kernel, p);
}

}  // namespace pb

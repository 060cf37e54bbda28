// One persistent kernel per decode token (batch 1, int8 weight-only).
//
// Why: at batch 1 a decode step of the 1.5B model is 140 dependent GEMVs of
// 0.4-2 us each; launched one by one (even from a CUDA graph) every kernel
// boundary drains the memory pipeline.  Here one CTA per SM stays resident for
// the whole token.  Each CTA owns a fixed slice of the output rows of every
// projection, and ALL weight bytes that CTA will ever need are laid out
// back to back in one private stream (built once at load time).  A producer
// warp walks that stream with bulk async copies (cp.async.bulk, completion on
// mbarriers) into a ring of shared-memory slots and never waits for
// activations, so HBM stays busy across the dependency points; eight consumer
// warps dequantise from shared memory with the activations held in registers
// and meet in warp-shuffle reductions.  The dependency points of the graph
// (q/k/v -> attention -> o -> gate/up -> down) are grid-wide barriers on a
// global counter.  Every wait is bounded: on expiry the kernel records an
// error code and returns.
//
// Arithmetic is that of examples/BuddyDeepSeekR1/subgraph0_decode_simplify.mlir
// :46-260 with the int8 GEMV of
// midend/lib/Conversion/MatMulOptimization/DequantMatMulVectorizationDecode.cpp:250-321
// and the attention recurrence of frontend/Python/ops/tosa.py:14245-14594.
#include "common.cuh"
#include "mega.cuh"

#include <cstddef>

namespace b200 {

namespace {

constexpr int kCW = 8;            // consumer warps
constexpr int kCT = kCW * 32;     // consumer threads
constexpr uint32_t kSpinLimit = 1u << 24;
constexpr float kSeed = -1.0e30f;

// ---- PTX wrappers ---------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      " selp.u32 %0, 1, 0, p;\n}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait.  Returns false when it gave up or the grid is already in the
// failed state; callers carry on with the same control flow (so CTA barriers
// stay matched) and the host discards the step.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, volatile int *err,
                                          volatile int *abort_flag) {
  if (*abort_flag)
    return false;
  for (uint32_t it = 0; it < kSpinLimit; ++it) {
    if (mbar_try_wait(bar, parity))
      return true;
    if ((it & 0xFFF) == 0xFFF && *err != 0)
      break;
  }
  *abort_flag = 1;
  return false;
}
__device__ __forceinline__ void bulk_g2s(void *dst, const void *src, uint32_t bytes,
                                         uint64_t *bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
          "r"(smem_u32(dst)),
      "l"(src), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void consumer_sync() {
  asm volatile("bar.sync 1, %0;" ::"n"(kCT) : "memory");
}
__device__ __forceinline__ unsigned ld_relaxed(const unsigned *p) {
  unsigned v;
  asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_relaxed(unsigned *p, unsigned v) {
  asm volatile("red.relaxed.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ float4 ldcg4(const float *p) {
  return __ldcg(reinterpret_cast<const float4 *>(p));
}
// Streamed rows hold u = q + 128 (the int8 weight with its sign bit flipped).
// Byte e of a word, moved to the low byte of an otherwise zero word, IS the
// float u * 2^-149 (a denormal), so the dequantisation is one PRMT and the
// multiply-accumulate one FFMA per weight.  The activations are pre-scaled by
// 2^64 to keep every product in the normal range (products are exact up to
// the usual single rounding of the FMA), and the offset 128 * sum(x) is
// subtracted once per row: sum x*q = 2^85 * sum (x*2^64)*(u*2^-149) - 128*sum x.
constexpr float kXScale = 18446744073709551616.0f;      // 2^64
constexpr float kAccScale = 38685626227668133590597632.0f;  // 2^85
__device__ __forceinline__ void dot_unit(const uint4 &w, const float (&x)[16], float (&a)[4]) {
  const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
  for (int j = 0; j < 4; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e)
      a[e] = fmaf(x[4 * j + e], __uint_as_float(__byte_perm(ws[j], 0u, 0x4440 + e)), a[e]);
}

__device__ __forceinline__ void rows_of(int N, int cta, int grid, int &begin, int &count) {
  const int base = N / grid, rem = N % grid;
  begin = cta * base + min(cta, rem);
  count = base + (cta < rem ? 1 : 0);
}

struct Shared {
  uint64_t full[kMegaMaxSlots];
  uint64_t empty[kMegaMaxSlots];
  float cs[64], sn[64];                 // cos / sin of this step's position
  float part[kCW][kMegaMaxRowsB];       // mode-B per-warp partial sums
  float2 rowinfo[kMegaMaxRowsB];        // (scale, bias) of the rows of a mode-B phase
  float red[kCW];
  float bestv[kCW];
  int besti[kCW];
  int abort_flag;
  int last_flag;
  // attention fold (aacc is written with 16-byte stores)
  float am[kCW][8], al[kCW][8];
  alignas(16) float aacc[kCW][8][128];
};
static_assert(offsetof(Shared, aacc) % 16 == 0, "aacc must be 16-byte aligned");
static_assert(offsetof(Shared, rowinfo) % 8 == 0, "rowinfo must be 8-byte aligned");

struct Ctx {
  const MegaParams &p;
  Shared &sh;
  uint8_t *ring;
  volatile int *err;
  int ctid, lane, warp;
  uint32_t stage;     // running stage counter (same sequence as the producer's)
  unsigned epoch;     // grid barriers passed
  unsigned barrier_base;
};

// Optional per-phase timeline (SM clock) of a few CTAs, for tuning.
__device__ __forceinline__ void trace(Ctx &c, int layer, int slot) {
  if (c.p.trace != nullptr && c.ctid == 0 && (blockIdx.x % c.p.trace_stride) == 0)
    c.p.trace[((size_t)(blockIdx.x / c.p.trace_stride) * (c.p.L + 1) + layer) * 12 + slot] =
        clock64();
}

// Grid-wide barrier over the consumer warps of every CTA.  After a failure
// anywhere in the grid it degenerates to the CTA-local barriers.
__device__ void grid_barrier(Ctx &c) {
  ++c.epoch;
  consumer_sync();
  if (c.ctid == 0) {
    __threadfence();   // release: this CTA's writes (ordered by the CTA barrier) before the arrival
    red_relaxed(c.p.barrier, 1u);
    // the counter is never reset: this launch's arrivals start at barrier_base
    const unsigned target = c.barrier_base + c.epoch * gridDim.x;
    volatile int *ab = &c.sh.abort_flag;
    uint32_t it = 0;
    while (!*ab && (int)(ld_relaxed(c.p.barrier) - target) < 0) {
      if (++it >= kSpinLimit) {
        atomicCAS((int *)c.err, 0, 100 + (int)c.epoch);
        *ab = 1;
        break;
      }
      if ((it & 0xFFF) == 0 && *c.err != 0)
        *ab = 1;
    }
    __threadfence();   // acquire: other CTAs' writes are visible after the CTA barrier below
  }
  consumer_sync();
}

// ---- activation sources ----------------------------------------------------------
// kind 0: vector v (optionally RMSNorm'ed with weight nw); kind 1: silu(g)*u.
struct XSrc {
  int kind;
  const float *v, *nw, *g, *u;
};

__device__ __forceinline__ void load_x4(const XSrc &xs, int k, float *dst) {
  if (xs.kind == 0) {
    const float4 t = ldcg4(xs.v + k);
    dst[0] = t.x; dst[1] = t.y; dst[2] = t.z; dst[3] = t.w;
  } else {
    const float4 g = ldcg4(xs.g + k), u = ldcg4(xs.u + k);
    const float gs[4] = {g.x, g.y, g.z, g.w}, us[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      // subgraph0_decode_simplify.mlir:226-231: (g * sigmoid(g)) * u
      const float s = 1.0f / (1.0f + expf(-gs[e]));
      dst[e] = __fmul_rn(__fmul_rn(gs[e], s), us[e]);
    }
  }
}

// epilogue kinds
enum { EP_STORE = 0, EP_RESIDUAL = 1, EP_LOGITS = 2 };
struct Epi {
  int kind;
  float *dst;
  const float *res;
};

__device__ __forceinline__ void emit(const Epi &e, int n, float v, float &bestv, int &besti) {
  if (e.kind == EP_RESIDUAL) {
    e.dst[n] = __fadd_rn(__ldcg(e.res + n), v);
  } else {
    e.dst[n] = v;
    if (e.kind == EP_LOGITS && (v > bestv || (v == bestv && n < besti))) {
      bestv = v;
      besti = n;
    }
  }
}

// One projection.  Mode A (K <= 1536): a warp owns two rows of every slot,
// activations in 48 registers per lane; mode B: all consumer threads share
// each row and the per-warp partial sums meet in shared memory.
__device__ void gemv_phase(Ctx &c, const MegaPhase &ph, const XSrc &xs, const Epi &ep,
                           float &bestv, int &besti) {
  const MegaParams &p = c.p;
  int row_begin, nrows;
  rows_of(ph.N, blockIdx.x, gridDim.x, row_begin, nrows);
  float xr[3][16];
  const int K = ph.K;
  const int units = K / 16;

  // ---- activations into registers (same k permutation as the packed rows) ----
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < 3; ++i) {
    const int u = ph.mode == 0 ? (i * 32 + c.lane) : (i * kCT + c.ctid);
    const bool active = nrows > 0 && u < units;
#pragma unroll
    for (int e = 0; e < 16; ++e)
      xr[i][e] = 0.f;
    if (active) {
      const int b = u >> 5, l = u & 31;
      const int Bs = min(512, K - 512 * b), q = Bs >> 2;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        load_x4(xs, 512 * b + j * q + 4 * l, &xr[i][4 * j]);
#pragma unroll
        for (int e = 0; e < 4; ++e)
          ss = __fadd_rn(ss, __fmul_rn(xr[i][4 * j + e], xr[i][4 * j + e]));
      }
    }
  }
  if (xs.kind == 0 && xs.nw != nullptr) {
    // RMSNorm, subgraph0_decode_simplify.mlir:60-72
    ss = warp_sum(ss);
    if (ph.mode == 1) {
      if (c.lane == 0)
        c.sh.red[c.warp] = ss;
      consumer_sync();
      ss = 0.f;
#pragma unroll
      for (int w = 0; w < kCW; ++w)
        ss += c.sh.red[w];
      consumer_sync();
    }
    const float rinv = rsqrtf(__fadd_rn(__fmul_rn(ss, 1.0f / (float)K), p.eps));
#pragma unroll
    for (int i = 0; i < 3; ++i) {
      const int u = ph.mode == 0 ? (i * 32 + c.lane) : (i * kCT + c.ctid);
      if (nrows > 0 && u < units) {
        const int b = u >> 5, l = u & 31;
        const int Bs = min(512, K - 512 * b), q = Bs >> 2;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float4 w4 = __ldg(reinterpret_cast<const float4 *>(xs.nw + 512 * b + j * q + 4 * l));
          xr[i][4 * j + 0] = __fmul_rn(w4.x, __fmul_rn(xr[i][4 * j + 0], rinv));
          xr[i][4 * j + 1] = __fmul_rn(w4.y, __fmul_rn(xr[i][4 * j + 1], rinv));
          xr[i][4 * j + 2] = __fmul_rn(w4.z, __fmul_rn(xr[i][4 * j + 2], rinv));
          xr[i][4 * j + 3] = __fmul_rn(w4.w, __fmul_rn(xr[i][4 * j + 3], rinv));
        }
      }
    }
  }
  // offset term 128 * sum(x) of this thread's activations, then the 2^64 pre-scale
  float sx = 0.f;
#pragma unroll
  for (int i = 0; i < 3; ++i)
#pragma unroll
    for (int e = 0; e < 16; ++e) {
      sx += xr[i][e];
      xr[i][e] *= kXScale;
    }
  const float off = -128.0f * sx;

  // ---- stream the rows --------------------------------------------------------
  volatile int *ab = &c.sh.abort_flag;
  int flush_base = 0;
  for (int r0 = 0; r0 < nrows; r0 += ph.rps) {
    const int rows = min(ph.rps, nrows - r0);
    const int slot = c.stage % p.slots;
    const uint32_t use = c.stage / p.slots;
    if (!mbar_wait(&c.sh.full[slot], use & 1, c.err, ab))
      atomicCAS((int *)c.err, 0, 200 + slot);
    const uint8_t *base = c.ring + (size_t)slot * p.slot_bytes;
    if (ph.mode == 0) {
      // rows c.warp and c.warp + 8 of the slot; clamp keeps the loads inside the slot
      const int ra = c.warp, rb = c.warp + kCW;
      const uint8_t *rowa = base + (size_t)min(ra, rows - 1) * ph.row_bytes;
      const uint8_t *rowb = base + (size_t)min(rb, rows - 1) * ph.row_bytes;
      float a[4] = {0.f, 0.f, 0.f, 0.f}, b[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int i = 0; i < 3; ++i) {
        const int u = i * 32 + c.lane;
        if (u < units) {
          const uint4 wa = *reinterpret_cast<const uint4 *>(rowa + u * 16);
          const uint4 wb = *reinterpret_cast<const uint4 *>(rowb + u * 16);
          dot_unit(wa, xr[i], a);
          dot_unit(wb, xr[i], b);
        }
      }
      float va = fmaf((a[0] + a[1]) + (a[2] + a[3]), kAccScale, off);
      float vb = fmaf((b[0] + b[1]) + (b[2] + b[3]), kAccScale, off);
      va = warp_sum(va);
      vb = warp_sum(vb);
      if (c.lane == 0 && ra < rows) {
        const float2 t = *reinterpret_cast<const float2 *>(rowa + K);
        emit(ep, row_begin + r0 + ra, __fadd_rn(__fmul_rn(va, t.x), t.y), bestv, besti);
      }
      if (c.lane == 1 && rb < rows) {
        const float2 t = *reinterpret_cast<const float2 *>(rowb + K);
        emit(ep, row_begin + r0 + rb, __fadd_rn(__fmul_rn(vb, t.x), t.y), bestv, besti);
      }
    } else {
      for (int r = 0; r < rows; r += 2) {
        const uint8_t *rowa = base + (size_t)r * ph.row_bytes;
        const uint8_t *rowb = base + (size_t)min(r + 1, rows - 1) * ph.row_bytes;
        float a[4] = {0.f, 0.f, 0.f, 0.f}, b[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int i = 0; i < 3; ++i) {
          const int u = i * kCT + c.ctid;
          if (u < units) {
            const uint4 wa = *reinterpret_cast<const uint4 *>(rowa + u * 16);
            const uint4 wb = *reinterpret_cast<const uint4 *>(rowb + u * 16);
            dot_unit(wa, xr[i], a);
            dot_unit(wb, xr[i], b);
          }
        }
        float va = fmaf((a[0] + a[1]) + (a[2] + a[3]), kAccScale, off);
        float vb = fmaf((b[0] + b[1]) + (b[2] + b[3]), kAccScale, off);
        va = warp_sum(va);
        vb = warp_sum(vb);
        if (c.lane == 0) {
          c.sh.part[c.warp][r0 + r - flush_base] = va;
          if (r + 1 < rows)
            c.sh.part[c.warp][r0 + r + 1 - flush_base] = vb;
        }
        if (c.ctid == 0) {
          c.sh.rowinfo[r0 + r - flush_base] = *reinterpret_cast<const float2 *>(rowa + K);
          if (r + 1 < rows)
            c.sh.rowinfo[r0 + r + 1 - flush_base] = *reinterpret_cast<const float2 *>(rowb + K);
        }
      }
    }
    __syncwarp();
    if (c.lane == 0)
      mbar_arrive(&c.sh.empty[slot]);
    ++c.stage;
    if (ph.mode == 1) {
      const int pending = r0 + rows - flush_base;
      if (pending + ph.rps > kMegaMaxRowsB || r0 + rows >= nrows) {
        // fold the per-warp partial sums of the pending rows (fixed warp order)
        consumer_sync();
        if (c.ctid < pending) {
          float s = 0.f;
#pragma unroll
          for (int w = 0; w < kCW; ++w)
            s += c.sh.part[w][c.ctid];
          const float2 t = c.sh.rowinfo[c.ctid];
          emit(ep, row_begin + flush_base + c.ctid, __fadd_rn(__fmul_rn(s, t.x), t.y), bestv,
               besti);
        }
        consumer_sync();
        flush_base = r0 + rows;
      }
    }
  }
}

// ---- attention -------------------------------------------------------------------
// Work item = (kv head, split).  The CTA applies (QK-norm and) RoPE to the G
// query heads of its kv head, the CTA whose range holds `pos` also rotates the
// new key and writes the K/V row, every warp scans every 8th row of the range,
// the CTA folds its warps, and the last CTA of a kv head to arrive folds the
// splits (in split order, so the result does not depend on arrival order).
template <int G>
__device__ void attention_phase(Ctx &c, int layer, int pos) {
  const MegaParams &p = c.p;
  constexpr int D = 128;
  const int items = p.kvh * p.splits;
  if ((int)blockIdx.x >= items)
    return;
  const int hk = blockIdx.x / p.splits, split = blockIdx.x % p.splits;
  const int len = pos + 1;
  const int chunk = (len + p.splits - 1) / p.splits;
  const int s0 = split * chunk, s1 = min(len, s0 + chunk);
  const int lane = c.lane, warp = c.warp;
  const float *qn = p.lvec[4 * layer + 2], *kn = p.lvec[4 * layer + 3];
  float *kc = p.kv[2 * layer] + (size_t)hk * p.max_len * D;
  float *vc = p.kv[2 * layer + 1] + (size_t)hk * p.max_len * D;
  const float scale = rsqrtf((float)D);
  const int jj = 4 * (lane & 15);       // rotary index of this lane's 4 dims
  const bool upper = lane >= 16;

  auto rope4 = [&](float (&v)[4], const float *nw) {
    if (nw != nullptr) {
      float s = 0.f;
#pragma unroll
      for (int e = 0; e < 4; ++e)
        s = __fadd_rn(s, __fmul_rn(v[e], v[e]));
      s = warp_sum(s);
      const float r = rsqrtf(__fadd_rn(__fmul_rn(s, 1.0f / (float)D), p.eps));
      const float4 w4 = __ldg(reinterpret_cast<const float4 *>(nw + 4 * lane));
      v[0] = __fmul_rn(w4.x, __fmul_rn(v[0], r));
      v[1] = __fmul_rn(w4.y, __fmul_rn(v[1], r));
      v[2] = __fmul_rn(w4.z, __fmul_rn(v[2], r));
      v[3] = __fmul_rn(w4.w, __fmul_rn(v[3], r));
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float other = __shfl_xor_sync(0xffffffffu, v[e], 16);
      const float cs = c.sh.cs[jj + e], sn = c.sh.sn[jj + e];
      // lower half: x*cos + (-x[j+64])*sin ; upper half: x*cos + x[j-64]*sin
      v[e] = __fadd_rn(__fmul_rn(v[e], cs), __fmul_rn(upper ? other : -other, sn));
    }
  };

  // new K / V row (written by the CTA whose range contains pos)
  if (pos >= s0 && pos < s1 && warp == 0) {
    const float4 k4 = ldcg4(p.qkv + p.qh * D + hk * D + 4 * lane);
    const float4 v4 = ldcg4(p.qkv + p.qh * D + p.kvh * D + hk * D + 4 * lane);
    float kv[4] = {k4.x, k4.y, k4.z, k4.w};
    rope4(kv, kn);
    const float4 ko = make_float4(kv[0], kv[1], kv[2], kv[3]);
    *reinterpret_cast<float4 *>(kc + (size_t)pos * D + 4 * lane) = ko;
    *reinterpret_cast<float4 *>(vc + (size_t)pos * D + 4 * lane) = v4;
    float *ks = p.kv_stage + (size_t)(2 * layer) * p.kvh * D + hk * D;
    float *vs = p.kv_stage + (size_t)(2 * layer + 1) * p.kvh * D + hk * D;
    *reinterpret_cast<float4 *>(ks + 4 * lane) = ko;
    *reinterpret_cast<float4 *>(vs + 4 * lane) = v4;
  }
  float qr[G][4];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    const float4 q4 = ldcg4(p.qkv + (size_t)(hk * G + g) * D + 4 * lane);
    qr[g][0] = q4.x; qr[g][1] = q4.y; qr[g][2] = q4.z; qr[g][3] = q4.w;
    rope4(qr[g], qn);
  }
  consumer_sync();  // the new row is visible to the whole CTA

  float m[G], l[G], acc[G][4];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    m[g] = kSeed;
    l[g] = 0.f;
    acc[g][0] = acc[g][1] = acc[g][2] = acc[g][3] = 0.f;
  }
  for (int j = s0 + warp; j < s1; j += 2 * kCW) {
    // two rows per iteration: their loads, dots and reductions are independent
    const int j2 = j + kCW;
    const bool two = j2 < s1;
    const float4 ka = ldcg4(kc + (size_t)j * D + 4 * lane);
    const float4 va = ldcg4(vc + (size_t)j * D + 4 * lane);
    const float4 kb = ldcg4(kc + (size_t)(two ? j2 : j) * D + 4 * lane);
    const float4 vb = ldcg4(vc + (size_t)(two ? j2 : j) * D + 4 * lane);
    float sa[G], sb[G];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float d = qr[g][0] * ka.x;
      d = fmaf(qr[g][1], ka.y, d);
      d = fmaf(qr[g][2], ka.z, d);
      sa[g] = fmaf(qr[g][3], ka.w, d);
      float e = qr[g][0] * kb.x;
      e = fmaf(qr[g][1], kb.y, e);
      e = fmaf(qr[g][2], kb.z, e);
      sb[g] = fmaf(qr[g][3], kb.w, e);
    }
#pragma unroll
    for (int g = 0; g < G; ++g) {
      sa[g] = warp_sum(sa[g]) * scale;
      sb[g] = warp_sum(sb[g]) * scale;
    }
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const float nm = fmaxf(m[g], two ? fmaxf(sa[g], sb[g]) : sa[g]);
      const float alpha = expf(m[g] - nm), pa = expf(sa[g] - nm);
      const float pb = two ? expf(sb[g] - nm) : 0.f;
      l[g] = fmaf(l[g], alpha, pa + pb);
      acc[g][0] = fmaf(acc[g][0], alpha, fmaf(pa, va.x, pb * vb.x));
      acc[g][1] = fmaf(acc[g][1], alpha, fmaf(pa, va.y, pb * vb.y));
      acc[g][2] = fmaf(acc[g][2], alpha, fmaf(pa, va.z, pb * vb.z));
      acc[g][3] = fmaf(acc[g][3], alpha, fmaf(pa, va.w, pb * vb.w));
      m[g] = nm;
    }
  }
#pragma unroll
  for (int g = 0; g < G; ++g) {
    if (lane == 0) {
      c.sh.am[warp][g] = m[g];
      c.sh.al[warp][g] = l[g];
    }
    *reinterpret_cast<float4 *>(&c.sh.aacc[warp][g][4 * lane]) =
        make_float4(acc[g][0], acc[g][1], acc[g][2], acc[g][3]);
  }
  consumer_sync();
  const int stride = D + 2;
  for (int idx = c.ctid; idx < G * D; idx += kCT) {
    const int g = idx / D, d = idx - g * D;
    float M = kSeed;
#pragma unroll
    for (int w = 0; w < kCW; ++w)
      M = fmaxf(M, c.sh.am[w][g]);
    float L = 0.f, A = 0.f;
#pragma unroll
    for (int w = 0; w < kCW; ++w) {
      const float b = expf(c.sh.am[w][g] - M);
      L = fmaf(c.sh.al[w][g], b, L);
      A = fmaf(c.sh.aacc[w][g][d], b, A);
    }
    float *part = p.attn_part + ((size_t)(hk * G + g) * p.splits + split) * stride;
    part[d] = A;
    if (d == 0) {
      part[D] = M;
      part[D + 1] = L;
    }
  }
  __threadfence();
  consumer_sync();
  if (c.ctid == 0) {
    const unsigned done = atomicAdd(&p.attn_count[hk], 1u);
    c.sh.last_flag = (done == (unsigned)p.splits - 1);
    if (c.sh.last_flag)
      p.attn_count[hk] = 0;
  }
  consumer_sync();
  if (c.sh.last_flag) {
    __threadfence();
    // fold the splits of this kv head (frontend/Python/ops/tosa.py:14502-14594):
    // weights exp(m_s - M) once per (head, split), then sums with independent loads
    const int S = p.splits;
    float *wts = &c.sh.aacc[0][0][0];           // [G][S] weights, then [G] totals
    for (int idx = c.ctid; idx < G * S; idx += kCT) {
      const int g = idx / S, sidx = idx - g * S;
      const float *part = p.attn_part + ((size_t)(hk * G + g) * S + sidx) * stride;
      c.sh.aacc[1][0][idx] = __ldcg(part + D);        // m
      c.sh.aacc[2][0][idx] = __ldcg(part + D + 1);    // l
    }
    consumer_sync();
    if (c.ctid < G) {
      const int g = c.ctid;
      float M = kSeed;
      for (int sidx = 0; sidx < S; ++sidx)
        M = fmaxf(M, c.sh.aacc[1][0][g * S + sidx]);
      float L = 0.f;
      for (int sidx = 0; sidx < S; ++sidx) {
        const float b = expf(c.sh.aacc[1][0][g * S + sidx] - M);
        wts[g * S + sidx] = b;
        L = fmaf(c.sh.aacc[2][0][g * S + sidx], b, L);
      }
      c.sh.aacc[3][0][g] = L;
    }
    consumer_sync();
    for (int idx = c.ctid; idx < G * D; idx += kCT) {
      const int g = idx / D, d = idx - g * D;
      const float *parts = p.attn_part + (size_t)(hk * G + g) * S * stride + d;
      float ar = 0.f;
#pragma unroll 8
      for (int sidx = 0; sidx < S; ++sidx)
        ar = fmaf(__ldcg(parts + (size_t)sidx * stride), wts[g * S + sidx], ar);
      p.attn[(size_t)(hk * G + g) * D + d] = __fdiv_rn(ar, c.sh.aacc[3][0][g]);
    }
  }
}

__device__ void attention_dispatch(Ctx &c, int layer, int pos) {
  switch (c.p.qh / c.p.kvh) {
  case 1: attention_phase<1>(c, layer, pos); break;
  case 2: attention_phase<2>(c, layer, pos); break;
  case 4: attention_phase<4>(c, layer, pos); break;
  case 6: attention_phase<6>(c, layer, pos); break;
  case 8: attention_phase<8>(c, layer, pos); break;
  default: break;  // rejected on the host
  }
}

} // namespace

__global__ void __launch_bounds__(kMegaThreads, 1) decode_step_kernel(const MegaParams p) {
  extern __shared__ __align__(128) uint8_t smem_raw[];
  Shared &sh = *reinterpret_cast<Shared *>(smem_raw);
  uint8_t *ring = smem_raw + ((sizeof(Shared) + 127) / 128) * 128;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int *err = p.error;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.slots; ++s) {
      mbar_init(&sh.full[s], 1);
      mbar_init(&sh.empty[s], kCW);
    }
    sh.abort_flag = 0;
    sh.last_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  const int token = p.state[0], pos = p.state[1];
  if (threadIdx.x < p.D / 2) {
    // subgraph0_decode_simplify.mlir:52-59
    const float th = __fmul_rn(__ldg(p.inv_freq + threadIdx.x), (float)pos);
    sh.cs[threadIdx.x] = cosf(th);
    sh.sn[threadIdx.x] = sinf(th);
  }
  __syncthreads();

  if (warp == kCW) {
    // ================= producer: walk this CTA's weight stream =================
    if (lane == 0) {
      const uint8_t *src = p.stream + p.cta_off[blockIdx.x];
      uint32_t g = 0;
      bool ok = true;
      for (int l = 0; l <= p.L && ok; ++l) {
        const int np = l < p.L ? 4 : 1;
        for (int pi = 0; pi < np && ok; ++pi) {
          const MegaPhase &ph = p.phase[l < p.L ? pi : 4];
          int rb, nrows;
          rows_of(ph.N, blockIdx.x, gridDim.x, rb, nrows);
          for (int r0 = 0; r0 < nrows; r0 += ph.rps) {
            const uint32_t bytes = (uint32_t)min(ph.rps, nrows - r0) * ph.row_bytes;
            const int slot = g % p.slots;
            const uint32_t use = g / p.slots;
            if (!mbar_wait(&sh.empty[slot], (use & 1) ^ 1, err, &sh.abort_flag)) {
              atomicCAS((int *)err, 0, 300 + slot);
              ok = false;
              break;
            }
            mbar_expect_tx(&sh.full[slot], bytes);
            bulk_g2s(ring + (size_t)slot * p.slot_bytes, src, bytes, &sh.full[slot]);
            src += bytes;
            ++g;
          }
        }
      }
      // never leave with copies of this CTA still in flight
      const uint32_t first = g > (uint32_t)p.slots ? g - p.slots : 0;
      for (uint32_t s = first; s < g; ++s) {
        uint32_t it = 0;
        while (!mbar_try_wait(&sh.full[s % p.slots], (s / p.slots) & 1) && ++it < (1u << 20)) {
        }
      }
    }
    return;
  }

  // ================= consumers ===================================================
  const unsigned barriers_per_launch = 5u * (unsigned)p.L + 1u;
  Ctx c{p, sh, ring, err, (int)threadIdx.x, lane, warp, 0u, 0u,
        (unsigned)p.state[4] * barriers_per_launch * gridDim.x};
  float bestv = -INFINITY;
  int besti = 0x7fffffff;
  const float *x_in = p.embed + (size_t)token * p.H;   // residual stream entering the layer
  for (int l = 0; l < p.L; ++l) {
    const float *in_norm = p.lvec[4 * l], *post_norm = p.lvec[4 * l + 1];
    trace(c, l, 0);
    {  // q | k | v  (+ bias) <- RMSNorm(x)
      const XSrc xs{0, x_in, in_norm, nullptr, nullptr};
      const Epi ep{EP_STORE, p.qkv, nullptr};
      gemv_phase(c, p.phase[0], xs, ep, bestv, besti);
    }
    trace(c, l, 1);
    grid_barrier(c);
    trace(c, l, 2);
    attention_dispatch(c, l, pos);
    trace(c, l, 3);
    grid_barrier(c);
    trace(c, l, 4);
    {  // x1 = x + attn @ Wo
      const XSrc xs{0, p.attn, nullptr, nullptr, nullptr};
      const Epi ep{EP_RESIDUAL, p.xb, x_in};
      gemv_phase(c, p.phase[1], xs, ep, bestv, besti);
    }
    trace(c, l, 5);
    grid_barrier(c);
    trace(c, l, 6);
    {  // gate | up <- RMSNorm(x1)
      const XSrc xs{0, p.xb, post_norm, nullptr, nullptr};
      const Epi ep{EP_STORE, p.gu, nullptr};
      gemv_phase(c, p.phase[2], xs, ep, bestv, besti);
    }
    trace(c, l, 7);
    grid_barrier(c);
    trace(c, l, 8);
    {  // x2 = x1 + (silu(gate) * up) @ Wdown
      const XSrc xs{1, nullptr, nullptr, p.gu, p.gu + p.F};
      const Epi ep{EP_RESIDUAL, p.xa, p.xb};
      gemv_phase(c, p.phase[3], xs, ep, bestv, besti);
    }
    trace(c, l, 9);
    grid_barrier(c);
    trace(c, l, 10);
    x_in = p.xa;
  }
  {  // logits <- RMSNorm(x) @ lm_head, with a running first-max
    const XSrc xs{0, x_in, p.final_norm, nullptr, nullptr};
    const Epi ep{EP_LOGITS, p.logits, nullptr};
    bestv = -INFINITY;
    besti = 0x7fffffff;
    trace(c, p.L, 0);
    gemv_phase(c, p.phase[4], xs, ep, bestv, besti);
    trace(c, p.L, 1);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bestv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, besti, o);
      if (ov > bestv || (ov == bestv && oi < besti)) {
        bestv = ov;
        besti = oi;
      }
    }
    if (c.lane == 0) {
      sh.bestv[c.warp] = bestv;
      sh.besti[c.warp] = besti;
    }
    consumer_sync();
    if (c.ctid == 0) {
      for (int w = 1; w < kCW; ++w)
        if (sh.bestv[w] > bestv || (sh.bestv[w] == bestv && sh.besti[w] < besti)) {
          bestv = sh.bestv[w];
          besti = sh.besti[w];
        }
      p.cand_val[blockIdx.x] = bestv;
      p.cand_idx[blockIdx.x] = besti;
    }
    grid_barrier(c);
  }
  if (blockIdx.x == 0 && c.warp == 0 && sh.abort_flag == 0) {
    // Sampler.h:101-104: first maximum
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = c.lane; i < (int)gridDim.x; i += 32) {
      const float v = __ldcg(p.cand_val + i);
      const int ix = __ldcg(p.cand_idx + i);
      if (v > bv || (v == bv && ix < bi)) {
        bv = v;
        bi = ix;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) {
        bv = ov;
        bi = oi;
      }
    }
    if (c.lane == 0) {
      const int next = bi == 0x7fffffff ? 0 : bi;
      const int cnt = p.state[3];
      if (cnt < p.history_cap)
        p.history[cnt] = next;
      p.state[3] = cnt + 1;
      p.state[2] = next;
      p.state[0] = next;
      p.state[1] = pos + 1;
      p.state[4] = p.state[4] + 1;   // launches completed (base of the barrier counter)
    }
  }
}

// ---- stream builder: packed rows of one projection -> per-CTA streams ---------------
// One CTA per source row: copies its K packed bytes and appends the 16-byte
// trailer {scale, bias, 0, 0}.  The source holds rows [row_offset,
// row_offset + gridDim.x) of a projection with N_total rows.
__global__ void mega_build_rows_kernel(const uint8_t *src, int K, int row_offset, int N_total,
                                       const float *scale, const float *bias, int grid_ctas,
                                       int row_bytes, const int64_t *cta_phase_off,
                                       uint8_t *stream) {
  const int n = blockIdx.x + row_offset;
  const int base = N_total / grid_ctas, rem = N_total % grid_ctas;
  // owner CTA of row n under rows_of()
  int cta;
  const int split = rem * (base + 1);
  if (n < split)
    cta = n / (base + 1);
  else
    cta = rem + (n - split) / base;
  const int begin = cta * base + min(cta, rem);
  uint8_t *dst = stream + cta_phase_off[cta] + (int64_t)(n - begin) * row_bytes;
  const uint4 *s4 = reinterpret_cast<const uint4 *>(src + (int64_t)blockIdx.x * K);
  uint4 *d4 = reinterpret_cast<uint4 *>(dst);
  for (int i = threadIdx.x; i < K / 16; i += blockDim.x) {
    uint4 v = s4[i];   // int8 q -> u = q + 128
    v.x ^= 0x80808080u; v.y ^= 0x80808080u; v.z ^= 0x80808080u; v.w ^= 0x80808080u;
    d4[i] = v;
  }
  if (threadIdx.x == 0)
    *reinterpret_cast<float4 *>(dst + K) =
        make_float4(scale[blockIdx.x], bias ? bias[blockIdx.x] : 0.f, 0.f, 0.f);
}

int mega_build_rows(const void *packed, int K, int n_rows, int row_offset, int N_total,
                    const float *scale, const float *bias, int grid_ctas, int row_bytes,
                    const int64_t *cta_phase_off_dev, void *stream_buf, cudaStream_t st) {
  mega_build_rows_kernel<<<n_rows, 128, 0, st>>>((const uint8_t *)packed, K, row_offset, N_total,
                                                 scale, bias, grid_ctas, row_bytes,
                                                 cta_phase_off_dev, (uint8_t *)stream_buf);
  B200_LAUNCH_CHECK();
  return B200_OK;
}

size_t mega_shared_bytes(int slots, int slot_bytes) {
  return ((sizeof(Shared) + 127) / 128) * 128 + (size_t)slots * slot_bytes;
}

int mega_launch(const MegaParams &p, int grid, size_t smem, cudaStream_t st) {
  static bool configured = false;
  if (!configured) {
    B200_CUDA(cudaFuncSetAttribute(decode_step_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   227 * 1024));
    configured = true;
  }
  void *args[] = {(void *)&p};
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kMegaThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;   // all CTAs co-resident, or the launch fails
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  B200_CUDA(cudaLaunchKernelExC(&cfg, (const void *)decode_step_kernel, args));
  count_launch();
  return B200_OK;
}

} // namespace b200

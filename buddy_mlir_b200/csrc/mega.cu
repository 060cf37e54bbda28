// One persistent kernel per decode token (batch 1, int8 weight-only).
//
// Why: at batch 1 a decode step of the 1.5B model is 140 dependent GEMVs of
// 0.4-2 us each; launched one by one (even from a CUDA graph) every kernel
// boundary drains the memory pipeline.  Here one CTA per SM stays resident for
// the whole token.
//
//  * Weights.  Each CTA owns a fixed slice of the output rows of every
//    projection, and ALL weight bytes that CTA will ever need are laid out back
//    to back in one private stream (built once at load time).  The stream is
//    pulled with bulk async copies (cp.async.bulk, completion on mbarriers)
//    into a ring of shared-memory slots; the warp that finishes a slot last
//    immediately refills it with the stage one ring-length ahead.  Refills never
//    wait for activations, so HBM stays busy across the dependency points of
//    the graph (the ring holds about one projection's worth of weights).
//  * Activations.  There is no grid-wide barrier.  Every activation vector
//    that crosses CTAs (q|k|v, attention output, the two residual streams, the
//    SiLU-gated MLP intermediate, attention split partials, argmax candidates)
//    is stored as 8-byte (value, tag) pairs written with one 64-bit store; the
//    tag names launch, layer and producer phase.  A consumer simply loads the
//    pairs it needs and retries until the tags match: data arrival IS the
//    synchronisation (no fence, no counter, no barrier), and CTAs drift apart
//    by at most one phase because every phase needs all outputs of the one
//    before.  Buffers alternate by layer parity, so a producer can never
//    overwrite a value a slower CTA still has to read.
//  * Math.  Sixteen warps dequantise from shared memory with the activations
//    in registers and meet in warp-shuffle reductions; groups of warps work on
//    different ring slots at the same time.
//
// Every wait (mbarrier or tag poll) is bounded: on expiry the kernel records an
// error code, all later waits fall through, control flow stays identical (so
// CTA barriers stay matched), and the host call fails.
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

constexpr int kCW = 16;           // warps (all of them consume)
constexpr int kCT = kCW * 32;     // threads
constexpr int kAW = 7;            // warps that scan the KV cache in the attention phase
constexpr uint32_t kSpinLimit = 1u << 26;      // poll count bound, and
constexpr unsigned long long kWaitNs = 1000000000ull;  // wall-time bound (1 s) of any single wait
__device__ __forceinline__ unsigned long long now_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
constexpr float kSeed = -1.0e30f;
constexpr int D = 128;            // head_dim (checked on the host)

// producer phases that tag their outputs
enum { T_QKV = 1, T_ATTN = 2, T_XB = 3, T_MID = 4, T_XA = 5, T_PART = 6, T_CAND = 7 };

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
// Bounded wait.  Returns false when it gave up or the CTA is already in the
// failed state; callers carry on with the same control flow.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, volatile int *err,
                                          volatile int *abort_flag) {
  if (*abort_flag)
    return false;
  unsigned long long t0 = 0;
  for (uint32_t it = 0; it < kSpinLimit; ++it) {
    if (mbar_try_wait(bar, parity))
      return true;
    if ((it & 0x3FF) == 0x3FF) {
      if (*err != 0)
        break;
      const unsigned long long t = now_ns();
      if (t0 == 0)
        t0 = t;
      else if (t - t0 > kWaitNs)
        break;
    }
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
__device__ __forceinline__ float4 ldcg4(const float *p) {
  return __ldcg(reinterpret_cast<const float4 *>(p));
}

// ---- tagged (value, tag) pairs ------------------------------------------------------
__device__ __forceinline__ void ll_store(uint2 *p, float v, uint32_t tag) {
  asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(__float_as_uint(v)),
               "r"(tag)
               : "memory");
}
__device__ __forceinline__ uint2 ll_load1(const uint2 *p) {
  uint2 v;
  asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
  return v;
}
// two consecutive pairs (p is 16-byte aligned)
__device__ __forceinline__ uint4 ll_load2(const uint2 *p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}

// Where stage g of this CTA's stream lives: stages per projection, rows, bytes.
struct StreamPlan {
  int n[5];            // stages of projection p in one layer (p = 4: lm_head)
  int rows[5];         // rows of projection p owned by this CTA
  int rps[5], row_bytes[5];
  long long off[5];    // byte offset of projection p inside a layer's part of the stream
  long long layer_bytes;
  int per_layer;       // stages per layer
  int total;           // stages per token
  int L;
  uint2 tab[kMegaMaxLayerStages];   // stage r of a layer: (byte offset inside the layer's part, bytes)
  int next_l[kMegaMaxSlots], next_r[kMegaMaxSlots];   // per ring slot: the stage it receives next
};

struct Shared {
  uint64_t full[kMegaMaxSlots];
  int done[kMegaMaxSlots];              // warps that finished the slot's current stage
  int issued[kMegaMaxSlots];            // stage last requested into the slot
  StreamPlan plan;
  const uint8_t *stream_base;
  float cs[64], sn[64];                 // cos / sin of this step's position
  float red[kCW], red2[kCW];
  float bestv[kCW];
  int besti[kCW];
  int abort_flag;
  float am[kAW][8], al[kAW][8];         // attention: per-warp (m, l)
  float fw[8 * kAW], fm[8];             // attention: fold of the warps (weights, m per head)
};

struct Ctx {
  const MegaParams &p;
  Shared &sh;
  float *xs;          // staged activations (shared memory)
  uint8_t *ring;
  volatile int *err;
  int ctid, lane, warp;
  int slot;           // ring slot of the next stage
  uint32_t parity;    // parity of that slot's current use
  int g;              // index of the next stage in this CTA's stream
  uint32_t tag_base;
  long long *tr;      // this CTA's trace rows, or null
};

__device__ __forceinline__ uint32_t tag_of(const Ctx &c, int layer, int what) {
  return c.tag_base + (uint32_t)((layer + 1) * 8 + what);
}

// Spin (bounded) until the pair at p carries `tag`.
__device__ __forceinline__ float ll_wait1(Ctx &c, const uint2 *p, uint32_t tag) {
  volatile int *ab = &c.sh.abort_flag;
  uint2 v = ll_load1(p);
  uint32_t it = 0;
  unsigned long long t0 = 0;
  while (v.y != tag && !*ab) {
    bool give_up = ++it >= kSpinLimit;
    if ((it & 0x3FF) == 0) {
      const unsigned long long t = now_ns();
      if (t0 == 0)
        t0 = t;
      give_up = give_up || *c.err != 0 || t - t0 > kWaitNs;
    }
    if (give_up) {
      atomicCAS((int *)c.err, 0, 400 + (int)(tag & 7));
      *ab = 1;
      break;
    }
    __nanosleep(it < 4 ? 40 : 200);   // keep the pollers of 148 CTAs from flooding L2
    v = ll_load1(p);
  }
  return __uint_as_float(v.x);
}
__device__ __forceinline__ uint4 ll_wait2(Ctx &c, const uint2 *p, uint32_t tag, uint4 v) {
  volatile int *ab = &c.sh.abort_flag;
  uint32_t it = 0;
  unsigned long long t0 = 0;
  while ((v.y != tag || v.w != tag) && !*ab) {
    bool give_up = ++it >= kSpinLimit;
    if ((it & 0x3FF) == 0) {
      const unsigned long long t = now_ns();
      if (t0 == 0)
        t0 = t;
      give_up = give_up || *c.err != 0 || t - t0 > kWaitNs;
    }
    if (give_up) {
      atomicCAS((int *)c.err, 0, 400 + (int)(tag & 7));
      *ab = 1;
      break;
    }
    __nanosleep(it < 4 ? 40 : 200);   // keep the pollers of 148 CTAs from flooding L2
    v = ll_load2(p);
  }
  return v;
}

constexpr float kXScale = 18446744073709551616.0f;          // 2^64
constexpr float kAccScale = 38685626227668133590597632.0f;  // 2^85
// Cooperative load of n activations (n even) into shared memory, ready for the
// row loops: multiplied by the RMSNorm weight (if any) and by 2^64.  `ss`
// receives this thread's share of sum(x^2) (of the raw values), `sx` its share
// of sum(x * weight).  The first vector of every thread is polled alone (cheap
// on L2) before the rest is requested.
__device__ __forceinline__ void put2(float *dst, const float *nw, int e, float a, float b, float &ss,
                                     float &sx) {
  ss = __fadd_rn(ss, __fmul_rn(a, a));
  ss = __fadd_rn(ss, __fmul_rn(b, b));
  if (nw != nullptr) {
    const float2 w = __ldg(reinterpret_cast<const float2 *>(nw + e));
    a = __fmul_rn(a, w.x);
    b = __fmul_rn(b, w.y);
  }
  sx += a + b;
  *reinterpret_cast<float2 *>(dst + e) = make_float2(a * kXScale, b * kXScale);
}
__device__ __forceinline__ void stage_tagged(Ctx &c, const uint2 *src, uint32_t tag, int n, float *dst,
                                             const float *nw, float &ss, float &sx) {
  const int nv = n >> 1;
  for (int base = 0; base < nv; base += kCT * 4) {
    uint4 r[4];
    int idx[4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
      idx[i] = base + i * kCT + c.ctid;
    if (idx[0] < nv) {
      r[0] = ll_load2(src + 2 * idx[0]);
      r[0] = ll_wait2(c, src + 2 * idx[0], tag, r[0]);
    }
#pragma unroll
    for (int i = 1; i < 4; ++i)
      if (idx[i] < nv)
        r[i] = ll_load2(src + 2 * idx[i]);
#pragma unroll
    for (int i = 0; i < 4; ++i)
      if (idx[i] < nv) {
        if (i > 0)
          r[i] = ll_wait2(c, src + 2 * idx[i], tag, r[i]);
        put2(dst, nw, 2 * idx[i], __uint_as_float(r[i].x), __uint_as_float(r[i].z), ss, sx);
      }
  }
}
__device__ __forceinline__ void stage_plain(Ctx &c, const float *src, int n, float *dst, const float *nw,
                                            float &ss, float &sx) {
  for (int i = c.ctid * 2; i < n; i += kCT * 2) {
    const float2 v = __ldg(reinterpret_cast<const float2 *>(src + i));
    put2(dst, nw, i, v.x, v.y, ss, sx);
  }
}

// Streamed rows hold u = q + 128 (the int8 weight with its sign bit flipped).
// A byte left in place inside an otherwise zeroed word IS a float: bits 0-7
// give u * 2^-149 (a denormal), bits 8-15 give u * 2^-141, bits 16-23 give
// u * 2^-133 (the step from denormal to normal numbers is continuous), and
// the top byte shifted down gives u * 2^-149 again.  So the dequantisation of
// a weight is ONE logic op (LOP3 / SHF) and its multiply-accumulate one FFMA.
// The four byte positions accumulate separately and are rescaled when they are
// added up.  The activations are pre-scaled by 2^64 to keep every product in
// the normal range (a product is exact up to the single rounding of the FMA),
// and the offset 128 * sum(x) is subtracted once per row:
//   sum x*q = 2^85 * (a0 + a1*2^-8 + a2*2^-16 + a3) - 128 * sum x.
__device__ __forceinline__ void dot_unit(const uint4 &w, const float (&x)[16], float (&a)[4]) {
  const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    a[0] = fmaf(x[4 * j + 0], __uint_as_float(ws[j] & 0x000000FFu), a[0]);
    a[1] = fmaf(x[4 * j + 1], __uint_as_float(ws[j] & 0x0000FF00u), a[1]);
    a[2] = fmaf(x[4 * j + 2], __uint_as_float(ws[j] & 0x00FF0000u), a[2]);
    a[3] = fmaf(x[4 * j + 3], __uint_as_float(ws[j] >> 24), a[3]);
  }
}
// a0 + a1 * 2^-8 + a2 * 2^-16 + a3 (the scalings are exact)
__device__ __forceinline__ float dot_total(const float (&a)[4]) {
  return (a[0] + a[3]) + fmaf(a[1], 0.00390625f, a[2] * 0.0000152587890625f);
}

__device__ __forceinline__ void rows_of(const MegaPhase &ph, int cta, int grid, int &begin,
                                        int &count) {
  // rows are dealt out in units of ph.unit rows (2 keeps gate/up pairs together)
  const int n = ph.N / ph.unit;
  const int base = n / grid, rem = n % grid;
  begin = (cta * base + min(cta, rem)) * ph.unit;
  count = (base + (cta < rem ? 1 : 0)) * ph.unit;
}

// Request stage g of this CTA's stream into ring slot `slot` (one thread).  A slot
// receives stages slot, slot + n_slots, .. in order, so its cursor (layer, stage
// within the layer) only ever moves forward by n_slots; the per-layer table
// turns the cursor into (address, bytes) without divisions.
__device__ __forceinline__ void issue_stage(Shared &sh, uint8_t *ring, int slot_bytes, int slot,
                                            int g, int n_slots) {
  StreamPlan &pl = sh.plan;
  if (g >= pl.total)
    return;
  int l = pl.next_l[slot], r = pl.next_r[slot];
  const uint8_t *src;
  uint32_t bytes;
  if (l < pl.L) {
    const uint2 e = pl.tab[r];
    src = sh.stream_base + (long long)l * pl.layer_bytes + e.x;
    bytes = e.y;
  } else {   // the lm_head follows the layers
    const int rows = min(pl.rps[4], pl.rows[4] - r * pl.rps[4]);
    bytes = (uint32_t)rows * pl.row_bytes[4];
    src = sh.stream_base + (long long)pl.L * pl.layer_bytes + (long long)r * pl.rps[4] * pl.row_bytes[4];
  }
  *(volatile int *)&sh.issued[slot] = g;
  mbar_expect_tx(&sh.full[slot], bytes);
  bulk_g2s(ring + (size_t)slot * slot_bytes, src, bytes, &sh.full[slot]);
  r += n_slots;
  while (l < pl.L && r >= pl.per_layer) {
    r -= pl.per_layer;
    ++l;
  }
  pl.next_l[slot] = l;
  pl.next_r[slot] = r;
}

// Wait until stage `want` has landed in `slot`.  The parity of an mbarrier only
// tells consecutive uses of a slot apart; warp groups work on different stages
// and can run more than one use ahead of the group that still owns the slot, so
// the wait first makes sure the slot has been re-requested for the wanted stage.
__device__ __forceinline__ bool stage_wait(Shared &sh, int slot, uint32_t parity, int want,
                                           volatile int *err, volatile int *ab) {
  volatile int *iq = &sh.issued[slot];
  if (*iq != want) {
    unsigned long long t0 = 0;
    uint32_t it = 0;
    while (*iq != want && !*ab) {
      if ((++it & 0x3FF) == 0) {
        const unsigned long long t = now_ns();
        if (t0 == 0)
          t0 = t;
        if (*err != 0 || t - t0 > kWaitNs) {
          *ab = 1;
          break;
        }
      }
    }
  }
  return mbar_wait(&sh.full[slot], parity, err, ab);
}

// Optional per-phase timeline (SM clock) of a few CTAs, for tuning.
__device__ __forceinline__ void trace(Ctx &c, int layer, int slot) {
  if (c.tr != nullptr && c.ctid == 0)
    c.tr[layer * kMegaTraceSlots + slot] = clock64();
}

// ---- activation source / result sink of a projection -----------------------------
struct XSrc {
  const uint2 *ll;      // tagged source, or
  const float *plain;   // plain f32 source (the embedding row)
  uint32_t tag;
  const float *nw;      // RMSNorm weight or null
};
enum { EP_STORE = 0, EP_RESIDUAL = 1, EP_LOGITS = 2, EP_SILU = 3 };
struct Epi {
  int kind;
  uint2 *dst;
  uint32_t tag;
  const uint2 *res_ll;   // residual (tagged) or
  const float *res_plain;
  uint32_t res_tag;
  float *logits;
};

__device__ __forceinline__ void emit(Ctx &c, const Epi &e, int n, float v, float &bestv,
                                     int &besti) {
  if (e.kind == EP_RESIDUAL) {
    const float r = e.res_ll ? ll_wait1(c, e.res_ll + n, e.res_tag) : __ldg(e.res_plain + n);
    ll_store(e.dst + n, __fadd_rn(r, v), e.tag);
  } else if (e.kind == EP_LOGITS) {
    e.logits[n] = v;
    if (v > bestv || (v == bestv && n < besti)) {
      bestv = v;
      besti = n;
    }
  } else {
    ll_store(e.dst + n, v, e.tag);
  }
}
__device__ __forceinline__ float silu_mul(float g, float u) {
  // subgraph0_decode_simplify.mlir:226-231: (g * sigmoid(g)) * u
  const float s = 1.0f / (1.0f + expf(-g));
  return __fmul_rn(__fmul_rn(g, s), u);
}

// One visit of a warp to a ring stage: the warp takes rows R*wig .. R*wig+R-1 of
// the stage.  The activations come from shared memory (already normalised and
// scaled; four LDS.128 per 16-byte weight unit, shared by the R rows), so the
// loop needs few registers whatever K is.  The R row sums are reduced across
// the warp "transposed": at each of the first log2(R) steps a lane hands half of
// its rows to its partner, so R rows cost R + 4 - log2(R).. shuffles instead of
// 5 R, and every lane ends up with the total of ONE row:
//   R = 8: row (lane>>2)&7 with bit order (16, 8, 4);  R = 4: (16, 8);  R = 1: row 0.
template <int R>
__device__ __forceinline__ void visit_rows(Ctx &c, const Epi &ep, const uint8_t *base, int rows,
                                           int row_bytes, int K, int units, int wig, int lane,
                                           const float *xsm, float off, float rinv, int first_row,
                                           int local_row, float &bestv, int &besti) {
  int ro[R];   // byte offsets of the warp's rows (clamped: loads stay inside the stage)
  float a[R][4];
#pragma unroll
  for (int q = 0; q < R; ++q) {
    ro[q] = min(R * wig + q, rows - 1) * row_bytes + lane * 16;
    a[q][0] = a[q][1] = a[q][2] = a[q][3] = 0.f;
  }
  if (R == 1) {
    // a single row per warp: four 512-byte blocks in flight, each with its own
    // accumulators, so that the loads and the FMA chains of the blocks overlap
    float b[3][4];
#pragma unroll
    for (int s = 0; s < 3; ++s)
      b[s][0] = b[s][1] = b[s][2] = b[s][3] = 0.f;
#pragma unroll 1
    for (int i0 = 0; i0 * 32 < units; i0 += 4) {
#pragma unroll
      for (int s = 0; s < 4; ++s) {
        const int i = i0 + s;
        if (i * 32 + lane < units) {
          const int qd = min(512, K - 512 * i) >> 2;
          const float *xp = xsm + 512 * i + 4 * lane;
          float x[16];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float4 t = *reinterpret_cast<const float4 *>(xp + j * qd);
            x[4 * j + 0] = t.x; x[4 * j + 1] = t.y; x[4 * j + 2] = t.z; x[4 * j + 3] = t.w;
          }
          const uint4 w = *reinterpret_cast<const uint4 *>(base + ro[0] + i * 512);
          if (s == 0)
            dot_unit(w, x, a[0]);
          else
            dot_unit(w, x, b[s - 1]);
        }
      }
    }
#pragma unroll
    for (int e = 0; e < 4; ++e)
      a[0][e] = (a[0][e] + b[0][e]) + (b[1][e] + b[2][e]);
  } else {
#pragma unroll 3
    for (int i = 0; i * 32 < units; ++i) {   // K / 512 blocks of 32 sixteen-byte units (the last may be short)
      const int u = i * 32 + lane;
      if (u < units) {
        const int qd = min(512, K - 512 * i) >> 2;   // k distance between the unit's four groups
        const float *xp = xsm + 512 * i + 4 * lane;
        float x[16];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float4 t = *reinterpret_cast<const float4 *>(xp + j * qd);
          x[4 * j + 0] = t.x; x[4 * j + 1] = t.y; x[4 * j + 2] = t.z; x[4 * j + 3] = t.w;
        }
        uint4 w[R];
#pragma unroll
        for (int q = 0; q < R; ++q)
          w[q] = *reinterpret_cast<const uint4 *>(base + ro[q] + i * 512);
#pragma unroll
        for (int q = 0; q < R; ++q)
          dot_unit(w[q], x, a[q]);
      }
    }
  }
  float v[R];
#pragma unroll
  for (int q = 0; q < R; ++q)
    v[q] = dot_total(a[q]);
  float tot;
  int rowc;
  if (R == 8) {
    const bool b4 = lane & 16, b3 = lane & 8, b2 = lane & 4;
    float t[4], s2[2];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float got = __shfl_xor_sync(0xffffffffu, b4 ? v[q] : v[q + 4], 16);
      t[q] = (b4 ? v[q + 4] : v[q]) + got;
    }
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      const float got = __shfl_xor_sync(0xffffffffu, b3 ? t[q] : t[q + 2], 8);
      s2[q] = (b3 ? t[q + 2] : t[q]) + got;
    }
    const float got = __shfl_xor_sync(0xffffffffu, b2 ? s2[0] : s2[1], 4);
    tot = (b2 ? s2[1] : s2[0]) + got;
    tot += __shfl_xor_sync(0xffffffffu, tot, 2);
    tot += __shfl_xor_sync(0xffffffffu, tot, 1);
    rowc = (b4 ? 4 : 0) + (b3 ? 2 : 0) + (b2 ? 1 : 0);
  } else if (R == 4) {
    const bool b4 = lane & 16, b3 = lane & 8;
    float t[2];
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      const float got = __shfl_xor_sync(0xffffffffu, b4 ? v[q] : v[q + 2], 16);
      t[q] = (b4 ? v[q + 2] : v[q]) + got;
    }
    const float got = __shfl_xor_sync(0xffffffffu, b3 ? t[0] : t[1], 8);
    tot = (b3 ? t[1] : t[0]) + got;
    tot += __shfl_xor_sync(0xffffffffu, tot, 4);
    tot += __shfl_xor_sync(0xffffffffu, tot, 2);
    tot += __shfl_xor_sync(0xffffffffu, tot, 1);
    rowc = (b4 ? 2 : 0) + (b3 ? 1 : 0);
  } else {
    tot = v[0];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
      tot += __shfl_xor_sync(0xffffffffu, tot, o);
    rowc = 0;
  }
  constexpr int kOwnerMask = R == 8 ? 3 : (R == 4 ? 7 : 31);   // one lane per row finishes it
  const int row = R * wig + rowc;
  const int rclamp = min(row, rows - 1);
  const float2 tr = *reinterpret_cast<const float2 *>(base + (size_t)rclamp * row_bytes + K);
  // sum x*q = 2^85 * tot - 128 * sum x; the RMSNorm factor applies to the whole row
  const float dotv = __fmul_rn(fmaf(tot, kAccScale, off), rinv);
  const float val = __fadd_rn(__fmul_rn(dotv, tr.x), tr.y);
  if (ep.kind == EP_SILU) {
    // rows (2j, 2j+1) = (gate_j, up_j) sit in partner lanes
    const float upv = __shfl_xor_sync(0xffffffffu, val, R == 8 ? 4 : 8);
    if ((lane & kOwnerMask) == 0 && (rowc & 1) == 0 && row + 1 < rows)
      ll_store(ep.dst + ((first_row + row) >> 1), silu_mul(val, upv), ep.tag);
  } else if ((lane & kOwnerMask) == 0 && row < rows) {
    emit(c, ep, first_row + row, val, bestv, besti);
  }
}

// One projection with rows of K <= 1536 weights.  All rows of the CTA are
// streamed through the ring in stages of 16 rows; R rows per warp and visit:
// 8 for long phases (two warps per stage, eight stages in flight), 4 for the
// gate|up pairs of short phases, 1 when the whole phase is one or two stages
// (q|k|v, o: all 16 warps take one row each).
__device__ __forceinline__ void gemv_phase(Ctx &c, int phase_index, const XSrc &xs, const Epi &ep,
                                           int tl) {
  const MegaPhase &ph = c.p.phase[phase_index];
  int row_begin, nrows;
  rows_of(ph, blockIdx.x, gridDim.x, row_begin, nrows);
  const int K = ph.K, row_bytes = ph.row_bytes, rps = ph.rps;
  const int units = K / 16;
  const int n_slots = c.p.slots, slot_bytes = c.p.slot_bytes;
  const float eps = c.p.eps;
  Shared &sh = c.sh;
  const int lane = c.lane, warp = c.warp;
  uint8_t *const ring = c.ring;
  float *const xsm = c.xs;
  int slot = c.slot, g = c.g;
  uint32_t parity = c.parity;
  const int nstages = (nrows + rps - 1) / rps;
  // rows per warp and visit: 8 when a ring slot is left for each of the 8 stage groups
  const int R = rps < 16 ? 1
                         : (nstages >= 5 && n_slots >= 8 ? 8 : ((nstages >= 3 || ep.kind == EP_SILU) ? 4 : 1));
  const int gw = rps / R;            // warps per group (= per stage)
  const int NG = kCW / gw;           // stage groups
  const int grp = warp / gw, wig = warp - grp * gw;
  const int nrounds = (nstages + NG - 1) / NG;

  // ---- stage the activation vector in shared memory ----------------------------
  float ss = 0.f, sx = 0.f;
  if (xs.ll != nullptr)
    stage_tagged(c, xs.ll, xs.tag, K, xsm, xs.nw, ss, sx);
  else
    stage_plain(c, xs.plain, K, xsm, xs.nw, ss, sx);
  ss = warp_sum(ss);
  sx = warp_sum(sx);
  if (lane == 0) {
    sh.red[warp] = ss;
    sh.red2[warp] = sx;
  }
  consumer_sync();
  trace(c, tl, 12 + 4 * phase_index);
  float rinv = 1.f, off;
  {
    float t = 0.f, t2 = 0.f;
#pragma unroll
    for (int w = 0; w < kCW; ++w) {
      t += sh.red[w];
      t2 += sh.red2[w];
    }
    // RMSNorm, subgraph0_decode_simplify.mlir:60-72 (the factor multiplies the row sums)
    if (xs.nw != nullptr)
      rinv = rsqrtf(__fadd_rn(__fmul_rn(t, 1.0f / (float)K), eps));
    off = -128.0f * t2;
  }

  // ---- stream the rows --------------------------------------------------------
  volatile int *ab = &sh.abort_flag;
  float bestv = -INFINITY;
  int besti = 0x7fffffff;
  int my_slot = slot + grp;
  uint32_t my_par = parity;
  while (my_slot >= n_slots) {
    my_slot -= n_slots;
    my_par ^= 1u;
  }
  for (int rd = 0; rd < nrounds; ++rd) {
    const int st = rd * NG + grp;
    if (st < nstages) {
      const int r0 = st * rps;
      const int rows = min(rps, nrows - r0);
      if (!stage_wait(sh, my_slot, my_par, g + st, c.err, ab))
        atomicCAS((int *)c.err, 0, 200 + my_slot);
      const uint8_t *base = ring + (size_t)my_slot * slot_bytes;
      if (R == 8)
        visit_rows<8>(c, ep, base, rows, row_bytes, K, units, wig, lane, xsm, off, rinv,
                      row_begin + r0, r0, bestv, besti);
      else if (R == 4)
        visit_rows<4>(c, ep, base, rows, row_bytes, K, units, wig, lane, xsm, off, rinv,
                      row_begin + r0, r0, bestv, besti);
      else
        visit_rows<1>(c, ep, base, rows, row_bytes, K, units, wig, lane, xsm, off, rinv,
                      row_begin + r0, r0, bestv, besti);
      // Release the slot; the warp of the group that finishes it last refills it
      // with the stage one ring-length ahead.  (No fence on purpose: the slot's
      // bytes were consumed by arithmetic the values above depend on, so every
      // read has completed; the counter reset is ordered before the next use of
      // the slot by the arrival of that stage's data.)
      __syncwarp();
      if (lane == 0 && atomicAdd(&sh.done[my_slot], 1) == gw - 1) {
        sh.done[my_slot] = 0;
        issue_stage(sh, ring, slot_bytes, my_slot, g + st + n_slots, n_slots);
      }
    }
    my_slot += NG;
    while (my_slot >= n_slots) {
      my_slot -= n_slots;
      my_par ^= 1u;
    }
  }
  // this phase used `nstages` stages of the ring
  g += nstages;
  slot += nstages % n_slots;
  parity ^= (uint32_t)((nstages / n_slots) & 1);
  if (slot >= n_slots) {
    slot -= n_slots;
    parity ^= 1u;
  }
  c.slot = slot;
  c.parity = parity;
  c.g = g;
  if (ep.kind == EP_LOGITS) {
    // this warp's first maximum, for the CTA's candidate
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bestv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, besti, o);
      if (ov > bestv || (ov == bestv && oi < besti)) {
        bestv = ov;
        besti = oi;
      }
    }
    if (lane == 0) {
      sh.bestv[warp] = bestv;
      sh.besti[warp] = besti;
    }
  }
  // the staged vector is reused by the next phase
  consumer_sync();
}

// ---- attention -------------------------------------------------------------------
// Work item = (kv head, split).  The CTA stages q|k|v of its kv head, applies
// (QK-norm and) RoPE to the G query heads, the CTA whose range holds `pos` also
// rotates the new key and writes the K/V row; eight warps scan every 8th row of
// the range with several rows in flight; the CTA folds its warps and publishes the
// split partial; then every CTA of the kv head folds one slice of the outputs
// over all splits (in split order: the result does not depend on timing).
// Ask L2 for the cache rows this CTA will scan in the coming attention phase.
// Called before the q|k|v projection, so the rows arrive while it runs.
__device__ __forceinline__ void attention_prefetch(const Ctx &c, int layer, int pos) {
  const MegaParams &p = c.p;
  const int S = p.splits;
  if ((int)blockIdx.x >= p.kvh * S)
    return;
  const int hk = blockIdx.x / S, split = blockIdx.x % S;
  const int len = pos + 1;
  const int chunk = (len + S - 1) / S;
  const int s0 = split * chunk, s1 = min(pos, s0 + chunk);   // row `pos` is written this step
  const char *kc = reinterpret_cast<const char *>(p.kv[2 * layer] + ((size_t)hk * p.max_len + s0) * D);
  const char *vc = reinterpret_cast<const char *>(p.kv[2 * layer + 1] + ((size_t)hk * p.max_len + s0) * D);
  const int lines = (s1 - s0) * (D * 4 / 128);
  for (int i = c.ctid; i < lines; i += kCT) {
    asm volatile("prefetch.global.L2 [%0];" ::"l"(kc + (size_t)i * 128));
    asm volatile("prefetch.global.L2 [%0];" ::"l"(vc + (size_t)i * 128));
  }
}

template <int G>
__device__ __noinline__ void attention_phase(Ctx &c, int layer, int pos) {
  const MegaParams &p = c.p;
  const int S = p.splits;
  if ((int)blockIdx.x >= p.kvh * S)
    return;
  const int hk = blockIdx.x / S, split = blockIdx.x % S;
  const int len = pos + 1;
  const int chunk = (len + S - 1) / S;
  const int s0 = split * chunk, s1 = min(len, s0 + chunk);
  const int lane = c.lane, warp = c.warp;
  const int par = layer & 1;
  const int QD = p.qh * D, KD = p.kvh * D;
  const float *qn = p.lvec[4 * layer + 2], *kn = p.lvec[4 * layer + 3];
  float *kc = p.kv[2 * layer] + (size_t)hk * p.max_len * D;
  float *vc = p.kv[2 * layer + 1] + (size_t)hk * p.max_len * D;
  const float scale = rsqrtf((float)D);
  const int jj = 4 * (lane & 15);       // rotary index of this lane's 4 dims
  const bool upper = lane >= 16;
  const bool scanner = warp < kAW;      // warps 0..kAW-1 scan; warp kAW writes the new cache row
  const bool has_new = pos >= s0 && pos < s1;
  constexpr int NB = G <= 4 ? 4 : 2;    // rows in flight per warp (register budget: 128)

  // ---- request the first rows of this warp: they do not depend on this step
  //      (row `pos` is this step's own k / v and is taken from shared memory below)
  float4 kr[NB], vr[NB];
#pragma unroll
  for (int i = 0; i < NB; ++i) {
    const int j = s0 + warp + i * kAW;
    kr[i] = vr[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (scanner && j < s1 && j != pos) {
      kr[i] = ldcg4(kc + (size_t)j * D + 4 * lane);
      vr[i] = ldcg4(vc + (size_t)j * D + 4 * lane);
    }
  }

  // ---- stage q (G heads), k, v of this kv head: xs[0 .. (G+2)*D), q and k rotated ----
  // subgraph0_decode_simplify.mlir:111-150: out[j] = x[j]*cos - x[j+64]*sin,
  // out[j+64] = x[j+64]*cos + x[j]*sin.  Without QK-norm the thread that stages
  // elements (j, j+1) of a head also stages (j+64, j+65) and rotates both pairs.
  {
    const uint2 *src = p.ll_qkv + (size_t)par * (QD + 2 * KD);
    const uint32_t tag = tag_of(c, layer, T_QKV);
    const bool fused_rope = qn == nullptr && kn == nullptr;
    const int t = c.ctid;
    if (t < (G + 1) * (D / 4)) {
      const int hh = t / (D / 4), j = 2 * (t - hh * (D / 4));   // head (G = the key), pair index
      const int base = hh < G ? hk * G * D + hh * D : QD + hk * D;
      uint4 lo = ll_load2(src + base + j), hi = ll_load2(src + base + j + D / 2);
      lo = ll_wait2(c, src + base + j, tag, lo);
      hi = ll_wait2(c, src + base + j + D / 2, tag, hi);
      float x0 = __uint_as_float(lo.x), x1 = __uint_as_float(lo.z);
      float y0 = __uint_as_float(hi.x), y1 = __uint_as_float(hi.z);
      if (fused_rope) {
        const float c0 = c.sh.cs[j], c1 = c.sh.cs[j + 1], n0 = c.sh.sn[j], n1 = c.sh.sn[j + 1];
        const float a0 = __fadd_rn(__fmul_rn(x0, c0), __fmul_rn(-y0, n0));
        const float a1 = __fadd_rn(__fmul_rn(x1, c1), __fmul_rn(-y1, n1));
        const float b0 = __fadd_rn(__fmul_rn(y0, c0), __fmul_rn(x0, n0));
        const float b1 = __fadd_rn(__fmul_rn(y1, c1), __fmul_rn(x1, n1));
        x0 = a0; x1 = a1; y0 = b0; y1 = b1;
      }
      *reinterpret_cast<float2 *>(c.xs + hh * D + j) = make_float2(x0, x1);
      *reinterpret_cast<float2 *>(c.xs + hh * D + j + D / 2) = make_float2(y0, y1);
    } else if (t < (G + 1) * (D / 4) + D / 2) {
      const int j = 2 * (t - (G + 1) * (D / 4));
      const uint2 *sp = src + QD + KD + hk * D + j;
      uint4 r = ll_load2(sp);
      r = ll_wait2(c, sp, tag, r);
      *reinterpret_cast<float2 *>(c.xs + (G + 1) * D + j) = make_float2(__uint_as_float(r.x), __uint_as_float(r.z));
    }
    consumer_sync();
    if (!fused_rope) {
      // QK-norm first (needs the whole head): warp hh normalises and rotates head hh in place
      if (warp <= G) {
        const float4 x4 = *reinterpret_cast<const float4 *>(c.xs + warp * D + 4 * lane);
        float v[4] = {x4.x, x4.y, x4.z, x4.w};
        const float *nw = warp < G ? qn : kn;
        if (nw != nullptr) {
          float ss = 0.f;
#pragma unroll
          for (int e = 0; e < 4; ++e)
            ss = __fadd_rn(ss, __fmul_rn(v[e], v[e]));
          ss = warp_sum(ss);
          const float r = rsqrtf(__fadd_rn(__fmul_rn(ss, 1.0f / (float)D), p.eps));
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
          v[e] = __fadd_rn(__fmul_rn(v[e], cs), __fmul_rn(upper ? other : -other, sn));
        }
        *reinterpret_cast<float4 *>(c.xs + warp * D + 4 * lane) = make_float4(v[0], v[1], v[2], v[3]);
      }
      consumer_sync();
    }
  }
  // this step's own key (rotated) and value: used by the scanning warps of the CTA
  // whose range holds `pos`, written to the cache by warp kAW of that CTA
  float4 knew = make_float4(0.f, 0.f, 0.f, 0.f), vnew = knew;
  if (has_new && warp <= kAW) {
    knew = *reinterpret_cast<const float4 *>(c.xs + G * D + 4 * lane);
    vnew = *reinterpret_cast<const float4 *>(c.xs + (G + 1) * D + 4 * lane);
    if (warp == kAW) {
      *reinterpret_cast<float4 *>(kc + (size_t)pos * D + 4 * lane) = knew;
      *reinterpret_cast<float4 *>(vc + (size_t)pos * D + 4 * lane) = vnew;
      float *ks = p.kv_stage + (size_t)(2 * layer) * p.kvh * D + hk * D;
      float *vs = p.kv_stage + (size_t)(2 * layer + 1) * p.kvh * D + hk * D;
      *reinterpret_cast<float4 *>(ks + 4 * lane) = knew;
      *reinterpret_cast<float4 *>(vs + 4 * lane) = vnew;
    }
  }
  trace(c, layer, 8);

  float *aacc = c.xs + (G + 2) * D;   // [kAW][G][D], beside the staged q | k | v
  if (scanner) {
    float qr[G][4];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const float4 q4 = *reinterpret_cast<const float4 *>(c.xs + g * D + 4 * lane);
      qr[g][0] = q4.x; qr[g][1] = q4.y; qr[g][2] = q4.z; qr[g][3] = q4.w;
    }
    float m[G], l[G], acc[G][4];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      m[g] = kSeed;
      l[g] = 0.f;
      acc[g][0] = acc[g][1] = acc[g][2] = acc[g][3] = 0.f;
    }
    for (int j0 = s0 + warp; j0 < s1; j0 += NB * kAW) {
      if (j0 != s0 + warp) {
        // later rounds: NB rows in flight, all loads issued before the first use
#pragma unroll
        for (int i = 0; i < NB; ++i) {
          const int j = min(j0 + i * kAW, s1 - 1);
          if (j != pos) {
            kr[i] = ldcg4(kc + (size_t)j * D + 4 * lane);
            vr[i] = ldcg4(vc + (size_t)j * D + 4 * lane);
          }
        }
      }
#pragma unroll
      for (int i = 0; i < NB; ++i)
        if (j0 + i * kAW == pos) {
          kr[i] = knew;
          vr[i] = vnew;
        }
      float s[NB][G];
#pragma unroll
      for (int i = 0; i < NB; ++i)
#pragma unroll
        for (int g = 0; g < G; ++g) {
          float d = qr[g][0] * kr[i].x;
          d = fmaf(qr[g][1], kr[i].y, d);
          d = fmaf(qr[g][2], kr[i].z, d);
          s[i][g] = fmaf(qr[g][3], kr[i].w, d);
        }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1)   // the NB * G reductions advance together
#pragma unroll
        for (int i = 0; i < NB; ++i)
#pragma unroll
          for (int g = 0; g < G; ++g)
            s[i][g] += __shfl_xor_sync(0xffffffffu, s[i][g], o);
#pragma unroll
      for (int i = 0; i < NB; ++i)
#pragma unroll
        for (int g = 0; g < G; ++g)
          s[i][g] *= scale;
      // one softmax update for the NB rows (tosa.py:14245-14252 applied to a block):
      // rows beyond the range get weight 0.  __expf: the arguments are <= 0 and
      // the error (about 1e-6 relative) is far inside the logits tolerance.
#pragma unroll
      for (int g = 0; g < G; ++g) {
        float nm = m[g];
#pragma unroll
        for (int i = 0; i < NB; ++i)
          if (j0 + i * kAW < s1)
            nm = fmaxf(nm, s[i][g]);
        const float alpha = __expf(m[g] - nm);
        float pw[NB];
#pragma unroll
        for (int i = 0; i < NB; ++i)
          pw[i] = (j0 + i * kAW < s1) ? __expf(s[i][g] - nm) : 0.f;
        float ll = l[g] * alpha, a0 = acc[g][0] * alpha, a1 = acc[g][1] * alpha,
              a2 = acc[g][2] * alpha, a3 = acc[g][3] * alpha;
#pragma unroll
        for (int i = 0; i < NB; ++i) {
          ll += pw[i];
          a0 = fmaf(pw[i], vr[i].x, a0);
          a1 = fmaf(pw[i], vr[i].y, a1);
          a2 = fmaf(pw[i], vr[i].z, a2);
          a3 = fmaf(pw[i], vr[i].w, a3);
        }
        l[g] = ll;
        acc[g][0] = a0; acc[g][1] = a1; acc[g][2] = a2; acc[g][3] = a3;
        m[g] = nm;
      }
    }
    // publish this warp's state to the CTA
#pragma unroll
    for (int g = 0; g < G; ++g) {
      if (lane == 0) {
        c.sh.am[warp][g] = m[g];
        c.sh.al[warp][g] = l[g];
      }
      *reinterpret_cast<float4 *>(aacc + ((size_t)warp * G + g) * D + 4 * lane) =
          make_float4(acc[g][0], acc[g][1], acc[g][2], acc[g][3]);
    }
  }
  trace(c, layer, 9);
  consumer_sync();
  // ---- fold the warps of this CTA (fixed warp order) ------------------------------
  // weights of the scanning warps' states: thread (g, w) takes one
  if (c.ctid < G * kAW) {
    const int g = c.ctid / kAW, w = c.ctid - g * kAW;
    float M = kSeed;
#pragma unroll
    for (int x = 0; x < kAW; ++x)
      M = fmaxf(M, c.sh.am[x][g]);
    c.sh.fw[g * kAW + w] = expf(c.sh.am[w][g] - M);
    if (w == 0)
      c.sh.fm[g] = M;
  }
  consumer_sync();
  const int stride = D + 2;
  uint2 *part = p.ll_part + (size_t)par * p.qh * S * stride;
  const uint32_t ptag = tag_of(c, layer, T_PART);
  for (int idx = c.ctid; idx < G * D; idx += kCT) {
    const int g = idx / D, d = idx - g * D;
    float A = 0.f;
#pragma unroll
    for (int w = 0; w < kAW; ++w)
      A = fmaf(aacc[((size_t)w * G + g) * D + d], c.sh.fw[g * kAW + w], A);
    uint2 *dst = part + ((size_t)(hk * G + g) * S + split) * stride;
    ll_store(dst + d, A, ptag);
    if (d == 0) {
      float L = 0.f;
#pragma unroll
      for (int w = 0; w < kAW; ++w)
        L = fmaf(c.sh.al[w][g], c.sh.fw[g * kAW + w], L);
      ll_store(dst + D, c.sh.fm[g], ptag);
      ll_store(dst + D + 1, L, ptag);
    }
  }
  consumer_sync();   // q | k | v and aacc (in xs) have been read: xs is reused below
  trace(c, layer, 10);
  // ---- fold the splits for this CTA's slice of the G*D outputs ----------------------
  // (frontend/Python/ops/tosa.py:14502-14594): weights exp(m_s - M), then sums in
  // split order.  A warp takes outputs warp, warp + 16, ..; its lanes take splits
  // lane, lane + 32, ..; the raw partials are requested first and stay in
  // registers while the (m, l) pairs of all splits are turned into weights.
  float *cm = c.xs, *cl = cm + G * S, *cw = cl + G * S, *cL = cw + G * S;
  const int per = (G * D + S - 1) / S;
  const int o_begin = split * per;
  const int o_cnt = max(0, min(per, G * D - o_begin));
  const int sl = (S + 31) >> 5;       // splits per lane
  constexpr int kMaxR = 8;            // (outputs per warp) x (splits per lane), checked on the host
  uint2 r[kMaxR];
  {
    int oo = 0, ss = 0;
#pragma unroll
    for (int a = 0; a < kMaxR; ++a) {
      const int o = warp + kCW * oo, si = lane + 32 * ss;
      r[a] = make_uint2(0u, 0u);
      if (o < o_cnt && si < S) {
        const int og = o_begin + o, g = og / D, d = og - g * D;
        r[a] = ll_load1(part + ((size_t)(hk * G + g) * S + si) * stride + d);
      }
      if (++ss == sl) {
        ss = 0;
        ++oo;
      }
    }
  }
  for (int idx = c.ctid; idx < G * S; idx += kCT) {
    const uint2 *src = part + ((size_t)hk * G * S + idx) * stride + D;   // idx = g * S + split
    uint4 v = ll_load2(src);
    v = ll_wait2(c, src, ptag, v);
    cm[idx] = __uint_as_float(v.x);
    cl[idx] = __uint_as_float(v.z);
  }
  consumer_sync();
  if (warp < G) {
    const int g = warp;
    float M = kSeed;
    for (int si = lane; si < S; si += 32)
      M = fmaxf(M, cm[g * S + si]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
      M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
    float L = 0.f;
    for (int si = lane; si < S; si += 32) {
      const float b = expf(cm[g * S + si] - M);
      cw[g * S + si] = b;
      L = fmaf(cl[g * S + si], b, L);
    }
    L = warp_sum(L);
    if (lane == 0)
      cL[g] = L;
  }
  consumer_sync();
  trace(c, layer, 11);
  {
    int oo = 0, ss = 0;
    float ar = 0.f;
#pragma unroll
    for (int a = 0; a < kMaxR; ++a) {
      const int o = warp + kCW * oo, si = lane + 32 * ss;   // o is the same for the whole warp
      const int og = o_begin + o, g = og / D, d = og - g * D;
      if (o < o_cnt && si < S) {
        float v = __uint_as_float(r[a].x);
        if (r[a].y != ptag)
          v = ll_wait1(c, part + ((size_t)(hk * G + g) * S + si) * stride + d, ptag);
        ar = fmaf(v, cw[g * S + si], ar);
      }
      if (++ss == sl) {
        ar = warp_sum(ar);
        if (lane == 0 && o < o_cnt)
          ll_store(p.ll_attn + (size_t)par * QD + (size_t)(hk * G + g) * D + d,
                   __fdiv_rn(ar, cL[g]), tag_of(c, layer, T_ATTN));
        ar = 0.f;
        ss = 0;
        ++oo;
      }
    }
  }
  consumer_sync();
}

__device__ __forceinline__ void attention_dispatch(Ctx &c, int layer, int pos) {
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

__global__ void __launch_bounds__(kMegaThreads, 1)
decode_step_kernel(const __grid_constant__ MegaParams p) {
  extern __shared__ __align__(128) uint8_t smem_raw[];
  Shared &sh = *reinterpret_cast<Shared *>(smem_raw);
  float *xs = reinterpret_cast<float *>(smem_raw + ((sizeof(Shared) + 127) / 128) * 128);
  uint8_t *ring = reinterpret_cast<uint8_t *>(xs + p.xs_floats);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int *err = p.error;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.slots; ++s) {
      mbar_init(&sh.full[s], 1);
      sh.done[s] = 0;
      sh.issued[s] = -1;
    }
    sh.abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    // this CTA's stream plan
    StreamPlan &pl = sh.plan;
    long long off = 0;
    pl.per_layer = 0;
    for (int i = 0; i < 5; ++i) {
      int rb, nr;
      rows_of(p.phase[i], blockIdx.x, gridDim.x, rb, nr);
      pl.rows[i] = nr;
      pl.rps[i] = p.phase[i].rps;
      pl.row_bytes[i] = p.phase[i].row_bytes;
      pl.n[i] = (nr + pl.rps[i] - 1) / pl.rps[i];
      if (i < 4) {
        pl.off[i] = off;
        off += (long long)nr * pl.row_bytes[i];
        pl.per_layer += pl.n[i];
      } else {
        pl.off[i] = 0;
      }
    }
    pl.layer_bytes = off;
    pl.L = p.L;
    pl.total = p.L * pl.per_layer + pl.n[4];
    {
      int r = 0;
      for (int i = 0; i < 4; ++i)
        for (int q = 0; q < pl.n[i]; ++q, ++r) {
          const int rows = min(pl.rps[i], pl.rows[i] - q * pl.rps[i]);
          pl.tab[r] = make_uint2((uint32_t)(pl.off[i] + (long long)q * pl.rps[i] * pl.row_bytes[i]),
                                 (uint32_t)rows * pl.row_bytes[i]);
        }
      for (int sl = 0; sl < p.slots; ++sl) {
        int l = 0, rr = sl;
        while (l < pl.L && rr >= pl.per_layer) {
          rr -= pl.per_layer;
          ++l;
        }
        pl.next_l[sl] = l;
        pl.next_r[sl] = rr;
      }
    }
    sh.stream_base = p.stream + p.cta_off[blockIdx.x];
  }
  const int token = p.state[0], pos = p.state[1];
  if (threadIdx.x < D / 2) {
    // subgraph0_decode_simplify.mlir:52-59
    const float th = __fmul_rn(__ldg(p.inv_freq + threadIdx.x), (float)pos);
    sh.cs[threadIdx.x] = cosf(th);
    sh.sn[threadIdx.x] = sinf(th);
  }
  __syncthreads();
  if (threadIdx.x == 0)   // fill the ring
    for (int s = 0; s < p.slots; ++s)
      issue_stage(sh, ring, p.slot_bytes, s, s, p.slots);

  // ================= consumers ===================================================
  const uint32_t tags_per_launch = 8u * (uint32_t)(p.L + 3);
  Ctx c{p, sh, xs, ring, err, (int)threadIdx.x, lane, warp, 0, 0u, 0,
        ((uint32_t)p.state[4] + 1u) * tags_per_launch,
        (p.trace != nullptr && blockIdx.x % p.trace_stride == 0)
            ? p.trace + (size_t)(blockIdx.x / p.trace_stride) * (p.L + 1) * kMegaTraceSlots
            : nullptr};
  const int H = p.H, QD = p.qh * D, KD = p.kvh * D;
  const float *embed_row = p.embed + (size_t)token * H;
  // One loop over (layer, projection) so that the projection body exists once:
  // step 0..3 of layer l = q|k|v, o, gate|up, down; layer L has the lm_head only.
  for (int l = 0; l <= p.L; ++l) {
    const int par = l & 1, ppar = par ^ 1;
    const bool last = l == p.L;
    // residual stream entering the layer: the embedding row, or layer l-1's output
    const uint2 *xin_ll = l == 0 ? nullptr : p.ll_xa + (size_t)ppar * H;
    const uint32_t xin_tag = tag_of(c, l - 1, T_XA);
    const int nsteps = last ? 1 : 4;
    for (int step = 0; step < nsteps; ++step) {
      XSrc xsrc;
      Epi ep;
      int phase_index;
      if (last) {              // logits <- RMSNorm(x) @ lm_head, with a running first-max
        phase_index = 4;
        xsrc = XSrc{xin_ll, embed_row, xin_tag, p.final_norm};
        ep = Epi{EP_LOGITS, nullptr, 0u, nullptr, nullptr, 0u, p.logits};
      } else if (step == 0) {  // q | k | v (+ bias) <- RMSNorm(x)
        phase_index = 0;
        xsrc = XSrc{xin_ll, embed_row, xin_tag, p.lvec[4 * l]};
        ep = Epi{EP_STORE, p.ll_qkv + (size_t)par * (QD + 2 * KD), tag_of(c, l, T_QKV),
                 nullptr, nullptr, 0u, nullptr};
      } else if (step == 1) {  // x1 = x + attn @ Wo
        phase_index = 1;
        xsrc = XSrc{p.ll_attn + (size_t)par * QD, nullptr, tag_of(c, l, T_ATTN), nullptr};
        ep = Epi{EP_RESIDUAL, p.ll_xb + (size_t)par * H, tag_of(c, l, T_XB),
                 xin_ll, embed_row, xin_tag, nullptr};
      } else if (step == 2) {  // silu(gate) * up <- RMSNorm(x1)
        phase_index = 2;
        xsrc = XSrc{p.ll_xb + (size_t)par * H, nullptr, tag_of(c, l, T_XB), p.lvec[4 * l + 1]};
        ep = Epi{EP_SILU, p.ll_mid + (size_t)par * p.F, tag_of(c, l, T_MID),
                 nullptr, nullptr, 0u, nullptr};
      } else {                 // x2 = x1 + mid @ Wdown
        phase_index = 3;
        xsrc = XSrc{p.ll_mid + (size_t)par * p.F, nullptr, tag_of(c, l, T_MID), nullptr};
        ep = Epi{EP_RESIDUAL, p.ll_xa + (size_t)par * H, tag_of(c, l, T_XA),
                 p.ll_xb + (size_t)par * H, nullptr, tag_of(c, l, T_XB), nullptr};
      }
      trace(c, l, step);
      if (!last && step == 0)
        attention_prefetch(c, l, pos);
      gemv_phase(c, phase_index, xsrc, ep, l);
      if (!last && step == 0) {
        trace(c, l, 6);
        {
          Ctx ca = c;   // the attention functions take the context by address; keep `c` in registers
          attention_dispatch(ca, l, pos);
        }
        trace(c, l, 7);
      }
    }
    trace(c, l, 4);
  }
  if (c.ctid == 0) {
    // the lm_head phase left one candidate per warp (and ended with a CTA barrier)
    float bestv = sh.bestv[0];
    int besti = sh.besti[0];
    for (int w = 1; w < kCW; ++w)
      if (sh.bestv[w] > bestv || (sh.bestv[w] == bestv && sh.besti[w] < besti)) {
        bestv = sh.bestv[w];
        besti = sh.besti[w];
      }
    const uint32_t ctag = tag_of(c, p.L, T_CAND);
    ll_store(p.ll_cand + 2 * blockIdx.x, bestv, ctag);
    ll_store(p.ll_cand + 2 * blockIdx.x + 1, __int_as_float(besti), ctag);
  }
  if (blockIdx.x == 0 && c.warp == 0) {
    // Sampler.h:101-104: first maximum over the per-CTA candidates
    const uint32_t ctag = tag_of(c, p.L, T_CAND);
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = c.lane; i < (int)gridDim.x; i += 32) {
      uint4 r = ll_load2(p.ll_cand + 2 * i);
      r = ll_wait2(c, p.ll_cand + 2 * i, ctag, r);
      const float v = __uint_as_float(r.x);
      const int ix = (int)r.z;
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
    if (c.lane == 0 && sh.abort_flag == 0) {
      const int next = bi == 0x7fffffff ? 0 : bi;
      const int cnt = p.state[3];
      if (cnt < p.history_cap)
        p.history[cnt] = next;
      p.state[3] = cnt + 1;
      p.state[2] = next;
      p.state[0] = next;
      p.state[1] = pos + 1;
      p.state[4] = p.state[4] + 1;   // launches completed (base of the tags)
    }
  }
  if (sh.abort_flag) {
    // an abandoned step may still have ring copies in flight: give them time
    // to land before the CTA (and its shared memory) goes away
    const unsigned long long t0 = now_ns();
    while (now_ns() - t0 < 2000000ull) {
    }
  }
}

// ---- stream builder: packed rows of one projection -> per-CTA streams ---------------
// One CTA per source row: copies its K packed bytes (flipping the sign bit:
// int8 q -> u = q + 128) and appends the 16-byte trailer {scale, bias, 0, 0}.
// Source row r becomes row r * row_stride + row_phase of a projection with
// N_total rows, dealt out to the CTAs in units of `unit` rows.
__global__ void mega_build_rows_kernel(const uint8_t *src, int K, int row_stride, int row_phase,
                                       int N_total, int unit, const float *scale,
                                       const float *bias, int grid_ctas, int row_bytes,
                                       const int64_t *cta_phase_off, uint8_t *stream) {
  const int n = blockIdx.x * row_stride + row_phase;
  const int nu = N_total / unit, un = n / unit;
  const int base = nu / grid_ctas, rem = nu % grid_ctas;
  int cta;
  const int split = rem * (base + 1);
  if (un < split)
    cta = un / (base + 1);
  else
    cta = rem + (un - split) / base;
  const int begin = (cta * base + min(cta, rem)) * unit;
  uint8_t *dst = stream + cta_phase_off[cta] + (int64_t)(n - begin) * row_bytes;
  const uint4 *s4 = reinterpret_cast<const uint4 *>(src + (int64_t)blockIdx.x * K);
  uint4 *d4 = reinterpret_cast<uint4 *>(dst);
  for (int i = threadIdx.x; i < K / 16; i += blockDim.x) {
    uint4 v = s4[i];
    v.x ^= 0x80808080u; v.y ^= 0x80808080u; v.z ^= 0x80808080u; v.w ^= 0x80808080u;
    d4[i] = v;
  }
  if (threadIdx.x == 0)
    *reinterpret_cast<float4 *>(dst + K) =
        make_float4(scale[blockIdx.x], bias ? bias[blockIdx.x] : 0.f, 0.f, 0.f);
}

int mega_build_rows(const void *packed, int K, int n_rows, int row_stride, int row_phase,
                    int N_total, int unit, const float *scale, const float *bias, int grid_ctas,
                    int row_bytes, const int64_t *cta_phase_off_dev, void *stream_buf,
                    cudaStream_t st) {
  mega_build_rows_kernel<<<n_rows, 128, 0, st>>>((const uint8_t *)packed, K, row_stride, row_phase,
                                                 N_total, unit, scale, bias, grid_ctas, row_bytes,
                                                 cta_phase_off_dev, (uint8_t *)stream_buf);
  B200_LAUNCH_CHECK();
  return B200_OK;
}

size_t mega_fixed_shared_bytes() { return ((sizeof(Shared) + 127) / 128) * 128; }

int mega_launch(const MegaParams &p, int grid, size_t smem, cudaStream_t st) {
  // the attribute belongs to the device's copy of the function: set it once per device
  static bool configured[64] = {};
  int dev = 0;
  B200_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    B200_CUDA(cudaFuncSetAttribute(decode_step_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   227 * 1024));
    if (dev >= 0 && dev < 64)
      configured[dev] = true;
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

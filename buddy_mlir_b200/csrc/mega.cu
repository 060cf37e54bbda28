// One persistent kernel per decode token (batch 1, int8 weight-only).
//
// Why: at batch 1 a decode step of the 1.5B model is 140 dependent GEMVs of
// 0.4-2 us each; launched one by one (even from a CUDA graph) every kernel
// boundary drains the memory pipeline.  Here one CTA per SM stays resident for
// the whole token.
//
//  * Weights.  Each CTA owns a fixed slice of the output rows of every
//    projection, and ALL weight bytes that CTA will ever need are laid out back
//    to back in one private stream (built once at load time) as ring stages:
//    a stage is a block of 16 rows x one K slice, followed by the rows' trailers
//    (scale, bias, sum of the row's weights).  The stream is pulled with bulk
//    async copies (cp.async.bulk, completion on mbarriers) into a ring of
//    shared-memory slots; every warp works on whole stages and refills the slot
//    it has just finished with the stage one ring-length ahead.  Refills never
//    wait for activations, so HBM stays busy across the dependency points of
//    the graph (the ring holds about half a layer's worth of weights).
//  * Activations.  There is no grid-wide barrier.  Every activation vector
//    that crosses CTAs (q|k|v, attention output, the two residual streams, the
//    SiLU-gated MLP intermediate, attention split partials, argmax candidates)
//    is stored as 8-byte (value, tag) pairs written with one 64-bit store; the
//    tag names launch, layer and producer phase.  A consumer simply loads the
//    pairs it needs and retries until the tags match: data arrival IS the
//    synchronisation, and CTAs drift apart by at most one phase because every
//    phase needs all outputs of the one before.  Buffers alternate by layer
//    parity, so a producer can never overwrite a value a slower CTA still has
//    to read.
//  * Math.  The activation vector of a projection is turned, once per phase,
//    into a 23-bit fixed-point number per element (one power-of-two scale per
//    vector, taken from its largest magnitude) and stored as three int8 planes
//    (high, middle, low byte).  The dot products with the int8 weights are
//    then integer tensor-core instructions (mma.sync m16n8k32 s8: sixteen
//    weight rows are the rows of A, the three planes are three columns of B), so
//    one instruction handles 16 rows x 32 k, the accumulation is exact, and
//    the per-plane sums are recombined in 64-bit integers before the single
//    conversion to float.  Because integer sums do not depend on their order,
//    K can be cut over warps freely (shared-memory atomics) and the result is
//    bit-identical for every schedule.
//
// Every wait (mbarrier or tag poll) is bounded: on expiry the kernel records an
// error code, all later waits fall through, control flow stays identical (so
// CTA barriers stay matched), and the host call fails.
//
// Arithmetic is that of examples/BuddyDeepSeekR1/subgraph0_decode_simplify.mlir
// :46-260 with the int8 GEMV of
// midend/lib/Conversion/MatMulOptimization/DequantMatMulVectorizationDecode.cpp:250-321
// (sum over k of x*q, then the per-channel scale) and the attention recurrence
// of frontend/Python/ops/tosa.py:14245-14594.
#include "common.cuh"
#include "mega.cuh"

#include <cstddef>

namespace b200 {

namespace {

constexpr int kCW = 16;           // warps (all of them consume)
constexpr int kCT = kCW * 32;     // threads
constexpr int kAW = 7;            // warps that scan the KV cache in the attention phase
constexpr int kMaxV = 10;         // (value, value) vectors per thread: K <= 2 * 512 * 10
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
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
// D (16x8, s32) += A (16x32, s8, row) * B (32x8, s8, col)
__device__ __forceinline__ void mma_s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                       uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
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

// One ring stage of this CTA's stream.
struct StageRef {
  uint32_t off;      // byte offset inside the layer's part of the stream (or the lm_head's)
  uint32_t bytes;
};

// What this CTA does in one projection (fixed for the whole run).
struct PhaseInfo {
  int row_begin, nrows, nrb;   // first row, rows, row blocks of 8
  int nstages;                 // ring stages = nrb * nks
  int nunits;                  // pieces of work = nstages * nkw (one warp each)
  int K, slice_bytes, nks, nkw, chunks, swizzle;   // chunks: 64-byte chunks of k per piece of work
  int first_stage;             // index of the phase's first stage inside a layer (projections 0..3)
};

struct Shared {
  uint64_t full[kMegaMaxSlots];
  int issued[kMegaMaxSlots];            // stage last requested into the slot
  int done[kMegaMaxSlots];              // warps that finished their piece of the slot's current stage
  int next_l[kMegaMaxSlots], next_r[kMegaMaxSlots];   // per ring slot: the stage it receives next
  PhaseInfo ph[5];
  StageRef tab[kMegaMaxLayerStages];    // stage r of a layer
  int per_layer, total, L;
  long long layer_bytes;
  const uint8_t *stream_base;
  int accw[kCW][48];                    // per warp: [plane][row] sums of the warp's current stage
  int acc[kMegaAccBlocks][48];          // per row block: [plane][row] partial sums (K cut over warps)
  int cnt[kMegaAccBlocks];              // slices of the block that have been added
  float cs[64], sn[64];                 // cos / sin of this step's position
  float red[2 * kCW];                   // per warp: (sum of squares, largest magnitude)
  float bestv[kCW];
  int besti[kCW];
  int abort_flag;
  float am[kAW][8], al[kAW][8];         // attention: per-warp (m, l)
  float fw[8 * kAW], fm[8];             // attention: fold of the warps (weights, m per head)
};

struct Ctx {
  const MegaParams &p;
  Shared &sh;
  float *xs;          // scratch (shared memory): activation planes, attention staging
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
    v = ll_load2(p);
  }
  return v;
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
  if (g >= sh.total)
    return;
  int l = sh.next_l[slot], r = sh.next_r[slot];
  const uint8_t *src;
  uint32_t bytes;
  if (l < sh.L) {
    const StageRef e = sh.tab[r];
    src = sh.stream_base + (long long)l * sh.layer_bytes + e.off;
    bytes = e.bytes;
  } else {   // the lm_head follows the layers: one K slice, blocks of 8 rows
    const PhaseInfo &pi = sh.ph[4];
    const int rows = min(kMegaBlockRows, pi.nrows - r * kMegaBlockRows);
    bytes = (uint32_t)rows * (pi.K + kMegaTrailer);
    src = sh.stream_base + (long long)sh.L * sh.layer_bytes +
          (long long)r * kMegaBlockRows * (pi.K + kMegaTrailer);
  }
  *(volatile int *)&sh.issued[slot] = g;
  mbar_expect_tx(&sh.full[slot], bytes);
  bulk_g2s(ring + (size_t)slot * slot_bytes, src, bytes, &sh.full[slot]);
  r += n_slots;
  while (l < sh.L && r >= sh.per_layer) {
    r -= sh.per_layer;
    ++l;
  }
  sh.next_l[slot] = l;
  sh.next_r[slot] = r;
}

// Wait until stage `want` has landed in `slot`.  The parity of an mbarrier only
// tells consecutive uses of a slot apart; warps work on different stages and can
// run more than one use ahead of the warp that still owns the slot, so the wait
// first makes sure the slot has been re-requested for the wanted stage.
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

__device__ __forceinline__ float silu_mul(float g, float u) {
  // subgraph0_decode_simplify.mlir:226-231: (g * sigmoid(g)) * u
  const float s = 1.0f / (1.0f + expf(-g));
  return __fmul_rn(__fmul_rn(g, s), u);
}

// ---- one projection -----------------------------------------------------------------
// 1. The activation vector (K values) is fetched by the whole CTA, multiplied by
//    the RMSNorm weight if there is one, and kept in registers while its largest
//    magnitude and sum of squares are reduced over the CTA.
// 2. With qs = 2^22 / 2^ceil(log2(max)) every value becomes the integer
//    X = rint(v * qs), |X| <= 2^22 (exact: qs is a power of two), stored as
//    three signed bytes  X = h * 65536 + (m + 128) * 256 + (l + 128)  in three
//    planes of K bytes in shared memory.
// 3. Every warp takes pieces of ring stages (16 rows x a k range).  Lane (g, t),
//    g = lane / 4, t = lane % 4, loads 16 weight bytes of row g and of row g + 8
//    and, if g < 3, the 16 bytes of plane g at the same k; two m16n8k32
//    instructions consume them (k runs over the lanes in fragment order, the same
//    for both operands, which is all a dot product needs).  After the k range,
//    lanes t = 0 hold the sums of planes 0 and 1 against rows g and g + 8, lanes
//    t = 1 those of plane 2.
// 4. The sums go to shared memory ([plane][row]; added atomically when K is cut
//    into several pieces, the warp that adds the last piece carries on), lanes
//    0..15 pick up one row each:
//      sum x*q = (Sh * 65536 + Sm * 256 + Sl + 32896 * sum q) / qs
//    in 64-bit integers, one conversion to float, then the RMSNorm factor, the
//    row's scale and bias, and the epilogue.
// One piece of work of a projection: which stage, which part of it, where it sits.
struct Piece {
  int st, sub, rb, ks, slot, rows;
  uint32_t par;
};
__device__ __forceinline__ Piece piece_of(const Ctx &c, const PhaseInfo &pi, int u, int n_slots) {
  // piece u = (stage st, part sub of its k range); stage st = (row block rb, slice ks)
  Piece q;
  q.st = u / pi.nkw;
  q.sub = u - q.st * pi.nkw;
  q.rb = q.st / pi.nks;
  q.ks = q.st - q.rb * pi.nks;
  const int lap = (c.slot + q.st) / n_slots;
  q.slot = c.slot + q.st - lap * n_slots;
  q.par = c.parity ^ (uint32_t)(lap & 1);
  q.rows = min(kMegaBlockRows, pi.nrows - q.rb * kMegaBlockRows);
  return q;
}

__device__ __forceinline__ void gemv_phase(Ctx &c, int phase_index, const XSrc &xs, const Epi &ep,
                                           int tl) {
  Shared &sh = c.sh;
  const PhaseInfo &pi = sh.ph[phase_index];
  const int K = pi.K;
  const int n_slots = c.p.slots, slot_bytes = c.p.slot_bytes;
  const int lane = c.lane, warp = c.warp, ctid = c.ctid;
  uint8_t *const ring = c.ring;
  int8_t *const planes = reinterpret_cast<int8_t *>(c.xs);
  const int pstride = c.p.plane_stride;
  volatile int *ab = &sh.abort_flag;

  // ---- 0. this warp's first piece: the index arithmetic does not depend on the
  //         activations, so it is done before they are waited for.  (The wait for
  //         the stage itself must stay behind the CTA barriers below: a stage late
  //         in a long projection is only requested once an earlier one has been
  //         consumed, which takes every warp's arrival at those barriers.)
  Piece pc = piece_of(c, pi, warp, n_slots);

  // ---- 1. fetch the activations: they stay in registers until their largest
  //         magnitude is known -------------------------------------------------------
  const int nv = K >> 1;               // vectors of two values
  float2 v[kMaxV];
  float ss = 0.f, amax = 0.f;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    // two batches of requests (all loads of a batch are in flight before the first
    // tag is looked at); vectors up to K = 512 * kMaxV need only the first
    uint4 r[kMaxV / 2];
#pragma unroll
    for (int i = 0; i < kMaxV / 2; ++i) {
      const int idx = (h * (kMaxV / 2) + i) * kCT + ctid;
      if (idx < nv) {
        if (xs.ll != nullptr) {
          r[i] = ll_load2(xs.ll + 2 * idx);
        } else {
          const float2 t = __ldg(reinterpret_cast<const float2 *>(xs.plain) + idx);
          r[i] = make_uint4(__float_as_uint(t.x), xs.tag, __float_as_uint(t.y), xs.tag);
        }
      }
    }
    if (xs.ll != nullptr) {
      // one retry loop for the batch: reload whatever does not carry the tag yet
      uint32_t it = 0;
      unsigned long long t0 = 0;
      for (;;) {
        bool ok = true;
#pragma unroll
        for (int i = 0; i < kMaxV / 2; ++i) {
          const int idx = (h * (kMaxV / 2) + i) * kCT + ctid;
          if (idx < nv && (r[i].y != xs.tag || r[i].w != xs.tag)) {
            r[i] = ll_load2(xs.ll + 2 * idx);
            ok = false;
          }
        }
        if (ok || *ab)
          break;
        bool give_up = ++it >= kSpinLimit;
        if ((it & 0x3FF) == 0) {
          const unsigned long long t = now_ns();
          if (t0 == 0)
            t0 = t;
          give_up = give_up || *c.err != 0 || t - t0 > kWaitNs;
        }
        if (give_up) {
          atomicCAS((int *)c.err, 0, 400 + (int)(xs.tag & 7));
          *ab = 1;
          break;
        }
      }
    }
#pragma unroll
    for (int i = 0; i < kMaxV / 2; ++i) {
      const int idx = (h * (kMaxV / 2) + i) * kCT + ctid;
      if (idx < nv) {
        float a = __uint_as_float(r[i].x), b = __uint_as_float(r[i].z);
        ss = __fadd_rn(ss, __fmul_rn(a, a));
        ss = __fadd_rn(ss, __fmul_rn(b, b));
        if (xs.nw != nullptr) {
          const float2 w = __ldg(reinterpret_cast<const float2 *>(xs.nw) + idx);
          a = __fmul_rn(a, w.x);
          b = __fmul_rn(b, w.y);
        }
        amax = fmaxf(amax, fmaxf(fabsf(a), fabsf(b)));
        v[h * (kMaxV / 2) + i] = make_float2(a, b);
      }
    }
  }
  ss = warp_sum(ss);
  amax = warp_max(amax);
  if (lane == 0)
    *reinterpret_cast<float2 *>(&sh.red[2 * warp]) = make_float2(ss, amax);
  consumer_sync();
  trace(c, tl, 12 + 4 * phase_index);
  float mult;   // turns the integer row sum into the (normalised) dot product
  {
    // every warp folds the 16 partial (sum, max) pairs with one shuffle tree
    float2 part = make_float2(0.f, 0.f);
    if (lane < kCW)
      part = *reinterpret_cast<const float2 *>(&sh.red[2 * lane]);
    float t = part.x, mx = part.y;
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) {
      t += __shfl_xor_sync(0xffffffffu, t, o);
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    }
    t = __shfl_sync(0xffffffffu, t, 0);
    mx = __shfl_sync(0xffffffffu, mx, 0);
    // qs = 2^(148 - e), e the biased exponent of the maximum: |v| < 2^(e - 126), so |v * qs| <= 2^22
    int e = (int)(__float_as_uint(mx) >> 23);
    e = min(max(e, 22), 253);
    const float qs = __uint_as_float((uint32_t)(275 - e) << 23);
    mult = __uint_as_float((uint32_t)(e - 21) << 23);   // 1 / qs
    // RMSNorm, subgraph0_decode_simplify.mlir:60-72 (the factor multiplies the row sums)
    if (xs.nw != nullptr)
      mult *= rsqrtf(__fadd_rn(__fmul_rn(t, 1.0f / (float)K), c.p.eps));
    // ---- 2. the three planes -----------------------------------------------------
#pragma unroll
    for (int i = 0; i < kMaxV; ++i) {
      const int idx = i * kCT + ctid;
      if (idx < nv) {
        const int xa = __float2int_rn(v[i].x * qs), xb = __float2int_rn(v[i].y * qs);
        // bytes 0,1 = high plane of both values, bytes 2,3 = middle plane; then the low plane
        const uint32_t hm = __byte_perm((uint32_t)xa, (uint32_t)xb, 0x5162) ^ 0x80800000u;
        const uint32_t lo = __byte_perm((uint32_t)xa, (uint32_t)xb, 0x0040) ^ 0x00008080u;
        *reinterpret_cast<uint16_t *>(planes + 2 * idx) = (uint16_t)(hm & 0xFFFFu);
        *reinterpret_cast<uint16_t *>(planes + pstride + 2 * idx) = (uint16_t)(hm >> 16);
        *reinterpret_cast<uint16_t *>(planes + 2 * pstride + 2 * idx) = (uint16_t)lo;
      }
    }
  }
  consumer_sync();
  trace(c, tl, 13 + 4 * phase_index);

  // ---- 3. the stages -------------------------------------------------------------
  const int g4 = lane >> 2, t4 = lane & 3;
  const int nkw = pi.nkw, chunks = pi.chunks, slice = pi.slice_bytes;
  const int per_block = pi.nks * nkw;     // pieces of work that add into one row block
  float bestv = -INFINITY;
  int besti = 0x7fffffff;
#pragma unroll 1
  for (int u = warp; u < pi.nunits; u += kCW) {
    if (u != warp)
      pc = piece_of(c, pi, u, n_slots);
#ifdef MEGA_FINE_TRACE
    const bool ftr = phase_index < 4 && u == warp;
    if (ftr) trace(c, tl, 32 + 8 * phase_index);
#endif
    if (!stage_wait(sh, pc.slot, pc.par, c.g + pc.st, c.err, ab))
      atomicCAS((int *)c.err, 0, 200 + pc.slot);
#ifdef MEGA_FINE_TRACE
    if (ftr) trace(c, tl, 33 + 8 * phase_index);
#endif
    const int rows = pc.rows, rb = pc.rb;
    const uint8_t *base = ring + (size_t)pc.slot * slot_bytes;
    // rows g4 and g4 + 8, clamped: loads stay inside the stage
    const int r_lo = min(g4, rows - 1), r_hi = min(g4 + 8, rows - 1);
    const int jb = pc.sub * chunks * 4;    // first 16-byte unit of this warp's k range inside the slice
    const uint32_t w_lo = smem_u32(base + r_lo * slice), w_hi = smem_u32(base + r_hi * slice);
    const int swz_lo = (r_lo & 1) ? pi.swizzle : 0, swz_hi = (r_hi & 1) ? pi.swizzle : 0;
    const uint32_t xrow = smem_u32(planes + min(g4, 2) * pstride + pc.ks * slice + jb * 16);
    const bool has_b = g4 < 3;
    int d0[4] = {0, 0, 0, 0}, d1[4] = {0, 0, 0, 0};
#pragma unroll 2
    for (int j = 0; j < chunks; ++j) {   // a chunk = 64 k = two instructions
      const int un = jb + (j << 2) + t4;
      const uint4 lo = lds128(w_lo + ((un ^ swz_lo) << 4));
      const uint4 hi = lds128(w_hi + ((un ^ swz_hi) << 4));
      uint4 x = make_uint4(0u, 0u, 0u, 0u);
      if (has_b)
        x = lds128(xrow + (((j << 2) + t4) << 4));
      mma_s8(d0, lo.x, hi.x, lo.y, hi.y, x.x, x.y);
      mma_s8(d1, lo.z, hi.z, lo.w, hi.w, x.z, x.w);
    }
#ifdef MEGA_FINE_TRACE
    if (ftr) trace(c, tl, 34 + 8 * phase_index);
#endif
    // lane (g4, t4): c0, c1 = row g4 x planes 2*t4, 2*t4 + 1; c2, c3 = row g4 + 8
    const int s0 = d0[0] + d1[0], s1 = d0[1] + d1[1], s2 = d0[2] + d1[2], s3 = d0[3] + d1[3];
    // ---- 4. [plane][row] sums to shared memory, one lane per row finishes -----------
    int *accp = per_block == 1 ? sh.accw[warp] : sh.acc[rb];
    bool last = true;
    if (per_block == 1) {
      if (t4 == 0) {
        accp[g4] = s0;
        accp[g4 + 8] = s2;
        accp[16 + g4] = s1;
        accp[16 + g4 + 8] = s3;
      } else if (t4 == 1) {
        accp[32 + g4] = s0;
        accp[32 + g4 + 8] = s2;
      }
      __syncwarp();
    } else {
      if (t4 == 0) {
        atomicAdd(&accp[g4], s0);
        atomicAdd(&accp[g4 + 8], s2);
        atomicAdd(&accp[16 + g4], s1);
        atomicAdd(&accp[16 + g4 + 8], s3);
      } else if (t4 == 1) {
        atomicAdd(&accp[32 + g4], s0);
        atomicAdd(&accp[32 + g4 + 8], s2);
      }
      __syncwarp();
      int old = 0;
      if (lane == 0) {
        __threadfence_block();
        old = atomicAdd(&sh.cnt[rb], 1);
      }
      old = __shfl_sync(0xffffffffu, old, 0);
      last = old == per_block - 1;
      if (last)
        __threadfence_block();
    }
#ifdef MEGA_FINE_TRACE
    if (ftr) trace(c, tl, 35 + 8 * phase_index);
#endif
    if (last && lane < kMegaBlockRows) {
      const int row = lane;
      const int rc = min(row, rows - 1);
      const long long Sh = ((volatile int *)accp)[rc], Sm = ((volatile int *)accp)[16 + rc],
                      Sl = ((volatile int *)accp)[32 + rc];
      if (per_block != 1) {   // ready for the next projection (all 16 entries: rows beyond the block hold sums of repeated rows)
        __syncwarp(0x0000ffffu);
        ((volatile int *)accp)[row] = 0;
        ((volatile int *)accp)[16 + row] = 0;
        ((volatile int *)accp)[32 + row] = 0;
        if (lane == 0)
          sh.cnt[rb] = 0;
      }
      const float4 tr = *reinterpret_cast<const float4 *>(base + rows * slice + rc * kMegaTrailer);
      const long long T = (Sh << 16) + (Sm << 8) + Sl + 32896ll * (long long)__float_as_int(tr.z);
      const float dotv = __fmul_rn(__ll2float_rn(T), mult);
      const float val = __fadd_rn(__fmul_rn(dotv, tr.x), tr.y);
      const int n = pi.row_begin + rb * kMegaBlockRows + row;
      if (ep.kind == EP_SILU) {
        // rows (2j, 2j+1) = (gate_j, up_j) sit in neighbouring lanes
        const float upv = __shfl_xor_sync(0x0000ffffu, val, 1);
        if ((row & 1) == 0 && row + 1 < rows)
          ll_store(ep.dst + (n >> 1), silu_mul(val, upv), ep.tag);
      } else if (row < rows) {
        if (ep.kind == EP_RESIDUAL) {
          const float r = ep.res_ll ? ll_wait1(c, ep.res_ll + n, ep.res_tag) : __ldg(ep.res_plain + n);
          ll_store(ep.dst + n, __fadd_rn(r, val), ep.tag);
        } else if (ep.kind == EP_LOGITS) {
          ep.logits[n] = val;
          if (val > bestv || (val == bestv && n < besti)) {
            bestv = val;
            besti = n;
          }
        } else {
          ll_store(ep.dst + n, val, ep.tag);
        }
      }
    }
    // Release the stage: the warp that finishes it last refills its slot with the
    // stage one ring-length ahead.  (No fence on purpose: the slot's bytes were
    // consumed by arithmetic the values above depend on, so every read has
    // completed; the counter reset is ordered before the next use of the slot by
    // the arrival of that stage's data.)
    __syncwarp();
#ifdef MEGA_FINE_TRACE
    if (ftr) trace(c, tl, 36 + 8 * phase_index);
#endif
    if (lane == 0 && (nkw == 1 || atomicAdd(&sh.done[pc.slot], 1) == nkw - 1)) {
      sh.done[pc.slot] = 0;
      issue_stage(sh, ring, slot_bytes, pc.slot, c.g + pc.st + n_slots, n_slots);
    }
#ifdef MEGA_FINE_TRACE
    if (ftr) trace(c, tl, 37 + 8 * phase_index);
#endif
  }
  trace(c, tl, 14 + 4 * phase_index);
  // this phase used `nstages` stages of the ring
  {
    int slot = c.slot + pi.nstages;
    uint32_t parity = c.parity;
    while (slot >= n_slots) {
      slot -= n_slots;
      parity ^= 1u;
    }
    c.slot = slot;
    c.parity = parity;
    c.g += pi.nstages;
  }
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
  // the planes are reused by the next phase
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
#pragma unroll 1
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
  uint8_t *ring = reinterpret_cast<uint8_t *>(xs) + p.xs_bytes;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int *err = p.error;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.slots; ++s) {
      mbar_init(&sh.full[s], 1);
      sh.issued[s] = -1;
      sh.done[s] = 0;
    }
    sh.abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    // this CTA's share of every projection and its stage table
    long long off = 0;
    int r = 0;
    for (int i = 0; i < 5; ++i) {
      const MegaPhase &ph = p.phase[i];
      PhaseInfo &pi = sh.ph[i];
      rows_of(ph, blockIdx.x, gridDim.x, pi.row_begin, pi.nrows);
      pi.nrb = (pi.nrows + kMegaBlockRows - 1) / kMegaBlockRows;
      pi.nstages = pi.nrb * ph.nks;
      pi.nunits = pi.nstages * ph.nkw;
      pi.K = ph.K;
      pi.slice_bytes = ph.slice_bytes;
      pi.nks = ph.nks;
      pi.nkw = ph.nkw;
      pi.chunks = ph.slice_bytes / 64 / ph.nkw;
      pi.swizzle = ph.swizzle;
      pi.first_stage = r;
      if (i < 4) {
        for (int b = 0; b < pi.nrb; ++b) {
          const int rows = min(kMegaBlockRows, pi.nrows - b * kMegaBlockRows);
          for (int k = 0; k < ph.nks; ++k, ++r) {
            const uint32_t bytes = (uint32_t)rows * (ph.slice_bytes + kMegaTrailer);
            if (r < kMegaMaxLayerStages)
              sh.tab[r] = StageRef{(uint32_t)off, bytes};
            off += bytes;
          }
        }
      }
    }
    sh.per_layer = r;
    sh.layer_bytes = off;
    sh.L = p.L;
    sh.total = p.L * sh.per_layer + sh.ph[4].nstages;
    for (int sl = 0; sl < p.slots; ++sl) {
      int l = 0, rr = sl;
      while (l < sh.L && rr >= sh.per_layer) {
        rr -= sh.per_layer;
        ++l;
      }
      sh.next_l[sl] = l;
      sh.next_r[sl] = rr;
    }
    sh.stream_base = p.stream + p.cta_off[blockIdx.x];
  }
  for (int i = threadIdx.x; i < kMegaAccBlocks * 48; i += blockDim.x)
    (&sh.acc[0][0])[i] = 0;
  if (threadIdx.x < kMegaAccBlocks)
    sh.cnt[threadIdx.x] = 0;
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
// One CTA per source row.  Source row r is row n = r * row_stride + row_phase of a
// projection with N_total rows, dealt out to the CTAs in units of ph.unit rows.
// Inside its CTA's part the row belongs to block b = local / 8, row i = local % 8;
// slice k of the block is the stage [rows x slice_bytes][rows x 16-byte trailer]
// at byte  b * 8 * (K + 16 * nks) + k * rows * (slice_bytes + 16).  The row's
// bytes are its int8 weights in natural k order (the source is the packed-row
// layout of the GEMV path, see packed_offset), with the two 64-byte halves of
// every 128 bytes swapped in odd rows when ph.swizzle is set (shared-memory
// banks: lanes of two rows then read different banks).  Trailer: {scale, bias,
// sum of the row's weights (int32), 0}.
__global__ void mega_build_rows_kernel(const uint8_t *src, int K, int row_stride, int row_phase,
                                       int N_total, MegaPhase ph, const float *scale,
                                       const float *bias, int grid_ctas,
                                       const int64_t *cta_phase_off, uint8_t *stream) {
  const int n = blockIdx.x * row_stride + row_phase;
  const int nu = N_total / ph.unit, un = n / ph.unit;
  const int base = nu / grid_ctas, rem = nu % grid_ctas;
  int cta;
  const int split = rem * (base + 1);
  if (un < split)
    cta = un / (base + 1);
  else
    cta = rem + (un - split) / base;
  const int begin = (cta * base + min(cta, rem)) * ph.unit;
  const int nrows = (base + (cta < rem ? 1 : 0)) * ph.unit;
  const int local = n - begin, b = local / kMegaBlockRows, ri = local % kMegaBlockRows;
  const int rows = min(kMegaBlockRows, nrows - b * kMegaBlockRows);
  uint8_t *block = stream + cta_phase_off[cta] +
                   (int64_t)b * kMegaBlockRows * ((int64_t)K + (int64_t)kMegaTrailer * ph.nks);
  const uint8_t *srow = src + (int64_t)blockIdx.x * packed_row_bytes(B200_W_I8, K);
  const int swz = (ri & 1) ? ph.swizzle : 0;
  int sum = 0;
  for (int w = threadIdx.x; w < K / 4; w += blockDim.x) {   // 4 consecutive k stay together in a packed row
    const int k = 4 * w;
    const uint32_t word = *reinterpret_cast<const uint32_t *>(srow + packed_offset(B200_W_I8, K, k, nullptr));
    sum += (int)(int8_t)(word & 0xFF) + (int)(int8_t)((word >> 8) & 0xFF) +
           (int)(int8_t)((word >> 16) & 0xFF) + (int)(int8_t)(word >> 24);
    const int ks = k / ph.slice_bytes, kk = k - ks * ph.slice_bytes;
    const int unit16 = (kk >> 4) ^ swz;
    uint8_t *dst = block + (int64_t)ks * rows * (ph.slice_bytes + kMegaTrailer) +
                   (int64_t)ri * ph.slice_bytes + unit16 * 16 + (kk & 15);
    *reinterpret_cast<uint32_t *>(dst) = word;
  }
  __shared__ int s_sum[32];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
    sum += __shfl_xor_sync(0xffffffffu, sum, o);
  if ((threadIdx.x & 31) == 0)
    s_sum[threadIdx.x >> 5] = sum;
  __syncthreads();
  if (threadIdx.x < ph.nks) {
    int total = 0;
    for (int w = 0; w < (int)(blockDim.x + 31) / 32; ++w)
      total += s_sum[w];
    uint8_t *tr = block + (int64_t)threadIdx.x * rows * (ph.slice_bytes + kMegaTrailer) +
                  (int64_t)rows * ph.slice_bytes + ri * kMegaTrailer;
    *reinterpret_cast<float4 *>(tr) = make_float4(scale[blockIdx.x], bias ? bias[blockIdx.x] : 0.f,
                                                  __int_as_float(total), 0.f);
  }
}

int mega_build_rows(const void *packed, int K, int n_rows, int row_stride, int row_phase,
                    int N_total, const MegaPhase &ph, const float *scale, const float *bias,
                    int grid_ctas, const int64_t *cta_phase_off_dev, void *stream_buf,
                    cudaStream_t st) {
  if (ph.nks > 128)
    return fail(B200_ELIMIT, "mega_build_rows: %d K slices", ph.nks);
  mega_build_rows_kernel<<<n_rows, 128, 0, st>>>((const uint8_t *)packed, K, row_stride, row_phase,
                                                 N_total, ph, scale, bias, grid_ctas,
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

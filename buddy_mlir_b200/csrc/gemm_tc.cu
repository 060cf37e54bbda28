// Dense weight-only-quantised GEMM on the 5th-generation tensor cores:
//   C[M,N] = A[M,K] (f32) * dequant(W)[N,K]^T, per-channel scale in the epilogue.
//
// This is the prefill / batched-decode path.  buddy-mlir's prefill GEMM
// (midend/lib/Conversion/MatMulOptimization/MatMulBlisVectorization.cpp:367-530)
// dequantises w = float(q) * scale while it packs B and then runs f32 FMAs; here
// the integer part and the scale are separated (sum_k a*q, then * scale[n]),
// which is the same product up to f32 rounding (the parity tests hold it to
// 1e-3 of the CPU restatement, as for the decode path).
//
// Operands.  int8 -> bf16 is exact (|q| <= 128 needs 8 significant bits), so
// the weight operand loses nothing.  The f32 activations are split into two
// bf16 terms, a = hi + lo (hi = bf16(a), lo = bf16(a - hi), 16 significant
// bits together), and every tile is multiplied twice, once per term, into the
// same f32 accumulator in tensor memory.  The split runs once per GEMM into a
// workspace, in the k order of the packed weight rows (a dot product does not
// care about the order of k as long as both operands agree), so the packed
// decode weights are used as they are: no second copy of the weights is kept.
//
// Two forms of the kernel (template PRE):
//  * converting (fewer than 256 rows: batched decode, HBM- and latency-bound).  One CTA
//    computes a 128 x 128 tile of C.  Warp 0 issues the TMA loads (cp.async.bulk.tensor,
//    no multicast) of the two activation tiles and of the raw int8 weight tile into a
//    3-stage ring of 32-element k blocks (64-byte swizzle rows); warps 2..9 convert the
//    int8 tile to bf16 in the swizzled layout the tensor core reads; warp 1 issues
//    tcgen05.mma (kind::f16, 128 x 128 x 16 per instruction, two terms x two k steps per
//    stage) and commits the stage back to the loader.  Few output tiles: the k range is
//    split over gridDim.z CTAs and a second kernel adds the partial tiles in split order.
//  * dense (256 rows and more: prefill).  A pass over the weights writes a slab of rows as
//    bf16 first (64 MB of workspace, a few percent of the GEMM's time); the GEMM then loads
//    both operands with TMA and nothing is converted in the main loop.  The main loop is
//    bound by the bytes brought from L2 into shared memory, so a CTA takes 256 weight rows
//    (one activation tile feeds two 128-column halves of a 256-column accumulator) when that
//    still leaves enough CTAs to fill the machine.
// Two CTAs are resident per SM (3 x 28 KB or 3 x 32 KB of ring, 128 or 256 of the 512
// tensor-memory columns each), so one CTA's epilogue runs under the other's main loop.
// Epilogue: warps 2..9 read the accumulator with tcgen05.ld (a thread owns a row), apply
// scale / bias / SiLU-gate, stage the tile in the idle ring and write whole rows with
// 16-byte stores (adding the residual there).
//
// Every wait is bounded (poll count and wall time); on expiry the CTA records
// an error, all roles fall through, tensor memory is released and the host
// call fails.
#include "common.cuh"

#include <cuda.h>

#include <algorithm>
#include <mutex>

namespace b200 {

namespace {

constexpr int BM = 128, BN = 128;              // output tile of one CTA
constexpr int kMaxStages = 8;
// warp 0 loader, warp 1 mma, then 8 conversion + epilogue warps (epilogue only when the
// weights arrive as bf16)
constexpr int kThreadsConv = 320, kThreadsPre = 320;
constexpr int kMaxPartialTiles = 320;          // split-K: 128 x 128 f32 partial tiles in the workspace
constexpr uint32_t kSpin = 1u << 26;
constexpr unsigned long long kWaitNs = 2000000000ull;

// Shared-memory stage for a k block of BKT elements (64: 128-byte swizzle rows, 32: 64-byte rows).
// PRE: the weight tile is loaded as bf16 (converted by a pass over the weights before the
// GEMM); else the raw int8 tile is loaded and converted by the CTA.
template <int BKT, bool PRE, int BNT = BN> struct Tile {
  static constexpr uint32_t A_BYTES = BM * BKT * 2;              // one bf16 term of the activations
  static constexpr uint32_t WRAW_BYTES = PRE ? 0 : BNT * BKT;    // int8 weights as stored
  static constexpr uint32_t WB_BYTES = BNT * BKT * 2;            // the weight tile as bf16
  static constexpr uint32_t STAGE_BYTES = 2 * A_BYTES + WRAW_BYTES + WB_BYTES;
  static constexpr uint32_t ROW_BYTES = BKT * 2;
};

struct Bars {
  uint64_t full[kMaxStages];   // TMA bytes of the stage have landed
  uint64_t ready[kMaxStages];  // the bf16 weight tile has been written (128 arrivals)
  uint64_t empty[kMaxStages];  // the tensor core is done with the stage
  uint64_t accum;              // all MMAs have completed
  uint32_t tmem_base;
  int abort_flag;
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ unsigned long long now_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint64_t *bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
               : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded wait; false when it gave up or the CTA already failed.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, volatile int *ab, int *err, int code) {
  unsigned long long t0 = 0;
  for (uint32_t it = 0; it < kSpin; ++it) {
    if (mbar_try(bar, parity))
      return !*ab;
    if ((it & 0x3FF) == 0x3FF) {
      if (*ab)
        return false;
      const unsigned long long t = now_ns();
      if (t0 == 0)
        t0 = t;
      else if (t - t0 > kWaitNs)
        break;
    }
  }
  atomicCAS(err, 0, code);
  *ab = 1;
  return false;
}
__device__ __forceinline__ void tma_load_2d(void *dst, const CUtensorMap *map, int x, int y, uint64_t *bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}
// K-major operand tile in shared memory, rows of 128 bytes (128-byte swizzle) or
// 64 bytes (64-byte swizzle): start address / 16, leading byte offset (unused for
// swizzled K-major: 1), stride byte offset = 8 rows, descriptor version 1,
// layout 2 (128-byte swizzle) or 4 (64-byte swizzle).
template <int BKT> __device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
  uint64_t d = 0;
  d |= (uint64_t)((addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)((8 * BKT * 2) >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)(BKT == 64 ? 2 : 4) << 61;
  return d;
}
// kind::f16 instruction descriptor: D = f32, A = B = bf16, both K-major, N = 128, M = 128.
template <int BNT> struct Idesc {
  static constexpr uint32_t value =
      (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BNT >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
};

template <int BNT>
__device__ __forceinline__ void mma_bf16(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(Idesc<BNT>::value), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tc_commit(uint64_t *bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

struct GemmParams {
  int M, N, K;                 // N = weight rows covered by this launch; K = packed k (multiple of 64)
  int n_off;                   // first weight row of the launch: scale, bias, residual and C are indexed n_off + n
  const float *scale;          // [N]
  const float *bias;           // [N] or null
  const float *residual;       // [M, ldr] or null
  float *C;                    // [M, ldc]
  int64_t ldc, ldr;
  int silu_pairs;              // rows (2j, 2j+1) of W are (gate_j, up_j): C[m, j] = silu(g) * u, ldc counts N/2 columns
  int stages;                  // ring depth (<= kMaxStages)
  int splits;                  // CTAs along K per output tile (gridDim.z); > 1: raw sums go to `partial`
  float *partial;              // [tiles][splits][128][128] f32
  int *error;
};

// scale / bias / residual, or the SiLU-gate of a (gate, up) column pair
__device__ __forceinline__ void store_plain(const GemmParams &p, int m, int n, float acc) {
  n += p.n_off;
  float y = __fmul_rn(acc, __ldg(p.scale + n));
  if (p.bias)
    y = __fadd_rn(y, __ldg(p.bias + n));
  if (p.residual)
    y = __fadd_rn(p.residual[(int64_t)m * p.ldr + n], y);
  p.C[(int64_t)m * p.ldc + n] = y;
}
__device__ __forceinline__ void store_pair(const GemmParams &p, int m, int n, float ag, float au) {
  n += p.n_off;
  float g = __fmul_rn(ag, __ldg(p.scale + n));
  float u = __fmul_rn(au, __ldg(p.scale + n + 1));
  if (p.bias) {
    g = __fadd_rn(g, __ldg(p.bias + n));
    u = __fadd_rn(u, __ldg(p.bias + n + 1));
  }
  const float sg = 1.0f / (1.0f + expf(-g));   // subgraph0_decode_simplify.mlir:226-231
  p.C[(int64_t)m * p.ldc + (n >> 1)] = __fmul_rn(__fmul_rn(g, sg), u);
}

// BNT: weight rows (output columns) per CTA: 128, or 256 on the dense path, where one
// activation tile then feeds twice the tensor-core work per byte brought in from L2.
template <int BKT, bool PRE, int BNT>
__global__ void __launch_bounds__(PRE ? kThreadsPre : kThreadsConv, BKT == 64 ? 1 : 2)
gemm_w8_tc_kernel(const __grid_constant__ CUtensorMap map_hi, const __grid_constant__ CUtensorMap map_lo,
                  const __grid_constant__ CUtensorMap map_w, const GemmParams p) {
  using T = Tile<BKT, PRE, BNT>;
  static_assert(PRE || BNT == BN, "the converting kernel takes 128 weight rows per CTA");
  constexpr int kEpiWarps = 8;
  extern __shared__ __align__(1024) uint8_t smem[];
  // 1024-byte alignment of every swizzled tile
  uint8_t *tiles = reinterpret_cast<uint8_t *>(((uintptr_t)smem + 1023) & ~(uintptr_t)1023);
  const int stages = p.stages;
  Bars &bars = *reinterpret_cast<Bars *>(tiles + stages * T::STAGE_BYTES);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BNT;
  // this CTA's share of the k blocks (split-K: blockIdx.z)
  const int nkb_all = p.K / BKT;
  const int kb0 = (int)((int64_t)nkb_all * blockIdx.z / p.splits);
  const int nkb = (int)((int64_t)nkb_all * (blockIdx.z + 1) / p.splits) - kb0;
  volatile int *ab = &bars.abort_flag;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(&bars.full[s], 1);
      mbar_init(&bars.ready[s], 256);
      mbar_init(&bars.empty[s], 1);
    }
    mbar_init(&bars.accum, 1);
    bars.abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {   // tensor memory: one warp allocates, the same warp frees
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&bars.tmem_base)), "n"(BNT) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = bars.tmem_base;

  if (warp == 0) {
    // ---- loader ------------------------------------------------------------------
    if (lane == 0) {
      for (int i = 0; i < nkb; ++i) {
        const int s = i % stages, use = i / stages;
        if (use > 0 && !mbar_wait(&bars.empty[s], (use - 1) & 1, ab, p.error, 701))
          break;
        uint8_t *st = tiles + s * T::STAGE_BYTES;
        const int kx = (kb0 + i) * BKT;
        mbar_expect_tx(&bars.full[s], 2 * T::A_BYTES + (PRE ? T::WB_BYTES : T::WRAW_BYTES));
        tma_load_2d(st, &map_hi, kx, m0, &bars.full[s]);
        tma_load_2d(st + T::A_BYTES, &map_lo, kx, m0, &bars.full[s]);
        tma_load_2d(st + 2 * T::A_BYTES, &map_w, kx, n0, &bars.full[s]);   // PRE: lands as the bf16 tile
      }
    }
  } else if (warp == 1) {
    // ---- tensor core issue (one thread) ------------------------------------------------
    if (lane == 0) {
      for (int i = 0; i < nkb; ++i) {
        const int s = i % stages, use = i / stages;
        if (!mbar_wait(&bars.full[s], use & 1, ab, p.error, 702))
          break;
        if (!PRE && !mbar_wait(&bars.ready[s], use & 1, ab, p.error, 703))
          break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t a_hi = smem_u32(tiles + s * T::STAGE_BYTES), a_lo = a_hi + T::A_BYTES,
                       wb = a_hi + 2 * T::A_BYTES + T::WRAW_BYTES;
#pragma unroll
        for (int k = 0; k < BKT / 16; ++k) {   // 16 bf16 = 32 bytes along the swizzled row
          const uint64_t db = smem_desc<BKT>(wb + k * 32);
          mma_bf16<BNT>(tmem, smem_desc<BKT>(a_hi + k * 32), db, (i | k) != 0);
          mma_bf16<BNT>(tmem, smem_desc<BKT>(a_lo + k * 32), db, 1u);
        }
        tc_commit(&bars.empty[s]);   // arrives when the MMAs above have read the stage
      }
      tc_commit(&bars.accum);
    }
  } else {
    bool alive = true;
    if (!PRE) {
      // ---- int8 -> bf16 conversion of the weight tile: 256 threads, two per weight row --------
      const int t = threadIdx.x - 64;           // 0..255
      const int r = t & 127, half = t >> 7;
      constexpr int NQ = BKT / 32;              // 16-byte units of raw weights per thread
      // 16-byte chunk c of row r of a swizzled tile sits at chunk c ^ swz(r)
      const int swz = BKT == 64 ? (r & 7) : ((r >> 1) & 3);
      for (int i = 0; i < nkb && alive; ++i) {
        const int s = i % stages, use = i / stages;
        if (!mbar_wait(&bars.full[s], use & 1, ab, p.error, 704)) {
          alive = false;
          break;
        }
        uint8_t *st = tiles + s * T::STAGE_BYTES;
        const uint4 *raw = reinterpret_cast<const uint4 *>(st + 2 * T::A_BYTES + r * BKT);
        uint8_t *dst = st + 2 * T::A_BYTES + T::WRAW_BYTES + r * T::ROW_BYTES;   // row r of the swizzled bf16 tile
#pragma unroll
        for (int qq = 0; qq < NQ; ++qq) {         // 16 int8 -> two 16-byte chunks of bf16
          // neighbouring rows start at different 16-byte units (fewer bank conflicts on the raw reads)
          const int q = half * NQ + ((qq + (r >> 1)) & (NQ - 1));
          const uint4 w = raw[q];
          const uint32_t ws[4] = {w.x ^ 0x80808080u, w.y ^ 0x80808080u, w.z ^ 0x80808080u, w.w ^ 0x80808080u};
          uint32_t o[8];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            // byte u = q + 128 placed in the mantissa of 2^23: (2^23 + u) - (2^23 + 128) = q, exact
            const float f0 = __uint_as_float(__byte_perm(ws[j], 0x4B000000u, 0x7440)) - 8388736.0f;
            const float f1 = __uint_as_float(__byte_perm(ws[j], 0x4B000000u, 0x7441)) - 8388736.0f;
            const float f2 = __uint_as_float(__byte_perm(ws[j], 0x4B000000u, 0x7442)) - 8388736.0f;
            const float f3 = __uint_as_float(__byte_perm(ws[j], 0x4B000000u, 0x7443)) - 8388736.0f;
            // an integer of magnitude <= 128 is its own bf16: keep the upper halves
            o[2 * j] = __byte_perm(__float_as_uint(f0), __float_as_uint(f1), 0x7632);
            o[2 * j + 1] = __byte_perm(__float_as_uint(f2), __float_as_uint(f3), 0x7632);
          }
          const int c0 = 2 * q, c1 = 2 * q + 1;
          *reinterpret_cast<uint4 *>(dst + ((c0 ^ swz) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
          *reinterpret_cast<uint4 *>(dst + ((c1 ^ swz) << 4)) = make_uint4(o[4], o[5], o[6], o[7]);
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic writes -> visible to the tensor core's reads
        mbar_arrive(&bars.ready[s]);
      }
    }
    // ---- epilogue ---------------------------------------------------------------------
    // A thread owns one accumulator row (its lane of tensor memory) and half of its columns.
    // Scaled values go to a padded tile in shared memory (the ring is idle by now; row stride
    // 132 floats keeps 16-byte stores of neighbouring rows on different banks), then the warps
    // write whole rows with 16-byte stores.
    const bool ok = alive && mbar_wait(&bars.accum, 0, ab, p.error, 705);
    constexpr int LDS = BN + 4;                       // row stride of the staging tile, in floats
    float *ep = reinterpret_cast<float *>(tiles);     // [BM][LDS]: 66 KB <= the ring
    const int width = p.splits > 1 ? BN : (p.silu_pairs ? BN / 2 : BN);
#pragma unroll 1
    for (int h = 0; h < BNT / BN; ++h) {   // 128 columns of the accumulator at a time
    const int n0h = n0 + h * BN;
    if (h > 0)   // the staging tile is free again once the previous half has been stored
      asm volatile("bar.sync 1, %0;" ::"n"(kEpiWarps * 32) : "memory");
    // rows of the tile beyond M hold nothing: warps whose 32 lanes are all dead skip the read
    if (ok && n0h < p.N && (warp & 3) * 32 < p.M - m0) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      // a warp reads the 32 lanes of tensor memory that match its rank within its warpgroup;
      // the two warps that share a lane quarter take half the columns each
      const int quad = warp & 3;
      const int row = quad * 32 + lane;
      const int cb0 = ((warp - 2) >> 2) * (BN / 2), cb1 = cb0 + BN / 2;
#pragma unroll 1
      for (int cb = cb0; cb < cb1; cb += 32) {
        uint32_t v[32];
        const uint32_t taddr = tmem + ((uint32_t)(quad * 32) << 16) + (uint32_t)(h * BN + cb);
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
            "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
            "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
            : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
              "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
              "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
              "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
            : "r"(taddr)
            : "memory");
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        float *erow = ep + row * LDS;
        if (p.splits > 1) {
          // split-K: raw sums of this CTA's k range; gemm_w8_combine_kernel adds the splits
#pragma unroll
          for (int j = 0; j < 32; j += 4)
            *reinterpret_cast<float4 *>(erow + cb + j) =
                make_float4(__uint_as_float(v[j]), __uint_as_float(v[j + 1]), __uint_as_float(v[j + 2]),
                            __uint_as_float(v[j + 3]));
        } else if (p.silu_pairs) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            float o[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int n = min(n0h + cb + j + 2 * e, p.N - 2) + p.n_off;   // columns beyond N are not stored
              const float2 sc2 = __ldg(reinterpret_cast<const float2 *>(p.scale + n));
              float g = __fmul_rn(__uint_as_float(v[j + 2 * e]), sc2.x);
              float u = __fmul_rn(__uint_as_float(v[j + 2 * e + 1]), sc2.y);
              if (p.bias) {
                g = __fadd_rn(g, __ldg(p.bias + n));
                u = __fadd_rn(u, __ldg(p.bias + n + 1));
              }
              const float sg = 1.0f / (1.0f + expf(-g));   // subgraph0_decode_simplify.mlir:226-231
              o[e] = __fmul_rn(__fmul_rn(g, sg), u);
            }
            *reinterpret_cast<float4 *>(erow + ((cb + j) >> 1)) = make_float4(o[0], o[1], o[2], o[3]);
          }
        } else {
#pragma unroll
          for (int j = 0; j < 32; j += 4) {
            float o[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int n = min(n0h + cb + j + e, p.N - 1) + p.n_off;
              float y = __fmul_rn(__uint_as_float(v[j + e]), __ldg(p.scale + n));
              if (p.bias)
                y = __fadd_rn(y, __ldg(p.bias + n));
              o[e] = y;
            }
            *reinterpret_cast<float4 *>(erow + cb + j) = make_float4(o[0], o[1], o[2], o[3]);
          }
        }
      }
    }
    // all epilogue warps, whether they hold data or gave up: named barrier 1
    asm volatile("bar.sync 1, %0;" ::"n"(kEpiWarps * 32) : "memory");
    if (ok && n0h < p.N) {
      const int ew = warp - 2;
      float *dst;
      int64_t ldd;
      int cols;                    // valid columns of this tile in the destination
      if (p.splits > 1) {
        const int64_t tile = (int64_t)blockIdx.y * gridDim.x + blockIdx.x;
        dst = p.partial + (tile * p.splits + blockIdx.z) * BM * BN;
        ldd = BN;
        cols = BN;
      } else if (p.silu_pairs) {
        dst = p.C + (int64_t)m0 * p.ldc + ((n0h + p.n_off) >> 1);
        ldd = p.ldc;
        cols = min(BN, p.N - n0h) >> 1;
      } else {
        dst = p.C + (int64_t)m0 * p.ldc + n0h + p.n_off;
        ldd = p.ldc;
        cols = min(BN, p.N - n0h);
      }
      const float *res = (p.residual && p.splits == 1 && !p.silu_pairs) ? p.residual + (int64_t)m0 * p.ldr + n0h + p.n_off : nullptr;
      const int rows = min(BM, p.M - m0);
      // 16-byte stores when the destination rows allow it
      const bool v4 = (ldd & 3) == 0 && ((uintptr_t)dst & 15) == 0 && (cols & 3) == 0 &&
                      (!res || ((p.ldr & 3) == 0 && ((uintptr_t)res & 15) == 0));
      if (v4) {
        const int per_row = width / 4;                 // float4 per row: 32 or 16
        for (int idx = ew * 32 + lane; idx < rows * per_row; idx += kEpiWarps * 32) {
          const int r = idx / per_row, c = (idx - r * per_row) * 4;
          if (c < cols) {
            float4 y = *reinterpret_cast<const float4 *>(ep + r * LDS + c);
            if (res) {
              const float4 q = *reinterpret_cast<const float4 *>(res + (int64_t)r * p.ldr + c);
              y.x = __fadd_rn(q.x, y.x);
              y.y = __fadd_rn(q.y, y.y);
              y.z = __fadd_rn(q.z, y.z);
              y.w = __fadd_rn(q.w, y.w);
            }
            *reinterpret_cast<float4 *>(dst + (int64_t)r * ldd + c) = y;
          }
        }
      } else {
        for (int r = ew; r < rows; r += kEpiWarps) {
          for (int c = lane; c < width; c += 32) {
            if (c < cols) {
              float y = ep[r * LDS + c];
              if (res)
                y = __fadd_rn(res[(int64_t)r * p.ldr + c], y);
              dst[(int64_t)r * ldd + c] = y;
            }
          }
        }
      }
    }
    }   // halves
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    if (*ab) {   // copies of an abandoned tile may still be in flight: let them land before the CTA ends
      const unsigned long long t0 = now_ns();
      while (now_ns() - t0 < 2000000ull) {
      }
    }
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "n"(BNT) : "memory");
  }
}

// int8 rows [rows][K] (packed k order) -> bf16, same order: the weight operand of the
// dense path.  One 16-byte unit per thread.
__global__ void __launch_bounds__(256)
weights_to_bf16_kernel(const uint8_t *w, int64_t units, uint4 *out) {
  for (int64_t u = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; u < units; u += (int64_t)gridDim.x * blockDim.x) {
    const uint4 x = __ldg(reinterpret_cast<const uint4 *>(w) + u);
    const uint32_t ws[4] = {x.x ^ 0x80808080u, x.y ^ 0x80808080u, x.z ^ 0x80808080u, x.w ^ 0x80808080u};
    uint32_t o[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float f0 = __uint_as_float(__byte_perm(ws[j], 0x4B000000u, 0x7440)) - 8388736.0f;
      const float f1 = __uint_as_float(__byte_perm(ws[j], 0x4B000000u, 0x7441)) - 8388736.0f;
      const float f2 = __uint_as_float(__byte_perm(ws[j], 0x4B000000u, 0x7442)) - 8388736.0f;
      const float f3 = __uint_as_float(__byte_perm(ws[j], 0x4B000000u, 0x7443)) - 8388736.0f;
      o[2 * j] = __byte_perm(__float_as_uint(f0), __float_as_uint(f1), 0x7632);
      o[2 * j + 1] = __byte_perm(__float_as_uint(f2), __float_as_uint(f3), 0x7632);
    }
    out[2 * u] = make_uint4(o[0], o[1], o[2], o[3]);
    out[2 * u + 1] = make_uint4(o[4], o[5], o[6], o[7]);
  }
}

// Split-K: add the splits of every output tile in split order, then the epilogue.
// grid (tiles, BM / 8): a CTA of 256 threads takes 8 rows of a tile, a thread 4 columns.
__global__ void __launch_bounds__(256)
gemm_w8_combine_kernel(const GemmParams p, int tiles_x) {
  const int tile = blockIdx.x;
  const int m0 = (tile / tiles_x) * BM, n0 = (tile % tiles_x) * BN;
  const int r = blockIdx.y * 8 + (threadIdx.x >> 5), c = (threadIdx.x & 31) * 4;
  const int m = m0 + r, n = n0 + c;
  if (m >= p.M || n >= p.N)
    return;
  const float *base = p.partial + (int64_t)tile * p.splits * BM * BN + r * BN + c;
  float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int z = 0; z < p.splits; ++z) {
    const float4 v = *reinterpret_cast<const float4 *>(base + (int64_t)z * BM * BN);
    a.x = __fadd_rn(a.x, v.x);
    a.y = __fadd_rn(a.y, v.y);
    a.z = __fadd_rn(a.z, v.z);
    a.w = __fadd_rn(a.w, v.w);
  }
  if (p.silu_pairs) {
    if (n + 1 < p.N)
      store_pair(p, m, n, a.x, a.y);
    if (n + 3 < p.N)
      store_pair(p, m, n + 2, a.z, a.w);
  } else {
    store_plain(p, m, n, a.x);
    if (n + 1 < p.N) store_plain(p, m, n + 1, a.y);
    if (n + 2 < p.N) store_plain(p, m, n + 2, a.z);
    if (n + 3 < p.N) store_plain(p, m, n + 3, a.w);
  }
}

// A[M,K] f32 -> hi/lo bf16 [Mpad, Kp] in the k order of the packed weight rows.
// Optional RMSNorm of every row first (y = w * (x * r), subgraph0_decode_simplify.mlir:60-72).
// A thread converts four consecutive k: they share a 16-byte unit of the packed row, so
// they land on four consecutive bf16.  Rows beyond M are written as zeros.
__global__ void __launch_bounds__(256)
split_activations_kernel(const float *A, int64_t lda, int M, int K, int Kp, const float *norm_w, float eps,
                         __nv_bfloat16 *hi, __nv_bfloat16 *lo) {
  const int m = blockIdx.x;
  __shared__ float s_red[32];
  float r = 1.f;
  const bool live = m < M;
  const float *arow = A + (int64_t)m * lda;
  const bool vec = (K & 3) == 0 && (lda & 3) == 0 && ((uintptr_t)A & 15) == 0;
  if (norm_w != nullptr && live) {
    float ss = 0.f;
    for (int k = threadIdx.x; k < K; k += blockDim.x) {
      const float x = arow[k];
      ss += x * x;
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0)
      s_red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float t = 0.f;
    for (int w = 0; w < (int)(blockDim.x + 31) / 32; ++w)
      t += s_red[w];
    r = rsqrtf(__fadd_rn(__fmul_rn(t, 1.0f / (float)K), eps));
  }
  uint2 *hrow = reinterpret_cast<uint2 *>(hi + (int64_t)m * Kp), *lrow = reinterpret_cast<uint2 *>(lo + (int64_t)m * Kp);
  for (int k = threadIdx.x * 4; k < Kp; k += blockDim.x * 4) {
    float a[4] = {0.f, 0.f, 0.f, 0.f};
    if (live && k < K) {
      if (vec) {
        const float4 v = *reinterpret_cast<const float4 *>(arow + k);
        a[0] = v.x; a[1] = v.y; a[2] = v.z; a[3] = v.w;
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e)
          if (k + e < K)
            a[e] = arow[k + e];
      }
      if (norm_w != nullptr) {
#pragma unroll
        for (int e = 0; e < 4; ++e)
          if (k + e < K)
            a[e] = __fmul_rn(norm_w[k + e], __fmul_rn(a[e], r));
      }
    }
    __nv_bfloat16 h[4], l[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      h[e] = __float2bfloat16_rn(a[e]);
      l[e] = __float2bfloat16_rn(a[e] - __bfloat162float(h[e]));
    }
    // position of k (a multiple of 4) in the packed row: a full block of 512 elements by shifts
    int64_t pos;
    if ((k | 511) < (K & ~511)) {
      const int kk = k & 511;
      pos = (k & ~511) + ((kk & 127) >> 2) * 16 + (kk >> 7) * 4;
    } else {
      pos = k < K ? packed_offset(B200_W_I8, K, k, nullptr) : k;
    }
    uint2 hv, lv;
    hv.x = (uint32_t)__bfloat16_as_ushort(h[0]) | ((uint32_t)__bfloat16_as_ushort(h[1]) << 16);
    hv.y = (uint32_t)__bfloat16_as_ushort(h[2]) | ((uint32_t)__bfloat16_as_ushort(h[3]) << 16);
    lv.x = (uint32_t)__bfloat16_as_ushort(l[0]) | ((uint32_t)__bfloat16_as_ushort(l[1]) << 16);
    lv.y = (uint32_t)__bfloat16_as_ushort(l[2]) | ((uint32_t)__bfloat16_as_ushort(l[3]) << 16);
    hrow[pos >> 2] = hv;
    lrow[pos >> 2] = lv;
  }
}

// ---- W8A8: int8 activations x int8 weights on the integer tensor-core path -----------------
// buddy-mlir's QuantizedMatmulOp (frontend/Python/ops/linalg.py:12728-12846): one scale for
// the whole activation tensor, s = max(absmax / 127, 1e-10), q = clamp(rne(x * (1 / s)), -128,
// 127), an exact i8 x i8 -> i32 contraction, y = float(acc) * (s * weight_scale[n]) (+ bias).
// Every step is reproduced operation by operation, so the result is bit-identical to the
// reference arithmetic.  Both operands are loaded by TMA as stored (64-byte swizzle applied by
// the copy), tcgen05.mma kind::i8 accumulates s32 in tensor memory: no conversion anywhere.
constexpr int BK8 = 64;                        // int8 per k block = one 64-byte swizzle row
constexpr int kStages8 = 5;                    // 5 x 16 KB: the ring also stages the epilogue tile
constexpr uint32_t kTile8 = BM * BK8;          // 8 KB per operand tile
constexpr uint32_t kIdescI8 = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);

__device__ __forceinline__ void mma_i8(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(kIdescI8), "r"(accumulate)
      : "memory");
}

struct W8A8Params {
  int M, N, K;
  const float *wscale, *bias;
  const float *act_scale;      // device scalar written by quantize_activations_kernel
  float *C;
  int64_t ldc;
  const float *residual;       // optional: C = residual + y (may be C itself)
  int64_t ldr;
  int silu_pairs;              // columns are (gate, up) pairs: C[m, j] = silu(y[m, 2j]) * y[m, 2j + 1]
  int *error;
};

__global__ void __launch_bounds__(kThreadsPre, 2)
gemm_w8a8_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                    const W8A8Params p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t *tiles = reinterpret_cast<uint8_t *>(((uintptr_t)smem + 1023) & ~(uintptr_t)1023);
  Bars &bars = *reinterpret_cast<Bars *>(tiles + kStages8 * 2 * kTile8);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int nkb = p.K / BK8;
  volatile int *ab = &bars.abort_flag;
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages8; ++s) {
      mbar_init(&bars.full[s], 1);
      mbar_init(&bars.empty[s], 1);
    }
    mbar_init(&bars.accum, 1);
    bars.abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&bars.tmem_base)), "n"(BN) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = bars.tmem_base;

  if (warp == 0) {
    if (lane == 0) {
      for (int i = 0; i < nkb; ++i) {
        const int s = i % kStages8, use = i / kStages8;
        if (use > 0 && !mbar_wait(&bars.empty[s], (use - 1) & 1, ab, p.error, 711))
          break;
        uint8_t *st = tiles + s * 2 * kTile8;
        mbar_expect_tx(&bars.full[s], 2 * kTile8);
        tma_load_2d(st, &map_a, i * BK8, m0, &bars.full[s]);
        tma_load_2d(st + kTile8, &map_w, i * BK8, n0, &bars.full[s]);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      for (int i = 0; i < nkb; ++i) {
        const int s = i % kStages8, use = i / kStages8;
        if (!mbar_wait(&bars.full[s], use & 1, ab, p.error, 712))
          break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t a = smem_u32(tiles + s * 2 * kTile8), w = a + kTile8;
#pragma unroll
        for (int k = 0; k < BK8 / 32; ++k)   // 32 int8 = 32 bytes along the swizzled row
          mma_i8(tmem, smem_desc<32>(a + k * 32), smem_desc<32>(w + k * 32), (i | k) != 0);
        tc_commit(&bars.empty[s]);
      }
      tc_commit(&bars.accum);
    }
  } else {
    const bool ok = mbar_wait(&bars.accum, 0, ab, p.error, 713);
    constexpr int LDS = BN + 4;
    float *ep = reinterpret_cast<float *>(tiles);   // [BM][LDS] staged in the idle ring
    if (ok) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const float sa = *p.act_scale;
      const int quad = warp & 3;
      const int row = quad * 32 + lane;
      const int cb0 = ((warp - 2) >> 2) * (BN / 2), cb1 = cb0 + BN / 2;
#pragma unroll 1
      for (int cb = cb0; cb < cb1; cb += 32) {
        uint32_t v[32];
        const uint32_t taddr = tmem + ((uint32_t)(quad * 32) << 16) + (uint32_t)cb;
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
            "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
            "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
            : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
              "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
              "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
              "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
            : "r"(taddr)
            : "memory");
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        float *erow = ep + row * LDS;
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
          float o[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int n = min(n0 + cb + j + e, p.N - 1);
            // linalg.py:12836-12846: float(acc) * (act_scale * weight_scale[n])
            float y = __fmul_rn(__int2float_rn((int)v[j + e]), __fmul_rn(sa, __ldg(p.wscale + n)));
            if (p.bias)
              y = __fadd_rn(y, __ldg(p.bias + n));
            o[e] = y;
          }
          *reinterpret_cast<float4 *>(erow + cb + j) = make_float4(o[0], o[1], o[2], o[3]);
        }
      }
    }
    asm volatile("bar.sync 1, %0;" ::"n"(8 * 32) : "memory");
    if (ok) {
      const int ew = warp - 2;
      const int rows = min(BM, p.M - m0), cols = min(BN, p.N - n0);
      if (p.silu_pairs) {   // subgraph0_decode_simplify.mlir:226-231 on neighbouring columns
        float *dst = p.C + (int64_t)m0 * p.ldc + (n0 >> 1);
        for (int r = ew; r < rows; r += 8)
          for (int c = lane; c < (cols >> 1); c += 32) {
            const float g = ep[r * LDS + 2 * c], u = ep[r * LDS + 2 * c + 1];
            const float s = 1.0f / (1.0f + expf(-g));
            dst[(int64_t)r * p.ldc + c] = __fmul_rn(__fmul_rn(g, s), u);
          }
      } else {
        float *dst = p.C + (int64_t)m0 * p.ldc + n0;
        const float *res = p.residual ? p.residual + (int64_t)m0 * p.ldr + n0 : nullptr;
        for (int r = ew; r < rows; r += 8)
          for (int c = lane; c < cols; c += 32) {
            float y = ep[r * LDS + c];
            if (res)
              y = __fadd_rn(res[(int64_t)r * p.ldr + c], y);
            dst[(int64_t)r * p.ldc + c] = y;
          }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    if (*ab) {
      const unsigned long long t0 = now_ns();
      while (now_ns() - t0 < 2000000ull) {
      }
    }
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "n"(BN) : "memory");
  }
}

// max |x| over the whole tensor (non-negative floats order like their bit patterns)
__global__ void __launch_bounds__(256)
absmax_kernel(const float *A, int64_t lda, int M, int K, uint32_t *out) {
  float mx = 0.f;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < (int64_t)M * K; i += (int64_t)gridDim.x * blockDim.x) {
    const int m = (int)(i / K), k = (int)(i - (int64_t)m * K);
    mx = fmaxf(mx, fabsf(A[(int64_t)m * lda + k]));
  }
  mx = warp_max(mx);
  if ((threadIdx.x & 31) == 0)
    atomicMax(out, __float_as_uint(mx));
}

// linalg.py:12728-12792 for four consecutive k per thread, written in the k order of the packed
// weight rows; thread 0 of the grid also leaves the scale for the GEMM's epilogue.
__global__ void __launch_bounds__(256)
quantize_activations_kernel(const float *A, int64_t lda, int M, int K, const uint32_t *absmax, float *scale_out,
                            uint32_t *q) {
  const float scale = fmaxf(__fmul_rn(__uint_as_float(*absmax), __fdiv_rn(1.0f, 127.0f)), 1e-10f);
  const float inv = __fdiv_rn(1.0f, scale);
  if (blockIdx.x == 0 && threadIdx.x == 0)
    *scale_out = scale;
  const int m = blockIdx.x;
  const float *arow = A + (int64_t)m * lda;
  uint32_t *qrow = q + (int64_t)m * (K / 4);
  for (int k = threadIdx.x * 4; k < K; k += blockDim.x * 4) {
    uint32_t pk = 0;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      float r = rintf(__fmul_rn(arow[k + e], inv));     // the f32 -> i32 cast rounds to nearest even
      r = fminf(fmaxf(r, -128.0f), 127.0f);
      pk |= ((uint32_t)(int)r & 0xFFu) << (8 * e);
    }
    int64_t pos;
    if ((k | 511) < (K & ~511)) {
      const int kk = k & 511;
      pos = (k & ~511) + ((kk & 127) >> 2) * 16 + (kk >> 7) * 4;
    } else {
      pos = packed_offset(B200_W_I8, K, k, nullptr);
    }
    qrow[pos >> 2] = pk;
  }
}

// The same split with a warp per row (eight rows per CTA) for aligned rows of up to 2048
// elements: the row is read once and stays in registers between the RMSNorm statistics and
// the conversion, and nothing waits on a CTA barrier.
template <int NV>   // float4 per lane: K <= 128 * NV
__global__ void __launch_bounds__(256)
split_activations_warp_kernel(const float *A, int64_t lda, int M, int K, const float *norm_w, float eps,
                              __nv_bfloat16 *hi, __nv_bfloat16 *lo) {
  const int lane = threadIdx.x & 31;
  const int m = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (m >= M)
    return;
  const float *arow = A + (int64_t)m * lda;
  float4 v[NV];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int k = (i * 32 + lane) * 4;
    v[i] = k < K ? *reinterpret_cast<const float4 *>(arow + k) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  float r = 1.f;
  if (norm_w != nullptr) {
    // the statistics in the order of the CTA-per-row kernel would differ in rounding only; both
    // stay far inside the tolerance of the contraction that follows
#pragma unroll
    for (int i = 0; i < NV; ++i)
      ss += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
    ss = warp_sum(ss);
    r = rsqrtf(__fadd_rn(__fmul_rn(ss, 1.0f / (float)K), eps));
  }
  uint2 *hrow = reinterpret_cast<uint2 *>(hi + (int64_t)m * K), *lrow = reinterpret_cast<uint2 *>(lo + (int64_t)m * K);
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int k = (i * 32 + lane) * 4;
    if (k >= K)
      break;
    float a[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
    if (norm_w != nullptr) {
      const float4 w4 = *reinterpret_cast<const float4 *>(norm_w + k);
      a[0] = __fmul_rn(w4.x, __fmul_rn(a[0], r));
      a[1] = __fmul_rn(w4.y, __fmul_rn(a[1], r));
      a[2] = __fmul_rn(w4.z, __fmul_rn(a[2], r));
      a[3] = __fmul_rn(w4.w, __fmul_rn(a[3], r));
    }
    uint32_t hb[4], lb[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const __nv_bfloat16 h = __float2bfloat16_rn(a[e]);
      hb[e] = __bfloat16_as_ushort(h);
      lb[e] = __bfloat16_as_ushort(__float2bfloat16_rn(a[e] - __bfloat162float(h)));
    }
    int64_t pos;
    if ((k | 511) < (K & ~511)) {
      const int kk = k & 511;
      pos = (k & ~511) + ((kk & 127) >> 2) * 16 + (kk >> 7) * 4;
    } else {
      pos = packed_offset(B200_W_I8, K, k, nullptr);
    }
    hrow[pos >> 2] = make_uint2(hb[0] | (hb[1] << 16), hb[2] | (hb[3] << 16));
    lrow[pos >> 2] = make_uint2(lb[0] | (lb[1] << 16), lb[2] | (lb[3] << 16));
  }
}

using EncodeFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                              const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn encode_fn() {
  static EncodeFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeFn>(p);
  });
  return fn;
}

int make_map(CUtensorMap *map, CUtensorMapDataType dt, int bk, void *base, uint64_t inner, uint64_t rows,
             uint64_t pitch_bytes, CUtensorMapSwizzle swz, int box_rows = 128) {
  EncodeFn fn = encode_fn();
  if (!fn)
    return fail(B200_ECUDA, "gemm_w8: cuTensorMapEncodeTiled is not available from this driver");
  const cuuint64_t dims[2] = {inner, rows};
  const cuuint64_t strides[1] = {pitch_bytes};
  const cuuint32_t box[2] = {(cuuint32_t)bk, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult rc = fn(map, dt, 2, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS)
    return fail(B200_ECUDA, "gemm_w8: cuTensorMapEncodeTiled failed (%d)", (int)rc);
  return B200_OK;
}

} // namespace

} // namespace b200

using namespace b200;

// Rows of bf16 weights the dense path converts at a time (a slab of the workspace).
constexpr int64_t kSlabElems = (int64_t)32 << 20;   // 64 MB of bf16
constexpr int kDenseRows = 256;                      // from this many rows on, convert the weights once per call

template <int BKT, bool PRE, int BNT>
static int gemm_launch(const void *wbase, __nv_bfloat16 *hi, __nv_bfloat16 *lo, int Mp, GemmParams &p, int stages,
                       cudaStream_t st) {
  const int K = p.K, N = p.N;
  const CUtensorMapSwizzle swz = BKT == 64 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B;
  CUtensorMap map_hi, map_lo, map_w;
  if (int rc = make_map(&map_hi, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, BKT, hi, K, p.M, (uint64_t)K * 2, swz))
    return rc;
  if (int rc = make_map(&map_lo, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, BKT, lo, K, p.M, (uint64_t)K * 2, swz))
    return rc;
  if (PRE) {
    if (int rc = make_map(&map_w, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, BKT, const_cast<void *>(wbase), K, N,
                          (uint64_t)K * 2, swz, BNT))
      return rc;
  } else {
    if (int rc = make_map(&map_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, BKT, const_cast<void *>(wbase), K, N, (uint64_t)K,
                          CU_TENSOR_MAP_SWIZZLE_NONE, BNT))
      return rc;
  }
  static int configured[64] = {};
  int dev = 0;
  B200_CUDA(cudaGetDevice(&dev));
  const int smem = stages * (int)Tile<BKT, PRE, BNT>::STAGE_BYTES + 1024 + 256;
  if (dev < 0 || dev >= 64 || configured[dev] < smem) {
    B200_CUDA(cudaFuncSetAttribute(gemm_w8_tc_kernel<BKT, PRE, BNT>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    if (dev >= 0 && dev < 64)
      configured[dev] = smem;
  }
  if ((size_t)stages * Tile<BKT, PRE, BNT>::STAGE_BYTES < (size_t)BM * (BN + 4) * 4)
    return fail(B200_EINVAL, "gemm_w8: the ring is smaller than the epilogue's staging tile");
  p.stages = stages;
  const dim3 grid((N + BNT - 1) / BNT, Mp / BM, p.splits);
  gemm_w8_tc_kernel<BKT, PRE, BNT><<<grid, PRE ? kThreadsPre : kThreadsConv, smem, st>>>(map_hi, map_lo, map_w, p);
  B200_LAUNCH_CHECK();
  if (p.splits > 1) {
    gemm_w8_combine_kernel<<<dim3(grid.x * grid.y, BM / 8), 256, 0, st>>>(p, (int)grid.x);
    B200_LAUNCH_CHECK();
  }
  return B200_OK;
}

extern "C" {

int64_t b200_gemm_w8_workspace_bytes(int M, int64_t K) {
  if (M < 1 || K < 1)
    return 0;
  const int64_t Mp = (M + BM - 1) / BM * BM, Kp = packed_k(B200_W_I8, K);
  // an error word, hi and lo (bf16), the split-K partial tiles, and for the dense path a slab of bf16 weights
  return 256 + 2 * Mp * Kp * 2 + (int64_t)kMaxPartialTiles * BM * BN * 4 + (M >= kDenseRows ? kSlabElems * 2 : 0);
}

int b200_gemm_w8(const b200_weight *w, const float *A, int M, int64_t lda, float *C, int64_t ldc,
                 const float *residual, int64_t ldr, const float *norm_weight, float norm_eps,
                 int silu_pairs, void *workspace, int64_t workspace_bytes, void *stream) {
  if (!w || !A || !C || !workspace)
    return fail(B200_EINVAL, "gemm_w8: null argument");
  if (w->kind != B200_W_I8 || w->scale_dtype != B200_F32 || !w->scale || !w->w)
    return fail(B200_EINVAL, "gemm_w8: int8 per-channel weights with f32 scales expected");
  if (M < 1 || w->K % 64 != 0 || w->N < 1 || (silu_pairs && (w->N & 1)))
    return fail(B200_EINVAL, "gemm_w8: M >= 1, K a multiple of 64, even N for gate/up pairs");
  if (((uintptr_t)w->w & 15) || ((uintptr_t)workspace & 255))
    return fail(B200_EINVAL, "gemm_w8: weight rows must be 16-byte aligned, the workspace 256-byte aligned");
  if (workspace_bytes < b200_gemm_w8_workspace_bytes(M, w->K))
    return fail(B200_EINVAL, "gemm_w8: workspace too small");
  if (int rc = ensure_device())
    return rc;
  cudaStream_t st = (cudaStream_t)stream;
  const int K = (int)w->K, N = (int)w->N;
  const int Mp = (M + BM - 1) / BM * BM;
  int *err = reinterpret_cast<int *>(workspace);
  __nv_bfloat16 *hi = reinterpret_cast<__nv_bfloat16 *>((char *)workspace + 256);
  __nv_bfloat16 *lo = hi + (int64_t)Mp * K;
  float *partial = reinterpret_cast<float *>(lo + (int64_t)Mp * K);
  __nv_bfloat16 *slab = reinterpret_cast<__nv_bfloat16 *>(partial + (int64_t)kMaxPartialTiles * BM * BN);
  B200_CUDA(cudaMemsetAsync(err, 0, 4, st));
  // rows M..Mp of the last tile are never written: the tensor maps end at row M and the TMA
  // unit fills what lies beyond with zeros
  // many rows: a warp per row (less work per row); few rows: a CTA per row (more threads on the few)
  const bool warp_rows = M >= 512 && (K & 3) == 0 && (lda & 3) == 0 && ((uintptr_t)A & 15) == 0 && K <= 2048 &&
                         (!norm_weight || ((uintptr_t)norm_weight & 15) == 0);
  if (warp_rows && K <= 1536)
    split_activations_warp_kernel<12><<<(M + 7) / 8, 256, 0, st>>>(A, lda, M, K, norm_weight, norm_eps, hi, lo);
  else if (warp_rows)
    split_activations_warp_kernel<16><<<(M + 7) / 8, 256, 0, st>>>(A, lda, M, K, norm_weight, norm_eps, hi, lo);
  else
    split_activations_kernel<<<M, 256, 0, st>>>(A, lda, M, K, K, norm_weight, norm_eps, hi, lo);
  B200_LAUNCH_CHECK();
  GemmParams p{};
  p.M = M;
  p.N = N;
  p.K = K;
  p.scale = (const float *)w->scale;
  p.bias = (const float *)w->bias;
  p.residual = residual;
  p.C = C;
  p.ldc = ldc;
  p.ldr = ldr;
  p.silu_pairs = silu_pairs;
  p.partial = partial;
  p.error = err;
  p.splits = 1;
  // 32-element k blocks (64-byte swizzle rows), three stages: two CTAs fit on an SM, so one
  // CTA's epilogue runs under the other's main loop
  constexpr int kBK = 32, kStages = 3;
  if (M >= kDenseRows) {
    // dense path: the weights of a slab of rows become bf16 once, then a plain bf16 x bf16 GEMM over the slab
    int64_t rows_per_slab = kSlabElems / K / BN * BN;
    for (int64_t r0 = 0; r0 < N; r0 += rows_per_slab) {
      const int64_t rows = N - r0 < rows_per_slab ? N - r0 : rows_per_slab;
      const int64_t units = rows * K / 16;
      weights_to_bf16_kernel<<<(unsigned)((units + 255) / 256 < 148 * 8 ? (units + 255) / 256 : 148 * 8), 256, 0, st>>>(
          (const uint8_t *)w->w + r0 * K, units, reinterpret_cast<uint4 *>(slab));
      B200_LAUNCH_CHECK();
      p.N = (int)rows;
      p.n_off = (int)r0;
      // 256 weight rows per CTA when that still leaves enough CTAs; else 128, split over K if few
      const int mt = Mp / BM;
      const bool wide = ((rows + 255) / 256) * mt >= 256;
      p.splits = 1;
      if (!wide) {
        const int tiles = (int)((rows + BN - 1) / BN) * mt;
        if (tiles < 148) {
          int splits = 296 / tiles;
          if (splits > K / kBK / 16)
            splits = K / kBK / 16;     // at least 16 k blocks per CTA
          if (splits * tiles > kMaxPartialTiles)
            splits = kMaxPartialTiles / tiles;
          p.splits = splits < 1 ? 1 : splits;
        }
      }
      const int rc = wide ? gemm_launch<kBK, true, 256>(slab, hi, lo, Mp, p, kStages, st)
                          : gemm_launch<kBK, true, 128>(slab, hi, lo, Mp, p, kStages, st);
      if (rc)
        return rc;
    }
    return B200_OK;
  }
  // split over K when the output tiles alone leave most SMs idle
  const int tiles = ((N + BN - 1) / BN) * (Mp / BM), nkb = K / kBK;
  if (tiles < 100) {
    int splits = kMaxPartialTiles / tiles;
    if (splits > nkb / 4)
      splits = nkb / 4;
    p.splits = splits < 1 ? 1 : splits;
  }
  return gemm_launch<kBK, false, 128>(w->w, hi, lo, Mp, p, kStages, st);
}

/* W8A8 (buddy-mlir's QuantizedMatmulOp): workspace = b200_gemm_w8a8_workspace_bytes(M, K). */
int64_t b200_gemm_w8a8_workspace_bytes(int M, int64_t K) {
  if (M < 1 || K < 1)
    return 0;
  return 256 + (int64_t)M * K;
}

int b200_gemm_w8a8(const b200_weight *w, const float *A, int M, int64_t lda, float *C, int64_t ldc,
                   void *workspace, int64_t workspace_bytes, void *stream) {
  return b200::gemm_w8a8_fused(w, A, M, lda, C, ldc, nullptr, 0, 0, workspace, workspace_bytes, (cudaStream_t)stream);
}

} // extern "C"

namespace b200 {
// b200_gemm_w8a8 with the f32 operations that follow a projection in the model folded into the
// store: residual != NULL gives C = residual + y (in place allowed), silu_pairs gives
// C[m, j] = silu(y[m, 2j]) * y[m, 2j + 1] over N / 2 columns.  The same roundings as the
// separate operations.
int gemm_w8a8_fused(const b200_weight *w, const float *A, int M, int64_t lda, float *C, int64_t ldc,
                    const float *residual, int64_t ldr, int silu_pairs, void *workspace, int64_t workspace_bytes,
                    cudaStream_t stream) {
  if (!w || !A || !C || !workspace)
    return fail(B200_EINVAL, "gemm_w8a8: null argument");
  if (silu_pairs && ((w->N & 1) || residual))
    return fail(B200_EINVAL, "gemm_w8a8: gate / up pairs need an even N and take no residual");
  if (w->kind != B200_W_I8 || w->scale_dtype != B200_F32 || !w->scale || !w->w)
    return fail(B200_EINVAL, "gemm_w8a8: int8 per-channel weights with f32 scales expected");
  if (M < 1 || w->K % BK8 != 0 || w->N < 1)
    return fail(B200_EINVAL, "gemm_w8a8: M >= 1 and K a multiple of %d expected", BK8);
  if (((uintptr_t)w->w & 15) || ((uintptr_t)workspace & 255))
    return fail(B200_EINVAL, "gemm_w8a8: weight rows must be 16-byte aligned, the workspace 256-byte aligned");
  if (workspace_bytes < b200_gemm_w8a8_workspace_bytes(M, w->K))
    return fail(B200_EINVAL, "gemm_w8a8: workspace too small");
  if (int rc = ensure_device())
    return rc;
  cudaStream_t st = (cudaStream_t)stream;
  const int K = (int)w->K, N = (int)w->N;
  int *err = reinterpret_cast<int *>(workspace);
  uint32_t *absmax = reinterpret_cast<uint32_t *>(workspace) + 1;
  float *act_scale = reinterpret_cast<float *>(workspace) + 2;
  uint32_t *q = reinterpret_cast<uint32_t *>((char *)workspace + 256);
  B200_CUDA(cudaMemsetAsync(workspace, 0, 16, st));
  const int64_t total = (int64_t)M * K;
  absmax_kernel<<<(unsigned)std::min<int64_t>((total + 255) / 256, 148 * 8), 256, 0, st>>>(A, lda, M, K, absmax);
  B200_LAUNCH_CHECK();
  quantize_activations_kernel<<<M, 256, 0, st>>>(A, lda, M, K, absmax, act_scale, q);
  B200_LAUNCH_CHECK();
  CUtensorMap map_a, map_w;
  if (int rc = make_map(&map_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, BK8, q, K, M, (uint64_t)K, CU_TENSOR_MAP_SWIZZLE_64B))
    return rc;
  if (int rc = make_map(&map_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, BK8, const_cast<void *>(w->w), K, N, (uint64_t)K,
                        CU_TENSOR_MAP_SWIZZLE_64B))
    return rc;
  W8A8Params p{};
  p.M = M;
  p.N = N;
  p.K = K;
  p.wscale = (const float *)w->scale;
  p.bias = (const float *)w->bias;
  p.act_scale = act_scale;
  p.C = C;
  p.ldc = ldc;
  p.residual = residual;
  p.ldr = ldr;
  p.silu_pairs = silu_pairs;
  p.error = err;
  static bool configured[64] = {};
  int dev = 0;
  B200_CUDA(cudaGetDevice(&dev));
  const int smem = kStages8 * 2 * (int)kTile8 + 1024 + 256;
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    B200_CUDA(cudaFuncSetAttribute(gemm_w8a8_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    if (dev >= 0 && dev < 64)
      configured[dev] = true;
  }
  const dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  gemm_w8a8_tc_kernel<<<grid, kThreadsPre, smem, st>>>(map_a, map_w, p);
  B200_LAUNCH_CHECK();
  return B200_OK;
}
} // namespace b200

extern "C" {

/* 0, or the code of the first bounded wait that gave up in the last b200_gemm_w8 on this workspace
 * (reads the error word; synchronises the stream). */
int b200_gemm_w8_status(void *workspace, void *stream) {
  if (!workspace)
    return fail(B200_EINVAL, "gemm_w8_status: null workspace");
  int code = 0;
  B200_CUDA(cudaMemcpyAsync(&code, workspace, 4, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
  B200_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
  if (code != 0)
    return fail(B200_ECUDA, "gemm_w8: a bounded wait gave up (code %d)", code);
  return B200_OK;
}

} // extern "C"

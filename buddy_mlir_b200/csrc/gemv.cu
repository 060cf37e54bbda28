// Decode GEMV over the packed device layout, M = 1..16 activation rows.
//
// One warp streams R output rows: every lane issues one 16-byte load per row
// and block (32 lanes x 16 B = 512 contiguous bytes of each row), dequantises
// in registers, multiplies with the activation groups read from shared
// memory, and the per-lane partial sums meet in a warp-shuffle tree.  HBM
// bound: each weight byte is read exactly once.
//
// Replaces the loops emitted by buddy-mlir's decode passes
//   midend/lib/Conversion/MatMulOptimization/DequantMatMulVectorizationDecode.cpp:250-321
//   midend/lib/Conversion/MatMulOptimization/Int4DequantMatMulVectorizationDecode.cpp:359-430
//   midend/lib/Conversion/MatMulOptimization/MatMulVectorizationDecode.cpp:94-192
// and, as fused prologue/epilogue, the RMSNorm, bias, residual and SiLU-gate
// ops of examples/BuddyDeepSeekR1/subgraph0_decode_simplify.mlir:60-72,75-76,
// 209,226-231,235.
#include "common.cuh"

namespace b200 {

struct GemvP {
  const void *x;
  const uint8_t *w;
  const void *scale;
  const float *bias;
  const float *residual;
  const float *norm_w;
  void *y;
  int64_t x_ld, y_ld, row_bytes;
  int K, Kp, N, M;
  int x_dtype, y_dtype, scale_dtype;
  int group, ngroups;
  int accumulate, silu_pairs;
  int kc;  // activation slab (elements) staged in shared memory at a time
  int fast_scales;  // int4 groups: the 8 f16 scales of a 1024-element block are one aligned 16-byte load
  int in_place4;    // int4 group-128, M = 1, f32 input: nibbles used in place (see gemv_kernel)
  TpPush push;      // ranks > 0: results go to every rank's staging buffer instead of y
  float eps;
};

__device__ __forceinline__ uint4 ld_stream(const void *p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

// Byte i of `word` as float(byte) + 2^23: the byte lands in the mantissa of
// 0x4B000000.  One PRMT; the caller subtracts the bias with one FADD.
__device__ __forceinline__ float byte_magic(uint32_t word, int i) {
  return __uint_as_float(__byte_perm(word, 0x4B000000u, 0x7650 + i));
}

template <int KIND> struct Dequant;

template <> struct Dequant<B200_W_I8> {
  static constexpr int G = 4;  // groups of 4 k per 16-byte unit
  // group j of the unit -> 4 floats
  static __device__ __forceinline__ void group(const uint4 &u, int j,
                                               float (&w)[4]) {
    const uint32_t word = (j == 0 ? u.x : j == 1 ? u.y : j == 2 ? u.z : u.w) ^
                          0x80808080u;  // signed -> offset-128
    constexpr float C = 8388608.0f + 128.0f;
#pragma unroll
    for (int e = 0; e < 4; ++e)
      w[e] = byte_magic(word, e) - C;
  }
};

template <> struct Dequant<B200_W_U4> {
  static constexpr int G = 8;
  static __device__ __forceinline__ void group(const uint4 &u, int j,
                                               float (&w)[4]) {
    const uint32_t word32 =
        (j >> 1) == 0 ? u.x : (j >> 1) == 1 ? u.y : (j >> 1) == 2 ? u.z : u.w;
    const uint32_t lo = word32 & 0x0F0F0F0Fu;         // elements 0 and 2
    const uint32_t hi = (word32 >> 4) & 0x0F0F0F0Fu;  // elements 1 and 3
    const int b = (j & 1) * 2;
    constexpr float C = 8388608.0f + 8.0f;  // zero-point 8 folded in
    w[0] = byte_magic(lo, b) - C;
    w[1] = byte_magic(hi, b) - C;
    w[2] = byte_magic(lo, b + 1) - C;
    w[3] = byte_magic(hi, b + 1) - C;
  }
};

template <> struct Dequant<B200_W_F32> {
  static constexpr int G = 1;
  static __device__ __forceinline__ void group(const uint4 &u, int,
                                               float (&w)[4]) {
    w[0] = __uint_as_float(u.x);
    w[1] = __uint_as_float(u.y);
    w[2] = __uint_as_float(u.z);
    w[3] = __uint_as_float(u.w);
  }
};

__device__ __forceinline__ float silu_mul(float g, float u) {
  // subgraph0_decode_simplify.mlir:226-231: (g * sigmoid(g)) * u
  const float s = 1.0f / (1.0f + expf(-g));
  return (g * s) * u;
}

// Single-row int8 decode (M = 1, per-channel scales): a weight byte is used in
// place.  With its sign bit flipped (u = q + 128) and the other bytes of the
// word masked off, the word read as a float is u * 2^-149 (byte 0, a denormal),
// u * 2^-141, u * 2^-133 (bytes 1, 2) or, shifted down, u * 2^-149 (byte 3).  So
// a weight costs one logic op and one FMA.  The staged activations carry a
// factor 2^64 (products stay in the normal range and are exact up to the FMA's
// single rounding), the four byte positions have their own accumulators, and
//   sum x*q = 2^85 * (a0 + a1*2^-8 + a2*2^-16 + a3) - 128 * sum x.
constexpr float kInPlaceX = 18446744073709551616.0f;          // 2^64
constexpr float kInPlaceAcc = 38685626227668133590597632.0f;  // 2^85

template <int KIND, int MT, int R, bool GROUPED>
__global__ void __launch_bounds__(256)
gemv_kernel(const GemvP p) {
  constexpr bool IN_PLACE = KIND == B200_W_I8 && MT == 1 && !GROUPED;
  // The same idea for group-wise int4 (zero-point 8): nibble e of a group of four
  // sits at bit 4e of a 16-bit half word, so masked in place it reads as
  // n * 2^(4e-149).  The staged activation k carries 2^(64 - 4*(k%4)), which
  // puts the four products of a group on one scale (2^-85); the zero-point term
  // -8 * (x0+x1+x2+x3) * 2^-85 of every group of four is staged beside the
  // activations.  One logic op and one FMA per weight, one FMA per four weights
  // for the group scale.
  const bool in_place4 = KIND == B200_W_U4 && MT == 1 && GROUPED && p.in_place4;
  __shared__ float s_sx[8];   // per-warp sums of the staged activations (IN_PLACE)
  extern __shared__ __align__(16) float xs[];  // [MT][kc]
  float *c4 = xs + (size_t)MT * p.kc;   // in_place4: zero-point terms, one per 4 activations
  __shared__ float s_red[8 * 16];
  __shared__ float s_push[8 * 4];   // tensor-parallel push: the CTA's row sums of one iteration
  __shared__ float s_rinv[16];

  using DQ = Dequant<KIND>;
  constexpr int E = KIND == B200_W_I8 ? 16 : (KIND == B200_W_U4 ? 32 : 4);
  constexpr int BLK = 32 * E;  // elements per full block

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = blockDim.x >> 5;
  // A CTA takes row groups base, base + gridDim.x * nwarps * R, ..: with a grid
  // capped at a few CTAs per SM the activation vector is staged (and its
  // RMSNorm statistics computed) once per CTA, not once per handful of rows.
  const int64_t gstride = (int64_t)gridDim.x * nwarps * R;
  const bool one_slab = p.kc >= p.Kp;

  // ---- optional fused RMSNorm statistics --------------------------------
  if (p.norm_w != nullptr) {
    for (int m = 0; m < p.M; ++m) {
      float s = 0.f;
      if (p.x_dtype == B200_F32 && (p.K & 3) == 0 && (p.x_ld & 3) == 0 &&
          (reinterpret_cast<uintptr_t>(p.x) & 15) == 0) {
        const float *xg = reinterpret_cast<const float *>(p.x) + (int64_t)m * p.x_ld;
        for (int k = threadIdx.x * 4; k < p.K; k += blockDim.x * 4) {
          const float4 v = __ldg(reinterpret_cast<const float4 *>(xg + k));
          s = fmaf(v.x, v.x, s);
          s = fmaf(v.y, v.y, s);
          s = fmaf(v.z, v.z, s);
          s = fmaf(v.w, v.w, s);
        }
      } else {
        for (int k = threadIdx.x; k < p.K; k += blockDim.x) {
          const float v = load_as_float(p.x, p.x_dtype, (int64_t)m * p.x_ld + k);
          s = fmaf(v, v, s);
        }
      }
      s = warp_sum(s);
      if (lane == 0)
        s_red[warp] = s;
      __syncthreads();
      if (threadIdx.x == 0) {
        float t = 0.f;
        for (int w = 0; w < nwarps; ++w)
          t += s_red[w];
        s_rinv[m] = rsqrtf(t * (1.0f / (float)p.K) + p.eps);
      }
      __syncthreads();
    }
  }

  bool staged = false;
  float sx_cta = 0.f;   // IN_PLACE: sum of the activations of the slab staged last
  for (int64_t base = (int64_t)blockIdx.x * nwarps * R; base < p.N; base += gstride) {
    const int64_t row0 = base + (int64_t)warp * R;
    float acc[R][MT];
    float a4[IN_PLACE ? R : 1][4];   // IN_PLACE: one accumulator per byte position
    float sx_total = 0.f;            // IN_PLACE: sum of the activations seen so far
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
      for (int m = 0; m < MT; ++m)
        acc[r][m] = 0.f;
#pragma unroll
    for (int r = 0; r < (IN_PLACE ? R : 1); ++r)
      a4[r][0] = a4[r][1] = a4[r][2] = a4[r][3] = 0.f;

    const uint8_t *rowp[R];
    int64_t srow[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      int64_t row = row0 + r;
      if (row >= p.N)
        row = p.N - 1;  // clamp: loads stay in bounds, result is discarded
      rowp[r] = p.w + row * p.row_bytes;
      srow[r] = row * p.ngroups;
    }

    for (int k0 = 0; k0 < p.Kp; k0 += p.kc) {
      const int kc = min(p.kc, p.Kp - k0);
      if (!(one_slab && staged)) {
        if (staged)
          __syncthreads();
        // ---- stage the activation slab (zero beyond K and beyond M) ----------
        float sx = 0.f;
        if (MT == 1 && p.x_dtype == B200_F32 && (p.K & 3) == 0 &&
            (reinterpret_cast<uintptr_t>(p.x) & 15) == 0) {
          // one f32 row: 16-byte loads, no index arithmetic per element
          const float *xg = reinterpret_cast<const float *>(p.x);
          const float rinv = p.norm_w != nullptr ? s_rinv[0] : 1.f;
          for (int i = threadIdx.x * 4; i < kc; i += blockDim.x * 4) {
            const int k = k0 + i;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (k < p.K) {
              v = __ldg(reinterpret_cast<const float4 *>(xg + k));
              if (p.norm_w != nullptr) {
                const float4 w4 = __ldg(reinterpret_cast<const float4 *>(p.norm_w + k));
                v.x = w4.x * (v.x * rinv);
                v.y = w4.y * (v.y * rinv);
                v.z = w4.z * (v.z * rinv);
                v.w = w4.w * (v.w * rinv);
              }
            }
            if (IN_PLACE) {
              sx += (v.x + v.y) + (v.z + v.w);
              v.x *= kInPlaceX; v.y *= kInPlaceX; v.z *= kInPlaceX; v.w *= kInPlaceX;
            }
            if (in_place4) {
              c4[i >> 2] = -8.0f * ((v.x + v.y) + (v.z + v.w)) * (1.0f / kInPlaceAcc);
              v.x *= kInPlaceX;                       // 2^64
              v.y *= kInPlaceX * 0.0625f;             // 2^60
              v.z *= kInPlaceX * 0.00390625f;         // 2^56
              v.w *= kInPlaceX * 0.000244140625f;     // 2^52
            }
            *reinterpret_cast<float4 *>(&xs[i]) = v;
          }
        } else {
          for (int i = threadIdx.x; i < MT * kc; i += blockDim.x) {
            const int m = i / kc, k = k0 + (i - m * kc);
            float v = 0.f;
            if (m < p.M && k < p.K) {
              v = load_as_float(p.x, p.x_dtype, (int64_t)m * p.x_ld + k);
              if (p.norm_w != nullptr)
                v = p.norm_w[k] * (v * s_rinv[m]);
            }
            if (IN_PLACE) {
              sx += v;
              v *= kInPlaceX;
            }
            xs[m * p.kc + (k - k0)] = v;
          }
        }
        if (IN_PLACE) {
          sx = warp_sum(sx);
          if (lane == 0)
            s_sx[warp] = sx;
        }
        __syncthreads();
        staged = true;
        if (IN_PLACE) {
          sx_cta = 0.f;
          for (int w = 0; w < nwarps; ++w)
            sx_cta += s_sx[w];
        }
      }

      if (IN_PLACE)
        sx_total += sx_cta;
      const int nblk = (kc + BLK - 1) / BLK;
#pragma unroll 2
      for (int b = 0; b < nblk; ++b) {
        const int kb = b * BLK;              // slab-relative element offset
        const int Bs = min(BLK, kc - kb);    // elements in this block
        if (lane * E < Bs) {
          const int q = Bs / DQ::G;
          const int64_t boff = (int64_t)((k0 + kb) / E) * 16 + lane * 16;
          uint4 wv[R];
#pragma unroll
          for (int r = 0; r < R; ++r)
            wv[r] = ld_stream(rowp[r] + boff);
          // int4 group scales of this block: eight consecutive f16 values per row
          uint4 sv[R];
          const bool vec_scales = GROUPED && p.fast_scales && Bs == BLK;
          if (vec_scales) {
#pragma unroll
            for (int r = 0; r < R; ++r)
              sv[r] = __ldg(reinterpret_cast<const uint4 *>(
                  reinterpret_cast<const __half *>(p.scale) + srow[r] + (k0 + kb) / p.group));
          }
          if (IN_PLACE) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float4 xv = *reinterpret_cast<const float4 *>(&xs[kb + j * q + 4 * lane]);
#pragma unroll
              for (int r = 0; r < R; ++r) {
                const uint32_t u = (j == 0 ? wv[r].x : j == 1 ? wv[r].y : j == 2 ? wv[r].z : wv[r].w) ^
                                   0x80808080u;
                a4[r][0] = fmaf(xv.x, __uint_as_float(u & 0x000000FFu), a4[r][0]);
                a4[r][1] = fmaf(xv.y, __uint_as_float(u & 0x0000FF00u), a4[r][1]);
                a4[r][2] = fmaf(xv.z, __uint_as_float(u & 0x00FF0000u), a4[r][2]);
                a4[r][3] = fmaf(xv.w, __uint_as_float(u >> 24), a4[r][3]);
              }
            }
          } else if (in_place4) {
#pragma unroll
            for (int wi = 0; wi < 4; ++wi) {   // word wi of the unit holds groups 2*wi (low half) and 2*wi+1
              const int ka = kb + (2 * wi) * q + 4 * lane, kb2 = ka + q;
              const float4 xa = *reinterpret_cast<const float4 *>(&xs[ka]);
              const float4 xb = *reinterpret_cast<const float4 *>(&xs[kb2]);
              const float ca = c4[ka >> 2], cb = c4[kb2 >> 2];
#pragma unroll
              for (int r = 0; r < R; ++r) {
                const uint32_t w32 = wi == 0 ? wv[r].x : wi == 1 ? wv[r].y : wi == 2 ? wv[r].z : wv[r].w;
                const uint32_t s32 = wi == 0 ? sv[r].x : wi == 1 ? sv[r].y : wi == 2 ? sv[r].z : sv[r].w;
                const uint32_t hw = w32 >> 16;
                float ta = fmaf(xa.x, __uint_as_float(w32 & 0x000Fu), ca);
                ta = fmaf(xa.y, __uint_as_float(w32 & 0x00F0u), ta);
                ta = fmaf(xa.z, __uint_as_float(w32 & 0x0F00u), ta);
                ta = fmaf(xa.w, __uint_as_float(w32 & 0xF000u), ta);
                float tb = fmaf(xb.x, __uint_as_float(hw & 0x000Fu), cb);
                tb = fmaf(xb.y, __uint_as_float(hw & 0x00F0u), tb);
                tb = fmaf(xb.z, __uint_as_float(hw & 0x0F00u), tb);
                tb = fmaf(xb.w, __uint_as_float(hw & 0xF000u), tb);
                const float2 sc2 = __half22float2(*reinterpret_cast<const __half2 *>(&s32));
                acc[r][0] = fmaf(ta, sc2.x, acc[r][0]);
                acc[r][0] = fmaf(tb, sc2.y, acc[r][0]);
              }
            }
          } else {
#pragma unroll
          for (int j = 0; j < DQ::G; ++j) {
            const int kx = kb + j * q + 4 * lane;
            float wf[R][4];
#pragma unroll
            for (int r = 0; r < R; ++r)
              DQ::group(wv[r], j, wf[r]);
            float sc[R];
            if (GROUPED) {
              if (vec_scales) {
#pragma unroll
                for (int r = 0; r < R; ++r) {
                  const uint32_t w32 = (j >> 1) == 0 ? sv[r].x : (j >> 1) == 1 ? sv[r].y
                                     : (j >> 1) == 2 ? sv[r].z : sv[r].w;
                  sc[r] = __half2float(__ushort_as_half((unsigned short)((j & 1) ? (w32 >> 16) : (w32 & 0xFFFFu))));
                }
              } else {
                const int g = (k0 + kx) / p.group;
#pragma unroll
                for (int r = 0; r < R; ++r)
                  sc[r] = load_as_float(p.scale, p.scale_dtype, srow[r] + g);
              }
            }
#pragma unroll
            for (int m = 0; m < MT; ++m) {
              const float4 xv =
                  *reinterpret_cast<const float4 *>(&xs[m * p.kc + kx]);
#pragma unroll
              for (int r = 0; r < R; ++r) {
                if (GROUPED) {
                  float t = xv.x * wf[r][0];
                  t = fmaf(xv.y, wf[r][1], t);
                  t = fmaf(xv.z, wf[r][2], t);
                  t = fmaf(xv.w, wf[r][3], t);
                  acc[r][m] = fmaf(t, sc[r], acc[r][m]);
                } else {
                  acc[r][m] = fmaf(xv.x, wf[r][0], acc[r][m]);
                  acc[r][m] = fmaf(xv.y, wf[r][1], acc[r][m]);
                  acc[r][m] = fmaf(xv.z, wf[r][2], acc[r][m]);
                  acc[r][m] = fmaf(xv.w, wf[r][3], acc[r][m]);
                }
              }
            }
          }
          }
        }
      }
    }

    // ---- reduce across lanes, epilogue --------------------------------------
    if (IN_PLACE) {
#pragma unroll
      for (int r = 0; r < R; ++r)
        acc[r][0] = (a4[r][0] + a4[r][3]) + fmaf(a4[r][1], 0.00390625f, a4[r][2] * 0.0000152587890625f);
    }
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
      for (int m = 0; m < MT; ++m)
        acc[r][m] = warp_sum(acc[r][m]);
    if (IN_PLACE) {
#pragma unroll
      for (int r = 0; r < R; ++r)
        acc[r][0] = fmaf(acc[r][0], kInPlaceAcc, -128.0f * sx_total);
    }
    if (in_place4) {
#pragma unroll
      for (int r = 0; r < R; ++r)
        acc[r][0] *= kInPlaceAcc;
    }

    if (p.push.ranks > 0) {
      // This rank's share of a tensor-parallel sum (M = 1).  The CTA's warps hold the sums of
      // nwarps * R consecutive rows: they are gathered in shared memory and sent to every
      // rank's staging buffer as 16-byte stores of two (value, tag) pairs (plain stores over
      // NVLink): a thread serves one peer and two rows, so the CTA's rows reach a peer as one
      // contiguous run instead of one 8-byte packet per row.
      const uint32_t seq = (uint32_t)(*p.push.step) * p.push.per_step + p.push.index;
      if (lane == 0) {
#pragma unroll
        for (int r = 0; r < R; ++r) {
          const int64_t row = row0 + r;
          float v = acc[r][0];
          if (row < p.N) {
            if (!GROUPED && p.scale != nullptr)
              v = v * load_as_float(p.scale, p.scale_dtype, row);
            if (p.bias != nullptr)
              v = p.bias[row] + v;
          }
          s_push[warp * R + r] = v;
        }
      }
      __syncthreads();
      const int rows_cta = nwarps * R;               // even: R >= 2 or an even number of warps
      const int units = (rows_cta + 1) / 2;          // 16-byte units per peer
      if ((int)threadIdx.x < p.push.ranks * units) {
        const int peer = threadIdx.x / units, u = threadIdx.x - peer * units;
        const int64_t row = base + 2 * u;
        uint2 *dst = p.push.peer[peer] + ((size_t)(seq % kTpRegions) * p.push.ranks + p.push.rank) * p.push.H;
        if (row + 1 < p.N && 2 * u + 1 < rows_cta && ((reinterpret_cast<uintptr_t>(dst + row) & 15) == 0))
          tagged_store2(dst + row, s_push[2 * u], s_push[2 * u + 1], seq + 1u);
        else {
          if (row < p.N)
            tagged_store(dst + row, s_push[2 * u], seq + 1u);
          if (row + 1 < p.N && 2 * u + 1 < rows_cta)
            tagged_store(dst + row + 1, s_push[2 * u + 1], seq + 1u);
        }
      }
      __syncthreads();
    } else if (lane == 0) {
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const int64_t row = row0 + r;
        if (row >= p.N)
          continue;
        float s = 1.f;
        if (!GROUPED && p.scale != nullptr)
          s = load_as_float(p.scale, p.scale_dtype, row);
#pragma unroll
        for (int m = 0; m < MT; ++m)
          if (m < p.M) {
            float v = acc[r][m];
            if (!GROUPED && p.scale != nullptr)
              v = v * s;
            if (p.bias != nullptr)
              v = p.bias[row] + v;
            acc[r][m] = v;
          }
      }
      if (p.silu_pairs) {
        // rows (2j, 2j+1) = (gate_j, up_j); R is even and row0 is even.
#pragma unroll
        for (int r = 0; r + 1 < R; r += 2) {
          const int64_t row = row0 + r;
          if (row + 1 >= p.N)
            continue;
          const int64_t col = row >> 1;
#pragma unroll
          for (int m = 0; m < MT; ++m)
            if (m < p.M) {
              const float v = silu_mul(acc[r][m], acc[r + 1][m]);
              const int64_t o = (int64_t)m * p.y_ld + col;
              if (p.y_dtype == B200_F32)
                ((float *)p.y)[o] = v;
              else
                ((__half *)p.y)[o] = __float2half_rn(v);
            }
        }
      } else {
#pragma unroll
        for (int r = 0; r < R; ++r) {
          const int64_t row = row0 + r;
          if (row >= p.N)
            continue;
#pragma unroll
          for (int m = 0; m < MT; ++m)
            if (m < p.M) {
              const int64_t o = (int64_t)m * p.y_ld + row;
              float v = acc[r][m];
              if (p.residual != nullptr)
                v = p.residual[o] + v;
              if (p.y_dtype == B200_F32) {
                if (p.accumulate)
                  v = ((float *)p.y)[o] + v;
                ((float *)p.y)[o] = v;
              } else {
                if (p.accumulate)
                  v = __half2float(((__half *)p.y)[o]) + v;
                ((__half *)p.y)[o] = __float2half_rn(v);
              }
            }
        }
      }
    }
  }
}

template <int KIND, int MT, int R, bool GROUPED>
static int launch(const GemvP &p, int warps, cudaStream_t st) {
  auto kern = gemv_kernel<KIND, MT, R, GROUPED>;
  const size_t smem = ((size_t)MT * p.kc + (p.in_place4 ? p.kc / 4 : 0)) * sizeof(float);
  if (smem > 40 * 1024) {  // dynamic + static shared memory may exceed the 48 KB default
    static thread_local size_t configured = 0;
    if (smem > configured) {
      B200_CUDA(cudaFuncSetAttribute(
          kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
      configured = 200 * 1024;
    }
  }
  const int64_t rows_per_cta = (int64_t)warps * R;
  int64_t grid = (p.N + rows_per_cta - 1) / rows_per_cta;
  // one resident wave: as many CTAs as fit on the device at once, each looping
  // over its row groups
  int occ = 0, dev = 0, sms = 0;
  B200_CUDA(cudaGetDevice(&dev));
  B200_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  B200_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kern, warps * 32, smem));
  if (occ < 1)
    occ = 1;
  const int64_t cap = (int64_t)sms * occ;
  if (grid > cap)
    grid = cap;
  kern<<<(unsigned)grid, warps * 32, smem, st>>>(p);
  B200_LAUNCH_CHECK();
  return B200_OK;
}

template <int KIND, bool GROUPED>
static int dispatch(const GemvP &p, int mt, int R, int warps,
                    cudaStream_t st) {
#define B200_CASE(MT_, R_)                                                     \
  if (mt == MT_ && R == R_)                                                    \
    return launch<KIND, MT_, R_, GROUPED>(p, warps, st);
  B200_CASE(1, 1) B200_CASE(1, 2) B200_CASE(1, 4)
  B200_CASE(2, 2) B200_CASE(4, 2) B200_CASE(8, 2) B200_CASE(16, 2)
#undef B200_CASE
  return fail(B200_EINVAL, "gemv: no kernel for M tile %d, R %d", mt, R);
}

} // namespace b200

using namespace b200;

extern "C" int b200_gemv(const b200_weight *w, const b200_gemv_args *a,
                         void *stream) {
  return gemv_run(w, a, nullptr, (cudaStream_t)stream);
}

int b200::gemv_run(const b200_weight *w, const b200_gemv_args *a, const TpPush *push,
                   cudaStream_t stream) {
  if (!w || !a || !w->w || !a->x || !a->y)
    return fail(B200_EINVAL, "gemv: null argument");
  if (a->M < 1 || a->M > 16)
    return fail(B200_EINVAL, "gemv: M=%d outside 1..16", a->M);
  if (w->K < 1 || w->N < 1 || w->K > (1 << 24))
    return fail(B200_EINVAL, "gemv: bad shape K=%lld N=%lld",
                (long long)w->K, (long long)w->N);
  if (w->kind != B200_W_F32 && w->kind != B200_W_I8 && w->kind != B200_W_U4)
    return fail(B200_EINVAL, "gemv: unknown weight kind %d", w->kind);
  if (w->kind != B200_W_F32 && !w->scale)
    return fail(B200_EINVAL, "gemv: quantised weight without scales");
  if (a->silu_pairs && (w->N & 1))
    return fail(B200_EINVAL, "gemv: silu_pairs needs an even N");
  if (a->silu_pairs && (a->accumulate || a->residual))
    return fail(B200_EINVAL, "gemv: silu_pairs excludes accumulate/residual");
  if (int rc = ensure_device())
    return rc;

  GemvP p{};
  if (push != nullptr) {
    if (a->M != 1 || a->silu_pairs || push->ranks < 2 || push->ranks > kTpMaxRanks || push->H != w->N)
      return fail(B200_EINVAL, "gemv: bad tensor-parallel push request");
    p.push = *push;
  }
  p.x = a->x;
  p.w = (const uint8_t *)w->w;
  p.scale = w->scale;
  p.bias = w->bias;
  p.residual = a->residual;
  p.norm_w = a->norm_weight;
  p.y = a->y;
  p.x_ld = a->x_ld ? a->x_ld : w->K;
  p.y_ld = a->y_ld ? a->y_ld : (a->silu_pairs ? w->N / 2 : w->N);
  p.K = (int)w->K;
  p.Kp = (int)packed_k(w->kind, w->K);
  p.row_bytes = packed_row_bytes(w->kind, w->K);
  p.N = (int)w->N;
  p.M = a->M;
  p.x_dtype = a->x_dtype;
  p.y_dtype = a->y_dtype;
  p.scale_dtype = w->scale_dtype;
  p.accumulate = a->accumulate;
  p.silu_pairs = a->silu_pairs;
  p.eps = a->norm_eps;
  bool grouped = false;
  p.group = p.Kp;
  p.ngroups = 1;
  if (w->kind == B200_W_U4 && w->group > 0 && w->group < w->K) {
    if (w->K % w->group != 0 || w->group % 4 != 0)
      return fail(B200_EINVAL, "gemv: group %d does not divide K=%lld",
                  w->group, (long long)w->K);
    grouped = true;
    p.group = w->group;
    p.ngroups = (int)(w->K / w->group);
  }

  const int mt = a->M == 1 ? 1 : a->M == 2 ? 2 : a->M <= 4 ? 4 : a->M <= 8 ? 8 : 16;
  // Activation slab: whole K when it fits, else a multiple of the largest
  // block (1024 elements) that keeps the staged tile under ~64 KB.
  int kc = p.Kp;
  const int budget = (64 * 1024) / (4 * mt);
  if (kc > budget)
    kc = (budget / 1024) * 1024;
  p.kc = kc;

  p.fast_scales = grouped && w->scale_dtype == B200_F16 && p.group * 8 == 1024 && p.ngroups % 8 == 0 &&
                  (reinterpret_cast<uintptr_t>(w->scale) & 15) == 0;

  p.in_place4 = p.fast_scales && a->M == 1 && a->x_dtype == B200_F32 && (w->K & 1023) == 0 &&
                (reinterpret_cast<uintptr_t>(a->x) & 15) == 0;

  // Rows per warp: the most that still gives every SM two CTAs of 8 warps.
  int R = 2, warps = 8;
  if (mt == 1) {
    const int64_t want = 2 * 148;
    if (w->N / (8 * 4) >= want)
      R = 4;
    else if (w->N / (8 * 2) >= want / 2 || a->silu_pairs)   // two rows share the staged activations
      R = 2;
    else
      R = 1;
  } else if (w->N / (8 * 2) < 2 * 148) {
    warps = 4;
  }
  cudaStream_t st = stream;
  switch (w->kind) {
  case B200_W_I8:
    return dispatch<B200_W_I8, false>(p, mt, R, warps, st);
  case B200_W_F32:
    return dispatch<B200_W_F32, false>(p, mt, R, warps, st);
  default:
    return grouped ? dispatch<B200_W_U4, true>(p, mt, R, warps, st)
                   : dispatch<B200_W_U4, false>(p, mt, R, warps, st);
  }
}

// CPU restatement of buddy-mlir's LLM decode arithmetic (test infrastructure
// only; see buddy_oracle.h for what it is pinned against).  Build with
// -ffp-contract=off: multiply and add are fused only where the reference
// emits vector.fma (written here as __builtin_fmaf).
#include "buddy_oracle.h"

#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <vector>
#ifdef _OPENMP
#include <omp.h>
#endif

namespace {

typedef _Float16 f16;

inline f16 bits_to_f16(uint16_t b) {
  f16 h;
  std::memcpy(&h, &b, 2);
  return h;
}
inline uint16_t f16_to_bits(f16 h) {
  uint16_t b;
  std::memcpy(&b, &h, 2);
  return b;
}
// f16 fused multiply-add: the product of two f16 values is exact in double
// and the sum is rounded once to f16.
inline f16 fma_f16(f16 a, f16 b, f16 c) {
  return (f16)((double)a * (double)b + (double)c);
}

// torch.round = round half to even; nearbyintf under the default rounding mode.
inline float rne(float v) { return std::nearbyintf(v); }

constexpr int64_t kTile = 32; // vector-size=32 in compile_pipeline.py:167-174

} // namespace

extern "C" {

int orc_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

// ---------------------------------------------------------------------------
// import_model.py:830-850
void orc_quantize_per_channel(const float *W, int64_t K, int64_t N, int bits,
                              int8_t *Q, float *scale) {
  const float qmax = bits == 4 ? 7.0f : 127.0f;
  const float lo = bits == 4 ? -8.0f : -128.0f;
  const float hi = bits == 4 ? 7.0f : 127.0f;
  std::vector<float> amax(N, 0.0f);
  for (int64_t k = 0; k < K; ++k)
    for (int64_t n = 0; n < N; ++n)
      amax[n] = std::max(amax[n], std::fabs(W[k * N + n]));
  for (int64_t n = 0; n < N; ++n)
    scale[n] = std::max(amax[n] / qmax, 1e-10f);
#pragma omp parallel for schedule(static)
  for (int64_t k = 0; k < K; ++k)
    for (int64_t n = 0; n < N; ++n) {
      float r = rne(W[k * N + n] / scale[n]);
      Q[k * N + n] = (int8_t)std::min(std::max(r, lo), hi);
    }
}

// import_model.py:810-815
void orc_pack_int4(const int8_t *flat, int64_t n, int8_t *packed) {
  for (int64_t i = 0; i < n / 2; ++i) {
    uint8_t low = (uint8_t)flat[2 * i] & 0x0F;
    uint8_t high = (uint8_t)(((uint8_t)flat[2 * i + 1] & 0x0F) << 4);
    packed[i] = (int8_t)(low | high);
  }
}

// ops/tosa.py:12158-12203
void orc_unpack_int4(const int8_t *packed, int64_t nbytes, int8_t *flat) {
  for (int64_t i = 0; i < nbytes; ++i) {
    int8_t b = packed[i];
    int8_t low = (int8_t)((int8_t)((uint8_t)(b & 0x0F) << 4) >> 4);
    int8_t high = (int8_t)(b >> 4);
    flat[2 * i] = low;
    flat[2 * i + 1] = high;
  }
}

void orc_quantize_w4_group(const float *W, int64_t K, int64_t N, int64_t G,
                           uint8_t *P, uint16_t *scale_f16) {
  const int64_t groups = K / G;
  std::vector<int8_t> u((size_t)K * N);
  for (int64_t g = 0; g < groups; ++g)
    for (int64_t n = 0; n < N; ++n) {
      float amax = 0.0f;
      for (int64_t k = g * G; k < (g + 1) * G; ++k)
        amax = std::max(amax, std::fabs(W[k * N + n]));
      f16 s16 = (f16)std::max(amax / 7.0f, 1e-10f);
      if ((float)s16 == 0.0f) // f16 underflow of a tiny scale
        s16 = bits_to_f16(0x0001);
      scale_f16[g * N + n] = f16_to_bits(s16);
      const float s = (float)s16;
      for (int64_t k = g * G; k < (g + 1) * G; ++k) {
        float r = rne(W[k * N + n] / s);
        r = std::min(std::max(r, -8.0f), 7.0f);
        u[k * N + n] = (int8_t)((int)r + 8);
      }
    }
  for (int64_t i = 0; i < K * N / 2; ++i)
    P[i] = (uint8_t)((u[2 * i] & 0x0F) | ((u[2 * i + 1] & 0x0F) << 4));
}

// ---------------------------------------------------------------------------
// DequantMatMulVectorizationDecode.cpp:250-321
void orc_gemv_w8_f32(const float *x, const int8_t *Q, const float *scale,
                     float *y, int64_t M, int64_t K, int64_t N) {
  const int64_t tiles = (N + kTile - 1) / kTile;
  for (int64_t m = 0; m < M; ++m) {
    const float *xm = x + m * K;
    float *ym = y + m * N;
#pragma omp parallel for schedule(static)
    for (int64_t t = 0; t < tiles; ++t) {
      const int64_t n0 = t * kTile;
      const int64_t w = std::min(kTile, N - n0);
      float acc[kTile];
      for (int64_t j = 0; j < kTile; ++j)
        acc[j] = 0.0f;
      if (w == kTile) {
        for (int64_t k = 0; k < K; ++k) {
          const float a = xm[k];
          const int8_t *row = Q + k * N + n0;
          for (int64_t j = 0; j < kTile; ++j)
            acc[j] = __builtin_fmaf(a, (float)row[j], acc[j]);
        }
      } else {
        for (int64_t k = 0; k < K; ++k) {
          const float a = xm[k];
          const int8_t *row = Q + k * N + n0;
          for (int64_t j = 0; j < w; ++j)
            acc[j] = __builtin_fmaf(a, (float)row[j], acc[j]);
        }
      }
      for (int64_t j = 0; j < w; ++j) {
        float v = acc[j] * scale[n0 + j];
        ym[n0 + j] = ym[n0 + j] + v;
      }
    }
  }
}

void orc_gemv_w8_f16(const uint16_t *x, const int8_t *Q, const uint16_t *scale,
                     uint16_t *y, int64_t M, int64_t K, int64_t N) {
  for (int64_t m = 0; m < M; ++m)
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
      f16 acc = (f16)0.0f;
      for (int64_t k = 0; k < K; ++k)
        acc = fma_f16(bits_to_f16(x[m * K + k]), (f16)(float)Q[k * N + n], acc);
      acc = acc * bits_to_f16(scale[n]);
      y[m * N + n] = f16_to_bits((f16)(bits_to_f16(y[m * N + n]) + acc));
    }
}

// Int4DequantMatMulVectorizationDecode.cpp:359-430
void orc_gemv_w4_f16(const uint16_t *x, const int8_t *P, const uint16_t *scale,
                     uint16_t *y, int64_t M, int64_t K, int64_t N) {
  for (int64_t m = 0; m < M; ++m)
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
      f16 acc = (f16)0.0f;
      for (int64_t k = 0; k < K; ++k) {
        int8_t b = P[k * (N / 2) + n / 2];
        int8_t q = (n & 1) ? (int8_t)(b >> 4)
                           : (int8_t)((int8_t)((uint8_t)(b & 0x0F) << 4) >> 4);
        acc = fma_f16(bits_to_f16(x[m * K + k]), (f16)(float)q, acc);
      }
      acc = acc * bits_to_f16(scale[n]);
      y[m * N + n] = f16_to_bits((f16)(bits_to_f16(y[m * N + n]) + acc));
    }
}

// MatMulVectorizationDecode.cpp:94-192
void orc_gemv_f32(const float *x, const float *B, float *y, int64_t M,
                  int64_t K, int64_t N) {
  const int64_t tiles = (N + kTile - 1) / kTile;
  for (int64_t m = 0; m < M; ++m) {
    const float *xm = x + m * K;
    float *ym = y + m * N;
#pragma omp parallel for schedule(static)
    for (int64_t t = 0; t < tiles; ++t) {
      const int64_t n0 = t * kTile;
      const int64_t w = std::min(kTile, N - n0);
      float acc[kTile];
      for (int64_t j = 0; j < kTile; ++j)
        acc[j] = j < w ? ym[n0 + j] : 0.0f;
      for (int64_t k = 0; k < K; ++k) {
        const float a = xm[k];
        const float *row = B + k * N + n0;
        for (int64_t j = 0; j < w; ++j)
          acc[j] = __builtin_fmaf(a, row[j], acc[j]);
      }
      for (int64_t j = 0; j < w; ++j)
        ym[n0 + j] = acc[j];
    }
  }
}

void orc_gemv_w4g_f32(const float *x, const uint8_t *P,
                      const uint16_t *scale_f16, float *y, int64_t M,
                      int64_t K, int64_t N, int64_t G) {
  const int64_t tiles = (N + kTile - 1) / kTile;
  const int64_t groups = K / G;
  for (int64_t m = 0; m < M; ++m) {
    const float *xm = x + m * K;
    float *ym = y + m * N;
#pragma omp parallel for schedule(static)
    for (int64_t t = 0; t < tiles; ++t) {
      const int64_t n0 = t * kTile;
      const int64_t w = std::min(kTile, N - n0);
      float tot[kTile];
      for (int64_t j = 0; j < kTile; ++j)
        tot[j] = 0.0f;
      for (int64_t g = 0; g < groups; ++g) {
        float acc[kTile];
        for (int64_t j = 0; j < kTile; ++j)
          acc[j] = 0.0f;
        for (int64_t k = g * G; k < (g + 1) * G; ++k) {
          const float a = xm[k];
          const uint8_t *row = P + k * (N / 2) + n0 / 2;
          for (int64_t j = 0; j < w; ++j) {
            uint8_t b = row[j >> 1];
            int u = (j & 1) ? (b >> 4) : (b & 0x0F);
            acc[j] = __builtin_fmaf(a, (float)(u - 8), acc[j]);
          }
        }
        for (int64_t j = 0; j < w; ++j) {
          float s = (float)bits_to_f16(scale_f16[g * N + n0 + j]);
          float v = acc[j] * s;
          tot[j] = tot[j] + v;
        }
      }
      for (int64_t j = 0; j < w; ++j)
        ym[n0 + j] = ym[n0 + j] + tot[j];
    }
  }
}

// pack_decode_weights.py:32-124
void orc_pack_panels_f32(const float *B, int64_t K, int64_t N, int64_t V,
                         float *packed) {
  for (int64_t n = 0; n < N; ++n)
    for (int64_t k = 0; k < K; ++k)
      packed[(n / V) * K * V + k * V + (n % V)] = B[k * N + n];
}

// MatMulVectorizationDecodePacked.cpp:128-266
void orc_gemv_f32_packed(const float *x, const float *packed, float *y,
                         int64_t K, int64_t N, int64_t V) {
#pragma omp parallel for schedule(static)
  for (int64_t p = 0; p < N / V; ++p) {
    std::vector<float> acc(V);
    for (int64_t j = 0; j < V; ++j)
      acc[j] = y[p * V + j];
    const float *panel = packed + p * K * V;
    for (int64_t k = 0; k < K; ++k)
      for (int64_t j = 0; j < V; ++j)
        acc[j] = __builtin_fmaf(x[k], panel[k * V + j], acc[j]);
    for (int64_t j = 0; j < V; ++j)
      y[p * V + j] = acc[j];
  }
}

// MatMulBlisVectorization.cpp:367-530
void orc_gemm_w8_prefill_f32(const float *A, const int8_t *Q,
                             const float *scale, float *C, int64_t M,
                             int64_t K, int64_t N) {
#pragma omp parallel for schedule(static)
  for (int64_t m = 0; m < M; ++m)
    for (int64_t n = 0; n < N; ++n) {
      float acc = C[m * N + n];
      for (int64_t k = 0; k < K; ++k) {
        float w = (float)Q[k * N + n] * scale[n];
        acc = __builtin_fmaf(A[m * K + k], w, acc);
      }
      C[m * N + n] = acc;
    }
}

// frontend/Python/ops/linalg.py:12728-12846 (QuantizedMatmulOp / QuantizedAddMMOp, the w8a8
// variant): one dynamic scale for the whole activation tensor, exact i8 x i8 -> i32
// contraction, result * (act_scale * weight_scale[n]) (+ bias).  The f32 -> i32 cast of the
// quantiser rounds to nearest even (tosa.cast).
void orc_matmul_w8a8(const float *A, const int8_t *Q, const float *scale, const float *bias,
                     float *C, int64_t M, int64_t K, int64_t N) {
  float amax = 0.0f;
  for (int64_t i = 0; i < M * K; ++i)
    amax = std::fmax(amax, std::fabs(A[i]));
  const float r127 = 1.0f / 127.0f;
  const float raw = amax * r127;
  const float s = raw > 1e-10f ? raw : 1e-10f;
  const float inv = 1.0f / s;
  std::vector<int8_t> q((size_t)(M * K));
  for (int64_t i = 0; i < M * K; ++i) {
    float v = std::nearbyintf(A[i] * inv);
    v = v < -128.0f ? -128.0f : (v > 127.0f ? 127.0f : v);
    q[(size_t)i] = (int8_t)v;
  }
  // exact integer sums: the order of the k loop does not matter, so it runs outermost over a
  // block of columns (contiguous weight rows) instead of striding down one column at a time
  const int64_t NB = 512, nblocks = (N + NB - 1) / NB;
#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t m = 0; m < M; ++m)
    for (int64_t nb = 0; nb < nblocks; ++nb) {
      const int64_t n0 = nb * NB, nn = std::min(NB, N - n0);
      int32_t acc[512];
      for (int64_t j = 0; j < nn; ++j)
        acc[j] = 0;
      for (int64_t k = 0; k < K; ++k) {
        const int32_t a = (int32_t)q[(size_t)(m * K + k)];
        const int8_t *w = Q + k * N + n0;
        for (int64_t j = 0; j < nn; ++j)
          acc[j] += a * (int32_t)w[j];
      }
      for (int64_t j = 0; j < nn; ++j) {
        const int64_t n = n0 + j;
        const float combined = s * scale[n];
        float y = (float)acc[j] * combined;
        if (bias)
          y = y + bias[n];
        C[m * N + n] = y;
      }
    }
}

// ---------------------------------------------------------------------------
// subgraph0_decode_simplify.mlir:60-72
void orc_rmsnorm(const float *x, const float *w, float *y, int64_t H,
                 float eps) {
  float s = 0.0f;
  for (int64_t i = 0; i < H; ++i) {
    float sq = x[i] * x[i];
    s = s + sq;
  }
  const float inv_h = 1.0f / (float)H;
  float t = s * inv_h;
  t = t + eps;
  const float r = 1.0f / std::sqrt(t);
  for (int64_t i = 0; i < H; ++i) {
    float xr = x[i] * r;
    y[i] = w[i] * xr;
  }
}

// subgraph0_decode_simplify.mlir:52-59, 86-105
void orc_rope(float *v, int64_t heads, int64_t D, const float *inv_freq,
              int64_t pos) {
  const int64_t half = D / 2;
  std::vector<float> c(D), s(D);
  for (int64_t j = 0; j < half; ++j) {
    float th = inv_freq[j] * (float)pos;
    c[j] = c[j + half] = std::cos(th);
    s[j] = s[j + half] = std::sin(th);
  }
  std::vector<float> rot(D);
  for (int64_t h = 0; h < heads; ++h) {
    float *p = v + h * D;
    for (int64_t j = 0; j < half; ++j) {
      rot[j] = -p[j + half];
      rot[j + half] = p[j];
    }
    for (int64_t j = 0; j < D; ++j) {
      float a = p[j] * c[j];
      float b = rot[j] * s[j];
      p[j] = a + b;
    }
  }
}

// subgraph0_decode_simplify.mlir:226-231
void orc_silu_mul(const float *g, const float *u, float *y, int64_t n) {
  for (int64_t i = 0; i < n; ++i) {
    float sg = 1.0f / (1.0f + std::exp(-g[i]));
    float si = g[i] * sg;
    y[i] = si * u[i];
  }
}

// Sampler.h:101-104
int64_t orc_argmax_first(const float *v, int64_t n) {
  int64_t best = 0;
  for (int64_t i = 1; i < n; ++i)
    if (v[i] > v[best])
      best = i;
  return best;
}

// ops/tosa.py:14130-14600
void orc_gqa_decode(const float *q, const float *Kc, const float *Vc,
                    float *out, int64_t q_heads, int64_t kv_heads,
                    int64_t max_len, int64_t D, int64_t pos) {
  const int64_t group = q_heads / kv_heads;
  int64_t splits = 4;
  if (max_len % (splits * 16) != 0)
    splits = 1;
  const int64_t split_len = max_len / splits;
  const float scale = 1.0f / std::sqrt((float)D);
  const int64_t chunks = D / 16;
  std::vector<float> pm(q_heads * splits), pl(q_heads * splits),
      pacc((size_t)q_heads * splits * D);

#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t h = 0; h < q_heads; ++h)
    for (int64_t s = 0; s < splits; ++s) {
      const int64_t hk = h / group;
      const float *qh = q + h * D;
      float m = -1.0e30f, l = 0.0f;
      std::vector<float> acc(D, 0.0f), accb(D);
      const int64_t end = (s + 1) * split_len;
      for (int64_t kb = s * split_len; kb < end; kb += 16) {
        const int64_t bs = std::min<int64_t>(16, end - kb);
        float sc[16];
        for (int64_t j = 0; j < 16; ++j)
          sc[j] = -INFINITY; // lanes past a ragged end never contribute
        for (int64_t j = 0; j < bs; ++j) {
          const int64_t k = kb + j;
          const float *kr = Kc + (hk * max_len + k) * D;
          float dv[16];
          for (int i = 0; i < 16; ++i)
            dv[i] = 0.0f;
          for (int64_t c = 0; c < chunks; ++c)
            for (int i = 0; i < 16; ++i)
              dv[i] = __builtin_fmaf(qh[c * 16 + i], kr[c * 16 + i], dv[i]);
          float dot = 0.0f;
          for (int i = 0; i < 16; ++i)
            dot = dot + dv[i];
          float scaled = dot * scale;
          float mask = (k <= pos) ? 0.0f : -INFINITY;
          sc[j] = scaled + mask;
        }
        float mb = sc[0];
        for (int64_t j = 1; j < 16; ++j)
          mb = std::max(mb, sc[j]);
        const float nm = mb > m ? mb : m;
        const float alpha = std::exp(m - nm);
        float p[16], lb = 0.0f;
        for (int64_t j = 0; j < 16; ++j) {
          p[j] = std::exp(sc[j] - nm);
          lb = lb + p[j];
        }
        float la = l * alpha;
        l = la + lb;
        for (int64_t d = 0; d < D; ++d)
          accb[d] = 0.0f;
        for (int64_t j = 0; j < bs; ++j) {
          const float *vr = Vc + (hk * max_len + kb + j) * D;
          for (int64_t d = 0; d < D; ++d)
            accb[d] = __builtin_fmaf(vr[d], p[j], accb[d]);
        }
        for (int64_t d = 0; d < D; ++d)
          acc[d] = __builtin_fmaf(acc[d], alpha, accb[d]);
        m = nm;
      }
      pm[h * splits + s] = m;
      pl[h * splits + s] = l;
      std::memcpy(&pacc[(size_t)(h * splits + s) * D], acc.data(),
                  D * sizeof(float));
    }

  for (int64_t h = 0; h < q_heads; ++h) {
    float mr = -1.0e30f, lr = 0.0f;
    std::vector<float> ar(D, 0.0f);
    for (int64_t s = 0; s < splits; ++s) {
      const float ms = pm[h * splits + s], ls = pl[h * splits + s];
      const float mn = ms > mr ? ms : mr;
      const float a = std::exp(mr - mn), b = std::exp(ms - mn);
      float t0 = lr * a, t1 = ls * b;
      lr = t0 + t1;
      const float *as = &pacc[(size_t)(h * splits + s) * D];
      for (int64_t d = 0; d < D; ++d) {
        float resc = ar[d] * a;
        ar[d] = __builtin_fmaf(as[d], b, resc);
      }
      mr = mn;
    }
    for (int64_t d = 0; d < D; ++d)
      out[h * D + d] = ar[d] / lr;
  }
}

// KVCacheManager.h:151-273 driven as in gen_session.py:1471-1506
int64_t orc_kv_overflow(float **kv, int64_t n_buffers, int64_t kv_heads,
                        int64_t max_len, int64_t D, int64_t position,
                        int64_t keep, float theta) {
  if (position < max_len)
    return -1;
  const int64_t cur = std::min(position, max_len);
  keep = std::min(std::max<int64_t>(keep, 0), cur - 1);
  const int64_t discard = std::max<int64_t>(1, (cur - keep) / 2);
  const int64_t src = keep + discard;
  if (src < cur) {
    const int64_t tail = cur - src;
    const size_t stride = (size_t)max_len * D;
    for (int64_t b = 0; b < n_buffers; ++b)
      for (int64_t h = 0; h < kv_heads; ++h) {
        float *hb = kv[b] + h * stride;
        std::memmove(hb + keep * D, hb + src * D, tail * D * sizeof(float));
        const int64_t clear = max_len - (keep + tail);
        if (clear > 0)
          std::memset(hb + (keep + tail) * D, 0, clear * D * sizeof(float));
      }
    const int64_t half = D / 2;
    std::vector<float> c(half), s(half);
    const float delta = -(float)discard;
    for (int64_t i = 0; i < half; ++i) {
      const float expo = (2.0f * (float)i) / (float)D;
      const float inv = 1.0f / (float)std::pow(theta, expo);
      const float ang = inv * delta;
      c[i] = std::cos(ang);
      s[i] = std::sin(ang);
    }
    for (int64_t b = 0; b < n_buffers; b += 2)
      for (int64_t h = 0; h < kv_heads; ++h)
        for (int64_t t = 0; t < tail; ++t) {
          float *tp = kv[b] + h * stride + (keep + t) * D;
          for (int64_t i = 0; i < half; ++i) {
            const float v1 = tp[i], v2 = tp[i + half];
            float a0 = v1 * c[i], a1 = v2 * s[i];
            float b0 = v1 * s[i], b1 = v2 * c[i];
            tp[i] = a0 - a1;
            tp[i + half] = b0 + b1;
          }
        }
  }
  return std::min(std::max<int64_t>(cur - discard, 0), max_len);
}

// ---------------------------------------------------------------------------
static void linear(const OrcLinear &L, const float *x, float *y) {
  for (int64_t n = 0; n < L.N; ++n)
    y[n] = 0.0f;
  switch (L.kind) {
  case ORC_LIN_F32:
    orc_gemv_f32(x, (const float *)L.w, y, 1, L.K, L.N);
    break;
  case ORC_LIN_W8:
    orc_gemv_w8_f32(x, (const int8_t *)L.w, (const float *)L.scale, y, 1, L.K,
                    L.N);
    break;
  case ORC_LIN_W4G:
    orc_gemv_w4g_f32(x, (const uint8_t *)L.w, (const uint16_t *)L.scale, y, 1,
                     L.K, L.N, L.group);
    break;
  case ORC_LIN_W4: {
    // the w4a16 variant: f16 activations, f16 accumulation
    // (Int4DequantMatMulVectorizationDecode.cpp:359-430)
    std::vector<uint16_t> xh((size_t)L.K), yh((size_t)L.N, f16_to_bits((f16)0.0f));
    for (int64_t k = 0; k < L.K; ++k)
      xh[(size_t)k] = f16_to_bits((f16)x[k]);
    orc_gemv_w4_f16(xh.data(), (const int8_t *)L.w, (const uint16_t *)L.scale, yh.data(), 1, L.K, L.N);
    for (int64_t n = 0; n < L.N; ++n)
      y[n] = (float)bits_to_f16(yh[(size_t)n]);
    break;
  }
  case ORC_LIN_W8H: {
    // the w8a16 variant: f16 activations, f16 accumulation (DequantMatMulVectorizationDecode.cpp:
    // 250-321 instantiated for f16)
    std::vector<uint16_t> xh((size_t)L.K), yh((size_t)L.N, f16_to_bits((f16)0.0f));
    for (int64_t k = 0; k < L.K; ++k)
      xh[(size_t)k] = f16_to_bits((f16)x[k]);
    orc_gemv_w8_f16(xh.data(), (const int8_t *)L.w, (const uint16_t *)L.scale, yh.data(), 1, L.K, L.N);
    for (int64_t n = 0; n < L.N; ++n)
      y[n] = (float)bits_to_f16(yh[(size_t)n]);
    break;
  }
  case ORC_LIN_W8Q:
    // the w8a8 variant: the row is the whole activation tensor of a decode step
    orc_matmul_w8a8(x, (const int8_t *)L.w, (const float *)L.scale, nullptr, y, 1, L.K, L.N);
    break;
  default:
    std::abort();
  }
  if (L.bias)
    for (int64_t n = 0; n < L.N; ++n)
      y[n] = L.bias[n] + y[n];
}

// M rows through one projection: row by row, except where the activation scale
// belongs to the whole [M, K] tensor
static void linear_rows(const OrcLinear &L, const float *X, float *Y, int64_t M) {
  if (L.kind == ORC_LIN_W8Q) {
    orc_matmul_w8a8(X, (const int8_t *)L.w, (const float *)L.scale, nullptr, Y, M, L.K, L.N);
    if (L.bias)
      for (int64_t r = 0; r < M; ++r)
        for (int64_t n = 0; n < L.N; ++n)
          Y[r * L.N + n] = L.bias[n] + Y[r * L.N + n];
    return;
  }
  for (int64_t r = 0; r < M; ++r)
    linear(L, X + r * L.K, Y + r * L.N);
}

void orc_prefill_rows(const OrcModel *m, const int64_t *tokens, int64_t M, float **kv, float *logits) {
  const int64_t H = m->hidden, D = m->head_dim, F = m->ffn;
  const int64_t QD = m->q_heads * D, KD = m->kv_heads * D;
  std::vector<float> x((size_t)(M * H)), h((size_t)(M * H)), q((size_t)(M * QD)), k((size_t)(M * KD)),
      v((size_t)(M * KD)), att((size_t)(M * QD)), o((size_t)(M * H)), g((size_t)(M * F)), u((size_t)(M * F)),
      mid((size_t)(M * F));
  for (int64_t r = 0; r < M; ++r)
    std::memcpy(&x[(size_t)(r * H)], m->embed + tokens[r] * H, (size_t)H * sizeof(float));
  for (int64_t l = 0; l < m->n_layers; ++l) {
    const OrcLayer &L = m->layers[l];
    for (int64_t r = 0; r < M; ++r)
      orc_rmsnorm(&x[(size_t)(r * H)], L.in_norm, &h[(size_t)(r * H)], H, m->eps);
    linear_rows(L.q, h.data(), q.data(), M);
    linear_rows(L.k, h.data(), k.data(), M);
    linear_rows(L.v, h.data(), v.data(), M);
    float *Kc = kv[2 * l], *Vc = kv[2 * l + 1];
    for (int64_t r = 0; r < M; ++r) {
      float *qr = &q[(size_t)(r * QD)], *kr = &k[(size_t)(r * KD)], *vr = &v[(size_t)(r * KD)];
      if (L.q_norm)
        for (int64_t i = 0; i < m->q_heads; ++i)
          orc_rmsnorm(qr + i * D, L.q_norm, qr + i * D, D, m->eps);
      if (L.k_norm)
        for (int64_t i = 0; i < m->kv_heads; ++i)
          orc_rmsnorm(kr + i * D, L.k_norm, kr + i * D, D, m->eps);
      orc_rope(qr, m->q_heads, D, m->inv_freq, r);
      orc_rope(kr, m->kv_heads, D, m->inv_freq, r);
      for (int64_t i = 0; i < m->kv_heads; ++i) {
        std::memcpy(Kc + (i * m->max_len + r) * D, kr + i * D, (size_t)D * sizeof(float));
        std::memcpy(Vc + (i * m->max_len + r) * D, vr + i * D, (size_t)D * sizeof(float));
      }
    }
    for (int64_t r = 0; r < M; ++r)   // causal: row r sees keys 0..r
      orc_gqa_decode(&q[(size_t)(r * QD)], Kc, Vc, &att[(size_t)(r * QD)], m->q_heads, m->kv_heads, m->max_len, D, r);
    linear_rows(L.o, att.data(), o.data(), M);
    for (int64_t i = 0; i < M * H; ++i)
      x[(size_t)i] = x[(size_t)i] + o[(size_t)i];
    for (int64_t r = 0; r < M; ++r)
      orc_rmsnorm(&x[(size_t)(r * H)], L.post_norm, &h[(size_t)(r * H)], H, m->eps);
    linear_rows(L.gate, h.data(), g.data(), M);
    linear_rows(L.up, h.data(), u.data(), M);
    orc_silu_mul(g.data(), u.data(), mid.data(), M * F);
    linear_rows(L.down, mid.data(), o.data(), M);
    for (int64_t i = 0; i < M * H; ++i)
      x[(size_t)i] = x[(size_t)i] + o[(size_t)i];
  }
  for (int64_t r = 0; r < M; ++r)
    orc_rmsnorm(&x[(size_t)(r * H)], m->final_norm, &h[(size_t)(r * H)], H, m->eps);
  linear_rows(m->lm_head, h.data(), logits, M);
}

void orc_decode_step(const OrcModel *m, int64_t token, int64_t pos, float **kv,
                     float *logits) {
  const int64_t H = m->hidden, D = m->head_dim;
  const int64_t QD = m->q_heads * D, KD = m->kv_heads * D;
  std::vector<float> x(m->embed + token * H, m->embed + (token + 1) * H);
  std::vector<float> h(H), q(QD), k(KD), v(KD), att(QD), o(H), g(m->ffn),
      u(m->ffn), mid(m->ffn), d(H);
  for (int64_t l = 0; l < m->n_layers; ++l) {
    const OrcLayer &L = m->layers[l];
    orc_rmsnorm(x.data(), L.in_norm, h.data(), H, m->eps);
    linear(L.q, h.data(), q.data());
    linear(L.k, h.data(), k.data());
    linear(L.v, h.data(), v.data());
    if (L.q_norm)
      for (int64_t i = 0; i < m->q_heads; ++i)
        orc_rmsnorm(&q[i * D], L.q_norm, &q[i * D], D, m->eps);
    if (L.k_norm)
      for (int64_t i = 0; i < m->kv_heads; ++i)
        orc_rmsnorm(&k[i * D], L.k_norm, &k[i * D], D, m->eps);
    orc_rope(q.data(), m->q_heads, D, m->inv_freq, pos);
    orc_rope(k.data(), m->kv_heads, D, m->inv_freq, pos);
    float *Kc = kv[2 * l], *Vc = kv[2 * l + 1];
    for (int64_t i = 0; i < m->kv_heads; ++i) {
      std::memcpy(Kc + (i * m->max_len + pos) * D, &k[i * D], D * sizeof(float));
      std::memcpy(Vc + (i * m->max_len + pos) * D, &v[i * D], D * sizeof(float));
    }
    orc_gqa_decode(q.data(), Kc, Vc, att.data(), m->q_heads, m->kv_heads,
                   m->max_len, D, pos);
    linear(L.o, att.data(), o.data());
    for (int64_t i = 0; i < H; ++i)
      x[i] = x[i] + o[i];
    orc_rmsnorm(x.data(), L.post_norm, h.data(), H, m->eps);
    linear(L.gate, h.data(), g.data());
    linear(L.up, h.data(), u.data());
    orc_silu_mul(g.data(), u.data(), mid.data(), m->ffn);
    linear(L.down, mid.data(), d.data());
    for (int64_t i = 0; i < H; ++i)
      x[i] = x[i] + d[i];
  }
  orc_rmsnorm(x.data(), m->final_norm, h.data(), H, m->eps);
  linear(m->lm_head, h.data(), logits);
}

} // extern "C"

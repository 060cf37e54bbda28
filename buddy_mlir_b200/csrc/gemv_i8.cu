// One decode row of the w8a8 graphs: QuantizedMatmulOp / QuantizedAddMMOp
// (frontend/Python/ops/linalg.py:12728-12910) with a single activation row.
// The row gets its dynamic scale s = max(absmax / 127, 1e-10), is rounded to
// int8 (nearest even) and contracted exactly with the int8 weight rows by
// dp4a; y[n] = float(acc) * (s * scale[n]) (+ bias[n]).  Integer sums do not
// depend on the order of k, so every step matches the tensor-core form of the
// same operation (b200_gemm_w8a8) bit for bit.
//
// The projection streams its weights once: HBM-bound, N * K bytes per call.
#include "common.cuh"

#include <cstdint>

namespace b200 {

// One CTA: optional RMSNorm (subgraph0_decode_simplify.mlir:60-72), absmax, quantise.  q is
// written in the k order of the packed weight rows.
__global__ void __launch_bounds__(1024)
quantize_row_kernel(const float *x, const float *norm_w, float eps, int K, uint32_t *q, float *scale_out) {
  __shared__ float red[32];
  __shared__ float bc;
  const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5, nw = blockDim.x >> 5;
  float rinv = 1.f;
  if (norm_w) {
    float s = 0.f;
    for (int i = tid; i < K; i += blockDim.x)
      s = __fadd_rn(s, __fmul_rn(x[i], x[i]));
    s = warp_sum(s);
    if (lane == 0)
      red[wid] = s;
    __syncthreads();
    if (tid == 0) {
      float t = 0.f;
      for (int i = 0; i < nw; ++i)
        t += red[i];
      bc = rsqrtf(__fadd_rn(__fmul_rn(t, 1.0f / (float)K), eps));
    }
    __syncthreads();
    rinv = bc;
    __syncthreads();
  }
  auto value = [&](int i) { return norm_w ? __fmul_rn(norm_w[i], __fmul_rn(x[i], rinv)) : x[i]; };
  float mx = 0.f;
  for (int i = tid; i < K; i += blockDim.x)
    mx = fmaxf(mx, fabsf(value(i)));
  mx = warp_max(mx);
  if (lane == 0)
    red[wid] = mx;
  __syncthreads();
  if (tid == 0) {
    float t = 0.f;
    for (int i = 0; i < nw; ++i)
      t = fmaxf(t, red[i]);
    bc = t;
  }
  __syncthreads();
  // linalg.py:12728-12792
  const float scale = fmaxf(__fmul_rn(bc, __fdiv_rn(1.0f, 127.0f)), 1e-10f);
  const float inv = __fdiv_rn(1.0f, scale);
  if (tid == 0)
    *scale_out = scale;
  for (int k = tid * 4; k < K; k += blockDim.x * 4) {
    uint32_t pk = 0;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      float r = rintf(__fmul_rn(value(k + e), inv));     // the f32 -> i32 cast rounds to nearest even
      r = fminf(fmaxf(r, -128.0f), 127.0f);
      pk |= ((uint32_t)(int)r & 0xFFu) << (8 * e);
    }
    q[packed_offset(B200_W_I8, K, k, nullptr) >> 2] = pk;
  }
}

struct GemvI8 {
  const int8_t *w;        // packed rows, K bytes each
  const uint32_t *q;      // the quantised activation row, same k order (unfused form)
  const float *act_scale, *wscale, *bias, *residual;
  const float *x, *norm_w;   // fused form: the f32 row, quantised by every CTA for itself
  float eps;
  float *y;
  int K, N, silu_pairs;
  int ksplit;             // warps per pair of rows: 1, 2, 4 or 8
};

__device__ __forceinline__ float block_reduce_256(float v, bool is_max, float *red) {
  v = is_max ? warp_max(v) : warp_sum(v);
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  __syncthreads();          // red may still be read from the previous reduction
  if (lane == 0)
    red[wid] = v;
  __syncthreads();
  float t = red[0];
#pragma unroll
  for (int i = 1; i < 8; ++i)
    t = is_max ? fmaxf(t, red[i]) : t + red[i];
  return t;
}

// A warp takes two neighbouring output rows at a time (a gate / up pair when silu_pairs):
// 16-byte streaming loads down both rows, the activation row from shared memory, dp4a into two
// int32 sums.  FUSED: the CTA first builds the int8 row itself from the f32 input (RMSNorm,
// absmax, rounding: the arithmetic of quantize_row_kernel; every CTA gets the same codes and
// the same scale), which saves a launch per projection; needs 5 K bytes of shared memory.
template <bool FUSED>
__global__ void __launch_bounds__(256)
gemv_i8_kernel(const GemvI8 p) {
  extern __shared__ __align__(16) uint8_t sq[];
  __shared__ float red[8];
  const int chunks = p.K >> 4;
  float sa;
  if (FUSED) {
    float *xs = reinterpret_cast<float *>(sq + p.K);
    const int tid = threadIdx.x;
    float s = 0.f;
    for (int i = tid; i < p.K; i += 256) {
      const float v = p.x[i];
      xs[i] = v;
      s = __fadd_rn(s, __fmul_rn(v, v));
    }
    if (p.norm_w) {
      const float t = block_reduce_256(s, false, red);
      const float rinv = rsqrtf(__fadd_rn(__fmul_rn(t, 1.0f / (float)p.K), p.eps));
      for (int i = tid; i < p.K; i += 256)
        xs[i] = __fmul_rn(p.norm_w[i], __fmul_rn(xs[i], rinv));
    }
    float mx = 0.f;
    for (int i = tid; i < p.K; i += 256)
      mx = fmaxf(mx, fabsf(xs[i]));
    mx = block_reduce_256(mx, true, red);     // its barriers also publish xs
    sa = fmaxf(__fmul_rn(mx, __fdiv_rn(1.0f, 127.0f)), 1e-10f);
    const float inv = __fdiv_rn(1.0f, sa);
    for (int k = tid * 4; k < p.K; k += 1024) {
      uint32_t pk = 0;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float r = rintf(__fmul_rn(xs[k + e], inv));
        r = fminf(fmaxf(r, -128.0f), 127.0f);
        pk |= ((uint32_t)(int)r & 0xFFu) << (8 * e);
      }
      reinterpret_cast<uint32_t *>(sq)[packed_offset(B200_W_I8, p.K, k, nullptr) >> 2] = pk;
    }
  } else {
    for (int i = threadIdx.x; i < chunks; i += blockDim.x)
      reinterpret_cast<int4 *>(sq)[i] = reinterpret_cast<const int4 *>(p.q)[i];
    sa = *p.act_scale;
  }
  __syncthreads();
  // ksplit warps share a pair of rows (each takes every ksplit-th group of 32 chunks), so that
  // a narrow projection still fills the SMs; their integer partial sums are added in any order
  __shared__ int part[8][2];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int ks = p.ksplit, per_cta = 8 / ks, sub = warp % ks, slot = warp / ks;
  const int pairs = (p.N + 1) >> 1;
  for (int base = blockIdx.x * per_cta; base < pairs; base += gridDim.x * per_cta) {
    const int pair = base + slot;
    const bool live = pair < pairs;
    const int n0 = pair * 2;
    const bool two = n0 + 1 < p.N;
    int a0 = 0, a1 = 0;
    if (live) {
      const int4 *r0 = reinterpret_cast<const int4 *>(p.w + (int64_t)n0 * p.K);
      const int4 *r1 = two ? r0 + chunks : r0;
#pragma unroll 4
      for (int c = sub * 32 + lane; c < chunks; c += 32 * ks) {
        const int4 w0 = __ldcs(r0 + c), w1 = __ldcs(r1 + c);
        const int4 qq = reinterpret_cast<const int4 *>(sq)[c];
        a0 = __dp4a(w0.x, qq.x, a0);
        a0 = __dp4a(w0.y, qq.y, a0);
        a0 = __dp4a(w0.z, qq.z, a0);
        a0 = __dp4a(w0.w, qq.w, a0);
        a1 = __dp4a(w1.x, qq.x, a1);
        a1 = __dp4a(w1.y, qq.y, a1);
        a1 = __dp4a(w1.z, qq.z, a1);
        a1 = __dp4a(w1.w, qq.w, a1);
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        a0 += __shfl_xor_sync(0xffffffffu, a0, o);
        a1 += __shfl_xor_sync(0xffffffffu, a1, o);
      }
    }
    if (ks > 1) {
      if (lane == 0) {
        part[warp][0] = a0;
        part[warp][1] = a1;
      }
      __syncthreads();
      if (sub == 0 && lane == 0)
        for (int j = 1; j < ks; ++j) {
          a0 += part[warp + j][0];
          a1 += part[warp + j][1];
        }
    }
    if (live && sub == 0 && lane == 0) {
      // linalg.py:12836-12846: float(acc) * (act_scale * weight_scale[n]), then the bias
      float y0 = __fmul_rn(__int2float_rn(a0), __fmul_rn(sa, p.wscale[n0]));
      float y1 = two ? __fmul_rn(__int2float_rn(a1), __fmul_rn(sa, p.wscale[n0 + 1])) : 0.f;
      if (p.bias) {
        y0 = __fadd_rn(y0, p.bias[n0]);
        if (two)
          y1 = __fadd_rn(y1, p.bias[n0 + 1]);
      }
      if (p.silu_pairs) {   // subgraph0_decode_simplify.mlir:226-231 on (gate, up) = rows (2j, 2j + 1)
        const float s = 1.0f / (1.0f + expf(-y0));
        p.y[n0 >> 1] = __fmul_rn(__fmul_rn(y0, s), y1);
      } else {
        if (p.residual) {
          y0 = __fadd_rn(p.residual[n0], y0);
          if (two)
            y1 = __fadd_rn(p.residual[n0 + 1], y1);
        }
        p.y[n0] = y0;
        if (two)
          p.y[n0 + 1] = y1;
      }
    }
    if (ks > 1)
      __syncthreads();     // part is rewritten by the next round
  }
}

int quantize_row_launch(const float *x, const float *norm_w, float eps, int64_t K, uint32_t *q, float *scale,
                        cudaStream_t st) {
  if (!x || !q || !scale || K < 64 || K % 64 != 0)
    return fail(B200_EINVAL, "quantize_row: K must be a positive multiple of 64");
  quantize_row_kernel<<<1, K >= 4096 ? 1024 : 512, 0, st>>>(x, norm_w, eps, (int)K, q, scale);
  B200_LAUNCH_CHECK();
  return B200_OK;
}

static int gemv_i8_check(const b200_weight *w, int silu_pairs) {
  if (w->kind != B200_W_I8 || w->scale_dtype != B200_F32 || !w->scale || !w->w || w->K % 64 != 0 ||
      ((uintptr_t)w->w & 15))
    return fail(B200_EINVAL, "gemv_i8: int8 per-channel weights with f32 scales and K a multiple of 64 expected");
  if (w->K > 48 * 1024)
    return fail(B200_ELIMIT, "gemv_i8: K = %lld exceeds the staged activation row (49152)", (long long)w->K);
  if (silu_pairs && (w->N & 1))
    return fail(B200_EINVAL, "gemv_i8: gate / up pairs need an even N");
  return B200_OK;
}

static GemvI8 gemv_i8_params(const b200_weight *w, const float *residual, float *y, int silu_pairs) {
  GemvI8 p{};
  p.w = (const int8_t *)w->w;
  p.wscale = (const float *)w->scale;
  p.bias = (const float *)w->bias;
  p.residual = residual;
  p.y = y;
  p.K = (int)w->K;
  p.N = (int)w->N;
  p.silu_pairs = silu_pairs;
  return p;
}

// warps per pair of rows: the fewest that still give every SM two CTAs
static int gemv_i8_ksplit(int64_t N) {
  const int64_t pairs = (N + 1) / 2;
  int ks = 1;
  while (ks < 8 && pairs * ks / 8 < 2 * 148)
    ks *= 2;
  return ks;
}
static unsigned gemv_i8_grid(int64_t N, int ks) {
  const int64_t per_cta = 8 / ks, ctas = ((N + 1) / 2 + per_cta - 1) / per_cta;
  return (unsigned)(ctas < 148 * 6 ? ctas : 148 * 6);
}

int gemv_i8_launch(const b200_weight *w, const uint32_t *q, const float *act_scale, const float *residual, float *y,
                   int silu_pairs, cudaStream_t st) {
  if (!w || !q || !act_scale || !y)
    return fail(B200_EINVAL, "gemv_i8: null argument");
  if (int rc = gemv_i8_check(w, silu_pairs)) return rc;
  GemvI8 p = gemv_i8_params(w, residual, y, silu_pairs);
  p.q = q;
  p.act_scale = act_scale;
  p.ksplit = gemv_i8_ksplit(w->N);
  gemv_i8_kernel<false><<<gemv_i8_grid(w->N, p.ksplit), 256, (size_t)w->K, st>>>(p);
  B200_LAUNCH_CHECK();
  return B200_OK;
}

// Fits the fused form: the int8 row and its f32 source in 48 KB of shared memory.
bool gemv_i8_fusable(int64_t K) { return K * 5 <= 48 * 1024; }

// One launch per projection: x (f32, not y) is normalised and quantised inside every CTA.
int gemv_i8_fused_launch(const b200_weight *w, const float *x, const float *norm_w, float eps, const float *residual,
                         float *y, int silu_pairs, cudaStream_t st) {
  if (!w || !x || !y || x == y)
    return fail(B200_EINVAL, "gemv_i8: null or aliased argument");
  if (int rc = gemv_i8_check(w, silu_pairs)) return rc;
  if (!gemv_i8_fusable(w->K))
    return fail(B200_ELIMIT, "gemv_i8: K = %lld does not fit the fused form", (long long)w->K);
  GemvI8 p = gemv_i8_params(w, residual, y, silu_pairs);
  p.x = x;
  p.norm_w = norm_w;
  p.eps = eps;
  p.ksplit = gemv_i8_ksplit(w->N);
  gemv_i8_kernel<true><<<gemv_i8_grid(w->N, p.ksplit), 256, (size_t)w->K * 5, st>>>(p);
  B200_LAUNCH_CHECK();
  return B200_OK;
}

} // namespace b200

// GQA decode attention: one query row per head against cache rows [0, pos].
//
// Replaces gqa_attention_fused_op (frontend/Python/ops/tosa.py:13931-14635).
// The reference walks all max_len cache rows under an additive -inf mask, in
// 4 k-splits of 16-row blocks, with the online-softmax recurrence
//   new_m = max(m, s); alpha = exp(m - new_m); p = exp(s - new_m);
//   l = l*alpha + p;   acc = acc*alpha + p*V
// seeded (-1e30, 0, 0), and folds the splits with the same recurrence
// (tosa.py:14245-14252, 14502-14594).  Masked rows contribute exactly 0, so
// this kernel scans only the live rows: the grid is (splits, kv_heads), one
// CTA serves the G query heads that share a kv head (each K/V row is loaded
// once for all of them), a warp owns every 4th row of the CTA's range, lanes
// own D/32 consecutive dims.  The split partials (m, l, acc) go to scratch;
// the last CTA of a kv head to finish folds them in split order, so the
// result does not depend on CTA scheduling.
#include "common.cuh"

#include <mutex>

namespace b200 {

constexpr int kAttnWarps = 8;
constexpr float kSeed = -1.0e30f;

template <int G, int VEC>
__global__ void __launch_bounds__(kAttnWarps * 32)
gqa_decode_kernel(const float *__restrict__ q, const float *__restrict__ kc,
                  const float *__restrict__ vc, float *__restrict__ out,
                  float *scratch, int q_heads, int kv_heads, int max_len,
                  int splits, const int32_t *posp) {
  constexpr int D = VEC * 32;
  const int split = blockIdx.x, hk = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int len = min(max(*posp, 0), max_len - 1) + 1;   // a position outside the cache never leaves it
  const int chunk = (len + splits - 1) / splits;
  const int s0 = split * chunk;
  const int s1 = min(len, s0 + chunk);
  const float scale = rsqrtf((float)D);

  float qr[G][VEC];
#pragma unroll
  for (int g = 0; g < G; ++g)
#pragma unroll
    for (int e = 0; e < VEC; ++e)
      qr[g][e] = q[(int64_t)(hk * G + g) * D + lane * VEC + e];

  float m[G], l[G], acc[G][VEC];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    m[g] = kSeed;
    l[g] = 0.f;
#pragma unroll
    for (int e = 0; e < VEC; ++e)
      acc[g][e] = 0.f;
  }

  const float *kbase = kc + (int64_t)hk * max_len * D + lane * VEC;
  const float *vbase = vc + (int64_t)hk * max_len * D + lane * VEC;
  // NB rows in flight per warp: all loads of a round are issued before the first use
  constexpr int NB = G <= 4 ? 4 : 2;
  for (int j0 = s0 + warp; j0 < s1; j0 += NB * kAttnWarps) {
    float kr[NB][VEC], vr[NB][VEC];
#pragma unroll
    for (int i = 0; i < NB; ++i) {
      const int j = min(j0 + i * kAttnWarps, s1 - 1);
      if (VEC == 4) {
        const float4 k4 = *reinterpret_cast<const float4 *>(kbase + (int64_t)j * D);
        const float4 v4 = *reinterpret_cast<const float4 *>(vbase + (int64_t)j * D);
        kr[i][0] = k4.x; kr[i][1] = k4.y; kr[i][2] = k4.z; kr[i][3] = k4.w;
        vr[i][0] = v4.x; vr[i][1] = v4.y; vr[i][2] = v4.z; vr[i][3] = v4.w;
      } else {
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
          kr[i][e] = kbase[(int64_t)j * D + e];
          vr[i][e] = vbase[(int64_t)j * D + e];
        }
      }
    }
#pragma unroll
    for (int i = 0; i < NB; ++i) {
      if (j0 + i * kAttnWarps >= s1)   // warp-uniform
        break;
      float s[G];
#pragma unroll
      for (int g = 0; g < G; ++g) {
        float d = 0.f;
#pragma unroll
        for (int e = 0; e < VEC; ++e)
          d = fmaf(qr[g][e], kr[i][e], d);
        s[g] = d;
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1)
#pragma unroll
        for (int g = 0; g < G; ++g)
          s[g] += __shfl_xor_sync(0xffffffffu, s[g], o);
#pragma unroll
      for (int g = 0; g < G; ++g) {
        s[g] *= scale;
        const float nm = fmaxf(m[g], s[g]);
        const float alpha = expf(m[g] - nm);
        const float p = expf(s[g] - nm);
        l[g] = fmaf(l[g], alpha, p);
#pragma unroll
        for (int e = 0; e < VEC; ++e)
          acc[g][e] = fmaf(acc[g][e], alpha, p * vr[i][e]);
        m[g] = nm;
      }
    }
  }

  // ---- fold the warps of this CTA (fixed warp order) -----------------------
  __shared__ float s_m[kAttnWarps][G], s_l[kAttnWarps][G];
  __shared__ float s_acc[kAttnWarps][G][D];
  __shared__ bool s_last;
#pragma unroll
  for (int g = 0; g < G; ++g) {
    if (lane == 0) {
      s_m[warp][g] = m[g];
      s_l[warp][g] = l[g];
    }
#pragma unroll
    for (int e = 0; e < VEC; ++e)
      s_acc[warp][g][lane * VEC + e] = acc[g][e];
  }
  __syncthreads();
  const int stride = D + 2;
  for (int idx = threadIdx.x; idx < G * D; idx += blockDim.x) {
    const int g = idx / D, d = idx - g * D;
    float M = kSeed;
#pragma unroll
    for (int w = 0; w < kAttnWarps; ++w)
      M = fmaxf(M, s_m[w][g]);
    float L = 0.f, A = 0.f;
#pragma unroll
    for (int w = 0; w < kAttnWarps; ++w) {
      const float b = expf(s_m[w][g] - M);
      L = fmaf(s_l[w][g], b, L);
      A = fmaf(s_acc[w][g][d], b, A);
    }
    float *part = scratch + ((int64_t)(hk * G + g) * splits + split) * stride;
    part[d] = A;
    if (d == 0) {
      part[D] = M;
      part[D + 1] = L;
    }
  }

  // ---- last CTA of this kv head folds the splits ----------------------------
  unsigned int *counters =
      reinterpret_cast<unsigned int *>(scratch + (int64_t)q_heads * splits * stride);
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int done = atomicAdd(&counters[hk], 1u);
    s_last = (done == (unsigned int)splits - 1);
    if (s_last)
      counters[hk] = 0;  // ready for the next launch
  }
  __syncthreads();
  if (!s_last)
    return;
  __threadfence();
  constexpr int kFoldSplits = 128;   // splits the parallel fold below keeps in shared memory
  if (splits <= kFoldSplits) {
    // Weights first (one warp per head: M = max m_s, w_s = exp(m_s - M), L = sum l_s w_s),
    // then every output is a sum of independent loads.  Same result as the running
    // recurrence of tosa.py:14502-14594 up to rounding, without its chain of
    // dependent loads over the splits.
    __shared__ float f_w[G][kFoldSplits];
    __shared__ float f_L[G];
    if (warp < G) {
      const float *parts = scratch + (int64_t)(hk * G + warp) * splits * stride + D;
      float ms[kFoldSplits / 32], ls[kFoldSplits / 32];
      float M = kSeed;
#pragma unroll
      for (int i = 0; i < kFoldSplits / 32; ++i) {
        const int sidx = lane + 32 * i;
        ms[i] = kSeed;
        ls[i] = 0.f;
        if (sidx < splits) {
          ms[i] = __ldcg(&parts[(int64_t)sidx * stride]);
          ls[i] = __ldcg(&parts[(int64_t)sidx * stride + 1]);
        }
        M = fmaxf(M, ms[i]);
      }
      M = warp_max(M);
      float L = 0.f;
#pragma unroll
      for (int i = 0; i < kFoldSplits / 32; ++i) {
        const int sidx = lane + 32 * i;
        const float b = expf(ms[i] - M);
        if (sidx < splits)
          f_w[warp][sidx] = b;
        L = fmaf(ls[i], b, L);
      }
      L = warp_sum(L);
      if (lane == 0)
        f_L[warp] = L;
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < G * D; idx += blockDim.x) {
      const int g = idx / D, d = idx - g * D;
      const float *parts = scratch + (int64_t)(hk * G + g) * splits * stride + d;
      float ar = 0.f;
      int sidx = 0;
      for (; sidx + 16 <= splits; sidx += 16) {   // 16 independent loads in flight
        float v[16];
#pragma unroll
        for (int u = 0; u < 16; ++u)
          v[u] = __ldcg(&parts[(int64_t)(sidx + u) * stride]);
#pragma unroll
        for (int u = 0; u < 16; ++u)
          ar = fmaf(v[u], f_w[g][sidx + u], ar);
      }
      for (; sidx < splits; ++sidx)
        ar = fmaf(__ldcg(&parts[(int64_t)sidx * stride]), f_w[g][sidx], ar);
      out[(int64_t)(hk * G + g) * D + d] = __fdiv_rn(ar, f_L[g]);
    }
    return;
  }
  for (int idx = threadIdx.x; idx < G * D; idx += blockDim.x) {
    const int g = idx / D, d = idx - g * D;
    const float *parts = scratch + (int64_t)(hk * G + g) * splits * stride;
    // tosa.py:14502-14594: running (m, l, acc) over the splits in order
    float mr = kSeed, lr = 0.f, ar = 0.f;
    for (int s = 0; s < splits; ++s) {
      const float ms = __ldcg(&parts[s * stride + D]);
      const float ls = __ldcg(&parts[s * stride + D + 1]);
      const float as = __ldcg(&parts[s * stride + d]);
      const float mn = ms > mr ? ms : mr;
      const float a = expf(mr - mn), b = expf(ms - mn);
      lr = __fadd_rn(__fmul_rn(lr, a), __fmul_rn(ls, b));
      ar = fmaf(as, b, __fmul_rn(ar, a));
      mr = mn;
    }
    out[(int64_t)(hk * G + g) * D + d] = __fdiv_rn(ar, lr);
  }
}

template <int G>
static int launch_g(const float *q, const float *kc, const float *vc,
                    float *out, float *scratch, int q_heads, int kv_heads,
                    int D, int max_len, int splits, const int32_t *pos,
                    cudaStream_t st) {
  dim3 grid(splits, kv_heads);
  if (D == 128)
    gqa_decode_kernel<G, 4><<<grid, kAttnWarps * 32, 0, st>>>(
        q, kc, vc, out, scratch, q_heads, kv_heads, max_len, splits, pos);
  else if (D == 64)
    gqa_decode_kernel<G, 2><<<grid, kAttnWarps * 32, 0, st>>>(
        q, kc, vc, out, scratch, q_heads, kv_heads, max_len, splits, pos);
  else
    return fail(B200_EINVAL, "gqa_decode: head_dim %d (64 or 128 supported)", D);
  B200_LAUNCH_CHECK();
  return B200_OK;
}

// Host-side argument check shared by both entry points; nothing touches the
// device before it has passed.
static int gqa_decode_check(const float *q, const float *kc, const float *vc, float *out,
                            const float *scratch, int q_heads, int kv_heads, int D, int max_len,
                            int splits, const int32_t *pos) {
  if (!q || !kc || !vc || !out || !scratch || !pos)
    return fail(B200_EINVAL, "gqa_decode: null argument");
  if (q_heads < 1 || kv_heads < 1 || kv_heads > q_heads || q_heads % kv_heads || splits < 1 ||
      splits > 1024 || max_len < 1)
    return fail(B200_EINVAL, "gqa_decode: bad shape");
  if (D != 64 && D != 128)
    return fail(B200_EINVAL, "gqa_decode: head_dim %d (64 or 128 supported)", D);
  const int G = q_heads / kv_heads;
  if (G != 1 && G != 2 && G != 3 && G != 4 && G != 6 && G != 8)
    return fail(B200_EINVAL, "gqa_decode: group size %d not built", G);
  return B200_OK;
}

int gqa_decode_launch(const float *q, const float *kc, const float *vc,
                      float *out, float *scratch, int q_heads, int kv_heads,
                      int D, int max_len, int splits, const int32_t *pos,
                      cudaStream_t st) {
  if (int rc = gqa_decode_check(q, kc, vc, out, scratch, q_heads, kv_heads, D, max_len, splits, pos))
    return rc;
  const int G = q_heads / kv_heads;
  switch (G) {
#define B200_G(G_)                                                             \
  case G_:                                                                     \
    return launch_g<G_>(q, kc, vc, out, scratch, q_heads, kv_heads, D,         \
                        max_len, splits, pos, st);
    B200_G(1) B200_G(2) B200_G(3) B200_G(4) B200_G(6) B200_G(8)
#undef B200_G
  default:
    return fail(B200_EINVAL, "gqa_decode: group size %d not built", G);
  }
}

// ---- scratch that lives in the library image ------------------------------------
// Split partials for b200_gqa_decode_static(): enough for 64 query heads x 32
// splits x (128 + 2) floats plus the arrival counters, about 1.07 MB.  Every
// GPU that loads this library keeps the array until the process exits.
constexpr int64_t kStaticScratchFloats = B200_GQA_STATIC_SCRATCH_FLOATS;
static __device__ __align__(256) float g_gqa_static_scratch[kStaticScratchFloats];

} // namespace b200

using namespace b200;

extern "C" {

int64_t b200_gqa_scratch_floats(int q_heads, int D, int splits) {
  // partials [q_heads][splits][D+2] + one arrival counter per kv head
  return (int64_t)q_heads * splits * (D + 2) + q_heads;
}

int b200_gqa_decode_static(const float *q, const float *k_cache, const float *v_cache, float *out,
                           int q_heads, int kv_heads, int D, int max_len, int splits,
                           const int32_t *pos, void *stream) {
  // Every argument is checked on the host first: a rejected call returns before
  // any device work (the counter clear below included).
  static const float kNotNull = 0.f;   // stands in for the scratch pointer during the check
  if (int rc = gqa_decode_check(q, k_cache, v_cache, out, &kNotNull, q_heads, kv_heads, D, max_len,
                                splits, pos))
    return rc;
  if (int rc = ensure_device())
    return rc;
  const int64_t need = b200_gqa_scratch_floats(q_heads, D, splits);
  if (need > kStaticScratchFloats)
    return fail(B200_ELIMIT,
                "gqa_decode_static: q_heads=%d x splits=%d x (D=%d + 2) needs %lld scratch floats, "
                "the built-in array holds %lld; use b200_gqa_decode with caller-owned scratch",
                q_heads, splits, D, (long long)need, (long long)kStaticScratchFloats);
  // Device address of the array, looked up once per device with that device
  // current.  (In host code the array's name is only a handle for this lookup,
  // never a pointer a kernel could use.)
  constexpr int kMaxDevices = 64;
  static float *addr[kMaxDevices] = {};
  static std::mutex mu;
  int dev = 0;
  B200_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices)
    return fail(B200_ELIMIT, "gqa_decode_static: device ordinal %d beyond %d", dev, kMaxDevices);
  float *scratch = nullptr;
  {
    std::lock_guard<std::mutex> lock(mu);
    if (addr[dev] == nullptr) {
      void *p = nullptr;
      cudaError_t e = cudaGetSymbolAddress(&p, g_gqa_static_scratch);
      if (e != cudaSuccess || p == nullptr)
        return fail(B200_ECUDA, "gqa_decode_static: cudaGetSymbolAddress: %s",
                    cudaGetErrorString(e));
      addr[dev] = static_cast<float *>(p);
    }
    scratch = addr[dev];
  }
  // The array keeps whatever the previous call (possibly of another shape)
  // left behind; only the arrival counters have to start at zero.
  cudaStream_t st = (cudaStream_t)stream;
  // (kv_heads <= q_heads was checked above, and the size check reserved q_heads counters)
  float *counters = scratch + (int64_t)q_heads * splits * (D + 2);
  B200_CUDA(cudaMemsetAsync(counters, 0, (size_t)kv_heads * sizeof(unsigned int), st));
  return gqa_decode_launch(q, k_cache, v_cache, out, scratch, q_heads, kv_heads, D, max_len,
                           splits, pos, st);
}

int b200_gqa_decode(const float *q, const float *k_cache, const float *v_cache,
                    float *out, float *scratch, int q_heads, int kv_heads,
                    int D, int max_len, int splits, const int32_t *pos,
                    void *stream) {
  if (int rc = ensure_device())
    return rc;
  return gqa_decode_launch(q, k_cache, v_cache, out, scratch, q_heads,
                           kv_heads, D, max_len, splits, pos,
                           (cudaStream_t)stream);
}

} // extern "C"

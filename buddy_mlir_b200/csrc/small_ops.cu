// The small f32 ops around the GEMVs of one decode step.  In buddy-mlir these
// are un-fused ATen decompositions; the concrete graph is
// examples/BuddyDeepSeekR1/subgraph0_decode_simplify.mlir:46-260.  Multiply
// and add stay separate roundings (__fmul_rn / __fadd_rn) wherever that IR
// has separate tosa.mul / tosa.add ops.
#include "common.cuh"

#include <cmath>
#include <vector>

namespace b200 {

// subgraph0_decode_simplify.mlir:60-72
__global__ void rmsnorm_kernel(const float *x, const float *w, float *y,
                               int64_t H, float eps) {
  __shared__ float red[32];
  __shared__ float rinv;
  const float *xr = x + (int64_t)blockIdx.x * H;
  float *yr = y + (int64_t)blockIdx.x * H;
  float s = 0.f;
  for (int64_t i = threadIdx.x; i < H; i += blockDim.x)
    s = __fadd_rn(s, __fmul_rn(xr[i], xr[i]));
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0)
    red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int i = 0; i < (int)(blockDim.x >> 5); ++i)
      t += red[i];
    rinv = rsqrtf(__fadd_rn(__fmul_rn(t, 1.0f / (float)H), eps));
  }
  __syncthreads();
  for (int64_t i = threadIdx.x; i < H; i += blockDim.x)
    yr[i] = __fmul_rn(w[i], __fmul_rn(xr[i], rinv));
}

// subgraph0_decode_simplify.mlir:226-231
__global__ void silu_mul_kernel(const float *g, const float *u, float *y,
                                int64_t n) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) {
    const float s = 1.0f / (1.0f + expf(-g[i]));
    y[i] = __fmul_rn(__fmul_rn(g[i], s), u[i]);
  }
}

// subgraph0_decode_simplify.mlir:52-59 (angles), 86-105 (rotate), 106-142 (KV
// write).  One CTA per head (q heads first, then kv heads), one thread per
// (j, j + D/2) pair.
__global__ void rope_kv_write_kernel(float *q, float *k, const float *v,
                                     float *k_cache, float *v_cache,
                                     const float *inv_freq,
                                     const float *q_norm, const float *k_norm,
                                     float eps, int q_heads, int kv_heads,
                                     int D, int max_len, const int32_t *posp,
                                     float *k_stage, float *v_stage) {
  __shared__ float red[8];
  const int half = D / 2;
  const int j = threadIdx.x;
  const int head = blockIdx.x;
  const bool is_q = head < q_heads;
  const int h = is_q ? head : head - q_heads;
  float *p = (is_q ? q : k) + (int64_t)h * D;
  const float *nw = is_q ? q_norm : k_norm;
  const int pos = *posp;
  float a = 0.f, b = 0.f;
  if (j < half) {
    a = p[j];
    b = p[j + half];
  }
  if (nw != nullptr) {
    // per-head RMSNorm over head_dim (Qwen3 q_norm / k_norm)
    float s = warp_sum(__fadd_rn(__fmul_rn(a, a), __fmul_rn(b, b)));
    if ((threadIdx.x & 31) == 0)
      red[threadIdx.x >> 5] = s;
    __syncthreads();
    float t = 0.f;
    for (int i = 0; i < (int)((blockDim.x + 31) >> 5); ++i)
      t += red[i];
    const float r = rsqrtf(__fadd_rn(__fmul_rn(t, 1.0f / (float)D), eps));
    if (j < half) {
      a = __fmul_rn(nw[j], __fmul_rn(a, r));
      b = __fmul_rn(nw[j + half], __fmul_rn(b, r));
    }
  }
  if (j >= half)
    return;
  const float th = __fmul_rn(inv_freq[j], (float)pos);
  const float c = cosf(th), s = sinf(th);
  // q' = q*cos + rotate_half(q)*sin, rotate_half(x) = [-x[half:], x[:half]]
  const float oa = __fadd_rn(__fmul_rn(a, c), __fmul_rn(-b, s));
  const float ob = __fadd_rn(__fmul_rn(b, c), __fmul_rn(a, s));
  p[j] = oa;
  p[j + half] = ob;
  if (!is_q) {
    const int64_t row = ((int64_t)h * max_len + pos) * D;
    k_cache[row + j] = oa;
    k_cache[row + j + half] = ob;
    const float va = v[(int64_t)h * D + j], vb = v[(int64_t)h * D + j + half];
    v_cache[row + j] = va;
    v_cache[row + j + half] = vb;
    if (k_stage != nullptr) {  // contiguous copy of the new rows for the host mirror
      k_stage[(int64_t)h * D + j] = oa;
      k_stage[(int64_t)h * D + j + half] = ob;
      v_stage[(int64_t)h * D + j] = va;
      v_stage[(int64_t)h * D + j + half] = vb;
    }
  }
}

// subgraph0_decode_simplify.mlir:46-49
__global__ void embed_kernel(const float *table, const int32_t *token, float *x,
                             int64_t H) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < H)
    x[i] = table[(int64_t)(*token) * H + i];
}

// Sampler.h:101-104 (std::max_element: first maximum).
__device__ __forceinline__ void better(float &bv, int &bi, float v, int i) {
  if (v > bv || (v == bv && i < bi)) {
    bv = v;
    bi = i;
  }
}
__device__ void block_argmax(float &bv, int &bi) {
  __shared__ float sv[32];
  __shared__ int si[32];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    better(bv, bi, ov, oi);
  }
  if ((threadIdx.x & 31) == 0) {
    sv[threadIdx.x >> 5] = bv;
    si[threadIdx.x >> 5] = bi;
  }
  __syncthreads();
  if (threadIdx.x < 32) {
    const int nw = blockDim.x >> 5;
    bv = threadIdx.x < nw ? sv[threadIdx.x] : -INFINITY;
    bi = threadIdx.x < nw ? si[threadIdx.x] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      better(bv, bi, ov, oi);
    }
  }
}
__global__ void argmax_part_kernel(const float *v, int64_t n, float *pv,
                                   int *pi) {
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x)
    better(bv, bi, v[i], (int)i);
  block_argmax(bv, bi);
  if (threadIdx.x == 0) {
    pv[blockIdx.x] = bv;
    pi[blockIdx.x] = bi;
  }
}
__global__ void argmax_final_kernel(const float *pv, const int *pi, int parts,
                                    int32_t *out) {
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < parts; i += blockDim.x)
    better(bv, bi, pv[i], pi[i]);
  block_argmax(bv, bi);
  if (threadIdx.x == 0)
    *out = bi == 0x7fffffff ? 0 : bi;
}

// KVCacheManager.h:151-194 (discard + move + zero) and :196-273 (rotate K by
// -discardLen positions), in two passes through a staging buffer because the
// move overlaps itself.
__global__ void kv_tail_stage_kernel(float *const *kv, int kv_heads,
                                     int max_len, int D, int src, int tail,
                                     const float *cs, const float *sn,
                                     float *stage) {
  // grid: (tail, kv_heads, n_buffers); thread: pair index
  const int t = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int half = D / 2, i = threadIdx.x;
  if (i >= half)
    return;
  const float *row = kv[b] + ((int64_t)h * max_len + src + t) * D;
  float *dst = stage + (((int64_t)b * kv_heads + h) * tail + t) * D;
  const float v1 = row[i], v2 = row[i + half];
  if ((b & 1) == 0) {  // K caches sit at even indices
    dst[i] = __fsub_rn(__fmul_rn(v1, cs[i]), __fmul_rn(v2, sn[i]));
    dst[i + half] = __fadd_rn(__fmul_rn(v1, sn[i]), __fmul_rn(v2, cs[i]));
  } else {
    dst[i] = v1;
    dst[i + half] = v2;
  }
}
__global__ void kv_tail_commit_kernel(float *const *kv, int kv_heads,
                                      int max_len, int D, int keep, int tail,
                                      const float *stage) {
  // grid: (max_len - keep, kv_heads, n_buffers)
  const int t = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  float *row = kv[b] + ((int64_t)h * max_len + keep + t) * D;
  const float *src = stage + (((int64_t)b * kv_heads + h) * tail + t) * D;
  for (int i = threadIdx.x; i < D; i += blockDim.x)
    row[i] = t < tail ? src[i] : 0.f;
}

int rope_kv_write_launch(float *q, float *k, const float *v, float *k_cache,
                         float *v_cache, const float *inv_freq,
                         const float *q_norm, const float *k_norm, float eps,
                         int q_heads, int kv_heads, int D, int max_len,
                         const int32_t *pos, float *k_stage, float *v_stage,
                         cudaStream_t st) {
  if (!q || !k || !v || !k_cache || !v_cache || !inv_freq || !pos)
    return fail(B200_EINVAL, "rope_kv_write: null argument");
  if (D < 2 || (D & 1) || D > 512 || q_heads < 1 || kv_heads < 1)
    return fail(B200_EINVAL, "rope_kv_write: bad head shape");
  const int threads = ((D / 2 + 31) / 32) * 32;
  rope_kv_write_kernel<<<q_heads + kv_heads, threads, 0, st>>>(
      q, k, v, k_cache, v_cache, inv_freq, q_norm, k_norm, eps, q_heads,
      kv_heads, D, max_len, pos, k_stage, v_stage);
  B200_LAUNCH_CHECK();
  return B200_OK;
}

} // namespace b200

using namespace b200;

extern "C" {

int b200_rmsnorm(const float *x, const float *w, float *y, int64_t rows,
                 int64_t H, float eps, void *stream) {
  if (!x || !w || !y || rows < 0 || H < 1)
    return fail(B200_EINVAL, "rmsnorm: bad argument");
  if (rows == 0)
    return B200_OK;
  if (int rc = ensure_device())
    return rc;
  rmsnorm_kernel<<<(unsigned)rows, 256, 0, (cudaStream_t)stream>>>(x, w, y, H,
                                                                   eps);
  B200_LAUNCH_CHECK();
  return B200_OK;
}

int b200_silu_mul(const float *g, const float *u, float *y, int64_t n,
                  void *stream) {
  if (!g || !u || !y || n < 0)
    return fail(B200_EINVAL, "silu_mul: bad argument");
  if (n == 0)
    return B200_OK;
  if (int rc = ensure_device())
    return rc;
  silu_mul_kernel<<<(unsigned)((n + 255) / 256), 256, 0,
                    (cudaStream_t)stream>>>(g, u, y, n);
  B200_LAUNCH_CHECK();
  return B200_OK;
}

int b200_rope_kv_write(float *q, float *k, const float *v, float *k_cache,
                       float *v_cache, const float *inv_freq,
                       const float *q_norm, const float *k_norm, float eps,
                       int q_heads, int kv_heads, int D, int max_len,
                       const int32_t *pos, void *stream) {
  if (int rc = ensure_device())
    return rc;
  return rope_kv_write_launch(q, k, v, k_cache, v_cache, inv_freq, q_norm,
                              k_norm, eps, q_heads, kv_heads, D, max_len, pos,
                              nullptr, nullptr, (cudaStream_t)stream);
}

int b200_embed(const float *table, const int32_t *token, float *x, int64_t H,
               void *stream) {
  if (!table || !token || !x || H < 1)
    return fail(B200_EINVAL, "embed: bad argument");
  if (int rc = ensure_device())
    return rc;
  embed_kernel<<<(unsigned)((H + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      table, token, x, H);
  B200_LAUNCH_CHECK();
  return B200_OK;
}

int b200_argmax_first(const float *v, int64_t n, int32_t *out, float *scratch,
                      void *stream) {
  if (!v || !out || !scratch || n < 1 || n > 0x7ffffff0)
    return fail(B200_EINVAL, "argmax_first: bad argument");
  if (int rc = ensure_device())
    return rc;
  int parts = (int)((n + 1023) / 1024);
  if (parts > 1024)
    parts = 1024;
  float *pv = scratch;
  int *pi = (int *)(scratch + 1024);
  argmax_part_kernel<<<parts, 256, 0, (cudaStream_t)stream>>>(v, n, pv, pi);
  B200_LAUNCH_CHECK();
  argmax_final_kernel<<<1, 256, 0, (cudaStream_t)stream>>>(pv, pi, parts, out);
  B200_LAUNCH_CHECK();
  return B200_OK;
}

int b200_kv_overflow(float **kv_dev, int n_buffers, int kv_heads, int max_len,
                     int D, int position, int keep, float theta,
                     int *new_position, void *stream) {
  if (!kv_dev || !new_position || n_buffers < 1 || kv_heads < 1 ||
      max_len < 1 || D < 2 || (D & 1) || D > 2048)
    return fail(B200_EINVAL, "kv_overflow: bad argument");
  // gen_session.py:1471-1506
  if (position < max_len) {
    *new_position = -1;
    return B200_OK;
  }
  if (int rc = ensure_device())
    return rc;
  const int cur = position < max_len ? position : max_len;
  keep = keep < 0 ? 0 : (keep > cur - 1 ? cur - 1 : keep);
  int discard = (cur - keep) / 2;
  if (discard < 1)
    discard = 1;
  const int src = keep + discard;
  cudaStream_t st = (cudaStream_t)stream;
  if (src < cur) {
    const int tail = cur - src, half = D / 2;
    // KVCacheManager.h:124-135 and :247-256, evaluated on the host in float
    // exactly as the reference does, so the rotation is bit-identical.
    std::vector<float> tab(2 * half);
    const float delta = -(float)discard;
    for (int i = 0; i < half; ++i) {
      const float expo = (2.0f * (float)i) / (float)D;
      const float inv = 1.0f / (float)std::pow(theta, expo);
      const float ang = inv * delta;
      tab[i] = std::cos(ang);
      tab[half + i] = std::sin(ang);
    }
    float *d_tab = nullptr, *stage = nullptr;
    const size_t stage_bytes =
        (size_t)n_buffers * kv_heads * tail * D * sizeof(float);
    B200_CUDA(cudaMallocAsync((void **)&d_tab, tab.size() * sizeof(float), st));
    B200_CUDA(cudaMallocAsync((void **)&stage, stage_bytes, st));
    B200_CUDA(cudaMemcpyAsync(d_tab, tab.data(), tab.size() * sizeof(float),
                              cudaMemcpyHostToDevice, st));
    B200_CUDA(cudaStreamSynchronize(st));  // tab is a host temporary
    const int threads = ((half + 31) / 32) * 32;
    kv_tail_stage_kernel<<<dim3(tail, kv_heads, n_buffers), threads, 0, st>>>(
        kv_dev, kv_heads, max_len, D, src, tail, d_tab, d_tab + half, stage);
    B200_LAUNCH_CHECK();
    kv_tail_commit_kernel<<<dim3(max_len - keep, kv_heads, n_buffers), 128, 0,
                            st>>>(kv_dev, kv_heads, max_len, D, keep, tail,
                                  stage);
    B200_LAUNCH_CHECK();
    B200_CUDA(cudaFreeAsync(stage, st));
    B200_CUDA(cudaFreeAsync(d_tab, st));
  }
  int np = cur - discard;
  *new_position = np < 0 ? 0 : (np > max_len ? max_len : np);
  return B200_OK;
}

} // extern "C"

// Prefill (many rows at once): the small ops around the dense GEMMs.
//
// buddy-mlir's prefill graph is the decode graph over all max_len rows with a
// causal mask (tools/buddy-codegen/compile_pipeline.py:207-220); its attention
// is flash_attention_for_cpu_prefill_op (frontend/Python/ops/tosa.py:4326-4700:
// blocks of 16 queries x 64 keys, online softmax seeded (-1e30, 0, 0), f32
// inside).  Here row m sits at position pos0 + m and attends to cache rows
// [0, pos0 + m]: the same recurrence over the same keys (masked keys contribute
// exactly 0 in the reference), with the work laid out for a GPU.
#include "common.cuh"

namespace b200 {

namespace {

constexpr float kSeed = -1.0e30f;

// subgraph0_decode_simplify.mlir:46-49, for M tokens
__global__ void embed_rows_kernel(const float *table, const int32_t *tokens, float *x, int64_t H) {
  const float4 *src = reinterpret_cast<const float4 *>(table + (int64_t)tokens[blockIdx.x] * H);
  float4 *dst = reinterpret_cast<float4 *>(x + (int64_t)blockIdx.x * H);
  for (int i = threadIdx.x; i < H / 4; i += blockDim.x)
    dst[i] = src[i];
}

// RoPE (and QK-norm) on the q and k heads of every row, K/V rows written to the
// cache: subgraph0_decode_simplify.mlir:52-59, 86-142 with pos = pos0 + row.
// grid (M, q_heads + kv_heads), one thread per (j, j + D/2) pair.
__global__ void rope_kv_rows_kernel(float *qkv, int64_t ld, float *k_cache, float *v_cache,
                                    const float *inv_freq, const float *q_norm, const float *k_norm,
                                    float eps, int q_heads, int kv_heads, int D, int max_len, int pos0) {
  __shared__ float red[8];
  const int half = D / 2;
  const int j = threadIdx.x;
  const int m = blockIdx.x, head = blockIdx.y;
  const bool is_q = head < q_heads;
  const int h = is_q ? head : head - q_heads;
  float *row = qkv + (int64_t)m * ld;
  float *p = row + (is_q ? 0 : q_heads * D) + (int64_t)h * D;
  const float *v = row + (q_heads + kv_heads) * D + (int64_t)h * D;
  const float *nw = is_q ? q_norm : k_norm;
  const int pos = pos0 + m;
  float a = 0.f, b = 0.f;
  if (j < half) {
    a = p[j];
    b = p[j + half];
  }
  if (nw != nullptr) {
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
  const float oa = __fadd_rn(__fmul_rn(a, c), __fmul_rn(-b, s));
  const float ob = __fadd_rn(__fmul_rn(b, c), __fmul_rn(a, s));
  p[j] = oa;
  p[j + half] = ob;
  if (!is_q) {
    const int64_t crow = ((int64_t)h * max_len + pos) * D;
    k_cache[crow + j] = oa;
    k_cache[crow + j + half] = ob;
    v_cache[crow + j] = v[j];
    v_cache[crow + j + half] = v[j + half];
  }
}

// Causal attention of M query rows over the cache: grid (M, kv_heads), 4 warps.
// The CTA serves the G query heads that share its kv head (each K/V row is
// loaded once for all of them); a warp owns every 4th key row, lanes own
// D/32 consecutive dims; the four warp states are folded in warp order.
template <int G, int VEC>
__global__ void __launch_bounds__(128)
gqa_prefill_kernel(const float *qkv, int64_t ld, const float *kc, const float *vc, float *out, int64_t ldo,
                   int q_heads, int max_len, int pos0) {
  constexpr int D = VEC * 32, W = 4;
  const int m = blockIdx.x, hk = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int len = min(pos0 + m, max_len - 1) + 1;
  const float scale = rsqrtf((float)D);
  const float *qrow = qkv + (int64_t)m * ld + (int64_t)hk * G * D;
  float qr[G][VEC];
#pragma unroll
  for (int g = 0; g < G; ++g)
#pragma unroll
    for (int e = 0; e < VEC; ++e)
      qr[g][e] = qrow[g * D + lane * VEC + e];
  float mx[G], l[G], acc[G][VEC];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    mx[g] = kSeed;
    l[g] = 0.f;
#pragma unroll
    for (int e = 0; e < VEC; ++e)
      acc[g][e] = 0.f;
  }
  const float *kbase = kc + (int64_t)hk * max_len * D + lane * VEC;
  const float *vbase = vc + (int64_t)hk * max_len * D + lane * VEC;
  for (int j = warp; j < len; j += W) {
    float kr[VEC], vr[VEC];
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
      kr[e] = kbase[(int64_t)j * D + e];
      vr[e] = vbase[(int64_t)j * D + e];
    }
    float s[G];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float d = 0.f;
#pragma unroll
      for (int e = 0; e < VEC; ++e)
        d = fmaf(qr[g][e], kr[e], d);
      s[g] = d;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
#pragma unroll
      for (int g = 0; g < G; ++g)
        s[g] += __shfl_xor_sync(0xffffffffu, s[g], o);
#pragma unroll
    for (int g = 0; g < G; ++g) {
      // tosa.py:14245-14252: new_m = max(m, s); alpha = exp(m - new_m); p = exp(s - new_m)
      s[g] *= scale;
      const float nm = fmaxf(mx[g], s[g]);
      const float alpha = expf(mx[g] - nm);
      const float pw = expf(s[g] - nm);
      l[g] = fmaf(l[g], alpha, pw);
#pragma unroll
      for (int e = 0; e < VEC; ++e)
        acc[g][e] = fmaf(acc[g][e], alpha, pw * vr[e]);
      mx[g] = nm;
    }
  }
  __shared__ float s_m[W][G], s_l[W][G];
  __shared__ float s_acc[W][G][D];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    if (lane == 0) {
      s_m[warp][g] = mx[g];
      s_l[warp][g] = l[g];
    }
#pragma unroll
    for (int e = 0; e < VEC; ++e)
      s_acc[warp][g][lane * VEC + e] = acc[g][e];
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * D; idx += blockDim.x) {
    const int g = idx / D, d = idx - g * D;
    float M = kSeed;
#pragma unroll
    for (int w = 0; w < W; ++w)
      M = fmaxf(M, s_m[w][g]);
    float L = 0.f, A = 0.f;
#pragma unroll
    for (int w = 0; w < W; ++w) {
      const float b = expf(s_m[w][g] - M);
      L = fmaf(s_l[w][g], b, L);
      A = fmaf(s_acc[w][g][d], b, A);
    }
    out[(int64_t)m * ldo + (int64_t)(hk * G + g) * D + d] = __fdiv_rn(A, L);
  }
}

template <int G>
int launch_prefill_attn(const float *qkv, int64_t ld, const float *kc, const float *vc, float *out, int64_t ldo,
                        int q_heads, int kv_heads, int D, int max_len, int pos0, int M, cudaStream_t st) {
  dim3 grid(M, kv_heads);
  if (D == 128)
    gqa_prefill_kernel<G, 4><<<grid, 128, 0, st>>>(qkv, ld, kc, vc, out, ldo, q_heads, max_len, pos0);
  else
    gqa_prefill_kernel<G, 2><<<grid, 128, 0, st>>>(qkv, ld, kc, vc, out, ldo, q_heads, max_len, pos0);
  B200_LAUNCH_CHECK();
  return B200_OK;
}

// ---- paged cache: rows of many sequences, K/V in fixed-size pages -------------------
// Page pool of one cache buffer: [n_pages][kv_heads][page][D] f32.  Row r of the batch
// belongs to sequence row_seq[r] at position row_pos[r]; block_table[seq][pos / page] is
// the page that holds the position.  (buddy-mlir has no paged cache; per sequence the
// arithmetic is that of the contiguous cache above.)
__global__ void rope_kv_paged_kernel(float *qkv, int64_t ld, float *k_pool, float *v_pool,
                                     const float *inv_freq, const float *q_norm, const float *k_norm, float eps,
                                     int q_heads, int kv_heads, int D, int page, const int32_t *row_seq,
                                     const int32_t *row_pos, const int32_t *block_table, int table_stride) {
  __shared__ float red[8];
  const int half = D / 2;
  const int j = threadIdx.x;
  const int m = blockIdx.x, head = blockIdx.y;
  const bool is_q = head < q_heads;
  const int h = is_q ? head : head - q_heads;
  float *row = qkv + (int64_t)m * ld;
  float *p = row + (is_q ? 0 : q_heads * D) + (int64_t)h * D;
  const float *v = row + (q_heads + kv_heads) * D + (int64_t)h * D;
  const float *nw = is_q ? q_norm : k_norm;
  const int pos = row_pos[m];
  float a = 0.f, b = 0.f;
  if (j < half) {
    a = p[j];
    b = p[j + half];
  }
  if (nw != nullptr) {
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
  const float oa = __fadd_rn(__fmul_rn(a, c), __fmul_rn(-b, s));
  const float ob = __fadd_rn(__fmul_rn(b, c), __fmul_rn(a, s));
  p[j] = oa;
  p[j + half] = ob;
  if (!is_q) {
    const int pg = block_table[(int64_t)row_seq[m] * table_stride + pos / page];
    const int64_t crow = (((int64_t)pg * kv_heads + h) * page + pos % page) * D;
    k_pool[crow + j] = oa;
    k_pool[crow + j + half] = ob;
    v_pool[crow + j] = v[j];
    v_pool[crow + j + half] = v[j + half];
  }
}

template <int G, int VEC>
__global__ void __launch_bounds__(128)
gqa_paged_kernel(const float *qkv, int64_t ld, const float *k_pool, const float *v_pool, float *out, int64_t ldo,
                 int kv_heads, int page, const int32_t *row_seq, const int32_t *row_pos, const int32_t *block_table,
                 int table_stride) {
  constexpr int D = VEC * 32, W = 4;
  const int m = blockIdx.x, hk = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int len = row_pos[m] + 1;
  const int32_t *table = block_table + (int64_t)row_seq[m] * table_stride;
  const float scale = rsqrtf((float)D);
  const float *qrow = qkv + (int64_t)m * ld + (int64_t)hk * G * D;
  float qr[G][VEC];
#pragma unroll
  for (int g = 0; g < G; ++g)
#pragma unroll
    for (int e = 0; e < VEC; ++e)
      qr[g][e] = qrow[g * D + lane * VEC + e];
  float mx[G], l[G], acc[G][VEC];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    mx[g] = kSeed;
    l[g] = 0.f;
#pragma unroll
    for (int e = 0; e < VEC; ++e)
      acc[g][e] = 0.f;
  }
  for (int j = warp; j < len; j += W) {
    const int pg = table[j / page];
    const int64_t crow = (((int64_t)pg * kv_heads + hk) * page + j % page) * D + lane * VEC;
    float kr[VEC], vr[VEC];
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
      kr[e] = k_pool[crow + e];
      vr[e] = v_pool[crow + e];
    }
    float s[G];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float d = 0.f;
#pragma unroll
      for (int e = 0; e < VEC; ++e)
        d = fmaf(qr[g][e], kr[e], d);
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
      const float nm = fmaxf(mx[g], s[g]);
      const float alpha = expf(mx[g] - nm);
      const float pw = expf(s[g] - nm);
      l[g] = fmaf(l[g], alpha, pw);
#pragma unroll
      for (int e = 0; e < VEC; ++e)
        acc[g][e] = fmaf(acc[g][e], alpha, pw * vr[e]);
      mx[g] = nm;
    }
  }
  __shared__ float s_m[W][G], s_l[W][G];
  __shared__ float s_acc[W][G][D];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    if (lane == 0) {
      s_m[warp][g] = mx[g];
      s_l[warp][g] = l[g];
    }
#pragma unroll
    for (int e = 0; e < VEC; ++e)
      s_acc[warp][g][lane * VEC + e] = acc[g][e];
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * D; idx += blockDim.x) {
    const int g = idx / D, d = idx - g * D;
    float M = kSeed;
#pragma unroll
    for (int w = 0; w < W; ++w)
      M = fmaxf(M, s_m[w][g]);
    float L = 0.f, A = 0.f;
#pragma unroll
    for (int w = 0; w < W; ++w) {
      const float b = expf(s_m[w][g] - M);
      L = fmaf(s_l[w][g], b, L);
      A = fmaf(s_acc[w][g][d], b, A);
    }
    out[(int64_t)m * ldo + (int64_t)(hk * G + g) * D + d] = __fdiv_rn(A, L);
  }
}

template <int G>
int launch_paged_attn(const float *qkv, int64_t ld, const float *kp, const float *vp, float *out, int64_t ldo,
                      int kv_heads, int D, int page, const int32_t *row_seq, const int32_t *row_pos,
                      const int32_t *block_table, int table_stride, int M, cudaStream_t st) {
  dim3 grid(M, kv_heads);
  if (D == 128)
    gqa_paged_kernel<G, 4><<<grid, 128, 0, st>>>(qkv, ld, kp, vp, out, ldo, kv_heads, page, row_seq, row_pos,
                                                 block_table, table_stride);
  else
    gqa_paged_kernel<G, 2><<<grid, 128, 0, st>>>(qkv, ld, kp, vp, out, ldo, kv_heads, page, row_seq, row_pos,
                                                 block_table, table_stride);
  B200_LAUNCH_CHECK();
  return B200_OK;
}

// The same scan for few rows with long histories (batched decode): the keys of a row
// are cut into chunks of kPagedChunk positions, one CTA of 8 warps per (row, kv head,
// chunk); a warp owns every 8th key of the chunk and keeps four K/V rows in flight.
// Partials (m, l, acc[D]) per query head go to `part`; gqa_paged_combine_kernel folds
// the chunks of a row in chunk order.
constexpr int kPagedChunk = 256;
template <int G, int VEC>
__global__ void __launch_bounds__(256)
gqa_paged_split_kernel(const float *qkv, int64_t ld, const float *k_pool, const float *v_pool, float *part,
                       int kv_heads, int page, const int32_t *row_seq, const int32_t *row_pos,
                       const int32_t *block_table, int table_stride) {
  constexpr int D = VEC * 32, W = 8, U = 4;
  const int m = blockIdx.x, hk = blockIdx.y, sp = blockIdx.z;
  const int len = row_pos[m] + 1;
  const int j0 = sp * kPagedChunk;
  if (j0 >= len)
    return;
  const int j1 = min(len, j0 + kPagedChunk);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int32_t *table = block_table + (int64_t)row_seq[m] * table_stride;
  const float scale = rsqrtf((float)D);
  const float *qrow = qkv + (int64_t)m * ld + (int64_t)hk * G * D;
  float qr[G][VEC];
#pragma unroll
  for (int g = 0; g < G; ++g)
#pragma unroll
    for (int e = 0; e < VEC; ++e)
      qr[g][e] = qrow[g * D + lane * VEC + e];
  float mx[G], l[G], acc[G][VEC];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    mx[g] = kSeed;
    l[g] = 0.f;
#pragma unroll
    for (int e = 0; e < VEC; ++e)
      acc[g][e] = 0.f;
  }
  for (int jb = j0 + warp; jb < j1; jb += W * U) {
    float kr[U][VEC], vr[U][VEC];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int j = jb + u * W;
      if (j < j1) {
        const int pg = table[j / page];
        const int64_t crow = (((int64_t)pg * kv_heads + hk) * page + j % page) * D + lane * VEC;
        if (VEC == 4) {
          const float4 a = *reinterpret_cast<const float4 *>(k_pool + crow);
          const float4 b = *reinterpret_cast<const float4 *>(v_pool + crow);
          kr[u][0] = a.x; kr[u][1] = a.y; kr[u][2 % VEC] = a.z; kr[u][3 % VEC] = a.w;
          vr[u][0] = b.x; vr[u][1] = b.y; vr[u][2 % VEC] = b.z; vr[u][3 % VEC] = b.w;
        } else {
#pragma unroll
          for (int e = 0; e < VEC; ++e) {
            kr[u][e] = k_pool[crow + e];
            vr[u][e] = v_pool[crow + e];
          }
        }
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (jb + u * W >= j1)
        break;
      float s[G];
#pragma unroll
      for (int g = 0; g < G; ++g) {
        float d = 0.f;
#pragma unroll
        for (int e = 0; e < VEC; ++e)
          d = fmaf(qr[g][e], kr[u][e], d);
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
        const float nm = fmaxf(mx[g], s[g]);
        const float alpha = expf(mx[g] - nm);
        const float pw = expf(s[g] - nm);
        l[g] = fmaf(l[g], alpha, pw);
#pragma unroll
        for (int e = 0; e < VEC; ++e)
          acc[g][e] = fmaf(acc[g][e], alpha, pw * vr[u][e]);
        mx[g] = nm;
      }
    }
  }
  __shared__ float s_m[W][G], s_l[W][G];
  __shared__ float s_acc[W][G][D];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    if (lane == 0) {
      s_m[warp][g] = mx[g];
      s_l[warp][g] = l[g];
    }
#pragma unroll
    for (int e = 0; e < VEC; ++e)
      s_acc[warp][g][lane * VEC + e] = acc[g][e];
  }
  __syncthreads();
  float *pout = part + (((int64_t)m * kv_heads + hk) * gridDim.z + sp) * G * (D + 2);
  for (int idx = threadIdx.x; idx < G * D; idx += blockDim.x) {
    const int g = idx / D, d = idx - g * D;
    float M = kSeed;
#pragma unroll
    for (int w = 0; w < W; ++w)
      M = fmaxf(M, s_m[w][g]);
    float L = 0.f, A = 0.f;
#pragma unroll
    for (int w = 0; w < W; ++w) {
      const float b = expf(s_m[w][g] - M);   // a warp that saw no key: l = 0, acc = 0
      L = fmaf(s_l[w][g], b, L);
      A = fmaf(s_acc[w][g][d], b, A);
    }
    pout[g * (D + 2) + 2 + d] = A;
    if (d == 0) {
      pout[g * (D + 2)] = M;
      pout[g * (D + 2) + 1] = L;
    }
  }
}

template <int G, int D>
__global__ void __launch_bounds__(128)
gqa_paged_combine_kernel(const float *part, float *out, int64_t ldo, int kv_heads, int chunks,
                         const int32_t *row_pos) {
  const int m = blockIdx.x, hk = blockIdx.y;
  const int n = (row_pos[m] + kPagedChunk) / kPagedChunk;   // chunks that hold keys of this row
  const float *pin = part + (((int64_t)m * kv_heads + hk) * chunks) * G * (D + 2);
  for (int idx = threadIdx.x; idx < G * D; idx += blockDim.x) {
    const int g = idx / D, d = idx - g * D;
    float M = kSeed;
    for (int c = 0; c < n; ++c)
      M = fmaxf(M, pin[(int64_t)(c * G + g) * (D + 2)]);
    float L = 0.f, A = 0.f;
    for (int c = 0; c < n; ++c) {
      const float *q = pin + (int64_t)(c * G + g) * (D + 2);
      const float b = expf(q[0] - M);
      L = fmaf(q[1], b, L);
      A = fmaf(q[2 + d], b, A);
    }
    out[(int64_t)m * ldo + (int64_t)(hk * G + g) * D + d] = __fdiv_rn(A, L);
  }
}

template <int G>
int launch_paged_split(const float *qkv, int64_t ld, const float *kp, const float *vp, float *out, int64_t ldo,
                       int kv_heads, int D, int page, const int32_t *row_seq, const int32_t *row_pos,
                       const int32_t *block_table, int table_stride, int M, float *part, int chunks,
                       cudaStream_t st) {
  dim3 grid(M, kv_heads, chunks), cgrid(M, kv_heads);
  if (D == 128) {
    gqa_paged_split_kernel<G, 4><<<grid, 256, 0, st>>>(qkv, ld, kp, vp, part, kv_heads, page, row_seq, row_pos,
                                                       block_table, table_stride);
    B200_LAUNCH_CHECK();
    gqa_paged_combine_kernel<G, 128><<<cgrid, 128, 0, st>>>(part, out, ldo, kv_heads, chunks, row_pos);
  } else {
    gqa_paged_split_kernel<G, 2><<<grid, 256, 0, st>>>(qkv, ld, kp, vp, part, kv_heads, page, row_seq, row_pos,
                                                       block_table, table_stride);
    B200_LAUNCH_CHECK();
    gqa_paged_combine_kernel<G, 64><<<cgrid, 128, 0, st>>>(part, out, ldo, kv_heads, chunks, row_pos);
  }
  B200_LAUNCH_CHECK();
  return B200_OK;
}

// one first-maximum per row of a [rows, n] matrix (Sampler.h:101-104)
__global__ void argmax_rows_kernel(const float *v, int64_t n, int32_t *out) {
  const float *row = v + (int64_t)blockIdx.x * n;
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  for (int64_t i = threadIdx.x; i < n; i += blockDim.x) {
    const float x = row[i];
    if (x > bv || (x == bv && (int)i < bi)) {
      bv = x;
      bi = (int)i;
    }
  }
  __shared__ float sv[32];
  __shared__ int si[32];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > bv || (ov == bv && oi < bi)) {
      bv = ov;
      bi = oi;
    }
  }
  if ((threadIdx.x & 31) == 0) {
    sv[threadIdx.x >> 5] = bv;
    si[threadIdx.x >> 5] = bi;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w)
      if (sv[w] > bv || (sv[w] == bv && si[w] < bi)) {
        bv = sv[w];
        bi = si[w];
      }
    out[blockIdx.x] = bi == 0x7fffffff ? 0 : bi;
  }
}

} // namespace

int rope_kv_paged_launch(float *qkv, int64_t ld, float *k_pool, float *v_pool, const float *inv_freq,
                         const float *q_norm, const float *k_norm, float eps, int q_heads, int kv_heads, int D,
                         int page, const int32_t *row_seq, const int32_t *row_pos, const int32_t *block_table,
                         int table_stride, int M, cudaStream_t st) {
  dim3 grid(M, q_heads + kv_heads);
  rope_kv_paged_kernel<<<grid, D / 2 < 32 ? 32 : D / 2, 0, st>>>(qkv, ld, k_pool, v_pool, inv_freq, q_norm, k_norm, eps,
                                                               q_heads, kv_heads, D, page, row_seq, row_pos,
                                                               block_table, table_stride);
  B200_LAUNCH_CHECK();
  return B200_OK;
}

int64_t gqa_paged_scratch_floats(int rows, int q_heads, int D, int max_context) {
  const int chunks = (max_context + kPagedChunk - 1) / kPagedChunk;
  return (int64_t)rows * chunks * q_heads * (D + 2);
}

// scratch: gqa_paged_scratch_floats(M, ..) floats, or null (then, and for more than
// kPagedSplitRows rows, every row is scanned by one CTA)
int gqa_paged_launch(const float *qkv, int64_t ld, const float *k_pool, const float *v_pool, float *out, int64_t ldo,
                     int q_heads, int kv_heads, int D, int page, const int32_t *row_seq, const int32_t *row_pos,
                     const int32_t *block_table, int table_stride, int M, float *scratch, int max_context,
                     cudaStream_t st) {
  if (D != 64 && D != 128)
    return fail(B200_EINVAL, "gqa_paged: head_dim %d (64 or 128 supported)", D);
  constexpr int kPagedSplitRows = 256;
  const bool split = scratch != nullptr && M <= kPagedSplitRows && max_context > kPagedChunk;
  const int chunks = (max_context + kPagedChunk - 1) / kPagedChunk;
  switch (q_heads / kv_heads) {
#define B200_G(G_)                                                                                          \
  case G_:                                                                                                  \
    if (split)                                                                                              \
      return launch_paged_split<G_>(qkv, ld, k_pool, v_pool, out, ldo, kv_heads, D, page, row_seq, row_pos, \
                                    block_table, table_stride, M, scratch, chunks, st);                     \
    return launch_paged_attn<G_>(qkv, ld, k_pool, v_pool, out, ldo, kv_heads, D, page, row_seq, row_pos,    \
                                 block_table, table_stride, M, st);
    B200_G(1) B200_G(2) B200_G(3) B200_G(4) B200_G(6) B200_G(8)
#undef B200_G
  default:
    return fail(B200_EINVAL, "gqa_paged: group size %d not built", q_heads / kv_heads);
  }
}

int argmax_rows_launch(const float *v, int64_t n, int rows, int32_t *out, cudaStream_t st) {
  argmax_rows_kernel<<<rows, 256, 0, st>>>(v, n, out);
  B200_LAUNCH_CHECK();
  return B200_OK;
}

int embed_rows_launch(const float *table, const int32_t *tokens_dev, float *x, int64_t H, int M, cudaStream_t st) {
  if (H % 4 != 0)
    return fail(B200_EINVAL, "embed_rows: hidden size must be a multiple of 4");
  embed_rows_kernel<<<M, 128, 0, st>>>(table, tokens_dev, x, H);
  B200_LAUNCH_CHECK();
  return B200_OK;
}

int rope_kv_rows_launch(float *qkv, int64_t ld, float *k_cache, float *v_cache, const float *inv_freq,
                        const float *q_norm, const float *k_norm, float eps, int q_heads, int kv_heads, int D,
                        int max_len, int pos0, int M, cudaStream_t st) {
  dim3 grid(M, q_heads + kv_heads);
  rope_kv_rows_kernel<<<grid, D / 2 < 32 ? 32 : D / 2, 0, st>>>(qkv, ld, k_cache, v_cache, inv_freq, q_norm, k_norm,
                                                              eps, q_heads, kv_heads, D, max_len, pos0);
  B200_LAUNCH_CHECK();
  return B200_OK;
}

int gqa_prefill_launch(const float *qkv, int64_t ld, const float *kc, const float *vc, float *out, int64_t ldo,
                       int q_heads, int kv_heads, int D, int max_len, int pos0, int M, cudaStream_t st) {
  if (D != 64 && D != 128)
    return fail(B200_EINVAL, "gqa_prefill: head_dim %d (64 or 128 supported)", D);
  switch (q_heads / kv_heads) {
#define B200_G(G_)                                                                                      \
  case G_:                                                                                              \
    return launch_prefill_attn<G_>(qkv, ld, kc, vc, out, ldo, q_heads, kv_heads, D, max_len, pos0, M, st);
    B200_G(1) B200_G(2) B200_G(3) B200_G(4) B200_G(6) B200_G(8)
#undef B200_G
  default:
    return fail(B200_EINVAL, "gqa_prefill: group size %d not built", q_heads / kv_heads);
  }
}

} // namespace b200

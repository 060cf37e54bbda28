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

// Causal attention tiled over query rows (flash style, f32 on the CUDA cores).
// A CTA takes BQ consecutive query rows of one kv head: R = BQ * G query vectors
// (row r = query row r / G, head hk * G + r % G) against tiles of 64 keys staged in
// shared memory, so a K/V row is read once per BQ query rows instead of once per
// row.  512 threads as 32 x 16: thread (ty, tx) owns query vectors 4ty..4ty+3; for
// the scores it owns keys tx, tx + 16, tx + 32, tx + 48 of the tile (rows of the K
// tile 16 apart: no bank conflicts), for the output the float4 column
// chunks tx + 16i.  Per key tile: S = Q K^T (register tile 4 x 4 over D), running
// max / sum per row across the 16 threads of a row (tosa.py:14245-14252, one update
// per tile instead of per key), P to shared memory, O += P V (register tile
// 4 x D/16).  The next K/V tile is fetched into registers while the current one
// is used.
template <int G, int D>
struct PrefillTile {
  static constexpr int BQ = G >= 6 ? 16 : (G >= 3 ? 32 : 64);
  static constexpr int R = BQ * G;           // <= 128
  static constexpr int KT = 64;              // keys per tile
  static constexpr int LDQ = D + 4, LDK = D + 4, LDP = KT + 4;
  static constexpr size_t smem_bytes = ((size_t)R * LDQ + (size_t)KT * LDK + (size_t)KT * D + (size_t)R * LDP) * 4;
};

// PAGED: kc / vc are page pools [n_pages][kv_heads][page][D] and `table` lists the
// pages of the one sequence all M rows belong to (positions pos0, pos0 + 1, ..).
template <int G, int D, bool PAGED>
__global__ void __launch_bounds__(512, 1)
gqa_prefill_tiled_kernel(const float *qkv, int64_t ld, const float *kc, const float *vc, float *out, int64_t ldo,
                         int max_len, int pos0, int M, const int32_t *table, int page, int kv_heads) {
  using T = PrefillTile<G, D>;
  constexpr int R = T::R, KT = T::KT, LDQ = T::LDQ, LDK = T::LDK, LDP = T::LDP, NCH = D / 64;
  extern __shared__ __align__(16) float sm[];
  float *Qs = sm, *Ks = Qs + R * LDQ, *Vs = Ks + KT * LDK, *Ps = Vs + KT * D;
  // heavy tiles (late rows, long histories) first
  const int qt = gridDim.x - 1 - blockIdx.x, hk = blockIdx.y;
  const int m0 = qt * T::BQ;
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const bool row_thread = 4 * ty < R;
  const float scale = rsqrtf((float)D);
  // keys this tile needs: up to the position of its last live row
  const int last_m = min(m0 + T::BQ, M) - 1;
  const int n_keys = min(pos0 + last_m, max_len - 1) + 1;
  const float *kbase = PAGED ? kc : kc + (int64_t)hk * max_len * D;
  const float *vbase = PAGED ? vc : vc + (int64_t)hk * max_len * D;

  // ---- stage Q: row r = (query row r / G, head r % G), G heads of a row are contiguous ----
  for (int idx = tid; idx < R * (D / 4); idx += 512) {
    const int r = idx / (D / 4), c = idx - r * (D / 4);
    const int m = m0 + r / G;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (m < M)
      v = *reinterpret_cast<const float4 *>(qkv + (int64_t)m * ld + (int64_t)(hk * G + r % G) * D + 4 * c);
    *reinterpret_cast<float4 *>(Qs + r * LDQ + 4 * c) = v;
  }
  // per-thread K/V fetch slots: KT * D / 4 float4 per tile over 512 threads
  constexpr int NF = KT * (D / 4) / 512;   // 4 (D = 128) or 2 (D = 64)
  float4 kf[NF], vf[NF];
  auto fetch = [&](int k0) {
#pragma unroll
    for (int i = 0; i < NF; ++i) {
      const int idx = tid + 512 * i;
      const int j = idx / (D / 4), c = idx - j * (D / 4);
      if (k0 + j < n_keys) {
        const int key = k0 + j;
        const int64_t roff = PAGED ? (((int64_t)table[key / page] * kv_heads + hk) * page + key % page) * D
                                   : (int64_t)key * D;
        kf[i] = __ldg(reinterpret_cast<const float4 *>(kbase + roff + 4 * c));
        vf[i] = __ldg(reinterpret_cast<const float4 *>(vbase + roff + 4 * c));
      } else {
        kf[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        vf[i] = kf[i];
      }
    }
  };
  auto stash = [&]() {
#pragma unroll
    for (int i = 0; i < NF; ++i) {
      const int idx = tid + 512 * i;
      const int j = idx / (D / 4), c = idx - j * (D / 4);
      *reinterpret_cast<float4 *>(Ks + j * LDK + 4 * c) = kf[i];
      *reinterpret_cast<float4 *>(Vs + j * D + 4 * c) = vf[i];
    }
  };

  float mrow[4], lrow[4], acc[4][NCH * 4];
  int qpos[4];
#pragma unroll
  for (int a = 0; a < 4; ++a) {
    mrow[a] = kSeed;
    lrow[a] = 0.f;
    const int m = m0 + (4 * ty + a) / G;
    qpos[a] = (row_thread && m < M) ? min(pos0 + m, max_len - 1) : -1;   // -1: every key is masked
#pragma unroll
    for (int c = 0; c < NCH * 4; ++c)
      acc[a][c] = 0.f;
  }

  fetch(0);
  for (int k0 = 0; k0 < n_keys; k0 += KT) {
    __syncthreads();            // the previous tile is no longer read (and Q is staged)
    stash();
    __syncthreads();
    if (k0 + KT < n_keys)
      fetch(k0 + KT);
    if (row_thread) {
      // ---- S = Q K^T for rows 4ty.., keys tx + 16b ------------------------------------
      float sc[4][4];
#pragma unroll
      for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b)
          sc[a][b] = 0.f;
      const float *qp = Qs + (4 * ty) * LDQ, *kp = Ks + tx * LDK;
#pragma unroll 4
      for (int d = 0; d < D; d += 4) {
        float4 q4[4], k4[4];
#pragma unroll
        for (int a = 0; a < 4; ++a)
          q4[a] = *reinterpret_cast<const float4 *>(qp + a * LDQ + d);
#pragma unroll
        for (int b = 0; b < 4; ++b)
          k4[b] = *reinterpret_cast<const float4 *>(kp + b * 16 * LDK + d);
#pragma unroll
        for (int a = 0; a < 4; ++a)
#pragma unroll
          for (int b = 0; b < 4; ++b) {
            sc[a][b] = fmaf(q4[a].x, k4[b].x, sc[a][b]);
            sc[a][b] = fmaf(q4[a].y, k4[b].y, sc[a][b]);
            sc[a][b] = fmaf(q4[a].z, k4[b].z, sc[a][b]);
            sc[a][b] = fmaf(q4[a].w, k4[b].w, sc[a][b]);
          }
      }
      // ---- running softmax per row: the 16 threads tx = 0..15 of a row hold its 64 scores ----
#pragma unroll
      for (int a = 0; a < 4; ++a) {
        float tm = kSeed;
#pragma unroll
        for (int b = 0; b < 4; ++b) {
          const int key = k0 + 16 * b + tx;
          sc[a][b] = key <= qpos[a] ? sc[a][b] * scale : kSeed;
          tm = fmaxf(tm, sc[a][b]);
        }
        tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, 1));
        tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, 2));
        tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, 4));
        tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, 8));
        const float nm = fmaxf(mrow[a], tm);
        const float alpha = expf(mrow[a] - nm);
        float ps = 0.f;
        float pw[4];
#pragma unroll
        for (int b = 0; b < 4; ++b) {
          const int key = k0 + 16 * b + tx;
          pw[b] = key <= qpos[a] ? expf(sc[a][b] - nm) : 0.f;
          ps += pw[b];
        }
        ps += __shfl_xor_sync(0xffffffffu, ps, 1);
        ps += __shfl_xor_sync(0xffffffffu, ps, 2);
        ps += __shfl_xor_sync(0xffffffffu, ps, 4);
        ps += __shfl_xor_sync(0xffffffffu, ps, 8);
        lrow[a] = fmaf(lrow[a], alpha, ps);
        mrow[a] = nm;
#pragma unroll
        for (int c = 0; c < NCH * 4; ++c)
          acc[a][c] *= alpha;
#pragma unroll
        for (int b = 0; b < 4; ++b)
          Ps[(4 * ty + a) * LDP + 16 * b + tx] = pw[b];
      }
    }
    // the 16 threads of a row sit in one warp: P of a row is complete after a warp sync
    __syncwarp();
    if (row_thread) {
      // ---- O += P V for rows 4ty.., column chunks tx + 16i ----------------------------
      const float *pp = Ps + (4 * ty) * LDP;
#pragma unroll 2
      for (int j = 0; j < KT; j += 4) {
        float4 p4[4];
#pragma unroll
        for (int a = 0; a < 4; ++a)
          p4[a] = *reinterpret_cast<const float4 *>(pp + a * LDP + j);
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
#pragma unroll
          for (int i = 0; i < NCH; ++i) {
            const float4 v4 = *reinterpret_cast<const float4 *>(Vs + (j + jj) * D + 4 * (tx + 16 * i));
#pragma unroll
            for (int a = 0; a < 4; ++a) {
              const float pv = jj == 0 ? p4[a].x : jj == 1 ? p4[a].y : jj == 2 ? p4[a].z : p4[a].w;
              acc[a][4 * i + 0] = fmaf(pv, v4.x, acc[a][4 * i + 0]);
              acc[a][4 * i + 1] = fmaf(pv, v4.y, acc[a][4 * i + 1]);
              acc[a][4 * i + 2] = fmaf(pv, v4.z, acc[a][4 * i + 2]);
              acc[a][4 * i + 3] = fmaf(pv, v4.w, acc[a][4 * i + 3]);
            }
          }
        }
      }
    }
  }
  if (row_thread) {
#pragma unroll
    for (int a = 0; a < 4; ++a) {
      const int r = 4 * ty + a;
      const int m = m0 + r / G;
      if (m < M) {
        float *orow = out + (int64_t)m * ldo + (int64_t)(hk * G + r % G) * D;
#pragma unroll
        for (int i = 0; i < NCH; ++i)
          *reinterpret_cast<float4 *>(orow + 4 * (tx + 16 * i)) =
              make_float4(__fdiv_rn(acc[a][4 * i], lrow[a]), __fdiv_rn(acc[a][4 * i + 1], lrow[a]),
                          __fdiv_rn(acc[a][4 * i + 2], lrow[a]), __fdiv_rn(acc[a][4 * i + 3], lrow[a]));
      }
    }
  }
}

template <int G, int D, bool PAGED>
int launch_prefill_tiled(const float *qkv, int64_t ld, const float *kc, const float *vc, float *out, int64_t ldo,
                         int kv_heads, int max_len, int pos0, int M, const int32_t *table, int page,
                         cudaStream_t st) {
  using T = PrefillTile<G, D>;
  static bool configured[64] = {};
  int dev = 0;
  B200_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    B200_CUDA(cudaFuncSetAttribute(gqa_prefill_tiled_kernel<G, D, PAGED>,
                                   cudaFuncAttributeMaxDynamicSharedMemorySize, (int)T::smem_bytes));
    if (dev >= 0 && dev < 64)
      configured[dev] = true;
  }
  dim3 grid((M + T::BQ - 1) / T::BQ, kv_heads);
  gqa_prefill_tiled_kernel<G, D, PAGED><<<grid, 512, T::smem_bytes, st>>>(qkv, ld, kc, vc, out, ldo, max_len, pos0,
                                                                         M, table, page, kv_heads);
  B200_LAUNCH_CHECK();
  return B200_OK;
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
// are cut into chunks of `chunk` positions (paged_chunk(): an eighth of the longest
// context, 32..256), one CTA of 8 warps per (row, kv head, chunk); a warp owns every 8th key of the chunk and keeps four K/V rows in flight.
// Partials (m, l, acc[D]) per query head go to `part`; the CTA that finishes a row's last
// chunk folds them in chunk order.
__host__ __device__ inline int paged_chunk(int max_context) {
  const int c = ((max_context + 7) / 8 + 31) / 32 * 32;
  return c < 32 ? 32 : (c > 256 ? 256 : c);
}
template <int G, int VEC>
__global__ void __launch_bounds__(256)
gqa_paged_split_kernel(const float *qkv, int64_t ld, const float *k_pool, const float *v_pool, float *part,
                       int kv_heads, int page, const int32_t *row_seq, const int32_t *row_pos,
                       const int32_t *block_table, int table_stride, int chunk, int *counters, float *out,
                       int64_t ldo) {
  constexpr int D = VEC * 32, W = 8;
  const int m = blockIdx.x, hk = blockIdx.y, sp = blockIdx.z;
  const int len = row_pos[m] + 1;
  const int j0 = sp * chunk;
  if (j0 >= len)
    return;
  const int j1 = min(len, j0 + chunk);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int32_t *table = block_table + (int64_t)row_seq[m] * table_stride;
  const float scale = rsqrtf((float)D);
  // the G query vectors of this kv head, shared by every lane (broadcast reads)
  __shared__ __align__(16) float s_q[G][D];
  const float *qrow = qkv + (int64_t)m * ld + (int64_t)hk * G * D;
  for (int i = threadIdx.x; i < G * D; i += blockDim.x)
    s_q[i / D][i % D] = qrow[i];
  __syncthreads();
  float mx[G], l[G], acc[G][VEC];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    mx[g] = kSeed;
    l[g] = 0.f;
#pragma unroll
    for (int e = 0; e < VEC; ++e)
      acc[g][e] = 0.f;
  }
  // A warp takes 32 keys at a time.  Scores: a lane owns one key and walks its K row (no
  // cross-lane reduction per key); softmax over the 32 keys with two warp reductions per query
  // head; values: a lane owns VEC dims, the 32 weights of a head arrive by shuffle.
  for (int jb = j0 + warp * 32; jb < j1; jb += W * 32) {
    const int j = jb + lane;
    const bool live = j < j1;
    int ridx = 0;     // row of the key inside the pool, in rows of D floats
    if (live)
      ridx = (table[j / page] * kv_heads + hk) * page + j % page;
    const float *kp = k_pool + (int64_t)ridx * D;
    float sc[G];
#pragma unroll
    for (int g = 0; g < G; ++g)
      sc[g] = 0.f;
    if (live) {
#pragma unroll 4
      for (int d = 0; d < D; d += 4) {
        const float4 k4 = *reinterpret_cast<const float4 *>(kp + d);
#pragma unroll
        for (int g = 0; g < G; ++g) {
          const float4 q4 = *reinterpret_cast<const float4 *>(&s_q[g][d]);
          sc[g] = fmaf(q4.x, k4.x, sc[g]);
          sc[g] = fmaf(q4.y, k4.y, sc[g]);
          sc[g] = fmaf(q4.z, k4.z, sc[g]);
          sc[g] = fmaf(q4.w, k4.w, sc[g]);
        }
      }
    }
    float pw[G];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const float sv = live ? sc[g] * scale : kSeed;
      const float nm = fmaxf(mx[g], warp_max(sv));
      // fast exponentials (2^-21 relative): the scan is bound by instruction issue
      const float alpha = __expf(mx[g] - nm);
      pw[g] = live ? __expf(sv - nm) : 0.f;
      l[g] = fmaf(l[g], alpha, warp_sum(pw[g]));
      mx[g] = nm;
#pragma unroll
      for (int e = 0; e < VEC; ++e)
        acc[g][e] *= alpha;
    }
    const int nk = min(32, j1 - jb);
    for (int t = 0; t < nk; ++t) {
      const int rt = __shfl_sync(0xffffffffu, ridx, t);
      const float *vp = v_pool + (int64_t)rt * D + lane * VEC;
      float vr[VEC];
      if (VEC == 4) {
        const float4 b = *reinterpret_cast<const float4 *>(vp);
        vr[0] = b.x; vr[1] = b.y; vr[2 % VEC] = b.z; vr[3 % VEC] = b.w;
      } else {
#pragma unroll
        for (int e = 0; e < VEC; ++e)
          vr[e] = vp[e];
      }
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const float pt = __shfl_sync(0xffffffffu, pw[g], t);
#pragma unroll
        for (int e = 0; e < VEC; ++e)
          acc[g][e] = fmaf(pt, vr[e], acc[g][e]);
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
  // The CTA that finishes a row's last chunk folds the chunks in chunk order (the counter
  // returns to zero for the next launch).
  const int n = (len + chunk - 1) / chunk;     // chunks that hold keys of this row
  __shared__ int s_last;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    int *cnt = counters + m * kv_heads + hk;
    const int prev = atomicAdd(cnt, 1);
    s_last = prev == n - 1;
    if (s_last)
      *cnt = 0;
  }
  __syncthreads();
  if (!s_last)
    return;
  __threadfence();
  const float *pin = part + (((int64_t)m * kv_heads + hk) * gridDim.z) * G * (D + 2);
  for (int idx = threadIdx.x; idx < G * D; idx += blockDim.x) {
    const int g = idx / D, d = idx - g * D;
    float M = kSeed;
    for (int c = 0; c < n; ++c)
      M = fmaxf(M, __ldcg(pin + (int64_t)(c * G + g) * (D + 2)));
    float L = 0.f, A = 0.f;
    for (int c = 0; c < n; ++c) {
      const float *q = pin + (int64_t)(c * G + g) * (D + 2);
      const float b = expf(__ldcg(q) - M);
      L = fmaf(__ldcg(q + 1), b, L);
      A = fmaf(__ldcg(q + 2 + d), b, A);
    }
    out[(int64_t)m * ldo + (int64_t)(hk * G + g) * D + d] = __fdiv_rn(A, L);
  }
}

template <int G>
int launch_paged_split(const float *qkv, int64_t ld, const float *kp, const float *vp, float *out, int64_t ldo,
                       int kv_heads, int D, int page, const int32_t *row_seq, const int32_t *row_pos,
                       const int32_t *block_table, int table_stride, int M, float *part, int *counters, int chunks,
                       int chunk, cudaStream_t st) {
  dim3 grid(M, kv_heads, chunks);
  if (D == 128)
    gqa_paged_split_kernel<G, 4><<<grid, 256, 0, st>>>(qkv, ld, kp, vp, part, kv_heads, page, row_seq, row_pos,
                                                       block_table, table_stride, chunk, counters, out, ldo);
  else
    gqa_paged_split_kernel<G, 2><<<grid, 256, 0, st>>>(qkv, ld, kp, vp, part, kv_heads, page, row_seq, row_pos,
                                                       block_table, table_stride, chunk, counters, out, ldo);
  B200_LAUNCH_CHECK();
  return B200_OK;
}

// one first-maximum per row of a [rows, n] matrix (Sampler.h:101-104); 1024 threads per row,
// 16-byte loads when the rows allow it
__global__ void __launch_bounds__(1024) argmax_rows_kernel(const float *v, int64_t n, int32_t *out) {
  const float *row = v + (int64_t)blockIdx.x * n;
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  auto take = [&](float x, int i) {
    if (x > bv || (x == bv && i < bi)) {
      bv = x;
      bi = i;
    }
  };
  if ((n & 3) == 0 && ((uintptr_t)row & 15) == 0) {
    for (int64_t i = (int64_t)threadIdx.x * 4; i < n; i += (int64_t)blockDim.x * 4) {
      const float4 x = *reinterpret_cast<const float4 *>(row + i);
      take(x.x, (int)i);
      take(x.y, (int)i + 1);
      take(x.z, (int)i + 2);
      take(x.w, (int)i + 3);
    }
  } else {
    for (int64_t i = threadIdx.x; i < n; i += blockDim.x)
      take(row[i], (int)i);
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
  const int chunk = paged_chunk(max_context);
  const int chunks = (max_context + chunk - 1) / chunk;
  // one completion counter per (row, kv head) in front (zero between launches), then the partials
  return (int64_t)rows * q_heads + (int64_t)rows * chunks * q_heads * (D + 2);
}

// scratch: gqa_paged_scratch_floats(scratch_rows, ..) floats whose first scratch_rows * q_heads
// words are zero, or null (then, and for more than scratch_rows or kPagedSplitRows rows, every
// row is scanned by one CTA)
int gqa_paged_launch(const float *qkv, int64_t ld, const float *k_pool, const float *v_pool, float *out, int64_t ldo,
                     int q_heads, int kv_heads, int D, int page, const int32_t *row_seq, const int32_t *row_pos,
                     const int32_t *block_table, int table_stride, int M, float *scratch, int scratch_rows,
                     int max_context, cudaStream_t st) {
  if (D != 64 && D != 128)
    return fail(B200_EINVAL, "gqa_paged: head_dim %d (64 or 128 supported)", D);
  constexpr int kPagedSplitRows = 256;
  const int chunk = paged_chunk(max_context);
  const bool split = scratch != nullptr && M <= scratch_rows && M <= kPagedSplitRows && max_context > chunk;
  int *counters = reinterpret_cast<int *>(scratch);
  float *part = scratch ? scratch + (int64_t)scratch_rows * q_heads : nullptr;
  const int chunks = (max_context + chunk - 1) / chunk;
  switch (q_heads / kv_heads) {
#define B200_G(G_)                                                                                          \
  case G_:                                                                                                  \
    if (split)                                                                                              \
      return launch_paged_split<G_>(qkv, ld, k_pool, v_pool, out, ldo, kv_heads, D, page, row_seq, row_pos, \
                                    block_table, table_stride, M, part, counters, chunks, chunk, st);       \
    return launch_paged_attn<G_>(qkv, ld, k_pool, v_pool, out, ldo, kv_heads, D, page, row_seq, row_pos,    \
                                 block_table, table_stride, M, st);
    B200_G(1) B200_G(2) B200_G(3) B200_G(4) B200_G(6) B200_G(8)
#undef B200_G
  default:
    return fail(B200_EINVAL, "gqa_paged: group size %d not built", q_heads / kv_heads);
  }
}

// M rows of ONE sequence at positions pos0 .. pos0 + M - 1 (a prefill chunk) over the paged
// pool: the attention kernel tiled over query rows.  seq_table: the sequence's row of the
// block table (device).  Needs M >= 64 and 16-byte aligned rows; else returns B200_ESTATE
// untouched and the caller uses gqa_paged_launch.
int gqa_paged_prefill_launch(const float *qkv, int64_t ld, const float *k_pool, const float *v_pool, float *out,
                             int64_t ldo, int q_heads, int kv_heads, int D, int page, const int32_t *seq_table,
                             int pos0, int M, int max_context, cudaStream_t st) {
  if ((D != 64 && D != 128) || M < 64 || (ld & 3) || (ldo & 3) || ((uintptr_t)qkv & 15) || ((uintptr_t)out & 15) ||
      ((uintptr_t)k_pool & 15) || ((uintptr_t)v_pool & 15))
    return B200_ESTATE;
  switch (q_heads / kv_heads) {
#define B200_G(G_)                                                                                                  \
  case G_:                                                                                                          \
    return D == 128 ? launch_prefill_tiled<G_, 128, true>(qkv, ld, k_pool, v_pool, out, ldo, kv_heads, max_context, \
                                                          pos0, M, seq_table, page, st)                             \
                    : launch_prefill_tiled<G_, 64, true>(qkv, ld, k_pool, v_pool, out, ldo, kv_heads, max_context,  \
                                                         pos0, M, seq_table, page, st);
    B200_G(1) B200_G(2) B200_G(3) B200_G(4) B200_G(6) B200_G(8)
#undef B200_G
  default:
    return B200_ESTATE;
  }
}

int argmax_rows_launch(const float *v, int64_t n, int rows, int32_t *out, cudaStream_t st) {
  argmax_rows_kernel<<<rows, 1024, 0, st>>>(v, n, out);
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
  // many rows: the tiled kernel (needs 16-byte aligned rows); few rows: one CTA per (row, kv head)
  const bool tiled = M >= 64 && (ld & 3) == 0 && (ldo & 3) == 0 && ((uintptr_t)qkv & 15) == 0 &&
                     ((uintptr_t)out & 15) == 0 && ((uintptr_t)kc & 15) == 0 && ((uintptr_t)vc & 15) == 0;
  switch (q_heads / kv_heads) {
#define B200_G(G_)                                                                                      \
  case G_:                                                                                              \
    if (tiled)                                                                                          \
      return D == 128 ? launch_prefill_tiled<G_, 128, false>(qkv, ld, kc, vc, out, ldo, kv_heads, max_len, pos0, \
                                                             M, nullptr, 0, st)                                 \
                      : launch_prefill_tiled<G_, 64, false>(qkv, ld, kc, vc, out, ldo, kv_heads, max_len, pos0, \
                                                            M, nullptr, 0, st);                                 \
    return launch_prefill_attn<G_>(qkv, ld, kc, vc, out, ldo, q_heads, kv_heads, D, max_len, pos0, M, st);
    B200_G(1) B200_G(2) B200_G(3) B200_G(4) B200_G(6) B200_G(8)
#undef B200_G
  default:
    return fail(B200_EINVAL, "gqa_prefill: group size %d not built", q_heads / kv_heads);
  }
}

} // namespace b200

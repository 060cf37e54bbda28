// The host-descriptor surface: per-op _mlir_ciface_buddy_* externs in the
// convention of buddy-mlir's runtime/external_kernels (callee-allocated
// result, strided MemRef descriptors, void return), and the core of the
// whole-entry _mlir_ciface_forward_decode replacement.
#include "common.cuh"
#include "../../include/buddy_b200_memref.h"

#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <tuple>
#include <vector>

using namespace b200;

namespace {

struct DevBuf {
  void *p = nullptr;
  ~DevBuf() { cudaFree(p); }
  int alloc(size_t bytes) {
    if (cudaMalloc(&p, bytes ? bytes : 16) != cudaSuccess) {
      (void)cudaGetLastError();
      p = nullptr;
      return fail(B200_ENOMEM, "cudaMalloc(%zu) failed", bytes);
    }
    return B200_OK;
  }
};

// Gather a strided rank-2 host tensor into a dense row-major host vector.
template <typename T, typename MR>
const T *dense2(const MR *m, std::vector<T> &tmp) {
  const T *base = m->aligned + m->offset;
  const intptr_t R = m->sizes[0], C = m->sizes[1];
  if (m->strides[1] == 1 && (m->strides[0] == C || R == 1))
    return base;
  tmp.resize((size_t)R * C);
  for (intptr_t i = 0; i < R; ++i)
    for (intptr_t j = 0; j < C; ++j)
      tmp[(size_t)i * C + j] = base[i * m->strides[0] + j * m->strides[1]];
  return tmp.data();
}

template <typename T, typename MR> void out2(MR *out, T *data, intptr_t R, intptr_t C) {
  out->allocated = data;
  out->aligned = data;
  out->offset = 0;
  out->sizes[0] = R;
  out->sizes[1] = C;
  out->strides[0] = C;
  out->strides[1] = 1;
}
template <typename MR> void out_null(MR *out) {
  out->allocated = nullptr;
  out->aligned = nullptr;
  out->offset = 0;
}

// ---- weight cache: one packed device copy per (host pointer, shape, kind) ----
struct CachedWeight {
  DevBuf w, scale;
  b200_weight desc{};
};
using Key = std::tuple<const void *, const void *, int64_t, int64_t, int, int>;
std::map<Key, CachedWeight *> g_cache;
std::mutex g_cache_mu;

// src: dense host tensor in the reference layout; scale: dense host scales
// [groups, N] in `sdt`.
int cached_weight(int kind, const void *src, const void *host_scale, int sdt,
                  int signed_nibbles, int64_t K, int64_t N, int64_t groups,
                  const void *key_w, const void *key_s, const b200_weight **out) {
  std::lock_guard<std::mutex> lock(g_cache_mu);
  Key key{key_w, key_s, K, N, kind, (int)groups};
  auto it = g_cache.find(key);
  if (it != g_cache.end()) {
    *out = &it->second->desc;
    return B200_OK;
  }
  if (int rc = ensure_device())
    return rc;
  auto *cw = new CachedWeight();
  DevBuf d_src, d_scale_src;
  const size_t src_bytes = kind == B200_W_F32 ? (size_t)K * N * 4
                         : kind == B200_W_I8  ? (size_t)K * N
                                              : (size_t)K * N / 2;
  int rc = d_src.alloc(src_bytes);
  if (!rc) rc = cw->w.alloc((size_t)packed_row_bytes(kind, K) * N);
  if (!rc && cudaMemcpy(d_src.p, src, src_bytes, cudaMemcpyHostToDevice) != cudaSuccess)
    rc = fail(B200_ECUDA, "weight upload failed");
  if (!rc) rc = b200_pack_weight(kind, d_src.p, K, N, signed_nibbles, cw->w.p, nullptr);
  if (!rc && kind != B200_W_F32) {
    const size_t sb = (size_t)groups * N * (sdt == B200_F32 ? 4 : 2);
    rc = d_scale_src.alloc(sb);
    if (!rc) rc = cw->scale.alloc(sb);
    if (!rc && cudaMemcpy(d_scale_src.p, host_scale, sb, cudaMemcpyHostToDevice) != cudaSuccess)
      rc = fail(B200_ECUDA, "scale upload failed");
    if (!rc) rc = b200_pack_scales(d_scale_src.p, sdt, groups, N, cw->scale.p, nullptr);
  }
  if (!rc && cudaDeviceSynchronize() != cudaSuccess)
    rc = fail(B200_ECUDA, "weight repack failed: %s", cudaGetErrorString(cudaGetLastError()));
  if (rc) {
    delete cw;
    return rc;
  }
  cw->desc.kind = kind;
  cw->desc.group = (kind == B200_W_U4 && groups > 1) ? (int)(K / groups) : 0;
  cw->desc.K = K;
  cw->desc.N = N;
  cw->desc.w = cw->w.p;
  cw->desc.scale = cw->scale.p;
  cw->desc.scale_dtype = sdt;
  g_cache[key] = cw;
  *out = &cw->desc;
  return B200_OK;
}

// y[M,N] = x[M,K] * W through the GEMV kernel, 16 activation rows at a time.
int run_gemv_host(const b200_weight *w, const void *x_host, int x_dtype, int M,
                  void *y_host, int y_dtype) {
  const int64_t K = w->K, N = w->N;
  const size_t xe = x_dtype == B200_F32 ? 4 : 2, ye = y_dtype == B200_F32 ? 4 : 2;
  DevBuf dx, dy;
  if (int rc = dx.alloc((size_t)M * K * xe)) return rc;
  if (int rc = dy.alloc((size_t)M * N * ye)) return rc;
  B200_CUDA(cudaMemcpy(dx.p, x_host, (size_t)M * K * xe, cudaMemcpyHostToDevice));
  for (int m0 = 0; m0 < M; m0 += 16) {
    b200_gemv_args a{};
    a.x = (const char *)dx.p + (size_t)m0 * K * xe;
    a.x_dtype = x_dtype;
    a.y = (char *)dy.p + (size_t)m0 * N * ye;
    a.y_dtype = y_dtype;
    a.M = M - m0 < 16 ? M - m0 : 16;
    if (int rc = b200_gemv(w, &a, nullptr)) return rc;
  }
  B200_CUDA(cudaMemcpy(y_host, dy.p, (size_t)M * N * ye, cudaMemcpyDeviceToHost));
  return B200_OK;
}

template <typename T> T *host_alloc(size_t n) {
  void *p = nullptr;
  const size_t bytes = n * sizeof(T);
  if (posix_memalign(&p, 64, ((bytes + 63) / 64) * 64 + 64) != 0)
    p = std::malloc(bytes ? bytes : 1);
  if (!p)
    fail(B200_ENOMEM, "host allocation of %zu bytes failed", bytes);
  return (T *)p;
}

} // namespace

extern "C" {

void b200_release_cached_weights(void) {
  std::lock_guard<std::mutex> lock(g_cache_mu);
  for (auto &kv : g_cache)
    delete kv.second;
  g_cache.clear();
}

void _mlir_ciface_buddy_matmul_f32(b200_memref_f32_2 *result, b200_memref_f32_2 *A,
                                   b200_memref_f32_2 *B) {
  out_null(result);
  const int64_t M = A->sizes[0], K = A->sizes[1], N = B->sizes[1];
  if (B->sizes[0] != K || M < 1 || K < 1 || N < 1) {
    fail(B200_EINVAL, "buddy_matmul_f32: shape mismatch");
    return;
  }
  std::vector<float> ta, tb;
  const float *a = dense2<float>(A, ta), *b = dense2<float>(B, tb);
  const b200_weight *w = nullptr;
  if (cached_weight(B200_W_F32, b, nullptr, B200_F32, 0, K, N, 1, B->aligned + B->offset,
                    nullptr, &w))
    return;
  float *y = host_alloc<float>((size_t)M * N);
  if (!y) return;
  if (run_gemv_host(w, a, B200_F32, (int)M, y, B200_F32)) {
    std::free(y);
    return;
  }
  out2(result, y, M, N);
}

void _mlir_ciface_buddy_gemv_w8_f32(b200_memref_f32_2 *result, b200_memref_f32_2 *A,
                                    b200_memref_i8_2 *W, b200_memref_f32_2 *scale) {
  out_null(result);
  const int64_t M = A->sizes[0], K = A->sizes[1], N = W->sizes[1];
  if (W->sizes[0] != K || scale->sizes[0] * scale->sizes[1] != N || M < 1) {
    fail(B200_EINVAL, "buddy_gemv_w8_f32: shape mismatch");
    return;
  }
  std::vector<float> ta, ts;
  std::vector<int8_t> tw;
  const float *a = dense2<float>(A, ta), *s = dense2<float>(scale, ts);
  const int8_t *q = dense2<int8_t>(W, tw);
  const b200_weight *w = nullptr;
  if (cached_weight(B200_W_I8, q, s, B200_F32, 1, K, N, 1, W->aligned + W->offset,
                    scale->aligned + scale->offset, &w))
    return;
  float *y = host_alloc<float>((size_t)M * N);
  if (!y) return;
  if (run_gemv_host(w, a, B200_F32, (int)M, y, B200_F32)) {
    std::free(y);
    return;
  }
  out2(result, y, M, N);
}

void _mlir_ciface_buddy_gemv_w4_f16(b200_memref_f16_2 *result, b200_memref_f16_2 *A,
                                    b200_memref_i8_2 *P, b200_memref_f16_2 *scale) {
  out_null(result);
  const int64_t M = A->sizes[0], K = A->sizes[1], N = P->sizes[1] * 2;
  if (P->sizes[0] != K || scale->sizes[0] * scale->sizes[1] != N || M < 1) {
    fail(B200_EINVAL, "buddy_gemv_w4_f16: shape mismatch");
    return;
  }
  std::vector<uint16_t> ta, ts;
  std::vector<int8_t> tw;
  const uint16_t *a = dense2<uint16_t>(A, ta), *s = dense2<uint16_t>(scale, ts);
  const int8_t *q = dense2<int8_t>(P, tw);
  const b200_weight *w = nullptr;
  if (cached_weight(B200_W_U4, q, s, B200_F16, 1, K, N, 1, P->aligned + P->offset,
                    scale->aligned + scale->offset, &w))
    return;
  uint16_t *y = host_alloc<uint16_t>((size_t)M * N);
  if (!y) return;
  if (run_gemv_host(w, a, B200_F16, (int)M, y, B200_F16)) {
    std::free(y);
    return;
  }
  out2(result, y, M, N);
}

void _mlir_ciface_buddy_gemv_w4g_f32(b200_memref_f32_2 *result, b200_memref_f32_2 *A,
                                     b200_memref_i8_2 *P, b200_memref_f16_2 *scale) {
  out_null(result);
  const int64_t M = A->sizes[0], K = A->sizes[1], N = P->sizes[1] * 2;
  const int64_t groups = scale->sizes[0];
  if (P->sizes[0] != K || scale->sizes[1] != N || groups < 1 || K % groups || M < 1) {
    fail(B200_EINVAL, "buddy_gemv_w4g_f32: shape mismatch");
    return;
  }
  std::vector<float> ta;
  std::vector<uint16_t> ts;
  std::vector<int8_t> tw;
  const float *a = dense2<float>(A, ta);
  const uint16_t *s = dense2<uint16_t>(scale, ts);
  const int8_t *q = dense2<int8_t>(P, tw);
  const b200_weight *w = nullptr;
  if (cached_weight(B200_W_U4, q, s, B200_F16, 0, K, N, groups, P->aligned + P->offset,
                    scale->aligned + scale->offset, &w))
    return;
  float *y = host_alloc<float>((size_t)M * N);
  if (!y) return;
  if (run_gemv_host(w, a, B200_F32, (int)M, y, B200_F32)) {
    std::free(y);
    return;
  }
  out2(result, y, M, N);
}

void _mlir_ciface_buddy_rmsnorm_f32(b200_memref_f32_2 *result, b200_memref_f32_2 *x,
                                    b200_memref_f32_1 *w, b200_memref_f32_1 *eps) {
  out_null(result);
  const int64_t R = x->sizes[0], H = x->sizes[1];
  if (w->sizes[0] != H || R < 1 || H < 1 || ensure_device()) {
    fail(B200_EINVAL, "buddy_rmsnorm_f32: shape mismatch or no device");
    return;
  }
  std::vector<float> tx, tw(H);
  const float *xd = dense2<float>(x, tx);
  for (int64_t i = 0; i < H; ++i)
    tw[i] = (w->aligned + w->offset)[i * w->strides[0]];
  DevBuf dx, dw, dy;
  if (dx.alloc(R * H * 4) || dw.alloc(H * 4) || dy.alloc(R * H * 4)) return;
  cudaMemcpy(dx.p, xd, R * H * 4, cudaMemcpyHostToDevice);
  cudaMemcpy(dw.p, tw.data(), H * 4, cudaMemcpyHostToDevice);
  if (b200_rmsnorm((float *)dx.p, (float *)dw.p, (float *)dy.p, R, H,
                   (eps->aligned + eps->offset)[0], nullptr))
    return;
  float *y = host_alloc<float>((size_t)R * H);
  if (!y) return;
  if (cudaMemcpy(y, dy.p, R * H * 4, cudaMemcpyDeviceToHost) != cudaSuccess) {
    fail(B200_ECUDA, "buddy_rmsnorm_f32: %s", cudaGetErrorString(cudaGetLastError()));
    std::free(y);
    return;
  }
  out2(result, y, R, H);
}

void _mlir_ciface_buddy_silu_mul_f32(b200_memref_f32_2 *result, b200_memref_f32_2 *g,
                                     b200_memref_f32_2 *u) {
  out_null(result);
  const int64_t R = g->sizes[0], C = g->sizes[1], n = R * C;
  if (u->sizes[0] != R || u->sizes[1] != C || n < 1 || ensure_device()) {
    fail(B200_EINVAL, "buddy_silu_mul_f32: shape mismatch or no device");
    return;
  }
  std::vector<float> tg, tu;
  const float *gd = dense2<float>(g, tg), *ud = dense2<float>(u, tu);
  DevBuf dg, du, dy;
  if (dg.alloc(n * 4) || du.alloc(n * 4) || dy.alloc(n * 4)) return;
  cudaMemcpy(dg.p, gd, n * 4, cudaMemcpyHostToDevice);
  cudaMemcpy(du.p, ud, n * 4, cudaMemcpyHostToDevice);
  if (b200_silu_mul((float *)dg.p, (float *)du.p, (float *)dy.p, n, nullptr)) return;
  float *y = host_alloc<float>((size_t)n);
  if (!y) return;
  if (cudaMemcpy(y, dy.p, n * 4, cudaMemcpyDeviceToHost) != cudaSuccess) {
    fail(B200_ECUDA, "buddy_silu_mul_f32: %s", cudaGetErrorString(cudaGetLastError()));
    std::free(y);
    return;
  }
  out2(result, y, R, C);
}

static void out4(b200_memref_f32_4 *out, float *data, const intptr_t *sizes) {
  out->allocated = out->aligned = data;
  out->offset = 0;
  intptr_t st = 1;
  for (int i = 3; i >= 0; --i) {
    out->sizes[i] = sizes[i];
    out->strides[i] = st;
    st *= sizes[i];
  }
}
static bool dense4(const b200_memref_f32_4 *m) {
  intptr_t st = 1;
  for (int i = 3; i >= 0; --i) {
    if (m->sizes[i] != 1 && m->strides[i] != st) return false;
    st *= m->sizes[i];
  }
  return true;
}

void _mlir_ciface_buddy_rope_f32(b200_memref_f32_4 *result, b200_memref_f32_4 *x,
                                 b200_memref_f32_1 *inv_freq, b200_memref_i64_1 *pos) {
  out_null(result);
  const int64_t heads = x->sizes[1], D = x->sizes[3], n = heads * D;
  if (x->sizes[0] != 1 || x->sizes[2] != 1 || !dense4(x) || inv_freq->sizes[0] != D / 2 ||
      inv_freq->strides[0] != 1 || ensure_device()) {
    fail(B200_EINVAL, "buddy_rope_f32: expects dense [1,heads,1,D] and inv_freq [D/2]");
    return;
  }
  // The fused device op rotates q and k and writes the cache row; here only the
  // rotation is wanted, so x plays q and a zeroed one-head dummy plays k and v,
  // written to row `pos` of a dummy cache of pos + 1 rows.
  const int32_t p32 = (int32_t)(pos->aligned + pos->offset)[0];
  if (p32 < 0) {
    fail(B200_EINVAL, "buddy_rope_f32: negative position");
    return;
  }
  DevBuf dq, dk, dv, dkc, dvc, dfreq, dpos;
  if (dq.alloc(n * 4) || dk.alloc(D * 4) || dv.alloc(D * 4) || dfreq.alloc(D / 2 * 4) ||
      dpos.alloc(4) || dkc.alloc((size_t)(p32 + 1) * D * 4) ||
      dvc.alloc((size_t)(p32 + 1) * D * 4))
    return;
  cudaMemcpy(dq.p, x->aligned + x->offset, n * 4, cudaMemcpyHostToDevice);
  cudaMemset(dk.p, 0, D * 4);
  cudaMemset(dv.p, 0, D * 4);
  cudaMemcpy(dfreq.p, inv_freq->aligned + inv_freq->offset, D / 2 * 4, cudaMemcpyHostToDevice);
  cudaMemcpy(dpos.p, &p32, 4, cudaMemcpyHostToDevice);
  if (b200_rope_kv_write((float *)dq.p, (float *)dk.p, (float *)dv.p, (float *)dkc.p,
                         (float *)dvc.p, (float *)dfreq.p, nullptr, nullptr, 0.f, (int)heads, 1,
                         (int)D, p32 + 1, (const int32_t *)dpos.p, nullptr))
    return;
  float *y = host_alloc<float>((size_t)n);
  if (!y) return;
  if (cudaMemcpy(y, dq.p, n * 4, cudaMemcpyDeviceToHost) != cudaSuccess) {
    fail(B200_ECUDA, "buddy_rope_f32: %s", cudaGetErrorString(cudaGetLastError()));
    std::free(y);
    return;
  }
  out4(result, y, x->sizes);
}

void _mlir_ciface_buddy_gqa_decode_f32(b200_memref_f32_4 *result, b200_memref_f32_4 *q,
                                       b200_memref_f32_4 *k_cache, b200_memref_f32_4 *v_cache,
                                       b200_memref_i64_1 *pos) {
  out_null(result);
  const int64_t QH = q->sizes[1], D = q->sizes[3], KH = k_cache->sizes[1], L = k_cache->sizes[2];
  const long long p = (pos->aligned + pos->offset)[0];
  if (!dense4(q) || !dense4(k_cache) || !dense4(v_cache) || k_cache->sizes[3] != D ||
      v_cache->sizes[1] != KH || v_cache->sizes[2] != L || p < 0 || p >= L || ensure_device()) {
    fail(B200_EINVAL, "buddy_gqa_decode_f32: shape mismatch or position out of range");
    return;
  }
  int splits = (int)(L / 64);
  splits = splits < 1 ? 1 : (splits > 32 ? 32 : splits);
  const size_t cache_bytes = (size_t)KH * L * D * 4;
  const size_t scratch_bytes = (size_t)b200_gqa_scratch_floats((int)QH, (int)D, splits) * 4;
  DevBuf dq, dk, dv, dout, dscr, dpos;
  if (dq.alloc(QH * D * 4) || dk.alloc(cache_bytes) || dv.alloc(cache_bytes) ||
      dout.alloc(QH * D * 4) || dscr.alloc(scratch_bytes) || dpos.alloc(4))
    return;
  const int32_t p32 = (int32_t)p;
  cudaMemcpy(dq.p, q->aligned + q->offset, QH * D * 4, cudaMemcpyHostToDevice);
  cudaMemcpy(dk.p, k_cache->aligned + k_cache->offset, cache_bytes, cudaMemcpyHostToDevice);
  cudaMemcpy(dv.p, v_cache->aligned + v_cache->offset, cache_bytes, cudaMemcpyHostToDevice);
  cudaMemcpy(dpos.p, &p32, 4, cudaMemcpyHostToDevice);
  cudaMemset(dscr.p, 0, scratch_bytes);
  if (b200_gqa_decode((float *)dq.p, (float *)dk.p, (float *)dv.p, (float *)dout.p,
                      (float *)dscr.p, (int)QH, (int)KH, (int)D, (int)L, splits,
                      (const int32_t *)dpos.p, nullptr))
    return;
  float *y = host_alloc<float>((size_t)QH * D);
  if (!y) return;
  if (cudaMemcpy(y, dout.p, QH * D * 4, cudaMemcpyDeviceToHost) != cudaSuccess) {
    fail(B200_ECUDA, "buddy_gqa_decode_f32: %s", cudaGetErrorString(cudaGetLastError()));
    std::free(y);
    return;
  }
  out4(result, y, q->sizes);
}

// ---- whole-entry core ---------------------------------------------------------
namespace {
struct ForwardSession {
  b200_model *model = nullptr;
  const void *w0 = nullptr, *w1 = nullptr;
  long long next_pos = -1;
  std::vector<float> rows;
};
ForwardSession g_fwd;
std::mutex g_fwd_mu;
} // namespace

void b200_forward_reset(void) {
  std::lock_guard<std::mutex> lock(g_fwd_mu);
  b200_model_destroy(g_fwd.model);
  g_fwd = ForwardSession();
}

int b200_forward_decode(const b200_model_config *cfg, const char *variant, int all_linear_w8,
                        const void *w0, int64_t n0, const void *w1, int64_t n1,
                        long long token, long long pos, float *const *host_kv,
                        float **logits_out) {
  if (!cfg || !variant || !w0 || !host_kv || !logits_out)
    return fail(B200_EINVAL, "forward_decode: null argument");
  std::lock_guard<std::mutex> lock(g_fwd_mu);
  ForwardSession &s = g_fwd;
  if (!s.model || s.w0 != w0 || s.w1 != w1) {
    // first call, or a different weight blob: (re)build the device session
    b200_model_destroy(s.model);
    s = ForwardSession();
    b200_model_config c = *cfg;
    c.tp_rank = 0;
    c.tp_size = 1;
    if (int rc = b200_model_create(&c, &s.model)) return rc;
    int rc = b200_model_load_blobs(s.model, variant, w0, n0, w1, n1, all_linear_w8);
    if (!rc) rc = b200_model_finalize(s.model);
    if (rc) {
      b200_model_destroy(s.model);
      s = ForwardSession();
      return rc;
    }
    s.w0 = w0;
    s.w1 = w1;
    s.rows.resize((size_t)2 * c.n_layers * c.kv_heads * c.head_dim);
  }
  const int nbuf = 2 * cfg->n_layers;
  if (pos != s.next_pos) {
    // hand-off from the host: everything before `pos` comes from host_kv
    for (int b = 0; b < nbuf; ++b)
      if (int rc = b200_model_kv_upload(s.model, b, host_kv[b], 0, (int)pos)) return rc;
  }
  float *logits = host_alloc<float>((size_t)cfg->vocab);
  if (!logits)
    return B200_ENOMEM;
  int rc = b200_model_decode(s.model, (int)token, (int)pos, logits, nullptr);
  if (!rc) rc = b200_model_read_new_kv_rows(s.model, s.rows.data());
  if (rc) {
    std::free(logits);
    s.next_pos = -1;
    return rc;
  }
  const size_t D = cfg->head_dim, KH = cfg->kv_heads, L = cfg->max_len;
  for (int b = 0; b < nbuf; ++b)
    for (size_t h = 0; h < KH; ++h)
      memcpy(host_kv[b] + (h * L + (size_t)pos) * D, &s.rows[((size_t)b * KH + h) * D], D * 4);
  s.next_pos = pos + 1;
  *logits_out = logits;
  return B200_OK;
}

} // extern "C"

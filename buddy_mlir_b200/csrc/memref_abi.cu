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
#include <string>
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

// ---- weight cache ---------------------------------------------------------------
// The quantised entries (gemv_w8 / gemv_w4 / gemv_w4g) take W and its scales as
// model weights: constant for as long as the caller keeps them at that address.
// Their packed device copies are cached under a key that names everything the
// packed bytes depend on (addresses, shape, kind, groups, strides, nibble
// signedness, scale type) and are checked on every hit against a fingerprint of
// the host bytes (up to 4096 evenly spaced 64-bit words of the weight and of
// the scales), so a buffer that was rewritten in place is repacked instead of
// silently reused.  The cache is bounded (BUDDY_B200_WEIGHT_CACHE_MB, default
// 8192): the least recently used copies are dropped first.
// _mlir_ciface_buddy_matmul_f32 does NOT use the cache: its B operand is any
// matmul operand of the graph (an activation, a transposed K, a scratch
// buffer), so it is uploaded on every call.
struct CachedWeight {
  DevBuf w, scale;
  b200_weight desc{};
  uint64_t fingerprint = 0;
  uint64_t last_use = 0;
  size_t bytes = 0;
};
struct WeightKey {
  const void *w, *s;
  int64_t K, N, groups, st0, st1;
  int kind, signed_nibbles, sdt;
  bool operator<(const WeightKey &o) const {
    return std::tie(w, s, K, N, groups, st0, st1, kind, signed_nibbles, sdt) <
           std::tie(o.w, o.s, o.K, o.N, o.groups, o.st0, o.st1, o.kind, o.signed_nibbles, o.sdt);
  }
};
std::map<WeightKey, CachedWeight *> g_cache;
std::mutex g_cache_mu;
uint64_t g_cache_clock = 0;
size_t g_cache_bytes = 0;

uint64_t fingerprint_bytes(const void *p, size_t bytes, uint64_t h, size_t samples = 4096) {
  const size_t words = bytes / 8;
  const uint64_t *q = (const uint64_t *)p;
  const size_t n = words < samples ? words : samples;
  for (size_t i = 0; i < n; ++i) {
    uint64_t v;
    memcpy(&v, q + (n > 1 ? i * (words - 1) / (n - 1) : 0), 8);
    h = (h ^ v) * 0x100000001B3ull;
    h ^= h >> 29;
  }
  const unsigned char *tail = (const unsigned char *)p + words * 8;
  for (size_t i = 0; i < bytes - words * 8; ++i)
    h = (h ^ tail[i]) * 0x100000001B3ull;
  return h ^ bytes;
}

size_t cache_limit_bytes() {
  const char *e = std::getenv("BUDDY_B200_WEIGHT_CACHE_MB");
  const long mb = e ? std::atol(e) : 8192;
  return (size_t)(mb > 0 ? mb : 0) << 20;
}

void cache_evict_to(size_t limit) {   // g_cache_mu held
  while (g_cache_bytes > limit && !g_cache.empty()) {
    auto victim = g_cache.begin();
    for (auto it = g_cache.begin(); it != g_cache.end(); ++it)
      if (it->second->last_use < victim->second->last_use)
        victim = it;
    g_cache_bytes -= victim->second->bytes;
    delete victim->second;
    g_cache.erase(victim);
  }
}

// Pack a dense host tensor in the reference layout (and its dense scales
// [groups, N] in `sdt`) into a fresh device copy.
int pack_weight_from_host(int kind, const void *src, const void *host_scale, int sdt,
                          int signed_nibbles, int64_t K, int64_t N, int64_t groups,
                          CachedWeight *cw) {
  if (int rc = ensure_device())
    return rc;
  DevBuf d_src, d_scale_src;
  const size_t src_bytes = kind == B200_W_F32 ? (size_t)K * N * 4
                         : kind == B200_W_I8  ? (size_t)K * N
                                              : (size_t)K * N / 2;
  const size_t packed_bytes = (size_t)packed_row_bytes(kind, K) * N;
  int rc = d_src.alloc(src_bytes);
  if (!rc) rc = cw->w.alloc(packed_bytes);
  if (!rc && cudaMemcpy(d_src.p, src, src_bytes, cudaMemcpyHostToDevice) != cudaSuccess)
    rc = fail(B200_ECUDA, "weight upload failed");
  if (!rc) rc = b200_pack_weight(kind, d_src.p, K, N, signed_nibbles, cw->w.p, nullptr);
  size_t sb = 0;
  if (!rc && kind != B200_W_F32) {
    sb = (size_t)groups * N * (sdt == B200_F32 ? 4 : 2);
    rc = d_scale_src.alloc(sb);
    if (!rc) rc = cw->scale.alloc(sb);
    if (!rc && cudaMemcpy(d_scale_src.p, host_scale, sb, cudaMemcpyHostToDevice) != cudaSuccess)
      rc = fail(B200_ECUDA, "scale upload failed");
    if (!rc) rc = b200_pack_scales(d_scale_src.p, sdt, groups, N, cw->scale.p, nullptr);
  }
  if (!rc && cudaDeviceSynchronize() != cudaSuccess)
    rc = fail(B200_ECUDA, "weight repack failed: %s", cudaGetErrorString(cudaGetLastError()));
  if (rc)
    return rc;
  cw->desc.kind = kind;
  cw->desc.group = (kind == B200_W_U4 && groups > 1) ? (int)(K / groups) : 0;
  cw->desc.K = K;
  cw->desc.N = N;
  cw->desc.w = cw->w.p;
  cw->desc.scale = cw->scale.p;
  cw->desc.scale_dtype = sdt;
  cw->bytes = packed_bytes + sb;
  return B200_OK;
}

// src / host_scale: dense host copies (what is packed and fingerprinted);
// key: what identifies the caller's tensor.  The returned descriptor stays
// valid until the next cache call (the entry points hold g_entry_mu).
int cached_weight(int kind, const void *src, const void *host_scale, int sdt,
                  int signed_nibbles, int64_t K, int64_t N, int64_t groups,
                  WeightKey key, const b200_weight **out) {
  std::lock_guard<std::mutex> lock(g_cache_mu);
  key.K = K; key.N = N; key.groups = groups;
  key.kind = kind; key.signed_nibbles = signed_nibbles; key.sdt = sdt;
  const size_t src_bytes = kind == B200_W_F32 ? (size_t)K * N * 4
                         : kind == B200_W_I8  ? (size_t)K * N
                                              : (size_t)K * N / 2;
  uint64_t fp = fingerprint_bytes(src, src_bytes, 0xCBF29CE484222325ull);
  if (host_scale)
    fp = fingerprint_bytes(host_scale, (size_t)groups * N * (sdt == B200_F32 ? 4 : 2), fp);
  auto it = g_cache.find(key);
  if (it != g_cache.end()) {
    if (it->second->fingerprint == fp) {
      it->second->last_use = ++g_cache_clock;
      *out = &it->second->desc;
      return B200_OK;
    }
    g_cache_bytes -= it->second->bytes;   // rewritten in place: repack
    delete it->second;
    g_cache.erase(it);
  }
  auto *cw = new CachedWeight();
  if (int rc = pack_weight_from_host(kind, src, host_scale, sdt, signed_nibbles, K, N, groups, cw)) {
    delete cw;
    return rc;
  }
  cw->fingerprint = fp;
  cw->last_use = ++g_cache_clock;
  const size_t limit = cache_limit_bytes();
  cache_evict_to(limit > cw->bytes ? limit - cw->bytes : 0);
  g_cache[key] = cw;
  g_cache_bytes += cw->bytes;
  *out = &cw->desc;
  return B200_OK;
}
template <typename MRW, typename MRS> WeightKey key_of(const MRW *W, const MRS *S) {
  WeightKey k{};
  k.w = W->aligned + W->offset;
  k.s = S ? (const void *)(S->aligned + S->offset) : nullptr;
  k.st0 = W->strides[0];
  k.st1 = W->strides[1];
  return k;
}
// One per-op call at a time: the calls come from the model's main thread
// (runtime/external_kernels convention), and a cache descriptor must outlive
// the call that uses it.
std::mutex g_entry_mu;

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
  g_cache_bytes = 0;
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
  // B is whatever the graph multiplies by (runtime_matmul_replace.py:27-55
  // rewrites every MatmulOp): packed afresh on every call, never cached.
  CachedWeight fresh;
  if (pack_weight_from_host(B200_W_F32, b, nullptr, B200_F32, 0, K, N, 1, &fresh))
    return;
  const b200_weight *w = &fresh.desc;
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
  std::lock_guard<std::mutex> entry(g_entry_mu);
  if (cached_weight(B200_W_I8, q, s, B200_F32, 1, K, N, 1, key_of(W, scale), &w))
    return;
  float *y = host_alloc<float>((size_t)M * N);
  if (!y) return;
  if (run_gemv_host(w, a, B200_F32, (int)M, y, B200_F32)) {
    std::free(y);
    return;
  }
  out2(result, y, M, N);
}

void _mlir_ciface_buddy_matmul_w8a8_f32(b200_memref_f32_2 *result, b200_memref_f32_2 *A,
                                        b200_memref_i8_2 *W, b200_memref_f32_2 *scale) {
  out_null(result);
  const int64_t M = A->sizes[0], K = A->sizes[1], N = W->sizes[1];
  if (W->sizes[0] != K || scale->sizes[0] * scale->sizes[1] != N || M < 1 || M > 0x7fffffff) {
    fail(B200_EINVAL, "buddy_matmul_w8a8_f32: shape mismatch");
    return;
  }
  std::vector<float> ta, ts;
  std::vector<int8_t> tw;
  const float *a = dense2<float>(A, ta), *s = dense2<float>(scale, ts);
  const int8_t *q = dense2<int8_t>(W, tw);
  const b200_weight *w = nullptr;
  std::lock_guard<std::mutex> entry(g_entry_mu);
  if (cached_weight(B200_W_I8, q, s, B200_F32, 1, K, N, 1, key_of(W, scale), &w))
    return;
  DevBuf da, dc, ws;
  const int64_t wsb = b200_gemm_w8a8_workspace_bytes((int)M, K);
  if (da.alloc((size_t)M * K * 4) || dc.alloc((size_t)M * N * 4) || ws.alloc((size_t)wsb))
    return;
  if (cudaMemcpy(da.p, a, (size_t)M * K * 4, cudaMemcpyHostToDevice) != cudaSuccess) {
    fail(B200_ECUDA, "buddy_matmul_w8a8_f32: upload failed");
    return;
  }
  if (b200_gemm_w8a8(w, (const float *)da.p, (int)M, K, (float *)dc.p, N, ws.p, wsb, nullptr) ||
      b200_gemm_w8_status(ws.p, nullptr))
    return;
  float *y = host_alloc<float>((size_t)M * N);
  if (!y) return;
  if (cudaMemcpy(y, dc.p, (size_t)M * N * 4, cudaMemcpyDeviceToHost) != cudaSuccess) {
    fail(B200_ECUDA, "buddy_matmul_w8a8_f32: download failed");
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
  std::lock_guard<std::mutex> entry(g_entry_mu);
  if (cached_weight(B200_W_U4, q, s, B200_F16, 1, K, N, 1, key_of(P, scale), &w))
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
  std::lock_guard<std::mutex> entry(g_entry_mu);
  if (cached_weight(B200_W_U4, q, s, B200_F16, 0, K, N, groups, key_of(P, scale), &w))
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
// One device session stands behind the two model entry points.  The reference
// entries are stateless (every call receives the host KV cache), this one keeps
// the cache on the device; `shadow` is a host copy of what the device cache
// holds, row for row, and decides when the device copy may be trusted.
extern "C++" {
namespace {
struct ForwardSession {
  b200_model *model = nullptr;
  const void *w0 = nullptr, *w1 = nullptr;
  uint64_t w_quick = 0;
  int64_t n0 = 0;
  std::string variant;
  // the same model in its other layout (plain <-> panel-packed decode blob), once recognised
  const void *alias_w0 = nullptr;
  uint64_t alias_quick = 0;
  int valid_rows = 0;                      // rows [0, valid_rows) of shadow == device cache
  std::vector<std::vector<float>> shadow;  // [2*layers][kv_heads*max_len*D]
  std::vector<float> rows;
  std::vector<float> logits;
  bool failed = false;
};
ForwardSession g_fwd;
std::mutex g_fwd_mu;
std::atomic<int> g_fwd_builds{0};   // sessions built since the last reset (diagnostic)

// The packed-decode spec hands the decode entry its own blob: every matmul weight in 32-column
// panels, Bpacked[n / 32][k][n % 32] == B[k, n] (pack_decode_weights.py:32-124), everything
// else byte for byte the plain blob the prefill entry gets.  Two blobs are taken for one model
// when 96 sampled elements agree under that map: 32 of the embedding (unpacked), 32 of layer
// 0's Wq and 32 of the lm_head (both panel-packed).
bool panels_of_same_model(const b200_model_config &c, const float *plain, const float *packed) {
  const int64_t H = c.hidden, D = c.head_dim, QD = (int64_t)c.q_heads * D, V = c.vocab;
  const int64_t total = [&] { int64_t nf = 0, ni = 0; b200_blob_elements(&c, "f32", &nf, &ni); return nf; }();
  for (int i = 0; i < 32; ++i) {
    const int64_t e = (V * H - 1) * i / 31;
    if (memcmp(plain + e, packed + e, 4) != 0)
      return false;
  }
  // blob order: embedding, layer 0 {input norm, Wq, ...}, ..., lm_head, inv_freq
  struct { int64_t off, K, N; } w[2] = {{V * H + H, H, QD}, {total - D / 2 - H * V, H, V}};
  for (auto &t : w) {
    if (t.N % 32 != 0)
      return false;
    for (int i = 0; i < 32; ++i) {
      const int64_t k = (t.K - 1) * i / 31, n = (t.N - 1) * ((i * 7) % 32) / 31;
      if (memcmp(plain + t.off + k * t.N + n, packed + t.off + ((n / 32) * t.K + k) * 32 + n % 32, 4) != 0)
        return false;
    }
  }
  return true;
}
std::atomic<int> g_fwd_status{0};   // first failure of the entry pair since the last reset (sticky)
inline int note_status(int rc) {
  if (rc != B200_OK) {
    int expected = 0;
    g_fwd_status.compare_exchange_strong(expected, rc);
  }
  return rc;
}

int session_for(ForwardSession &s, const b200_model_config *cfg, const char *variant,
                int all_linear_w8, const void *w0, int64_t n0, const void *w1, int64_t n1) {
  // the blobs are the model: same addresses, sizes and sampled contents = same session.  Every
  // call samples 64 words spread over each blob (a few microseconds beside a millisecond step).
  // n0 counts elements of the float blob: f16 in the f16, w4a16 and w8a16 variants
  const size_t e0 = (!strcmp(variant, "w4a16") || !strcmp(variant, "w8a16") || !strcmp(variant, "f16") ||
                     !strcmp(variant, "bf16")) ? 2 : 4;
  const uint64_t seed = 0xCBF29CE484222325ull;
  uint64_t quick = fingerprint_bytes(w0, (size_t)n0 * e0, seed, 64);
  if (w1)
    quick = fingerprint_bytes(w1, (size_t)n1, quick, 64);
  if (s.model && s.w0 == w0 && s.w1 == w1 && s.w_quick == quick)
    return B200_OK;
  if (s.model && s.alias_w0 == w0 && !w1 && s.alias_quick == quick)
    return B200_OK;
  if (s.model && !w1 && !s.w1 && n0 == s.n0) {
    const bool now_packed = !strcmp(variant, "f32p32"), was_packed = s.variant == "f32p32";
    if ((now_packed && s.variant == "f32") || (was_packed && !strcmp(variant, "f32"))) {
      const float *plain = (const float *)(now_packed ? s.w0 : w0), *packed = (const float *)(now_packed ? w0 : s.w0);
      if (panels_of_same_model(*cfg, plain, packed)) {
        s.alias_w0 = w0;
        s.alias_quick = quick;
        return B200_OK;
      }
    }
  }
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
  s.w_quick = quick;
  s.n0 = n0;
  s.variant = variant;
  g_fwd_builds.fetch_add(1);
  s.rows.resize((size_t)2 * c.n_layers * c.kv_heads * c.head_dim);
  s.shadow.assign((size_t)2 * c.n_layers,
                  std::vector<float>((size_t)c.kv_heads * c.max_len * c.head_dim, 0.f));
  s.valid_rows = 0;
  return B200_OK;
}

// Host-side element of the cache and the logits: float, or IEEE half as uint16_t (the
// reference's f16 / w8a16 / w4a16 variants, tools/buddy-codegen/gen_config.py:37-49).
// The device session and its shadow stay f32; half buffers are converted at the boundary.
inline void to_host(float *dst, const float *src, size_t n) { memcpy(dst, src, n * 4); }
inline void to_host(uint16_t *dst, const float *src, size_t n) {
  for (size_t i = 0; i < n; ++i)
    dst[i] = __half_as_ushort(__float2half_rn(src[i]));
}
inline void from_host(float *dst, const float *src, size_t n) { memcpy(dst, src, n * 4); }
inline void from_host(float *dst, const uint16_t *src, size_t n) {
  for (size_t i = 0; i < n; ++i)
    dst[i] = __half2float(__ushort_as_half(src[i]));
}
// bfloat16 on the host (the bf16 variant): the same 16 bits of storage, another conversion
struct Bf16 { uint16_t bits; };
static_assert(sizeof(Bf16) == 2, "Bf16 must alias uint16_t storage");
inline uint16_t bf16_rn(float f) {       // round to nearest even, as arith.truncf does
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7F800000u) == 0x7F800000u)       // inf / nan: keep the class
    return (uint16_t)((u >> 16) | ((u & 0xFFFFu) ? 0x40u : 0u));
  return (uint16_t)((u + 0x7FFFu + ((u >> 16) & 1u)) >> 16);
}
inline void to_host(Bf16 *dst, const float *src, size_t n) {
  for (size_t i = 0; i < n; ++i)
    dst[i].bits = bf16_rn(src[i]);
}
inline void from_host(float *dst, const Bf16 *src, size_t n) {
  for (size_t i = 0; i < n; ++i) {
    const uint32_t u = (uint32_t)src[i].bits << 16;
    memcpy(&dst[i], &u, 4);
  }
}
inline bool same_row(const Bf16 *host, const float *shadow, size_t n) {
  for (size_t i = 0; i < n; ++i)
    if (host[i].bits != bf16_rn(shadow[i]))
      return false;
  return true;
}
inline bool same_row(const float *host, const float *shadow, size_t n) { return memcmp(host, shadow, n * 4) == 0; }
inline bool same_row(const uint16_t *host, const float *shadow, size_t n) {
  for (size_t i = 0; i < n; ++i)
    if (host[i] != __half_as_ushort(__float2half_rn(shadow[i])))
      return false;
  return true;
}

// Does the host cache still hold, in rows [0, pos), what the device cache holds?
// Row pos-1 of every buffer depends on every earlier token of the sequence, row
// 0 and the middle row catch a rewritten or shifted cache
// (handleKVCacheOverflow, gen_session.py:1471-1506): three rows per head and
// buffer are compared bit for bit.
// HL: rows per kv head of the HOST buffers (max_len, or the cache size of a tier of the
// tiered-cache spec); the shadow and the device cache always hold max_len rows.
template <typename T>
bool host_matches_device(const ForwardSession &s, const b200_model_config *cfg,
                         T *const *host_kv, long long pos, size_t HL) {
  if (pos > s.valid_rows)
    return false;
  if (pos == 0)
    return true;
  const size_t D = cfg->head_dim, KH = cfg->kv_heads, L = cfg->max_len;
  const long long probe[3] = {0, (pos - 1) / 2, pos - 1};
  for (size_t b = 0; b < s.shadow.size(); ++b)
    for (size_t h = 0; h < KH; ++h)
      for (long long r : probe)
        if (!same_row(host_kv[b] + (h * HL + (size_t)r) * D, s.shadow[b].data() + (h * L + (size_t)r) * D, D))
          return false;
  return true;
}

template <typename T>
int forward_decode(const b200_model_config *cfg, const char *variant, int all_linear_w8,
                   const void *w0, int64_t n0, const void *w1, int64_t n1,
                   long long token, long long pos, T *const *host_kv, T **logits_out, int host_len = 0) {
  if (!cfg || !variant || !w0 || !host_kv || !logits_out)
    return fail(B200_EINVAL, "forward_decode: null argument");
  *logits_out = nullptr;
  const size_t HL = host_len > 0 ? (size_t)host_len : (size_t)cfg->max_len;
  if (pos < 0 || pos >= cfg->max_len || (size_t)pos >= HL)
    return fail(B200_EINVAL, "forward_decode: position %lld outside the cache (max_len %d, host rows %zu)", pos,
                cfg->max_len, HL);
  std::lock_guard<std::mutex> lock(g_fwd_mu);
  ForwardSession &s = g_fwd;
  if (int rc = session_for(s, cfg, variant, all_linear_w8, w0, n0, w1, n1)) return rc;
  const int nbuf = 2 * cfg->n_layers;
  const size_t D = cfg->head_dim, KH = cfg->kv_heads, L = cfg->max_len;
  if (!host_matches_device(s, cfg, host_kv, pos, HL)) {
    // hand-off from the host (CPU prefill, another sequence, a shifted cache):
    // everything before `pos` comes from host_kv
    for (int b = 0; b < nbuf; ++b) {
      for (size_t h = 0; h < KH; ++h)
        from_host(s.shadow[b].data() + h * L * D, host_kv[b] + h * HL * D, (size_t)pos * D);
      if (int rc = b200_model_kv_upload(s.model, b, s.shadow[b].data(), 0, (int)pos)) return rc;
    }
    s.valid_rows = (int)pos;
  }
  T *logits = host_alloc<T>((size_t)cfg->vocab);
  if (!logits)
    return B200_ENOMEM;
  float *lf = reinterpret_cast<float *>(logits);     // float host: decode straight into the result
  if (sizeof(T) != 4) {
    s.logits.resize((size_t)cfg->vocab);
    lf = s.logits.data();
  }
  int rc = b200_model_decode(s.model, (int)token, (int)pos, lf, nullptr);
  if (!rc) rc = b200_model_read_new_kv_rows(s.model, s.rows.data());
  if (rc) {
    std::free(logits);
    s.valid_rows = 0;
    return rc;
  }
  if (sizeof(T) != 4)
    to_host(logits, lf, (size_t)cfg->vocab);
  for (int b = 0; b < nbuf; ++b)
    for (size_t h = 0; h < KH; ++h) {
      const float *row = &s.rows[((size_t)b * KH + h) * D];
      to_host(host_kv[b] + (h * HL + (size_t)pos) * D, row, D);
      memcpy(s.shadow[b].data() + (h * L + (size_t)pos) * D, row, D * 4);
    }
  if (s.valid_rows < pos + 1)
    s.valid_rows = (int)pos + 1;
  *logits_out = logits;
  return B200_OK;
}

template <typename T>
int forward_prefill(const b200_model_config *cfg, const char *variant, int all_linear_w8,
                    const void *w0, int64_t n0, const void *w1, int64_t n1,
                    const long long *tokens, int n_rows, T *const *host_kv_out, T *logits_out,
                    int host_len = 0) {
  if (!cfg || !variant || !w0 || !tokens || !host_kv_out || !logits_out)
    return fail(B200_EINVAL, "forward_prefill: null argument");
  const size_t HL = host_len > 0 ? (size_t)host_len : (size_t)cfg->max_len;
  if (n_rows < 1 || n_rows > cfg->max_len || (size_t)n_rows > HL)
    return fail(B200_EINVAL, "forward_prefill: %d rows, the cache holds %d (host rows %zu)", n_rows, cfg->max_len, HL);
  for (int i = 0; i < n_rows; ++i)
    if (tokens[i] < 0 || tokens[i] >= cfg->vocab)
      return fail(B200_EINVAL, "forward_prefill: token %lld at row %d outside the vocabulary",
                  tokens[i], i);
  std::lock_guard<std::mutex> lock(g_fwd_mu);
  ForwardSession &s = g_fwd;
  if (int rc = session_for(s, cfg, variant, all_linear_w8, w0, n0, w1, n1)) return rc;
  const int nbuf = 2 * cfg->n_layers;
  const size_t D = cfg->head_dim, KH = cfg->kv_heads, L = cfg->max_len;
  s.valid_rows = 0;
  // All rows in one pass (dense GEMMs + causal attention); the cache stays on the
  // device for the decode calls that follow.
  {
    std::vector<int32_t> ids((size_t)n_rows);
    for (int i = 0; i < n_rows; ++i)
      ids[(size_t)i] = (int32_t)tokens[i];
    if (sizeof(T) == 4) {
      // [rows, vocab] f32 is hundreds of megabytes: pinned for the duration of the copy, the
      // device-to-host transfer runs at link speed instead of through a bounce buffer
      const size_t bytes = (size_t)n_rows * cfg->vocab * 4;
      const bool pinned = bytes >= ((size_t)32 << 20) &&
                          cudaHostRegister(logits_out, bytes, cudaHostRegisterDefault) == cudaSuccess;
      if (!pinned)
        (void)cudaGetLastError();
      const int rc = b200_model_prefill(s.model, ids.data(), n_rows, 0, reinterpret_cast<float *>(logits_out), 1, nullptr);
      if (pinned)
        cudaHostUnregister(logits_out);
      if (rc)
        return rc;
    } else {
      std::vector<float> lf((size_t)n_rows * cfg->vocab);
      if (int rc = b200_model_prefill(s.model, ids.data(), n_rows, 0, lf.data(), 1, nullptr))
        return rc;
      to_host(logits_out, lf.data(), lf.size());
    }
  }
  for (int b = 0; b < nbuf; ++b) {
    if (int rc = b200_model_kv_download(s.model, b, s.shadow[b].data(), 0, n_rows)) return rc;
    for (size_t h = 0; h < KH; ++h) {
      to_host(host_kv_out[b] + h * HL * D, s.shadow[b].data() + h * L * D, (size_t)n_rows * D);
      if ((size_t)n_rows < HL)   // rows the prefill did not reach read as zero
        memset(host_kv_out[b] + (h * HL + (size_t)n_rows) * D, 0, (HL - (size_t)n_rows) * D * sizeof(T));
    }
  }
  s.valid_rows = n_rows;
  return B200_OK;
}
} // namespace
} // extern "C++"

void b200_forward_reset(void) {
  std::lock_guard<std::mutex> lock(g_fwd_mu);
  b200_model_destroy(g_fwd.model);
  g_fwd = ForwardSession();
  g_fwd_status.store(0);
  g_fwd_builds.store(0);
}

int b200_forward_status(void) { return g_fwd_status.load(); }
int b200_forward_session_builds(void) { return g_fwd_builds.load(); }

int b200_forward_decode(const b200_model_config *cfg, const char *variant, int all_linear_w8,
                        const void *w0, int64_t n0, const void *w1, int64_t n1,
                        long long token, long long pos, float *const *host_kv,
                        float **logits_out) {
  return note_status(forward_decode<float>(cfg, variant, all_linear_w8, w0, n0, w1, n1, token, pos, host_kv, logits_out));
}
int b200_forward_decode_f16(const b200_model_config *cfg, const char *variant, int all_linear_w8,
                            const void *w0, int64_t n0, const void *w1, int64_t n1,
                            long long token, long long pos, uint16_t *const *host_kv,
                            uint16_t **logits_out) {
  return note_status(forward_decode<uint16_t>(cfg, variant, all_linear_w8, w0, n0, w1, n1, token, pos, host_kv, logits_out));
}
int b200_forward_prefill(const b200_model_config *cfg, const char *variant, int all_linear_w8,
                         const void *w0, int64_t n0, const void *w1, int64_t n1,
                         const long long *tokens, int n_rows, float *const *host_kv_out,
                         float *logits_out) {
  return note_status(forward_prefill<float>(cfg, variant, all_linear_w8, w0, n0, w1, n1, tokens, n_rows, host_kv_out, logits_out));
}
// The tiered-cache spec (models/deepseek_r1/specs/f32_tiered_kv_cache.json,
// gen_session.py:303-800): one prefill / decode symbol per cache size; the host buffers of a
// tier hold host_len rows per kv head, the device session always holds max_len rows.
int b200_forward_decode_tier(const b200_model_config *cfg, const char *variant, int all_linear_w8,
                             const void *w0, int64_t n0, const void *w1, int64_t n1,
                             long long token, long long pos, float *const *host_kv, int host_len,
                             float **logits_out) {
  return note_status(forward_decode<float>(cfg, variant, all_linear_w8, w0, n0, w1, n1, token, pos, host_kv,
                                           logits_out, host_len));
}
int b200_forward_prefill_tier(const b200_model_config *cfg, const char *variant, int all_linear_w8,
                              const void *w0, int64_t n0, const void *w1, int64_t n1,
                              const long long *tokens, int n_rows, float *const *host_kv_out, int host_len,
                              float *logits_out) {
  return note_status(forward_prefill<float>(cfg, variant, all_linear_w8, w0, n0, w1, n1, tokens, n_rows,
                                            host_kv_out, logits_out, host_len));
}
// bfloat16 cache and logits on the host, carried as uint16_t (the reference's bf16 variant,
// tools/buddy-codegen/gen_config.py:40-44)
int b200_forward_decode_bf16(const b200_model_config *cfg, const char *variant, int all_linear_w8,
                             const void *w0, int64_t n0, const void *w1, int64_t n1,
                             long long token, long long pos, uint16_t *const *host_kv,
                             uint16_t **logits_out) {
  return note_status(forward_decode<Bf16>(cfg, variant, all_linear_w8, w0, n0, w1, n1, token, pos,
                                          reinterpret_cast<Bf16 *const *>(host_kv),
                                          reinterpret_cast<Bf16 **>(logits_out)));
}
int b200_forward_prefill_bf16(const b200_model_config *cfg, const char *variant, int all_linear_w8,
                              const void *w0, int64_t n0, const void *w1, int64_t n1,
                              const long long *tokens, int n_rows, uint16_t *const *host_kv_out,
                              uint16_t *logits_out) {
  return note_status(forward_prefill<Bf16>(cfg, variant, all_linear_w8, w0, n0, w1, n1, tokens, n_rows,
                                           reinterpret_cast<Bf16 *const *>(host_kv_out),
                                           reinterpret_cast<Bf16 *>(logits_out)));
}
int b200_forward_prefill_f16(const b200_model_config *cfg, const char *variant, int all_linear_w8,
                             const void *w0, int64_t n0, const void *w1, int64_t n1,
                             const long long *tokens, int n_rows, uint16_t *const *host_kv_out,
                             uint16_t *logits_out) {
  return note_status(forward_prefill<uint16_t>(cfg, variant, all_linear_w8, w0, n0, w1, n1, tokens, n_rows, host_kv_out,
                                   logits_out));
}

} // extern "C"

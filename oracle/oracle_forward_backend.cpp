// Test infrastructure (never shipped): the model-entry contract of buddy_b200_memref.h --
// b200_forward_prefill / b200_forward_decode and their _tier forms -- implemented with the CPU
// restatement instead of the device session.  The generated model-entry shims
// (buddy_mlir_b200/gen_model_entry.py) are linked against this library for one purpose: to run
// the reference's generated ModelSession over the SAME shim source on a machine without a GPU
// and compare the ids it generates with the restatement's, which exercises the shim's ABI
// logic (results allocated, aliased or filled in place; the tiered session's cache moves) with
// real numbers.  Nothing in the product loads it.
//
// The host cache is the truth on every call, as the reference's entries are stateless: the
// rows before `pos` are read from it, the new row is written back.  Variants: f32, f32p32
// (decode blob of the packed-decode spec), w8a32, w8a8; f32 cache and logits.
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "buddy_b200.h"
#include "buddy_oracle.h"

namespace {

std::string g_error;

struct Model {
  OrcModel m{};
  std::vector<OrcLayer> layers;
  std::vector<std::vector<float>> plain;      // un-panelled copies of packed weights
  std::vector<std::vector<float>> kv_store;
  std::vector<float *> kv;
};

// blob walk: the module's parameters in first-use order, then the rotary buffer
// (frontend/Python/frontend.py:922-933); quantised tensors of w8a32 / w8a8 live in the int8 blob,
// their scales at the end of the float blob (quantize.py:577-589)
std::unique_ptr<Model> build(const b200_model_config &c, const std::string &variant, const float *fb, int64_t nf,
                             const int8_t *ib, int64_t ni) {
  auto M = std::make_unique<Model>();
  const int64_t H = c.hidden, D = c.head_dim, QD = (int64_t)c.q_heads * D, KD = (int64_t)c.kv_heads * D, F = c.ffn,
                V = c.vocab;
  const bool quant = variant == "w8a32" || variant == "w8a8", panels = variant == "f32p32";
  if (!(variant == "f32" || quant || panels) || c.qk_norm)
    return nullptr;
  const float *fp = fb;
  const int8_t *ip = ib;
  auto takef = [&](int64_t n) { const float *p = fp; fp += n; return p; };
  struct Pending { OrcLinear *L; };
  std::vector<OrcLinear *> pending;
  auto flinear = [&](OrcLinear &L, int64_t K, int64_t N, bool bias) {
    L = OrcLinear{};
    L.kind = ORC_LIN_F32;
    L.K = K;
    L.N = N;
    const float *w = takef(K * N);
    if (panels) {   // Bpacked[n / 32][k][n % 32] == B[k, n]
      M->plain.emplace_back((size_t)(K * N));
      float *dst = M->plain.back().data();
      for (int64_t pn = 0; pn < N / 32; ++pn)
        for (int64_t k = 0; k < K; ++k)
          std::memcpy(dst + k * N + pn * 32, w + (pn * K + k) * 32, 32 * sizeof(float));
      w = dst;
    }
    L.w = w;
    L.bias = bias ? takef(N) : nullptr;
  };
  auto qlinear = [&](OrcLinear &L, int64_t K, int64_t N) {
    if (!quant) {
      flinear(L, K, N, false);
      return;
    }
    L = OrcLinear{};
    L.kind = variant == "w8a8" ? ORC_LIN_W8Q : ORC_LIN_W8;
    L.K = K;
    L.N = N;
    L.w = ip;
    ip += K * N;
    pending.push_back(&L);
  };
  M->layers.assign((size_t)c.n_layers, OrcLayer{});
  M->m.hidden = H; M->m.n_layers = c.n_layers; M->m.q_heads = c.q_heads; M->m.kv_heads = c.kv_heads;
  M->m.head_dim = D; M->m.ffn = F; M->m.vocab = V; M->m.max_len = c.max_len; M->m.eps = c.eps;
  M->m.embed = takef(V * H);
  for (auto &L : M->layers) {
    L.in_norm = takef(H);
    flinear(L.q, H, QD, c.qkv_bias);
    flinear(L.k, H, KD, c.qkv_bias);
    flinear(L.v, H, KD, c.qkv_bias);
    qlinear(L.o, QD, H);
    L.post_norm = takef(H);
    qlinear(L.gate, H, F);
    qlinear(L.up, H, F);
    qlinear(L.down, F, H);
  }
  M->m.layers = M->layers.data();
  M->m.final_norm = takef(H);
  qlinear(M->m.lm_head, H, V);
  M->m.inv_freq = takef(D / 2);
  for (OrcLinear *L : pending)
    L->scale = takef(L->N);
  if (fp - fb != nf || (quant && ip - ib != ni))
    return nullptr;
  M->kv_store.assign((size_t)(2 * c.n_layers), std::vector<float>((size_t)c.kv_heads * c.max_len * D, 0.f));
  for (auto &b : M->kv_store)
    M->kv.push_back(b.data());
  return M;
}

Model *model_for(const b200_model_config *cfg, const char *variant, const void *w0, int64_t n0, const void *w1,
                 int64_t n1) {
  static std::map<std::pair<const void *, std::string>, std::unique_ptr<Model>> cache;
  auto key = std::make_pair(w0, std::string(variant));
  auto it = cache.find(key);
  if (it == cache.end()) {
    auto M = build(*cfg, variant, (const float *)w0, n0, (const int8_t *)w1, n1);
    if (!M) {
      g_error = std::string("oracle backend: cannot build a model from the blobs of variant ") + variant;
      return nullptr;
    }
    it = cache.emplace(key, std::move(M)).first;
  }
  return it->second.get();
}

// host cache [kv_heads, HL, D] <-> restatement cache [kv_heads, max_len, D], rows [0, n)
void rows_in(Model &M, const b200_model_config &c, float *const *host, int64_t HL, int64_t n) {
  const int64_t D = c.head_dim;
  for (size_t b = 0; b < M.kv.size(); ++b)
    for (int64_t h = 0; h < c.kv_heads; ++h)
      std::memcpy(M.kv[b] + h * c.max_len * D, host[b] + h * HL * D, (size_t)(n * D) * sizeof(float));
}

int decode(const b200_model_config *cfg, const char *variant, const void *w0, int64_t n0, const void *w1, int64_t n1,
           long long token, long long pos, float *const *host_kv, int host_len, float **logits_out) {
  if (!cfg || !variant || !w0 || !host_kv || !logits_out)
    return -1;
  *logits_out = nullptr;
  const int64_t HL = host_len > 0 ? host_len : cfg->max_len, D = cfg->head_dim;
  if (pos < 0 || pos >= cfg->max_len || pos >= HL || token < 0 || token >= cfg->vocab) {
    g_error = "oracle backend: token or position out of range";
    return -1;
  }
  Model *M = model_for(cfg, variant, w0, n0, w1, n1);
  if (!M)
    return -1;
  rows_in(*M, *cfg, host_kv, HL, pos);
  float *logits = (float *)std::malloc((size_t)cfg->vocab * sizeof(float));
  orc_decode_step(&M->m, token, pos, M->kv.data(), logits);
  for (size_t b = 0; b < M->kv.size(); ++b)
    for (int64_t h = 0; h < cfg->kv_heads; ++h)
      std::memcpy(host_kv[b] + (h * HL + pos) * D, M->kv[b] + (h * cfg->max_len + pos) * D, (size_t)D * sizeof(float));
  *logits_out = logits;
  return 0;
}

int prefill(const b200_model_config *cfg, const char *variant, const void *w0, int64_t n0, const void *w1, int64_t n1,
            const long long *tokens, int n_rows, float *const *host_kv_out, int host_len, float *logits_out) {
  if (!cfg || !variant || !w0 || !tokens || !host_kv_out || !logits_out)
    return -1;
  const int64_t HL = host_len > 0 ? host_len : cfg->max_len, D = cfg->head_dim;
  if (n_rows < 1 || n_rows > cfg->max_len || n_rows > HL) {
    g_error = "oracle backend: row count outside the cache";
    return -1;
  }
  Model *M = model_for(cfg, variant, w0, n0, w1, n1);
  if (!M)
    return -1;
  std::vector<int64_t> ids(tokens, tokens + n_rows);
  orc_prefill_rows(&M->m, ids.data(), n_rows, M->kv.data(), logits_out);
  for (size_t b = 0; b < M->kv.size(); ++b)
    for (int64_t h = 0; h < cfg->kv_heads; ++h) {
      float *dst = host_kv_out[b] + h * HL * D;
      std::memcpy(dst, M->kv[b] + h * cfg->max_len * D, (size_t)(n_rows * D) * sizeof(float));
      std::memset(dst + n_rows * D, 0, (size_t)((HL - n_rows) * D) * sizeof(float));
    }
  return 0;
}

} // namespace

extern "C" {

const char *b200_last_error(void) { return g_error.c_str(); }

int b200_forward_decode(const b200_model_config *cfg, const char *variant, int, const void *w0, int64_t n0,
                        const void *w1, int64_t n1, long long token, long long pos, float *const *host_kv,
                        float **logits_out) {
  return decode(cfg, variant, w0, n0, w1, n1, token, pos, host_kv, 0, logits_out);
}
int b200_forward_prefill(const b200_model_config *cfg, const char *variant, int, const void *w0, int64_t n0,
                         const void *w1, int64_t n1, const long long *tokens, int n_rows, float *const *host_kv_out,
                         float *logits_out) {
  return prefill(cfg, variant, w0, n0, w1, n1, tokens, n_rows, host_kv_out, 0, logits_out);
}
int b200_forward_decode_tier(const b200_model_config *cfg, const char *variant, int, const void *w0, int64_t n0,
                             const void *w1, int64_t n1, long long token, long long pos, float *const *host_kv,
                             int host_len, float **logits_out) {
  return decode(cfg, variant, w0, n0, w1, n1, token, pos, host_kv, host_len, logits_out);
}
int b200_forward_prefill_tier(const b200_model_config *cfg, const char *variant, int, const void *w0, int64_t n0,
                              const void *w1, int64_t n1, const long long *tokens, int n_rows,
                              float *const *host_kv_out, int host_len, float *logits_out) {
  return prefill(cfg, variant, w0, n0, w1, n1, tokens, n_rows, host_kv_out, host_len, logits_out);
}

} // extern "C"

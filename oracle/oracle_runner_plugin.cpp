// Test infrastructure (never shipped): the CPU restatement behind buddy-mlir's
// own host loop.  A runner plugin with the ABI buddy-cli loads
// (runtime/include/buddy/runtime/core/InferenceRunner.h:104-114,
// models/deepseek_r1/DeepSeekR1RunnerPlugin.cpp:19-26) whose LLMSession
// (runtime/include/buddy/runtime/llm/LLMSession.h:41-82) runs orc_decode_step;
// generation, sampling, stop rules and the clock are the reference's own
// runGeneration and Sampler (runtime/llm/TextGeneration.cpp:157-277), compiled
// from the buddy-mlir tree into this library.  This is the CPU baseline the
// bench times beside the GPU path: tokens/s as the reference measures them
// (TextGeneration.cpp:135-152).
//
// Weights: RunConfig::weightsPath names the f32 blob in the reference's order
// (frontend/Python/graph/graph.py:836-863).  ORC_RUNNER_MODEL = a stock name
// (deepseek_r1_1p5b, tiny_qwen2) or "hidden=..,n_layers=..,...";
// ORC_RUNNER_ALL_LINEAR_W8=1 quantises every linear layer to int8 per output
// channel with the restated quantiser (the metric's configuration).
// ORC_RUNNER_KV_PREFIX=<rows>,<seed>: prefill() fills rows [0, rows) of every
// cache buffer with seeded N(0,1) values instead of computing them and sets
// the position there, so that the decode loop is timed at a long context
// without a CPU prefill of that length (the GPU bench seeds its cache the
// same way).  Prompts are token ids separated by spaces.
#include "buddy/runtime/core/InferenceRunner.h"
#include "buddy/runtime/llm/TextGeneration.h"

#include <cmath>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <iostream>
#include <random>
#include <sstream>
#include <stdexcept>

#include "buddy_oracle.h"

namespace {

struct Shape {
  int64_t hidden = 0, n_layers = 0, q_heads = 0, kv_heads = 0, head_dim = 0, ffn = 0, vocab = 0, max_len = 0;
  float eps = 1e-6f;
  int qkv_bias = 1;
};

Shape parse_shape() {
  const char *env = std::getenv("ORC_RUNNER_MODEL");
  const std::string spec = env ? env : "deepseek_r1_1p5b";
  Shape s;
  if (spec == "deepseek_r1_1p5b") {
    s = Shape{1536, 28, 12, 2, 128, 8960, 151936, 1024, 1e-6f, 1};
  } else if (spec == "tiny_qwen2") {
    s = Shape{256, 2, 4, 2, 64, 512, 1024, 128, 1e-6f, 1};
  } else {
    std::stringstream ss(spec);
    std::string kv;
    while (std::getline(ss, kv, ',')) {
      const size_t eq = kv.find('=');
      if (eq == std::string::npos)
        continue;
      const std::string k = kv.substr(0, eq);
      const double v = std::atof(kv.c_str() + eq + 1);
      if (k == "hidden") s.hidden = (int64_t)v;
      else if (k == "n_layers") s.n_layers = (int64_t)v;
      else if (k == "q_heads") s.q_heads = (int64_t)v;
      else if (k == "kv_heads") s.kv_heads = (int64_t)v;
      else if (k == "head_dim") s.head_dim = (int64_t)v;
      else if (k == "ffn") s.ffn = (int64_t)v;
      else if (k == "vocab") s.vocab = (int64_t)v;
      else if (k == "max_len") s.max_len = (int64_t)v;
      else if (k == "eps") s.eps = (float)v;
      else if (k == "qkv_bias") s.qkv_bias = (int)v;
    }
  }
  if (s.hidden < 1 || s.n_layers < 1 || s.q_heads < 1 || s.kv_heads < 1 || s.head_dim < 2 || s.ffn < 1 ||
      s.vocab < 1 || s.max_len < 1)
    throw std::runtime_error("[oracle runner] ORC_RUNNER_MODEL does not describe a model: " + spec);
  return s;
}

class OracleSession : public buddy::runtime::LLMSession {
public:
  explicit OracleSession(const Shape &s) : s_(s) {
    logits_.resize((size_t)s.vocab);
    kv_store_.assign((size_t)(2 * s.n_layers), std::vector<float>((size_t)(s.kv_heads * s.max_len * s.head_dim), 0.f));
    for (auto &b : kv_store_)
      kv_.push_back(b.data());
  }

  void loadWeights(const std::vector<std::string> &paths) override {
    if (paths.size() != 1)
      throw std::runtime_error("[oracle runner] one f32 blob expected");
    std::ifstream f(paths[0], std::ios::binary | std::ios::ate);
    if (!f)
      throw std::runtime_error("[oracle runner] cannot open " + paths[0]);
    const std::streamsize n = f.tellg();
    f.seekg(0);
    blob_.resize((size_t)n / 4);
    f.read(reinterpret_cast<char *>(blob_.data()), (std::streamsize)(blob_.size() * 4));
    const char *all = std::getenv("ORC_RUNNER_ALL_LINEAR_W8");
    const bool w8 = all && all[0] == '1';
    // blob walk (parameters as the traced graph first uses them, then the rotary buffer,
    // frontend/Python/frontend.py:922-933): embedding, per layer {in norm, Wq, [q bias,] Wk, [k bias,]
    // Wv, [v bias,] Wo, post norm, Wgate, Wup, Wdown}, final norm, lm_head, inv_freq; every matmul
    // weight [K,N] row-major
    const int64_t H = s_.hidden, D = s_.head_dim, QD = s_.q_heads * D, KD = s_.kv_heads * D, F = s_.ffn, V = s_.vocab;
    size_t off = 0;
    auto take = [&](int64_t count) {
      if (off + (size_t)count > blob_.size())
        throw std::runtime_error("[oracle runner] the blob is shorter than the model");
      const float *p = blob_.data() + off;
      off += (size_t)count;
      return p;
    };
    auto linear = [&](int64_t K, int64_t N, bool with_bias) {
      OrcLinear L{};
      L.K = K;
      L.N = N;
      const float *W = take(K * N);
      L.bias = with_bias ? take(N) : nullptr;
      if (w8) {
        q_.emplace_back((size_t)(K * N));
        sc_.emplace_back((size_t)N);
        orc_quantize_per_channel(W, K, N, 8, q_.back().data(), sc_.back().data());
        L.kind = ORC_LIN_W8;
        L.w = q_.back().data();
        L.scale = sc_.back().data();
      } else {
        L.kind = ORC_LIN_F32;
        L.w = W;
      }
      return L;
    };
    model_ = OrcModel{};
    model_.hidden = H; model_.n_layers = s_.n_layers; model_.q_heads = s_.q_heads; model_.kv_heads = s_.kv_heads;
    model_.head_dim = D; model_.ffn = F; model_.vocab = V; model_.max_len = s_.max_len; model_.eps = s_.eps;
    model_.embed = take(V * H);
    layers_.assign((size_t)s_.n_layers, OrcLayer{});
    for (auto &L : layers_) {
      L.in_norm = take(H);
      L.q = linear(H, QD, s_.qkv_bias);
      L.k = linear(H, KD, s_.qkv_bias);
      L.v = linear(H, KD, s_.qkv_bias);
      L.o = linear(QD, H, false);
      L.post_norm = take(H);
      L.gate = linear(H, F, false);
      L.up = linear(H, F, false);
      L.down = linear(F, H, false);
    }
    model_.layers = layers_.data();
    model_.final_norm = take(H);
    model_.lm_head = linear(H, V, false);
    model_.inv_freq = take(D / 2);
    if (off != blob_.size())
      throw std::runtime_error("[oracle runner] the blob is longer than the model");
  }

  void prefill(buddy::Text<size_t, 2> &tokens) override {
    const int n = (int)tokens.getTokenCnt();
    if (n < 1 || n > s_.max_len)
      throw std::runtime_error("[oracle runner] prompt length outside 1..max_len");
    int start = 0;
    if (const char *pre = std::getenv("ORC_RUNNER_KV_PREFIX")) {
      long rows = 0, seed = 0;
      if (std::sscanf(pre, "%ld,%ld", &rows, &seed) == 2 && rows > 0 && rows + n <= s_.max_len) {
        std::mt19937_64 rng((uint64_t)seed);
        std::normal_distribution<float> nd(0.f, 1.f);
        for (auto &b : kv_store_)
          for (int64_t h = 0; h < s_.kv_heads; ++h)
            for (int64_t r = 0; r < rows; ++r)
              for (int64_t d = 0; d < s_.head_dim; ++d)
                b[(size_t)((h * s_.max_len + r) * s_.head_dim + d)] = nd(rng);
        start = (int)rows;
      }
    }
    // the rows of the prompt, one decode step each (the restatement has no batched prefill)
    prefill_rows_.assign((size_t)n * s_.vocab, 0.f);
    for (int i = 0; i < n; ++i)
      orc_decode_step(&model_, (int64_t)tokens.getData()[i], start + i, kv_.data(),
                      prefill_rows_.data() + (size_t)i * s_.vocab);
    position_ = start + n;
    last_is_decode_ = false;
  }

  void decode(int tokenId) override {
    orc_decode_step(&model_, tokenId, position_, kv_.data(), logits_.data());
    position_ += 1;
    last_is_decode_ = true;
  }

  void resetPosition() override { position_ = 0; }
  int position() const override { return position_; }
  const float *logitsData(int tokenOffset = 0) const override {
    if (last_is_decode_)
      return logits_.data();
    return prefill_rows_.data() + (size_t)tokenOffset * s_.vocab;
  }
  int vocabSize() const override { return (int)s_.vocab; }

  bool handleKVCacheOverflow(int keepTokenNum, float ropeTheta = 10000.0f) override {
    const int64_t np = orc_kv_overflow(kv_.data(), (int64_t)kv_.size(), s_.kv_heads, s_.max_len, s_.head_dim,
                                       position_, keepTokenNum, ropeTheta);
    if (np < 0)
      return false;
    position_ = (int)np;
    return true;
  }

private:
  Shape s_;
  OrcModel model_{};
  std::vector<OrcLayer> layers_;
  std::vector<float> blob_;
  std::vector<std::vector<int8_t>> q_;
  std::vector<std::vector<float>> sc_;
  std::vector<std::vector<float>> kv_store_;
  std::vector<float *> kv_;
  std::vector<float> logits_, prefill_rows_;
  int position_ = 0;
  bool last_is_decode_ = false;
};

class OracleRunner : public buddy::runtime::InferenceRunner {
public:
  void run(const buddy::runtime::RunConfig &cfg) override {
    const Shape shape = parse_shape();
    OracleSession session(shape);
    session.loadWeights({cfg.weightsPath});
    buddy::runtime::TextCodec codec;
    codec.maxTokenLen = (int)shape.max_len;
    const std::string prompt = cfg.prompt;
    codec.tokenize = [prompt](buddy::Text<size_t, 2> &t, const std::string &) {
      buddy::Text<size_t, 2> ids;
      std::stringstream ss(prompt);
      long long id;
      while (ss >> id)
        ids.appendTokenIdx((size_t)id);
      t = std::move(ids);
    };
    codec.detokenize = [](buddy::Text<size_t, 2> &t) {
      std::string s;
      for (size_t i = 0; i < t.getTokenCnt(); ++i)
        s += (i ? " " : "") + std::to_string(t.getData()[i]);
      return s;
    };
    buddy::Sampler sampler(cfg.samplerConfig);
    const buddy::runtime::GenerationResult r =
        buddy::runtime::runGeneration(cfg.prompt, session, cfg.vocabPath, cfg.maxNewTokens, {}, sampler, codec,
                                      cfg.suppressStats, cfg.streamJsonl);
    std::cout << "[ids] " << r.text << std::endl;
    // the reference's own figures (TextGeneration.cpp:135-152), in a form a script can read
    std::cout << "[stats] prefill_s " << r.prefillSecs << " decode_s " << r.decodeSecs << " tokens "
              << r.generatedTokens << " threads " << orc_num_threads() << std::endl;
    if (!cfg.suppressStats)
      buddy::runtime::printStats(r);
  }
};

} // namespace

extern "C" buddy::runtime::InferenceRunner *buddy_create_inference_runner_v1() { return new OracleRunner(); }

extern "C" void buddy_destroy_inference_runner_v1(buddy::runtime::InferenceRunner *runner) { delete runner; }

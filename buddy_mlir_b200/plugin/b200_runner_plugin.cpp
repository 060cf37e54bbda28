// Runner plugin for buddy-cli: the two symbols buddy-cli resolves in a model's
// runner library (runtime/include/buddy/runtime/core/InferenceRunner.h:107-114,
// models/deepseek_r1/DeepSeekR1RunnerPlugin.cpp:19-26) over the device-resident
// session of libbuddy_b200_kernels.so.
//
// B200Session implements buddy-mlir's LLMSession
// (runtime/include/buddy/runtime/llm/LLMSession.h:41-82): weights from the
// reference's arg0*.data blobs, prefill (all prompt rows in one dense pass),
// decode, logits on the host, KV overflow.  B200Runner::run() hands it to the
// reference's own generation loop, runGeneration
// (runtime/llm/TextGeneration.cpp:157-277), compiled from the buddy-mlir tree
// into this library together with its Sampler: tokens, timing and stop rules
// are the reference's, only the session is new.
//
// Built against a buddy-mlir checkout (BUDDY_MLIR_ROOT); nothing of it is
// copied.  Model shapes: BUDDY_B200_MODEL = a stock name (deepseek_r1_1p5b,
// tiny_qwen2) or "hidden=..,n_layers=..,q_heads=..,kv_heads=..,head_dim=..,
// ffn=..,vocab=..,max_len=..[,qkv_bias=0|1]".  RunConfig::weightsPath: one
// file (f32 variant) or "float.data,int8.data" (w8a32); BUDDY_B200_VARIANT
// names another of the reference's variants (f16, bf16, w8a8, w8a16, w4a16:
// tools/buddy-codegen/gen_config.py:37-71) whose files those then are.
// BUDDY_B200_ALL_LINEAR_W8=1 quantises every linear layer of an f32 blob on
// the device.  Prompts are token ids separated by spaces unless
// BUDDY_B200_TOKENIZER=deepseek_r1 asks for the reference's tokenizer.
// BUDDY_B200_PACK_CACHE=<file> keeps the packed device layout of the weights on disk.
#include "buddy/runtime/core/InferenceRunner.h"
#include "buddy/runtime/llm/TextGeneration.h"

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <iostream>
#include <sstream>
#include <stdexcept>

#include "buddy_b200.h"

namespace {

b200_model_config stock_config(const std::string &name) {
  b200_model_config c{};
  if (name == "deepseek_r1_1p5b")
    c = b200_model_config{1536, 28, 12, 2, 128, 8960, 151936, 1024, 1e-6f, 1e4f, 1, 0, 0, 1};
  else if (name == "tiny_qwen2")
    c = b200_model_config{256, 2, 4, 2, 64, 512, 1024, 128, 1e-6f, 1e4f, 1, 0, 0, 1};
  return c;
}

b200_model_config parse_config() {
  const char *env = std::getenv("BUDDY_B200_MODEL");
  const std::string spec = env ? env : "deepseek_r1_1p5b";
  b200_model_config c = stock_config(spec);
  if (c.hidden > 0)
    return c;
  c = b200_model_config{0, 0, 0, 0, 0, 0, 0, 0, 1e-6f, 1e4f, 1, 0, 0, 1};
  std::stringstream ss(spec);
  std::string kv;
  while (std::getline(ss, kv, ',')) {
    const size_t eq = kv.find('=');
    if (eq == std::string::npos)
      continue;
    const std::string k = kv.substr(0, eq);
    const double v = std::atof(kv.c_str() + eq + 1);
    if (k == "hidden") c.hidden = (int)v;
    else if (k == "n_layers") c.n_layers = (int)v;
    else if (k == "q_heads") c.q_heads = (int)v;
    else if (k == "kv_heads") c.kv_heads = (int)v;
    else if (k == "head_dim") c.head_dim = (int)v;
    else if (k == "ffn") c.ffn = (int)v;
    else if (k == "vocab") c.vocab = (int)v;
    else if (k == "max_len") c.max_len = (int)v;
    else if (k == "eps") c.eps = (float)v;
    else if (k == "rope_theta") c.rope_theta = (float)v;
    else if (k == "qkv_bias") c.qkv_bias = (int)v;
  }
  if (c.hidden < 1 || c.n_layers < 1 || c.vocab < 1)
    throw std::runtime_error("[buddy_b200] BUDDY_B200_MODEL does not describe a model: " + spec);
  return c;
}

void check(int rc, const char *what) {
  if (rc != 0)
    throw std::runtime_error(std::string("[buddy_b200] ") + what + ": " + b200_last_error());
}

template <typename T> std::vector<T> read_file(const std::string &path) {
  std::ifstream f(path, std::ios::binary | std::ios::ate);
  if (!f)
    throw std::runtime_error("[buddy_b200] cannot open " + path);
  const std::streamsize n = f.tellg();
  f.seekg(0);
  std::vector<T> v((size_t)n / sizeof(T));
  f.read(reinterpret_cast<char *>(v.data()), (std::streamsize)(v.size() * sizeof(T)));
  return v;
}

class B200Session : public buddy::runtime::LLMSession {
public:
  explicit B200Session(const b200_model_config &cfg) : cfg_(cfg) {
    check(b200_model_create(&cfg_, &model_), "model_create");
    logits_.resize((size_t)cfg_.vocab);
  }
  ~B200Session() override { b200_model_destroy(model_); }

  // gen_session.py:1301-1338: one file per weight blob, in the variant's order.
  // BUDDY_B200_PACK_CACHE=<file>: the packed device layout is read from that file when it
  // exists (no blob walk, no quantisation) and written there after the first load.
  void loadWeights(const std::vector<std::string> &paths) override {
    if (paths.empty() || paths.size() > 2)
      throw std::runtime_error("[buddy_b200] one (f32) or two (w8a32) weight files expected");
    const char *venv = std::getenv("BUDDY_B200_VARIANT");
    const std::string variant = venv && venv[0] ? venv : (paths.size() == 1 ? "f32" : "w8a32");
    const bool two_files = variant == "w8a32" || variant == "w8a8" || variant == "w8a16" || variant == "w4a16";
    if (two_files != (paths.size() == 2))
      throw std::runtime_error("[buddy_b200] variant " + variant + " takes " + (two_files ? "two weight files" : "one weight file"));
    const char *cache = std::getenv("BUDDY_B200_PACK_CACHE");
    if (cache && std::ifstream(cache).good()) {
      if (b200_model_load_packed(model_, cache) == 0) {
        if (variant == "w8a8")     // the arithmetic is not part of the packed weights
          check(b200_model_set_activation_int8(model_, 1), "set_activation_int8");
        check(b200_model_finalize(model_), "finalize");
        return;
      }
      std::cerr << "[buddy_b200] ignoring the pack cache: " << b200_last_error() << "\n";
      b200_model_destroy(model_);           // a partly filled model: start again from the blobs
      model_ = nullptr;
      check(b200_model_create(&cfg_, &model_), "model_create");
    }
    // the float blob holds 16-bit elements in the f16-activation variants and in bf16
    const size_t fsize = (variant == "f32" || variant == "w8a32" || variant == "w8a8") ? 4 : 2;
    const std::vector<char> fb = read_file<char>(paths[0]);
    const char *all = std::getenv("BUDDY_B200_ALL_LINEAR_W8");
    if (!two_files) {
      check(b200_model_load_blobs(model_, variant.c_str(), fb.data(), (int64_t)(fb.size() / fsize), nullptr, 0,
                                  variant == "f32" && all && all[0] == '1'),
            "load_blobs");
    } else {
      const std::vector<int8_t> ib = read_file<int8_t>(paths[1]);
      check(b200_model_load_blobs(model_, variant.c_str(), fb.data(), (int64_t)(fb.size() / fsize), ib.data(),
                                  (int64_t)ib.size(), 0),
            "load_blobs");
    }
    if (cache && b200_model_save_packed(model_, cache) != 0)
      std::cerr << "[buddy_b200] the pack cache was not written: " << b200_last_error() << "\n";
    check(b200_model_finalize(model_), "finalize");
  }

  // gen_session.py:1345-1373; the runtime reads row tokenCnt - 1 (TextGeneration.cpp:190-194)
  void prefill(buddy::Text<size_t, 2> &tokens) override {
    const int n = (int)tokens.getTokenCnt();
    if (n < 1 || n > cfg_.max_len)
      throw std::runtime_error("[buddy_b200] prompt length outside 1..max_len");
    // The w8a8 prefill graph takes its activation scales over every row of the token container,
    // padding included (gen_session.py:1345-1373 passes the whole container), so all of it runs.
    int rows = n;
    if (b200_model_activation_int8(model_))
      rows = (int)std::min<size_t>(tokens.getSize(), (size_t)cfg_.max_len);
    if (rows < n)
      rows = n;
    std::vector<int32_t> ids((size_t)rows);
    for (int i = 0; i < rows; ++i)
      ids[(size_t)i] = (int32_t)tokens.getData()[i];
    prefill_rows_.assign((size_t)rows * cfg_.vocab, 0.f);
    check(b200_model_prefill(model_, ids.data(), rows, 0, prefill_rows_.data(), 1, nullptr), "prefill");
    position_ = n;
    last_is_decode_ = false;
  }

  void decode(int tokenId) override {
    check(b200_model_decode(model_, tokenId, position_, logits_.data(), nullptr), "decode");
    position_ += 1;
    last_is_decode_ = true;
  }

  void resetPosition() override { position_ = 0; }
  int position() const override { return position_; }
  const float *logitsData(int tokenOffset = 0) const override {
    if (last_is_decode_)
      return logits_.data();
    return prefill_rows_.data() + (size_t)tokenOffset * cfg_.vocab;
  }
  int vocabSize() const override { return cfg_.vocab; }

  // gen_session.py:1471-1506 / KVCacheManager.h:151-273, on the device cache
  bool handleKVCacheOverflow(int keepTokenNum, float ropeTheta = 10000.0f) override {
    int new_pos = -1;
    check(b200_model_kv_overflow(model_, position_, keepTokenNum, ropeTheta, &new_pos), "kv_overflow");
    if (new_pos < 0)
      return false;
    position_ = new_pos;
    return true;
  }

private:
  b200_model_config cfg_;
  b200_model *model_ = nullptr;
  int position_ = 0;
  bool last_is_decode_ = false;
  std::vector<float> logits_, prefill_rows_;
};

class B200Runner : public buddy::runtime::InferenceRunner {
public:
  void run(const buddy::runtime::RunConfig &cfg) override {
    const b200_model_config mc = parse_config();
    B200Session session(mc);
    std::vector<std::string> paths;
    {
      std::stringstream ss(cfg.weightsPath);
      std::string p;
      while (std::getline(ss, p, ','))
        if (!p.empty())
          paths.push_back(p);
    }
    session.loadWeights(paths);
    const char *tk = std::getenv("BUDDY_B200_TOKENIZER");
    const bool ref_tokenizer = tk && !std::strcmp(tk, "deepseek_r1");
    buddy::runtime::TextCodec codec;
    codec.maxTokenLen = mc.max_len;
    if (ref_tokenizer) {
      const int max_len = mc.max_len;
      codec.tokenize = [max_len](buddy::Text<size_t, 2> &t, const std::string &vocab) {
        t.tokenizeDeepSeekR1(vocab, (size_t)max_len);
      };
      codec.detokenize = [](buddy::Text<size_t, 2> &t) { return t.revertDeepSeekR1(); };
    } else {
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
    }
    buddy::Sampler sampler(cfg.samplerConfig);
    const buddy::runtime::GenerationResult r =
        buddy::runtime::runGeneration(cfg.prompt, session, cfg.vocabPath, cfg.maxNewTokens, {}, sampler, codec,
                                      cfg.suppressStats, cfg.streamJsonl);
    if (!ref_tokenizer)
      std::cout << "[ids] " << r.text << std::endl;
    if (!cfg.suppressStats)
      buddy::runtime::printStats(r);
  }
};

} // namespace

extern "C" buddy::runtime::InferenceRunner *buddy_create_inference_runner_v1() { return new B200Runner(); }

extern "C" void buddy_destroy_inference_runner_v1(buddy::runtime::InferenceRunner *runner) { delete runner; }

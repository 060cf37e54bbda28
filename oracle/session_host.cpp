// Test infrastructure: buddy-mlir's own host stack over a model-entry library.
//
// The ModelSession that tools/buddy-codegen/gen_session.py GENERATES for a model (here: for
// the small test model, generated at build time into oracle/_ref/generated/ and compiled
// unmodified) loads a model library the way the reference does -- dlopen, then
// _mlir_ciface_forward_prefill and _mlir_ciface_forward_decode by name
// (gen_session.py:1127-1141) -- reads the weight files (:1301-1338), owns the KV cache and the
// prefill / decode ABI structs (:908-972), and is driven by the reference's own generation
// loop and sampler (runtime/llm/TextGeneration.cpp:157-277, Sampler.h:62-104).  Pointing it at
// a shim built by buddy_mlir_b200/gen_model_entry.py is the drop-in test of boundary B2:
// nothing on the host side is this project's code except this main().
//
//   session_host <model.so> <weights[,weights2]> <vocab.txt> <max_new_tokens> <pad_id> "<prompt token ids>"
//
// Prints "[ids] <generated ids>" like the runner-plugin host.
#include "buddy/runtime/llm/TextGeneration.h"
#include "buddy/runtime/models/ModelSession.h"

#include <cstdlib>
#include <iostream>
#include <sstream>
#include <string>
#include <vector>

int main(int argc, char **argv) {
  if (argc < 7) {
    std::cerr << "usage: session_host <model.so> <weights[,more]> <vocab.txt> <max_new_tokens> <pad_id> <prompt ids>\n";
    return 2;
  }
  try {
    buddy::runtime::ModelSession::Config cfg;
    cfg.modelSoPath = argv[1];
    auto session = buddy::runtime::ModelSession::create(cfg);
    std::vector<std::string> paths;
    {
      std::stringstream ss(argv[2]);
      std::string p;
      while (std::getline(ss, p, ','))
        if (!p.empty())
          paths.push_back(p);
    }
    session->loadWeights(paths);
    const std::string vocab = argv[3];
    const int max_new = std::atoi(argv[4]);
    const size_t pad = (size_t)std::atoll(argv[5]);
    const std::string prompt = argv[6];
    const int max_len = cfg.maxTokenLen;
    buddy::runtime::TextCodec codec;
    codec.maxTokenLen = max_len;
    // what the reference's tokenizers leave behind: max_len entries, the prompt first, pad after
    codec.tokenize = [prompt, pad, max_len](buddy::Text<size_t, 2> &t, const std::string &) {
      buddy::Text<size_t, 2> ids;
      std::stringstream ss(prompt);
      long long id;
      size_t n = 0;
      while (ss >> id) {
        ids.appendTokenIdx((size_t)id);
        ++n;
      }
      for (size_t i = n; i < (size_t)max_len; ++i)
        ids.appendTokenIdx(pad);
      ids.setTokenCnt(n);
      t = std::move(ids);
    };
    codec.detokenize = [](buddy::Text<size_t, 2> &t) {
      std::string s;
      for (size_t i = 0; i < t.getTokenCnt(); ++i)
        s += (i ? " " : "") + std::to_string(t.getData()[i]);
      return s;
    };
    buddy::SamplerConfig sc;
    sc.temperature = 0.0f;   // greedy
    buddy::Sampler sampler(sc);
    const buddy::runtime::GenerationResult r =
        buddy::runtime::runGeneration(prompt, *session, vocab, max_new, {}, sampler, codec, true, false);
    std::cout << "[ids] " << r.text << std::endl;
  } catch (const std::exception &e) {
    std::cerr << "session_host failed: " << e.what() << "\n";
    return 1;
  }
  return 0;
}

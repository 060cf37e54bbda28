// Thin C wrapper around buddy-mlir's own host headers, compiled from the
// reference source tree where it lies (never copied).  Test infrastructure
// only: it lets the tests compare the CPU restatement's argmax and KV-overflow
// handling with the reference's real code.
//
//   runtime/include/buddy/runtime/llm/Sampler.h        (Sampler::sample)
//   runtime/include/buddy/runtime/llm/KVCacheManager.h (discardKVCache,
//       buildInverseRopeFreqs, adjustKeyCacheRope)
//
// The overflow driver below repeats the call sequence of the generated
// ModelSession::handleKVCacheOverflow (tools/buddy-codegen/gen_session.py:1471-1506).
#include "buddy/runtime/llm/KVCacheManager.h"
#include "buddy/runtime/llm/Sampler.h"

#include <algorithm>
#include <cstdint>
#include <vector>

extern "C" {

int ref_greedy_sample(const float *logits, int64_t n) {
  buddy::SamplerConfig cfg; // temperature 0 = greedy
  buddy::Sampler sampler(cfg);
  std::vector<int> recent;
  return sampler.sample(logits, (size_t)n, recent);
}

int64_t ref_kv_overflow(float **kv, int64_t nBuffers, int64_t headNum,
                        int64_t maxTokenLen, int64_t hiddenSize,
                        int64_t position, int64_t keepTokenNum, float theta) {
  if (position < maxTokenLen)
    return -1;
  const int currentTokens = (int)std::min(position, maxTokenLen);
  int keep = std::clamp((int)keepTokenNum, 0, currentTokens - 1);
  const int discardLen = std::max(1, (currentTokens - keep) / 2);
  buddy::kvcache::discardKVCache(kv, (int)nBuffers, (int)headNum,
                                 (int)maxTokenLen, (int)hiddenSize, keep,
                                 discardLen, currentTokens);
  auto inv = buddy::kvcache::buildInverseRopeFreqs(theta, (int)hiddenSize);
  buddy::kvcache::adjustKeyCacheRope(kv, (int)nBuffers, (int)headNum,
                                     (int)maxTokenLen, (int)hiddenSize, keep,
                                     discardLen, currentTokens, inv);
  return std::clamp(currentTokens - discardLen, 0, (int)maxTokenLen);
}
}

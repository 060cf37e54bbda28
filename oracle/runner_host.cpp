// Test infrastructure: the few lines of buddy-cli that load a runner plugin
// (tools/buddy-cli/buddy-cli.cpp:195-252): dlopen the runner library, resolve
// buddy_create_inference_runner_v1 / buddy_destroy_inference_runner_v1, fill a
// RunConfig and call run().  buddy-cli itself needs LLVMSupport and
// FlatBuffers and cannot be linked here; RunConfig and InferenceRunner come
// from the buddy-mlir tree (BUDDY_MLIR_ROOT), nothing is copied.
//
//   runner_host <plugin.so> <weights[,weights2]> <vocab.txt> <max_new_tokens> "<prompt>"
#include "buddy/runtime/core/InferenceRunner.h"

#include <dlfcn.h>

#include <cstdlib>
#include <iostream>

int main(int argc, char **argv) {
  if (argc < 6) {
    std::cerr << "usage: runner_host <plugin.so> <weights> <vocab> <max_new_tokens> <prompt>\n";
    return 2;
  }
  void *h = dlopen(argv[1], RTLD_NOW | RTLD_LOCAL);
  if (!h) {
    std::cerr << "dlopen failed: " << dlerror() << "\n";
    return 1;
  }
  auto create = reinterpret_cast<buddy::runtime::CreateInferenceRunnerFn>(dlsym(h, "buddy_create_inference_runner_v1"));
  auto destroy = reinterpret_cast<buddy::runtime::DestroyInferenceRunnerFn>(dlsym(h, "buddy_destroy_inference_runner_v1"));
  if (!create || !destroy) {
    std::cerr << "runner symbols not found\n";
    return 1;
  }
  buddy::runtime::RunConfig cfg;
  cfg.weightsPath = argv[2];
  cfg.vocabPath = argv[3];
  cfg.maxNewTokens = std::atoi(argv[4]);
  cfg.prompt = argv[5];
  cfg.samplerConfig.temperature = 0.0f;   // greedy (Sampler.h:62-104)
  int rc = 0;
  buddy::runtime::InferenceRunner *runner = create();
  try {
    runner->run(cfg);
  } catch (const std::exception &e) {
    std::cerr << "run failed: " << e.what() << "\n";
    rc = 1;
  }
  destroy(runner);
  return rc;
}

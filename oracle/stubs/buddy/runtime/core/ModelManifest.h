// Stand-in for buddy-mlir's runtime/include/buddy/runtime/core/ModelManifest.h, used only to
// compile the reference's GENERATED ModelSession (tools/buddy-codegen/gen_session.py) for the
// drop-in test of the model-entry shims.  The real header reads a .rax package through
// FlatBuffers-generated code, which is not part of a plain checkout; the generated session
// touches it in one place, createFromRax(), which this test never calls.  Test infrastructure:
// nothing shipped includes it.
#ifndef BUDDY_B200_ORACLE_MODEL_MANIFEST_STANDIN_H
#define BUDDY_B200_ORACLE_MODEL_MANIFEST_STANDIN_H

#include <stdexcept>
#include <string>
#include <vector>

namespace buddy {
namespace runtime {

struct ModelManifest {
  std::string soPath;
  std::vector<std::string> dependentSoPaths;
  static ModelManifest loadFromRax(const std::string &path) {
    throw std::runtime_error("ModelManifest stand-in: .rax packages are not read here (" + path + ")");
  }
};

} // namespace runtime
} // namespace buddy

#endif

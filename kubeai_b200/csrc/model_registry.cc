// Model designs by the "architecture" string of their config.json.  The Llama family is the engine's built-in kernel
// sequence (engine.cu) and is recognised by HF's "model_type": "llama"; every other design implements Model (model.h)
// and registers its factory here.
#include "model.h"

namespace b200 {
namespace {
struct Entry {
  const char* arch;
  ModelFactory make;
};
const Entry kModels[] = {
    {"Nomanex", make_nomanex},
    {"Zinavik", make_zinavik},
    {"Mulenex", make_mulenex},
    {"Nagilix", make_nagilix},
};
}  // namespace

ModelFactory find_model_factory(const std::string& arch) {
  for (const Entry& e : kModels)
    if (arch == e.arch) return e.make;
  return nullptr;
}

std::string registered_architectures() {
  std::string s = "llama";
  for (const Entry& e : kModels) s += std::string(", ") + e.arch;
  return s;
}

}  // namespace b200

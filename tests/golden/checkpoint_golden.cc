// Opens a model folder with the reference's own safetensors reader (src/model/
// safetensors.cc, unmodified) and prints, one JSON object a tensor in name order, its
// element type, shape and an FNV-1a hash of its bytes.  make_golden.sh runs it over the
// folder that this repository's `write_random_model` writes for config_cases/tiny_b.json
// with seed 7; the output is committed as checkpoint_golden.jsonl, and
// tests/test_scheduler_golden.py writes that folder again, reads it with this repository's
// own reader and compares: the writer's files are what the reference reads, the two
// readers see the same bytes, and the seeded weights are the same every time.
#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <string>
#include <vector>

#include "inferx/model/safetensors.h"

int main(int argc, char** argv) {
  if (argc != 2) return 2;
  auto ck = inferx::model::Checkpoint::Open(argv[1]);
  if (!ck.ok()) {
    std::fprintf(stderr, "open: %s\n", ck.status().ToString().c_str());
    return 1;
  }
  std::vector<std::string> names = ck->Names();
  std::sort(names.begin(), names.end());
  for (const std::string& name : names) {
    const inferx::model::TensorEntry* e = ck->FindEntry(name);
    auto t = ck->Get(name);
    if (e == nullptr || !t.ok()) {
      std::fprintf(stderr, "%s: not readable\n", name.c_str());
      return 1;
    }
    const unsigned char* p = static_cast<const unsigned char*>(t->data());
    uint64_t h = 1469598103934665603ULL;
    for (size_t i = 0; i < e->nbytes(); ++i) {
      h ^= p[i];
      h *= 1099511628211ULL;
    }
    const std::string dtype(inferx::DataTypeName(e->dtype));
    std::printf("{\"name\": \"%s\", \"dtype\": \"%s\", \"shape\": [", name.c_str(),
                dtype.c_str());
    const auto dims = e->shape.Dims();
    for (size_t d = 0; d < dims.size(); ++d)
      std::printf("%s%lld", d ? ", " : "", (long long)dims[d]);
    std::printf("], \"nbytes\": %zu, \"fnv1a\": \"%016llx\"}\n", e->nbytes(),
                (unsigned long long)h);
  }
  return 0;
}

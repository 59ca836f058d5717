// A small driver around the reference engine's library (libllmi.a of fernandojcardenas/llm-inference-cpp), used only
// by make_golden.py to record outputs that the command-line programs do not print:
//
//   reference_driver sampling  IN.f32 ROWS N TEMPERATURE TOP_K TOP_P OUT.f32
//       llmi::sampling_probabilities (src/model/sampling.cpp:11-58) of ROWS rows of N logits each
//   reference_driver portions  MODEL_DIR IDS PORTION OUT.f32
//       llmi::Transformer::forward_cached (src/model/transformer.cpp:192-306) over the comma-separated IDS in
//       portions of PORTION tokens, every new position's logits — a sequence continued by several tokens at a time
//
// It is not part of the library: it links the reference, which the library never does.
#include <cstdio>
#include <cstdlib>
#include <string>
#include <vector>

#include "llmi/model/model.hpp"
#include "llmi/model/sampling.hpp"
#include "llmi/model/transformer.hpp"

static std::vector<float> read_floats(const char* path, std::size_t count) {
  std::vector<float> v(count);
  std::FILE* f = std::fopen(path, "rb");
  if (!f || std::fread(v.data(), sizeof(float), count, f) != count) {
    std::fprintf(stderr, "cannot read %zu floats from %s\n", count, path);
    std::exit(1);
  }
  std::fclose(f);
  return v;
}

static void write_floats(const char* path, const std::vector<float>& v) {
  std::FILE* f = std::fopen(path, "wb");
  if (!f || std::fwrite(v.data(), sizeof(float), v.size(), f) != v.size()) {
    std::fprintf(stderr, "cannot write %s\n", path);
    std::exit(1);
  }
  std::fclose(f);
}

int main(int argc, char** argv) {
  const std::string mode = argc > 1 ? argv[1] : "";
  if (mode == "sampling" && argc == 9) {
    const std::size_t rows = std::strtoul(argv[3], nullptr, 10), n = std::strtoul(argv[4], nullptr, 10);
    llmi::SamplingConfig cfg;
    cfg.temperature = std::strtof(argv[5], nullptr);
    cfg.top_k = std::strtoul(argv[6], nullptr, 10);
    cfg.top_p = std::strtof(argv[7], nullptr);
    const std::vector<float> logits = read_floats(argv[2], rows * n);
    std::vector<float> out;
    for (std::size_t r = 0; r < rows; ++r) {
      const std::vector<float> p = llmi::sampling_probabilities(logits.data() + r * n, n, cfg);
      out.insert(out.end(), p.begin(), p.end());
    }
    write_floats(argv[8], out);
    return 0;
  }
  if (mode == "portions" && argc == 6) {
    auto model = llmi::Model::load(argv[2]);
    if (!model) {
      std::fprintf(stderr, "%s\n", model.error().c_str());
      return 1;
    }
    auto net = llmi::Transformer::load(model.value());
    if (!net) {
      std::fprintf(stderr, "%s\n", net.error().c_str());
      return 1;
    }
    std::vector<llmi::TokenId> ids;
    for (const char* s = argv[3]; *s;) {
      char* end = nullptr;
      ids.push_back(static_cast<llmi::TokenId>(std::strtoul(s, &end, 10)));
      s = (*end == ',') ? end + 1 : end;
    }
    const std::size_t portion = std::strtoul(argv[4], nullptr, 10);
    auto cache = net.value().new_cache(ids.size());
    if (!cache) {
      std::fprintf(stderr, "%s\n", cache.error().c_str());
      return 1;
    }
    std::vector<float> out;
    for (std::size_t a = 0; a < ids.size(); a += portion) {
      const std::size_t b = a + portion < ids.size() ? a + portion : ids.size();
      const std::vector<llmi::TokenId> part(ids.begin() + static_cast<long>(a), ids.begin() + static_cast<long>(b));
      auto logits = net.value().forward_cached(part, cache.value(), /*all_positions=*/true);
      if (!logits) {
        std::fprintf(stderr, "%s\n", logits.error().c_str());
        return 1;
      }
      out.insert(out.end(), logits.value().begin(), logits.value().end());
    }
    write_floats(argv[5], out);
    return 0;
  }
  std::fprintf(stderr, "usage: reference_driver sampling IN ROWS N T K P OUT | portions MODEL_DIR IDS PORTION OUT\n");
  return 2;
}

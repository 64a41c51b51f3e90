// kuiper_generate: greedy generation with a batched model, from token ids.
//
//   kuiper_generate --model DIR [--dtype bfloat16|float32] [--new N] [--eos ID] [--max-tokens N] [--page N]
//                   --prompt "1 2 3" [--prompt "4 5" ...]
//
// All prompts form one batch: one prompt step, then one token per live request and step (model::BatchScheduler::
// generate).  Prints one line of generated ids per prompt.
#include <cstdio>
#include <cstdlib>
#include <sstream>
#include <string>
#include <vector>

#include "model/sequence_model.h"

int main(int argc, char** argv) {
  std::string dir, dtype = "bfloat16";
  model::SequenceOptions opt;
  int32_t n_new = 16, eos = -1;
  std::vector<std::vector<int32_t>> prompts;
  for (int i = 1; i < argc; ++i) {
    const std::string a = argv[i];
    auto next = [&]() -> const char* { return i + 1 < argc ? argv[++i] : ""; };
    if (a == "--model") dir = next();
    else if (a == "--dtype") dtype = next();
    else if (a == "--new") n_new = std::atoi(next());
    else if (a == "--eos") eos = std::atoi(next());
    else if (a == "--max-tokens") opt.max_tokens = std::atoi(next());
    else if (a == "--page") opt.page_tokens = std::atoi(next());
    else if (a == "--prompt") {
      std::istringstream ss(next());
      std::vector<int32_t> p;
      int32_t t;
      while (ss >> t) p.push_back(t);
      prompts.push_back(p);
    } else {
      std::fprintf(stderr, "unknown argument %s\n", a.c_str());
      return 2;
    }
  }
  if (dir.empty() || prompts.empty() || (dtype != "bfloat16" && dtype != "float32")) {
    std::fprintf(stderr, "usage: %s --model DIR [--dtype bfloat16|float32] [--new N] [--eos ID] [--max-tokens N] "
                         "[--page N] --prompt \"ids\" [--prompt ...]\n", argv[0]);
    return 2;
  }
  opt.compute = dtype == "float32" ? model::ComputeType::kFloat32 : model::ComputeType::kBFloat16;
  opt.max_seqs = static_cast<int32_t>(prompts.size());
  std::unique_ptr<model::SequenceModel> m;
  if (base::Status st = model::create_sequence_model(dir, opt, &m); !st) {
    std::fprintf(stderr, "cannot load %s: %s\n", dir.c_str(), st.get_err_msg().c_str());
    return 2;
  }
  model::BatchScheduler scheduler(m.get());
  std::vector<std::vector<int32_t>> generated;
  if (base::Status st = scheduler.generate(prompts, n_new, eos, &generated); !st) {
    std::fprintf(stderr, "generation failed: %s\n", st.get_err_msg().c_str());
    return 1;
  }
  for (const auto& g : generated) {
    for (size_t i = 0; i < g.size(); ++i) std::printf("%s%d", i ? " " : "", g[i]);
    std::printf("\n");
  }
  return 0;
}

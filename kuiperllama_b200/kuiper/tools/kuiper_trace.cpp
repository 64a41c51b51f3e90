// kuiper_trace: replay a trace of serving steps through a batched model and write the logits that are asked for.
//
//   kuiper_trace --model DIR --dtype bfloat16|float32 --out DIR [--max-tokens N] [--max-seqs N] [--page N]
//                [--residual]
//
// Standard input carries one JSON object per line:
//     {"step": 3, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": ["a"]}
// Every entry brings the next tokens of one request (a new id starts a request); all entries of a step run as one
// batch through model::BatchScheduler and the sequence-batch engine.  "want" lists the positions among the entry's
// tokens whose logits are written, in entry order, as little-endian fp32 [rows, vocab] to OUT/<step>.f32 (no file
// when nothing is wanted).  Requests named in "end" are retired after the step and their cache pages are reused.
// After each step the tool prints "done <step>" and flushes.  --residual also writes the residual stream after every
// layer run of the step to OUT/<step>.residual.f32 ([layer runs, tokens, width]).
// Exit codes: 0 end of input, 1 a step failed, 2 bad arguments or model.
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <iostream>
#include <string>
#include <vector>

#include "model/sequence_model.h"

namespace {
bool write_floats(const std::string& path, const std::vector<float>& data) {
  FILE* f = std::fopen(path.c_str(), "wb");
  if (f == nullptr) return false;
  const size_t n = std::fwrite(data.data(), sizeof(float), data.size(), f);
  return std::fclose(f) == 0 && n == data.size();
}
}  // namespace

int main(int argc, char** argv) {
  std::string dir, dtype = "bfloat16", out;
  model::SequenceOptions opt;
  opt.max_tokens = 8192;
  opt.max_seqs = 256;  // a slot costs one page-table row and one spare page per layer run
  bool residual = false;
  for (int i = 1; i < argc; ++i) {
    const std::string a = argv[i];
    auto next = [&]() -> const char* { return i + 1 < argc ? argv[++i] : ""; };
    if (a == "--model") dir = next();
    else if (a == "--dtype") dtype = next();
    else if (a == "--out") out = next();
    else if (a == "--max-tokens") opt.max_tokens = std::atoi(next());
    else if (a == "--max-seqs") opt.max_seqs = std::atoi(next());
    else if (a == "--page") opt.page_tokens = std::atoi(next());
    else if (a == "--residual") residual = true;
    else {
      std::fprintf(stderr, "unknown argument %s\n", a.c_str());
      return 2;
    }
  }
  if (dir.empty() || out.empty() || opt.max_tokens <= 0 || (dtype != "bfloat16" && dtype != "float32")) {
    std::fprintf(stderr, "usage: %s --model DIR --dtype bfloat16|float32 --out DIR [--max-tokens N] [--max-seqs N] "
                         "[--page N] [--residual]\n", argv[0]);
    return 2;
  }
  opt.compute = dtype == "float32" ? model::ComputeType::kFloat32 : model::ComputeType::kBFloat16;
  std::unique_ptr<model::SequenceModel> m;
  if (base::Status st = model::create_sequence_model(dir, opt, &m); !st) {
    std::fprintf(stderr, "cannot load %s: %s\n", dir.c_str(), st.get_err_msg().c_str());
    return 2;
  }
  model::BatchScheduler scheduler(m.get());
  std::string line;
  while (std::getline(std::cin, line)) {
    if (line.find_first_not_of(" \t\r\n") == std::string::npos) continue;
    long long step = -1;
    std::vector<model::RequestStep> entries;
    std::vector<std::string> finished;
    size_t wanted = 0;
    try {
      const model::json::Value v = model::json::parse(line);
      step = v.at("step").as_int();
      for (const auto& e : v.at("entries").array) {
        model::RequestStep r;
        r.id = e.at("id").as_string();
        for (const auto& t : e.at("tokens").array) r.tokens.push_back(static_cast<int32_t>(t.as_int()));
        if (e.has("want"))
          for (const auto& t : e.at("want").array) r.want.push_back(static_cast<int32_t>(t.as_int()));
        wanted += r.want.size();
        entries.push_back(std::move(r));
      }
      if (v.has("end"))
        for (const auto& e : v.at("end").array) finished.push_back(e.as_string());
    } catch (const std::exception& e) {
      std::fprintf(stderr, "bad step: %s\n", e.what());
      return 1;
    }
    model::StepResult res;
    base::Status st;
    if (residual) {  // the scheduler's path, with the residual trace switched on for this step
      std::vector<model::RequestStep> one = entries;
      st = scheduler.run(one, {}, &res, true, true);
      model::StepResult none;
      if (st) st = scheduler.run({}, finished, &none, false);
    } else {
      st = scheduler.run(entries, finished, &res, true);
    }
    if (!st) {
      std::fprintf(stderr, "step %lld failed: %s\n", step, st.get_err_msg().c_str());
      return 1;
    }
    if (wanted > 0 && !write_floats(out + "/" + std::to_string(step) + ".f32", res.logits)) {
      std::fprintf(stderr, "cannot write into %s\n", out.c_str());
      return 1;
    }
    if (residual && !write_floats(out + "/" + std::to_string(step) + ".residual.f32", res.residual)) return 1;
    std::printf("done %lld\n", step);
    std::fflush(stdout);
  }
  return 0;
}

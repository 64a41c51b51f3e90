// Fobolorn: a decoder-only family served by the sequence-batch engine.
//
//   x = embed[token]
//   layers in the order config "layers" lists them; config "loop" {start, stop, times} runs layers start..stop-1
//   `times` times in a row with the same weights (every pass keeps a cache of its own) and adds row t of the tensor
//   'loop.step' to x right before the first layer of pass t
//   layer:  x += LN_1b(mixer(LN_1(x)));  x += LN_2b(ff(LN_2(x)))   (layer norms with weight and bias; ff optional)
//   mixer 'attention': grouped-query softmax attention without rotation; per-head RMS norm of queries and keys with a
//       shared weight; the query is scaled by 1 + c ln(floor((p + 1) / n) + 1) at position p; scores times a
//       configured scale; a sigmoid gate per head on the output, read from the mixer's input
//   ff 'moe': softmax router over all experts, the top-k renormalised and scaled, SwiGLU experts, plus a shared SwiGLU
//       expert scaled by a sigmoid gate per token
//   logits = head(LN_final(x))
//
// The class only translates config.json and the tensor names into the engine's layer descriptors; every size and
// constant comes from the configuration or from a tensor's shape.
#ifndef KLLM_KUIPER_MODEL_FOBOLORN_H_
#define KLLM_KUIPER_MODEL_FOBOLORN_H_
#include "sequence_model.h"

namespace model {
class FobolornModel final : public SequenceModel {
 protected:
  base::Status build(const json::Value& config, const SafetensorsFile& weights) override;
  base::Status check_folder(const json::Value& config, const SafetensorsFile& weights) override;

 private:
  base::Status build_attention(const json::Value& mixer, const SafetensorsFile& w, const std::string& prefix,
                               kllm_seq_attention* out);
  base::Status build_moe(const json::Value& mlp, const SafetensorsFile& w, const std::string& prefix, kllm_seq_moe* out);
  base::Status load_norm(const SafetensorsFile& w, const std::string& name, kllm_seq_norm* out);
};
}  // namespace model
#endif  // KLLM_KUIPER_MODEL_FOBOLORN_H_

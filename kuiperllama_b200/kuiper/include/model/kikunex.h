// Kikunex: a decoder-only family served by the sequence-batch engine.
//
//   x = N(embed[token]; 'embed.norm');  this x is the embedding output
//   layers in the order config "layers" lists them; config "loop" {start, stop, times} runs layers start..stop-1
//   `times` times in a row with the same weights (every pass keeps a cache / state of its own); before each pass but
//   the first the embedding output is added to x, and before every pass row t of 'loop.step'
//   N(v; g) = v / sqrt(mean(v^2) + eps) * g with ONE number g per norm
//   layer:  x += mixer(shift(N(x; norm1)));  x += ff(N(x; norm2))   (ff optional)
//   shift:  h_t <- h_t + (h_(t-1) - h_t) * 'shift', element by element, zeros before the first token
//   mixer 'latent_attention': queries and keys / values through low-rank latents, rotary positions on a separate
//       part of each query head and on one key part shared by all heads, a sliding window, a per-head sink in the
//       softmax denominator, a sigmoid gate per head
//   mixer 'lightning': linear attention with a per-head decay (silu on q, k, v), RMS norm over the heads, sigmoid gate
//   ff 'dense': down(xIELU(up h));  ff 'moe': sigmoid router with a correction for the choice and a limit to the best
//       groups of experts, squared-ReLU experts, weights = scores * scale
//   logits = head(N(x; 'final.norm')) * logit_scale
//
// The class only translates config.json and the tensor names into the engine's layer descriptors; every size and
// constant comes from the configuration or from a tensor's shape.
#ifndef KLLM_KUIPER_MODEL_KIKUNEX_H_
#define KLLM_KUIPER_MODEL_KIKUNEX_H_
#include "sequence_model.h"

namespace model {
class KikunexModel final : public SequenceModel {
 protected:
  base::Status build(const json::Value& config, const SafetensorsFile& weights) override;
  base::Status check_folder(const json::Value& config, const SafetensorsFile& weights) override;

 private:
  base::Status build_latent(const json::Value& mixer, const SafetensorsFile& w, const std::string& prefix,
                            kllm_seq_latent* out);
  base::Status build_lightning(const json::Value& mixer, const SafetensorsFile& w, const std::string& prefix,
                               kllm_seq_linear* out);
  base::Status build_dense(const json::Value& mlp, const SafetensorsFile& w, const std::string& prefix, kllm_seq_dense* out);
  base::Status build_moe(const json::Value& mlp, const SafetensorsFile& w, const std::string& prefix, kllm_seq_moe* out);
  base::Status scalar_norm(const SafetensorsFile& w, const std::string& name, kllm_seq_norm* out);
};
}  // namespace model
#endif  // KLLM_KUIPER_MODEL_KIKUNEX_H_

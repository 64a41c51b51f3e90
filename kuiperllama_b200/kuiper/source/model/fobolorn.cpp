#include "model/fobolorn.h"

#include <string>
#include <vector>

namespace model {
KLLM_REGISTER_SEQUENCE_MODEL("Fobolorn", FobolornModel);

namespace {
int32_t get_int(const json::Value& v, const char* key) { return static_cast<int32_t>(v.at(key).as_int()); }
}  // namespace

base::Status FobolornModel::load_norm(const SafetensorsFile& w, const std::string& name, kllm_seq_norm* out) {
  base::Status st;
  const StTensor* weight = need(w, name, &st);
  const StTensor* bias = need(w, name + ".b", &st);
  if (!st) return st;
  if (st = upload_f32(weight, width_, &out->w); !st) return st;
  return upload_f32(bias, width_, &out->b);
}

base::Status FobolornModel::build_attention(const json::Value& c, const SafetensorsFile& w, const std::string& p,
                                            kllm_seq_attention* a) {
  a->heads = get_int(c, "heads");
  a->kv_heads = get_int(c, "kv_heads");
  a->dim = get_int(c, "dim");
  a->vdim = get_int(c, "vdim");
  a->scale = static_cast<float>(c.at("scale").as_number());
  a->temp_coef = 0.f, a->temp_every = 0;
  if (c.has("q_temp")) {
    a->temp_coef = static_cast<float>(c.at("q_temp").at("coef").as_number());
    a->temp_every = get_int(c.at("q_temp"), "every");
  }
  if (a->heads <= 0 || a->kv_heads <= 0 || a->heads % a->kv_heads != 0 || a->dim <= 0 || a->vdim <= 0)
    return base::error::ModelParseError(p + ": bad head configuration");
  a->qk_norm = 1, a->gate = 1;
  base::Status st;
  const StTensor *q = need(w, p + "q", &st), *k = need(w, p + "k", &st), *v = need(w, p + "v", &st), *g = need(w, p + "g", &st),
                 *o = need(w, p + "o", &st), *qn = need(w, p + "q.norm", &st), *kn = need(w, p + "k.norm", &st);
  if (!st) return st;
  if (q->numel() != int64_t(a->heads) * a->dim * width_ || k->numel() != int64_t(a->kv_heads) * a->dim * width_ ||
      v->numel() != int64_t(a->kv_heads) * a->vdim * width_ || g->numel() != int64_t(a->heads) * width_)
    return base::error::ModelParseError(p + ": projection shapes do not fit the configuration");
  if (st = upload_compute({q, k, v, g}, width_, &a->w_in); !st) return st;
  if (st = upload_compute({o}, int64_t(a->heads) * a->vdim, &a->w_out); !st) return st;
  if (o->numel() != int64_t(width_) * a->heads * a->vdim) return base::error::ModelParseError(p + "o: unexpected shape");
  if (st = upload_f32(qn, a->dim, &a->q_norm_w); !st) return st;
  return upload_f32(kn, a->dim, &a->k_norm_w);
}

base::Status FobolornModel::build_moe(const json::Value& c, const SafetensorsFile& w, const std::string& p, kllm_seq_moe* m) {
  const json::Value& r = c.at("router");
  m->experts = get_int(r, "experts");
  m->top = get_int(r, "top");
  m->router_scale = r.has("scale") ? static_cast<float>(r.at("scale").as_number()) : 1.0f;
  m->ff = get_int(c.at("expert"), "ff");
  if (m->experts <= 0 || m->top <= 0 || m->top > m->experts || m->ff <= 0)
    return base::error::ModelParseError(p + ": bad router configuration");
  base::Status st;
  std::vector<const StTensor*> gate_up, down;
  for (int e = 0; e < m->experts; ++e) {
    const std::string ep = p + "e" + std::to_string(e) + ".";
    const StTensor *g = need(w, ep + "gate", &st), *u = need(w, ep + "up", &st), *d = need(w, ep + "down", &st);
    if (!st) return st;
    if (g->numel() != int64_t(m->ff) * width_ || u->numel() != g->numel() || d->numel() != g->numel())
      return base::error::ModelParseError(ep + ": expert shapes do not fit the configuration");
    gate_up.push_back(g), gate_up.push_back(u), down.push_back(d);
  }
  if (st = upload_compute(gate_up, width_, &m->gate_up); !st) return st;
  if (st = upload_compute(down, m->ff, &m->down); !st) return st;
  if (st = upload_f32(need(w, p + "router", &st), int64_t(m->experts) * width_, &m->w_router); !st) return st;
  m->shared_ff = 0;
  if (c.has("shared")) {
    m->shared_ff = get_int(c.at("shared"), "ff");
    if (m->shared_ff <= 0) return base::error::ModelParseError(p + "shared: bad size");
    const StTensor *g = need(w, p + "shared.gate", &st), *u = need(w, p + "shared.up", &st), *d = need(w, p + "shared.down", &st),
                   *sg = need(w, p + "shared.sg", &st);
    if (!st) return st;
    if (g->numel() != int64_t(m->shared_ff) * width_ || u->numel() != g->numel() || d->numel() != g->numel())
      return base::error::ModelParseError(p + "shared: shapes do not fit the configuration");
    if (st = upload_compute({g, u}, width_, &m->shared_gate_up); !st) return st;
    if (st = upload_compute({d}, m->shared_ff, &m->shared_down); !st) return st;
    if (st = upload_f32(sg, width_, &m->w_shared_gate); !st) return st;
  }
  return base::error::Success();
}

// every tensor the configuration implies, by name
base::Status FobolornModel::check_folder(const json::Value& config, const SafetensorsFile& w) {
  base::Status st;
  for (const char* name : {"embed", "head", "final.norm", "final.norm.b"}) need(w, name, &st);
  const auto& layers = config.at("layers").array;
  for (size_t i = 0; i < layers.size(); ++i) {
    const std::string p = "l" + std::to_string(i) + ".";
    if (layers[i].at("type").as_string() != "attention")
      return base::error::FunctionNotImplement("layer " + std::to_string(i) + ": unknown mixer");
    std::vector<std::string> names = {"norm1", "norm1.b", "norm1b", "norm1b.b", "mix.q", "mix.k", "mix.v", "mix.g", "mix.o",
                                      "mix.q.norm", "mix.k.norm"};
    if (layers[i].has("mlp")) {
      const json::Value& mc = layers[i].at("mlp");
      for (const char* n : {"norm2", "norm2.b", "norm2b", "norm2b.b", "mlp.router"}) names.push_back(n);
      for (int e = 0; e < get_int(mc.at("router"), "experts"); ++e)
        for (const char* n : {"gate", "up", "down"}) names.push_back("mlp.e" + std::to_string(e) + "." + n);
      if (mc.has("shared"))
        for (const char* n : {"gate", "up", "down", "sg"}) names.push_back(std::string("mlp.shared.") + n);
    }
    for (const std::string& n : names) need(w, p + n, &st);
  }
  return st;
}

base::Status FobolornModel::build(const json::Value& config, const SafetensorsFile& w) {
  vocab_ = get_int(config, "vocab");
  width_ = get_int(config, "width");
  norm_eps_ = static_cast<float>(config.at("norm").at("eps").as_number());
  if (vocab_ <= 0 || width_ <= 0) return base::error::ModelParseError("bad vocab / width");
  const auto& layers = config.at("layers").array;
  if (layers.empty()) return base::error::ModelParseError("no layers");
  base::Status st;
  layers_.assign(layers.size(), kllm_seq_layer{});
  for (size_t i = 0; i < layers.size(); ++i) {
    const json::Value& lc = layers[i];
    kllm_seq_layer& L = layers_[i];
    const std::string p = "l" + std::to_string(i) + ".";
    const std::string& type = lc.at("type").as_string();
    if (type != "attention") return base::error::FunctionNotImplement("layer " + std::to_string(i) + ": unknown mixer '" + type + "'");
    L.mixer_kind = KLLM_SEQ_MIXER_ATTENTION;
    if (st = load_norm(w, p + "norm1", &L.pre_mixer); !st) return st;
    if (st = load_norm(w, p + "norm1b", &L.post_mixer); !st) return st;
    if (st = build_attention(lc.at("mixer"), w, p + "mix.", &L.attn); !st) return st;
    L.ff_kind = KLLM_SEQ_FF_NONE;
    if (lc.has("mlp")) {
      const json::Value& mc = lc.at("mlp");
      const std::string kind = mc.has("kind") ? mc.at("kind").as_string() : "moe";
      if (kind != "moe") return base::error::FunctionNotImplement("layer " + std::to_string(i) + ": unknown feed-forward '" + kind + "'");
      L.ff_kind = KLLM_SEQ_FF_MOE;
      if (st = load_norm(w, p + "norm2", &L.pre_ff); !st) return st;
      if (st = load_norm(w, p + "norm2b", &L.post_ff); !st) return st;
      if (st = build_moe(mc, w, p + "mlp.", &L.moe); !st) return st;
    }
  }
  // the order of layer runs
  const int32_t n = static_cast<int32_t>(layers.size());
  int32_t start = 0, stop = 0, times = 1;
  if (config.has("loop")) {
    const json::Value& lp = config.at("loop");
    start = get_int(lp, "start"), stop = get_int(lp, "stop"), times = get_int(lp, "times");
    if (start < 0 || stop < start || stop > n || times < 1) return base::error::ModelParseError("bad loop");
  }
  run_layer_.clear(), run_add_.clear();
  for (int32_t i = 0; i < start; ++i) run_layer_.push_back(i), run_add_.push_back(-1);
  if (stop > start)
    for (int32_t t = 0; t < times; ++t)
      for (int32_t i = start; i < stop; ++i) run_layer_.push_back(i), run_add_.push_back(i == start ? t : -1);
  for (int32_t i = stop; i < n; ++i) run_layer_.push_back(i), run_add_.push_back(-1);
  if (stop > start) {
    if (st = upload_f32(need(w, "loop.step", &st), int64_t(times) * width_, &run_vectors_); !st) return st;
  }
  if (st = upload_compute({need(w, "embed", &st)}, width_, &embed_); !st) return st;
  if (st = upload_compute({need(w, "head", &st)}, width_, &head_); !st) return st;
  if (w.find("embed")->numel() != int64_t(vocab_) * width_ || w.find("head")->numel() != int64_t(vocab_) * width_)
    return base::error::ModelParseError("embed / head do not fit vocab x width");
  return load_norm(w, "final.norm", &final_norm_);
}
}  // namespace model

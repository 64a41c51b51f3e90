#include "model/kikunex.h"

#include <cmath>
#include <string>
#include <vector>

namespace model {
KLLM_REGISTER_SEQUENCE_MODEL("Kikunex", KikunexModel);

namespace {
int32_t get_int(const json::Value& v, const char* key) { return static_cast<int32_t>(v.at(key).as_int()); }
bool present(const json::Value& v, const char* key) { return v.has(key) && !v.at(key).is_null(); }
double softplus(double z) { return z > 30.0 ? z : std::log1p(std::exp(z)); }
bool shaped(const StTensor* t, int64_t rows, int64_t cols) {
  return t != nullptr && t->shape.size() == 2 && t->shape[0] == rows && t->shape[1] == cols;
}
}  // namespace

base::Status KikunexModel::scalar_norm(const SafetensorsFile& w, const std::string& name, kllm_seq_norm* out) {
  base::Status st;
  const StTensor* g = need(w, name, &st);
  if (!st) return st;
  out->b = nullptr, out->kind = KLLM_SEQ_NORM_RMS;
  return upload_broadcast(g, width_, &out->w);
}

base::Status KikunexModel::build_latent(const json::Value& c, const SafetensorsFile& w, const std::string& p,
                                        kllm_seq_latent* a) {
  a->heads = get_int(c, "heads"), a->dim = get_int(c, "dim"), a->rot_dim = get_int(c, "rot_dim"), a->vdim = get_int(c, "vdim");
  a->q_rank = get_int(c, "q_rank"), a->kv_rank = get_int(c, "kv_rank");
  a->scale = static_cast<float>(c.at("scale").as_number());
  a->window = present(c, "mask") ? get_int(c.at("mask"), "size") : 0;
  a->rope_dims = 0, a->rope_base = 1.f;
  if (present(c, "rot")) {
    a->rope_dims = get_int(c.at("rot"), "dims");
    a->rope_base = static_cast<float>(c.at("rot").at("base").as_number());
  }
  if (a->heads <= 0 || a->dim <= 0 || a->rot_dim < 0 || a->vdim <= 0 || a->q_rank <= 0 || a->kv_rank <= 0 || a->window < 0 ||
      a->rope_dims < 0 || a->rope_dims > a->rot_dim || (a->rope_dims & 1))
    return base::error::ModelParseError(p + ": bad mixer configuration");
  base::Status st;
  const StTensor *dq = need(w, p + "dq", &st), *dqn = need(w, p + "dq.norm", &st), *uq = need(w, p + "uq", &st),
                 *dkv = need(w, p + "dkv", &st), *dkvn = need(w, p + "dkv.norm", &st), *uk = need(w, p + "uk", &st),
                 *uv = need(w, p + "uv", &st), *g = need(w, p + "g", &st), *o = need(w, p + "o", &st);
  if (!st) return st;
  const int64_t H = a->heads;
  if (!shaped(dq, a->q_rank, width_) || !shaped(uq, H * (a->dim + a->rot_dim), a->q_rank) ||
      !shaped(dkv, a->kv_rank + a->rot_dim, width_) || !shaped(uk, H * a->dim, a->kv_rank) ||
      !shaped(uv, H * a->vdim, a->kv_rank) || !shaped(g, H, width_) || !shaped(o, width_, H * a->vdim))
    return base::error::ModelParseError(p + ": tensor shapes do not fit the configuration");
  if (st = upload_compute({dq, dkv, g}, width_, &a->w_in); !st) return st;
  if (st = upload_compute({uq}, a->q_rank, &a->w_uq); !st) return st;
  if (st = upload_compute({uk}, a->kv_rank, &a->w_uk); !st) return st;
  if (st = upload_compute({uv}, a->kv_rank, &a->w_uv); !st) return st;
  if (st = upload_compute({o}, H * a->vdim, &a->w_out); !st) return st;
  if (st = upload_f32(dqn, a->q_rank, &a->q_norm_w); !st) return st;
  if (st = upload_f32(dkvn, a->kv_rank, &a->kv_norm_w); !st) return st;
  a->sink = nullptr;
  if (const StTensor* sink = w.find(p + "sink"); sink != nullptr)
    if (st = upload_f32(sink, H, &a->sink); !st) return st;
  return base::error::Success();
}

base::Status KikunexModel::build_lightning(const json::Value& c, const SafetensorsFile& w, const std::string& p,
                                           kllm_seq_linear* a) {
  a->heads = get_int(c, "heads"), a->dim = get_int(c, "dim"), a->vdim = get_int(c, "vdim");
  if (a->heads <= 0 || a->dim <= 0 || a->vdim <= 0) return base::error::ModelParseError(p + ": bad mixer configuration");
  // one decay per head, or one number for all heads
  std::vector<float> lam;
  if (c.at("decay").is_array()) {
    for (const auto& v : c.at("decay").array) lam.push_back(static_cast<float>(v.as_number()));
  } else {
    lam.assign(static_cast<size_t>(a->heads), static_cast<float>(c.at("decay").as_number()));
  }
  if (static_cast<int64_t>(lam.size()) != a->heads) return base::error::ModelParseError(p + ": one decay per head is needed");
  for (float v : lam)
    if (!(v > 0.f) || v > 1.f) return base::error::ModelParseError(p + ": a decay must lie in (0, 1]");
  base::Status st;
  const StTensor *q = need(w, p + "q", &st), *k = need(w, p + "k", &st), *v = need(w, p + "v", &st), *g = need(w, p + "g", &st),
                 *o = need(w, p + "o", &st), *n = need(w, p + "norm", &st);
  if (!st) return st;
  const int64_t qn = int64_t(a->heads) * a->dim, vn = int64_t(a->heads) * a->vdim;
  if (!shaped(q, qn, width_) || !shaped(k, qn, width_) || !shaped(v, vn, width_) || !shaped(g, vn, width_) ||
      !shaped(o, width_, vn))
    return base::error::ModelParseError(p + ": tensor shapes do not fit the configuration");
  if (st = upload_compute({q, k, v, g}, width_, &a->w_in); !st) return st;
  if (st = upload_compute({o}, vn, &a->w_out); !st) return st;
  if (st = upload_f32(n, vn, &a->out_norm_w); !st) return st;
  return upload_values(lam, &a->decay);
}

base::Status KikunexModel::build_dense(const json::Value& c, const SafetensorsFile& w, const std::string& p,
                                       kllm_seq_dense* f) {
  f->ff = get_int(c, "ff");
  if (f->ff <= 0) return base::error::ModelParseError(p + ": bad size");
  base::Status st;
  const StTensor *up = need(w, p + "up", &st), *down = need(w, p + "down", &st), *act = need(w, p + "act", &st);
  if (!st) return st;
  if (!shaped(up, f->ff, width_) || !shaped(down, width_, f->ff))
    return base::error::ModelParseError(p + ": tensor shapes do not fit the configuration");
  std::vector<float> pq;
  if (st = read_values(act, 2, &pq); !st) return st;
  // xIELU: z > 0: softplus(p) z^2 + z / 2;  z <= 0: (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2
  f->act = KLLM_SEQ_ACT_XIELU;
  f->act_a = static_cast<float>(softplus(pq[0]));
  f->act_b = static_cast<float>(0.5 + softplus(pq[1]));
  if (st = upload_compute({up}, width_, &f->up); !st) return st;
  return upload_compute({down}, f->ff, &f->down);
}

base::Status KikunexModel::build_moe(const json::Value& c, const SafetensorsFile& w, const std::string& p, kllm_seq_moe* m) {
  const json::Value& r = c.at("router");
  m->experts = get_int(r, "experts");
  m->top = get_int(r, "top");
  m->router_scale = r.has("scale") ? static_cast<float>(r.at("scale").as_number()) : 1.0f;
  m->ff = get_int(c.at("expert"), "ff");
  m->router_kind = KLLM_SEQ_ROUTER_SIGMOID;
  m->act = KLLM_SEQ_ACT_RELU2;
  m->groups = 0, m->groups_keep = 0;
  if (present(r, "groups")) {
    m->groups = get_int(r.at("groups"), "count");
    m->groups_keep = get_int(r.at("groups"), "keep");
    if (m->groups <= 0 || m->experts % m->groups != 0 || m->groups_keep <= 0 || m->groups_keep > m->groups)
      return base::error::ModelParseError(p + ": bad expert groups");
  }
  if (m->experts <= 0 || m->top <= 0 || m->top > m->experts || m->ff <= 0)
    return base::error::ModelParseError(p + ": bad router configuration");
  base::Status st;
  std::vector<const StTensor*> up, down;
  for (int e = 0; e < m->experts; ++e) {
    const std::string ep = p + "e" + std::to_string(e) + ".";
    const StTensor *u = need(w, ep + "up", &st), *d = need(w, ep + "down", &st);
    if (!st) return st;
    if (!shaped(u, m->ff, width_) || !shaped(d, width_, m->ff))
      return base::error::ModelParseError(ep + ": expert shapes do not fit the configuration");
    up.push_back(u), down.push_back(d);
  }
  if (st = upload_compute(up, width_, &m->gate_up); !st) return st;
  if (st = upload_compute(down, m->ff, &m->down); !st) return st;
  if (st = upload_f32(need(w, p + "router", &st), int64_t(m->experts) * width_, &m->w_router); !st) return st;
  m->correction = nullptr;
  if (const StTensor* corr = w.find(p + "correction"); corr != nullptr)
    if (st = upload_f32(corr, m->experts, &m->correction); !st) return st;
  m->shared_ff = 0;
  return base::error::Success();
}

// every tensor the configuration implies, by name
base::Status KikunexModel::check_folder(const json::Value& config, const SafetensorsFile& w) {
  base::Status st;
  for (const char* name : {"embed", "embed.norm", "head", "final.norm"}) need(w, name, &st);
  const auto& layers = config.at("layers").array;
  for (size_t i = 0; i < layers.size(); ++i) {
    const std::string p = "l" + std::to_string(i) + ".";
    const std::string& type = layers[i].at("type").as_string();
    std::vector<std::string> names = {"norm1", "shift", "mix.g", "mix.o"};
    if (type == "latent_attention") {
      for (const char* n : {"mix.dq", "mix.dq.norm", "mix.uq", "mix.dkv", "mix.dkv.norm", "mix.uk", "mix.uv", "mix.sink"})
        names.push_back(n);
    } else if (type == "lightning") {
      for (const char* n : {"mix.q", "mix.k", "mix.v", "mix.norm"}) names.push_back(n);
    } else {
      return base::error::FunctionNotImplement("layer " + std::to_string(i) + ": unknown mixer '" + type + "'");
    }
    if (present(layers[i], "mlp")) {
      const json::Value& mc = layers[i].at("mlp");
      names.push_back("norm2");
      if (mc.at("kind").as_string() == "dense") {
        for (const char* n : {"mlp.up", "mlp.down", "mlp.act"}) names.push_back(n);
      } else {
        names.push_back("mlp.router"), names.push_back("mlp.correction");
        for (int e = 0; e < get_int(mc.at("router"), "experts"); ++e)
          for (const char* n : {"up", "down"}) names.push_back("mlp.e" + std::to_string(e) + "." + n);
      }
    }
    for (const std::string& n : names) need(w, p + n, &st);
  }
  return st;
}

base::Status KikunexModel::build(const json::Value& config, const SafetensorsFile& w) {
  vocab_ = get_int(config, "vocab");
  width_ = get_int(config, "width");
  norm_eps_ = static_cast<float>(config.at("norm").at("eps").as_number());
  logit_scale_ = config.has("logit_scale") ? static_cast<float>(config.at("logit_scale").as_number()) : 1.0f;
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
    if (st = scalar_norm(w, p + "norm1", &L.pre_mixer); !st) return st;
    if (st = upload_f32(need(w, p + "shift", &st), width_, &L.shift); !st) return st;
    if (type == "latent_attention") {
      L.mixer_kind = KLLM_SEQ_MIXER_LATENT;
      if (st = build_latent(lc.at("mixer"), w, p + "mix.", &L.latent); !st) return st;
    } else if (type == "lightning") {
      L.mixer_kind = KLLM_SEQ_MIXER_LINEAR;
      if (st = build_lightning(lc.at("mixer"), w, p + "mix.", &L.linear); !st) return st;
    } else {
      return base::error::FunctionNotImplement("layer " + std::to_string(i) + ": unknown mixer '" + type + "'");
    }
    L.ff_kind = KLLM_SEQ_FF_NONE;
    if (present(lc, "mlp")) {
      const json::Value& mc = lc.at("mlp");
      const std::string& kind = mc.at("kind").as_string();
      if (st = scalar_norm(w, p + "norm2", &L.pre_ff); !st) return st;
      if (kind == "dense") {
        L.ff_kind = KLLM_SEQ_FF_DENSE;
        if (st = build_dense(mc, w, p + "mlp.", &L.dense); !st) return st;
      } else if (kind == "moe") {
        L.ff_kind = KLLM_SEQ_FF_MOE;
        if (st = build_moe(mc, w, p + "mlp.", &L.moe); !st) return st;
      } else {
        return base::error::FunctionNotImplement("layer " + std::to_string(i) + ": unknown feed-forward '" + kind + "'");
      }
    }
  }
  // the order of layer runs
  const int32_t n = static_cast<int32_t>(layers.size());
  int32_t start = 0, stop = 0, times = 1;
  if (present(config, "loop")) {
    const json::Value& lp = config.at("loop");
    start = get_int(lp, "start"), stop = get_int(lp, "stop"), times = get_int(lp, "times");
    if (start < 0 || stop < start || stop > n || times < 1) return base::error::ModelParseError("bad loop");
  }
  run_layer_.clear(), run_add_.clear(), run_embed_.clear();
  auto push = [&](int32_t layer, int32_t add, int32_t embed) {
    run_layer_.push_back(layer), run_add_.push_back(add), run_embed_.push_back(embed);
  };
  for (int32_t i = 0; i < start; ++i) push(i, -1, 0);
  if (stop > start)
    for (int32_t t = 0; t < times; ++t)
      for (int32_t i = start; i < stop; ++i) push(i, i == start ? t : -1, i == start && t > 0 ? 1 : 0);
  for (int32_t i = stop; i < n; ++i) push(i, -1, 0);
  if (stop > start) {
    if (st = upload_f32(need(w, "loop.step", &st), int64_t(times) * width_, &run_vectors_); !st) return st;
  }
  const StTensor *embed = need(w, "embed", &st), *head = need(w, "head", &st);
  if (!st) return st;
  if (!shaped(embed, vocab_, width_) || !shaped(head, vocab_, width_))
    return base::error::ModelParseError("embed / head do not fit vocab x width");
  if (st = upload_compute({embed}, width_, &embed_); !st) return st;
  if (st = upload_compute({head}, width_, &head_); !st) return st;
  if (st = scalar_norm(w, "embed.norm", &embed_norm_); !st) return st;
  return scalar_norm(w, "final.norm", &final_norm_);
}
}  // namespace model

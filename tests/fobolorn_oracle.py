"""A plain, slow restatement of the Fobolorn family in float64 torch: one function per mechanism, whole sequences at
once, no cache, no batching.  It shares nothing with the product path (C++ / CUDA); the tests compare the two.

Also here: a writer for model folders (config.json + model.safetensors with bf16 tensors) and a generator of small
random configurations and weights.
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np
import torch

F = torch.float64


# ---- mechanisms -------------------------------------------------------------------------------------------------------
def layer_norm(v, weight, bias, eps):
    mu = v.mean(-1, keepdim=True)
    var = ((v - mu) ** 2).mean(-1, keepdim=True)
    return (v - mu) / torch.sqrt(var + eps) * weight + bias


def unit_rms(v, weight, eps):
    return v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps) * weight


def query_temperature(positions, coef, every):
    return 1.0 + coef * torch.log(torch.floor((positions + 1) / every) + 1.0)


def gated_attention(h, tw, c, eps):
    """h [n, width]; tw: this mixer's tensors by short name; c: the mixer's config."""
    n = h.shape[0]
    nq, nkv, dk, dv = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    q = unit_rms((h @ tw["q"].T).reshape(n, nq, dk), tw["q.norm"], eps)
    k = unit_rms((h @ tw["k"].T).reshape(n, nkv, dk), tw["k.norm"], eps)
    v = (h @ tw["v"].T).reshape(n, nkv, dv)
    pos = torch.arange(n, dtype=F)
    if c.get("q_temp"):
        q = q * query_temperature(pos, c["q_temp"]["coef"], c["q_temp"]["every"])[:, None, None]
    gate = torch.sigmoid(h @ tw["g"].T)
    visible = pos[None, :] <= pos[:, None]
    group = nq // nkv
    heads = []
    for a in range(nq):
        s = (q[:, a] @ k[:, a // group].T) * c["scale"]
        s = torch.where(visible, s, torch.full_like(s, -math.inf))
        heads.append(torch.softmax(s, dim=-1) @ v[:, a // group] * gate[:, a:a + 1])
    return torch.cat(heads, dim=-1) @ tw["o"].T


def swiglu(h, gate, up, down):
    z = h @ gate.T
    return (z * torch.sigmoid(z) * (h @ up.T)) @ down.T


def route(h, router_w, top, scale):
    score = torch.softmax(h @ router_w.T, dim=-1)
    val, idx = torch.topk(score, top, dim=-1)
    return idx, val / (val.sum(-1, keepdim=True) + 1e-20) * scale


def mixture(h, tw, c):
    idx, wgt = route(h, tw["router"], c["router"]["top"], c["router"].get("scale", 1.0))
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(idx.shape[1]):
            e = int(idx[t, j])
            out[t] += wgt[t, j] * swiglu(h[t:t + 1], tw[f"e{e}.gate"], tw[f"e{e}.up"], tw[f"e{e}.down"])[0]
    if c.get("shared"):
        out = out + swiglu(h, tw["shared.gate"], tw["shared.up"], tw["shared.down"]) * torch.sigmoid(h @ tw["shared.sg"].T)
    return out


def layer_order(cfg):
    """[(layer index, pass number or None)]: the pass number is set on the first layer of each pass of the loop."""
    n = len(cfg["layers"])
    lp = cfg.get("loop")
    if not lp or lp["stop"] <= lp["start"]:
        return [(i, None) for i in range(n)]
    order = [(i, None) for i in range(lp["start"])]
    for t in range(lp["times"]):
        order += [(i, t if i == lp["start"] else None) for i in range(lp["start"], lp["stop"])]
    return order + [(i, None) for i in range(lp["stop"], n)]


def sub(weights, prefix):
    return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


def forward(cfg, weights, tokens, residuals=None):
    """Logits [n, vocab] of one whole sequence; `residuals` (a list) receives the stream after every layer run."""
    w = {k: v.to(F) for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.tensor(tokens)]
    for i, t in layer_order(cfg):
        if t is not None:
            x = x + w["loop.step"][t]
        c, p = cfg["layers"][i], f"l{i}."
        h = layer_norm(x, w[p + "norm1"], w[p + "norm1.b"], eps)
        y = gated_attention(h, sub(w, p + "mix."), c["mixer"], eps)
        x = x + layer_norm(y, w[p + "norm1b"], w[p + "norm1b.b"], eps)
        if c.get("mlp"):
            h = layer_norm(x, w[p + "norm2"], w[p + "norm2.b"], eps)
            y = mixture(h, sub(w, p + "mlp."), c["mlp"])
            x = x + layer_norm(y, w[p + "norm2b"], w[p + "norm2b.b"], eps)
        if residuals is not None:
            residuals.append(x.clone())
    return layer_norm(x, w["final.norm"], w["final.norm.b"], eps) @ w["head"].T


def greedy(cfg, weights, prompt, n_new):
    ids = list(prompt)
    out = []
    for _ in range(n_new):
        nxt = int(torch.argmax(forward(cfg, weights, ids)[-1]))
        out.append(nxt)
        ids.append(nxt)
    return out


# ---- model folders ------------------------------------------------------------------------------------------------------
def bf16_round(t):
    return t.to(torch.float32).to(torch.bfloat16).to(torch.float32)


def make_config(width=64, vocab=96, layers=2, heads=4, kv_heads=2, dim=16, vdim=24, experts=4, top=2, ff=32,
                shared_ff=48, loop=None, q_temp=(0.5, 8), scale=None, router_scale=1.5, mlp=True, eps=1e-5):
    def one(i):
        mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
                 "scale": scale if scale is not None else dim ** -0.5}
        if q_temp:
            mixer["q_temp"] = {"coef": q_temp[0], "every": q_temp[1]}
        ml = None
        has = mlp[i] if isinstance(mlp, (list, tuple)) else mlp
        if has:
            ml = {"kind": "moe", "router": {"experts": experts, "top": top, "scale": router_scale}, "expert": {"ff": ff}}
            if shared_ff:
                ml["shared"] = {"ff": shared_ff}
        return {"type": "attention", "mixer": mixer, "mlp": ml}
    cfg = {"architecture": "Fobolorn", "vocab": vocab, "width": width, "norm": {"eps": eps},
           "layers": [one(i) for i in range(layers)]}
    if loop:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return cfg


def make_weights(cfg, seed=0, sharp=1.0):
    """Random bf16-representable weights.  `sharp` multiplies the query norm weights: > 1 makes the softmax peaky, so
    that single keys (far ones too) carry the output."""
    g = torch.Generator().manual_seed(seed)
    W, V = cfg["width"], cfg["vocab"]

    def rnd(*shape, std=1.0):
        return bf16_round(torch.randn(*shape, generator=g) * std)
    w = {"embed": rnd(V, W), "head": rnd(V, W, std=W ** -0.5),
         "final.norm": bf16_round(1 + 0.1 * torch.randn(W, generator=g)), "final.norm.b": rnd(W, std=0.1)}
    if cfg.get("loop"):
        w["loop.step"] = rnd(cfg["loop"]["times"], W, std=0.5)
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        names = ["norm1", "norm1b"] + (["norm2", "norm2b"] if L.get("mlp") else [])
        for nm in names:
            w[p + nm] = bf16_round(1 + 0.1 * torch.randn(W, generator=g))
            w[p + nm + ".b"] = rnd(W, std=0.1)
        m = L["mixer"]
        w[p + "mix.q"] = rnd(m["heads"] * m["dim"], W, std=W ** -0.5)
        w[p + "mix.k"] = rnd(m["kv_heads"] * m["dim"], W, std=W ** -0.5)
        w[p + "mix.v"] = rnd(m["kv_heads"] * m["vdim"], W, std=W ** -0.5)
        w[p + "mix.g"] = rnd(m["heads"], W, std=W ** -0.5)
        w[p + "mix.o"] = rnd(W, m["heads"] * m["vdim"], std=(m["heads"] * m["vdim"]) ** -0.5)
        w[p + "mix.q.norm"] = bf16_round(sharp * (1 + 0.1 * torch.randn(m["dim"], generator=g)))
        w[p + "mix.k.norm"] = bf16_round(1 + 0.1 * torch.randn(m["dim"], generator=g))
        ml = L.get("mlp")
        if ml:
            ff = ml["expert"]["ff"]
            w[p + "mlp.router"] = rnd(ml["router"]["experts"], W, std=2 * W ** -0.5)
            for e in range(ml["router"]["experts"]):
                w[p + f"mlp.e{e}.gate"] = rnd(ff, W, std=W ** -0.5)
                w[p + f"mlp.e{e}.up"] = rnd(ff, W, std=W ** -0.5)
                w[p + f"mlp.e{e}.down"] = rnd(W, ff, std=ff ** -0.5)
            if ml.get("shared"):
                sf = ml["shared"]["ff"]
                w[p + "mlp.shared.gate"] = rnd(sf, W, std=W ** -0.5)
                w[p + "mlp.shared.up"] = rnd(sf, W, std=W ** -0.5)
                w[p + "mlp.shared.down"] = rnd(W, sf, std=sf ** -0.5)
                w[p + "mlp.shared.sg"] = rnd(1, W, std=W ** -0.5)
    return w


def write_model(folder, cfg, weights):
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(cfg))
    header, blobs, at = {}, [], 0
    for name, t in weights.items():
        u = t.to(torch.float32).contiguous().numpy().view(np.uint32)
        assert not (u & 0xffff).any(), f"{name} is not bf16-representable"
        raw = (u >> 16).astype("<u2").tobytes()
        header[name] = {"dtype": "BF16", "shape": list(t.shape), "data_offsets": [at, at + len(raw)]}
        blobs.append(raw)
        at += len(raw)
    head = json.dumps(header).encode()
    head += b" " * (-len(head) % 8)
    with open(folder / "model.safetensors", "wb") as f:
        f.write(struct.pack("<Q", len(head)) + head + b"".join(blobs))
    return folder

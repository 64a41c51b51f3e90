"""A slow float64 restatement of the Kikunex family, one function per mechanism.

It shares no code with the product path: numpy only, whole sequences, no cache and no state (every function sees the
complete sequence).  `weights` maps tensor names to float64 arrays; `config` is the parsed config.json.

    tokens --embed--> scalar RMS norm --> layer runs --> scalar RMS norm --> head * logit_scale

    layer:  x += mixer(shift(norm1(x)));  x += ff(norm2(x))            (ff optional)
    loop:   layers start..stop-1 run `times` times; before pass t > 0 the embedding output is added to x, and before
            every pass row t of 'loop.step'
"""
from __future__ import annotations

import math

import numpy as np


# ---- small pieces ------------------------------------------------------------------------------------------------------
def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) along the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def scalar_norm(x, g, eps):
    """RMS norm whose weight is one number."""
    assert np.ndim(g) == 0
    return rms_unit(x, eps) * float(g)


def vector_norm(x, w, eps):
    return rms_unit(x, eps) * w


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def softplus(z):
    return math.log1p(math.exp(z))


def silu(z):
    return z * sigmoid(z)


def token_shift(h, mu):
    """Row t becomes h[t] + (h[t-1] - h[t]) * mu, with zeros before the first row."""
    prev = np.vstack([np.zeros_like(h[:1]), h[:-1]])
    return h + (prev - h) * mu


def rotate(v, positions, dims, base):
    """Rotary positions on the first `dims` coordinates of v [T, ..., n]: coordinate i pairs with i + dims/2."""
    half = dims // 2
    freq = base ** (-2.0 * np.arange(half) / dims)
    ang = positions[:, None] * freq[None, :]                      # [T, half]
    shape = (v.shape[0],) + (1,) * (v.ndim - 2) + (half,)
    c, s = np.cos(ang).reshape(shape), np.sin(ang).reshape(shape)
    a, b = v[..., :half], v[..., half:dims]
    out = v.copy()
    out[..., :half] = a * c - b * s
    out[..., half:dims] = b * c + a * s
    return out


# ---- mixers -----------------------------------------------------------------------------------------------------------
def latent_attention(h, w, p, m, eps):
    """h [T, width]; w: weights; p: tensor prefix '<layer>.mix.'; m: the mixer's configuration."""
    T = h.shape[0]
    H, dn, dr, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = np.arange(T, dtype=np.float64)
    cq = vector_norm(h @ w[p + "dq"].T, w[p + "dq.norm"], eps)
    q = (cq @ w[p + "uq"].T).reshape(T, H, dn + dr)
    q_plain, q_rot = q[..., :dn], rotate(q[..., dn:], pos, m["rot"]["dims"], m["rot"]["base"])
    dkv = h @ w[p + "dkv"].T
    c = vector_norm(dkv[:, :rank], w[p + "dkv.norm"], eps)
    k_rot = rotate(dkv[:, rank:], pos, m["rot"]["dims"], m["rot"]["base"])     # [T, dr], one for all heads
    k_plain = (c @ w[p + "uk"].T).reshape(T, H, dn)
    v = (c @ w[p + "uv"].T).reshape(T, H, dv)
    gate = sigmoid(h @ w[p + "g"].T)                                            # [T, H]
    window = m["mask"]["size"] if m.get("mask") else T
    out = np.zeros((T, H, dv))
    for i in range(T):
        lo = max(0, i - window + 1)
        for hd in range(H):
            s = (k_plain[lo:i + 1, hd] @ q_plain[i, hd] + k_rot[lo:i + 1] @ q_rot[i, hd]) * m["scale"]
            sink = w[p + "sink"][hd]
            top = max(s.max(), sink)
            e = np.exp(s - top)
            out[i, hd] = (e @ v[lo:i + 1, hd]) / (e.sum() + math.exp(sink - top))
    out = out * gate[:, :, None]
    return out.reshape(T, H * dv) @ w[p + "o"].T


def lightning(h, w, p, m, eps):
    T = h.shape[0]
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ w[p + "q"].T).reshape(T, H, dk)
    k = silu(h @ w[p + "k"].T).reshape(T, H, dk)
    v = silu(h @ w[p + "v"].T).reshape(T, H, dv)
    out = np.zeros((T, H, dv))
    for hd in range(H):
        S = np.zeros((dk, dv))
        lam = m["decay"][hd]
        for t in range(T):
            S = lam * S + np.outer(k[t, hd], v[t, hd])
            out[t, hd] = S.T @ q[t, hd]
    o = vector_norm(out.reshape(T, H * dv), w[p + "norm"], eps) * sigmoid(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


# ---- feed-forward ------------------------------------------------------------------------------------------------------
def xielu(z, p, q):
    ap, aq = softplus(p), 0.5 + softplus(q)
    neg = np.minimum(z, 0.0)
    return np.where(z > 0, ap * z * z + 0.5 * z, aq * (np.exp(neg) - 1.0 - neg) + 0.5 * z)


def dense_ff(h, w, p):
    a = w[p + "act"]
    return xielu(h @ w[p + "up"].T, float(a[0]), float(a[1])) @ w[p + "down"].T


def route(h, w, p, r):
    """Returns (chosen experts [T, top], weights [T, top])."""
    s = sigmoid(h @ w[p + "router"].T)
    choice = s + w[p + "correction"]
    E, top = r["experts"], r["top"]
    groups = r.get("groups")
    if groups:
        size = E // groups["count"]
        per = choice.reshape(-1, groups["count"], size)
        gscore = np.sort(per, axis=-1)[..., -min(2, size):].sum(-1)            # [T, groups]
        kept = np.argsort(-gscore, axis=-1, kind="stable")[:, :groups["keep"]]
        allowed = np.zeros_like(gscore, dtype=bool)
        np.put_along_axis(allowed, kept, True, axis=-1)
        choice = np.where(np.repeat(allowed, size, axis=-1), choice, -np.inf)
    idx = np.argsort(-choice, axis=-1, kind="stable")[:, :top]
    return idx, np.take_along_axis(s, idx, axis=-1) * r["scale"]


def moe_ff(h, w, p, c):
    idx, wt = route(h, w, p, c["router"])
    out = np.zeros((h.shape[0], w[p + "e0.down"].shape[0]))
    for t in range(h.shape[0]):
        for e, g in zip(idx[t], wt[t]):
            z = np.maximum(w[f"{p}e{e}.up"] @ h[t], 0.0)
            out[t] += g * (w[f"{p}e{e}.down"] @ (z * z))
    return out


# ---- the model ----------------------------------------------------------------------------------------------------------
def layer_runs(config):
    """[(layer, pass number or None)]: pass number on the first layer of each pass of the loop."""
    n = len(config["layers"])
    lp = config.get("loop") or {"start": 0, "stop": 0, "times": 1}
    runs = [(i, None) for i in range(lp["start"])]
    for t in range(lp["times"]):
        runs += [(i, t if i == lp["start"] else None) for i in range(lp["start"], lp["stop"])]
    return runs + [(i, None) for i in range(lp["stop"], n)]


def forward(config, weights, tokens):
    """Returns (logits [T, vocab], residual stream after every layer run [runs, T, width])."""
    w, eps = weights, config["norm"]["eps"]
    x0 = scalar_norm(w["embed"][np.asarray(tokens)], w["embed.norm"], eps)
    x = x0.copy()
    trace = []
    for i, t in layer_runs(config):
        L = config["layers"][i]
        pre = f"l{i}."
        if t is not None:
            if t > 0:
                x = x + x0
            x = x + w["loop.step"][t]
        h = token_shift(scalar_norm(x, w[pre + "norm1"], eps), w[pre + "shift"])
        mixer = {"latent_attention": latent_attention, "lightning": lightning}[L["type"]]
        x = x + mixer(h, w, pre + "mix.", L["mixer"], eps)
        if L.get("mlp"):
            h2 = scalar_norm(x, w[pre + "norm2"], eps)
            ff = dense_ff(h2, w, pre + "mlp.") if L["mlp"]["kind"] == "dense" else moe_ff(h2, w, pre + "mlp.", L["mlp"])
            x = x + ff
        trace.append(x.copy())
    logits = scalar_norm(x, w["final.norm"], eps) @ w["head"].T * config["logit_scale"]
    return logits, np.stack(trace)


def greedy(config, weights, prompt, n_new):
    """Greedy continuation by recomputing the whole sequence (lowest index on ties)."""
    seq, out = list(prompt), []
    for _ in range(n_new):
        logits, _ = forward(config, weights, seq)
        out.append(int(np.argmax(logits[-1])))
        seq.append(out[-1])
    return out


# ---- small random models for the tests ------------------------------------------------------------------------------------
def latent_mixer(heads=4, dim=12, rot_dim=8, vdim=10, kv_rank=24, q_rank=20, window=16, base=10000.0, scale=None,
                 rot_dims=None):
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
                      "mask": {"size": window}, "rot": {"base": base, "dims": rot_dim if rot_dims is None else rot_dims},
                      "scale": (dim + rot_dim) ** -0.5 if scale is None else scale}}


def lightning_mixer(heads=3, dim=8, vdim=12, decay=None):
    decay = [math.exp(-1.0 / (2.0 + 7.0 * h)) for h in range(heads)] if decay is None else list(decay)
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay}}


def dense_mlp(ff=40):
    return {"kind": "dense", "ff": ff}


def moe_mlp(experts=6, top=2, ff=16, groups=(3, 2), scale=1.5):
    r = {"experts": experts, "top": top, "scale": scale}
    if groups:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "expert": {"ff": ff}, "router": r}


def make_config(width=48, vocab=61, layers=(), loop=None, eps=3e-6, logit_scale=0.7):
    """layers: [(mixer dict, mlp dict or None)]."""
    cfg = {"architecture": "Kikunex", "vocab": vocab, "width": width, "norm": {"eps": eps}, "logit_scale": logit_scale,
           "layers": [dict(m, mlp=f) for m, f in layers]}
    if loop:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return cfg


def bf16_round(a):
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    u = ((u + 0x7fff + ((u >> 16) & 1)) >> 16) << 16
    return u.astype(np.uint32).view(np.float32).astype(np.float64).reshape(np.shape(a))


def make_weights(cfg, seed=0, sharp=1.0):
    """Random bf16-representable weights.  `sharp` multiplies the query latent's norm weight: > 1 makes the softmax
    peaky, so that single keys (those at a window's edge too) carry the output."""
    rng = np.random.default_rng(seed)
    W, V = cfg["width"], cfg["vocab"]

    def rnd(*shape, std=1.0, mean=0.0):
        return bf16_round(mean + std * rng.standard_normal(shape))
    w = {"embed": rnd(V, W), "embed.norm": rnd(mean=1.0, std=0.1), "head": rnd(V, W, std=W ** -0.5),
         "final.norm": rnd(mean=1.0, std=0.1)}
    if cfg.get("loop"):
        w["loop.step"] = rnd(cfg["loop"]["times"], W, std=0.5)
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        w[p + "norm1"] = rnd(mean=1.0, std=0.1)
        w[p + "shift"] = bf16_round(rng.uniform(0.0, 1.0, W))
        H = m["heads"]
        if L["type"] == "latent_attention":
            w[p + "mix.dq"] = rnd(m["q_rank"], W, std=W ** -0.5)
            w[p + "mix.dq.norm"] = rnd(m["q_rank"], mean=1.0, std=0.1) * sharp
            w[p + "mix.dq.norm"] = bf16_round(w[p + "mix.dq.norm"])
            w[p + "mix.uq"] = rnd(H * (m["dim"] + m["rot_dim"]), m["q_rank"], std=m["q_rank"] ** -0.5)
            w[p + "mix.dkv"] = rnd(m["kv_rank"] + m["rot_dim"], W, std=W ** -0.5)
            w[p + "mix.dkv.norm"] = rnd(m["kv_rank"], mean=1.0, std=0.1)
            w[p + "mix.uk"] = rnd(H * m["dim"], m["kv_rank"], std=m["kv_rank"] ** -0.5)
            w[p + "mix.uv"] = rnd(H * m["vdim"], m["kv_rank"], std=m["kv_rank"] ** -0.5)
            w[p + "mix.sink"] = rnd(H)
            w[p + "mix.g"] = rnd(H, W, std=W ** -0.5)
            w[p + "mix.o"] = rnd(W, H * m["vdim"], std=(H * m["vdim"]) ** -0.5)
        else:
            for n, rows in (("q", H * m["dim"]), ("k", H * m["dim"]), ("v", H * m["vdim"]), ("g", H * m["vdim"])):
                w[p + "mix." + n] = rnd(rows, W, std=W ** -0.5)
            w[p + "mix.norm"] = rnd(H * m["vdim"], mean=1.0, std=0.1)
            w[p + "mix.o"] = rnd(W, H * m["vdim"], std=(H * m["vdim"]) ** -0.5)
        f = L.get("mlp")
        if not f:
            continue
        w[p + "norm2"] = rnd(mean=1.0, std=0.1)
        if f["kind"] == "dense":
            w[p + "mlp.up"] = rnd(f["ff"], W, std=W ** -0.5)
            w[p + "mlp.down"] = rnd(W, f["ff"], std=f["ff"] ** -0.5)
            w[p + "mlp.act"] = rnd(2, std=0.7)
        else:
            E, ff = f["router"]["experts"], f["expert"]["ff"]
            for e in range(E):
                w[f"{p}mlp.e{e}.up"] = rnd(ff, W, std=W ** -0.5)
                w[f"{p}mlp.e{e}.down"] = rnd(W, ff, std=ff ** -0.5)
            w[p + "mlp.router"] = rnd(E, W, std=2.0 * W ** -0.5)
            w[p + "mlp.correction"] = rnd(E, std=0.3)
    return w


def write_model(folder, cfg, weights):
    """config.json and model.safetensors (bfloat16) in `folder`."""
    import json
    import struct
    from pathlib import Path
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(cfg))
    header, blobs, at = {}, [], 0
    for name, a in weights.items():
        u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
        assert not (u & 0xffff).any(), f"{name} is not bf16-representable"
        raw = (u >> 16).astype("<u2").tobytes()
        header[name] = {"dtype": "BF16", "shape": list(np.shape(a)), "data_offsets": [at, at + len(raw)]}
        blobs.append(raw)
        at += len(raw)
    head = json.dumps(header).encode()
    head += b" " * (-len(head) % 8)
    with open(folder / "model.safetensors", "wb") as f:
        f.write(struct.pack("<Q", len(head)) + head + b"".join(blobs))
    return folder

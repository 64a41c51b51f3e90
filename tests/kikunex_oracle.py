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
    window = m["mask"]["size"]
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

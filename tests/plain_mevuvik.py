"""Mevuvik in float64 NumPy, one function per mechanism, token by token where that is the
plainest form.  It shares no code with the package: the tests compare the engine with it.

A model is a dict `cfg` (the nested config.json of the design) and a dict of float64 arrays
by tensor name.  `forward(cfg, w, tokens)` gives the logits of every position of one
sequence; `forward(..., layers_out=[])` also collects the residual stream after every layer
run (a layer inside the repeated stretch counts once per pass).

    start:   x = N(embed[token]) * g_embed
    layer:   x <- x + r * ls1 * mixer(N(x) * g1);  x <- x + r * ls2 * ff(N(x) * g2)
    repeat:  layers [start, stop) run `times` times; pass t begins with x <- x + step[t]
    output:  cap * tanh(head . (N(x) * g_final) / cap)

with N(x) = x / sqrt(mean(x^2) + eps), every g a single number, r = residual_mult.
"""
from __future__ import annotations

import math

import numpy as np


def rms(x, eps):
    return x / np.sqrt((x ** 2).mean(axis=-1, keepdims=True) + eps)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-np.clip(z, -700.0, 700.0)))


def log_sigmoid(z):
    return -np.logaddexp(0.0, -z)


def relu_squared(z):
    return np.maximum(z, 0.0) ** 2


def softmax(s):
    e = np.exp(s - s.max())
    return e / e.sum()


def rotate_half(x, p, base):
    """x [..., n]: dimension i turns with dimension i + n/2 by the angle p * base^(-2i/n)."""
    n = x.shape[-1]
    half = n // 2
    ang = p * base ** (-2.0 * np.arange(half) / n)
    c, s = np.cos(ang), np.sin(ang)
    u, v = x[..., :half], x[..., half:]
    return np.concatenate([u * c - v * s, v * c + u * s], axis=-1)


def latent_attention(h, m, t, eps):
    """h [T, W] -> [T, W].  Queries pass a normed latent; every token leaves a normed latent
    row c (keys and values are its projections) and one turned key part shared by all heads."""
    H, d, r, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    base = m["rot"]["base"]
    assert m["rot"]["dims"] == r
    T = h.shape[0]
    cq = rms(h @ t["dq"].T, eps) * t["dq.norm"]
    q = (cq @ t["uq"].T).reshape(T, H, d + r)
    kv = h @ t["dkv"].T
    c = rms(kv[:, :R], eps) * t["dkv.norm"]
    k_rot = np.stack([rotate_half(kv[p, R:], p, base) for p in range(T)])
    k = (c @ t["uk"].T).reshape(T, H, d)
    v = (c @ t["uv"].T).reshape(T, H, dv)
    out = np.zeros((T, H, dv))
    for i in range(T):
        for hh in range(H):
            q_rot = rotate_half(q[i, hh, d:], i, base)
            s = (k[:i + 1, hh] @ q[i, hh, :d] + k_rot[:i + 1] @ q_rot) * m["scale"]
            out[i, hh] = softmax(s) @ v[:i + 1, hh]
    return out.reshape(T, H * dv) @ t["o"].T


def gated_grouped_attention(h, m, t):
    """Grouped heads without positions; head j's result is multiplied by sigmoid(W_g h)_j."""
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = (h @ t["q"].T).reshape(T, H, d)
    k = (h @ t["k"].T).reshape(T, G, d)
    v = (h @ t["v"].T).reshape(T, G, dv)
    gate = sigmoid(h @ t["g"].T)                                  # [T, H]
    out = np.zeros((T, H, dv))
    for i in range(T):
        for hh in range(H):
            g = hh // (H // G)
            s = k[:i + 1, g] @ q[i, hh] * m["scale"]
            out[i, hh] = softmax(s) @ v[:i + 1, g] * gate[i, hh]
    return out.reshape(T, H * dv) @ t["o"].T


def matrix_memory(h, m, t, eps, state=None):
    """The matrix memory with exponential gates kept stable by a running maximum.  Per head:
    C [d, dv], n [d], mx (a number, 0 at the start).  Returns (output, state)."""
    H, d, dv, cap = m["heads"], m["dim"], m["vdim"], m["gate_cap"]
    T = h.shape[0]
    q = (h @ t["q"].T).reshape(T, H, d) * d ** -0.5
    k = (h @ t["k"].T).reshape(T, H, d)
    v = (h @ t["v"].T).reshape(T, H, dv)
    log_i = cap * np.tanh((h @ t["i"].T + t["i.b"]) / cap)          # [T, H]
    log_f = log_sigmoid(cap * np.tanh((h @ t["f"].T + t["f.b"]) / cap))
    if state is None:
        state = [(np.zeros((d, dv)), np.zeros(d), 0.0) for _ in range(H)]
    out = np.zeros((T, H, dv))
    for hh in range(H):
        C, n, mx = state[hh]
        for i in range(T):
            new = max(log_f[i, hh] + mx, log_i[i, hh])
            keep, take = math.exp(log_f[i, hh] + mx - new), math.exp(log_i[i, hh] - new)
            C = keep * C + take * np.outer(k[i, hh], v[i, hh])
            n = keep * n + take * k[i, hh]
            mx = new
            out[i, hh] = C.T @ q[i, hh] / (max(abs(n @ q[i, hh]), math.exp(-mx)) + 1e-6)
        state[hh] = (C, n, mx)
    y = rms(out, eps).reshape(T, H * dv) * t["norm"] * sigmoid(h @ t["g"].T)
    return y @ t["o"].T, state


def _sub(w, prefix):
    return {k[len(prefix):]: v for k, v in w.items() if k.startswith(prefix)}


def parallel_mixer(h, m, t, eps):
    left = gated_grouped_attention(h, m["left"], _sub(t, "left."))
    right, _ = matrix_memory(h, m["right"], _sub(t, "right."), eps)
    return m["left_scale"] * left + m["right_scale"] * right


def dense(h, t):
    return relu_squared(h @ t["up"].T) @ t["down"].T


def route(z, correction, top, scale):
    """Chosen experts and their weights for one token's router logits [E]: the choice looks at
    sigmoid(z) + correction, the weights are sigmoid(z) of the chosen, normalised, times scale."""
    s = sigmoid(z)
    chosen = np.argsort(-(s + correction), kind="stable")[:top]
    return chosen, s[chosen] / (s[chosen].sum() + 1e-20) * scale


def moe(h, mlp, t):
    r = mlp["router"]
    out = np.zeros_like(h)
    for i in range(h.shape[0]):
        chosen, weights = route(t["router"] @ h[i], t["correction"], r["top"], r["scale"])
        for e, wgt in zip(chosen, weights):
            out[i] += wgt * (t[f"e{e}.down"] @ relu_squared(t[f"e{e}.up"] @ h[i]))
    return out


def feed_forward(h, mlp, t):
    if mlp["kind"] == "dense":
        return dense(h, t)
    if mlp["kind"] == "moe":
        return moe(h, mlp, t)
    raise ValueError(mlp["kind"])


def layer(cfg, w, i, x):
    eps, r = cfg["norm"]["eps"], cfg["residual_mult"]
    p = f"l{i}."
    L = cfg["layers"][i]
    h = rms(x, eps) * w[p + "norm1"]
    if L["type"] == "latent_attention":
        y = latent_attention(h, L["mixer"], _sub(w, p + "mix."), eps)
    elif L["type"] == "parallel":
        y = parallel_mixer(h, L["mixer"], _sub(w, p + "mix."), eps)
    else:
        raise ValueError(L["type"])
    x = x + r * w[p + "ls1"] * y
    if L.get("mlp") is not None:
        h = rms(x, eps) * w[p + "norm2"]
        x = x + r * w[p + "ls2"] * feed_forward(h, L["mlp"], _sub(w, p + "mlp."))
    return x


def run_order(cfg):
    """[(layer, pass or None: the first layer of pass t adds step[t])]"""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    a, b, times = loop["start"], loop["stop"], loop["times"]
    order = [(i, None) for i in range(a)]
    for t in range(times):
        order += [(i, t if i == a else None) for i in range(a, b)]
    return order + [(i, None) for i in range(b, n)]


def forward(cfg, w, tokens, layers_out=None):
    eps = cfg["norm"]["eps"]
    x = rms(w["embed"][np.asarray(tokens)], eps) * w["embed.norm"]
    for i, t in run_order(cfg):
        if t is not None:
            x = x + w["loop.step"][t]
        x = layer(cfg, w, i, x)
        if layers_out is not None:
            layers_out.append(x.copy())
    h = rms(x, eps) * w["final.norm"]
    logits = h @ w["head"].T
    cap = cfg.get("logit_softcap")
    return cap * np.tanh(logits / cap) if cap else logits

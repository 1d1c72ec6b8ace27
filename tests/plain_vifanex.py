"""Vifanex in float64 NumPy, one function per mechanism, token by token where that is the
plainest form.  It shares no code with the package: the tests compare the engine with it.

A model is a dict `cfg` (the nested config.json of the design) and a dict of float64 arrays
by tensor name.  `forward(cfg, w, tokens)` gives the logits of every position of one
sequence; `forward(..., layers_out=[])` also collects the sum of the residual streams after
every layer.

    streams:  x_1 .. x_S = embedding * scale
    sublayer: u = sum_s a[s] x_s;  y = f(rms(u));  x_t <- sum_s M[s, t] x_s + b[t] y
    output:   cap * tanh(head . rms(sum_s x_s) / cap)
"""
from __future__ import annotations

import math

import numpy as np

GLU_ALPHA = 1.702
UNIT_EPS = 1e-6


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-np.clip(z, -700.0, 700.0)))


def softplus(z):
    return np.where(z > 30.0, z, np.log1p(np.exp(np.minimum(z, 30.0))))


def rms_norm(x, w, eps):
    return x / np.sqrt((x ** 2).mean(axis=-1, keepdims=True) + eps) * w


# ---- several residual streams ---------------------------------------------------------------

def streams_read(xs, a):
    """xs [S, T, W], a [S] -> what the sub-layer reads, [T, W]."""
    return sum(a[s] * xs[s] for s in range(xs.shape[0]))


def streams_write(xs, y, mix, b):
    """All streams at once from the old ones: x_t = sum_s mix[s, t] x_s + b[t] y."""
    S = xs.shape[0]
    return np.stack([sum(mix[s, t] * xs[s] for s in range(S)) + b[t] * y for t in range(S)])


# ---- the clamped gated feed-forward and the mixture -----------------------------------------

def glu_clamp(x, t, limit, bias):
    """x [W] -> [W]."""
    g = t["gate"] @ x + (t["gate.b"] if bias else 0.0)
    u = t["up"] @ x + (t["up.b"] if bias else 0.0)
    g = np.minimum(g, limit)
    u = np.clip(u, -limit, limit)
    y = t["down"] @ (g * sigmoid(GLU_ALPHA * g) * (u + 1.0))
    return y + (t["down.b"] if bias else 0.0)


def route(scores, top, groups, keep):
    """Chosen experts of one token's scores [E]: groups of neighbours, a group's score its
    largest member, experts of the `keep` best groups only."""
    E = scores.shape[0]
    size = E // groups
    best = [scores[g * size:(g + 1) * size].max() for g in range(groups)]
    kept = np.argsort(-np.asarray(best), kind="stable")[:keep]
    allowed = np.full(E, -np.inf)
    for g in kept:
        allowed[g * size:(g + 1) * size] = scores[g * size:(g + 1) * size]
    return np.argsort(-allowed, kind="stable")[:top]


def _sub(w, prefix):
    return {k[len(prefix):]: v for k, v in w.items() if k.startswith(prefix)}


def moe(h, mlp, t):
    r = mlp["router"]
    out = np.zeros_like(h)
    for i in range(h.shape[0]):
        z = t["router"] @ h[i]
        s = np.exp(z - z.max())
        s /= s.sum()
        groups = r.get("groups") or {"count": 1, "keep": 1}
        for e in route(s, r["top"], groups["count"], groups["keep"]):
            out[i] += s[e] * r.get("scale", 1.0) * glu_clamp(h[i], _sub(t, f"e{e}."),
                                                            mlp["expert"]["limit"], False)
        if mlp.get("shared") is not None:
            out[i] += glu_clamp(h[i], _sub(t, "shared."), mlp["shared"]["limit"], False)
    return out


# ---- attention --------------------------------------------------------------------------------

def rotation_frequencies(rot):
    dims = rot["dims"]
    f = np.array([rot["base"] ** (-2.0 * i / dims) for i in range(dims // 2)])
    sc = rot.get("scaling")
    if sc:
        out = []
        for fi in f:
            wavelength = 2.0 * math.pi / fi
            if wavelength < sc["original"] / sc["high"]:
                out.append(fi)
            elif wavelength > sc["original"] / sc["low"]:
                out.append(fi / sc["factor"])
            else:
                s = (sc["original"] / wavelength - sc["low"]) / (sc["high"] - sc["low"])
                out.append((1.0 - s) * fi / sc["factor"] + s * fi)
        f = np.array(out)
    return f


def rotate_pairs(x, p, freq):
    """One head's vector x at position p: pair (2i, 2i+1) turns by p * freq[i]."""
    y = x.copy()
    for i, fi in enumerate(freq):
        c, s = math.cos(p * fi), math.sin(p * fi)
        y[2 * i] = x[2 * i] * c - x[2 * i + 1] * s
        y[2 * i + 1] = x[2 * i + 1] * c + x[2 * i] * s
    return y


def attention(h, m, t, eps, first_values):
    """h [T, W] -> ([T, W], this layer's own values before mixing [T, G, dv])."""
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = rms_norm(h @ t["q"].T + t["q.b"], t["q.norm"], eps).reshape(T, H, d)
    k = rms_norm(h @ t["k"].T + t["k.b"], t["k.norm"], eps).reshape(T, G, d)
    v = (h @ t["v"].T + t["v.b"]).reshape(T, G, dv)
    own = v
    if m.get("rot"):
        f = rotation_frequencies(m["rot"])
        q = np.stack([[rotate_pairs(q[i, a], i, f) for a in range(H)] for i in range(T)])
        k = np.stack([[rotate_pairs(k[i, a], i, f) for a in range(G)] for i in range(T)])
    if m.get("v_mix") and first_values is not None:
        lam = float(t["vmix"])
        v = (1.0 - lam) * v + lam * first_values
    window = (m.get("mask") or {}).get("size")
    out = np.zeros((T, H, dv))
    for i in range(T):
        lo = 0 if window is None else max(0, i - window + 1)
        for a in range(H):
            g = a // (H // G)
            s = k[lo:i + 1, g] @ q[i, a] * m["scale"]
            e = np.exp(s - s.max())
            out[i, a] = (e / e.sum()) @ v[lo:i + 1, g]
    return out.reshape(T, H * dv) @ t["o"].T, own


# ---- the gated delta rule -----------------------------------------------------------------------

def conv_silu(x, filt):
    """x [T, C], filt [C, taps] (last column the current token's), zeros before the start."""
    T, taps = x.shape[0], filt.shape[1]
    y = np.zeros_like(x)
    for i in range(T):
        for j in range(taps):
            src = i - (taps - 1 - j)
            if src >= 0:
                y[i] += filt[:, j] * x[src]
    return y * sigmoid(y)


def unit(x):
    return x / np.sqrt((x ** 2).sum(axis=-1, keepdims=True) + UNIT_EPS)


def delta_step(S, q, k, v, beta, g):
    """One token of one head.  S [d, dv]; q, k, g [d]; v [dv].  Returns (S, o)."""
    S = g[:, None] * S
    u = beta * (v - S.T @ k)
    S = S + np.outer(k, u)
    return S, S.T @ q


def gated_delta(h, m, t, eps):
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = unit(conv_silu(h @ t["q"].T, t["q.conv"]).reshape(T, G, d)) * d ** -0.5
    k = unit(conv_silu(h @ t["k"].T, t["k.conv"]).reshape(T, G, d))
    v = conv_silu(h @ t["v"].T, t["v.conv"]).reshape(T, H, dv)
    beta = sigmoid(h @ t["b"].T)
    rate = np.exp(t["A_log"])[None, :, None]
    g = np.exp(-rate * softplus((h @ t["a1"].T) @ t["a2"].T + t["dt_bias"]).reshape(T, H, d))
    gate = sigmoid((h @ t["g1"].T) @ t["g2"].T).reshape(T, H, dv)
    o = np.zeros((T, H, dv))
    for a in range(H):
        S = np.zeros((d, dv))
        kv = a // (H // G)
        for i in range(T):
            S, o[i, a] = delta_step(S, q[i, kv], k[i, kv], v[i, a], beta[i, a], g[i, a])
    o = o / np.sqrt((o ** 2).mean(axis=-1, keepdims=True) + eps) * t["norm"] * gate
    return o.reshape(T, H * dv) @ t["o"].T


# ---- the model ------------------------------------------------------------------------------------

def forward(cfg, w, tokens, layers_out=None):
    eps = cfg["norm"]["eps"]
    x = w["embed"][np.asarray(tokens)] * (cfg.get("embedding") or {}).get("scale", 1.0)
    S = cfg.get("streams")
    xs = np.stack([x] * (S or 1))
    first_values = None

    def sublayer(xs, prefix, hc, f):
        if S is None:
            return xs + f(rms_norm(xs[0], w[prefix], eps))[None]
        y = f(rms_norm(streams_read(xs, w[hc + ".in"]), w[prefix], eps))
        return streams_write(xs, y, w[hc + ".mix"], w[hc + ".out"])

    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        m, t = layer["mixer"], _sub(w, p + "mix.")
        if layer["type"] == "attention":
            def mixer(h):
                nonlocal first_values
                y, own = attention(h, m, t, eps, first_values if m.get("v_mix") else None)
                if m.get("v_mix") and first_values is None:
                    first_values = own
                return y
        elif layer["type"] == "channel_delta":
            mixer = lambda h: gated_delta(h, m, t, eps)
        else:
            raise ValueError(layer["type"])
        xs = sublayer(xs, p + "norm1", p + "hc1", mixer)
        mlp = layer.get("mlp")
        if mlp is not None:
            tm = _sub(w, p + "mlp.")
            if mlp["kind"] == "dense":
                ff = lambda h: np.stack([glu_clamp(r, tm, mlp["limit"], True) for r in h])
            else:
                ff = lambda h: moe(h, mlp, tm)
            xs = sublayer(xs, p + "norm2", p + "hc2", ff)
        if layers_out is not None:
            layers_out.append(xs.sum(axis=0))
    logits = rms_norm(xs.sum(axis=0), w["final.norm"], eps) @ w["head"].T
    cap = cfg.get("logit_softcap")
    return cap * np.tanh(logits / cap) if cap else logits

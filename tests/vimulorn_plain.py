"""A plain, slow statement of the Vimulorn design in float64 numpy: one function per mechanism, token-by-token
where the design is recurrent, no cache (every call sees the whole sequence).  It is the oracle of the tests and
shares nothing with the product: the product's kernels, state manager and loader are compared against it."""
from __future__ import annotations

import math

import numpy as np


def f64(a):
    return np.asarray(a, np.float64)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def softplus(z):
    return np.logaddexp(0.0, z)


def silu(z):
    return z * sigmoid(z)


def dyt(x, p, name):
    """Dynamic tanh: no statistics, tanh(alpha x) w + b."""
    return np.tanh(f64(p[name + ".alpha"]) * x) * f64(p[name]) + f64(p[name + ".b"])


def rms(x, eps, w=None):
    y = x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)
    return y if w is None else y * f64(w)


def short_conv(u, w):
    """u [T, C], w [C, taps]; tap taps-1 multiplies the current token, zeros before the start."""
    T, taps = u.shape[0], w.shape[1]
    w = f64(w)
    y = np.zeros_like(u)
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                y[t] += w[:, j] * u[s]
    return y


def softmax_rows(s, extra=None):
    """Row-wise softmax over the finite entries of s; `extra` [rows] joins the denominator only."""
    m = s.max(-1, keepdims=True)
    if extra is not None:
        m = np.maximum(m, extra[:, None])
    e = np.exp(s - m)
    d = e.sum(-1, keepdims=True)
    if extra is not None:
        d = d + np.exp(extra[:, None] - m)
    return e / d


def latent_attention(h, p, pre, mx, eps):
    T = h.shape[0]
    H, D, Dv = mx["heads"], mx["dim"], mx["vdim"]
    cq = rms(h @ f64(p[pre + "dq"]).T, eps, p[pre + "dq.norm"])
    q = (cq @ f64(p[pre + "uq"]).T).reshape(T, H, D)
    c = rms(h @ f64(p[pre + "dkv"]).T, eps, p[pre + "dkv.norm"])
    k = (c @ f64(p[pre + "uk"]).T).reshape(T, H, D)
    v = (c @ f64(p[pre + "uv"]).T).reshape(T, H, Dv)
    gate = sigmoid(h @ f64(p[pre + "g"]).T)                      # [T, H]
    out = np.zeros((T, H, Dv))
    causal = np.tril(np.ones((T, T), bool))
    for a in range(H):
        s = (q[:, a] @ k[:, a].T) * mx["scale"]
        s = np.where(causal, s, -np.inf)
        out[:, a] = softmax_rows(s) @ v[:, a]
    out = out * gate[:, :, None]
    return out.reshape(T, H * Dv) @ f64(p[pre + "o"]).T


def channel_delta(h, p, pre, mx, eps):
    T = h.shape[0]
    H, G, D, Dv = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
    q = silu(short_conv(h @ f64(p[pre + "q"]).T, p[pre + "q.conv"])).reshape(T, G, D)
    k = silu(short_conv(h @ f64(p[pre + "k"]).T, p[pre + "k.conv"])).reshape(T, G, D)
    v = silu(short_conv(h @ f64(p[pre + "v"]).T, p[pre + "v.conv"])).reshape(T, H, Dv)
    q = q / np.sqrt((q * q).sum(-1, keepdims=True) + 1e-6) * D ** -0.5
    k = k / np.sqrt((k * k).sum(-1, keepdims=True) + 1e-6)
    beta = sigmoid(h @ f64(p[pre + "b"]).T)                      # [T, H]
    dt = softplus((h @ f64(p[pre + "a1"]).T) @ f64(p[pre + "a2"]).T + f64(p[pre + "dt_bias"])).reshape(T, H, D)
    decay = np.exp(-np.exp(f64(p[pre + "A_log"]))[None, :, None] * dt)
    gate = sigmoid((h @ f64(p[pre + "g1"]).T) @ f64(p[pre + "g2"]).T).reshape(T, H, Dv)
    out = np.zeros((T, H, Dv))
    rep = H // G
    for a in range(H):
        S = np.zeros((D, Dv))
        for t in range(T):
            kk, qq = k[t, a // rep], q[t, a // rep]
            S = decay[t, a][:, None] * S
            u = beta[t, a] * (v[t, a] - S.T @ kk)
            S = S + np.outer(kk, u)
            out[t, a] = S.T @ qq
    out = rms(out, eps, p[pre + "norm"]) * gate
    return out.reshape(T, H * Dv) @ f64(p[pre + "o"]).T


def window_attention(h, p, pre, mx, eps):
    T = h.shape[0]
    H, G, D, Dv, W = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"], mx["mask"]["size"]
    q = short_conv(h @ f64(p[pre + "q"]).T, p[pre + "q.conv"]).reshape(T, H, D)
    k = short_conv(h @ f64(p[pre + "k"]).T, p[pre + "k.conv"]).reshape(T, G, D)
    v = short_conv(h @ f64(p[pre + "v"]).T, p[pre + "v.conv"]).reshape(T, G, Dv)
    q, k = rms(q, eps), rms(k, eps)
    i, j = np.arange(T)[:, None], np.arange(T)[None, :]
    seen = (i - j >= 0) & (i - j < W)
    sink = f64(p[pre + "sink"])
    out = np.zeros((T, H, Dv))
    rep = H // G
    for a in range(H):
        s = (q[:, a] @ k[:, a // rep].T) * mx["scale"]
        s = np.where(seen, s, -np.inf)
        out[:, a] = softmax_rows(s, np.full(T, sink[a])) @ v[:, a // rep]
    return out.reshape(T, H * Dv) @ f64(p[pre + "o"]).T


def dense_ff(h, p, pre, ml):
    lim = ml["limit"]
    g = np.minimum(h @ f64(p[pre + "gate"]).T, lim)
    u = np.clip(h @ f64(p[pre + "up"]).T, -lim, lim)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ f64(p[pre + "down"]).T


MIXERS = {"latent_attention": latent_attention, "channel_delta": channel_delta, "attention": window_attention}


def layer_runs(cfg):
    """Indices of the layers in the order they run (the looped span repeated)."""
    n = len(cfg["layers"])
    lp = cfg.get("loop") or {"start": 0, "stop": 0, "times": 1}
    runs, first = [], []
    for r in range(lp["times"]):
        for i in range(lp["start"], lp["stop"]):
            runs.append(i)
            first.append(r > 0 and i == lp["start"])
    head = list(range(0, lp["start"]))
    tail = list(range(lp["stop"], n))
    return head + runs + tail, [False] * len(head) + first + [False] * len(tail)


def forward(cfg, p, tokens, trace=None):
    """Logits [T, vocab] of one sequence; `trace` (a list) receives the residual stream after every layer run."""
    eps = cfg["norm"]["eps"]
    x0 = f64(p["embed"])[np.asarray(tokens)]
    x = x0.copy()
    order, readd = layer_runs(cfg)
    for i, again in zip(order, readd):
        if again:
            x = x + x0
        L = cfg["layers"][i]
        pre = "l%d." % i
        y = MIXERS[L["type"]](dyt(x, p, pre + "norm1"), p, pre + "mix.", L["mixer"], eps)
        x = x + dyt(y, p, pre + "norm1b")
        if L.get("mlp"):
            y = dense_ff(dyt(x, p, pre + "norm2"), p, pre + "mlp.", L["mlp"])
            x = x + dyt(y, p, pre + "norm2b")
        if trace is not None:
            trace.append(x.copy())
    return dyt(x, p, "final.norm") @ f64(p["head"]).T

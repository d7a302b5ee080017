"""Plain float64 statement of the Bovinex design, one function per mechanism, token loops and no cache: the slow oracle
the runtime is compared with.  It shares no code with calm_b200 (numpy only; tensors come in as float64 arrays).

Notation: x [T, width] is one sequence's residual stream, h = norm(x) the input every sublayer of a layer reads,
p the position of a token (0 for the first)."""
from __future__ import annotations

import math
from typing import Dict, List

import numpy as np


def rms_norm(x: np.ndarray, w: np.ndarray, eps: float, around_zero: bool) -> np.ndarray:
    """x / sqrt(mean(x^2) + eps) times w, or times (1 + w) when the checkpoint keeps the weight as its offset from one."""
    r = x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)
    return r * (1.0 + w) if around_zero else r * w


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def yarn_frequencies(dims: int, base: float, sc: dict | None):
    """Per pair i < dims/2: the angle step f_i, and the factor on cos and sin."""
    half = dims // 2
    f = np.array([base ** (-2.0 * i / dims) for i in range(half)])
    if not sc:
        return f, 1.0
    factor, orig = float(sc["factor"]), float(sc["original"])

    def where(turns):
        return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(where(float(sc["fast"]))), 0)
    hi = min(math.ceil(where(float(sc["slow"]))), dims - 1)
    ramp = np.clip((np.arange(half) - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(v: np.ndarray, pos: np.ndarray, rot: dict) -> np.ndarray:
    """v [T, heads, dim]: the first rot.dims channels of every head turn by position, channel i with channel i + dims/2."""
    dims = int(rot["dims"])
    f, mag = yarn_frequencies(dims, float(rot["base"]), rot.get("scaling"))
    ang = pos[:, None].astype(np.float64) * f[None, :]
    c, s = (np.cos(ang) * mag)[:, None, :], (np.sin(ang) * mag)[:, None, :]
    half = dims // 2
    a, b = v[..., :half], v[..., half:dims]
    out = v.copy()
    out[..., :half] = a * c - b * s
    out[..., half:dims] = b * c + a * s
    return out


def visible(i: int, j: int, size: int, keep_first: int) -> bool:
    return j <= i and (i - j < size or j < keep_first)


def attention_mixer(h: np.ndarray, W: Dict[str, np.ndarray], mx: dict, eps: float) -> np.ndarray:
    """Grouped-query attention: biased projections, one RMS norm over the whole q (and k) projection, partial rotation,
    a sliding window that keeps the first tokens, a sigmoid gate on the concatenated heads."""
    T = h.shape[0]
    H, G, D, Dv = int(mx["heads"]), int(mx["kv_heads"]), int(mx["dim"]), int(mx["vdim"])
    q = h @ W["q"].T + W["q.b"]
    k = h @ W["k"].T + W["k.b"]
    v = h @ W["v"].T + W["v.b"]
    q = rms_norm(q, W["q.norm"], eps, False).reshape(T, H, D)
    k = rms_norm(k, W["k.norm"], eps, False).reshape(T, G, D)
    v = v.reshape(T, G, Dv)
    pos = np.arange(T)
    if mx.get("rot"):
        q, k = rotate(q, pos, mx["rot"]), rotate(k, pos, mx["rot"])
    mask = mx.get("mask") or {}
    size, keep = int(mask.get("size", 0)) or (1 << 60), int(mask.get("keep_first", 0))
    out = np.zeros((T, H, Dv))
    for i in range(T):
        js = [j for j in range(i + 1) if visible(i, j, size, keep)]
        for hd in range(H):
            g = hd // (H // G)
            s = np.array([q[i, hd] @ k[j, g] for j in js]) * float(mx["scale"])
            p = np.exp(s - s.max())
            p /= p.sum()
            out[i, hd] = sum(pj * v[j, g] for pj, j in zip(p, js))
    gate = sigmoid(h @ W["g"].T)
    return (out.reshape(T, H * Dv) * gate) @ W["o"].T


def gla_mixer(h: np.ndarray, W: Dict[str, np.ndarray], mx: dict, eps: float, state: np.ndarray | None = None):
    """Gated linear attention: per head S <- diag(alpha) S + k v^T, o = S^T q, with one decay per key channel."""
    T = h.shape[0]
    H, D, Dv = int(mx["heads"]), int(mx["dim"]), int(mx["vdim"])
    q = (h @ W["q"].T).reshape(T, H, D) * D ** -0.5
    k = (h @ W["k"].T).reshape(T, H, D)
    v = (h @ W["v"].T).reshape(T, H, Dv)
    z = (h @ W["a1"].T) @ W["a2"].T + W["a2.b"]
    alpha = (sigmoid(z) ** (1.0 / float(mx["tau"]))).reshape(T, H, D)
    S = np.zeros((H, D, Dv)) if state is None else state.copy()
    o = np.zeros((T, H, Dv))
    for t in range(T):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = np.einsum("hdv,hd->hv", S, q[t])
    o = rms_norm(o, W["norm"], eps, False).reshape(T, H * Dv)
    return (o * silu(h @ W["g"].T)) @ W["o"].T, S


def dense_ff(h: np.ndarray, W: Dict[str, np.ndarray]) -> np.ndarray:
    return np.maximum(h @ W["up"].T, 0.0) ** 2 @ W["down"].T


def route(h: np.ndarray, W: Dict[str, np.ndarray], top: int):
    """Per token: which `top` experts score highest at the router, and their mixing weights (a softmax restricted to those scores)."""
    z = h @ W["router"].T + W["router.b"]
    idx = np.argsort(-z, axis=-1, kind="stable")[:, :top]
    zs = np.take_along_axis(z, idx, -1)
    p = np.exp(zs - zs.max(-1, keepdims=True))
    return idx, p / p.sum(-1, keepdims=True)


def moe_ff(h: np.ndarray, W: Dict[str, np.ndarray], ml: dict) -> np.ndarray:
    top = int(ml["router"]["top"])
    idx, wts = route(h, W, top)
    out = np.zeros((h.shape[0], W["e0.down"].shape[0]))
    for t in range(h.shape[0]):
        for e, w in zip(idx[t], wts[t]):
            a = silu(W[f"e{e}.gate"] @ h[t]) * (W[f"e{e}.up"] @ h[t])
            out[t] += w * (W[f"e{e}.down"] @ a)
    return out


def sub(tensors: Dict[str, np.ndarray], prefix: str) -> Dict[str, np.ndarray]:
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def forward(cfg: dict, tensors: Dict[str, np.ndarray], tokens: List[int], layers_out: list | None = None) -> np.ndarray:
    """Logits [T, vocab] of one sequence fed whole; layers_out collects the residual stream after every layer."""
    eps = float(cfg["norm"]["eps"])
    x = tensors["embed"][np.asarray(tokens)] * float(cfg["embedding"]["scale"])
    for i, lc in enumerate(cfg["layers"]):
        h = rms_norm(x, tensors[f"l{i}.norm1"], eps, True)
        Wm = sub(tensors, f"l{i}.mix.")
        if lc["type"] == "attention":
            y = attention_mixer(h, Wm, lc["mixer"], eps)
        elif lc["type"] == "gla":
            y, _ = gla_mixer(h, Wm, lc["mixer"], eps)
        else:
            raise ValueError(lc["type"])
        ml = lc.get("mlp")
        if ml:
            Wf = sub(tensors, f"l{i}.mlp.")
            y = y + (dense_ff(h, Wf) if ml["kind"] == "dense" else moe_ff(h, Wf, ml))
        x = x + y
        if layers_out is not None:
            layers_out.append(x.copy())
    return rms_norm(x, tensors["final.norm"], eps, True) @ tensors["head"].T

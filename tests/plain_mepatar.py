"""Mepatar, stated plainly: dense numpy in 64-bit, one function per mechanism,
whole sequences at once, token-by-token loops for the recurrences, no cache
and no kernels.  Shares nothing with the package; the tests hold the
package's steps to this.

Notation: T tokens, W width, weights are stored [out, in] and applied as
y = x @ w.T.  ``w`` maps tensor names to float64 arrays; ``cfg`` is the
config.json dictionary.
"""
from __future__ import annotations

import json
import struct

import numpy as np


def read_safetensors(path) -> dict:
    """name -> float64 array (integers stay integers)."""
    raw = open(path, "rb").read()
    n = struct.unpack("<Q", raw[:8])[0]
    header = json.loads(raw[8:8 + n])
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        lo, hi = meta["data_offsets"]
        buf = raw[8 + n + lo:8 + n + hi]
        if meta["dtype"] == "BF16":
            a = (np.frombuffer(buf, dtype="<u2").astype(np.uint32) << 16).view(np.float32).astype(np.float64)
        elif meta["dtype"] == "F32":
            a = np.frombuffer(buf, dtype="<f4").astype(np.float64)
        elif meta["dtype"] == "I32":
            a = np.frombuffer(buf, dtype="<i4")
        else:
            raise ValueError(f"{name}: dtype {meta['dtype']}")
        out[name] = a.reshape(meta["shape"])
    return out


# ---- small pieces ---------------------------------------------------------------------------------
def unit_rms(x, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(np.sqrt(2.0 / np.pi) * (z + 0.044715 * z ** 3)))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.log1p(np.exp(-np.abs(z))) + np.maximum(z, 0.0)


def group_norm(x, weight, groups, eps):
    """x [T, W] cut into ``groups`` equal consecutive parts, each divided by its own root mean square."""
    T, W = x.shape
    parts = x.reshape(T, groups, W // groups)
    return unit_rms(parts, eps).reshape(T, W) * weight


def causal_conv(x, taps):
    """x [T, C], taps [C, K] with the last column the current token's: y_t = sum_j taps[:, j] x_(t - K + 1 + j)."""
    T, C = x.shape
    K = taps.shape[1]
    padded = np.concatenate([np.zeros((K - 1, C)), x], axis=0)
    y = np.zeros_like(x)
    for j in range(K):
        y += padded[j:j + T] * taps[:, j][None, :]
    return y


def rotary_angles(pos, dims, base):
    i = np.arange(dims // 2, dtype=np.float64)
    return np.asarray(pos, dtype=np.float64)[:, None] * (float(base) ** (-2.0 * i / dims))[None, :]


def rotate(x, pos, dims, base, layout):
    """x [T, heads, d]: the first ``dims`` numbers of every head rotated in pairs, (i, i + dims/2) for layout
    "half" and (2i, 2i + 1) for "interleaved"; (u, v) -> (u cos a - v sin a, v cos a + u sin a)."""
    out = x.copy()
    if dims == 0:
        return out
    a = rotary_angles(pos, dims, base)
    c, s = np.cos(a)[:, None, :], np.sin(a)[:, None, :]
    if layout == "half":
        u, v = x[..., :dims // 2], x[..., dims // 2:dims]
        out[..., :dims // 2] = u * c - v * s
        out[..., dims // 2:dims] = v * c + u * s
    elif layout == "interleaved":
        u, v = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = u * c - v * s
        out[..., 1:dims:2] = v * c + u * s
    else:
        raise ValueError(layout)
    return out


# ---- mixers -----------------------------------------------------------------------------------------
def retention(h, w, p, m, eps):
    """Linear attention with one fixed decay per head, no softmax and no denominator."""
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    pos = np.arange(T)
    q = (h @ w[p + "q"].T).reshape(T, H, d)
    k = (h @ w[p + "k"].T).reshape(T, H, d)
    v = (h @ w[p + "v"].T).reshape(T, H, dv)
    rot = m.get("rot") or dict(dims=0, base=10000.0)
    q = rotate(q, pos, rot["dims"], rot["base"], "half")
    k = rotate(k, pos, rot["dims"], rot["base"], "half") * d ** -0.5
    o = np.zeros((T, H, dv))
    for a in range(H):
        S = np.zeros((d, dv))
        for t in range(T):
            S = m["decay"][a] * S + np.outer(k[t, a], v[t, a])
            o[t, a] = S.T @ q[t, a]
    o = unit_rms(o, eps).reshape(T, H * dv) * silu(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


def visible(i, j, size, keep_first):
    return j <= i and (i - j < size or j < keep_first)


def attention(h, w, p, m, eps):
    """Grouped-query softmax attention with biases, a norm on q and k, interleaved partial rotation, a number per
    head on the scores, and a sliding window that keeps the first tokens."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = np.arange(T)
    q = (h @ w[p + "q"].T + w[p + "q.b"]).reshape(T, H, d)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).reshape(T, G, d)
    v = (h @ w[p + "v"].T + w[p + "v.b"]).reshape(T, G, dv)
    q = unit_rms(q, eps) * w[p + "q.norm"]
    k = unit_rms(k, eps) * w[p + "k.norm"]
    rot = m.get("rot") or dict(dims=0, base=10000.0)
    q = rotate(q, pos, rot["dims"], rot["base"], "interleaved")
    k = rotate(k, pos, rot["dims"], rot["base"], "interleaved")
    mask = m.get("mask")
    size = mask["size"] if mask else T + 1
    keep = mask.get("keep_first", 0) if mask else 0
    see = np.array([[visible(i, j, size, keep) for j in range(T)] for i in range(T)])
    out = np.zeros((T, H, dv))
    for a in range(H):
        g = a // (H // G)
        s = (q[:, a] @ k[:, g].T) * m["scale"] * w[p + "temp"][a]
        s = np.where(see, s, -np.inf)
        s = np.exp(s - s.max(axis=1, keepdims=True))
        out[:, a] = (s / s.sum(axis=1, keepdims=True)) @ v[:, g]
    return out.reshape(T, H * dv) @ w[p + "o"].T + w[p + "o.b"]


def delta(h, w, p, m, eps):
    """Gated delta rule."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(causal_conv(h @ w[p + "q"].T, w[p + "q.conv"])).reshape(T, G, d)
    k = silu(causal_conv(h @ w[p + "k"].T, w[p + "k.conv"])).reshape(T, G, d)
    v = silu(causal_conv(h @ w[p + "v"].T, w[p + "v.conv"])).reshape(T, H, dv)
    q = q / np.sqrt((q * q).sum(-1, keepdims=True) + 1e-6) * d ** -0.5
    k = k / np.sqrt((k * k).sum(-1, keepdims=True) + 1e-6)
    beta = sigmoid(h @ w[p + "b"].T)                                             # [T, H]
    g = np.exp(-np.exp(w[p + "A_log"]) * softplus(h @ w[p + "a"].T + w[p + "dt_bias"]))   # [T, H]
    o = np.zeros((T, H, dv))
    for a in range(H):
        c = a // (H // G)
        S = np.zeros((d, dv))
        for t in range(T):
            S = g[t, a] * S
            u = beta[t, a] * (v[t, a] - S.T @ k[t, c])
            S = S + np.outer(k[t, c], u)
            o[t, a] = S.T @ q[t, c]
    o = unit_rms(o, eps) * w[p + "norm"]
    o = o.reshape(T, H * dv) * silu(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


MIXERS = {"retention": retention, "attention": attention, "delta": delta}


# ---- feed-forwards ----------------------------------------------------------------------------------
def dense_ff(h, w, p):
    return (gelu_tanh(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def expert(h, w, p, limit):
    g = np.minimum(h @ w[p + "gate"].T, limit)
    u = np.clip(h @ w[p + "up"].T, -limit, limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].T


def router_scores(h, w, p):
    z = h @ w[p + "router"].T
    e = np.exp(z - z.max(axis=-1, keepdims=True))
    return e / e.sum(axis=-1, keepdims=True)


def moe_ff(h, w, p, mlp, margins=None):
    E, top, limit = mlp["router"]["experts"], mlp["router"]["top"], mlp["expert"]["limit"]
    s = router_scores(h, w, p)
    out = np.zeros((h.shape[0], w[p + "e0.down"].shape[0]))
    order = np.argsort(-s, axis=-1, kind="stable")
    if margins is not None and top < E:
        rows = np.arange(h.shape[0])
        margins.append((s[rows, order[:, top - 1]] - s[rows, order[:, top]]) / s[rows, order[:, top - 1]])
    for e in range(E):
        rows = np.nonzero((order[:, :top] == e).any(axis=1))[0]
        if rows.size:
            out[rows] += s[rows, e][:, None] * expert(h[rows], w, f"{p}e{e}.", limit)
    return out


# ---- the model --------------------------------------------------------------------------------------
def layer(x, w, cfg, i, margins=None):
    L = cfg["layers"][i]
    p = f"l{i}."
    eps, groups = cfg["norm"]["eps"], cfg["norm"].get("groups", 1)
    h = group_norm(x, w[p + "norm1"], groups, eps)
    if (cfg.get("canon") or {}).get("taps"):
        h = h + causal_conv(h, w[p + "canon1"])
    y = MIXERS[L["type"]](h, w, p + "mix.", L["mixer"], eps)
    mlp = L.get("mlp")
    if mlp is not None:
        f = group_norm(x, w[p + "norm2"], groups, eps)
        y = y + (dense_ff(f, w, p + "mlp.") if mlp["kind"] == "dense" else moe_ff(f, w, p + "mlp.", mlp, margins))
    return x + y


def forward(tokens, w, cfg, keep_layers=False, margins=None):
    """Logits [T, vocab] of one sequence (and the residual stream after every layer, if asked)."""
    x = w["embed"][np.asarray(tokens)] * (cfg.get("embedding") or {}).get("scale", 1.0)
    after = []
    for i in range(len(cfg["layers"])):
        x = layer(x, w, cfg, i, margins)
        if keep_layers:
            after.append(x.copy())
    logits = group_norm(x, w["final.norm"], cfg["norm"].get("groups", 1), cfg["norm"]["eps"]) @ w["head"].T
    return (logits, np.stack(after)) if keep_layers else logits

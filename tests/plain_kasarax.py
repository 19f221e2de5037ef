"""Kasarax, stated plainly: dense numpy in 64-bit, one function per mechanism,
whole sequences at once, token-by-token loops for the recurrence, no cache
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


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def one_plus_norm(x, weight, eps):
    """RMS norm whose stored weight sits around zero: unit_rms(x) (1 + weight)."""
    return unit_rms(x, eps) * (1.0 + weight)


def plain_norm(x, weight, eps):
    return unit_rms(x, eps) * weight


def causal_conv(x, taps):
    """x [T, C], taps [C, K] with the last column the current token's: y_t = sum_j taps[:, j] x_(t - K + 1 + j)."""
    T, C = x.shape
    K = taps.shape[1]
    padded = np.concatenate([np.zeros((K - 1, C)), x], axis=0)
    y = np.zeros_like(x)
    for j in range(K):
        y += padded[j:j + T] * taps[:, j][None, :]
    return y


def rotate_interleaved(x, pos, dims, base):
    """x [T, heads, d]: numbers (2i, 2i + 1), i < dims / 2, of every head turn by pos * base^(-2i / dims)."""
    out = x.copy()
    i = np.arange(dims // 2)
    a = np.asarray(pos, dtype=np.float64)[:, None] * base ** (-2.0 * i / dims)[None, :]       # [T, dims / 2]
    c, s = np.cos(a)[:, None, :], np.sin(a)[:, None, :]
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def query_temperature(pos, coef, every):
    """The factor on the query at position p: 1 + coef ln(floor((p + 1) / every) + 1)."""
    p = np.asarray(pos, dtype=np.int64)
    return 1.0 + coef * np.log((p + 1) // every + 1.0)


def sink_softmax_attention(q, k, v, scale, sink):
    """q [T, H, d], k [T, G, d], v [T, G, dv]; causal; the softmax's denominator has one more term exp(sink[h])
    (``sink`` [H]) that has neither key nor value.  Returns [T, H, dv]."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = np.zeros((T, H, v.shape[2]))
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale                                                    # [T, T]
        s = np.where(np.tril(np.ones((T, T), dtype=bool)), s, -np.inf)
        m = np.maximum(s.max(axis=1, keepdims=True), sink[h])
        e = np.exp(s - m)
        out[:, h] = (e @ v[:, g]) / (e.sum(axis=1, keepdims=True) + np.exp(sink[h] - m))
    return out


# ---- mixers -----------------------------------------------------------------------------------------
def gated_attention(h, w, p, m, pos):
    """Mixer 'attention': biased projections, no rotation, a query factor that grows with the logarithm of the
    position, one added to the softmax's denominator, a sigmoid gate per head on the heads' outputs."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T + w[p + "q.b"]).reshape(T, H, d)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).reshape(T, G, d)
    v = (h @ w[p + "v"].T + w[p + "v.b"]).reshape(T, G, dv)
    if m.get("q_temp"):
        q = q * query_temperature(pos, m["q_temp"]["coef"], m["q_temp"]["every"])[:, None, None]
    o = sink_softmax_attention(q, k, v, m["scale"], np.zeros(H))
    o = o * sigmoid(h @ w[p + "g"].T)[:, :, None]
    return o.reshape(T, H * dv) @ w[p + "o"].T + w[p + "o.b"]


def conv_attention(h, w, p, m, pos, eps):
    """Left half of mixer 'parallel': projections, a short causal convolution on each, RMS norm over the whole of q
    and of k, interleaved rotation of part of each head, softmax with a learned sink per head."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q, k, v = h @ w[p + "q"].T, h @ w[p + "k"].T, h @ w[p + "v"].T
    if m.get("conv"):
        q, k, v = causal_conv(q, w[p + "q.conv"]), causal_conv(k, w[p + "k.conv"]), causal_conv(v, w[p + "v.conv"])
    q = plain_norm(q, w[p + "q.norm"], eps).reshape(T, H, d)
    k = plain_norm(k, w[p + "k.norm"], eps).reshape(T, G, d)
    rot = m.get("rot")
    if rot and rot["dims"]:
        q = rotate_interleaved(q, pos, rot["dims"], rot["base"])
        k = rotate_interleaved(k, pos, rot["dims"], rot["base"])
    o = sink_softmax_attention(q, k, v.reshape(T, G, dv), m["scale"], w[p + "sink"])
    return o.reshape(T, H * dv) @ w[p + "o"].T


def lightning_scan(q, k, v, decay, state=None):
    """S_t = decay_h S_(t-1) + k_t v_t^T, o_t = S_t^T q_t.  q, k [T, H, d], v [T, H, dv].  Returns (o, S)."""
    T, H, d = q.shape
    dv = v.shape[2]
    S = np.zeros((H, d, dv)) if state is None else state.copy()
    o = np.zeros((T, H, dv))
    for t in range(T):
        for h in range(H):
            S[h] = decay[h] * S[h] + np.outer(k[t, h], v[t, h])
            o[t, h] = S[h].T @ q[t, h]
    return o, S


def lightning_attention(h, w, p, m, eps):
    """Right half of mixer 'parallel'."""
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ w[p + "q"].T).reshape(T, H, d)
    k = silu(h @ w[p + "k"].T).reshape(T, H, d)
    v = silu(h @ w[p + "v"].T).reshape(T, H, dv)
    o, _ = lightning_scan(q, k, v, np.asarray(m["decay"], dtype=np.float64))
    z = plain_norm(o.reshape(T, H * dv), w[p + "norm"], eps) * sigmoid(h @ w[p + "g"].T)
    return z @ w[p + "o"].T


def parallel_mixer(h, w, p, m, pos, eps):
    left = conv_attention(h, w, p + "left.", m["left"], pos, eps)
    right = lightning_attention(h, w, p + "right.", m["right"], eps)
    return 0.5 * (plain_norm(left, w[p + "left.out"], eps) + plain_norm(right, w[p + "right.out"], eps))


# ---- feed-forwards -------------------------------------------------------------------------------------
def dense_ff(h, w, p):
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def router_choice(h, w, p, f, margins=None):
    """(chosen experts [T, top], their weights [T, top]): sigmoid scores, the largest, as they are.  ``margins``
    (a list) receives, per token, how far the last chosen logit is above the first one that is not."""
    z = h @ w[p + "router"].T
    top = f["router"]["top"]
    ids = np.argsort(-z, axis=1, kind="stable")[:, :top]                      # the sigmoid keeps the order
    if margins is not None:
        zs = -np.sort(-z, axis=1)
        margins.append(zs[:, top - 1] - zs[:, top] if top < z.shape[1] else np.full(len(z), np.inf))
    return ids, sigmoid(np.take_along_axis(z, ids, axis=1))


def expert_ff(h, w, p, f, margins=None):
    """Each chosen expert reads its weight times h: sum_e down_e relu(up_e (s_e h))^2."""
    ids, wt = router_choice(h, w, p, f, margins)
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e, s in zip(ids[t], wt[t]):
            a = np.maximum(w[f"{p}e{e}.up"] @ (s * h[t]), 0.0) ** 2
            out[t] += w[f"{p}e{e}.down"] @ a
    return out


# ---- the model -------------------------------------------------------------------------------------------
def layer_forward(x, w, cfg, i, pos, margins=None):
    L = cfg["layers"][i]
    eps = cfg["norm"]["eps"]
    p = f"l{i}."
    h = one_plus_norm(x, w[p + "norm1"], eps)
    if L["type"] == "attention":
        y = gated_attention(h, w, p + "mix.", L["mixer"], pos)
    elif L["type"] == "parallel":
        y = parallel_mixer(h, w, p + "mix.", L["mixer"], pos, eps)
    else:
        raise ValueError(L["type"])
    f = L.get("mlp")
    if f is not None:
        y = y + (dense_ff(h, w, p + "mlp.") if f["kind"] == "dense" else expert_ff(h, w, p + "mlp.", f, margins))
    return x + y


def forward(tokens, w, cfg, return_layers=False, margins=None):
    """Logits [T, vocab] of one sequence from position 0 (and the stream after every layer).  ``margins`` (a list)
    receives one array [T] per layer with experts: the routers' margins."""
    tokens = np.asarray(tokens)
    pos = np.arange(len(tokens))
    x = w["embed"][tokens]
    layers = []
    for i in range(len(cfg["layers"])):
        x = layer_forward(x, w, cfg, i, pos, margins)
        layers.append(x)
    logits = (one_plus_norm(x, w["final.norm"], cfg["norm"]["eps"]) @ w["embed"].T) * cfg["logit_scale"]
    return (logits, np.stack(layers)) if return_layers else logits

"""Small Kasarax configurations for the tests, their model folders and plain logits.

The cases differ from one another in every size.  Together they cover: the
two mixers in different orders, layers with a dense feed-forward, with
experts and with none; attention with one key/value head per head and with
several heads per key/value head, keys larger and smaller than values, query
factors that step every 1, 7 and 50 positions and none; left halves with
convolutions of 1 to 5 taps, rotation of none, part and all of a head;
right halves with one head and several, decays from 0.5 to 1; one, some and
all experts chosen; logit scales on both sides of one; sizes that are no
multiple of 8, and a width that is no multiple of 4.

Weights are random but not all alike: the one-plus norm weights well away
from zero, plain norm weights away from one, biases and sinks that matter,
decays near 1 (so that the states remember).
"""
from __future__ import annotations

import json
import math
import tempfile
from pathlib import Path

import numpy as np


def attention(heads, kv_heads, dim, vdim, coef=None, every=None, scale=None):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale or 1.0 / math.sqrt(dim))
    if every:
        m["q_temp"] = dict(coef=coef, every=every)
    return dict(type="attention", mixer=m)


def left(heads, kv_heads, dim, vdim, conv, dims=0, base=10000.0, scale=None):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, conv=conv, scale=scale or 1.0 / math.sqrt(dim))
    if dims:
        m["rot"] = dict(base=base, dims=dims)
    return m


def right(heads, dim, vdim, decay):
    return dict(heads=heads, dim=dim, vdim=vdim, decay=list(decay))


def parallel(l, r):
    return dict(type="parallel", mixer=dict(left=l, right=r))


def dense(ff):
    return dict(kind="dense", ff=ff)


def moe(experts, top, ff):
    return dict(kind="moe", router=dict(experts=experts, top=top), expert=dict(ff=ff))


def layer(mix, mlp):
    return dict(mix, mlp=mlp)


# A: a parallel layer first; part of the left heads rotated, three taps; two of six and all of four experts; a
#    layer without a feed-forward; the query factor steps every 7 positions.
CASE_A = dict(
    architecture="Kasarax", width=64, vocab=200, norm=dict(eps=1e-5), logit_scale=0.7,
    layers=[layer(parallel(left(4, 2, 16, 24, 3, dims=8, base=100.0), right(2, 16, 8, [0.9, 0.995])), moe(6, 2, 24)),
            layer(attention(4, 2, 16, 8, coef=0.3, every=7), dense(96)),
            layer(parallel(left(2, 2, 24, 16, 2, dims=24, base=1000.0), right(3, 8, 24, [0.5, 0.97, 1.0])), None),
            layer(attention(6, 3, 8, 16, coef=1.1, every=1, scale=0.5), moe(4, 4, 16))])
# B: a convolution of one tap (a factor per channel, nothing kept between steps), no rotation, every head its own key/value head; one lightning head; attention
#    without a query factor; one expert chosen of five; logit scale one.
CASE_B = dict(
    architecture="Kasarax", width=96, vocab=130, norm=dict(eps=1e-6), logit_scale=1.0,
    layers=[layer(attention(3, 3, 32, 32), moe(5, 1, 40)),
            layer(parallel(left(6, 6, 16, 16, 1), right(1, 32, 48, [0.99])), dense(64)),
            layer(attention(6, 1, 16, 48, coef=0.8, every=50, scale=0.2), None)])
# C: sizes that are no multiple of 8; five taps; large epsilon; logit scale above one.
CASE_C = dict(
    architecture="Kasarax", width=40, vocab=90, norm=dict(eps=1e-3), logit_scale=2.5,
    layers=[layer(parallel(left(6, 3, 12, 20, 5, dims=6, base=70.0), right(5, 12, 10, [0.8, 0.9, 0.95, 0.99, 0.999])),
                  moe(3, 2, 12)),
            layer(attention(2, 1, 20, 12, coef=0.5, every=3), dense(56)),
            layer(parallel(left(3, 1, 12, 12, 2, dims=12, base=30.0), right(2, 20, 12, [0.7, 0.999])), moe(7, 3, 20))])
# D: sizes in multiples of 16 with prompts of several hundred tokens (the tensor-core kernels' tiles, the grouped
#    products of long prompts); four taps; decays a hair below one.
CASE_D = dict(
    architecture="Kasarax", width=128, vocab=320, norm=dict(eps=1e-6), logit_scale=0.25,
    layers=[layer(attention(8, 2, 64, 48, coef=0.4, every=50), dense(192)),
            layer(parallel(left(4, 4, 32, 32, 4, dims=32, base=20000.0), right(4, 32, 16, [0.96, 0.99, 0.998, 0.9995])),
                  moe(8, 3, 48)),
            layer(parallel(left(8, 2, 48, 64, 3, dims=16, base=300.0), right(8, 16, 16, [0.9] * 4 + [0.999] * 4)),
                  dense(64)),
            layer(attention(4, 4, 32, 32, coef=0.2, every=128), moe(12, 2, 32)),
            layer(parallel(left(2, 1, 128, 64, 2, dims=64, base=5000.0), right(2, 64, 64, [0.98, 1.0])), moe(8, 3, 48))])

# E: a width and a vocabulary that are multiples of neither 8 nor 4 (rows that start off 16-byte boundaries); head
#    sizes of 10 and 6; an attention layer last; seven taps.
CASE_E = dict(
    architecture="Kasarax", width=38, vocab=77, norm=dict(eps=1e-5), logit_scale=1.7,
    layers=[layer(parallel(left(2, 2, 10, 6, 7, dims=4, base=50.0), right(3, 6, 10, [0.93, 0.99, 0.9999])), dense(30)),
            layer(parallel(left(4, 1, 6, 10, 1, dims=6, base=9.0), right(1, 10, 6, [0.97])), moe(5, 2, 9)),
            layer(attention(5, 5, 6, 10, coef=0.7, every=11), moe(2, 1, 14))])

CASES = {"A": (CASE_A, 3, 8), "B": (CASE_B, 5, 16), "C": (CASE_C, 7, 32), "D": (CASE_D, 9, 16),
         "E": (CASE_E, 11, 4)}                                                                # config, seed, page

_made: dict = {}
_plain: dict = {}


def random_tensors(cfg: dict, seed: int, std: float = 0.12) -> dict:
    """name -> float32 array for every tensor of the model, by name."""
    rng = np.random.default_rng(seed)
    W = cfg["width"]
    n = lambda *shape, s=std: rng.normal(0.0, s, size=shape)
    near_one = lambda *shape: 1.0 + rng.uniform(-0.3, 0.3, size=shape)
    near_zero = lambda *shape: rng.uniform(-0.4, 0.6, size=shape)
    t = {"embed": n(cfg["vocab"], W, s=0.5), "final.norm": near_zero(W)}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        q = p + "mix."
        t[p + "norm1"] = near_zero(W)
        if L["type"] == "attention":
            H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            t.update({q + "q": n(H * d, W, s=0.25), q + "k": n(G * d, W, s=0.25), q + "v": n(G * dv, W),
                      q + "o": n(W, H * dv), q + "q.b": n(H * d, s=0.3), q + "k.b": n(G * d, s=0.3),
                      q + "v.b": n(G * dv, s=0.3), q + "o.b": n(W, s=0.3), q + "g": n(H, W, s=0.4)})
        else:
            a, s = m["left"], m["right"]
            H, G, d, dv, K = a["heads"], a["kv_heads"], a["dim"], a["vdim"], a["conv"]
            b = q + "left."
            t.update({b + "q": n(H * d, W), b + "k": n(G * d, W), b + "v": n(G * dv, W), b + "o": n(W, H * dv),
                      b + "q.norm": near_one(H * d) * 2.0, b + "k.norm": near_one(G * d) * 2.0,
                      b + "sink": n(H, s=1.5), q + "left.out": near_one(W), q + "right.out": near_one(W)})
            if K >= 1:
                t.update({b + "q.conv": n(H * d, K, s=0.6), b + "k.conv": n(G * d, K, s=0.6),
                          b + "v.conv": n(G * dv, K, s=0.6)})
            H, d, dv = s["heads"], s["dim"], s["vdim"]
            b = q + "right."
            t.update({b + "q": n(H * d, W), b + "k": n(H * d, W), b + "v": n(H * dv, W), b + "g": n(H * dv, W),
                      b + "o": n(W, H * dv), b + "norm": near_one(H * dv)})
        f = L["mlp"]
        if f:
            if f["kind"] == "dense":
                t.update({p + "mlp.gate": n(f["ff"], W), p + "mlp.up": n(f["ff"], W), p + "mlp.down": n(W, f["ff"])})
            else:
                t[p + "mlp.router"] = n(f["router"]["experts"], W, s=0.2)
                for e in range(f["router"]["experts"]):
                    F = f["expert"]["ff"]
                    t.update({f"{p}mlp.e{e}.up": n(F, W, s=0.3), f"{p}mlp.e{e}.down": n(W, F)})
    return {k: np.asarray(v, dtype=np.float32) for k, v in t.items()}


def write_model(cfg: dict, seed: int, out_dir, change=None) -> Path:
    """config.json and model.safetensors (bfloat16) for ``cfg``; ``change(tensors)`` may edit the arrays first."""
    import torch
    from railgun_b200.weights.safetensors_io import write_safetensors
    out_dir = Path(out_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    tensors = random_tensors(cfg, seed)
    if change is not None:
        change(tensors)
    (out_dir / "config.json").write_text(json.dumps(cfg))
    write_safetensors(out_dir / "model.safetensors",
                      {k: torch.from_numpy(v).to(torch.bfloat16) for k, v in tensors.items()})
    return out_dir


def model_dir(name: str) -> Path:
    if name not in _made:
        cfg, seed, _ = CASES[name]
        _made[name] = write_model(cfg, seed, tempfile.mkdtemp(prefix=f"rg_kasarax_{name}_"))
    return _made[name]


class Plain:
    """The plain statement over a model folder."""

    def __init__(self, folder):
        import plain_kasarax as P
        self.P = P
        self.cfg = json.loads((Path(folder) / "config.json").read_text())
        self.w = P.read_safetensors(Path(folder) / "model.safetensors")

    def forward(self, ids):
        return self.P.forward(ids, self.w, self.cfg)

    def forward_with_margins(self, ids):
        """(logits, per position the smallest router margin of any layer; inf without experts)."""
        m = []
        logits = self.P.forward(ids, self.w, self.cfg, margins=m)
        return logits, (np.min(np.stack(m), axis=0) if m else np.full(len(ids), np.inf))

    def greedy(self, prompt, n):
        ids = list(prompt)
        for _ in range(n):
            ids.append(int(np.argmax(self.forward(ids)[-1])))
        return ids[len(prompt):]


def plain_model(name: str) -> Plain:
    if name not in _plain:
        _plain[name] = Plain(model_dir(name))
    return _plain[name]


def prompts(vocab: int, lengths, seed: int):
    rng = np.random.default_rng(seed)
    return [rng.integers(0, vocab, size=n).tolist() for n in lengths]

"""Small Mepatar configurations for the tests, their model folders and plain logits.

The cases differ from one another in every size.  Together they cover: the
three mixers in different orders, layers with a dense feed-forward, with
experts and with none; norms in 1, 2, 3 and 5 groups; input convolutions of
1 to 5 taps and none; retention with one head and several, rotation of all,
part and none of a head, values larger and smaller than keys; attention
with one key/value head per head and several heads per key/value head,
windows shorter than a page, longer than any prompt and none, kept first
tokens of 0, 1, more than a page and more than the window; the delta rule
with as many query/key heads as value heads and fewer, convolutions of 1 to
5 taps; experts of which all, some and one are chosen.

Weights are random but not all alike: norm weights and temperatures away
from one, biases that matter, decays near 1 (so that the states remember).
"""
from __future__ import annotations

import json
import math
import tempfile
from pathlib import Path

import numpy as np


def retention(heads, dim, vdim, decay, dims=None, base=10000.0):
    m = dict(heads=heads, dim=dim, vdim=vdim, decay=list(decay))
    if dims:
        m["rot"] = dict(base=base, dims=dims)
    return dict(type="retention", mixer=m)


def attention(heads, kv_heads, dim, vdim, dims=0, base=10000.0, window=0, keep=0, scale=None):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale or 1.0 / math.sqrt(dim))
    if dims:
        m["rot"] = dict(base=base, dims=dims)
    if window:
        m["mask"] = dict(size=window, keep_first=keep)
    return dict(type="attention", mixer=m)


def delta(heads, kv_heads, dim, vdim, conv):
    return dict(type="delta", mixer=dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, conv=conv))


def dense(ff):
    return dict(kind="dense", ff=ff)


def moe(experts, top, ff, limit):
    return dict(kind="moe", router=dict(experts=experts, top=top), expert=dict(ff=ff, limit=limit))


def layer(mix, mlp):
    return dict(mix, mlp=mlp)


# A: two norm groups, three taps; windowed attention keeping three first tokens (window shorter than two pages);
#    retention with part of the head rotated; delta with fewer query/key heads; experts and a dense layer.
CASE_A = dict(
    architecture="Mepatar", width=64, vocab=200, norm=dict(eps=1e-5, groups=2), embedding=dict(scale=3.0),
    canon=dict(taps=3),
    layers=[layer(attention(4, 2, 16, 24, dims=8, base=100.0, window=11, keep=3), moe(6, 2, 24, 1.5)),
            layer(retention(2, 16, 24, [0.9, 0.995], dims=8, base=1000.0), dense(96)),
            layer(delta(4, 2, 16, 8, 3), None),
            layer(retention(3, 8, 8, [0.5, 0.97, 1.0]), moe(4, 4, 16, 0.7))])
# B: one norm group, no input convolution; full attention (no mask) with every head its own key/value head and no
#    rotation; delta with a convolution of one tap; retention with one head; all experts but one chosen.
CASE_B = dict(
    architecture="Mepatar", width=96, vocab=130, norm=dict(eps=1e-6, groups=1), embedding=dict(scale=1.0),
    layers=[layer(delta(3, 3, 24, 16, 1), dense(64)),
            layer(attention(6, 6, 16, 16), moe(5, 4, 40, 3.0)),
            layer(retention(1, 32, 48, [0.99], dims=32, base=50.0), None)])
# C: three norm groups, one tap (h + w h); a window of one with one kept token, a window longer than any prompt
#    with more kept tokens than a page; one expert chosen of many.
CASE_C = dict(
    architecture="Mepatar", width=48, vocab=64, norm=dict(eps=1e-3, groups=3), embedding=dict(scale=0.5),
    canon=dict(taps=1),
    layers=[layer(attention(2, 1, 8, 8, dims=8, base=10.0, window=1, keep=1), moe(9, 1, 8, 0.3)),
            layer(delta(2, 1, 8, 24, 5), dense(16)),
            layer(attention(3, 3, 24, 8, dims=12, base=30.0, window=1000, keep=20), None)])
# D: sizes in multiples of 16 with prompts of several hundred tokens; five taps; windows that end inside pages, kept
#    tokens beyond a page; decays a hair below one.
CASE_D = dict(
    architecture="Mepatar", width=128, vocab=320, norm=dict(eps=1e-6, groups=2), embedding=dict(scale=11.3),
    canon=dict(taps=5),
    layers=[layer(retention(4, 32, 16, [0.96, 0.99, 0.998, 0.9995], dims=32, base=100000.0), dense(192)),
            layer(delta(4, 4, 48, 64, 3), moe(8, 3, 48, 1.0)),
            layer(attention(8, 2, 64, 48, dims=32, base=20000.0, window=130, keep=4), moe(8, 3, 48, 1.0)),
            layer(attention(4, 4, 32, 32, dims=32, base=300.0, window=50, keep=37), dense(64)),
            layer(delta(8, 2, 16, 16, 2), moe(12, 2, 32, 2.0))])
# E: five norm groups; sizes that are no multiple of 8; kept tokens more than the window.
CASE_E = dict(
    architecture="Mepatar", width=40, vocab=90, norm=dict(eps=1e-5, groups=5), embedding=dict(scale=6.0),
    canon=dict(taps=2),
    layers=[layer(attention(6, 3, 12, 20, dims=6, base=70.0, window=5, keep=9), moe(3, 2, 12, 1.0)),
            layer(retention(5, 12, 10, [0.8, 0.9, 0.95, 0.99, 0.999], dims=12, base=70.0), dense(56)),
            layer(delta(6, 3, 12, 10, 4), moe(7, 3, 20, 0.5))])

CASES = {"A": (CASE_A, 3, 8), "B": (CASE_B, 5, 16), "C": (CASE_C, 7, 4), "D": (CASE_D, 9, 16),
         "E": (CASE_E, 11, 32)}                                                              # config, seed, page

_made: dict = {}
_plain: dict = {}


def random_tensors(cfg: dict, seed: int, std: float = 0.12) -> dict:
    """name -> float32 array for every tensor of the model, by name."""
    rng = np.random.default_rng(seed)
    W = cfg["width"]
    K0 = (cfg.get("canon") or {}).get("taps", 0)
    n = lambda *shape, s=std: rng.normal(0.0, s, size=shape)
    near_one = lambda *shape: 1.0 + rng.uniform(-0.3, 0.3, size=shape)
    t = {"embed": n(cfg["vocab"], W, s=0.5), "final.norm": near_one(W), "head": n(cfg["vocab"], W)}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        q = p + "mix."
        t[p + "norm1"] = near_one(W)
        if K0:
            t[p + "canon1"] = n(W, K0, s=0.4)
        if L["type"] == "retention":
            H, d, dv = m["heads"], m["dim"], m["vdim"]
            t.update({q + "q": n(H * d, W), q + "k": n(H * d, W), q + "v": n(H * dv, W), q + "g": n(H * dv, W),
                      q + "o": n(W, H * dv)})
        elif L["type"] == "attention":
            H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            t.update({q + "q": n(H * d, W), q + "k": n(G * d, W), q + "v": n(G * dv, W), q + "o": n(W, H * dv),
                      q + "q.b": n(H * d, s=0.3), q + "k.b": n(G * d, s=0.3), q + "v.b": n(G * dv, s=0.3),
                      q + "o.b": n(W, s=0.3), q + "q.norm": near_one(d) * 2.0, q + "k.norm": near_one(d) * 2.0,
                      q + "temp": rng.uniform(0.5, 2.0, size=H)})
        else:
            H, G, d, dv, K = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
            t.update({q + "q": n(G * d, W), q + "k": n(G * d, W), q + "v": n(H * dv, W), q + "g": n(H * dv, W),
                      q + "q.conv": n(G * d, K, s=0.6), q + "k.conv": n(G * d, K, s=0.6), q + "v.conv": n(H * dv, K, s=0.6),
                      q + "b": n(H, W), q + "a": n(H, W), q + "A_log": rng.normal(-2.0, 1.0, size=H),
                      q + "dt_bias": rng.normal(-1.0, 1.0, size=H), q + "norm": near_one(dv), q + "o": n(W, H * dv)})
        f = L["mlp"]
        if f:
            t[p + "norm2"] = near_one(W)
            if f["kind"] == "dense":
                t.update({p + "mlp.gate": n(f["ff"], W), p + "mlp.up": n(f["ff"], W), p + "mlp.down": n(W, f["ff"])})
            else:
                t[p + "mlp.router"] = n(f["router"]["experts"], W, s=0.5)
                for e in range(f["router"]["experts"]):
                    F = f["expert"]["ff"]
                    t.update({f"{p}mlp.e{e}.gate": n(F, W, s=0.3), f"{p}mlp.e{e}.up": n(F, W, s=0.3),
                              f"{p}mlp.e{e}.down": n(W, F)})
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
        _made[name] = write_model(cfg, seed, tempfile.mkdtemp(prefix=f"rg_mepatar_{name}_"))
    return _made[name]


class Plain:
    """The plain statement over a model folder."""

    def __init__(self, folder):
        import plain_mepatar as P
        self.P = P
        self.cfg = json.loads((Path(folder) / "config.json").read_text())
        self.w = P.read_safetensors(Path(folder) / "model.safetensors")

    def forward(self, ids):
        return self.P.forward(ids, self.w, self.cfg)

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

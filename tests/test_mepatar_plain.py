"""The plain statement of Mepatar against loop-level formulas, and the package's
configuration, description and tensor list for the design (no GPU)."""
import json
import math

import numpy as np
import pytest

import mepatar_cases as C
import plain_mepatar as P


def weights(cfg, seed=1):
    return {k: v.astype(np.float64) for k, v in C.random_tensors(cfg, seed).items()}


def test_group_norm_norms_each_part_on_its_own():
    rng = np.random.default_rng(0)
    x = rng.normal(size=(3, 12))
    x[:, 4:8] *= 100.0                                     # one loud part must not quieten the others
    w = rng.uniform(0.5, 2.0, size=12)
    for groups in (1, 2, 3, 4, 12):
        got = P.group_norm(x, w, groups, 1e-5)
        n = 12 // groups
        for t in range(3):
            for g in range(groups):
                part = x[t, g * n:(g + 1) * n]
                ref = part / math.sqrt((part ** 2).mean() + 1e-5) * w[g * n:(g + 1) * n]
                assert np.allclose(got[t, g * n:(g + 1) * n], ref, atol=1e-12)
    assert not np.allclose(P.group_norm(x, w, 1, 1e-5), P.group_norm(x, w, 3, 1e-5))


def test_causal_convolution_reads_the_past_only_and_the_last_column_is_now():
    rng = np.random.default_rng(1)
    x, taps = rng.normal(size=(9, 5)), rng.normal(size=(5, 4))
    got = P.causal_conv(x, taps)
    for t in range(9):
        ref = np.zeros(5)
        for j in range(4):
            s = t - 3 + j
            if s >= 0:
                ref += taps[:, j] * x[s]
        assert np.allclose(got[t], ref, atol=1e-12)
    one = np.zeros((4, 1)); one[0, 0] = 1.0
    assert np.allclose(P.causal_conv(one, np.array([[1.0, 2.0, 3.0]]))[:, 0], [3.0, 2.0, 1.0, 0.0])
    assert np.allclose(P.causal_conv(x, taps[:, :1]), x * taps[:, 0])                     # one tap: no past


def test_rotation_layouts_pair_the_right_numbers():
    rng = np.random.default_rng(0)
    x = rng.normal(size=(4, 2, 12))
    pos = np.array([0, 1, 300, 4000])
    for layout in ("half", "interleaved"):
        for dims in (0, 4, 12):
            got = P.rotate(x, pos, dims, 50.0, layout)
            for t in range(4):
                for h in range(2):
                    ref = x[t, h].copy()
                    for i in range(dims // 2):
                        a = pos[t] * 50.0 ** (-2.0 * i / dims)
                        lo, hi = (i, i + dims // 2) if layout == "half" else (2 * i, 2 * i + 1)
                        u, v = x[t, h, lo], x[t, h, hi]
                        ref[lo], ref[hi] = u * math.cos(a) - v * math.sin(a), v * math.cos(a) + u * math.sin(a)
                    assert np.allclose(got[t, h], ref, atol=1e-12)


def test_window_with_kept_first_tokens():
    see = lambda i, size, keep: [j for j in range(i + 1) if P.visible(i, j, size, keep)]
    assert see(9, 3, 0) == [7, 8, 9]
    assert see(9, 3, 2) == [0, 1, 7, 8, 9]
    assert see(3, 3, 2) == [0, 1, 2, 3]                    # the window still reaches the kept tokens: once each
    assert see(9, 1, 1) == [0, 9] and see(0, 1, 1) == [0]
    assert see(9, 2, 20) == list(range(10))                # more kept tokens than there are
    assert not P.visible(3, 4, 100, 100)                   # never the future


def test_retention_equals_its_sum_form():
    """o_t = sum_(s <= t) decay^(t - s) (q_t . k_s) v_s: the recurrence unrolled."""
    cfg = C.CASE_A
    w = weights(cfg)
    m, eps = cfg["layers"][1]["mixer"], cfg["norm"]["eps"]
    rng = np.random.default_rng(2)
    T = 11
    h = rng.normal(size=(T, cfg["width"]))
    got = P.retention(h, w, "l1.mix.", m, eps)
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    pos = np.arange(T)
    q = P.rotate((h @ w["l1.mix.q"].T).reshape(T, H, d), pos, m["rot"]["dims"], m["rot"]["base"], "half")
    k = P.rotate((h @ w["l1.mix.k"].T).reshape(T, H, d), pos, m["rot"]["dims"], m["rot"]["base"], "half") / math.sqrt(d)
    v = (h @ w["l1.mix.v"].T).reshape(T, H, dv)
    gate = P.silu(h @ w["l1.mix.g"].T).reshape(T, H, dv)
    z = np.zeros((T, H, dv))
    for t in range(T):
        for a in range(H):
            o = sum(m["decay"][a] ** (t - s) * (q[t, a] @ k[s, a]) * v[s, a] for s in range(t + 1))
            z[t, a] = o / math.sqrt((o ** 2).mean() + eps) * gate[t, a]
    assert np.allclose(got, z.reshape(T, -1) @ w["l1.mix.o"].T, atol=1e-10)


def test_delta_rule_writes_before_it_reads():
    """With beta = 1 and no decay, reading with the key just written returns the value just written."""
    rng = np.random.default_rng(3)
    d, dv = 6, 4
    S = np.zeros((d, dv))
    for _ in range(5):
        k = rng.normal(size=d); k /= np.linalg.norm(k)
        v = rng.normal(size=dv)
        S = S + np.outer(k, 1.0 * (v - S.T @ k))
        assert np.allclose(S.T @ k, v, atol=1e-12)
    # the function's own order: decay, correction, write, read
    cfg = C.CASE_A
    w = weights(cfg)
    m = cfg["layers"][2]["mixer"]
    T = 7
    h = rng.normal(size=(T, cfg["width"]))
    got = P.delta(h, w, "l2.mix.", m, 1e-5)
    H, G, dd, dvv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    conv = lambda n: P.silu(P.causal_conv(h @ w[f"l2.mix.{n}"].T, w[f"l2.mix.{n}.conv"]))
    q, k, v = conv("q").reshape(T, G, dd), conv("k").reshape(T, G, dd), conv("v").reshape(T, H, dvv)
    z = np.zeros((T, H, dvv))
    for a in range(H):
        c = a // (H // G)
        S = np.zeros((dd, dvv))
        for t in range(T):
            qq = q[t, c] / math.sqrt((q[t, c] ** 2).sum() + 1e-6) / math.sqrt(dd)
            kk = k[t, c] / math.sqrt((k[t, c] ** 2).sum() + 1e-6)
            beta = 1.0 / (1.0 + math.exp(-(w["l2.mix.b"][a] @ h[t])))
            x = w["l2.mix.a"][a] @ h[t] + w["l2.mix.dt_bias"][a]
            g = math.exp(-math.exp(w["l2.mix.A_log"][a]) * math.log1p(math.exp(x)))
            S = g * S
            S = S + np.outer(kk, beta * (v[t, a] - S.T @ kk))
            o = S.T @ qq
            z[t, a] = o / math.sqrt((o ** 2).mean() + 1e-5) * w["l2.mix.norm"]
    z = z.reshape(T, -1) * P.silu(h @ w["l2.mix.g"].T)
    assert np.allclose(got, z @ w["l2.mix.o"].T, atol=1e-10)


def test_attention_against_loops():
    cfg = C.CASE_A
    w = weights(cfg)
    m, eps = cfg["layers"][0]["mixer"], cfg["norm"]["eps"]
    rng = np.random.default_rng(4)
    T = 19
    h = rng.normal(size=(T, cfg["width"]))
    got = P.attention(h, w, "l0.mix.", m, eps)
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    size, keep = m["mask"]["size"], m["mask"]["keep_first"]
    dims, base = m["rot"]["dims"], m["rot"]["base"]

    def head(x, norm, pos):
        x = x / math.sqrt((x ** 2).mean() + eps) * norm
        out = x.copy()
        for i in range(dims // 2):
            a = pos * base ** (-2.0 * i / dims)
            out[2 * i] = x[2 * i] * math.cos(a) - x[2 * i + 1] * math.sin(a)
            out[2 * i + 1] = x[2 * i + 1] * math.cos(a) + x[2 * i] * math.sin(a)
        return out

    rows = np.zeros((T, H * dv))
    for t in range(T):
        qt = (w["l0.mix.q"] @ h[t] + w["l0.mix.q.b"]).reshape(H, d)
        for a in range(H):
            c = a // (H // G)
            qa = head(qt[a], w["l0.mix.q.norm"], t)
            seen = [j for j in range(t + 1) if t - j < size or j < keep]
            s, vs = [], []
            for j in seen:
                kj = head((w["l0.mix.k"] @ h[j] + w["l0.mix.k.b"]).reshape(G, d)[c], w["l0.mix.k.norm"], j)
                s.append((qa @ kj) * m["scale"] * w["l0.mix.temp"][a])
                vs.append((w["l0.mix.v"] @ h[j] + w["l0.mix.v.b"]).reshape(G, dv)[c])
            p = np.exp(np.array(s) - max(s)); p /= p.sum()
            rows[t, a * dv:(a + 1) * dv] = p @ np.array(vs)
    assert np.allclose(got, rows @ w["l0.mix.o"].T + w["l0.mix.o.b"], atol=1e-10)


def test_experts_clamp_and_keep_their_scores_as_they_are():
    cfg = C.CASE_A
    w = weights(cfg)
    mlp = cfg["layers"][0]["mlp"]
    rng = np.random.default_rng(5)
    h = rng.normal(size=(8, cfg["width"])) * 3.0
    w["l0.mlp.router"] = w["l0.mlp.router"] * 0.05         # scores that are not one-hot
    got = P.moe_ff(h, w, "l0.mlp.", mlp)
    E, top, limit = mlp["router"]["experts"], mlp["router"]["top"], mlp["expert"]["limit"]
    clamped = False
    for t in range(8):
        z = w["l0.mlp.router"] @ h[t]
        s = np.exp(z - z.max()); s /= s.sum()
        ref = np.zeros(cfg["width"])
        for e in np.argsort(-s)[:top]:
            g, u = w[f"l0.mlp.e{e}.gate"] @ h[t], w[f"l0.mlp.e{e}.up"] @ h[t]
            clamped |= bool((g > limit).any() and (u < -limit).any() and (u > limit).any())
            g, u = np.minimum(g, limit), np.clip(u, -limit, limit)
            ref += s[e] * (w[f"l0.mlp.e{e}.down"] @ (g / (1.0 + np.exp(-1.702 * g)) * (u + 1.0)))
        assert np.allclose(got[t], ref, atol=1e-10)
        assert s[np.argsort(-s)[:top]].sum() < 1.0 - 1e-6                      # not renormalised
    assert clamped
    assert abs(P.gelu_tanh(np.array([1.0]))[0] - 0.8411919906082768) < 1e-12


def test_layer_is_parallel_on_one_stream():
    cfg = C.CASE_A
    w = weights(cfg)
    x = np.random.default_rng(6).normal(size=(6, cfg["width"]))
    eps, groups = cfg["norm"]["eps"], cfg["norm"]["groups"]
    h = P.group_norm(x, w["l1.norm1"], groups, eps)
    h = h + P.causal_conv(h, w["l1.canon1"])
    f = P.group_norm(x, w["l1.norm2"], groups, eps)
    ref = x + P.retention(h, w, "l1.mix.", cfg["layers"][1]["mixer"], eps) + P.dense_ff(f, w, "l1.mlp.")
    assert np.allclose(P.layer(x, w, cfg, 1), ref, atol=1e-12)
    assert np.allclose(P.layer(x, w, cfg, 2), x + P.delta(
        (lambda g: g + P.causal_conv(g, w["l2.canon1"]))(P.group_norm(x, w["l2.norm1"], groups, eps)), w, "l2.mix.",
        cfg["layers"][2]["mixer"], eps), atol=1e-12)                           # a layer without a feed-forward


@pytest.mark.parametrize("name", sorted(C.CASES))
def test_prefix_property(name):
    """Causal everywhere: the logits of a prefix are the first rows of the logits of the whole."""
    cfg, seed, _ = C.CASES[name]
    w = weights(cfg, seed)
    ids = C.prompts(cfg["vocab"], [40], seed=1)[0]
    whole = P.forward(ids, w, cfg)
    assert np.allclose(P.forward(ids[:17], w, cfg), whole[:17], atol=1e-9)
    assert np.isfinite(whole).all() and np.abs(whole).max() > 1e-3


# ---- the package's side, without a GPU -------------------------------------------------------------

@pytest.mark.parametrize("name", sorted(C.CASES))
def test_configuration_description_and_tensor_list(name):
    from railgun_b200.config.registry import architecture_name, architecture_of
    from railgun_b200.parts.model import expected_tensors
    cfg, seed, _ = C.CASES[name]
    arch = architecture_of(architecture_name(cfg))
    assert arch.name == "Mepatar"
    c = arch.config_from_dict(cfg)
    again = arch.config_from_dict(json.loads(json.dumps(c.to_dict())))
    assert again == c
    spec = arch.model_spec(c)
    assert len(spec.layers) == len(cfg["layers"]) and spec.vocab_size == cfg["vocab"]
    specs = expected_tensors(spec)
    made = C.random_tensors(cfg, seed)
    assert set(specs) == set(made)
    for k, s in specs.items():
        assert tuple(s.shape) == made[k].shape, k


def test_configuration_errors_are_named():
    from railgun_b200.config.base import ConfigError
    from railgun_b200.config.mepatar import MepatarConfig
    good = json.loads(json.dumps(C.CASE_A))
    for change, word in ((lambda d: d["layers"][0].update(type="hyena"), "hyena"),
                         (lambda d: d["layers"][1]["mixer"].update(decay=[0.5]), "decays"),
                         (lambda d: d["norm"].update(groups=7), "groups"),
                         (lambda d: d["layers"][0]["mixer"].update(kv_heads=3), "share"),
                         (lambda d: d["layers"][0]["mlp"]["router"].update(top=99), "top"),
                         (lambda d: d["layers"][0]["mixer"]["rot"].update(dims=7), "rot.dims")):
        bad = json.loads(json.dumps(good))
        change(bad)
        with pytest.raises(ConfigError) as e:
            MepatarConfig.from_dict(bad)
        assert word in str(e.value)

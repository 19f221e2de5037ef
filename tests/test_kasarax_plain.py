"""The plain statement of Kasarax against loop-level formulas, and the package's
configuration, description and tensor list for the design (no GPU)."""
import json
import math

import numpy as np
import pytest

import kasarax_cases as C
import plain_kasarax as P


def weights(cfg, seed=1):
    return {k: v.astype(np.float64) for k, v in C.random_tensors(cfg, seed).items()}


def test_norm_weights_are_stored_around_zero():
    rng = np.random.default_rng(0)
    x, w = rng.normal(size=(3, 12)) * 7.0, rng.uniform(-0.5, 0.5, size=12)
    got = P.one_plus_norm(x, w, 1e-5)
    for t in range(3):
        assert np.allclose(got[t], x[t] / math.sqrt((x[t] ** 2).mean() + 1e-5) * (1.0 + w), atol=1e-12)
    assert np.allclose(P.one_plus_norm(x, np.zeros(12), 0.0) ** 2, x ** 2 / (x ** 2).mean(axis=1, keepdims=True))
    big = P.one_plus_norm(x * 1e-4, w, 1.0)                # eps sits inside the root
    assert np.abs(big).max() < 1e-2


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


def test_interleaved_rotation_pairs_neighbours():
    rng = np.random.default_rng(0)
    x = rng.normal(size=(4, 2, 12))
    pos = np.array([0, 1, 300, 4000])
    for dims in (4, 12):
        got = P.rotate_interleaved(x, pos, dims, 50.0)
        for t in range(4):
            for h in range(2):
                ref = x[t, h].copy()
                for i in range(dims // 2):
                    a = pos[t] * 50.0 ** (-2.0 * i / dims)
                    u, v = x[t, h, 2 * i], x[t, h, 2 * i + 1]
                    ref[2 * i], ref[2 * i + 1] = u * math.cos(a) - v * math.sin(a), v * math.cos(a) + u * math.sin(a)
                assert np.allclose(got[t, h], ref, atol=1e-12)
        assert np.array_equal(got[..., dims:], x[..., dims:])


def test_query_factor_steps_with_the_position():
    f = P.query_temperature(np.arange(50), 0.25, 10)
    assert np.all(f[:9] == 1.0) and f[9] == 1.0 + 0.25 * math.log(2.0)        # position 9: (9 + 1) / 10 = 1
    assert f[18] == f[9] and f[19] == 1.0 + 0.25 * math.log(3.0)
    assert np.allclose(P.query_temperature([0, 1, 2], 2.0, 1), [1.0 + 2.0 * math.log(k + 2.0) for k in range(3)])


def test_sink_softmax_against_loops():
    """The sink's term is exp(sink), unscaled, once, with no value; a sink of score 0 adds one."""
    rng = np.random.default_rng(3)
    T, H, G, d, dv = 6, 4, 2, 5, 3
    q, k, v = rng.normal(size=(T, H, d)), rng.normal(size=(T, G, d)), rng.normal(size=(T, G, dv))
    sink = np.array([0.0, 2.0, -50.0, 1.0])
    got = P.sink_softmax_attention(q, k, v, 0.7, sink)
    for t in range(T):
        for h in range(H):
            g = h // 2
            e = [math.exp(0.7 * float(q[t, h] @ k[j, g])) for j in range(t + 1)]
            den = sum(e) + math.exp(sink[h])
            assert np.allclose(got[t, h], sum(e[j] * v[j, g] for j in range(t + 1)) / den, atol=1e-12)
    plain = P.sink_softmax_attention(q, k, v, 0.7, np.full(H, -1e9))
    assert np.allclose(got[:, 2], plain[:, 2], atol=1e-12) and not np.allclose(got[:, 0], plain[:, 0], atol=1e-3)
    assert np.all(np.abs(got[0, 0]) < np.abs(v[0, 0]))                          # one key and the sink: less than v


def test_lightning_equals_its_sum_form_and_continues_from_a_state():
    """o_t = sum_(s <= t) decay^(t - s) (q_t . k_s) v_s: the recurrence unrolled."""
    rng = np.random.default_rng(4)
    T, H, d, dv = 9, 3, 4, 5
    q, k, v = rng.normal(size=(T, H, d)), rng.normal(size=(T, H, d)), rng.normal(size=(T, H, dv))
    decay = np.array([0.5, 0.9, 1.0])
    o, S = P.lightning_scan(q, k, v, decay)
    for t in range(T):
        for h in range(H):
            ref = sum(decay[h] ** (t - s) * float(q[t, h] @ k[s, h]) * v[s, h] for s in range(t + 1))
            assert np.allclose(o[t, h], ref, atol=1e-12)
    o1, S1 = P.lightning_scan(q[:4], k[:4], v[:4], decay)
    o2, S2 = P.lightning_scan(q[4:], k[4:], v[4:], decay, S1)
    assert np.allclose(np.concatenate([o1, o2]), o, atol=1e-12) and np.allclose(S2, S, atol=1e-12)


def test_mixers_against_loops():
    cfg = C.CASE_A
    w = weights(cfg)
    rng = np.random.default_rng(5)
    T = 11
    h = rng.normal(size=(T, cfg["width"]))
    pos = np.arange(T)
    # the attention mixer: biases, the query factor, one added to the denominator, a gate per head
    m = cfg["layers"][1]["mixer"]
    p = "l1.mix."
    got = P.gated_attention(h, w, p, m, pos)
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    for t in range(T):
        heads = []
        f = 1.0 + m["q_temp"]["coef"] * math.log((t + 1) // m["q_temp"]["every"] + 1)
        gate = 1.0 / (1.0 + np.exp(-(w[p + "g"] @ h[t])))
        for hd in range(H):
            g = hd // (H // G)
            qv = (w[p + "q"][hd * d:(hd + 1) * d] @ h[t] + w[p + "q.b"][hd * d:(hd + 1) * d]) * f
            e, vs = [], []
            for j in range(t + 1):
                kv = w[p + "k"][g * d:(g + 1) * d] @ h[j] + w[p + "k.b"][g * d:(g + 1) * d]
                vs.append(w[p + "v"][g * dv:(g + 1) * dv] @ h[j] + w[p + "v.b"][g * dv:(g + 1) * dv])
                e.append(math.exp(m["scale"] * float(qv @ kv)))
            heads.append(gate[hd] * sum(a * b for a, b in zip(e, vs)) / (1.0 + sum(e)))
        assert np.allclose(got[t], w[p + "o"] @ np.concatenate(heads) + w[p + "o.b"], atol=1e-10)
    # the parallel mixer: each half normed over the width with its own weight, half the sum
    m = cfg["layers"][0]["mixer"]
    p = "l0.mix."
    eps = cfg["norm"]["eps"]
    left = P.conv_attention(h, w, p + "left.", m["left"], pos, eps)
    right = P.lightning_attention(h, w, p + "right.", m["right"], eps)
    got = P.parallel_mixer(h, w, p, m, pos, eps)
    for t in range(T):
        a = left[t] / math.sqrt((left[t] ** 2).mean() + eps) * w[p + "left.out"]
        b = right[t] / math.sqrt((right[t] ** 2).mean() + eps) * w[p + "right.out"]
        assert np.allclose(got[t], 0.5 * (a + b), atol=1e-12)
    # the left half norms ALL of q at once, before the heads are cut
    a = m["left"]
    q = P.causal_conv(h @ w[p + "left.q"].T, w[p + "left.q.conv"])
    qn = q / np.sqrt((q ** 2).mean(axis=1, keepdims=True) + eps) * w[p + "left.q.norm"]
    per_head = P.unit_rms(q.reshape(T, a["heads"], a["dim"]), eps).reshape(T, -1) * w[p + "left.q.norm"]
    assert not np.allclose(qn, per_head, atol=1e-3)


def test_experts_read_their_weight_times_the_input():
    cfg = C.CASE_A
    w = weights(cfg)
    rng = np.random.default_rng(6)
    h = rng.normal(size=(7, cfg["width"]))
    f = cfg["layers"][0]["mlp"]
    p = "l0.mlp."
    got = P.expert_ff(h, w, p, f)
    ids, wt = P.router_choice(h, w, p, f)
    for t in range(7):
        z = w[p + "router"] @ h[t]
        s = 1.0 / (1.0 + np.exp(-z))
        chosen = sorted(range(len(s)), key=lambda e: -s[e])[:f["router"]["top"]]
        assert list(ids[t]) == chosen and np.allclose(wt[t], s[chosen])
        ref = np.zeros(cfg["width"])
        for e in chosen:
            ref += w[f"{p}e{e}.down"] @ np.maximum(w[f"{p}e{e}.up"] @ (s[e] * h[t]), 0.0) ** 2
        assert np.allclose(got[t], ref, atol=1e-12)
    assert wt.sum(axis=1).max() > 1.0 or wt.sum(axis=1).min() < 1.0              # not renormalized


def test_the_layer_has_one_norm_and_the_model_is_causal():
    cfg = C.CASE_C
    w = weights(cfg)
    ids = C.prompts(cfg["vocab"], [14], seed=1)[0]
    logits, layers = P.forward(ids, w, cfg, return_layers=True)
    x = w["embed"][np.asarray(ids)]
    h = P.one_plus_norm(x, w["l0.norm1"], cfg["norm"]["eps"])
    L = cfg["layers"][0]
    y = P.parallel_mixer(h, w, "l0.mix.", L["mixer"], np.arange(14), cfg["norm"]["eps"]) + P.expert_ff(
        h, w, "l0.mlp.", L["mlp"])
    assert np.allclose(layers[0], x + y, atol=1e-12)
    last = P.one_plus_norm(layers[-1], w["final.norm"], cfg["norm"]["eps"]) @ w["embed"].T * cfg["logit_scale"]
    assert np.allclose(logits, last, atol=1e-12)
    other = list(ids)
    other[9] = (ids[9] + 1) % cfg["vocab"]
    moved = P.forward(other, w, cfg)
    assert np.allclose(moved[:9], logits[:9], atol=1e-12) and not np.allclose(moved[9:], logits[9:], atol=1e-6)


# ---- the package's side, without a GPU ------------------------------------------------------------------

@pytest.mark.parametrize("name", sorted(C.CASES))
def test_configuration_round_trip_and_tensor_list(name):
    from railgun_b200.config.kasarax import KasaraxConfig
    from railgun_b200.config.registry import architecture_of
    from railgun_b200.parts.model import expected_tensors
    cfg = C.CASES[name][0]
    typed = KasaraxConfig.from_dict(json.loads(json.dumps(cfg)))
    assert typed.to_dict() == cfg
    arch = architecture_of("Kasarax")
    spec = arch.model_spec(typed)
    expected = expected_tensors(spec)
    made = C.random_tensors(cfg, 0)
    assert set(expected) == set(made)
    assert all(tuple(expected[k].shape) == made[k].shape for k in made)
    assert len(spec.layers) == len(cfg["layers"]) and all(L.arrangement == "parallel_residual" for L in spec.layers)
    for L, c in zip(spec.layers, cfg["layers"]):
        assert len(L.branches()) == (2 if c["mlp"] else 1)
        assert all(b.norm == L.branches()[0].norm for b in L.branches())       # one norm for both


def test_configuration_errors():
    from railgun_b200.config.base import ConfigError
    from railgun_b200.config.kasarax import KasaraxConfig
    good = json.loads(json.dumps(C.CASE_A))

    def broken(change):
        c = json.loads(json.dumps(good))
        change(c)
        with pytest.raises(ConfigError):
            KasaraxConfig.from_dict(c)

    broken(lambda c: c.pop("width"))
    broken(lambda c: c.pop("norm"))
    broken(lambda c: c.update(layers=[]))
    broken(lambda c: c["layers"][0].update(type="retention"))
    broken(lambda c: c["layers"][0]["mixer"].pop("right"))
    broken(lambda c: c["layers"][0]["mixer"]["right"].update(decay=[0.5]))
    broken(lambda c: c["layers"][0]["mixer"]["left"].update(kv_heads=3))
    broken(lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=7))
    broken(lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=18))
    broken(lambda c: c["layers"][1]["mixer"]["q_temp"].update(every=0))
    broken(lambda c: c["layers"][1]["mixer"].pop("scale"))
    broken(lambda c: c["layers"][0]["mlp"]["router"].update(top=7))
    broken(lambda c: c["layers"][1]["mlp"].update(kind="sparse"))


def test_registry_knows_the_design(tmp_path):
    from railgun_b200.config.registry import known_architectures, load_config
    assert "Kasarax" in known_architectures()
    (tmp_path / "config.json").write_text(json.dumps(C.CASE_B))
    arch, cfg = load_config(tmp_path)
    assert arch.name == "Kasarax" and cfg.width == 96 and cfg.logit_scale == 1.0
    assert cfg.layers[0].mixer.temp_every == 0 and cfg.layers[2].mixer.temp_every == 50
    assert cfg.layers[1].mixer.left.conv == 1 and cfg.layers[1].mixer.left.rot_dims == 0

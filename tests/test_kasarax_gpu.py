"""Kasarax on the GPU against the plain statement: each mechanism alone, then
the model through the step function in several cuts and both precisions, then
generation through the engine, its scheduler and the command line."""
import json
import os
import subprocess
import sys
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import helpers
import kasarax_cases as C
import plain_kasarax as P

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DEV = torch.device("cuda:0")
DTYPES = ["float32", "bfloat16"]
TORCH = {"float32": torch.float32, "bfloat16": torch.bfloat16}
# bfloat16: the test weights are several times larger than a trained model's, so rounding alone moves a few
# logits in a hundred by some 1e-2 of the largest, the same in every cut; a lost key, state, tap or sink is caught
# by the tests of the mechanisms alone, where it changes a row by its whole size.  Where a router's choice is a
# close call, rounding may choose the other expert: those positions are held to LOOSE only, and so may be a few
# that come after them in their request.
TOL = {"float32": 5e-5, "bfloat16": 6e-2}
LOOSE = 1.5
CLOSE_CALL = 0.06                                   # of router logits, in bfloat16


def rel(got, ref):
    got = got.double().cpu().numpy() if isinstance(got, torch.Tensor) else np.asarray(got, dtype=np.float64)
    ref = ref.double().cpu().numpy() if isinstance(ref, torch.Tensor) else np.asarray(ref, dtype=np.float64)
    return np.abs(got - ref).max() / np.abs(ref).max()


def dev(x, dtype=None):
    t = torch.as_tensor(x)
    return t.to(DEV, dtype=dtype) if dtype is not None else t.to(DEV)


def step_batch(lengths, starts, slots):
    """What the kernels of the state mixers read of a step: requests packed one after another."""
    cu = np.concatenate([[0], np.cumsum(lengths)]).astype(np.int32)
    return SimpleNamespace(cu_seqlens=dev(cu), num_requests=len(lengths),
                           req_of_token=dev(np.repeat(np.arange(len(lengths)), lengths).astype(np.int32)),
                           start_pos=dev(np.asarray(starts, dtype=np.int32)),
                           state_slots=dev(np.asarray(slots, dtype=np.int32)),
                           positions=dev(np.concatenate([s + np.arange(n) for s, n in zip(starts, lengths)]).astype(np.int32)))


# ---- norms ---------------------------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,W,n", [(3, 24, 2), (5, 64, 1), (300, 256, 2), (2, 41, 3), (7, 2050, 2), (33, 4100, 4)])
def test_normed_sum_alone(T, W, n, dtype):
    """Every input is brought to unit size on its own: one loud input does not drown the others."""
    from railgun_b200 import ops
    rng = np.random.default_rng(T + W)
    ys = [torch.tensor(rng.normal(size=(T, W)) * (100.0 if b == 0 else 0.01), dtype=TORCH[dtype]) for b in range(n)]
    ws = [rng.uniform(0.5, 2, size=W) for _ in range(n)]
    cs = [0.5, 0.25, 2.0, 1.0][:n]
    got = ops.norm_sum([dev(y) for y in ys], [dev(w, torch.float32) for w in ws], cs, 1e-6)
    ref = sum(c * P.plain_norm(y.double().numpy(), w, 1e-6) for y, w, c in zip(ys, ws, cs))
    assert got.dtype == torch.float32 and rel(got, ref) < 3e-6


@pytest.mark.parametrize("dtype", DTYPES)
def test_one_norm_feeds_both_branches(dtype):
    """A layer whose mixer and feed-forward are given the same norm: one normed row, stored weight plus one."""
    from railgun_b200.engine.runner import ModelRunner
    cfg, _, page = C.CASES["A"]
    runner = ModelRunner(C.model_dir("A"), dtype=dtype, page_size=page, max_tokens=64, max_requests=1)
    norms = [b.norm for b in runner.model.layers[0].branches]
    assert len(norms) == 2 and norms[0].params == norms[1].params
    w = C.plain_model("A").w
    assert rel(norms[0].weight, 1.0 + w["l0.norm1"]) < 1e-7
    assert rel(runner.model.final_norm.weight, (1.0 + w["final.norm"]) * cfg["logit_scale"]) < 1e-6


# ---- what attention does per token before the attention kernels ------------------------------------------

@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_prepare_whole_norm_and_query_factor(dtype):
    """Norm over all q heads at once and over all k heads at once (a loud head quietens the others), rotation in
    pairs (2i, 2i + 1) of the first numbers only, the query factor stepping with the position, 32-bit rows
    rounded once into the storage type."""
    from railgun_b200 import ops
    from railgun_b200.parts.latent_attention import rotary_frequencies
    rng = np.random.default_rng(11)
    for H, G, d, dv, dims, every in ((4, 2, 16, 8, 8, 7), (6, 2, 128, 80, 64, 1), (3, 3, 24, 40, 0, 31), (2, 1, 12, 12, 12, 0)):
        T, page = 9, 4
        D = -(-max(d, dv) // 16) * 16
        qkv = rng.normal(size=(T, (H + G) * d + G * dv))
        qkv[:, :d] *= 20.0                                                    # the first q head is loud
        qkv = torch.tensor(qkv, dtype=torch.float32)
        qn, kn = rng.uniform(0.5, 2, size=H * d), rng.uniform(0.5, 2, size=G * d)
        factor = np.full(H, 0.37)
        pos = np.array([0, 1, 5, 6, 7, 13, 70000, 62, 63])
        slots = torch.tensor([5, 4, -1, 7, 0, 1, 2, 11, 3], dtype=torch.int32)
        cache = torch.zeros((3, 2, G, page, D), dtype=TORCH[dtype], device=DEV)
        q = ops.attention_prepare(dev(qkv), cache, dev(qn, torch.float32), dev(kn, torch.float32), 1e-5,
                                  rotary_frequencies(dims, 300.0).to(DEV), dims, True, dev(pos.astype(np.int32)),
                                  dev(slots), dev(factor, torch.float32), H, G, d, dv, D, norm_whole=True,
                                  temp_coef=0.45, temp_every=every, out_dtype=TORCH[dtype])
        assert q.dtype == TORCH[dtype]
        x = qkv.double().numpy()
        q_ref = P.plain_norm(x[:, :H * d], qn, 1e-5).reshape(T, H, d)
        k_ref = P.plain_norm(x[:, H * d:(H + G) * d], kn, 1e-5).reshape(T, G, d)
        if dims:
            q_ref, k_ref = P.rotate_interleaved(q_ref, pos, dims, 300.0), P.rotate_interleaved(k_ref, pos, dims, 300.0)
        temp = P.query_temperature(pos, 0.45, every) if every else np.ones(T)
        tol = 3e-6 if dtype == "float32" else 8e-3
        assert rel(q[:, :, :d], q_ref * 0.37 * temp[:, None, None]) < tol
        for h in range(1, H):                                                 # quiet heads are held to their own size
            assert rel(q[:, h, :d], (q_ref * 0.37 * temp[:, None, None])[:, h]) < tol
        assert float(q[:, :, d:].abs().max()) == 0.0 if D > d else True
        for t in range(T):
            s = int(slots[t])
            if s >= 0:
                assert rel(cache[s // page, 0, :, s % page, :d], k_ref[t]) < tol
                assert rel(cache[s // page, 1, :, s % page, :dv], x[t, (H + G) * d:].reshape(G, dv)) < tol
        assert float(cache[2, :, :, 0].abs().max()) == 0.0 and float(cache[1, :, :, 2].abs().max()) == 0.0   # places 8, 6


# ---- attention kernels with a sink and a gate ---------------------------------------------------------------

def paged_kv(k, v, page, D, dtype, seed):
    """Keys and values [n, G, *] behind a block table whose pages are in a shuffled order."""
    n, G = k.shape[:2]
    pages = -(-n // page)
    order = np.random.default_rng(seed).permutation(pages + 3)[:pages]
    cache = torch.zeros((pages + 3, 2, G, page, D), dtype=dtype)
    for j in range(n):
        cache[order[j // page], 0, :, j % page, :k.shape[2]] = k[j].to(dtype)
        cache[order[j // page], 1, :, j % page, :v.shape[2]] = v[j].to(dtype)
    return cache, torch.tensor(order[None, :].astype(np.int32))


def plain_sink_rows(q, k, v, pos, sink, gate):
    """q [H, d] at position ``pos`` over keys k [n, G, d], values v [n, G, dv]; scale already inside q."""
    H, G = q.shape[0], k.shape[1]
    grp = torch.arange(H) // (H // G)
    s = torch.einsum("hd,jhd->hj", q, k[:pos + 1][:, grp])
    m = torch.maximum(s.max(dim=1).values, sink)
    e = torch.exp(s - m[:, None])
    o = torch.einsum("hj,jhd->hd", e, v[:pos + 1][:, grp]) / (e.sum(dim=1) + torch.exp(sink - m))[:, None]
    return o * torch.sigmoid(gate)[:, None]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,d,dv,page", [(4, 2, 16, 8, 8), (6, 2, 112, 80, 16), (3, 3, 24, 40, 16), (2, 1, 16, 16, 4),
                                           (8, 8, 32, 32, 32), (5, 1, 12, 20, 16), (4, 4, 64, 64, 16),
                                           (16, 2, 128, 128, 64), (12, 1, 64, 32, 16), (4, 2, 160, 96, 16),
                                           (2, 1, 256, 64, 16), (6, 2, 144, 144, 8), (3, 1, 40, 200, 16)])
def test_sink_attention_kernels_alone(H, G, d, dv, page, dtype):
    """Head 0 of the last query points at one key (the first, at page borders, far back, the last); head 1 has a
    sink so large that most of its weight goes nowhere, head 2 (if there is one) a sink that does not matter; the
    gates differ per head.  A sink that is left out, counted per split or scaled, or a gate on the wrong head,
    changes a row by its whole size.  The query is a single token and the end of a portion of 70; in bfloat16
    also through the tensor-core kernels (the split kernel in one part and in several, and the flash-style one)."""
    from railgun_b200 import ops
    n = 333
    D = -(-max(d, dv) // 16) * 16
    rng = np.random.default_rng(H * d + page)
    for key in (0, page - 1, page, 150, n - page - 1, n - 1):
        k = torch.tensor(rng.normal(size=(n, G, d)), dtype=TORCH[dtype]).double()
        v = torch.tensor(rng.normal(size=(n, G, dv)), dtype=TORCH[dtype]).double()
        q = torch.tensor(rng.normal(size=(H, d)) * d ** -0.5, dtype=TORCH[dtype]).double()
        k[key, 0] = (k[key, 0] * 1.5).to(TORCH[dtype]).double()                             # a loud key
        q[0] = (k[key, 0] * 4.0).to(TORCH[dtype]).double()
        sink = torch.tensor(rng.normal(size=H) * 2.0, dtype=torch.float32)
        sink[1 % H] = 9.0
        if H > 2:
            sink[2] = -30.0
        cache, table = paged_kv(k, v, page, D, TORCH[dtype], key)
        for portion in (1, 70):
            qs = torch.zeros((portion, H, D), dtype=TORCH[dtype])
            qs[:, :, :d] = torch.tensor(rng.normal(size=(portion, H, d)) * d ** -0.5, dtype=TORCH[dtype])
            qs[-1, :, :d] = q.to(TORCH[dtype])
            # the gate lives behind other columns of a wider buffer, as it does behind q, k and v
            wide = torch.tensor(rng.normal(size=(portion, 5 + H)) * 2.0, dtype=TORCH[dtype])
            gate = wide[:, 5:]
            ref = plain_sink_rows(q, k, v, n - 1, sink.double(), gate[-1].double())
            no_sink = plain_sink_rows(q, k, v, n - 1, torch.full((H,), -1e9, dtype=torch.float64), gate[-1].double())
            assert (ref[1 % H] - no_sink[1 % H]).abs().max() > 0.5 * no_sink[1 % H].abs().max()   # the sink matters
            positions = torch.arange(n - portion, n, dtype=torch.int32)
            wide_dev = dev(wide)
            got = ops.paged_attention_general(dev(qs).view(portion, H * D), H * D, dev(cache), dev(table),
                                              dev(torch.zeros(portion, dtype=torch.int32)), dev(positions), H, G, D,
                                              0, 1.0, 0, sink=dev(sink), gate=wide_dev[:, 5:])
            assert rel(got[-1].view(H, D)[:, :dv], ref) < (2e-5 if dtype == "float32" else 2e-2), f"key {key}"
            assert D == dv or float(got.view(portion, H, D)[:, :, dv:].abs().max()) == 0.0
            e = portion // 2                                                   # an earlier query of the portion
            ref_e = plain_sink_rows(qs[e, :, :d].double(), k, v, int(positions[e]), sink.double(), gate[e].double())
            assert rel(got[e].view(H, D)[:, :dv], ref_e) < (2e-5 if dtype == "float32" else 2e-2)
            if dtype == "bfloat16":
                outs = []
                if portion == 1:
                    for splits in (1, 3, 8):
                        o = torch.full((1, H * D), 7.0, dtype=torch.bfloat16, device=DEV)
                        ops.decode_attention(dev(qs).view(1, H * D), H * D, o, dev(cache), dev(table), None, 1,
                                             dev(torch.zeros(1, dtype=torch.int32)), dev(positions), H, G, D, 0,
                                             1.0, splits, sink=dev(sink), gate=wide_dev[:, 5:])
                        outs.append(o)
                    o = torch.full((1, H * D), 7.0, dtype=torch.bfloat16, device=DEV)
                    ops.decode_attention(dev(qs).view(1, H * D), H * D, o, dev(cache), dev(table), None, 1,
                                         dev(torch.zeros(1, dtype=torch.int32)), dev(positions), H, G, D, 0,
                                         1.0, 4, fused_reduce=True, sink=dev(sink), gate=wide_dev[:, 5:])
                    outs.append(o)
                else:
                    tiles = torch.tensor([[0, 64, 0], [64, portion - 64, 0]], dtype=torch.int32)
                    o = torch.full((portion, H * D), 7.0, dtype=torch.bfloat16, device=DEV)
                    ops.prefill_attention(dev(qs).view(portion, H * D), H * D, o, dev(cache), dev(table), dev(tiles),
                                          dev(positions), H, G, D, 0, 1.0, sink=dev(sink), gate=wide_dev[:, 5:])
                    outs.append(o)
                for o in outs:
                    assert rel(o[-1].view(H, D)[:, :dv], ref) < 2e-2, f"key {key}, tensor cores"
                    assert rel(o, got) < 3e-2


def test_attention_kernels_without_sink_are_unchanged():
    """No sink and no gate: the plain softmax, as the other designs use the kernels."""
    from railgun_b200 import ops
    rng = np.random.default_rng(1)
    H, G, d, n, page = 4, 2, 32, 100, 16
    k = torch.tensor(rng.normal(size=(n, G, d)), dtype=torch.bfloat16).double()
    v = torch.tensor(rng.normal(size=(n, G, d)), dtype=torch.bfloat16).double()
    q = torch.tensor(rng.normal(size=(H, d)) * 0.3, dtype=torch.bfloat16)
    cache, table = paged_kv(k, v, page, d, torch.bfloat16, 0)
    grp = torch.arange(H) // (H // G)
    s = torch.einsum("hd,jhd->hj", q.double(), k[:, grp])
    ref = torch.einsum("hj,jhd->hd", torch.softmax(s, dim=-1), v[:, grp])
    pos = dev(torch.tensor([n - 1], dtype=torch.int32))
    zero = dev(torch.zeros(1, dtype=torch.int32))
    got = ops.paged_attention_general(dev(q).view(1, H * d), H * d, dev(cache), dev(table), zero, pos, H, G, d, 0, 1.0)
    o = torch.empty((1, H * d), dtype=torch.bfloat16, device=DEV)
    ops.decode_attention(dev(q).view(1, H * d), H * d, o, dev(cache), dev(table), None, 1, zero, pos, H, G, d, 0, 1.0, 2)
    assert rel(got.view(H, d), ref) < 2e-2 and rel(o.view(H, d), ref) < 2e-2


# ---- lightning attention -------------------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,d,dv", [(2, 16, 8), (1, 32, 48), (5, 12, 10), (4, 64, 32), (3, 128, 64), (2, 200, 72)])
def test_lightning_alone(H, d, dv, dtype):
    """silu on q, k and v; S carried in the slot from an earlier step beside a new request in a dirty slot and a
    single token; a far key made loud and the last query pointed at it; one root mean square over all heads with a
    weight of that size; a sigmoid gate."""
    from railgun_b200 import ops
    from railgun_b200.parts.latent_attention import rotary_frequencies
    rng = np.random.default_rng(H + d)
    lengths, starts, slots = [40, 75, 1], [0, 33, 9], [2, 0, 3]
    T = sum(lengths)
    cols = 2 * H * d + 2 * H * dv
    proj = rng.normal(size=(T, cols)) * 0.7
    proj[45, H * d:H * d + d] = 3.0                                            # a loud key early in request 1 ...
    proj[114, :d] = 3.0                                                        # ... that its last query asks for
    proj = torch.tensor(proj, dtype=TORCH[dtype])
    decay = np.linspace(1.0, 0.9, H)
    state0 = rng.normal(size=(4, H, dv, d)) * 0.3
    state = dev(state0, torch.float32)
    batch = step_batch(lengths, starts, slots)
    q, k, v = ops.retention_prepare(dev(proj), 0, H * d, rotary_frequencies(0, 10.0).to(DEV), 0, batch.positions, H, d,
                                    1.0, silu=True, v_off=2 * H * d, dv=dv)
    x = proj.double().numpy()
    qr, kr = P.silu(x[:, :H * d]).reshape(T, H, d), P.silu(x[:, H * d:2 * H * d]).reshape(T, H, d)
    vr = P.silu(x[:, 2 * H * d:2 * H * d + H * dv]).reshape(T, H, dv)
    assert rel(q, qr) < 2e-6 and rel(k, kr) < 2e-6 and rel(v.view(T, H, dv), vr) < 2e-6
    o = ops.state_scan(q.view(T, H * d), k.view(T, H * d), v, state, batch, H, d, dv, decay=dev(decay, torch.float32))
    refs, at = [], 0
    for n, start, slot in zip(lengths, starts, slots):
        S0 = None if start == 0 else np.transpose(state0[slot], (0, 2, 1))
        ro, S = P.lightning_scan(qr[at:at + n], kr[at:at + n], vr[at:at + n], decay, S0)
        refs.append(ro)
        assert rel(state[slot], np.transpose(S, (0, 2, 1))) < 3e-5
        at += n
    ref = np.concatenate(refs)
    assert rel(o, ref) < 3e-5
    assert np.abs(ref[114, 0]).max() > 5 * np.median(np.abs(ref[:, 0]))      # the far key is heard
    w = rng.uniform(0.5, 2, size=H * dv)
    z = ops.head_norm_gate(o, dev(proj)[:, 2 * H * d + H * dv:], dev(w, torch.float32), 1e-5, TORCH[dtype], whole=True,
                           gate_kind="sigmoid")
    zr = P.plain_norm(ref.reshape(T, H * dv), w, 1e-5) * P.sigmoid(x[:, 2 * H * d + H * dv:])
    assert rel(z, zr) < (3e-5 if dtype == "float32" else 8e-3)


# ---- the experts ---------------------------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,layer", [("A", 0), ("A", 3), ("B", 0), ("C", 0), ("C", 2), ("D", 1), ("D", 3)])
def test_experts_alone(name, layer, dtype):
    """Sigmoid scores, the largest chosen, not renormalized, on the experts' input: with the square of relu a
    weight that sat on the output instead would give other numbers (s against s^2)."""
    from railgun_b200.engine.runner import ModelRunner
    cfg, _, page = C.CASES[name]
    plain = C.plain_model(name)
    runner = ModelRunner(C.model_dir(name), dtype=dtype, page_size=page, max_tokens=64, max_requests=1)
    rng = np.random.default_rng(layer)
    mlp = cfg["layers"][layer]["mlp"]
    p = f"l{layer}.mlp."
    for T in (1, 5, 70, 1100):
        h = torch.tensor(rng.normal(size=(T, cfg["width"])) * 0.7, dtype=torch.float32).to(TORCH[dtype])
        x = h.double().numpy()
        ref = P.expert_ff(x, plain.w, p, mlp)
        margins = []
        P.router_choice(x, plain.w, p, mlp, margins)
        got = runner.model.layers[layer].ffn.forward(h.to(DEV), None).float().cpu().numpy()
        sure = margins[0] > (1e-4 if dtype == "float32" else CLOSE_CALL)
        assert T < 70 or sure.sum() >= 0.5 * T
        if not sure.any():
            continue
        assert rel(got[sure], ref[sure]) < TOL[dtype]
        ids, wt = P.router_choice(x, plain.w, p, mlp)
        on_output = np.zeros_like(x)
        for t in range(T):
            for e, sc in zip(ids[t], wt[t]):
                on_output[t] += sc * (plain.w[f"{p}e{e}.down"] @ np.maximum(plain.w[f"{p}e{e}.up"] @ x[t], 0.0) ** 2)
        assert rel(on_output[sure], ref[sure]) > 1e-2


# ---- the model through the step function ---------------------------------------------------------------

LENGTHS = {"A": [1, 2, 9, 12, 40, 77, 150, 64], "B": [1, 3, 17, 64, 100, 33], "C": [1, 6, 10, 33, 90, 65],
           "D": [2, 131, 260, 400, 55, 129, 181], "E": [1, 2, 5, 23, 70, 41]}
PORTIONS = {"D": (130, 2, 64, 7, 128, 3, 65, 2, 33, 129)}
MIXED = {"D": (5, 1, 2, 70, 1, 1, 3, 140, 1, 2, 128, 17)}
TAIL = {"D": 140, "B": 60}                          # the query factor's steps at 50, 100 and 128 fall on decoded tokens
_oracle: dict = {}


def oracle(name):
    if name not in _oracle:
        cfg = C.CASES[name][0]
        reqs = {f"r{i}": p for i, p in enumerate(C.prompts(cfg["vocab"], LENGTHS[name], seed=21))}
        plain = C.plain_model(name)
        both = {k: plain.forward_with_margins(v) for k, v in reqs.items()}
        _oracle[name] = (reqs, {k: v[0] for k, v in both.items()}, {k: v[1] for k, v in both.items()})
    return _oracle[name][:2]


def margins_of(name):
    oracle(name)
    return _oracle[name][2]


def make_trace(mode, reqs, name):
    if mode == "whole":
        return helpers.trace_whole(reqs)
    if mode == "tail":
        return helpers.trace_tail_decode(reqs, TAIL.get(name, 32))
    if mode == "every_token":
        return helpers.trace_tail_decode(reqs, 10 ** 6)
    if mode == "portions":
        return helpers.trace_portions(reqs, **({"sizes": PORTIONS[name]} if name in PORTIONS else {}))
    if mode == "mixed":
        return helpers.trace_mixed(reqs, max_live=4, seed=5, **({"sizes": MIXED[name]} if name in MIXED else {}))
    raise ValueError(mode)


def replay(folder, cfg, page, dtype, steps, out_dir, **more):
    from railgun_b200.engine.runner import ModelRunner
    from railgun_b200.replay import Replayer
    runner = ModelRunner(folder, dtype=dtype, page_size=page, max_tokens=helpers.peak_tokens(steps, 64),
                         max_requests=4, **more)
    rp = Replayer(runner, out_dir)
    for s in steps:
        rp.feed(s)
    runner.check_device_errors()
    runner.alloc.check()
    assert runner.alloc.num_requests() == 0
    return helpers.collect(steps, out_dir, cfg["vocab"])


def replay_case(name, dtype, steps, out_dir, page=None, **more):
    cfg, _, own_page = C.CASES[name]
    return replay(C.model_dir(name), cfg, page or own_page, dtype, steps, out_dir, **more)


def compare(rows, reqs, logits, tol, what, margins=None):
    """Every position within ``tol`` of the largest logit.  With ``margins`` (bfloat16: per request and position the
    smallest router margin): positions whose routing is a close call are held to LOOSE only, and of the others at
    most one in fifty may be over ``tol`` (they come after a close call that went the other way)."""
    worst, held, over = 0.0, 0, 0
    for name, toks in reqs.items():
        ref = logits[name]
        scale = np.abs(ref).max()
        for p in range(len(toks)):
            err = np.abs(rows[(name, p)] - ref[p]).max() / scale
            if margins is None:
                assert err <= tol, (f"{what}: request {name} (length {len(toks)}) first differs at position {p}: "
                                    f"relative error {err:.3e}")
            else:
                assert err <= LOOSE, f"{what}: request {name} position {p}: relative error {err:.3e}"
                clear = margins[name][p] >= CLOSE_CALL
                held += clear
                over += bool(clear and err > tol)
            worst = max(worst, err)
    if margins is not None:
        total = sum(len(t) for t in reqs.values())
        assert held >= 0.5 * total and over <= 1 + 0.02 * held, f"{what}: {over} of {held} clear positions over {tol}"
    return worst


@pytest.mark.parametrize("mode", ["whole", "tail", "portions", "mixed"])
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(C.CASES))
def test_replay_matches_plain(name, dtype, mode, tmp_path):
    """Whole prompts; the last tokens one by one; portions down to two tokens, cut inside pages and inside the
    reach of the convolutions; up to four live requests in a pool so small that pages and state slots are used
    again.  Every position of every request is compared, the first tokens included."""
    reqs, logits = oracle(name)
    rows = replay_case(name, dtype, make_trace(mode, reqs, name), tmp_path)
    margins = margins_of(name) if dtype == "bfloat16" else None
    print(f"{name} {dtype} {mode}: worst relative error "
          f"{compare(rows, reqs, logits, TOL[dtype], f'{name} {dtype} {mode}', margins):.3e}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C", "E"])
def test_every_token_decoded_alone_matches_whole_prompts(name, dtype, tmp_path):
    """Token-by-token decoding from the first token on (through the decode graphs and with graphs off): states
    and convolution tails that start from nothing, query factors that step between decoded tokens."""
    reqs, logits = oracle(name)
    few = dict(list(reqs.items())[1:5])
    steps = make_trace("every_token", few, name)
    margins = margins_of(name) if dtype == "bfloat16" else None
    compare(replay_case(name, dtype, steps, tmp_path / "g"), few, logits, TOL[dtype], "decoded", margins)
    compare(replay_case(name, dtype, steps, tmp_path / "e", use_graphs=False), few, logits, TOL[dtype],
            "decoded, no graphs", margins)


@pytest.mark.parametrize("page", [2, 64])
def test_other_page_sizes(page, tmp_path):
    reqs, logits = oracle("A")
    for mode in ("portions", "mixed"):
        steps = make_trace(mode, reqs, "A")
        compare(replay_case("A", "float32", steps, tmp_path / mode, page=page), reqs, logits, TOL["float32"],
                f"page {page}")


def test_batch_of_unequal_requests_equals_each_alone(tmp_path):
    """One step with four prompts of unequal length beside one another, then single tokens of all four in one
    step: the rows equal those of each request run alone."""
    reqs, logits = oracle("D")
    names = list(reqs)[:4]
    together = [{"step": 0, "entries": [{"id": n, "tokens": reqs[n][:-1], "want": list(range(len(reqs[n]) - 1))}
                                         for n in names], "end": []},
                {"step": 1, "entries": [{"id": n, "tokens": reqs[n][-1:], "want": [0]} for n in names], "end": names}]
    alone, k = [], 0
    for n in names:
        alone.append({"step": k, "entries": [{"id": n, "tokens": reqs[n][:-1], "want": list(range(len(reqs[n]) - 1))}],
                      "end": []})
        alone.append({"step": k + 1, "entries": [{"id": n, "tokens": reqs[n][-1:], "want": [0]}], "end": [n]})
        k += 2
    for dtype in DTYPES:
        a = replay_case("D", dtype, together, tmp_path / f"t{dtype}")
        b = replay_case("D", dtype, alone, tmp_path / f"a{dtype}")
        compare(a, {n: reqs[n] for n in names}, logits, TOL[dtype], "together",
                margins_of("D") if dtype == "bfloat16" else None)
        apart = [key for key in a
                 if np.abs(a[key] - b[key]).max() > (2e-5 if dtype == "float32" else 0.25) * np.abs(b[key]).max()]
        assert len(apart) <= (0 if dtype == "float32" else 1 + 0.02 * len(a)), apart[:5]


def test_sinks_and_sharp_attention_show(tmp_path):
    """With sinks as large as the largest scores (and the attention layers' scores doubled) a sink that is forgotten, counted once per split or scaled, or one key too many, moves the logits
    by far more than the tolerance.  Prompts, portions, decoding and mixed batches."""
    cfg, seed, page = C.CASES["D"]

    def sharpen(t):
        for i, L in enumerate(cfg["layers"]):
            if L["type"] == "parallel":
                t[f"l{i}.mix.left.sink"] = np.abs(t[f"l{i}.mix.left.sink"]) * 2.0 + 6.0
            else:
                t[f"l{i}.mix.q"] *= 2.0

    folder = C.write_model(cfg, seed + 1, tmp_path / "model", change=sharpen)
    plain = C.Plain(folder)
    reqs = {f"s{i}": p for i, p in enumerate(C.prompts(cfg["vocab"], [190, 135, 52, 300], seed=4))}
    logits = {k: plain.forward(v) for k, v in reqs.items()}
    # the sinks matter: the same model with its learned sinks far below every score answers differently, and so
    # does the one whose attention layers have no sink of score 0
    w2 = dict(plain.w)
    for i, L in enumerate(cfg["layers"]):
        if L["type"] == "parallel":
            w2[f"l{i}.mix.left.sink"] = plain.w[f"l{i}.mix.left.sink"] - 60.0
    moved = P.forward(reqs["s0"], w2, cfg)
    scale = np.abs(logits["s0"]).max()
    assert np.abs(moved[-1] - logits["s0"][-1]).max() > 50 * TOL["float32"] * scale
    for mode in ("whole", "tail", "portions", "mixed"):
        steps = make_trace(mode, reqs, "D")
        rows = replay(folder, cfg, page, "float32", steps, tmp_path / mode)
        compare(rows, reqs, logits, TOL["float32"], f"sharp {mode}")
    both = {k: plain.forward_with_margins(v) for k, v in reqs.items()}
    rows = replay(folder, cfg, page, "bfloat16", make_trace("mixed", reqs, "D"), tmp_path / "bf16")
    compare(rows, reqs, logits, 2 * TOL["bfloat16"], "sharp mixed bfloat16", {k: v[1] for k, v in both.items()})


def test_states_remember_a_far_token(tmp_path):
    """A model whose left halves are silenced (their output norms' weights are zero), so that only the lightning
    states carry anything from token to token, and in which one token of the vocabulary has keys and values ten
    times louder than the others in the first layer: a prompt that has that token in second place still differs
    from one that does not after 300 more tokens, most of them decoded one by one, and both equal the plain
    model's."""
    cfg, _, page = C.CASES["D"]
    only = dict(cfg, layers=[L for L in cfg["layers"] if L["type"] == "parallel"])
    loud, j = 11, 5

    def change(t):
        for i in range(len(only["layers"])):
            t[f"l{i}.mix.left.out"] *= 0.0
        t["embed"][loud] = 0.0
        t["embed"][loud, j] = 3.0                                              # all of the row in one place ...
        t["l0.mix.right.k"][:, j] *= 10.0                                      # ... that keys and values listen to
        t["l0.mix.right.v"][:, j] *= 10.0

    folder = C.write_model(only, 17, tmp_path / "model", change=change)
    plain = C.Plain(folder)
    b = [t if t != loud else loud + 1 for t in C.prompts(cfg["vocab"], [310], seed=9)[0]]
    a = list(b)
    a[1] = loud
    reqs = {"a": a, "b": b}
    logits = {k: plain.forward(v) for k, v in reqs.items()}
    scale = np.abs(logits["a"]).max()
    assert np.abs(logits["a"][-1] - logits["b"][-1]).max() > 20 * TOL["float32"] * scale
    steps = helpers.trace_tail_decode(reqs, 250)
    compare(replay(folder, only, page, "float32", steps, tmp_path / "o"), reqs, logits, TOL["float32"], "far")


def test_attention_hears_a_far_token(tmp_path):
    """An attention-only model: prompts that differ in the first token only differ at the end of 400 tokens,
    in portions and decoded across page borders."""
    cfg, _, page = C.CASES["D"]
    only = dict(cfg, layers=[L for L in cfg["layers"] if L["type"] == "attention"])
    folder = C.write_model(only, 23, tmp_path / "model")
    plain = C.Plain(folder)
    a = C.prompts(cfg["vocab"], [400], seed=10)[0]
    b = list(a)
    b[0] = (a[0] + 7) % cfg["vocab"]
    reqs = {"a": a, "b": b}
    logits = {k: plain.forward(v) for k, v in reqs.items()}
    assert np.abs(logits["a"][-1] - logits["b"][-1]).max() > 20 * TOL["float32"] * np.abs(logits["a"]).max()
    for mode in ("tail", "portions"):
        compare(replay(folder, only, page, "float32", make_trace(mode, reqs, "D"), tmp_path / mode), reqs, logits,
                TOL["float32"], f"far {mode}")


# ---- generation through the engine and the command line -----------------------------------------------

def greedy_consistent(plain, prompt, out, tol):
    """How many generated tokens are the plain model's choice given the tokens before them (teacher-forced), up
    to ``tol`` of the largest absolute logit."""
    logits = plain.forward(list(prompt) + list(out))
    return sum(int(logits[len(prompt) - 1 + i][t] >= logits[len(prompt) - 1 + i].max() - tol * np.abs(logits).max())
               for i, t in enumerate(out))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "C"])
def test_greedy_generation_through_the_engine(name, dtype):
    """Prompts of one token and more, prefilled in portions by the scheduler beside decoding requests."""
    from railgun_b200.engine.engine import Engine
    from railgun_b200.engine.request import SamplingParams
    cfg, _, page = C.CASES[name]
    prompts = C.prompts(cfg["vocab"], [1, 2, 9, 40, 63, 100], seed=2)
    plain = C.plain_model(name)
    eng = Engine(C.model_dir(name), dtype=dtype, block_size=page, num_gpu_blocks=1024 // page, max_num_seqs=4,
                 max_num_batched_tokens=64, max_prefill_chunk=24, max_model_len=256)
    outs = eng.generate(prompts, SamplingParams(max_new_tokens=10))
    good = 0
    for p, o in zip(prompts, outs):
        assert o.finish_reason == "max_tokens" and len(o.token_ids) == 10
        good += greedy_consistent(plain, p, o.token_ids, 1e-4 if dtype == "float32" else 6e-2)
        if dtype == "float32":
            assert o.token_ids == plain.greedy(p, 10)
    assert good == 60
    assert eng.stats()["num_free_blocks"] == 1024 // page and not eng.has_unfinished()


def test_long_decoding_through_the_engine():
    from railgun_b200.engine.engine import Engine
    from railgun_b200.engine.request import SamplingParams
    cfg, _, page = C.CASES["A"]
    plain = C.plain_model("A")
    prompt = C.prompts(cfg["vocab"], [3], seed=8)[0]
    eng = Engine(C.model_dir("A"), dtype="float32", block_size=page, num_gpu_blocks=100, max_num_seqs=2,
                 max_model_len=400)
    out = eng.generate([prompt], SamplingParams(max_new_tokens=300))[0]
    assert len(out.token_ids) == 300
    assert greedy_consistent(plain, prompt, out.token_ids, 1e-4) == 300


def test_command_line_and_trace_runner(tmp_path):
    d = C.model_dir("C")
    plain = C.plain_model("C")
    prompt = [7, 80, 3, 55]
    res = subprocess.run([sys.executable, "-m", "railgun_b200", "generate", "-m", str(d), "--prompt-ids",
                          ",".join(map(str, prompt)), "--max-tokens", "6", "--dtype", "f32", "--block-size", "8"],
                         cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    line = [l for l in res.stdout.splitlines() if l and l[0].isdigit()][0]
    assert [int(t) for t in line.split(",")] == plain.greedy(prompt, 6)
    toks = C.prompts(90, [30], seed=6)[0]
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": toks[:19], "want": [0, 18]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": toks[19:21], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": toks[21:], "want": [8]}], "end": ["a"]}]
    res = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", str(d), "--dtype", "float32", "--out",
                          str(tmp_path), "--max-tokens", "64"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                         cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    assert [l for l in res.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    ref = plain.forward(toks)
    got0 = np.fromfile(tmp_path / "0.f32", dtype="<f4").reshape(2, 90)
    got2 = np.fromfile(tmp_path / "2.f32", dtype="<f4").reshape(1, 90)
    assert not (tmp_path / "1.f32").exists()
    scale = np.abs(ref).max()
    assert np.abs(got0 - ref[[0, 18]]).max() < 1e-4 * scale and np.abs(got2[0] - ref[29]).max() < 1e-4 * scale

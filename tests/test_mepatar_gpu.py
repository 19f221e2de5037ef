"""Mepatar on the GPU against the plain statement: each mechanism alone, then
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
import mepatar_cases as C
import plain_mepatar as P

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DEV = torch.device("cuda:0")
DTYPES = ["float32", "bfloat16"]
TORCH = {"float32": torch.float32, "bfloat16": torch.bfloat16}
# bfloat16: the test weights are several times larger than a trained model's, so rounding alone moves a few
# logits in a hundred by some 1e-2 of the largest, the same in every cut; a lost key, state or tap is caught
# by the tests of the mechanisms alone, where it changes a row by its whole size
TOL = {"float32": 5e-5, "bfloat16": 6e-2}


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


# ---- the norm in groups ------------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,W,groups", [(3, 24, 1), (5, 64, 2), (9, 48, 3), (300, 256, 4), (2, 40, 5), (70, 1536, 6),
                                          (4, 30, 3), (6, 42, 7), (33, 2050, 1)])
def test_group_norm_alone(T, W, groups, dtype):
    """The residual takes the pending rows in 32-bit; two norms read the same sum; one loud part stays alone."""
    from railgun_b200 import ops
    rng = np.random.default_rng(T + W)
    x = rng.normal(size=(T, W)).astype(np.float32)
    x[:, :W // groups] *= 50.0
    y = torch.tensor(rng.normal(size=(T, W)), dtype=TORCH[dtype])
    w1, w2 = rng.uniform(0.5, 2, size=W).astype(np.float32), rng.uniform(0.5, 2, size=W).astype(np.float32)
    resid = dev(x.copy())
    a, b = ops.add_group_rmsnorm(resid, y.to(DEV), [dev(w1), dev(w2)], groups, 1e-5, TORCH[dtype])
    total = x.astype(np.float64) + y.double().numpy()
    assert rel(resid, total) < 1e-6
    tol = 2e-6 if dtype == "float32" else 6e-3
    assert rel(a, P.group_norm(total, w1, groups, 1e-5)) < tol and rel(b, P.group_norm(total, w2, groups, 1e-5)) < tol
    rows = dev(np.array([T - 1, 0], dtype=np.int32))
    (c,) = ops.add_group_rmsnorm(resid, None, [dev(w1)], groups, 1e-5, torch.float32, rows=rows)
    assert rel(c, P.group_norm(total, w1, groups, 1e-5)[[T - 1, 0]]) < 2e-6


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("I", [24, 12, 7, 512])
def test_gated_activations_alone(I, dtype):
    """gate | up rows through the three gated activations, with numbers on both sides of the clamps."""
    from railgun_b200 import ops
    rng = np.random.default_rng(I)
    gu = torch.tensor(rng.normal(size=(37, 2 * I)) * 2.0, dtype=TORCH[dtype])
    g, u = gu[:, :I].double().numpy(), gu[:, I:].double().numpy()
    silu = lambda z: z / (1.0 + np.exp(-z))
    want = {"silu": silu(g) * u, "gelu_tanh": P.gelu_tanh(g) * u,
            "clamped_swish": np.minimum(g, 1.25) / (1.0 + np.exp(-1.702 * np.minimum(g, 1.25))) * (np.clip(u, -1.25, 1.25) + 1.0)}
    for kind, ref in want.items():
        got = ops.gated_activation(gu.to(DEV), kind, 1.25)
        assert rel(got, ref) < (2e-6 if dtype == "float32" else 6e-3), kind


# ---- the short convolution and its state ---------------------------------------------------------------

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("C_,K", [(48, 4), (40, 1), (200, 2), (64, 5), (300, 3)])
def test_convolution_continues_from_the_state(C_, K, dtype):
    """Three requests side by side: a new one, one that continues from its slot's tail, one that brings a single
    token; then the slots hold the last K - 1 inputs, also where the step brought fewer than that."""
    from railgun_b200 import ops
    rng = np.random.default_rng(C_ + K)
    lengths, starts, slots = [5, 7, 1], [0, 9, 3], [2, 1, 3]
    T = sum(lengths)
    x = torch.tensor(rng.normal(size=(T, C_ + 8)), dtype=TORCH[dtype])
    taps = rng.normal(size=(C_, K))
    state = torch.tensor(rng.normal(size=(4, max(K - 1, 0), C_)), dtype=torch.float32)
    st = dev(state.clone()) if K > 1 else None
    batch = step_batch(lengths, starts, slots)
    xin = x.double().numpy()[:, 8:]
    past = lambda s: state[s].double().numpy()
    ref = np.concatenate([P.causal_conv(xin[:5], taps),
                          P.causal_conv(np.concatenate([past(1), xin[5:12]]), taps)[K - 1:],
                          P.causal_conv(np.concatenate([past(3), xin[12:]]), taps)[K - 1:]])
    tol = 2e-6 if dtype == "float32" else 8e-3
    plain = ops.causal_conv(dev(x), 8, dev(np.ascontiguousarray(taps.T), torch.float32), st, batch, torch.float32)
    assert rel(plain, ref) < 2e-6
    assert rel(ops.causal_conv(dev(x), 8, dev(np.ascontiguousarray(taps.T), torch.float32), st, batch, TORCH[dtype], residual=True), ref + xin) < tol
    assert rel(ops.causal_conv(dev(x), 8, dev(np.ascontiguousarray(taps.T), torch.float32), st, batch, torch.float32, silu=True), P.silu(ref)) < 2e-6
    if K > 1:
        assert torch.equal(st.cpu(), state)                                   # reading changes nothing
        ops.conv_state_update(dev(x), 8, st, batch)
        after = st.cpu().double().numpy()
        assert np.array_equal(after[0], past(0))                              # nobody's slot
        assert np.array_equal(after[2], np.concatenate([np.zeros((K - 1, C_)), xin[:5]])[-(K - 1):])
        assert np.array_equal(after[1], xin[5:12][-(K - 1):])
        assert np.array_equal(after[3], np.concatenate([past(3), xin[12:]])[-(K - 1):])


# ---- the matrix-state scans ----------------------------------------------------------------------------

def plain_scan(q, k, v, S, decay=None, g=None, beta=None):
    """One head: q, k [T, d], v [T, dv], S [d, dv] (changed in place).  Returns o [T, dv]."""
    o = np.zeros_like(v)
    for t in range(q.shape[0]):
        if beta is None:
            S *= decay
            S += np.outer(k[t], v[t])
        else:
            S *= g[t]
            S += np.outer(k[t], beta[t] * (v[t] - S.T @ k[t]))
        o[t] = S.T @ q[t]
    return o


@pytest.mark.parametrize("rule", ["retention", "delta"])
@pytest.mark.parametrize("H,Hqk,d,dv", [(4, 4, 32, 16), (4, 2, 16, 8), (3, 1, 8, 24), (1, 1, 32, 48), (5, 5, 12, 10),
                                        (2, 2, 128, 128), (8, 4, 64, 256), (2, 1, 200, 72), (1, 1, 256, 20)])
def test_state_scan_alone(H, Hqk, d, dv, rule):
    """Two requests in one step (one new with a slot full of another request's numbers, one continuing), then
    the continuing one token by token: rows and states equal the plain loop's.  One key far back is made loud
    and the last query points at it, so a state that forgets or starts late shows in full."""
    from railgun_b200 import ops
    rng = np.random.default_rng(H * d + dv)
    n0, n1, tail = 37, 130, 5
    T = n0 + n1
    q = rng.normal(size=(T + tail, Hqk, d)) * 0.3
    k = rng.normal(size=(T + tail, Hqk, d)) * 0.3
    v = rng.normal(size=(T + tail, H, dv))
    if rule == "delta":
        k /= np.linalg.norm(k, axis=-1, keepdims=True)
        q[-1] = 3.0 * k[n0 + 2]
    else:
        k[n0 + 2] *= 6.0
        q[-1] = k[n0 + 2]
    state0 = rng.normal(size=(3, H, dv, d))                           # the slots hold S transposed
    decay = np.linspace(0.97, 0.9995, H) if rule == "retention" else None
    g = rng.uniform(0.9, 1.0, size=(T + tail, H)) if rule == "delta" else None
    beta = rng.uniform(0.1, 1.0, size=(T + tail, H)) if rule == "delta" else None
    f32 = lambda a: dev(np.ascontiguousarray(a), torch.float32) if a is not None else None
    state = f32(state0)
    args = dict(decay=f32(decay)) if rule == "retention" else {}

    def run(lo, hi, lengths, starts, slots):
        more = dict(args) if rule == "retention" else dict(g=f32(g[lo:hi]), beta=f32(beta[lo:hi]))
        return ops.state_scan(f32(q[lo:hi].reshape(hi - lo, -1)), f32(k[lo:hi].reshape(hi - lo, -1)),
                              f32(v[lo:hi].reshape(hi - lo, -1)), state, step_batch(lengths, starts, slots), H, d, dv, **more)

    got = [run(0, T, [n0, n1], [0, 11], [2, 0])]
    for t in range(T, T + tail):
        got.append(run(t, t + 1, [1], [11 + n1 + t - T], [0]))
    got = torch.cat(got).cpu().double().numpy()
    grp = H // Hqk
    for h in range(H):
        S_new, S_old = np.zeros((d, dv)), state0[0, h].T.copy()
        kw = lambda lo, hi: dict(decay=decay[h]) if rule == "retention" else dict(g=g[lo:hi, h], beta=beta[lo:hi, h])
        ref0 = plain_scan(q[:n0, h // grp], k[:n0, h // grp], v[:n0, h], S_new, **kw(0, n0))
        ref1 = plain_scan(q[n0:, h // grp], k[n0:, h // grp], v[n0:, h], S_old, **kw(n0, T + tail))
        assert rel(got[:n0, h], ref0) < 2e-5 and rel(got[n0:, h], ref1) < 2e-5 and rel(got[-1, h], ref1[-1]) < 2e-5
        assert rel(state[2, h], S_new.T) < 2e-5 and rel(state[0, h], S_old.T) < 2e-5
    assert np.array_equal(state[1].cpu().numpy(), state0[1].astype(np.float32))           # nobody's slot


@pytest.mark.parametrize("dtype", DTYPES)
def test_prepare_kernels_alone(dtype):
    """Rotation in pairs (i, i + dims/2) at positions up to 70000 with k scaled; unit vectors, beta and the decay
    of the delta rule; the heads' norm with and without a weight times silu of the gate."""
    from railgun_b200 import ops
    from railgun_b200.parts.latent_attention import rotary_frequencies
    rng = np.random.default_rng(5)
    for H, d, dims in ((3, 16, 8), (2, 32, 32), (4, 12, 0), (1, 64, 2)):
        T = 6
        proj = torch.tensor(rng.normal(size=(T, 2 * H * d + 5)), dtype=TORCH[dtype])
        pos = np.array([0, 1, 2, 500, 70000, 3])
        q, k = ops.retention_prepare(dev(proj), 0, H * d, rotary_frequencies(dims, 300.0).to(DEV), dims,
                                     dev(pos.astype(np.int32)), H, d, 0.37)
        x = proj.double().numpy()
        assert rel(q, P.rotate(x[:, :H * d].reshape(T, H, d), pos, dims, 300.0, "half")) < 3e-6
        assert rel(k, 0.37 * P.rotate(x[:, H * d:2 * H * d].reshape(T, H, d), pos, dims, 300.0, "half")) < 3e-6
    for H, G, d in ((4, 2, 16), (3, 3, 24), (6, 1, 40)):
        T = 5
        qkv = rng.normal(size=(T, 2 * G * d + 7)).astype(np.float32)
        ab = torch.tensor(rng.normal(size=(T, 2 * H)) * 3.0, dtype=torch.float32)
        A, bias = rng.normal(size=H).astype(np.float32), rng.normal(size=H).astype(np.float32)
        buf = dev(qkv.copy())
        beta, g = ops.delta_prepare(buf, G, d, 0.25, 1e-6, dev(ab), 0, H, dev(A), dev(bias), H)
        x = qkv.astype(np.float64)
        unit = lambda a: a / np.sqrt((a * a).sum(-1, keepdims=True) + 1e-6)
        assert rel(buf[:, :G * d], 0.25 * unit(x[:, :G * d].reshape(T, G, d)).reshape(T, -1)) < 2e-6
        assert rel(buf[:, G * d:2 * G * d], unit(x[:, G * d:2 * G * d].reshape(T, G, d)).reshape(T, -1)) < 2e-6
        assert np.array_equal(buf[:, 2 * G * d:].cpu().numpy(), qkv[:, 2 * G * d:])
        assert rel(beta, P.sigmoid(ab.double().numpy()[:, :H])) < 2e-6
        assert rel(g, np.exp(-np.exp(A.astype(np.float64)) * P.softplus(ab.double().numpy()[:, H:] + bias))) < 2e-6
    for H, dv in ((3, 8), (2, 80), (5, 33)):
        T = 4
        o = rng.normal(size=(T, H, dv)).astype(np.float32) * 7.0
        gate = torch.tensor(rng.normal(size=(T, H * dv + 3)), dtype=TORCH[dtype])
        w = rng.uniform(0.5, 2, size=dv).astype(np.float32)
        tol = 2e-6 if dtype == "float32" else 8e-3
        for weight in (None, w):
            got = ops.head_norm_gate(dev(o), dev(gate)[:, :H * dv], dev(weight) if weight is not None else None, 1e-5,
                                     TORCH[dtype])
            ref = P.unit_rms(o.astype(np.float64), 1e-5) * (weight if weight is not None else 1.0)
            assert rel(got, ref.reshape(T, -1) * P.silu(gate.double().numpy()[:, :H * dv])) < tol


# ---- windowed attention that keeps the first tokens, over hand-made rows ----------------------------------

def paged_kv(k, v, page, D, seed, dtype):
    """k [n, G, d] and v [n, G, dv] of one request over shuffled pages: (cache [pages, 2, G, page, D], table [1, blocks])."""
    n, G = k.shape[:2]
    blocks = -(-n // page)
    ids = np.random.default_rng(seed).permutation(blocks + 5)[:blocks]
    cache = torch.full((blocks + 5, 2, G, page, D), 1e4, dtype=dtype)        # a row read from a wrong place is far off
    for j in range(n):
        cache[ids[j // page], 0, :, j % page] = 0
        cache[ids[j // page], 1, :, j % page] = 0
        cache[ids[j // page], 0, :, j % page, :k.shape[2]] = k[j].to(dtype)
        cache[ids[j // page], 1, :, j % page, :v.shape[2]] = v[j].to(dtype)
    return cache, torch.tensor(ids, dtype=torch.int32)[None]


def plain_window_rows(q, k, v, pos, window, keep):
    """q [H, d] at position ``pos`` over keys k [n, G, d], values v [n, G, dv]; scale already inside q."""
    H, G = q.shape[0], k.shape[1]
    seen = [j for j in range(pos + 1) if not window or pos - j < window or j < keep]
    grp = torch.arange(H) // (H // G)
    s = torch.einsum("hd,jhd->hj", q, k[seen][:, grp])
    return torch.einsum("hj,jhd->hd", torch.softmax(s, dim=-1), v[seen][:, grp])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,d,dv,page,window,keep", [(4, 2, 16, 8, 8, 37, 3), (6, 2, 112, 80, 16, 130, 5),
                                                       (3, 3, 24, 40, 16, 50, 20), (2, 1, 16, 16, 4, 1, 1),
                                                       (8, 8, 32, 32, 32, 100, 0), (5, 1, 12, 20, 16, 0, 0),
                                                       (4, 4, 64, 64, 16, 20, 33), (6, 3, 48, 16, 64, 300, 2),
                                                       (4, 2, 32, 32, 16, 40, 70), (16, 2, 128, 128, 16, 64, 65)])
def test_window_attention_kernel_alone(H, G, d, dv, page, window, keep, dtype):
    """Head 0 of the last query points at one key: far back, at page borders, just inside and just outside the
    window, the last kept token and the first one that is not kept.  A key that is lost, seen twice or taken
    from the neighbouring place changes the row by its whole size.  The query is a single token, and the end
    of a portion of 70; in bfloat16 also through the tensor-core kernels (the split kernel for single tokens, in
    one part and in several, and the flash-style kernel for the portion)."""
    from railgun_b200 import ops
    n = 333
    D = -(-max(d, dv) // 16) * 16
    rng = np.random.default_rng(H * d + window)
    keys_at = [0, 1, page - 1, page, n - 2 * page, n - page - 1, 150, n - 2, n - 1]
    if window:
        keys_at += [n - window, n - window - 1, n - window + 1]
    if keep:
        keys_at += [keep - 1, keep, keep + 1]
    for key in sorted({x for x in keys_at if 0 <= x < n}):
        k = torch.tensor(rng.normal(size=(n, G, d)), dtype=TORCH[dtype]).double()
        v = torch.tensor(rng.normal(size=(n, G, dv)), dtype=TORCH[dtype]).double()
        q = torch.tensor(rng.normal(size=(H, d)) * d ** -0.5, dtype=TORCH[dtype]).double()
        k[key, 0] = (k[key, 0] * 1.5).to(TORCH[dtype]).double()                             # a loud key
        q[0] = (k[key, 0] * 4.0).to(TORCH[dtype]).double()
        ref = plain_window_rows(q, k, v, n - 1, window, keep)
        visible = not window or n - 1 - key < window or key < keep
        without = plain_window_rows(q, torch.cat([k[:key], k[key + 1:]]), torch.cat([v[:key], v[key + 1:]]),
                                    n - 2, 0, 0) if visible and not window else None
        if without is not None:
            assert (ref[0] - without[0]).abs().max() > 0.3 * ref[0].abs().max()            # the key matters
        cache, table = paged_kv(k, v, page, D, key, TORCH[dtype])
        for portion in (1, 70):
            qs = torch.zeros((portion, H, D), dtype=TORCH[dtype])
            qs[:, :, :d] = torch.tensor(rng.normal(size=(portion, H, d)) * d ** -0.5, dtype=TORCH[dtype])
            qs[-1, :, :d] = q.to(TORCH[dtype])
            positions = torch.arange(n - portion, n, dtype=torch.int32)
            got = ops.paged_attention_general(dev(qs).view(portion, H * D), H * D, dev(cache), dev(table),
                                              dev(torch.zeros(portion, dtype=torch.int32)), dev(positions), H, G, D,
                                              window, 1.0, keep)
            assert rel(got[-1].view(H, D)[:, :dv], ref) < (2e-5 if dtype == "float32" else 2e-2), f"key {key}"
            assert D == dv or float(got.view(portion, H, D)[:, :, dv:].abs().max()) == 0.0
            if dtype == "bfloat16":
                outs = []
                if portion == 1:
                    for splits in (1, 3, 8):
                        o = torch.full((1, H * D), 7.0, dtype=torch.bfloat16, device=DEV)
                        ops.decode_attention(dev(qs).view(1, H * D), H * D, o, dev(cache), dev(table), None, 1,
                                             dev(torch.zeros(1, dtype=torch.int32)), dev(positions), H, G, D, window,
                                             1.0, splits, keep_first=keep)
                        outs.append(o)
                else:
                    tiles = torch.tensor([[0, 64, 0], [64, portion - 64, 0]], dtype=torch.int32)
                    o = torch.full((portion, H * D), 7.0, dtype=torch.bfloat16, device=DEV)
                    ops.prefill_attention(dev(qs).view(portion, H * D), H * D, o, dev(cache), dev(table), dev(tiles),
                                          dev(positions), H, G, D, window, 1.0, keep_first=keep)
                    outs.append(o)
                for o in outs:
                    assert rel(o[-1].view(H, D)[:, :dv], ref) < 2e-2, f"key {key}, tensor cores"
                    assert rel(o, got) < 3e-2
            # an earlier query of the portion, whose window ends elsewhere
            if portion > 1:
                e = 31
                ref_e = plain_window_rows(qs[e, :, :d].double(), k, v, int(positions[e]), window, keep)
                assert rel(got[e].view(H, D)[:, :dv], ref_e) < (2e-5 if dtype == "float32" else 2e-2)


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_prepare_alone(dtype):
    """Bias is in the rows already; norm per head with one weight for all heads, rotation in pairs (2i, 2i + 1) of
    the first numbers only, the head's factor on q, zeros behind d and dv, k and v at their places of the cache."""
    from railgun_b200 import ops
    from railgun_b200.parts.latent_attention import rotary_frequencies
    rng = np.random.default_rng(7)
    for H, G, d, dv, dims in ((4, 2, 16, 8, 8), (6, 2, 128, 80, 64), (3, 3, 24, 40, 0), (2, 1, 12, 12, 12)):
        T, page = 9, 4
        D = -(-max(d, dv) // 16) * 16
        qkv = torch.tensor(rng.normal(size=(T, (H + G) * d + G * dv)), dtype=TORCH[dtype])
        qn, kn = rng.uniform(0.5, 2, size=d), rng.uniform(0.5, 2, size=d)
        factor = rng.uniform(0.05, 0.5, size=H)
        pos = np.array([0, 1, 2, 3, 500, 501, 70000, 5, 6])
        slots = torch.tensor([5, 4, -1, 7, 0, 1, 2, 11, 3], dtype=torch.int32)
        cache = torch.zeros((3, 2, G, page, D), dtype=TORCH[dtype], device=DEV)
        q = ops.attention_prepare(dev(qkv), cache, dev(qn, torch.float32), dev(kn, torch.float32), 1e-5,
                                  rotary_frequencies(dims, 300.0).to(DEV), dims, True, dev(pos.astype(np.int32)),
                                  dev(slots), dev(factor, torch.float32), H, G, d, dv, D)
        x = qkv.double().numpy()
        q_ref = P.rotate(P.unit_rms(x[:, :H * d].reshape(T, H, d), 1e-5) * qn, pos, dims, 300.0, "interleaved")
        k_ref = P.rotate(P.unit_rms(x[:, H * d:(H + G) * d].reshape(T, G, d), 1e-5) * kn, pos, dims, 300.0, "interleaved")
        tol = 3e-6 if dtype == "float32" else 8e-3
        assert rel(q[:, :, :d], q_ref * factor[None, :, None]) < tol
        assert float(q[:, :, d:].abs().max()) == 0.0 if D > d else True
        for t in range(T):
            s = int(slots[t])
            if s >= 0:
                assert rel(cache[s // page, 0, :, s % page, :d], k_ref[t]) < tol
                assert torch.equal(cache[s // page, 1, :, s % page, :dv].cpu(), qkv[t, (H + G) * d:].view(G, dv))
        assert float(cache[2, :, :, 0].abs().max()) == 0.0 and float(cache[1, :, :, 2].abs().max()) == 0.0   # places 8, 6


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,layer", [("A", 0), ("A", 3), ("B", 1), ("C", 0), ("D", 1), ("E", 2)])
def test_experts_alone(name, layer, dtype):
    """Inputs large enough that gate and up run into the limit on both sides; the weights are the chosen experts'
    softmax scores over all experts as they are."""
    from railgun_b200.engine.runner import ModelRunner
    cfg, _, page = C.CASES[name]
    plain = C.plain_model(name)
    runner = ModelRunner(C.model_dir(name), dtype=dtype, page_size=page, max_tokens=64, max_requests=1)
    rng = np.random.default_rng(layer)
    mlp = cfg["layers"][layer]["mlp"]
    for T in (1, 5, 70, 300):
        h = torch.tensor(rng.normal(size=(T, cfg["width"])) * 0.7, dtype=torch.float32).to(TORCH[dtype])
        margins = []
        ref = P.moe_ff(h.double().numpy(), plain.w, f"l{layer}.mlp.", mlp, margins)
        got = runner.model.layers[layer].ffn.forward(h.to(DEV), None).float().cpu().numpy()
        sure = np.ones(T, dtype=bool) if not margins else margins[0] > (1e-4 if dtype == "float32" else 3e-2)
        assert sure.sum() >= 0.6 * T
        assert rel(got[sure], ref[sure]) < TOL[dtype]


# ---- the model through the step function ---------------------------------------------------------------

LENGTHS = {"A": [1, 2, 9, 12, 40, 77, 150, 64], "B": [1, 3, 17, 64, 100, 33], "C": [1, 5, 21, 60, 130, 4],
           "D": [2, 131, 260, 400, 55, 129, 181], "E": [1, 6, 10, 33, 90, 65]}
PORTIONS = {"D": (130, 2, 64, 7, 128, 3, 65, 2, 33, 129)}
MIXED = {"D": (5, 1, 2, 70, 1, 1, 3, 140, 1, 2, 128, 17)}
TAIL = {"D": 140}                                   # the windows of 130 and 50 pass over decoded tokens
_oracle: dict = {}


def oracle(name):
    if name not in _oracle:
        cfg = C.CASES[name][0]
        reqs = {f"r{i}": p for i, p in enumerate(C.prompts(cfg["vocab"], LENGTHS[name], seed=21))}
        plain = C.plain_model(name)
        _oracle[name] = (reqs, {k: plain.forward(v) for k, v in reqs.items()})
    return _oracle[name]


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


def compare(rows, reqs, logits, tol, what):
    worst = 0.0
    for name, toks in reqs.items():
        ref = logits[name]
        scale = np.abs(ref).max()
        for p in range(len(toks)):
            err = np.abs(rows[(name, p)] - ref[p]).max() / scale
            assert err <= tol, (f"{what}: request {name} (length {len(toks)}) first differs at position {p}: "
                                f"relative error {err:.3e}")
            worst = max(worst, err)
    return worst


@pytest.mark.parametrize("mode", ["whole", "tail", "portions", "mixed"])
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(C.CASES))
def test_replay_matches_plain(name, dtype, mode, tmp_path):
    """Whole prompts; the last tokens one by one; portions down to two tokens, cut inside pages, windows and
    the reach of the convolutions; up to four live requests in a pool so small that pages and state slots are
    used again.  Every position of every request is compared, the first tokens included."""
    reqs, logits = oracle(name)
    rows = replay_case(name, dtype, make_trace(mode, reqs, name), tmp_path)
    print(f"{name} {dtype} {mode}: worst relative error "
          f"{compare(rows, reqs, logits, TOL[dtype], f'{name} {dtype} {mode}'):.3e}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "C", "E"])
def test_every_token_decoded_alone_matches_whole_prompts(name, dtype, tmp_path):
    """Token-by-token decoding from the first token on (through the decode graphs and with graphs off): states
    and convolution tails that start from nothing, windows that pass over decoded tokens."""
    reqs, logits = oracle(name)
    few = dict(list(reqs.items())[2:7])
    steps = make_trace("every_token", few, name)
    compare(replay_case(name, dtype, steps, tmp_path / "g"), few, logits, TOL[dtype], "decoded")
    compare(replay_case(name, dtype, steps, tmp_path / "e", use_graphs=False), few, logits, TOL[dtype],
            "decoded, no graphs")


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
        compare(a, {n: reqs[n] for n in names}, logits, TOL[dtype], "together")
        for key in a:
            assert np.abs(a[key] - b[key]).max() <= (2e-5 if dtype == "float32" else 0.25) * np.abs(b[key]).max(), key


def test_sharp_attention_shows_the_edges_of_the_window(tmp_path):
    """With the weights of the norms on q and k made several times larger the softmax is sharp: a few keys hold
    most of the weight, so one key too many or too few at the window's edge, or a kept token that is lost,
    moves the logits by far more than the tolerance.  Prompts, portions, and decoding across both windows."""
    cfg, seed, page = C.CASES["D"]

    def sharpen(t):
        for i, L in enumerate(cfg["layers"]):
            if L["type"] == "attention":
                t[f"l{i}.mix.q.norm"] *= 2.5
                t[f"l{i}.mix.k.norm"] *= 2.5

    folder = C.write_model(cfg, seed + 1, tmp_path / "model", change=sharpen)
    plain = C.Plain(folder)
    reqs = {f"s{i}": p for i, p in enumerate(C.prompts(cfg["vocab"], [190, 135, 52, 300], seed=4))}
    logits = {k: plain.forward(v) for k, v in reqs.items()}
    # the windows matter: the same model with windows one token longer answers differently
    other = json.loads(json.dumps(cfg))
    for L in other["layers"]:
        if L["type"] == "attention":
            L["mixer"]["mask"]["size"] += 1
    moved = P.forward(reqs["s0"], plain.w, other)
    assert np.abs(moved[-1] - logits["s0"][-1]).max() > 50 * TOL["float32"] * np.abs(logits["s0"]).max()
    for mode in ("whole", "tail", "portions", "mixed"):
        steps = make_trace(mode, reqs, "D")
        rows = replay(folder, cfg, page, "float32", steps, tmp_path / mode)
        compare(rows, reqs, logits, TOL["float32"], f"sharp {mode}")


def test_states_remember_a_far_token(tmp_path):
    """Two prompts that differ in their second token only: after 300 more tokens, most of them decoded one by
    one, the logits still differ (the decays are close to one), and both equal the plain model's."""
    cfg, _, page = C.CASES["D"]
    only_states = dict(cfg, layers=[L for L in cfg["layers"] if L["type"] != "attention"])
    folder = C.write_model(only_states, 17, tmp_path / "model")
    plain = C.Plain(folder)
    a = C.prompts(cfg["vocab"], [310], seed=9)[0]
    b = list(a)
    b[1] = (a[1] + 1) % cfg["vocab"]
    reqs = {"a": a, "b": b}
    logits = {k: plain.forward(v) for k, v in reqs.items()}
    scale = np.abs(logits["a"]).max()
    assert np.abs(logits["a"][-1] - logits["b"][-1]).max() > 20 * TOL["float32"] * scale
    steps = helpers.trace_tail_decode(reqs, 250)
    compare(replay(folder, only_states, page, "float32", steps, tmp_path / "o"), reqs, logits, TOL["float32"], "far")


# ---- generation through the engine and the command line -----------------------------------------------

def greedy_consistent(plain, prompt, out, tol):
    """How many generated tokens are the plain model's choice given the tokens before them (teacher-forced), up
    to ``tol`` of the largest absolute logit."""
    logits = plain.forward(list(prompt) + list(out))
    return sum(int(logits[len(prompt) - 1 + i][t] >= logits[len(prompt) - 1 + i].max() - tol * np.abs(logits).max())
               for i, t in enumerate(out))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "E"])
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
    d = C.model_dir("E")
    plain = C.plain_model("E")
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

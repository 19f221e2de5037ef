"""Mixers whose memory is a matrix per head, and the short convolution that
can sit in front of any mixer.

"retention": linear attention with one fixed decay per head and neither
softmax nor denominator (Sun et al., "Retentive Network: A Successor to
Transformer for Large Language Models").  With q, k [heads, d] (their first
``rot_dims`` numbers rotated in pairs (i, i + rot_dims/2), k times d^-1/2)
and v [heads, dv]:
    S_t = decay_h S_(t-1) + k_t v_t^T,   o_t = S_t^T q_t
    out = W_o (unit_rms(o_t) per head * silu(W_g h))

"gated_delta": the gated delta rule (Yang et al., "Gated Delta Networks:
Improving Mamba2 with Delta Rule").  q, k [qk_heads, d] and v [heads, dv]
each pass a causal convolution per channel and silu; q and k become unit
vectors (q times d^-1/2); beta = sigmoid(W_b h),
g = exp(-exp(A_log) softplus(W_a h + dt_bias)) per head:
    S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
    out = W_o (unit_rms(o) per head * weight * silu(W_g h))

"input_conv": a wrapper.  The inner mixer reads h + conv(h), a causal
convolution per channel over the request's tokens, instead of h.

Between steps a request keeps, in its state slot and in 32-bit: S of every
head (transposed, [dv, d]), and the last taps - 1 inputs of every
convolution.  Everything from the projections' outputs to the rounding
before the output product is 32-bit.
"""
from __future__ import annotations

import torch

from .. import ops
from ..cache.manager import StateNeed
from ..weights.loader import TensorSpec
from .base import CacheView, Mixer
from .latent_attention import rotary_frequencies
from .registry import MIXERS, register_mixer


def _base(p, prefix):
    return prefix + (p.get("base") if p.get("base") is not None else "mix.")


class Retention(Mixer):
    """params: ``hidden_size``, ``num_heads``, ``head_dim``, ``v_dim``, ``decay`` (one number per head),
    ``rot_dims``, ``rot_base``, ``eps`` (of the heads' norm), ``k_scale`` (None: head_dim^-1/2), ``base`` (what
    the tensor names start with after the prefix, default "mix."; the tensors are q, k, v, g, o).  Optional:
    ``activation`` "silu" (on q, k and v, as lightning attention has it; default none), ``norm`` "whole" (one
    root mean square over all heads' outputs with the weight tensor ``norm`` [heads * v_dim]; default "head":
    every head by its own, no weight), ``gate`` "sigmoid" (default "silu")."""

    @classmethod
    def tensor_specs(cls, p, prefix):
        W, H, d, dv = p["hidden_size"], p["num_heads"], p["head_dim"], p["v_dim"]
        b = _base(p, prefix)
        out = {b + "q": TensorSpec((H * d, W)), b + "k": TensorSpec((H * d, W)), b + "v": TensorSpec((H * dv, W)),
               b + "g": TensorSpec((H * dv, W)), b + "o": TensorSpec((W, H * dv))}
        if p.get("norm") == "whole":
            out[b + "norm"] = TensorSpec((H * dv,), init="norm")
        return out

    @classmethod
    def cache_need(cls, p):
        return StateNeed((int(p["num_heads"]), int(p["v_dim"]), int(p["head_dim"])), "float32")     # S transposed

    def __init__(self, p, prefix, env, tensors):
        super().__init__(p, prefix, env, tensors)
        self.H, self.d, self.dv = int(p["num_heads"]), int(p["head_dim"]), int(p["v_dim"])
        decay = [float(x) for x in p["decay"]]
        if len(decay) != self.H:
            raise ValueError(f"{len(decay)} decays for {self.H} heads")
        self.decay = torch.tensor(decay, dtype=torch.float32, device=env.device)
        self.rot_dims = int(p.get("rot_dims") or 0)
        if self.rot_dims % 2 or not 0 <= self.rot_dims <= self.d:
            raise ValueError(f"{self.rot_dims} rotated numbers do not fit a head of {self.d}")
        self.eps = float(p.get("eps") or 0.0)
        self.k_scale = float(p["k_scale"]) if p.get("k_scale") is not None else float(self.d) ** -0.5
        act, norm, gate = p.get("activation"), p.get("norm") or "head", p.get("gate") or "silu"
        if act not in (None, "silu") or norm not in ("head", "whole") or gate not in ops.HEAD_GATES:
            raise ValueError(f"retention: activation {act!r}, norm {norm!r} or gate {gate!r} is not known")
        self.silu, self.whole, self.gate = act == "silu", norm == "whole", gate
        b = _base(p, prefix)
        self.w_in = torch.cat([tensors.get(b + n, env.dtype) for n in ("q", "k", "v", "g")], dim=0).contiguous()
        tensors.drop(b + "q", b + "k", b + "v", b + "g")
        self.w_o = tensors.get(b + "o", env.dtype)
        self.norm = tensors.get(b + "norm", torch.float32).contiguous() if self.whole else None
        base = float(p.get("rot_base") or 10000.0)
        self.freq = tensors.shared_part(("rotary_frequencies", self.rot_dims, base),
                                        lambda: rotary_frequencies(self.rot_dims, base).to(env.device))

    def input_weight(self):
        """The matrix of the first product, for a wrapper that computes the first products of several mixers that
        read the same rows as one."""
        return self.w_in

    def adopt_input_weight(self, view):
        self.w_in = view

    def forward(self, x, batch, cache, writes=True, proj=None):
        H, d, dv = self.H, self.d, self.dv
        if proj is None:
            proj = ops.linear(x, self.w_in)                                  # [T, q | k | v | gate]
        if self.silu:
            q, k, v = ops.retention_prepare(proj, 0, H * d, self.freq, self.rot_dims, batch.positions, H, d,
                                            self.k_scale, silu=True, v_off=2 * H * d, dv=dv)
        else:
            q, k = ops.retention_prepare(proj, 0, H * d, self.freq, self.rot_dims, batch.positions, H, d, self.k_scale)
            v = proj[:, 2 * H * d:2 * H * d + H * dv]
        o = ops.state_scan(q.view(-1, H * d), k.view(-1, H * d), v, cache.state, batch, H, d, dv, decay=self.decay)
        z = ops.head_norm_gate(o, proj[:, 2 * H * d + H * dv:], self.norm, self.eps, self.env.dtype, whole=self.whole,
                               gate_kind=self.gate)
        return ops.linear(z, self.w_o)


class GatedDelta(Mixer):
    """params: ``hidden_size``, ``num_heads`` (value heads), ``num_qk_heads``, ``head_dim``, ``v_dim``, ``taps``
    (of the convolutions on q, k and v), ``eps`` (of the heads' norm), ``unit_eps`` (inside the root that makes
    q and k unit vectors, default 1e-6), ``q_scale`` (None: head_dim^-1/2), ``base`` (default "mix."; the
    tensors are q, k, v, q.conv, k.conv, v.conv, b, a, A_log, dt_bias, g, norm, o)."""

    @classmethod
    def tensor_specs(cls, p, prefix):
        W, H, G, d, dv, K = (p["hidden_size"], p["num_heads"], p["num_qk_heads"], p["head_dim"], p["v_dim"],
                             p["taps"])
        b = _base(p, prefix)
        return {b + "q": TensorSpec((G * d, W)), b + "k": TensorSpec((G * d, W)), b + "v": TensorSpec((H * dv, W)),
                b + "q.conv": TensorSpec((G * d, K)), b + "k.conv": TensorSpec((G * d, K)),
                b + "v.conv": TensorSpec((H * dv, K)), b + "b": TensorSpec((H, W)), b + "a": TensorSpec((H, W)),
                b + "A_log": TensorSpec((H,)), b + "dt_bias": TensorSpec((H,)), b + "g": TensorSpec((H * dv, W)),
                b + "norm": TensorSpec((dv,), init="norm"), b + "o": TensorSpec((W, H * dv))}

    @classmethod
    def cache_need(cls, p):
        H, G, d, dv, K = p["num_heads"], p["num_qk_heads"], p["head_dim"], p["v_dim"], p["taps"]
        need = [StateNeed((int(H), int(dv), int(d)), "float32")]            # S transposed
        if K > 1:
            need.append(StateNeed((int(K) - 1, 2 * G * d + H * dv), "float32"))
        return tuple(need)

    def __init__(self, p, prefix, env, tensors):
        super().__init__(p, prefix, env, tensors)
        self.H, self.G, self.d, self.dv, self.K = (int(p["num_heads"]), int(p["num_qk_heads"]), int(p["head_dim"]),
                                                   int(p["v_dim"]), int(p["taps"]))
        if self.H % self.G:
            raise ValueError(f"{self.H} heads cannot share {self.G} query/key heads")
        self.eps = float(p.get("eps") or 0.0)
        self.unit_eps = float(p["unit_eps"]) if p.get("unit_eps") is not None else 1e-6
        self.q_scale = float(p["q_scale"]) if p.get("q_scale") is not None else float(self.d) ** -0.5
        b = _base(p, prefix)
        f32 = lambda n: tensors.get(b + n, torch.float32).contiguous()
        self.w_in = torch.cat([tensors.get(b + n, env.dtype) for n in ("q", "k", "v", "g")], dim=0).contiguous()
        self.w_ba = torch.cat([tensors.get(b + n, env.dtype) for n in ("b", "a")], dim=0).contiguous()
        tensors.drop(b + "q", b + "k", b + "v", b + "g", b + "b", b + "a")
        self.taps = torch.cat([f32("q.conv"), f32("k.conv"), f32("v.conv")], dim=0).t().contiguous()    # [taps, channels]
        self.A_log, self.dt_bias, self.norm = f32("A_log"), f32("dt_bias"), f32("norm")
        self.w_o = tensors.get(b + "o", env.dtype)

    def forward(self, x, batch, cache, writes=True):
        H, G, d, dv = self.H, self.G, self.d, self.dv
        C = 2 * G * d + H * dv
        proj = ops.linear(x, self.w_in)                                      # [T, q | k | v | gate]
        ba = ops.linear(x, self.w_ba, out_dtype=torch.float32)               # [T, b | a], kept in 32-bit
        conv_state = cache.parts[1].state if self.K > 1 else None
        qkv = ops.causal_conv(proj, 0, self.taps, conv_state, batch, torch.float32, silu=True)
        if writes and conv_state is not None:
            ops.conv_state_update(proj, 0, conv_state, batch)
        beta, g = ops.delta_prepare(qkv, G, d, self.q_scale, self.unit_eps, ba, 0, H, self.A_log, self.dt_bias, H)
        o = ops.state_scan(qkv[:, :G * d], qkv[:, G * d:2 * G * d], qkv[:, 2 * G * d:], cache.parts[0].state, batch,
                           H, d, dv, g=g, beta=beta)
        z = ops.head_norm_gate(o, proj[:, C:], self.norm, self.eps, self.env.dtype)
        return ops.linear(z, self.w_o)


class InputConv(Mixer):
    """params: ``channels``, ``taps``, ``name`` (the taps' tensor name after the prefix, [channels, taps], last
    column the current token's), ``inner`` (the PartSpec of the mixer that reads h + conv(h))."""

    @classmethod
    def tensor_specs(cls, p, prefix):
        inner = p["inner"]
        out = dict(MIXERS.get(inner.kind).tensor_specs(inner.params, prefix))
        out[prefix + p["name"]] = TensorSpec((p["channels"], p["taps"]))
        return out

    @classmethod
    def _inner_needs(cls, p):
        inner = p["inner"]
        need = MIXERS.get(inner.kind).cache_need(inner.params)
        return (tuple(need), True) if isinstance(need, (tuple, list)) else ((need,), False)

    @classmethod
    def cache_need(cls, p):
        needs, _ = cls._inner_needs(p)
        own = (StateNeed((int(p["taps"]) - 1, int(p["channels"])), "float32"),) if p["taps"] > 1 else (None,)
        return own + needs

    def __init__(self, p, prefix, env, tensors):
        super().__init__(p, prefix, env, tensors)
        inner = p["inner"]
        self.inner = MIXERS.get(inner.kind)(inner.params, prefix, env, tensors)
        self.inner_composite = self._inner_needs(p)[1]
        self.K = int(p["taps"])
        self.taps = tensors.get(prefix + p["name"], torch.float32).t().contiguous()                # [taps, channels]
        self.graph_safe = getattr(self.inner, "graph_safe", True)

    def forward(self, x, batch, cache, writes=True):
        state = cache.parts[0].state if self.K > 1 else None
        h = ops.causal_conv(x, 0, self.taps, state, batch, self.env.dtype, residual=True)
        if writes and state is not None:
            ops.conv_state_update(x, 0, state, batch)
        view = CacheView(cache.cache_id, parts=cache.parts[1:]) if self.inner_composite else cache.parts[1]
        return self.inner.forward(h, batch, view, writes)


register_mixer("retention", Retention)
register_mixer("gated_delta", GatedDelta)
register_mixer("input_conv", InputConv)

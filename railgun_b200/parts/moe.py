"""A mixture of experts with a softmax or sigmoid router.

Router logits are 32-bit; scores are their softmax over all router outputs
(or the sigmoid of each);
the ``top`` outputs with the largest score + correction are chosen, and their
weights are the scores themselves over their sum.  The first ``experts``
outputs stand for gated feed-forwards down(silu(gate h) * (up h)), the
``identity`` outputs after them for experts that return their input.  An
optional shared expert of the same form runs for every token and is added.
Experts without a gate, down(act(up h)), and experts whose weight multiplies
their input instead of their output, sum_e expert_e(w_e h), are options.

The experts' matrices are stacked at load ([E, 2F, W] gate rows then up rows,
[E, W, F]); the step groups its (token, choice) pairs by expert on the device
and runs both products over the groups, so nothing is read back to the host
and the step stays capturable.
"""
from __future__ import annotations

import torch

from .. import ops
from ..weights.loader import TensorSpec
from .base import FeedForward
from .mlp import SwiGLU
from .registry import register_feed_forward


class RoutedExperts(FeedForward):
    """params: ``hidden_size``, ``experts``, ``identity``, ``top``,
    ``expert_size`` (an expert's inner size), ``shared_size`` (the shared
    expert's, or None), ``base`` (tensor names after the prefix start with it:
    ``<base>e<i>.gate|up|down``, ``<base>router``, ``<base>correction``,
    ``<base>shared.gate|up|down``).  Optional: ``correction`` False (no
    correction tensor: the largest scores are chosen), ``renormalize`` False
    (the weights are the chosen scores themselves), ``activation`` ("silu",
    "gelu_tanh" or "clamped_swish" with ``limit``: g' sigmoid(1.702 g') (u' + 1),
    g' = min(g, limit), u' = clamp(u, -limit, limit)), ``scoring`` "sigmoid"
    (default "softmax"), ``gated`` False (experts ``<base>e<i>.up|down`` without a
    gate; ``activation`` is then one of ``ops.ACTIVATIONS``, e.g. "relu2"),
    ``scale_input`` True (a chosen expert reads its weight times the token's row,
    and the experts' outputs are added as they are; not with identity or shared
    experts)."""

    @classmethod
    def tensor_specs(cls, p, prefix):
        W, E, N, F = p["hidden_size"], p["experts"], p["experts"] + p["identity"], p["expert_size"]
        b = prefix + p.get("base", "mlp.")
        out = {b + "router": TensorSpec((N, W))}
        if p.get("correction", True):
            out[b + "correction"] = TensorSpec((N,))
        for e in range(E):
            if p.get("gated", True):
                out[f"{b}e{e}.gate"] = TensorSpec((F, W))
            out[f"{b}e{e}.up"] = TensorSpec((F, W))
            out[f"{b}e{e}.down"] = TensorSpec((W, F))
        if p.get("shared_size"):
            out.update(SwiGLU.tensor_specs(cls._shared_params(p), prefix))
        return out

    @staticmethod
    def _shared_params(p):
        b = p.get("base", "mlp.")
        return dict(hidden_size=p["hidden_size"], intermediate_size=p["shared_size"],
                    names=(b + "shared.gate", b + "shared.up", b + "shared.down"))

    def __init__(self, p, prefix, env, tensors):
        super().__init__(p, prefix, env, tensors)
        self.E, self.top = int(p["experts"]), int(p["top"])
        self.N = self.E + int(p["identity"])
        if not 1 <= self.top <= self.N:
            raise ValueError(f"{self.top} choices among {self.N} router outputs")
        b = prefix + p.get("base", "mlp.")
        self.router = tensors.get(b + "router", torch.float32)
        self.correction = tensors.get(b + "correction", torch.float32) if p.get("correction", True) else None
        self.renormalize = bool(p.get("renormalize", True))
        self.act = p.get("activation") or "silu"
        self.limit = float(p.get("limit") or 0.0)
        self.gated = bool(p.get("gated", True))
        self.scoring = p.get("scoring") or "softmax"
        self.scale_input = bool(p.get("scale_input", False))
        if self.scoring not in ops.MOE_SCORINGS:
            raise ValueError(f"router scoring {self.scoring!r} is not known; known: {sorted(ops.MOE_SCORINGS)}")
        known = ops.GATED_ACTIVATIONS if self.gated else ops.ACTIVATIONS
        if self.act not in known:
            raise ValueError(f"activation {self.act!r} is not known; known: {sorted(known)}")
        if self.scale_input and (self.N != self.E or p.get("shared_size")):
            raise ValueError("experts that read their weight times the input go without identity and shared experts")
        if self.E and not self.gated:
            self.w_gate_up = torch.stack([tensors.get(f"{b}e{e}.up", env.dtype) for e in range(self.E)]).contiguous()
            self.w_down = torch.stack([tensors.get(f"{b}e{e}.down", env.dtype) for e in range(self.E)]).contiguous()
            tensors.drop(*[f"{b}e{e}.{n}" for e in range(self.E) for n in ("up", "down")])
        elif self.E:
            self.w_gate_up = torch.stack([torch.cat([tensors.get(f"{b}e{e}.gate", env.dtype),
                                                     tensors.get(f"{b}e{e}.up", env.dtype)], dim=0)
                                          for e in range(self.E)]).contiguous()                    # [E, 2F, W]
            self.w_down = torch.stack([tensors.get(f"{b}e{e}.down", env.dtype) for e in range(self.E)]).contiguous()
            tensors.drop(*[f"{b}e{e}.{n}" for e in range(self.E) for n in ("gate", "up", "down")])
        self.shared = SwiGLU(self._shared_params(p), prefix, env, tensors) if p.get("shared_size") else None

    def forward(self, x, batch):
        T = x.shape[0]
        ids, weights = ops.moe_route(x, self.router, self.correction, self.top, self.renormalize, self.scoring)
        y = pair_pos = None
        if self.E:
            places = T * self.top
            rows = ops.moe_tile_rows(x.dtype, places, self.E, self.w_gate_up.shape[2], self.w_down.shape[2])
            sorted_pair, pair_pos, tiles = ops.moe_align(ids, self.E, rows)
            src, div = sorted_pair, self.top
            if self.scale_input:
                # the experts' rows in expert order, each already times its weight; the sum then takes them as they are
                x_in, src, div = ops.moe_scaled_rows(x, sorted_pair, self.top, weights, places), None, 1
                weights = None
            else:
                x_in = x
            if self.gated:
                act = ops.moe_grouped_gemm(x_in, src, div, self.w_gate_up, tiles, places, True, rows,
                                           act=self.act, limit=self.limit)
            else:
                act = ops.moe_grouped_gemm(x_in, src, div, self.w_gate_up, tiles, places, False, rows,
                                           plain_act=self.act)
            y = ops.moe_grouped_gemm(act, None, 1, self.w_down, tiles, places, False, rows)
        else:
            pair_pos = ids
        shared = self.shared.forward(x, batch) if self.shared is not None else None
        return ops.moe_combine(x, y, shared, ids, weights, pair_pos, self.E)


register_feed_forward("routed_experts", RoutedExperts)

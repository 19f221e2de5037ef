"""Mixers side by side: every branch reads the same input, and the result is
the sum of the branches' outputs, each times a constant.

A branch is any mixer that can hand out what goes into its output product
(``mix(x, batch, cache, writes, out, out_scale, proj)`` -> [T, out_features],
``w_o`` [hidden, out_features]) and takes its first product from outside
(``w_in`` [in_features, hidden]; ``proj`` = x w_in^T).  ONE product with the
branches' input matrices stacked feeds them all; they write side by side
into one buffer, already multiplied by their constants in 32-bit before the
one rounding, and ONE product with the output matrices side by side gives
sum_b c_b W_o,b z_b.  What the branches keep between steps is asked for as a
tuple of needs, one per branch.

With ``out_norms`` every branch's output is RMS-normed over the width with a
weight of its own before the sum, sum_b c_b norm_b(branch_b(x)): the branches
are then any mixers, run one after the other through their ``forward``, and
the norms, constants and sum are one kernel (ops.norm_sum, 32-bit); branches
that hand out the matrix of their first product (``input_weight()``) get that
product from here, one for all of them.
"""
from __future__ import annotations

import torch

from .. import ops
from ..weights.loader import TensorSpec
from .base import CacheView, Mixer
from .registry import MIXERS, register_mixer


class Parallel(Mixer):
    """params: ``branches``: ((PartSpec of a mixer, constant), ...).  Optional ``out_norms``: one tensor name
    (after the prefix, [hidden_size], a plain weight) per branch, with ``hidden_size`` and ``eps``."""

    @classmethod
    def tensor_specs(cls, p, prefix):
        out = {}
        for spec, _ in p["branches"]:
            out.update(MIXERS.get(spec.kind).tensor_specs(spec.params, prefix))
        for name in p.get("out_norms") or ():
            out[prefix + name] = TensorSpec((int(p["hidden_size"]),), init="norm")
        return out

    @classmethod
    def _branch_needs(cls, p):
        """Per branch: (its needs as a tuple, whether it asked for a tuple itself)."""
        out = []
        for spec, _ in p["branches"]:
            need = MIXERS.get(spec.kind).cache_need(spec.params)
            out.append((tuple(need), True) if isinstance(need, (tuple, list)) else ((need,), False))
        return out

    @classmethod
    def cache_need(cls, p):
        # one flat tuple: a branch that keeps several things itself gets that many places in a row
        return tuple(n for needs, _ in cls._branch_needs(p) for n in needs)

    def _views(self, cache):
        """The branches' cache views out of this mixer's: a branch that asked for a tuple of needs sees a view with
        one part per need, as it would alone."""
        views, at = [], 0
        for needs, composite in self._needs:
            views.append(CacheView(cache.cache_id, parts=cache.parts[at:at + len(needs)]) if composite
                         else cache.parts[at])
            at += len(needs)
        return views

    def __init__(self, p, prefix, env, tensors):
        super().__init__(p, prefix, env, tensors)
        self.parts = [MIXERS.get(spec.kind)(spec.params, prefix, env, tensors) for spec, _ in p["branches"]]
        self.scales = [float(c) for _, c in p["branches"]]
        self._needs = self._branch_needs(p)
        self.graph_safe = all(getattr(part, "graph_safe", True) for part in self.parts)
        self.out_norms = None
        if p.get("out_norms"):
            if len(p["out_norms"]) != len(self.parts) or len(self.parts) > 4:
                raise ValueError("'parallel' with out_norms: one norm per branch, four branches at most")
            self.out_norms = [tensors.get(prefix + n, torch.float32).contiguous() for n in p["out_norms"]]
            self.eps = float(p["eps"])
            # branches that hand out the matrix of their first product get that product from here: one product
            # over the matrices stacked by rows, of which every branch reads its columns
            self.stacked, self.in_cols = None, []
            ws = [part.input_weight() if hasattr(part, "input_weight") else None for part in self.parts]
            if len(ws) > 1 and all(w is not None for w in ws):
                self.stacked = torch.cat(ws, dim=0).contiguous()
                at = 0
                for part, w in zip(self.parts, ws):
                    part.adopt_input_weight(self.stacked[at:at + w.shape[0]])
                    self.in_cols.append((at, at + w.shape[0]))
                    at += w.shape[0]
            return
        for part in self.parts:
            if not all(hasattr(part, a) for a in ("mix", "w_o", "w_in")):
                raise ValueError(f"{type(part).__name__} cannot be a branch of 'parallel': it has no mix(), w_in and w_o")
        self.w_in = torch.cat([part.w_in for part in self.parts], dim=0).contiguous()
        self.w_o = torch.cat([part.w_o for part in self.parts], dim=1).contiguous()
        self.widths = [int(part.out_features) for part in self.parts]
        self.in_widths = [int(part.w_in.shape[0]) for part in self.parts]
        # the stacked matrices are the ones that are kept: the branches see their share of them
        at = off = 0
        for part, n_in, n in zip(self.parts, self.in_widths, self.widths):
            part.w_in = self.w_in[at:at + n_in]
            part.w_o = self.w_o[:, off:off + n]
            for name in ("w_qkv", "w_yx"):
                if hasattr(part, name):
                    setattr(part, name, part.w_in)
            at += n_in
            off += n
        self.graph_safe = all(getattr(part, "graph_safe", True) for part in self.parts)

    def forward(self, x, batch, cache, writes=True):
        if self.out_norms is not None:
            if self.stacked is not None:
                proj = ops.linear(x, self.stacked)
                ys = [part.forward(x, batch, view, writes, proj=proj[:, a:b])
                      for part, view, (a, b) in zip(self.parts, self._views(cache), self.in_cols)]
            else:
                ys = [part.forward(x, batch, view, writes) for part, view in zip(self.parts, self._views(cache))]
            return ops.norm_sum(ys, self.out_norms, self.scales, self.eps)
        T = x.shape[0]
        proj = ops.linear(x, self.w_in)
        z = torch.empty((T, sum(self.widths)), dtype=self.env.dtype, device=self.w_o.device)
        off = at = 0
        for part, c, n, n_in, view in zip(self.parts, self.scales, self.widths, self.in_widths, self._views(cache)):
            part.mix(x, batch, view, writes, out=z[:, off:off + n], out_scale=c, proj=proj[:, at:at + n_in])
            off += n
            at += n_in
        return ops.linear(z, self.w_o)


register_mixer("parallel", Parallel)

"""RMSNorm, fused with the residual add that precedes it.

y = w * r / sqrt(mean(r^2) + eps), r = residual (+ pending), all in 32-bit
with one rounding at the end.  The reference builds the norm with
candle_nn::rms_norm(H, eps) (crates/vllm-models/src/llama/architecture.rs:27-28,108)
and adds residuals with separate ops (:53,58).
"""
from __future__ import annotations

import torch

from .. import ops
from ..weights.loader import TensorSpec
from .base import Norm
from .registry import register_norm


class RMSNorm(Norm):
    """params: ``size``, ``eps``, ``name`` (weight tensor name after the prefix);
    optional ``scale_name`` (a second per-feature vector, a layer scale, that
    multiplies the normed value) and ``mult`` (a constant that does): both are
    multiplied into the weight at load, in 32-bit; ``groups`` (default 1): the
    row is cut into that many equal consecutive parts and each part is divided
    by its own root mean square; ``one_plus`` (default false): the stored
    weight sits around zero and the normed value is multiplied by 1 + w."""

    @classmethod
    def tensor_specs(cls, params, prefix):
        out = {prefix + params["name"]: TensorSpec((params["size"],), init="norm")}
        if params.get("scale_name"):
            out[prefix + params["scale_name"]] = TensorSpec((params["size"],), init="norm")
        return out

    def __init__(self, params, prefix, env, tensors):
        super().__init__(params, prefix, env, tensors)
        self.eps = float(params["eps"])
        self.weight = tensors.get(prefix + params["name"], torch.float32)
        if params.get("one_plus"):
            self.weight = self.weight + 1.0
        if params.get("scale_name"):
            self.weight = self.weight * tensors.get(prefix + params["scale_name"], torch.float32)
        if params.get("mult") is not None and float(params["mult"]) != 1.0:
            self.weight = self.weight * float(params["mult"])
        self.weight = self.weight.contiguous()
        self.groups = int(params.get("groups") or 1)
        if self.groups < 1 or int(params["size"]) % self.groups:
            raise ValueError(f"rows of {params['size']} do not split into {self.groups} equal groups")

    fuses_pending_linear = True
    fuses_post_norm = True
    fuses_pending_sum = True

    def add_norm(self, resid, pending, rows=None):
        if self.groups > 1 or isinstance(pending, ops.PendingSum):
            if isinstance(pending, (ops.PendingLinear, ops.PendingNormed)):
                pending = pending.materialize()
            return ops.add_group_rmsnorm(resid, pending, [self.weight], self.groups, self.eps, self.env.dtype, rows)[0]
        if isinstance(pending, ops.PendingNormed):
            return ops.add_postnorm_rmsnorm(resid, pending, self.weight, self.eps, self.env.dtype, rows)
        if isinstance(pending, ops.PendingLinear):
            # small decode batches: the product adds its result to the residual itself and prepares this
            # norm; the product that reads the result finishes it
            if rows is None and self.env.dtype == torch.bfloat16 and ops.skinny_fused_ok(pending.x, pending.weight, resid):
                return ops.skinny_gemm_residual(pending.x, pending.weight, resid, self.weight, self.eps)
            if rows is None and self.env.dtype == torch.bfloat16 and ops.tc_stream_fused_ok(pending.x, pending.weight, resid):
                return ops.tc_stream_gemm_residual(pending.x, pending.weight, resid, self.weight, self.eps)
            pending = pending.materialize()
        return ops.add_rmsnorm(resid, pending, self.weight, self.eps, self.env.dtype, rows)


register_norm("rmsnorm", RMSNorm)

"""Dense gated feed-forward: down(act(gate(x)) * up(x)), act = silu
(crates/vllm-models/src/llama/architecture.rs:75-85) unless the model names
another one.  gate and up are one matrix here, stacked by rows at load.
"""
from __future__ import annotations

import torch

from .. import ops
from ..weights.loader import TensorSpec
from .base import FeedForward
from .registry import register_feed_forward


class SwiGLU(FeedForward):
    """params: ``hidden_size``, ``intermediate_size``; optional ``names`` (the
    gate, up and down matrices' names after the prefix) and ``activation``
    ("silu", the default, or "gelu_tanh": the products' fused epilogues are
    silu's, another activation runs as a kernel of its own)."""

    NAMES = ("mlp.gate_proj.weight", "mlp.up_proj.weight", "mlp.down_proj.weight")

    @classmethod
    def tensor_specs(cls, p, prefix):
        H, I = p["hidden_size"], p["intermediate_size"]
        gate, up, down = p.get("names") or cls.NAMES
        return {prefix + gate: TensorSpec((I, H)), prefix + up: TensorSpec((I, H)), prefix + down: TensorSpec((H, I))}

    def __init__(self, p, prefix, env, tensors):
        super().__init__(p, prefix, env, tensors)
        n_gate, n_up, n_down = (prefix + n for n in (p.get("names") or self.NAMES))
        gate, up = tensors.get(n_gate, env.dtype), tensors.get(n_up, env.dtype)
        # bfloat16 with I % 8 == 0: gate and up rows interleaved in blocks of 8, which lets the decode
        # product apply SiLU-mul in its epilogue; otherwise gate rows, then up rows
        self.act = p.get("activation") or "silu"
        if self.act not in ops.GATED_ACTIVATIONS:
            raise ValueError(f"gated activation {self.act!r} is not known; known: {sorted(ops.GATED_ACTIVATIONS)}")
        self.interleaved = env.dtype == torch.bfloat16 and p["intermediate_size"] % 8 == 0 and self.act == "silu"
        self.w_gate_up = (ops.interleave_gate_up(gate, up) if self.interleaved
                          else torch.cat([gate, up], dim=0).contiguous())
        tensors.drop(n_gate, n_up)
        self.w_down = tensors.get(n_down, env.dtype)

    takes_normed_rows = True
    defers_output = True

    def forward(self, x, batch, defer=False):
        if self.act != "silu":
            if isinstance(x, ops.NormedRows):
                x = x.materialize()
            act = ops.gated_activation(ops.linear(x, self.w_gate_up), self.act)
            return ops.PendingLinear(act, self.w_down) if defer else ops.linear(act, self.w_down)
        if isinstance(x, ops.NormedRows):
            if self.interleaved and ops.skinny_scaled_ok(x, self.w_gate_up):
                act = ops.skinny_gemm_scaled(x, self.w_gate_up, silu_mul=True)   # decode: norm, product and SiLU-mul in one
                return ops.PendingLinear(act, self.w_down) if defer else ops.linear(act, self.w_down)
            if self.interleaved and ops.tc_stream_scaled_ok(x, self.w_gate_up):
                act = ops.tc_stream_gemm(x, self.w_gate_up, silu_mul=True)       # the same for 17 to 64 rows
                return ops.PendingLinear(act, self.w_down) if defer else ops.linear(act, self.w_down)
            x = x.materialize()
        if self.interleaved and x.shape[0] <= ops.SKINNY_AUTO_ROWS and ops.skinny_gemm_ok(x, self.w_gate_up):
            act = ops.skinny_gemm(x, self.w_gate_up, silu_mul=True)              # decode: weights streamed once
        elif (self.interleaved and x.shape[0] <= ops.TC_STREAM_AUTO_ROWS and ops.tc_stream_ok(x, self.w_gate_up)):
            # decode batches of 17 to 32 rows: the swapped-operand tcgen05 product, SiLU-mul in its epilogue
            act = ops.tc_stream_gemm(x, self.w_gate_up, silu_mul=True)
        elif self.interleaved and x.shape[0] >= ops.TC_GEMM_MIN_ROWS and ops.tc_gemm_ok(x, self.w_gate_up):
            # prefill: tcgen05 on CTA pairs, SiLU-mul in the epilogue
            act = ops.tc_gemm(x, self.w_gate_up, silu_mul=True, tile="256x256")
        else:
            act = ops.silu_mul(ops.linear(x, self.w_gate_up), interleaved=self.interleaved)
        return ops.PendingLinear(act, self.w_down) if defer else ops.linear(act, self.w_down)


class DenseMLP(FeedForward):
    """down(act(up(x))) without a gate.  params: ``hidden_size``,
    ``intermediate_size``, ``activation`` ("relu2": the square of relu, "relu",
    "gelu_tanh", "silu"), ``names`` (the up and down matrices' names after the
    prefix)."""

    @classmethod
    def tensor_specs(cls, p, prefix):
        H, I = p["hidden_size"], p["intermediate_size"]
        up, down = p["names"]
        return {prefix + up: TensorSpec((I, H)), prefix + down: TensorSpec((H, I))}

    def __init__(self, p, prefix, env, tensors):
        super().__init__(p, prefix, env, tensors)
        if p["activation"] not in ops.ACTIVATIONS:
            raise ValueError(f"activation {p['activation']!r} is not known; known: {sorted(ops.ACTIVATIONS)}")
        self.act = p["activation"]
        up, down = p["names"]
        self.w_up = tensors.get(prefix + up, env.dtype)
        self.w_down = tensors.get(prefix + down, env.dtype)

    def forward(self, x, batch):
        return ops.linear(ops.activation(ops.linear(x, self.w_up), self.act), self.w_down)


register_feed_forward("swiglu", SwiGLU)
register_feed_forward("dense_mlp", DenseMLP)

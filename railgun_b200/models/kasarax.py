"""Kasarax as a description in parts.

Layers in the order the configuration lists them.  A layer is a mixer and
(unless it has none) a feed-forward side by side on the same stream behind
ONE norm that both read (arrangement "parallel_residual" with the same norm
on both branches): h = norm1(x); x <- x + (mixer(h) + ff(h)).  Norm weights
are stored around zero and applied as 1 + w.

Mixers: "attention" is grouped-query softmax attention ("gqa_attention")
with biases, keys and values of different sizes, no rotation, a query factor
1 + coef ln(floor((p + 1) / every) + 1) at position p, a sink of score 0 in
the softmax's denominator and a sigmoid gate per head on the heads' outputs.
"parallel" is two mixers that read the same input, each output RMS-normed over
the width with a weight of its own, half their sum ("parallel" with
``out_norms``): on the left attention without biases behind a short causal
convolution on q, k and v, with RMS norms over the whole of q and of k,
interleaved rotation of part of each head and a learned sink per head; on the
right lightning attention ("retention" with silu on q, k and v, no rotation,
one RMS norm over all heads' outputs and a sigmoid gate):
S_t = decay_h S_(t-1) + k_t v_t^T, o_t = S_t^T q_t.

Feed-forwards: down(silu(gate h) * up h), or routed experts down(relu(up
.)^2) chosen by the largest sigmoid router scores, whose scores multiply the
experts' INPUT and are not renormalized.  Final norm, then the embedding
matrix as the head, times ``logit_scale`` (multiplied into the final norm's
weight, which is the same product).

Tensor names: ``embed``, ``l<i>.norm1``, ``l<i>.mix.*`` (``.left.*`` and
``.right.*`` in a parallel mixer), ``l<i>.mlp.gate|up|down`` or
``l<i>.mlp.router`` and ``l<i>.mlp.e<j>.up|down``, ``final.norm``.
"""
from __future__ import annotations

from ..config.kasarax import KasaraxConfig
from ..config.registry import Architecture, register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, SubLayer


def _mixer_spec(c: KasaraxConfig, L) -> PartSpec:
    W, m = c.width, L.mixer
    if L.type == "attention":
        return PartSpec("gqa_attention", dict(
            hidden_size=W, num_heads=m.heads, num_kv_heads=m.kv_heads, head_dim=m.dim, v_dim=m.vdim, scale=m.scale,
            rot_dims=0, eps=c.norm_eps, window=0, bias=True, qk_norm=False, head_temp=False,
            q_temp=(m.temp_coef, m.temp_every) if m.temp_every else None, sink="zero", out_gate=True))
    a, s = m.left, m.right
    left = PartSpec("gqa_attention", dict(
        hidden_size=W, num_heads=a.heads, num_kv_heads=a.kv_heads, head_dim=a.dim, v_dim=a.vdim, scale=a.scale,
        rot_dims=a.rot_dims, rot_base=a.rot_base, rot_layout="interleaved", eps=c.norm_eps, window=0, bias=False,
        qk_norm="whole", head_temp=False, sink="learned", conv=a.conv, base="mix.left."))
    right = PartSpec("retention", dict(
        hidden_size=W, num_heads=s.heads, head_dim=s.dim, v_dim=s.vdim, decay=tuple(s.decay), rot_dims=0,
        eps=c.norm_eps, k_scale=1.0, activation="silu", norm="whole", gate="sigmoid", base="mix.right."))
    return PartSpec("parallel", dict(branches=((left, 0.5), (right, 0.5)), out_norms=("mix.left.out", "mix.right.out"),
                                     hidden_size=W, eps=c.norm_eps))


def _ffn_spec(c: KasaraxConfig, f) -> PartSpec:
    if f.kind == "dense":
        return PartSpec("swiglu", dict(hidden_size=c.width, intermediate_size=f.ff, activation="silu",
                                       names=("mlp.gate", "mlp.up", "mlp.down")))
    return PartSpec("routed_experts", dict(
        hidden_size=c.width, experts=f.experts, identity=0, top=f.top, expert_size=f.ff, shared_size=None, base="mlp.",
        correction=False, renormalize=False, scoring="sigmoid", gated=False, activation="relu2", scale_input=True))


def kasarax_model_spec(c: KasaraxConfig) -> ModelSpec:
    W = c.width

    def norm(name, mult=None):
        return PartSpec("rmsnorm", dict(size=W, eps=c.norm_eps, name=name, one_plus=True, mult=mult))

    layers = []
    for i, L in enumerate(c.layers):
        subs = [SubLayer(norm("norm1"), _mixer_spec(c, L), "mixer")]
        if L.mlp is not None:
            subs.append(SubLayer(norm("norm1"), _ffn_spec(c, L.mlp), "ffn"))
        layers.append(LayerSpec(prefix=f"l{i}.", sublayers=tuple(subs), arrangement="parallel_residual"))
    return ModelSpec(
        hidden_size=W, vocab_size=c.vocab, max_position=c.max_position,
        embedding=PartSpec("token_embedding", dict(vocab_size=c.vocab, hidden_size=W, name="embed")),
        layers=tuple(layers),
        final_norm=norm("final.norm", mult=c.logit_scale),
        head=PartSpec("lm_head", dict(vocab_size=c.vocab, hidden_size=W, name="embed")),
    )


KASARAX = register_architecture(Architecture(
    name="Kasarax",
    config_from_dict=KasaraxConfig.from_dict,
    model_spec=kasarax_model_spec,
    description="mixer and feed-forward side by side behind one norm: gated attention with a logarithmic query "
                "factor and a zero sink, or convolved attention with a learned sink beside lightning attention, "
                "each normed and halved; dense or input-weighted relu-squared experts; tied head with a logit scale",
    family="Kasarax",
), replace=True)

"""Mepatar as a description in parts.

Embedding times a constant; layers in the order the configuration lists them.
A layer is a mixer and (unless it has none) a feed-forward side by side on
the same stream, each behind a norm of its own (arrangement
"parallel_residual"): x <- x + (mixer(norm1(x)) + ff(norm2(x))).  The norms
are RMS norms in groups: the row is cut into equal consecutive parts and each
is divided by its own root mean square.  Every mixer reads h + conv(h), a
short causal convolution per channel over the request's tokens
("input_conv").  Mixers: "retention" (linear attention with a fixed decay per
head), "attention" (grouped-query softmax attention with biases, a norm on q
and k, interleaved rotation, a number per head on the scores and a sliding
window that keeps the first tokens: "gqa_attention"), "delta" (the gated
delta rule behind convolutions on q, k and v: "gated_delta").  Feed-forwards:
down(gelu_tanh(gate x) * up x), or routed experts with a clamped gated
activation whose weights are the chosen experts' softmax scores as they are.
Final norm (in groups too), then the head.

Tensor names: ``embed``, ``l<i>.norm1|norm2``, ``l<i>.canon1``,
``l<i>.mix.*``, ``l<i>.mlp.gate|up|down`` or ``l<i>.mlp.router`` and
``l<i>.mlp.e<j>.gate|up|down``, ``final.norm``, ``head``.
"""
from __future__ import annotations

from ..config.mepatar import MepatarConfig
from ..config.registry import Architecture, register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, SubLayer


def _mixer_spec(c: MepatarConfig, L) -> PartSpec:
    W, m = c.width, L.mixer
    if L.type == "retention":
        inner = PartSpec("retention", dict(
            hidden_size=W, num_heads=m.heads, head_dim=m.dim, v_dim=m.vdim, decay=tuple(m.decay),
            rot_dims=m.rot_dims, rot_base=m.rot_base, eps=c.norm_eps))
    elif L.type == "attention":
        inner = PartSpec("gqa_attention", dict(
            hidden_size=W, num_heads=m.heads, num_kv_heads=m.kv_heads, head_dim=m.dim, v_dim=m.vdim, scale=m.scale,
            rot_dims=m.rot_dims, rot_base=m.rot_base, rot_layout="interleaved", eps=c.norm_eps, window=m.window,
            keep_first=m.keep_first, bias=True, qk_norm=True, head_temp=True))
    else:
        inner = PartSpec("gated_delta", dict(
            hidden_size=W, num_heads=m.heads, num_qk_heads=m.kv_heads, head_dim=m.dim, v_dim=m.vdim, taps=m.conv,
            eps=c.norm_eps))
    if not c.canon_taps:
        return inner
    return PartSpec("input_conv", dict(channels=W, taps=c.canon_taps, name="canon1", inner=inner))


def _ffn_spec(c: MepatarConfig, f) -> PartSpec:
    if f.kind == "dense":
        return PartSpec("swiglu", dict(hidden_size=c.width, intermediate_size=f.ff, activation="gelu_tanh",
                                       names=("mlp.gate", "mlp.up", "mlp.down")))
    return PartSpec("routed_experts", dict(
        hidden_size=c.width, experts=f.experts, identity=0, top=f.top, expert_size=f.ff, shared_size=None, base="mlp.",
        correction=False, renormalize=False, activation="clamped_swish", limit=f.limit))


def mepatar_model_spec(c: MepatarConfig) -> ModelSpec:
    W = c.width

    def norm(name):
        return PartSpec("rmsnorm", dict(size=W, eps=c.norm_eps, name=name, groups=c.norm_groups))

    layers = []
    for i, L in enumerate(c.layers):
        subs = [SubLayer(norm("norm1"), _mixer_spec(c, L), "mixer")]
        if L.mlp is not None:
            subs.append(SubLayer(norm("norm2"), _ffn_spec(c, L.mlp), "ffn"))
        layers.append(LayerSpec(prefix=f"l{i}.", sublayers=tuple(subs), arrangement="parallel_residual"))
    return ModelSpec(
        hidden_size=W, vocab_size=c.vocab, max_position=c.max_position,
        embedding=PartSpec("token_embedding", dict(vocab_size=c.vocab, hidden_size=W, name="embed",
                                                   scale=c.embedding_scale)),
        layers=tuple(layers),
        final_norm=norm("final.norm"),
        head=PartSpec("lm_head", dict(vocab_size=c.vocab, hidden_size=W, name="head")),
    )


MEPATAR = register_architecture(Architecture(
    name="Mepatar",
    config_from_dict=MepatarConfig.from_dict,
    model_spec=mepatar_model_spec,
    description="parallel mixer and feed-forward on one stream behind grouped norms and an input convolution: "
                "retention, gated delta rule and windowed softmax attention that keeps the first tokens; "
                "routed experts with a clamped gated activation",
    family="Mepatar",
), replace=True)

"""Block arrangements: how a layer's parts sit around the residual stream.

"prenorm": for every branch of the layer in turn, x = x + part(norm(x)); the
usual block is x = x + mixer(norm(x)); x = x + ffn(norm(x))
(crates/vllm-models/src/llama/architecture.rs:47-58).  Each addition is done
inside the next norm's kernel, in 32-bit; at small decode batches the
addition moves into the kernel of the product before it and the norm into the
kernel of the product after it (ops.PendingLinear, ops.NormedRows).

"sandwich": a norm behind each part as well as before it,
x = x + post_norm(part(norm(x))); constant factors on the branch (a residual
multiplier, a per-feature layer scale) are part of the post-norm's weight.
The post-norm, the 32-bit addition and the next branch's norm are one kernel
(ops.PendingNormed).

"hyper": S copies of the residual stream instead of one (hyper-connections).
A branch reads u = sum_s a[s] x_s through its norm, and its output y changes
every copy at once: x_t <- sum_s M[s, t] x_s + b[t] y, with a [S], M [S, S]
(indexed [from, to]) and b [S] tensors of the branch.  All copies start as the
embedding's output and are summed into one stream at the end.  The update by
one branch and the read of the next are one kernel (ops.hyper_step), as the
pre-norm block's addition lives in the next norm's kernel.

"parallel_residual": the layer's branches all read the same stream, each
through a norm of its own, and their outputs are added to it together:
x = x + (mixer(norm1(x)) + ffn(norm2(x))).  The sum of the branches' outputs,
its addition to the 32-bit residual and the next layer's norms are one
kernel (ops.PendingSum, ops.add_group_rmsnorm): the norms of one layer differ
in their weights only, so the row's statistics are computed once.  Branches
that are given the SAME norm (the same tensor with the same constants) read
one normed row: h = norm(x); x = x + (mixer(h) + ffn(h)).

"reinject" (a stream operation): x <- W [x; x0] with x0 the embedding's
output, for models that feed the input again at the start of a pass over a
span of layers.
"""
from __future__ import annotations

import torch

from .. import ops
from ..weights.loader import TensorSpec
from .base import Arrangement, StreamOp, normed_input
from .registry import register_arrangement, register_stream_op


class PreNorm(Arrangement):
    def run(self, layer, stream, batch, cache, writes):
        for b in layer.branches:
            h = normed_input(b.norm, b.part, stream)
            more = dict(defer=True) if getattr(b.part, "defers_output", False) else {}
            if b.role == "mixer":
                stream.pending = b.part.forward(h, batch, cache, writes, **more)
            else:
                stream.pending = b.part.forward(h, batch, **more)


class Sandwich(Arrangement):
    def run(self, layer, stream, batch, cache, writes):
        for b in layer.branches:
            if b.post_norm is None:
                raise ValueError("the 'sandwich' arrangement needs a post_norm on every branch")
            h = normed_input(b.norm, b.part, stream)
            y = b.part.forward(h, batch, cache, writes) if b.role == "mixer" else b.part.forward(h, batch)
            stream.pending = ops.PendingNormed(y, b.post_norm.weight, b.post_norm.eps)


class ParallelResidual(Arrangement):
    """Up to two branches side by side on the same stream."""

    def run(self, layer, stream, batch, cache, writes):
        bs = layer.branches
        if len(bs) > 2:
            raise ValueError("the 'parallel_residual' arrangement takes one or two branches")
        norms = [b.norm for b in bs]
        same = all(getattr(n, "fuses_pending_sum", False) and hasattr(n, "groups") for n in norms) and len(
            {(n.groups, n.eps, n.env.dtype) for n in norms}) == 1
        pending = stream.pending
        if isinstance(pending, (ops.PendingLinear, ops.PendingNormed)):
            pending = pending.materialize()
        if same:
            # branches behind one and the same norm share its output
            shared = len(norms) == 2 and norms[0].prefix == norms[1].prefix and norms[0].params == norms[1].params
            hs = ops.add_group_rmsnorm(stream.resid, pending, [n.weight for n in (norms[:1] if shared else norms)],
                                       norms[0].groups, norms[0].eps, norms[0].env.dtype)
            if shared:
                hs = [hs[0], hs[0]]
        else:
            # norms of different kinds: the first one adds what is pending, the others read the sum
            hs = []
            for b in bs:
                hs.append(normed_input(b.norm, None, stream))
                stream.pending = None
        ys = []
        for b, h in zip(bs, hs):
            ys.append(b.part.forward(h, batch, cache, writes) if b.role == "mixer" else b.part.forward(h, batch))
        stream.pending = ops.PendingSum(ys)


class HyperWiring:
    """One branch's hyper-connection coefficients, 32-bit on the device."""

    def __init__(self, a, M, b):
        self.a, self.M, self.b = a, M, b


class Hyper(Arrangement):
    """A branch's ``wiring``: ``streams`` (S) and ``name`` (its tensors are
    ``<prefix><name>.in`` [S], ``.out`` [S] and ``.mix`` [S, S])."""

    @classmethod
    def tensor_specs(cls, sublayer, prefix):
        w = sublayer.wiring
        if not w:
            raise ValueError("the 'hyper' arrangement needs `wiring` (streams, name) on every branch")
        S, n = int(w["streams"]), prefix + w["name"]
        return {n + ".in": TensorSpec((S,), init="norm"), n + ".out": TensorSpec((S,), init="norm"),
                n + ".mix": TensorSpec((S, S), init="eye")}

    def bind(self, sublayer, prefix, env, tensors):
        n = prefix + sublayer.wiring["name"]
        get = lambda x: tensors.get(n + x, torch.float32).contiguous()
        return HyperWiring(get(".in"), get(".mix"), get(".out"))

    @staticmethod
    def _fold(stream):
        """The copies' sum (with the last branch's update) becomes the one stream again."""
        y, w = stream.pending if stream.pending is not None else (None, None)
        stream.resid = ops.hyper_step(stream.copies, None, y, w.M if w else None, w.b if w else None, None, None, 0.0,
                                      torch.float32)
        stream.pending, stream.copies = None, None

    def run(self, layer, stream, batch, cache, writes):
        for b in layer.branches:
            w = b.wiring
            weight, eps = b.norm.weight, b.norm.eps
            if stream.copies is None:
                # the first branch of the step: every copy is the embedding's output
                if stream.pending is not None:
                    raise ValueError("the 'hyper' arrangement starts from a stream with nothing pending")
                T, W = stream.resid.shape
                stream.copies = torch.empty((T, w.a.numel(), W), dtype=torch.float32, device=stream.resid.device)
                h = ops.hyper_step(stream.copies, stream.resid, None, None, None, w.a, weight, eps, self_dtype(b))
                stream.resid = None
                stream.closer = self._fold
            else:
                y, prev = stream.pending
                h = ops.hyper_step(stream.copies, None, y, prev.M, prev.b, w.a, weight, eps, self_dtype(b))
            y = b.part.forward(h, batch, cache, writes) if b.role == "mixer" else b.part.forward(h, batch)
            stream.pending = (y, w)


def self_dtype(branch):
    return branch.part.env.dtype


class Reinject(StreamOp):
    """params: ``hidden_size``, ``name`` (the matrix [H, 2 H], the stream's half first)."""

    @classmethod
    def tensor_specs(cls, p, prefix):
        return {p["name"]: TensorSpec((p["hidden_size"], 2 * p["hidden_size"]))}

    def __init__(self, p, prefix, env, tensors):
        super().__init__(p, prefix, env, tensors)
        self.H = p["hidden_size"]
        self.weight = tensors.get(p["name"], env.dtype)

    def begin(self, stream, batch):
        # [x | x0] in the activation type: the right half is filled here, once per step
        both = torch.empty((stream.resid.shape[0], 2 * self.H), dtype=self.env.dtype, device=stream.resid.device)
        ops.add_postnorm_rmsnorm(stream.resid, None, None, 0.0, None, out=both[:, self.H:])
        stream.kept[self] = both

    def apply(self, stream, batch):
        both = stream.kept[self]
        # what is pending is added (32-bit), the sum goes into the left half, the product is the new stream
        pending = stream.pending.materialize() if isinstance(stream.pending, ops.PendingLinear) else stream.pending
        ops.add_postnorm_rmsnorm(stream.resid, pending, None, 0.0, None, out=both[:, :self.H])
        stream.pending = None
        stream.resid = ops.linear(both, self.weight, out_dtype=torch.float32)


register_arrangement("prenorm", PreNorm)
register_arrangement("sandwich", Sandwich)
register_arrangement("hyper", Hyper)
register_arrangement("parallel_residual", ParallelResidual)
register_stream_op("reinject", Reinject)

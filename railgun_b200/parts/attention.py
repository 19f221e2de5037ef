"""Grouped-query attention over the paged cache.

q, k, v = x Wq^T, x Wk^T, x Wv^T (crates/vllm-models/src/llama/attention.rs:94-96);
positions are encoded into q and k, k and v go to the cache, then every query
attends its request's keys up to its own position (and not further back than
the window, if there is one), and the result goes through Wo (:133).  The
three projections are one matrix here, stacked by rows at load, which gives
the same numbers as three products.
"""
from __future__ import annotations

import os

import torch

from .. import ops
from ..cache.manager import PagedKVNeed, StateNeed
from ..weights.loader import TensorSpec
from .base import Mixer
from .latent_attention import rotary_frequencies
from .registry import register_mixer, POSITION_ENCODINGS


# The tcgen05 flash kernel takes portions of prompts when the head size is 64 and pages hold 8..128 tokens;
# RAILGUN_B200_TC_ATTENTION=0 sends them to the mma.sync kernel instead.
USE_TC_ATTENTION = os.environ.get("RAILGUN_B200_TC_ATTENTION", "1") != "0"


class PagedAttention(Mixer):
    """params: ``hidden_size``, ``num_heads``, ``num_kv_heads``, ``head_dim``,
    ``window`` (0: none), ``scale`` (None: head_dim^-0.5), ``position``
    (a PartSpec or None)."""

    @classmethod
    def tensor_specs(cls, p, prefix):
        H, nh, nkv, d = p["hidden_size"], p["num_heads"], p["num_kv_heads"], p["head_dim"]
        return {
            prefix + "self_attn.q_proj.weight": TensorSpec((nh * d, H)),
            prefix + "self_attn.k_proj.weight": TensorSpec((nkv * d, H)),
            prefix + "self_attn.v_proj.weight": TensorSpec((nkv * d, H)),
            prefix + "self_attn.o_proj.weight": TensorSpec((H, nh * d)),
        }

    @classmethod
    def cache_need(cls, p):
        return PagedKVNeed(p["num_kv_heads"], p["head_dim"], int(p.get("window") or 0))

    def __init__(self, p, prefix, env, tensors):
        super().__init__(p, prefix, env, tensors)
        self.nh, self.nkv, self.d = p["num_heads"], p["num_kv_heads"], p["head_dim"]
        if self.nh % self.nkv:
            raise ValueError(f"{self.nh} heads cannot share {self.nkv} key/value heads")
        if self.d > 256:
            raise ValueError(f"head size {self.d} is above the attention kernels' limit of 256")
        self.window = int(p.get("window") or 0)
        self.scale = float(p["scale"]) if p.get("scale") is not None else float(self.d) ** -0.5
        a = prefix + "self_attn."
        pos = p.get("position")
        self.position = None
        if pos is not None:
            self.position = tensors.shared_part(("position", pos), lambda: POSITION_ENCODINGS.get(pos.kind)(
                pos.params, prefix, env, tensors))
        wq, wk = tensors.get(a + "q_proj.weight", env.dtype), tensors.get(a + "k_proj.weight", env.dtype)
        # With a rotary table and a head size in steps of 16, q and k rows are kept in the order in which every
        # 16 rows hold 8 whole rotation pairs (q . k does not notice; the cache then holds k in that order): the
        # projection of a few single tokens can then rotate and write the cache in its own kernel.
        self.paired8 = getattr(self.position, "rotary_table", None) is not None and self.d % 16 == 0
        if self.paired8:
            wq, wk = ops.reorder_rope_rows(wq, self.nh, self.d), ops.reorder_rope_rows(wk, self.nkv, self.d)
        self.w_qkv = torch.cat([wq, wk, tensors.get(a + "v_proj.weight", env.dtype)], dim=0).contiguous()
        tensors.drop(a + "q_proj.weight", a + "k_proj.weight", a + "v_proj.weight")
        self.w_o = tensors.get(a + "o_proj.weight", env.dtype)

    takes_normed_rows = True
    defers_output = True

    def forward(self, x, batch, cache, writes=True, defer=False):
        nh, nkv, d = self.nh, self.nkv, self.d
        slots = batch.slot_mapping[cache.group]
        if self.paired8 and self.env.dtype == torch.bfloat16 and ops.skinny_rope_ok(x, self.w_qkv, d):
            # a few single tokens: projection, rotation and cache write in one kernel
            qkv = ops.skinny_gemm_rope_cache(x, self.w_qkv, self.position.rotary_table, batch.positions,
                                             slots if writes else None, cache.kv, nh, nkv, d, batch.err_flag)
        elif (self.paired8 and self.env.dtype == torch.bfloat16 and batch.decode_only
              and ops.tc_stream_rope_ok(x, self.w_qkv, d)):
            # 17 to 64 single tokens: the same in the streaming tcgen05 product
            qkv = ops.tc_stream_gemm_rope_cache(x, self.w_qkv, self.position.rotary_table, batch.positions,
                                                slots if writes else None, cache.kv, nh, nkv, d, batch.err_flag)
        else:
            qkv = ops.linear(x, self.w_qkv)
            kv_dest = (cache.kv, slots) if writes else None
            wrote = False
            if self.position is not None:
                if self.paired8:
                    wrote = self.position.apply(qkv, batch, nh, nkv, d, kv_dest, paired8=True)
                else:
                    wrote = self.position.apply(qkv, batch, nh, nkv, d, kv_dest)
            if writes and not wrote:
                ops.rope_cache_write(qkv, None, batch.positions, slots, cache.kv, nh, nkv, d, cache.page_size,
                                     batch.err_flag)
        out = self.attend(qkv, batch, cache)
        return ops.PendingLinear(out, self.w_o) if defer else ops.linear(out, self.w_o)

    def attend(self, qkv, batch, cache):
        """Pick the attention kernels for this step's shape and precision:
        bfloat16 with a head size in steps of 16 runs on the tensor cores
        (requests with several tokens through the flash-style kernel, single
        tokens through the split kernel); everything else, and all of the
        32-bit path, through the general kernel."""
        nh, nkv, d = self.nh, self.nkv, self.d
        table = batch.block_table[cache.group]
        if qkv.dtype != torch.bfloat16 or d % 16:
            return ops.paged_attention_general(qkv, qkv.shape[1], cache.kv, table, batch.req_of_token,
                                               batch.positions, nh, nkv, d, self.window, self.scale)
        out = torch.empty((qkv.shape[0], nh * d), dtype=qkv.dtype, device=qkv.device)
        kv_tiles = nkv * (-(-(nh // nkv) // 8))
        if batch.decode_only:
            n = batch.num_tokens
            ops.decode_attention(qkv, qkv.shape[1], out, cache.kv, table, None, n, batch.req_of_token,
                                 batch.positions, nh, nkv, d, self.window, self.scale,
                                 ops.decode_splits(n, kv_tiles, batch.max_context_len))
            return out
        if batch.num_prefill_tiles:
            if USE_TC_ATTENTION and batch.num_prefill_tiles128 and ops.prefill_attention_tc_ok(
                    qkv, cache.kv, d, cache.page_size):
                ops.prefill_attention_tc(qkv, out, cache.kv, table, batch.prefill_tiles128, batch.positions,
                                         nh, nkv, d, self.window, self.scale)
            else:
                ops.prefill_attention(qkv, qkv.shape[1], out, cache.kv, table, batch.prefill_tiles, batch.positions,
                                      nh, nkv, d, self.window, self.scale)
        if batch.num_decode_rows:
            n = batch.num_decode_rows
            ops.decode_attention(qkv, qkv.shape[1], out, cache.kv, table, batch.decode_rows, n, batch.req_of_token,
                                 batch.positions, nh, nkv, d, self.window, self.scale,
                                 ops.decode_splits(n, kv_tiles, batch.max_context_len))
        return out


register_mixer("paged_attention", PagedAttention)


class NormedAttention(Mixer):
    """Grouped-query softmax attention with the options that recent designs add to it, each a parameter:
    biases on the four projections, an RMS norm on q and k before the rotation (per head, with one weight vector
    for all q heads and one for all k heads, or over the whole of q and the whole of k with weights of that
    size), a short causal convolution per channel on q, k and v directly behind the projections, rotation of
    the first ``rot_dims`` numbers of a head in either layout, a learned number per head on the scores
    (``head_temp``), a query factor that grows with the logarithm of the position (``q_temp``), a sink in the
    softmax's denominator (of score 0, or a learned score per head), a sigmoid gate per head on the heads'
    outputs, values of another size than keys, and a sliding window that keeps the request's first
    ``keep_first`` tokens visible (at their true positions).

    Keys, queries and values are padded with zeros to one size D (a multiple of 16 that holds both), so the
    key/value pages and the attention kernels are the ordinary ones; the output product's matrix gets zero
    columns to match.  The score's scale, the head's number and the position's factor are multiplied into q, in
    32-bit, before its one rounding; the sink and the gate are applied where the attention kernels divide by
    the denominator.

    params: ``hidden_size``, ``num_heads``, ``num_kv_heads``, ``head_dim``, ``v_dim``, ``scale`` (None:
    head_dim^-1/2), ``rot_dims``, ``rot_base``, ``rot_layout`` ("interleaved": pairs (2i, 2i + 1), or "half":
    pairs (i, i + rot_dims/2)), ``eps`` (of the q and k norms), ``window`` (0: none), ``keep_first``,
    ``bias``, ``head_temp`` (booleans, default true), ``qk_norm`` (true, the default: per head; "whole"; false),
    ``q_temp`` (None, or (coef, every): q at position p times 1 + coef ln(floor((p + 1) / every) + 1)),
    ``sink`` (None, "zero" or "learned"), ``out_gate`` (default false), ``conv`` (taps; 0: none; 1: a factor per
    channel),
    ``base`` (what the tensor names start with after the prefix, default "mix."; the tensors are q, k, v, o,
    their biases <name>.b, q.norm, k.norm, temp, sink [heads], g [heads, hidden_size], and q.conv, k.conv,
    v.conv [channels, taps] with the last column the current token's).

    With a convolution the request keeps, beside its pages, the last taps - 1 projected rows (32-bit) in its
    state slot."""

    @classmethod
    def _base(cls, p, prefix):
        return prefix + (p.get("base") if p.get("base") is not None else "mix.")

    @classmethod
    def _padded(cls, p) -> int:
        return -(-max(int(p["head_dim"]), int(p["v_dim"])) // 16) * 16

    @classmethod
    def _taps(cls, p) -> int:
        return max(0, int(p.get("conv") or 0))

    @classmethod
    def tensor_specs(cls, p, prefix):
        W, H, G, d, dv = p["hidden_size"], p["num_heads"], p["num_kv_heads"], p["head_dim"], p["v_dim"]
        b = cls._base(p, prefix)
        out = {b + "q": TensorSpec((H * d, W)), b + "k": TensorSpec((G * d, W)), b + "v": TensorSpec((G * dv, W)),
               b + "o": TensorSpec((W, H * dv))}
        if p.get("bias", True):
            out.update({b + "q.b": TensorSpec((H * d,)), b + "k.b": TensorSpec((G * d,)),
                        b + "v.b": TensorSpec((G * dv,)), b + "o.b": TensorSpec((W,))})
        norm = p.get("qk_norm", True)
        if norm:
            whole = norm == "whole"
            out[b + "q.norm"] = TensorSpec((H * d if whole else d,), init="norm")
            out[b + "k.norm"] = TensorSpec((G * d if whole else d,), init="norm")
        if p.get("head_temp", True):
            out[b + "temp"] = TensorSpec((H,), init="norm")
        if p.get("sink") == "learned":
            out[b + "sink"] = TensorSpec((H,))
        if p.get("out_gate"):
            out[b + "g"] = TensorSpec((H, W))
        K = cls._taps(p)
        if K >= 1:
            out.update({b + "q.conv": TensorSpec((H * d, K)), b + "k.conv": TensorSpec((G * d, K)),
                        b + "v.conv": TensorSpec((G * dv, K))})
        return out

    @classmethod
    def cache_need(cls, p):
        window = int(p.get("window") or 0)
        pages = PagedKVNeed(int(p["num_kv_heads"]), cls._padded(p), window,
                            keep_first=int(p.get("keep_first") or 0) if window else 0)
        K = cls._taps(p)
        if K <= 1:
            return pages
        H, G, d, dv = int(p["num_heads"]), int(p["num_kv_heads"]), int(p["head_dim"]), int(p["v_dim"])
        return (pages, StateNeed((K - 1, (H + G) * d + G * dv), "float32"))

    def __init__(self, p, prefix, env, tensors):
        super().__init__(p, prefix, env, tensors)
        self.H, self.G, self.d, self.dv = (int(p["num_heads"]), int(p["num_kv_heads"]), int(p["head_dim"]),
                                           int(p["v_dim"]))
        self.D = self._padded(p)
        self.C = (self.H + self.G) * self.d + self.G * self.dv
        if self.H % self.G:
            raise ValueError(f"{self.H} heads cannot share {self.G} key/value heads")
        if self.D > 256:
            raise ValueError(f"head size {self.D} is above the attention kernels' limit of 256")
        self.rot_dims = int(p.get("rot_dims") or 0)
        if self.rot_dims % 2 or not 0 <= self.rot_dims <= self.d:
            raise ValueError(f"{self.rot_dims} rotated numbers do not fit a head of {self.d}")
        layout = p.get("rot_layout") or "interleaved"
        if layout not in ("interleaved", "half"):
            raise ValueError(f"rotation layout {layout!r} is not known; known: ['half', 'interleaved']")
        self.interleaved = layout == "interleaved"
        self.window = int(p.get("window") or 0)
        self.keep_first = int(p.get("keep_first") or 0) if self.window else 0
        self.eps = float(p.get("eps") or 0.0)
        scale = float(p["scale"]) if p.get("scale") is not None else float(self.d) ** -0.5
        b = self._base(p, prefix)
        names = ["q", "k", "v"] + (["g"] if p.get("out_gate") else [])
        self.out_gate = bool(p.get("out_gate"))
        self.w_qkv = torch.cat([tensors.get(b + n, env.dtype) for n in names], dim=0).contiguous()
        self.b_qkv = self.b_o = None
        if p.get("bias", True):
            biases = [tensors.get(b + n, env.dtype) for n in ("q.b", "k.b", "v.b")]
            if self.out_gate:                                        # the gate's rows of the product have no bias
                biases.append(torch.zeros(self.H, dtype=env.dtype, device=biases[0].device))
            self.b_qkv = torch.cat(biases, dim=0).contiguous()
            self.b_o = tensors.get(b + "o.b", env.dtype).contiguous()
        tensors.drop(b + "q", b + "k", b + "v", b + "g", b + "q.b", b + "k.b", b + "v.b")
        w_o = tensors.get(b + "o", env.dtype)
        if self.D != self.dv:
            # zero columns where the attention's output rows carry padding
            padded = torch.zeros((w_o.shape[0], self.H, self.D), dtype=w_o.dtype, device=w_o.device)
            padded[:, :, :self.dv] = w_o.view(w_o.shape[0], self.H, self.dv)
            w_o = padded.view(w_o.shape[0], self.H * self.D)
            tensors.drop(b + "o")
        self.w_o = w_o.contiguous()
        norm = p.get("qk_norm", True)
        if norm not in (True, False, None, "whole", "head"):
            raise ValueError(f"qk_norm {norm!r} is not known; known: true (per head), 'whole', false")
        self.norm_whole = norm == "whole"
        self.q_norm = tensors.get(b + "q.norm", torch.float32).contiguous() if norm else None
        self.k_norm = tensors.get(b + "k.norm", torch.float32).contiguous() if norm else None
        # what every q head is multiplied by: the score's scale times the head's own number
        self.factor = torch.full((self.H,), scale, dtype=torch.float32, device=env.device)
        if p.get("head_temp", True):
            self.factor = (self.factor * tensors.get(b + "temp", torch.float32)).contiguous()
        temp = p.get("q_temp")
        self.temp_coef, self.temp_every = (float(temp[0]), int(temp[1])) if temp else (0.0, 0)
        if self.temp_every < 0:
            raise ValueError(f"q_temp.every {self.temp_every} must be positive")
        sink = p.get("sink")
        if sink not in (None, "zero", "learned"):
            raise ValueError(f"sink {sink!r} is not known; known: None, 'zero', 'learned'")
        self.sink = None
        if sink == "zero":
            self.sink = torch.zeros(self.H, dtype=torch.float32, device=env.device)
        elif sink == "learned":
            self.sink = tensors.get(b + "sink", torch.float32).contiguous()
        self.K = self._taps(p)
        self.taps = None
        if self.K >= 1:
            self.taps = torch.cat([tensors.get(b + n, torch.float32) for n in ("q.conv", "k.conv", "v.conv")],
                                  dim=0).t().contiguous()                                  # [taps, channels]
        base = float(p.get("rot_base") or 10000.0)
        self.freq = tensors.shared_part(("rotary_frequencies", self.rot_dims, base),
                                        lambda: rotary_frequencies(self.rot_dims, base).to(env.device))

    def input_weight(self):
        """The matrix of this mixer's first product, for a wrapper that computes the first products of several
        mixers that read the same rows as one (None: the product has a bias and stays here)."""
        return self.w_qkv if self.b_qkv is None else None

    def adopt_input_weight(self, view):
        self.w_qkv = view

    def forward(self, x, batch, cache, writes=True, proj=None):
        H, G, d, dv, D, C = self.H, self.G, self.d, self.dv, self.D, self.C
        if proj is None:
            proj = ops.linear(x, self.w_qkv, bias=self.b_qkv)                 # [T, q | k | v (| gate)]
        pages = cache.parts[0] if self.K > 1 else cache
        qkv = proj if proj.shape[1] == C else proj[:, :C]
        if self.K >= 1:
            state = cache.parts[1].state if self.K > 1 else None
            qkv = ops.causal_conv(qkv, 0, self.taps, state, batch, torch.float32)
            if writes and state is not None:
                ops.conv_state_update(proj, 0, state, batch)
        slots = batch.slot_mapping[pages.group] if writes else None
        q = ops.attention_prepare(qkv, pages.kv, self.q_norm, self.k_norm, self.eps, self.freq, self.rot_dims,
                                  self.interleaved, batch.positions, slots, self.factor, H, G, d, dv, D,
                                  norm_whole=self.norm_whole, temp_coef=self.temp_coef, temp_every=self.temp_every,
                                  out_dtype=self.env.dtype)
        gate = proj[:, C:] if self.out_gate else None
        out = self.attend(q.view(-1, H * D), batch, pages, gate)
        return ops.linear(out, self.w_o, bias=self.b_o)

    def attend(self, q, batch, cache, gate=None):
        """bfloat16 runs on the tensor cores (requests with several tokens through the flash-style kernel, single
        tokens through the split kernel; both know the window, the kept first tokens, the sink and the gate); the
        32-bit path runs the general kernel."""
        H, G, D = self.H, self.G, self.D
        table = batch.block_table[cache.group]
        if q.dtype != torch.bfloat16:
            return ops.paged_attention_general(q, q.shape[1], cache.kv, table, batch.req_of_token, batch.positions,
                                               H, G, D, self.window, 1.0, self.keep_first, sink=self.sink, gate=gate)
        out = torch.empty((q.shape[0], H * D), dtype=q.dtype, device=q.device)
        kv_tiles = G * (-(-(H // G) // 8))
        reach = batch.max_context_len
        if self.window:
            reach = min(reach, self.window + self.keep_first)
        if batch.num_prefill_tiles:
            ops.prefill_attention(q, q.shape[1], out, cache.kv, table, batch.prefill_tiles, batch.positions,
                                  H, G, D, self.window, 1.0, self.keep_first, sink=self.sink, gate=gate)
        n = batch.num_tokens if batch.decode_only else batch.num_decode_rows
        if n:
            ops.decode_attention(q, q.shape[1], out, cache.kv, table, None if batch.decode_only else batch.decode_rows,
                                 n, batch.req_of_token, batch.positions, H, G, D, self.window, 1.0,
                                 ops.decode_splits(n, kv_tiles, reach), keep_first=self.keep_first, sink=self.sink,
                                 gate=gate)
        return out


register_mixer("gqa_attention", NormedAttention)

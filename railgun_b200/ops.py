"""Python entry points of the hand-written sm_100a kernels.

Each function checks its arguments (device, dtype, contiguity, sizes), calls
the ``extern "C"`` launcher on the current CUDA stream and raises on any
error.  There is no CPU path and no library fallback: without a CUDA device,
or if a library fails to build, these raise.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_int, c_float, c_void_p, c_longlong

import torch

from . import native

F32, BF16 = 0, 1


class KernelError(RuntimeError):
    pass


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"unsupported dtype {t.dtype}: kernels take float32 or bfloat16")


def _check(t: torch.Tensor, name: str, dtype=None) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor (there is no CPU path)")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")


def _check_rows(t: torch.Tensor, name: str, dtype=None) -> None:
    """Like ``_check`` for a matrix whose rows may be further apart than its width (a slice of columns)."""
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor (there is no CPU path)")
    if t.dim() != 2 or t.stride(1) != 1 or t.stride(0) < t.shape[1]:
        raise KernelError(f"{name} must be a matrix with unit column stride")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")


def _ptr(t) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> c_void_p:
    """The current CUDA stream of the current device (what torch.cuda.stream and graph capture set)."""
    if _raw_stream is not None:
        return c_void_p(_raw_stream(torch.cuda.current_device()))
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _ok(code: int, what: str) -> None:
    if code == 0:
        return
    if code == 10001:
        raise KernelError(f"{what}: the kernel refuses these sizes or dtypes")
    raise KernelError(f"{what}: CUDA error {code}")


class LaunchCounter:
    """Counts launches of this package's own kernels (library matrix products
    are not counted).  A replayed CUDA graph adds the launches it captured."""

    def __init__(self):
        self.value = 0


_COUNTER = LaunchCounter()
_fn_cache: dict = {}


def launch_counter() -> LaunchCounter:
    return _COUNTER


# Programmatic dependent launch: a kernel may start (and fetch weights) while the kernel before it drains.
# RAILGUN_B200_PDL=0 switches it off.
PDL_ENABLED = os.environ.get("RAILGUN_B200_PDL", "1") != "0"
_pdl_set: set = set()


def _fn(lib_name: str, fn_name: str):
    fn = _fn_cache.get(fn_name)
    if fn is None:
        lib = native.load(lib_name)
        if lib_name not in _pdl_set:
            lib.rg_set_pdl.restype = None
            lib.rg_set_pdl(c_int(1 if PDL_ENABLED else 0))
            _pdl_set.add(lib_name)
        fn = getattr(lib, fn_name)
        fn.restype = c_int
        _fn_cache[fn_name] = fn
    _COUNTER.value += 1
    return fn


def embedding(ids: torch.Tensor, table: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    """residual [T, H] float32 = table[ids] * scale."""
    _check(ids, "ids", torch.int32)
    _check(table, "table")
    T, (V, H) = ids.numel(), table.shape
    out = torch.empty((T, H), dtype=torch.float32, device=table.device)
    _ok(_fn("embedding", "rg_embedding")(_ptr(ids), _ptr(table), c_int(_dtype_code(table)), _ptr(out),
                                         c_int(T), c_int(H), c_int(V), c_float(scale), _stream()), "embedding")
    return out


def add_rmsnorm(resid: torch.Tensor, pending, weight: torch.Tensor, eps: float, out_dtype,
                rows: torch.Tensor | None = None) -> torch.Tensor:
    """resid += pending (in place, 32-bit), then RMSNorm of resid.  With
    ``rows`` (int32 indices) only those rows are normed and resid is untouched."""
    _check(resid, "resid", torch.float32)
    _check(weight, "weight", torch.float32)
    T, H = resid.shape
    if weight.numel() != H:
        raise KernelError(f"norm weight has {weight.numel()} elements, rows have {H}")
    if pending is not None:
        _check(pending, "pending")
        if pending.shape != resid.shape:
            raise KernelError(f"pending {tuple(pending.shape)} vs residual {tuple(resid.shape)}")
    n_out = T
    if rows is not None:
        _check(rows, "rows", torch.int32)
        n_out = rows.numel()
    out = torch.empty((n_out, H), dtype=out_dtype, device=resid.device)
    _ok(_fn("norm", "rg_add_rmsnorm")(
        _ptr(resid), _ptr(pending), c_int(_dtype_code(pending) if pending is not None else 0), _ptr(weight),
        c_float(eps), _ptr(out), c_int(_dtype_code(out)), _ptr(rows), c_int(n_out), c_int(H), _stream()),
        "add_rmsnorm")
    return out



class PendingSum:
    """The outputs of several parts that read the same stream (a mixer and a
    feed-forward side by side), still to be added to it: first to one another,
    then to the residual, in 32-bit, inside the next norm's kernel."""

    def __init__(self, parts):
        self.parts = [p for p in parts if p is not None]
        if not 1 <= len(self.parts) <= 2:
            raise KernelError(f"a pending sum holds one or two outputs, not {len(self.parts)}")

    def materialize(self) -> torch.Tensor:
        """The sum as one 32-bit tensor, for a norm that takes tensors only."""
        out = self.parts[0].to(torch.float32, copy=True)
        for p in self.parts[1:]:
            out += p
        return out


def add_group_rmsnorm(resid: torch.Tensor, pending, weights, groups: int, eps: float, out_dtype,
                      rows: torch.Tensor | None = None):
    """resid += (the sum of ``pending``: None, a tensor, or a ``PendingSum`` of
    up to two) in place, in 32-bit; then RMSNorm of resid in ``groups`` equal
    consecutive parts, each divided by its own root mean square, once per
    weight vector in ``weights`` (one or two: branches that read the same
    stream through norms of their own).  Returns one output per weight.  With
    ``rows`` (int32 indices) only those rows are normed and resid is untouched."""
    _check(resid, "resid", torch.float32)
    T, H = resid.shape
    if groups < 1 or H % groups:
        raise KernelError(f"rows of {H} do not split into {groups} equal groups")
    if not 1 <= len(weights) <= 2:
        raise KernelError("add_group_rmsnorm: one or two weight vectors")
    for w in weights:
        _check(w, "weight", torch.float32)
        if w.numel() != H:
            raise KernelError(f"norm weight has {w.numel()} elements, rows have {H}")
    parts = pending.parts if isinstance(pending, PendingSum) else ([pending] if pending is not None else [])
    for p in parts:
        _check(p, "pending")
        if p.shape != resid.shape:
            raise KernelError(f"pending {tuple(p.shape)} vs residual {tuple(resid.shape)}")
    n_out = T
    if rows is not None:
        _check(rows, "rows", torch.int32)
        n_out = rows.numel()
    outs = [torch.empty((n_out, H), dtype=out_dtype, device=resid.device) for _ in weights]
    p1 = parts[0] if parts else None
    p2 = parts[1] if len(parts) > 1 else None
    _ok(_fn("norm", "rg_add_group_rmsnorm")(
        _ptr(resid), _ptr(p1), c_int(_dtype_code(p1) if p1 is not None else 0), _ptr(p2),
        c_int(_dtype_code(p2) if p2 is not None else 0), _ptr(weights[0]), _ptr(weights[1] if len(weights) > 1 else None),
        c_float(eps), _ptr(outs[0]), _ptr(outs[1] if len(outs) > 1 else None), c_int(_dtype_code(outs[0])), _ptr(rows),
        c_int(n_out), c_int(H), c_int(groups), _stream()), "add_group_rmsnorm")
    return outs


def norm_sum(ys, weights, consts, eps: float) -> torch.Tensor:
    """float32 [T, H] = sum_b consts[b] * RMSNorm(ys[b]; weights[b], eps): up to four [T, H] tensors of one type,
    each divided by its rows' root mean square, times its weight [H] (float32) and its constant, added in order."""
    n = len(ys)
    if not 1 <= n <= 4 or len(weights) != n or len(consts) != n:
        raise KernelError("norm_sum: one to four inputs, each with a weight and a constant")
    T, H = ys[0].shape
    for y, w in zip(ys, weights):
        _check(y, "y", ys[0].dtype)
        _check(w, "weight", torch.float32)
        if tuple(y.shape) != (T, H) or w.numel() != H:
            raise KernelError(f"norm_sum: input {tuple(y.shape)} or weight of {w.numel()} does not match [{T}, {H}]")
    out = torch.empty((T, H), dtype=torch.float32, device=ys[0].device)
    yp = (c_void_p * n)(*[y.data_ptr() for y in ys])
    wp = (c_void_p * n)(*[w.data_ptr() for w in weights])
    cs = (c_float * n)(*[float(c) for c in consts])
    _ok(_fn("norm", "rg_norm_sum")(yp, wp, cs, c_int(n), c_int(_dtype_code(ys[0])), c_float(eps), _ptr(out), c_int(T),
                                   c_int(H), _stream()), "norm_sum")
    return out


class PendingNormed:
    """A part's output that is still to be RMS-normed (``weight``, ``eps``; the
    weight holds whatever constant factors follow the norm) before it is added
    to the residual: a norm that follows does both inside its own kernel;
    ``materialize()`` computes the normed rows in 32-bit."""

    __slots__ = ("y", "weight", "eps")

    def __init__(self, y, weight, eps: float):
        self.y, self.weight, self.eps = y, weight, float(eps)

    @property
    def shape(self):
        return self.y.shape

    def materialize(self) -> torch.Tensor:
        out = torch.zeros(self.y.shape, dtype=torch.float32, device=self.y.device)
        add_postnorm_rmsnorm(out, self, None, 0.0, None)
        return out


def add_postnorm_rmsnorm(resid: torch.Tensor, pending, weight, eps: float, out_dtype, rows: torch.Tensor | None = None,
                         out: torch.Tensor | None = None):
    """resid += post-norm of ``pending`` (a ``PendingNormed``; a plain tensor is
    added as it is; None adds nothing), in place and in 32-bit; then the
    RMSNorm (``weight``, ``eps``) of the new rows in ``out_dtype``.  With
    ``weight`` None and an ``out_dtype`` the rows are returned unnormed (a copy
    of the stream in that type); with ``out_dtype`` None nothing is returned.
    ``rows`` as in ``add_rmsnorm``.  ``out``: a [rows, H] view to write into,
    whose rows may be further apart than H."""
    _check(resid, "resid", torch.float32)
    T, H = resid.shape
    post_w, post_eps, y = None, 0.0, pending
    if isinstance(pending, PendingNormed):
        post_w, post_eps, y = pending.weight, pending.eps, pending.y
        _check(post_w, "post-norm weight", torch.float32)
        if post_w.numel() != H:
            raise KernelError(f"post-norm weight has {post_w.numel()} elements, rows have {H}")
    if y is not None:
        _check(y, "pending")
        if y.shape != resid.shape:
            raise KernelError(f"pending {tuple(y.shape)} vs residual {tuple(resid.shape)}")
    if weight is not None:
        _check(weight, "weight", torch.float32)
        if weight.numel() != H:
            raise KernelError(f"norm weight has {weight.numel()} elements, rows have {H}")
    n_out = T
    if rows is not None:
        _check(rows, "rows", torch.int32)
        n_out = rows.numel()
    if out is None and out_dtype is not None:
        out = torch.empty((n_out, H), dtype=out_dtype, device=resid.device)
    if out is not None:
        if (not out.is_cuda or out.dim() != 2 or out.shape != (n_out, H) or out.stride(1) != 1
                or out.stride(0) < H):
            raise KernelError(f"out must be a CUDA [rows, {H}] view with unit column stride")
    _ok(_fn("norm", "rg_add_postnorm_rmsnorm")(
        _ptr(resid), _ptr(y), c_int(_dtype_code(y) if y is not None else 0), _ptr(post_w), c_float(post_eps),
        _ptr(weight), c_float(eps), _ptr(out), c_int(_dtype_code(out) if out is not None else 0),
        c_int(out.stride(0) if out is not None else H), _ptr(rows), c_int(n_out), c_int(H), _stream()),
        "add_postnorm_rmsnorm")
    return out


def softcap_(logits: torch.Tensor, cap: float) -> torch.Tensor:
    """logits <- cap * tanh(logits / cap), in place (32-bit)."""
    _check(logits, "logits", torch.float32)
    if not cap > 0.0:
        raise KernelError(f"a soft cap must be positive, got {cap}")
    _ok(_fn("activation", "rg_softcap")(_ptr(logits), c_float(cap), c_longlong(logits.numel()), _stream()), "softcap")
    return logits


def latent_rope_cache(proj: torch.Tensor, kv_off: int, qa, cache, norm_w: torch.Tensor, eps: float,
                      freq: torch.Tensor, rot_dims: int, positions: torch.Tensor, slots, H: int, dn: int, dr: int,
                      R: int, q_in_place: bool = False, interleaved: bool = False) -> None:
    """Per token of ``proj`` [T, H (dn + dr) + R + dr] (queries per head as
    [dn plain | dr rotated], then at ``kv_off`` the compressed key/value vector
    [R | dr]): rotate every head's rotated part into ``qa`` [T, H, R + dr][:, :, R:],
    and write [RMS norm of the R latent numbers times ``norm_w`` | rotated key
    part] into row ``slots[t]`` of ``cache`` [pages, page, R + dr] (``slots``
    None or a negative slot: no write).  Rotation: pairs (i, i + rot_dims / 2), or
    (2i, 2i + 1) with ``interleaved``, by position * ``freq[i]`` (64-bit
    frequencies and angles, 32-bit rotation).  ``q_in_place``: the rotated parts also
    replace the unrotated ones in ``proj`` (``qa`` may then be None)."""
    _check(proj, "proj")
    if qa is None and not q_in_place:
        raise KernelError("latent_rope_cache: nowhere to put the rotated query parts")
    if qa is not None:
        _check(qa, "qa", proj.dtype)
    _check(norm_w, "norm_w", torch.float32)
    _check(freq, "freq", torch.float64)
    _check(positions, "positions", torch.int32)
    T = proj.shape[0]
    D = R + dr
    if (proj.shape[1] < kv_off + D or kv_off < H * (dn + dr) or (qa is not None and qa.shape != (T, H, D))
            or positions.numel() != T):
        raise KernelError(f"latent_rope_cache: proj {tuple(proj.shape)}, qa {None if qa is None else tuple(qa.shape)} "
                          f"do not match {H} heads x ({dn} + {dr}), latent {R}")
    if norm_w.numel() != R or freq.numel() < rot_dims // 2:
        raise KernelError("latent_rope_cache: norm weight or frequency table of the wrong size")
    if slots is not None:
        _check(slots, "slots", torch.int32)
        _check(cache, "cache", proj.dtype)
        if cache.shape[-1] != D:
            raise KernelError(f"latent cache rows hold {cache.shape[-1]} numbers, the mixer writes {D}")
    _ok(_fn("attention_latent", "rg_latent_rope_cache")(
        _ptr(proj), c_int(proj.stride(0)), c_int(kv_off), _ptr(qa), _ptr(cache if slots is not None else None),
        c_int(_dtype_code(proj)), _ptr(norm_w), c_float(eps), _ptr(freq), c_int(rot_dims),
        c_int(1 if interleaved else 0), _ptr(positions),
        _ptr(slots), c_int(T), c_int(H), c_int(dn), c_int(dr), c_int(R), c_int(1 if q_in_place else 0), _stream()),
        "latent_rope_cache")


def latent_expand_context(cache: torch.Tensor, block_table: torch.Tensor, cu_seqlens: torch.Tensor,
                          context_lens: torch.Tensor, w_uk: torch.Tensor, w_uv: torch.Tensor, H: int, dn: int, dr: int,
                          dv: int, R: int):
    """The contexts of the step's requests that bring several tokens, expanded from the latent cache
    [pages, page, R + dr] into ordinary key/value pages [requests * max_blocks, 2, H, page, dn + dr] (keys
    [U_k c | rotated part], values U_v c zero-padded to dn + dr), numbered request by request.  Returns (pages,
    their block table [requests, max_blocks])."""
    _check(cache, "cache")
    _check(block_table, "block_table", torch.int32)
    _check(cu_seqlens, "cu_seqlens", torch.int32)
    _check(context_lens, "context_lens", torch.int32)
    _check(w_uk, "w_uk", cache.dtype)
    _check(w_uv, "w_uv", cache.dtype)
    n_req, MB = block_table.shape
    page, D = cache.shape[1], cache.shape[2]
    if D != R + dr or w_uk.shape != (H * dn, R) or w_uv.shape != (H * dv, R) or dv > dn + dr:
        raise KernelError("latent_expand_context: sizes do not match")
    N = n_req * MB * page
    lat = torch.empty((N, R), dtype=cache.dtype, device=cache.device)
    _ok(_fn("attention_latent", "rg_latent_gather")(
        _ptr(cache), _ptr(block_table), c_int(MB), _ptr(cu_seqlens), _ptr(context_lens), _ptr(lat),
        c_int(_dtype_code(cache)), c_int(n_req), c_int(page), c_int(R), c_int(D), _stream()), "latent_gather")
    kn = linear(lat, w_uk)
    vv = linear(lat, w_uv)
    kv = torch.empty((n_req * MB, 2, H, page, dn + dr), dtype=cache.dtype, device=cache.device)
    _ok(_fn("attention_latent", "rg_latent_pack_kv")(
        _ptr(kn), _ptr(vv), _ptr(cache), _ptr(block_table), c_int(MB), _ptr(cu_seqlens), _ptr(context_lens), _ptr(kv),
        c_int(_dtype_code(cache)), c_int(n_req), c_int(page), c_int(H), c_int(dn), c_int(dr), c_int(dv), c_int(R),
        _stream()), "latent_pack_kv")
    table = torch.arange(n_req * MB, dtype=torch.int32, device=cache.device).view(n_req, MB)
    return kv, table


def latent_attention_general(qa: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor,
                             req_of_token: torch.Tensor, positions: torch.Tensor, R: int, window: int,
                             scale: float, sink: torch.Tensor | None = None) -> torch.Tensor:
    """Attention of ``qa`` [T, H, D] over the latent cache [pages, page, D]: the
    scores use all D numbers of a cache row, the values are its first R.
    ``sink`` [H] float32: exp(sink[h]) joins head h's softmax denominator.
    Returns [T, H, R].  32-bit arithmetic, any sizes with R <= 1024."""
    _check(qa, "qa")
    _check(cache, "cache", qa.dtype)
    _check(block_table, "block_table", torch.int32)
    _check(req_of_token, "req_of_token", torch.int32)
    _check(positions, "positions", torch.int32)
    T, H, D = qa.shape
    if cache.dim() != 3 or cache.shape[2] != D or R > D:
        raise KernelError(f"latent cache {tuple(cache.shape)} does not match queries of {D} numbers, latent {R}")
    if sink is not None:
        _check(sink, "sink", torch.float32)
        if sink.numel() != H:
            raise KernelError(f"{sink.numel()} sinks for {H} heads")
    out = torch.empty((T, H, R), dtype=qa.dtype, device=qa.device)
    _ok(_fn("attention_latent", "rg_latent_attention_general")(
        _ptr(qa), _ptr(out), _ptr(cache), c_int(_dtype_code(qa)), _ptr(block_table), c_int(block_table.shape[1]),
        _ptr(req_of_token), _ptr(positions), c_int(T), c_int(H), c_int(R), c_int(D), c_int(cache.shape[1]),
        c_int(window or 0), c_float(scale), _ptr(sink), _stream()), "latent_attention_general")
    return out


# RAILGUN_B200_LATENT_MMA=0 sends everything that would run the tensor-core latent-cache kernel to the general one.
USE_LATENT_MMA = os.environ.get("RAILGUN_B200_LATENT_MMA", "1") != "0"


def latent_attention_mma_ok(dtype, H: int, R: int, D: int) -> bool:
    """Whether the tensor-core kernels take these sizes: bfloat16, latent and row sizes in steps of 16, a latent
    of at most 512 numbers, a row that fits shared memory."""
    if not USE_LATENT_MMA or dtype != torch.bfloat16 or R % 16 or D % 16 or not 16 <= R <= 512 or D < R:
        return False
    return (64 + 64) * (D + 8) * 2 + 4 * 16 * 40 * 2 + 4 * 128 * 4 <= 227 * 1024


def latent_decode_splits(n_tokens: int, head_chunks: int, max_context: int) -> int:
    """How many shares a single token's context is cut into: enough blocks to fill the device twice, at least
    64 keys a share."""
    by_residency = 296 // max(1, n_tokens * head_chunks)
    by_length = -(-max_context // 64)
    return max(1, min(by_residency, by_length, 64))


def latent_attention_mma(qa: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor, tiles,
                         rows, n_items: int, req_of_token: torch.Tensor, positions: torch.Tensor, R: int, window: int,
                         scale: float, num_splits: int = 1, sink: torch.Tensor | None = None, select=None,
                         out_scale: float = 1.0, score_from: int = 0) -> None:
    """Attention over the latent cache on the tensor cores, into ``out`` [T, H, R].  With ``tiles`` [n, 3]
    (first row, rows <= 64, request): requests with several tokens.  Without: ``n_items`` single tokens
    (``rows``, or rows 0..n_items-1), every context cut into ``num_splits`` shares that a second kernel adds.
    ``sink`` [H] float32: exp(sink[h]) joins head h's denominator.  ``select`` = (dv, heads per group): head h
    keeps only columns [(h // heads per group) dv, + dv) of its R output numbers, and ``out`` is a [T, H dv] view
    (rows may be further apart).  ``out_scale`` multiplies the result.  ``score_from`` (a multiple of 16): the
    scores use the row's numbers from there on only; the queries must be zero before it."""
    _check(qa, "qa", torch.bfloat16)
    _check(cache, "cache", torch.bfloat16)
    _check(block_table, "block_table", torch.int32)
    _check(req_of_token, "req_of_token", torch.int32)
    _check(positions, "positions", torch.int32)
    T, H, D = qa.shape
    sel_dv, sel_hpg, out_ld = 0, 1, 0
    if select is not None:
        sel_dv, sel_hpg = int(select[0]), int(select[1])
        _check_out_view(out, T, H * sel_dv, torch.bfloat16, "latent_attention_mma")
        out_ld = out.stride(0)
        if sel_dv < 2 or sel_dv % 2 or sel_hpg < 1 or -(-H // sel_hpg) * sel_dv > R:
            raise KernelError(f"latent_attention_mma: cannot select {sel_dv} of {R} columns per group of {sel_hpg} heads")
    else:
        _check(out, "out", torch.bfloat16)
        if out.shape != (T, H, R):
            raise KernelError(f"latent_attention_mma: out {tuple(out.shape)} is not [{T}, {H}, {R}]")
    if sink is not None:
        _check(sink, "sink", torch.float32)
        if sink.numel() != H:
            raise KernelError(f"{sink.numel()} sinks for {H} heads")
    if cache.dim() != 3 or cache.shape[2] != D or not latent_attention_mma_ok(qa.dtype, H, R, D):
        raise KernelError(f"latent_attention_mma: queries {tuple(qa.shape)}, cache {tuple(cache.shape)}, latent {R}")
    for t, name in ((tiles, "tiles"), (rows, "rows")):
        if t is not None:
            _check(t, name, torch.int32)
    part_o = part_ml = None
    if tiles is None and num_splits > 1:
        part_o = torch.empty((T, H, num_splits, R), dtype=torch.float32, device=qa.device)
        part_ml = torch.empty((T, H, num_splits, 2), dtype=torch.float32, device=qa.device)
        _COUNTER.value += 1                                   # the kernel that adds the shares
    _ok(_fn("attention_latent_mma", "rg_latent_attention_mma")(
        _ptr(qa), _ptr(out), _ptr(part_o), _ptr(part_ml), _ptr(cache), _ptr(block_table), c_int(block_table.shape[1]),
        _ptr(tiles), _ptr(rows), c_int(n_items), _ptr(req_of_token), _ptr(positions), c_int(H), c_int(R), c_int(D),
        c_int(cache.shape[1]), c_int(window or 0), c_float(scale), c_int(num_splits if tiles is None else 1),
        _ptr(sink), c_int(sel_dv), c_int(sel_hpg), c_int(out_ld), c_float(out_scale), c_int(score_from), _stream()),
        "latent_attention_mma")


MOE_TILE_ROWS = 32


MOE_SCORINGS = {"softmax": 0, "sigmoid": 1}


def moe_route(x: torch.Tensor, router: torch.Tensor, correction, top: int, renormalize: bool = True,
              scoring: str = "softmax"):
    """Router of a mixture of experts: softmax of the 32-bit logits ``router`` x
    over all N outputs (``scoring`` "sigmoid": the sigmoid of each logit
    instead); the ``top`` outputs with the largest score + correction
    (``correction`` None: the largest scores); weights = their scores over
    their sum, or with ``renormalize`` False the scores themselves.  Returns
    (ids int32 [T, top], weights float32 [T, top])."""
    _check(x, "x")
    _check(router, "router", torch.float32)
    if correction is not None:
        _check(correction, "correction", torch.float32)
    if scoring not in MOE_SCORINGS:
        raise KernelError(f"moe_route: scoring {scoring!r} is not known; known: {sorted(MOE_SCORINGS)}")
    T, W = x.shape
    N = router.shape[0]
    if router.shape[1] != W or (correction is not None and correction.numel() != N):
        raise KernelError(f"router {tuple(router.shape)} or its correction do not match rows of {W}")
    ids = torch.empty((T, top), dtype=torch.int32, device=x.device)
    weights = torch.empty((T, top), dtype=torch.float32, device=x.device)
    _ok(_fn("moe", "rg_moe_route")(_ptr(x), c_int(_dtype_code(x)), _ptr(router), _ptr(correction), _ptr(ids),
                                   _ptr(weights), c_int(T), c_int(W), c_int(N), c_int(top), c_int(1 if renormalize else 0),
                                   c_int(MOE_SCORINGS[scoring]), _stream()), "moe_route")
    return ids, weights


def moe_align(ids: torch.Tensor, num_experts: int, tile_rows: int = MOE_TILE_ROWS):
    """Group the (token, choice) pairs of ``ids`` [T, top] by expert (outputs
    from ``num_experts`` on have no expert behind them and get no place).
    Returns (sorted_pair [P], pair_pos [P] (-1: no place), tiles [max_tiles, 3]
    = (expert or -1, first place, places))."""
    _check(ids, "ids", torch.int32)
    P = ids.numel()
    max_tiles = (P + tile_rows - 1) // tile_rows + num_experts
    sorted_pair = torch.empty(P, dtype=torch.int32, device=ids.device)
    pair_pos = torch.empty(P, dtype=torch.int32, device=ids.device)
    tiles = torch.empty((max_tiles, 3), dtype=torch.int32, device=ids.device)
    _ok(_fn("moe", "rg_moe_align")(_ptr(ids), c_int(P), c_int(num_experts), c_int(tile_rows), _ptr(sorted_pair),
                                   _ptr(pair_pos), _ptr(tiles), c_int(max_tiles), _stream()), "moe_align")
    return sorted_pair, pair_pos, tiles


GATED_ACTIVATIONS = {"silu": 0, "gelu_tanh": 1, "clamped_swish": 2}


def gated_activation(gate_up: torch.Tensor, kind: str = "silu", limit: float = 0.0) -> torch.Tensor:
    """[T, 2I] = gate | up -> [T, I] = act(gate) * up in 32-bit: "silu", "gelu_tanh", or "clamped_swish":
    g' sigmoid(1.702 g') (u' + 1) with g' = min(g, limit), u' = clamp(u, -limit, limit)."""
    _check(gate_up, "gate_up")
    if kind not in GATED_ACTIVATIONS:
        raise KernelError(f"unknown gated activation {kind!r}; known: {sorted(GATED_ACTIVATIONS)}")
    T, two_i = gate_up.shape
    if two_i % 2:
        raise KernelError("gated_activation: last dimension must be even")
    out = torch.empty((T, two_i // 2), dtype=gate_up.dtype, device=gate_up.device)
    _ok(_fn("activation", "rg_gated_activation")(_ptr(gate_up), _ptr(out), c_int(_dtype_code(gate_up)), c_int(T),
                                                 c_int(two_i // 2), c_int(GATED_ACTIVATIONS[kind]), c_float(limit),
                                                 _stream()), "gated_activation")
    return out


def moe_grouped_gemm(a: torch.Tensor, src, src_div: int, w: torch.Tensor, tiles: torch.Tensor, places: int,
                     gated: bool, tile_rows: int = MOE_TILE_ROWS, act: str = "silu", limit: float = 0.0,
                     plain_act: str | None = None) -> torch.Tensor:
    """out[pos] = W_e a_row(pos) for every place of the tile list, e the tile's
    expert; ``w`` [E, N, K] (``gated``: [E, 2 N, K] = gate rows then up rows and
    out = silu(gate) * up, or another gated activation ``act``; not gated:
    ``plain_act`` names an activation on the product, see ``ACTIVATIONS``).  Row ``pos`` of the input is ``a[src[pos] // src_div]``
    or, without ``src``, ``a[pos]``.  Returns [places, N]; rows that belong to no
    tile are not written.  bfloat16 with rows on 16-byte boundaries runs on the
    tensor cores (tiles of 32 places: mma.sync, weight-streaming; tiles of 128:
    the grouped tcgen05 product, whose bounded waits ``tc_gemm_check`` reports
    on), everything else in 32-bit arithmetic on the CUDA cores (tiles of 32)."""
    _check(a, "a")
    _check(w, "w", a.dtype)
    _check(tiles, "tiles", torch.int32)
    if src is not None:
        _check(src, "src", torch.int32)
    E, rows_w, K = w.shape
    N = rows_w // 2 if gated else rows_w
    if a.shape[1] != K or (gated and rows_w % 2):
        raise KernelError(f"moe_grouped_gemm: a {tuple(a.shape)} vs w {tuple(w.shape)}")
    if tile_rows == 128:
        if not moe_grouped_gemm_tc_ok(a.dtype, K, a.stride(0)):
            raise KernelError("moe_grouped_gemm: tiles of 128 places are for the tensor-core path")
        # prompts: the tcgen05 product over the tile list (its rows come through TMA, so they are gathered
        # into expert order first); gate and up as one product, silu * up by the activation kernel
        if src is not None:
            rows = torch.empty((places, K), dtype=a.dtype, device=a.device)
            _ok(_fn("moe", "rg_moe_gather_rows")(_ptr(a), c_int(a.stride(0)), _ptr(src), c_int(src_div), _ptr(rows),
                                                 c_int(places), c_int(K), _stream()), "moe_gather_rows")
            a = rows
        elif a.shape[0] != places:
            raise KernelError(f"moe_grouped_gemm: {a.shape[0]} rows for {places} places")
        err = _tc_err.get(a.device)
        if err is None:
            err = _tc_err[a.device] = torch.zeros(1, dtype=torch.int32, device=a.device)
        global _tc_unchecked
        _tc_unchecked = True
        wide = torch.empty((places, rows_w), dtype=a.dtype, device=a.device)
        _ok(_fn("gemm_tcgen05", "rg_tc_gemm_grouped")(
            _ptr(a), c_int(a.stride(0)), c_int(places), _ptr(w), c_int(E), c_int(rows_w), c_int(K), _ptr(wide),
            c_int(rows_w), _ptr(tiles), c_int(tiles.shape[0]), _ptr(err), _stream()), "tc_gemm_grouped")
        if not gated:
            return activation(wide, plain_act) if plain_act else wide
        return silu_mul(wide) if act == "silu" else gated_activation(wide, act, limit)
    if act not in GATED_ACTIVATIONS:
        raise KernelError(f"unknown gated activation {act!r}; known: {sorted(GATED_ACTIVATIONS)}")
    if plain_act is not None and (gated or plain_act not in ACTIVATIONS):
        raise KernelError(f"moe_grouped_gemm: activation {plain_act!r} on a product without a gate; known: "
                          f"{sorted(ACTIVATIONS)}")
    act_code = GATED_ACTIVATIONS[act] if gated else (ACTIVATIONS[plain_act] if plain_act else -1)
    out = torch.empty((places, N), dtype=a.dtype, device=a.device)
    if moe_grouped_gemm_tc_ok(a.dtype, K, a.stride(0)):
        _ok(_fn("moe", "rg_moe_grouped_gemm_mma")(
            _ptr(a), c_int(a.stride(0)), _ptr(src), c_int(src_div), _ptr(w), _ptr(out), c_int(N), _ptr(tiles),
            c_int(tiles.shape[0]), c_int(tile_rows), c_int(N), c_int(K), c_int(1 if gated else 0),
            c_int(act_code), c_float(limit), _stream()), "moe_grouped_gemm_mma")
        return out
    _ok(_fn("moe", "rg_moe_grouped_gemm")(
        _ptr(a), c_int(a.stride(0)), _ptr(src), c_int(src_div), _ptr(w), _ptr(out), c_int(N), c_int(_dtype_code(a)),
        _ptr(tiles), c_int(tiles.shape[0]), c_int(tile_rows), c_int(N), c_int(K), c_int(1 if gated else 0),
        c_int(act_code), c_float(limit), _stream()), "moe_grouped_gemm")
    return out


def moe_grouped_gemm_tc_ok(dtype, K: int, lda: int) -> bool:
    """Whether the grouped product runs on the tensor cores: bfloat16, rows that start on 16-byte boundaries."""
    return dtype == torch.bfloat16 and K % 8 == 0 and lda % 8 == 0 and K >= 8


def moe_tile_rows(dtype, pairs: int, num_experts: int, K1: int, K2: int) -> int:
    """Places per tile of the grouped products: 128 (the tcgen05 product) once an expert gets 64 places on
    average (prompts: every weight row that is read serves 128 rows), else 32."""
    tc = moe_grouped_gemm_tc_ok(dtype, K1, K1) and moe_grouped_gemm_tc_ok(dtype, K2, K2)
    return 128 if tc and pairs >= 64 * max(1, num_experts) else MOE_TILE_ROWS


def moe_scaled_rows(x: torch.Tensor, sorted_pair: torch.Tensor, top: int, weights: torch.Tensor,
                    places: int) -> torch.Tensor:
    """[places, W]: place ``pos`` holds weights[pair] * x[pair // top] for the pair ``sorted_pair[pos]`` (32-bit
    product, one rounding): the input of experts whose weight multiplies what they read.  Places without a pair
    are not written."""
    _check_rows(x, "x")
    _check(sorted_pair, "sorted_pair", torch.int32)
    _check(weights, "weights", torch.float32)
    if sorted_pair.numel() < places or weights.numel() != x.shape[0] * top:
        raise KernelError("moe_scaled_rows: sizes do not match")
    out = torch.empty((places, x.shape[1]), dtype=x.dtype, device=x.device)
    _ok(_fn("moe", "rg_moe_gather_scaled_rows")(_ptr(x), c_int(_dtype_code(x)), c_int(x.stride(0)), _ptr(sorted_pair),
                                                c_int(top), _ptr(weights), _ptr(out), c_int(places), c_int(x.shape[1]),
                                                _stream()), "moe_scaled_rows")
    return out


def moe_combine(x: torch.Tensor, y, shared, ids: torch.Tensor, weights, pair_pos: torch.Tensor,
                num_experts: int) -> torch.Tensor:
    """float32 [T, W] = sum over a token's choices of weight * (the expert's
    row of ``y``, or the token's own row of ``x`` for a choice with no expert
    behind it), plus ``shared`` if given.  ``weights`` None: every weight is 1."""
    _check(x, "x")
    T, W = x.shape
    top = ids.shape[1]
    if y is not None:
        _check(y, "y", x.dtype)
    if shared is not None:
        _check(shared, "shared", x.dtype)
        if shared.shape != x.shape:
            raise KernelError(f"shared {tuple(shared.shape)} vs x {tuple(x.shape)}")
    out = torch.empty((T, W), dtype=torch.float32, device=x.device)
    _ok(_fn("moe", "rg_moe_combine")(_ptr(x), _ptr(y), _ptr(shared), c_int(_dtype_code(x)), _ptr(ids), _ptr(weights),
                                     _ptr(pair_pos), _ptr(out), c_int(T), c_int(W), c_int(num_experts), c_int(top),
                                     _stream()), "moe_combine")
    return out



# ---- hyper-connections, talking-heads attention, the gated recurrence, plain activations ---------------

def hyper_step(copies, x0, y, mix, outc, inc, norm_w, eps: float, out_dtype, out: torch.Tensor | None = None):
    """One pass over the copies of a hyper-connected residual stream ``copies`` [T, S, W] (32-bit, in
    place).  With ``x0`` [T, W]: every copy becomes x0 (the start).  With ``y`` [T, W]: every copy t becomes
    sum_s ``mix``[s, t] copy_s + ``outc``[t] y, all from the old copies.  Then u = sum_s ``inc``[s] copy_s
    (``inc`` None: the plain sum) is returned RMS-normed with ``norm_w`` in ``out_dtype``, or unnormed when
    ``norm_w`` is None; nothing is returned when ``out_dtype`` is None."""
    _check(copies, "copies", torch.float32)
    T, S, W = copies.shape
    for t, name, n in ((mix, "mix", S * S), (outc, "out", S), (inc, "in", S), (norm_w, "norm weight", W)):
        if t is not None:
            _check(t, name, torch.float32)
            if t.numel() != n:
                raise KernelError(f"hyper_step: {name} has {t.numel()} elements, expected {n}")
    for t, name in ((x0, "x0"), (y, "y")):
        if t is not None:
            _check(t, name)
            if t.shape != (T, W):
                raise KernelError(f"hyper_step: {name} {tuple(t.shape)} does not match copies {tuple(copies.shape)}")
    if x0 is not None and x0.dtype != torch.float32:
        raise KernelError("hyper_step: x0 must be float32")
    if out is None and out_dtype is not None:
        out = torch.empty((T, W), dtype=out_dtype, device=copies.device)
    if out is not None and (out.shape != (T, W) or out.stride(1) != 1):
        raise KernelError("hyper_step: out must be [T, W] with unit column stride")
    _ok(_fn("hyper", "rg_hyper_step")(
        _ptr(copies), _ptr(x0), _ptr(y), c_int(_dtype_code(y) if y is not None else 0), _ptr(mix), _ptr(outc), _ptr(inc),
        _ptr(norm_w), c_float(eps), _ptr(out), c_int(_dtype_code(out) if out is not None else 0),
        c_int(out.stride(0) if out is not None else W), c_int(T), c_int(S), c_int(W), _stream()), "hyper_step")
    return out


def talking_prepare(qkv: torch.Tensor, q_out, cache, q_norm, k_norm, eps: float, freq: torch.Tensor,
                    rot_dims: int, positions: torch.Tensor, slots, H: int, G: int, d: int, dv: int,
                    qa: torch.Tensor | None = None, talk=None, scale: float = 1.0,
                    qc: torch.Tensor | None = None) -> None:
    """Per token of ``qkv`` [T, H d + G d + G dv]: every q and k head is RMS-normed over its d numbers
    (``q_norm`` / ``k_norm`` [d] float32, None: no norm) and its first ``rot_dims`` numbers are rotated in
    pairs (i, i + rot_dims / 2) by position * ``freq[i]`` (float64); q goes to ``q_out`` [T, H, d] (if given),
    the values and the keys to row ``slots[t]`` of ``cache`` [pages, page, G dv + G d] (negative slot or None: no
    write).  ``qa`` [T, H, G dv + G d] (if given) receives the queries of the tensor-core form: zeros, then for
    every key/value head c the numbers ``scale`` * sum over the heads g of c of ``talk``[h, g] q_g; ``qc``
    [T, H, G d] (if given) the same without the zeros."""
    _check_rows(qkv, "qkv")
    if qc is not None:
        _check(qc, "qc", qkv.dtype)
        if qc.shape != (qkv.shape[0], H, G * d):
            raise KernelError(f"talking_prepare: qc {tuple(qc.shape)} is not [T, {H}, {G * d}]")
    if q_out is None and qa is None and qc is None:
        raise KernelError("talking_prepare: nowhere to put the queries")
    _check(freq, "freq", torch.float64)
    _check(positions, "positions", torch.int32)
    T = qkv.shape[0]
    if q_out is not None:
        _check(q_out, "q_out", qkv.dtype)
    if qa is not None:
        _check(qa, "qa", qkv.dtype)
        if qa.shape != (T, H, G * (d + dv)):
            raise KernelError(f"talking_prepare: qa {tuple(qa.shape)} is not [T, {H}, {G * (d + dv)}]")
    if talk is not None:
        _check(talk, "talk", torch.float32)
    if (qkv.shape[1] != (H + G) * d + G * dv or (q_out is not None and q_out.shape != (T, H, d))
            or positions.numel() != T):
        raise KernelError(f"talking_prepare: qkv {tuple(qkv.shape)} does not match {H} + {G} heads of {d}, values of {dv}")
    for w, name in ((q_norm, "q_norm"), (k_norm, "k_norm")):
        if w is not None:
            _check(w, name, torch.float32)
            if w.numel() != d:
                raise KernelError(f"talking_prepare: {name} has {w.numel()} elements, heads have {d}")
    if (q_norm is None) != (k_norm is None):
        raise KernelError("talking_prepare: q and k are normed together or not at all")
    if freq.numel() < rot_dims // 2:
        raise KernelError("talking_prepare: frequency table too short")
    if slots is not None:
        _check(slots, "slots", torch.int32)
        _check(cache, "cache", qkv.dtype)
        if cache.shape[-1] != G * (d + dv):
            raise KernelError(f"cache rows hold {cache.shape[-1]} numbers, the mixer writes {G * (d + dv)}")
    _ok(_fn("attention_talking", "rg_talking_prepare")(
        _ptr(qkv), c_int(_dtype_code(qkv)), c_int(qkv.stride(0)), _ptr(q_out), _ptr(cache if slots is not None else None),
        _ptr(q_norm), _ptr(k_norm), c_float(eps), _ptr(freq), c_int(rot_dims), _ptr(positions), _ptr(slots), c_int(T),
        c_int(H), c_int(G), c_int(d), c_int(dv), _ptr(qa), _ptr(talk), c_float(scale), _ptr(qc), _stream()), "talking_prepare")


# Up to this many key numbers side by side the flash form is the faster one for prompts (measured on B200: at 128
# 111 us against 168 for 2,048 tokens, at 256 455 against 427: that kernel holds one block per SM at head size 256).
TALKING_FLASH_MAX_KEYS = 128


def talking_flash_ok(dtype, G: int, d: int, dv: int) -> bool:
    """Whether prompts of talking-heads attention can run on the flash kernel of paged attention: bfloat16, all key
    heads side by side within the head sizes at which that kernel is the faster form, values no larger than that."""
    return dtype == torch.bfloat16 and (G * d) % 16 == 0 and 16 <= G * d <= TALKING_FLASH_MAX_KEYS and dv <= G * d


def talking_prefill_flash(qc: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor, batch, G: int, d: int,
                          dv: int, out: torch.Tensor, out_scale: float = 1.0) -> None:
    """Talking-heads attention of the step's requests that bring several tokens, from mixed queries ``qc``
    [T, H, G d]: their contexts are laid out as temporary key/value pages (every key/value head sees all key heads
    side by side and its own values, zero-padded), the flash kernel of paged attention runs over them, and the
    first ``dv`` numbers of every head's output, times ``out_scale``, go to those requests' rows of ``out``
    [T, H dv] (rows may be further apart).  Causal, no window."""
    _check(qc, "qc", torch.bfloat16)
    _check(cache, "cache", torch.bfloat16)
    T, H, Gd = qc.shape
    if Gd != G * d or cache.dim() != 3 or cache.shape[2] != G * (d + dv) or not talking_flash_ok(qc.dtype, G, d, dv):
        raise KernelError(f"talking_prefill_flash: queries {tuple(qc.shape)}, cache {tuple(cache.shape)}")
    _check_out_view(out, T, H * dv, qc.dtype, "talking_prefill_flash")
    n_req, MB = block_table.shape
    page = cache.shape[1]
    kv = torch.empty((n_req * MB, 2, G, page, Gd), dtype=cache.dtype, device=cache.device)
    _ok(_fn("attention_talking", "rg_talking_pack_kv")(
        _ptr(cache), _ptr(block_table), c_int(MB), _ptr(batch.cu_seqlens), _ptr(batch.context_lens), _ptr(kv),
        c_int(_dtype_code(cache)), c_int(n_req), c_int(page), c_int(G), c_int(d), c_int(dv), _stream()), "talking_pack_kv")
    table = torch.arange(n_req * MB, dtype=torch.int32, device=cache.device).view(n_req, MB)
    wide = torch.empty((T, H * Gd), dtype=qc.dtype, device=qc.device)
    prefill_attention(qc, H * Gd, wide, kv, table, batch.prefill_tiles, batch.positions, H, G, Gd, 0, 1.0)
    _ok(_fn("attention_talking", "rg_talking_select")(
        _ptr(wide), _ptr(out), c_int(out.stride(0)), c_float(out_scale), c_int(_dtype_code(wide)), _ptr(batch.cu_seqlens),
        _ptr(batch.req_of_token), c_int(T), c_int(H), c_int(Gd), c_int(dv), _stream()), "talking_select")


def _check_out_view(out, T: int, n: int, dtype, what: str):
    if not out.is_cuda or out.dtype != dtype or out.dim() != 2 or out.shape != (T, n) or out.stride(1) != 1:
        raise KernelError(f"{what}: out must be a CUDA [{T}, {n}] view of {dtype} with unit column stride")


def talking_attention_general(q: torch.Tensor, cache: torch.Tensor, talk, block_table: torch.Tensor,
                              req_of_token: torch.Tensor, positions: torch.Tensor, G: int, dv: int, window: int,
                              scale: float, out: torch.Tensor | None = None, out_scale: float = 1.0) -> torch.Tensor:
    """Attention of ``q`` [T, H, d] over cache rows [pages, page, G dv + G d] (values, then keys) with the heads' scores mixed by
    ``talk`` [H, H] (float32; None: no mixing) before the softmax.  Returns [T, H dv] times ``out_scale``
    (``out``: a view to write into, rows may be further apart).  32-bit arithmetic, H dv <= 4096."""
    _check(q, "q")
    _check(cache, "cache", q.dtype)
    _check(block_table, "block_table", torch.int32)
    _check(req_of_token, "req_of_token", torch.int32)
    _check(positions, "positions", torch.int32)
    T, H, d = q.shape
    if cache.dim() != 3 or cache.shape[2] != G * (d + dv) or H % G:
        raise KernelError(f"talking attention: cache {tuple(cache.shape)} does not match {G} heads of {d} + {dv}")
    if talk is not None:
        _check(talk, "talk", torch.float32)
        if talk.shape != (H, H):
            raise KernelError(f"talking attention: mixing matrix {tuple(talk.shape)} for {H} heads")
    if out is None:
        out = torch.empty((T, H * dv), dtype=q.dtype, device=q.device)
    _check_out_view(out, T, H * dv, q.dtype, "talking attention")
    _ok(_fn("attention_talking", "rg_talking_attention_general")(
        _ptr(q), _ptr(out), c_int(out.stride(0)), c_float(out_scale), _ptr(cache), c_int(_dtype_code(q)), _ptr(talk),
        _ptr(block_table), c_int(block_table.shape[1]), _ptr(req_of_token), _ptr(positions), c_int(T), c_int(H), c_int(G),
        c_int(d), c_int(dv), c_int(cache.shape[1]), c_int(window or 0), c_float(scale), _stream()),
        "talking_attention_general")
    return out


def recurrent_conv(proj: torch.Tensor, x_off: int, xb: torch.Tensor, taps: torch.Tensor, cb: torch.Tensor,
                   state: torch.Tensor, batch, halves_blocks: int = 0):
    """u [T, C] float32: the causal convolution (``taps`` [C, K], bias ``cb``) of proj[:, x_off:x_off + C] + ``xb``
    per channel along each request's tokens, continued from the request's state slot (``state`` [slots, K, C]:
    rows 0..K-2 the last inputs) unless the request starts at position 0.  With ``halves_blocks`` = B > 0 also
    returns u as two bfloat16 numbers per element, u = hi + lo to 2^-17, laid out [T, B, 2, C / B] (per block of
    channels the hi numbers, then the lo numbers): (u, halves)."""
    _check_rows(proj, "proj")
    for t, name in ((xb, "xb"), (taps, "taps"), (cb, "cb"), (state, "state")):
        _check(t, name, torch.float32)
    C, K = taps.shape
    T = proj.shape[0]
    if state.shape[1:] != (K, C) or proj.shape[1] < x_off + C or xb.numel() != C or cb.numel() != C:
        raise KernelError("recurrent_conv: sizes do not match")
    u = torch.empty((T, C), dtype=torch.float32, device=proj.device)
    halves = None
    if halves_blocks:
        if C % halves_blocks:
            raise KernelError(f"recurrent_conv: {C} channels do not split into {halves_blocks} blocks")
        halves = torch.empty((T, halves_blocks, 2, C // halves_blocks), dtype=torch.bfloat16, device=proj.device)
    _ok(_fn("recurrent", "rg_recurrent_conv")(
        _ptr(proj), c_int(_dtype_code(proj)), c_int(proj.stride(0)), c_int(x_off), _ptr(xb), _ptr(taps), _ptr(cb),
        _ptr(state), _ptr(batch.cu_seqlens), _ptr(batch.req_of_token), _ptr(batch.start_pos), _ptr(batch.state_slots),
        _ptr(u), c_int(T), c_int(C), c_int(K), _ptr(halves), c_int(C // halves_blocks if halves_blocks else 0),
        _stream()), "recurrent_conv")
    return (u, halves) if halves_blocks else u


# Steps whose longest portion is at most this many tokens compute gates and recurrence in one kernel.
RECURRENT_FUSED_MAX_TOKENS = 4


def recurrent_scan(proj: torch.Tensor, y_off: int, x_off: int, yb, xb, u: torch.Tensor, gates: torch.Tensor, rb, ib, lam,
                   decay: float, state: torch.Tensor, batch, out: torch.Tensor | None = None,
                   out_scale: float = 1.0) -> torch.Tensor:
    """The recurrence S_t = a_t S_(t-1) + sqrt(1 - a_t^2) i_t u_t along each request's tokens, with
    a = exp(-``decay`` sigmoid(gates_r + rb) softplus(lam)) and i = sigmoid(gates_i + ib) (``gates``
    [blocks, T, 2 bs] float32), from the request's state (row K-1 of its slot) or from zero at position 0;
    returns S_t gelu_tanh(proj[:, y_off:] + yb) times ``out_scale`` as [T, C] in proj's type, and leaves S and
    the convolution's last K-1 inputs in the slot."""
    _check_rows(proj, "proj")
    for t, name in ((yb, "yb"), (xb, "xb"), (u, "u"), (gates, "gates"), (rb, "rb"), (ib, "ib"), (lam, "lam"),
                    (state, "state")):
        _check(t, name, torch.float32)
    T, C = u.shape
    K = state.shape[1]
    blocks, bs = gates.shape[0], gates.shape[2] // 2
    if gates.shape != (blocks, T, 2 * bs) or blocks * bs != C or state.shape[2] != C or proj.shape[0] != T:
        raise KernelError("recurrent_scan: sizes do not match")
    if out is None:
        out = torch.empty((T, C), dtype=proj.dtype, device=proj.device)
    _check_out_view(out, T, C, proj.dtype, "recurrent_scan")
    R = batch.cu_seqlens.numel() - 1
    # portions of several tokens: the gates of all tokens in one parallel kernel, then the bare recurrence
    ab = None
    if batch.max_query_len > RECURRENT_FUSED_MAX_TOKENS:
        ab = torch.empty((2, T, C), dtype=torch.float32, device=proj.device)
        _COUNTER.value += 2
    _ok(_fn("recurrent", "rg_recurrent_scan")(
        _ptr(proj), c_int(_dtype_code(proj)), c_int(proj.stride(0)), c_int(y_off), c_int(x_off), _ptr(yb), _ptr(xb),
        _ptr(u), _ptr(gates), _ptr(rb), _ptr(ib), _ptr(lam), c_float(decay), _ptr(state), _ptr(batch.cu_seqlens),
        _ptr(batch.start_pos), _ptr(batch.state_slots), _ptr(out), c_int(out.stride(0)), c_float(out_scale), c_int(T),
        c_int(R), c_int(C), c_int(K), c_int(bs), _ptr(ab), c_int(batch.max_query_len), _stream()), "recurrent_scan")
    return out


# ---- short convolutions with state, matrix-state mixers (retention, delta rule), attention's per-token work -------

def causal_conv(x: torch.Tensor, x_off: int, taps: torch.Tensor, state, batch, out_dtype, residual: bool = False,
                silu: bool = False, out: torch.Tensor | None = None) -> torch.Tensor:
    """[T, C]: per channel the causal convolution of x[:, x_off:x_off + C] with ``taps`` [K, C] (tap-major: what the
    tensor files hold as [C, K], transposed once at load; last row: the
    current token's) along each request's tokens, continued from the K - 1 inputs in the request's state slot
    (``state`` [slots, K - 1, C] float32; None when K = 1) unless the request starts at position 0.  ``silu``:
    the activation on the convolution; ``residual``: x is added.  32-bit arithmetic, one rounding into
    ``out_dtype``.  The state is not changed (``conv_state_update`` does that, afterwards)."""
    _check_rows(x, "x")
    _check(taps, "taps", torch.float32)
    K, C = taps.shape
    T = x.shape[0]
    if x.shape[1] < x_off + C:
        raise KernelError(f"causal_conv: {C} channels from column {x_off} of rows of {x.shape[1]}")
    if K > 1:
        _check(state, "state", torch.float32)
        if tuple(state.shape[1:]) != (K - 1, C):
            raise KernelError(f"causal_conv: state {tuple(state.shape)} is not [slots, {K - 1}, {C}]")
    if out is None:
        out = torch.empty((T, C), dtype=out_dtype, device=x.device)
    _check_out_view(out, T, C, out_dtype, "causal_conv")
    _ok(_fn("state_mixers", "rg_causal_conv")(
        _ptr(x), c_int(_dtype_code(x)), c_int(x.stride(0)), c_int(x_off), _ptr(taps), _ptr(state if K > 1 else None),
        _ptr(batch.cu_seqlens), _ptr(batch.req_of_token), _ptr(batch.start_pos), _ptr(batch.state_slots), _ptr(out),
        c_int(_dtype_code(out)), c_int(out.stride(0)), c_int(T), c_int(C), c_int(K), c_int(1 if residual else 0),
        c_int(1 if silu else 0), _stream()), "causal_conv")
    return out


def conv_state_update(x: torch.Tensor, x_off: int, state: torch.Tensor, batch) -> None:
    """Leave the last K - 1 inputs x[:, x_off:x_off + C] of every request of the step in its slot of ``state``
    [slots, K - 1, C] (older ones move up when the step brought fewer than K - 1 tokens)."""
    _check_rows(x, "x")
    _check(state, "state", torch.float32)
    K1, C = state.shape[1:]
    if K1 < 1:
        return
    _ok(_fn("state_mixers", "rg_conv_state_update")(
        _ptr(x), c_int(_dtype_code(x)), c_int(x.stride(0)), c_int(x_off), _ptr(state), _ptr(batch.cu_seqlens),
        _ptr(batch.start_pos), _ptr(batch.state_slots), c_int(batch.num_requests), c_int(C), c_int(K1 + 1), _stream()),
        "conv_state_update")


def retention_prepare(proj: torch.Tensor, q_off: int, k_off: int, freq: torch.Tensor, rot_dims: int,
                      positions: torch.Tensor, H: int, d: int, k_scale: float, silu: bool = False, v_off: int = -1,
                      dv: int = 0):
    """q, k [T, H, d] float32 from the columns of ``proj`` at ``q_off`` and ``k_off``: the first ``rot_dims`` numbers
    of every head rotated in pairs (i, i + rot_dims / 2) by position * ``freq[i]`` (float64), k times ``k_scale``.
    ``silu``: the activation on q and k (before the rotation).  With ``v_off`` >= 0 also v [T, H dv] float32 from
    the columns at ``v_off``, with the same activation; returns (q, k) or (q, k, v)."""
    _check_rows(proj, "proj")
    _check(freq, "freq", torch.float64)
    _check(positions, "positions", torch.int32)
    T = proj.shape[0]
    if proj.shape[1] < max(q_off, k_off) + H * d or freq.numel() < rot_dims // 2 or (
            v_off >= 0 and (dv < 1 or proj.shape[1] < v_off + H * dv)):
        raise KernelError("retention_prepare: sizes do not match")
    q = torch.empty((T, H, d), dtype=torch.float32, device=proj.device)
    k = torch.empty((T, H, d), dtype=torch.float32, device=proj.device)
    v = torch.empty((T, H * dv), dtype=torch.float32, device=proj.device) if v_off >= 0 else None
    _ok(_fn("state_mixers", "rg_retention_prepare")(
        _ptr(proj), c_int(_dtype_code(proj)), c_int(proj.stride(0)), c_int(q_off), c_int(k_off), _ptr(freq),
        c_int(rot_dims), _ptr(positions), _ptr(q), _ptr(k), c_int(T), c_int(H), c_int(d), c_float(k_scale),
        c_int(1 if silu else 0), c_int(max(v_off, 0)), c_int(dv), _ptr(v), _stream()),
        "retention_prepare")
    return (q, k) if v is None else (q, k, v)


def delta_prepare(qkv: torch.Tensor, G: int, d: int, q_scale: float, unit_eps: float, ab: torch.Tensor, b_off: int,
                  a_off: int, A_log: torch.Tensor, dt_bias: torch.Tensor, H: int):
    """In place on ``qkv`` [T, >= 2 G d] float32: the G query heads (from column 0) and the G key heads (from
    column G d) become unit vectors, x / sqrt(sum(x^2) + ``unit_eps``), the queries times ``q_scale``.  Returns
    beta = sigmoid(ab[:, b_off:b_off + H]) and g = exp(-exp(A_log) softplus(ab[:, a_off:a_off + H] + dt_bias)),
    both [T, H] float32."""
    _check_rows(qkv, "qkv", torch.float32)
    _check_rows(ab, "ab")
    _check(A_log, "A_log", torch.float32)
    _check(dt_bias, "dt_bias", torch.float32)
    T = qkv.shape[0]
    if qkv.shape[1] < 2 * G * d or ab.shape[0] != T or ab.shape[1] < max(a_off, b_off) + H or A_log.numel() != H \
            or dt_bias.numel() != H:
        raise KernelError("delta_prepare: sizes do not match")
    beta = torch.empty((T, H), dtype=torch.float32, device=qkv.device)
    g = torch.empty((T, H), dtype=torch.float32, device=qkv.device)
    _ok(_fn("state_mixers", "rg_delta_prepare")(
        _ptr(qkv), c_int(qkv.stride(0)), c_int(G), c_int(d), c_float(q_scale), c_float(unit_eps), _ptr(ab),
        c_int(_dtype_code(ab)), c_int(ab.stride(0)), c_int(b_off), c_int(a_off), _ptr(A_log), _ptr(dt_bias), _ptr(beta),
        _ptr(g), c_int(T), c_int(H), _stream()), "delta_prepare")
    return beta, g


def state_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, state: torch.Tensor, batch, H: int, d: int, dv: int,
               decay: torch.Tensor | None = None, g: torch.Tensor | None = None,
               beta: torch.Tensor | None = None) -> torch.Tensor:
    """A matrix S [d, dv] per head carried along each request's tokens, 32-bit, from the request's slot of ``state``
    [slots, H, dv, d] (S transposed; zeros at position 0) and left there.  With ``decay`` [H]: S <- decay_h S + k v^T; with ``g``
    and ``beta`` [T, H]: S <- g S, u = beta (v - S^T k), S <- S + k u^T.  Either way o = S^T q after the update.
    ``q``, ``k``: float32 [T, Hqk * d] views (head h reads head h / (H / Hqk)); ``v``: [T, H * dv] view, float32 or
    bfloat16.
    Returns o [T, H, dv] float32."""
    for t, name in ((q, "q"), (k, "k")):
        _check_rows(t, name, torch.float32)
    _check_rows(v, "v")
    _check(state, "state", torch.float32)
    T = q.shape[0]
    Hqk = q.shape[1] // d
    if q.shape[1] != Hqk * d or k.shape != q.shape or v.shape != (T, H * dv) or Hqk < 1 or H % Hqk \
            or tuple(state.shape[1:]) != (H, dv, d):
        raise KernelError(f"state_scan: q {tuple(q.shape)}, k {tuple(k.shape)}, v {tuple(v.shape)}, state "
                          f"{tuple(state.shape)} do not match {H} heads of {d} x {dv}")
    for t, name, n in ((decay, "decay", H), (g, "g", T * H), (beta, "beta", T * H)):
        if t is not None:
            _check(t, name, torch.float32)
            if t.numel() != n:
                raise KernelError(f"state_scan: {name} has {t.numel()} elements, expected {n}")
    if (decay is None) == (g is None) or (beta is not None and g is None):
        raise KernelError("state_scan: a fixed decay per head, or g and beta per token")
    o = torch.empty((T, H, dv), dtype=torch.float32, device=q.device)
    _ok(_fn("state_mixers", "rg_state_scan")(
        _ptr(q), c_int(q.stride(0)), _ptr(k), c_int(k.stride(0)), _ptr(v), c_int(_dtype_code(v)), c_int(v.stride(0)),
        _ptr(decay), _ptr(g),
        _ptr(beta), _ptr(state), _ptr(batch.cu_seqlens), _ptr(batch.start_pos), _ptr(batch.state_slots), _ptr(o),
        c_int(batch.num_requests), c_int(H), c_int(Hqk), c_int(d), c_int(dv), _stream()), "state_scan")
    return o


def state_scan_rows(rows: int) -> None:
    """For measurements: make ``state_scan`` give every thread ``rows`` rows of S (4, 8, 16 or 32) instead of the
    launcher's own choice; 0 gives the choice back."""
    _fn("state_mixers", "rg_state_scan_rows")(c_int(rows))


HEAD_GATES = {"silu": 0, "sigmoid": 1}


def head_norm_gate(o: torch.Tensor, gate: torch.Tensor, weight, eps: float, out_dtype, whole: bool = False,
                   gate_kind: str = "silu") -> torch.Tensor:
    """[T, H dv] in ``out_dtype``: every head of ``o`` [T, H, dv] (float32) divided by its root mean square (``eps``
    inside the root), times ``weight`` [dv] (None: no weight), times silu(``gate``) ([T, H dv] view) or, with
    ``gate_kind`` "sigmoid", sigmoid(``gate``).  ``whole``: one root mean square over all H dv numbers of a token
    and a weight of that size."""
    _check(o, "o", torch.float32)
    _check_rows(gate, "gate")
    T, H, dv = o.shape
    if gate.shape != (T, H * dv):
        raise KernelError(f"head_norm_gate: gate {tuple(gate.shape)} vs o {tuple(o.shape)}")
    if gate_kind not in HEAD_GATES:
        raise KernelError(f"head_norm_gate: gate {gate_kind!r} is not known; known: {sorted(HEAD_GATES)}")
    if weight is not None:
        _check(weight, "weight", torch.float32)
        if weight.numel() != (H * dv if whole else dv):
            raise KernelError(f"head_norm_gate: weight has {weight.numel()} elements, expected "
                              f"{H * dv if whole else dv}")
    out = torch.empty((T, H * dv), dtype=out_dtype, device=o.device)
    _ok(_fn("state_mixers", "rg_head_norm_gate")(
        _ptr(o), _ptr(gate), c_int(_dtype_code(gate)), c_int(gate.stride(0)), c_int(0), _ptr(weight), c_float(eps),
        _ptr(out), c_int(_dtype_code(out)), c_int(T), c_int(H), c_int(dv), c_int(1 if whole else 0),
        c_int(HEAD_GATES[gate_kind]), _stream()), "head_norm_gate")
    return out


def attention_prepare(qkv: torch.Tensor, kv_cache, q_norm, k_norm, eps: float, freq: torch.Tensor, rot_dims: int,
                      interleaved: bool, positions: torch.Tensor, slots, factor, H: int, G: int, d: int, dv: int,
                      D: int, norm_whole: bool = False, temp_coef: float = 0.0, temp_every: int = 0,
                      out_dtype=None) -> torch.Tensor:
    """Per token of ``qkv`` [T, H d + G d + G dv] (a view whose rows may be further apart): q and k RMS-normed,
    per head over d (``q_norm`` / ``k_norm`` [d] float32) or, with ``norm_whole``, all q heads together and all k
    heads together (weights [H d] and [G d]); None: no norm.  Then their first ``rot_dims`` numbers rotated in
    pairs (2i, 2i + 1) (``interleaved``) or (i, i + rot_dims / 2) by position * ``freq[i]`` (float64), q head h
    times ``factor[h]`` (float32 [H] or None) and, with ``temp_every`` > 0, times
    1 + ``temp_coef`` ln(floor((position + 1) / ``temp_every``) + 1).
    Returns q [T, H, D] in ``out_dtype`` (default: qkv's; 32-bit rows may be rounded to bfloat16 here, once); k and
    v go to place ``slots[t]`` of ``kv_cache`` [pages, 2, G, page, D] of that type (negative slot or None: no
    write).  D >= max(d, dv): the rest of every row is zeros."""
    _check_rows(qkv, "qkv")
    _check(freq, "freq", torch.float64)
    _check(positions, "positions", torch.int32)
    T = qkv.shape[0]
    out_dtype = out_dtype or qkv.dtype
    if qkv.shape[1] != (H + G) * d + G * dv or positions.numel() != T or freq.numel() < rot_dims // 2:
        raise KernelError(f"attention_prepare: qkv {tuple(qkv.shape)} does not match {H} + {G} heads of {d}, values of {dv}")
    if out_dtype != qkv.dtype and qkv.dtype != torch.float32:
        raise KernelError("attention_prepare: only 32-bit rows can be written in another type")
    for w, name, n in ((q_norm, "q_norm", H * d if norm_whole else d), (k_norm, "k_norm", G * d if norm_whole else d),
                       (factor, "factor", H)):
        if w is not None:
            _check(w, name, torch.float32)
            if w.numel() != n:
                raise KernelError(f"attention_prepare: {name} has {w.numel()} elements, expected {n}")
    page_size = 1
    if slots is not None:
        _check(slots, "slots", torch.int32)
        _check(kv_cache, "kv_cache", out_dtype)
        page_size = kv_cache.shape[3]
        if tuple(kv_cache.shape[1:]) != (2, G, page_size, D):
            raise KernelError(f"kv cache shape {tuple(kv_cache.shape)} does not match {G} heads of {D}")
    q = torch.empty((T, H, D), dtype=out_dtype, device=qkv.device)
    _ok(_fn("attention_prepare", "rg_attention_prepare")(
        _ptr(qkv), c_int(_dtype_code(qkv)), c_int(qkv.stride(0)), _ptr(q), c_int(_dtype_code(q)),
        _ptr(kv_cache if slots is not None else None),
        _ptr(q_norm), _ptr(k_norm), c_int(1 if norm_whole else 0), c_float(eps), _ptr(freq), c_int(rot_dims),
        c_int(1 if interleaved else 0), _ptr(positions), _ptr(slots), _ptr(factor), c_float(temp_coef),
        c_int(temp_every), c_int(T), c_int(H), c_int(G), c_int(d), c_int(dv), c_int(D),
        c_int(page_size), _stream()), "attention_prepare")
    return q


def _sink_and_gate(sink, gate, nh: int, T: int, dtype):
    """Checks of the attention kernels' optional ``sink`` [heads] float32 (exp(sink[h]) joins head h's softmax
    denominator, once, unscaled, with neither key nor value) and ``gate`` ([T, heads] view in the kernels' storage
    type: head h's output at token t is multiplied by sigmoid(gate[t, h])).  Returns the gate's row stride."""
    if sink is not None:
        _check(sink, "sink", torch.float32)
        if sink.numel() != nh:
            raise KernelError(f"{sink.numel()} sinks for {nh} heads")
    if gate is None:
        return 0
    _check_rows(gate, "gate", dtype)
    if gate.shape[0] < T or gate.shape[1] != nh:
        raise KernelError(f"gate {tuple(gate.shape)} does not match {T} tokens of {nh} heads")
    return gate.stride(0)


ACTIVATIONS = {"relu2": 0, "relu": 1, "gelu_tanh": 2, "silu": 3}


def activation(x: torch.Tensor, kind: str, in_place: bool = True) -> torch.Tensor:
    """Elementwise activation computed in 32-bit: relu2 (the square of relu), relu, gelu_tanh, silu."""
    _check(x, "x")
    if kind not in ACTIVATIONS:
        raise KernelError(f"unknown activation {kind!r}; known: {sorted(ACTIVATIONS)}")
    out = x if in_place else torch.empty_like(x)
    _ok(_fn("activation", "rg_activation")(_ptr(x), _ptr(out), c_int(_dtype_code(x)), c_int(ACTIVATIONS[kind]),
                                           c_longlong(x.numel()), _stream()), "activation")
    return out


def residual_add(resid: torch.Tensor, pending: torch.Tensor) -> None:
    _check(resid, "resid", torch.float32)
    _check(pending, "pending")
    if pending.shape != resid.shape:
        raise KernelError(f"pending {tuple(pending.shape)} vs residual {tuple(resid.shape)}")
    _ok(_fn("norm", "rg_residual_add")(_ptr(resid), _ptr(pending), c_int(_dtype_code(pending)),
                                       c_longlong(resid.numel()), _stream()), "residual_add")


def silu_mul(gate_up: torch.Tensor, interleaved: bool = False) -> torch.Tensor:
    """[T, 2I] -> [T, I]: silu(gate) * up.  Plain storage: gate is the first
    half of a row, up the second.  ``interleaved``: blocks of 8 gate columns
    followed by their 8 up columns (the storage ``interleave_gate_up`` makes)."""
    _check(gate_up, "gate_up")
    T, two_i = gate_up.shape
    if two_i % 2 or (interleaved and two_i % 16):
        raise KernelError("silu_mul: last dimension must be even (a multiple of 16 when interleaved)")
    out = torch.empty((T, two_i // 2), dtype=gate_up.dtype, device=gate_up.device)
    name = "rg_silu_mul_interleaved" if interleaved else "rg_silu_mul"
    _ok(_fn("activation", name)(_ptr(gate_up), _ptr(out), c_int(_dtype_code(gate_up)),
                                c_int(T), c_int(two_i // 2), _stream()), "silu_mul")
    return out


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """Stack gate [I, K] and up [I, K] as blocks of 8 gate rows followed by the
    8 matching up rows, so that one 16-row tensor-core tile holds a gate
    element and its up element in the same thread (I % 8 == 0)."""
    I, K = gate.shape
    if I % 8 or up.shape != gate.shape:
        raise KernelError("interleave_gate_up: both [I, K] with I a multiple of 8")
    return torch.stack([gate.view(I // 8, 8, K), up.view(I // 8, 8, K)], dim=1).reshape(2 * I, K).contiguous()


SKINNY_MAX_ROWS = 64           # what the kernel takes
SKINNY_AUTO_ROWS = 16          # up to here it beats the library product on B200 (measured, with the fused
                               # residual / norm / rotary variants in a decoder layer), so linear() uses it


def skinny_gemm_ok(x: torch.Tensor, weight: torch.Tensor) -> bool:
    """Can the weight-streaming decode product take this shape?"""
    return (x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.dim() == 2
            and 0 < x.shape[0] <= SKINNY_MAX_ROWS and x.shape[1] % 8 == 0 and x.stride(1) == 1
            and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and weight.is_contiguous())


def skinny_gemm(x: torch.Tensor, weight: torch.Tensor, out_dtype=None, silu_mul: bool = False) -> torch.Tensor:
    """y = x W^T for up to 64 rows of x, reading W once at memory speed.
    ``silu_mul``: W is interleaved gate|up storage and y = silu(gate) * up."""
    if not skinny_gemm_ok(x, weight):
        raise KernelError(f"skinny_gemm refuses x {tuple(x.shape)} {x.dtype}, W {tuple(weight.shape)} {weight.dtype}: "
                          "bfloat16, at most 64 rows, K a multiple of 8")
    M, K = x.shape
    N = weight.shape[0]
    if weight.shape[1] != K:
        raise KernelError(f"skinny_gemm: x has {K} columns, W has {weight.shape[1]}")
    out_dtype = out_dtype or torch.bfloat16
    if silu_mul and (N % 16 or out_dtype != torch.bfloat16):
        raise KernelError("skinny_gemm: the SiLU-mul epilogue needs N % 16 == 0 and bfloat16 output")
    out = torch.empty((M, N // 2 if silu_mul else N), dtype=out_dtype, device=x.device)
    _ok(_fn("gemm_skinny", "rg_skinny_gemm")(
        _ptr(weight), _ptr(x), c_int(x.stride(0)), _ptr(out), c_int(out.shape[1]), c_int(_dtype_code(out)),
        c_int(1 if silu_mul else 0), c_int(M), c_int(N), c_int(K), _stream()), "skinny_gemm")
    return out


SKINNY_FUSED_MAX_ROWS = 16     # what the fused variants (residual epilogue, norm prologue) are compiled for


class NormedRows:
    """RMSNorm of the residual rows, not finished yet: ``scaled`` holds
    bf16(residual * norm weight) and ``partials`` [>= blocks, ld] the partial
    sums of squares of the residual rows, one row per block of the product that
    last added to the residual.  A product that follows multiplies its sums by
    1 / rms (``linear`` and ``skinny_gemm_scaled`` take this in place of a
    tensor); ``materialize()`` runs the norm kernel on the residual."""

    __slots__ = ("resid", "scaled", "partials", "blocks", "weight", "eps", "dtype")

    def __init__(self, resid, scaled, partials, blocks: int, weight, eps: float, dtype):
        self.resid, self.scaled, self.partials, self.blocks = resid, scaled, partials, blocks
        self.weight, self.eps, self.dtype = weight, eps, dtype

    @property
    def shape(self):
        return self.resid.shape

    def materialize(self) -> torch.Tensor:
        return add_rmsnorm(self.resid, None, self.weight, self.eps, self.dtype)


class PendingLinear:
    """A part's output x W^T, not computed yet: a norm that follows adds it to
    the residual inside the product's own kernel; ``materialize()`` runs the
    product."""

    __slots__ = ("x", "weight")

    def __init__(self, x, weight):
        self.x, self.weight = x, weight

    @property
    def shape(self):
        return (self.x.shape[0], self.weight.shape[0])

    def materialize(self) -> torch.Tensor:
        return linear(self.x, self.weight)


def skinny_fused_ok(x: torch.Tensor, weight: torch.Tensor, resid: torch.Tensor) -> bool:
    """Can x W^T be added to ``resid`` inside the decode product (which then
    also prepares the next norm)?  Only where ``linear`` would use that product."""
    return (x.shape[0] <= min(SKINNY_AUTO_ROWS, SKINNY_FUSED_MAX_ROWS) and skinny_gemm_ok(x, weight)
            and resid.dtype == torch.float32 and resid.is_contiguous() and resid.shape == (x.shape[0], weight.shape[0])
            and resid.shape[1] % 8 == 0)


def skinny_gemm_residual(x: torch.Tensor, weight: torch.Tensor, resid: torch.Tensor, norm_weight: torch.Tensor,
                         eps: float) -> NormedRows:
    """resid += x W^T (32-bit, in place), and the RMSNorm (``norm_weight``,
    ``eps``) of the new rows but for the factor 1 / rms, which the product that
    reads the result applies."""
    if not (x.shape[0] <= SKINNY_FUSED_MAX_ROWS and skinny_gemm_ok(x, weight)):
        raise KernelError(f"skinny_gemm_residual refuses x {tuple(x.shape)} {x.dtype}, W {tuple(weight.shape)}")
    _check(resid, "resid", torch.float32)
    _check(norm_weight, "norm_weight", torch.float32)
    M, K = x.shape
    N = weight.shape[0]
    if weight.shape[1] != K or resid.shape != (M, N) or norm_weight.numel() != N:
        raise KernelError(f"skinny_gemm_residual: x {tuple(x.shape)}, W {tuple(weight.shape)}, residual "
                          f"{tuple(resid.shape)}, norm weight {norm_weight.numel()}")
    ld = 8 * ((M + 7) // 8)
    partials = torch.empty(((N + 15) // 16, ld), dtype=torch.float32, device=x.device)
    scaled = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    blocks = c_int(0)
    _ok(_fn("gemm_skinny_fused", "rg_skinny_gemm_residual")(
        _ptr(weight), _ptr(x), c_int(x.stride(0)), _ptr(resid), c_int(resid.stride(0)), _ptr(norm_weight), _ptr(scaled),
        c_int(M), c_int(N), c_int(K), _ptr(partials), c_int(ld), ctypes.byref(blocks), _stream()),
        "skinny_gemm_residual")
    return NormedRows(resid, scaled, partials, blocks.value, norm_weight, eps, torch.bfloat16)


def skinny_scaled_ok(rows: NormedRows, weight: torch.Tensor) -> bool:
    return (rows.dtype == torch.bfloat16 and rows.shape[0] <= min(SKINNY_AUTO_ROWS, SKINNY_FUSED_MAX_ROWS)
            and skinny_gemm_ok(rows.scaled, weight) and rows.shape[1] == weight.shape[1])


def skinny_gemm_scaled(rows: NormedRows, weight: torch.Tensor, silu_mul: bool = False) -> torch.Tensor:
    """y = rmsnorm(residual rows) W^T from the unfinished norm ``rows``: the
    product over the scaled rows, its 32-bit sums multiplied by 1 / rms before
    the epilogue; ``silu_mul`` as in ``skinny_gemm``.  bfloat16 out."""
    if not skinny_scaled_ok(rows, weight):
        raise KernelError(f"skinny_gemm_scaled refuses rows {tuple(rows.shape)}, W {tuple(weight.shape)} {weight.dtype}")
    x = rows.scaled
    M, K = x.shape
    N = weight.shape[0]
    if silu_mul and N % 16:
        raise KernelError("skinny_gemm_scaled: the SiLU-mul epilogue needs N % 16 == 0")
    out = torch.empty((M, N // 2 if silu_mul else N), dtype=torch.bfloat16, device=x.device)
    _ok(_fn("gemm_skinny_fused", "rg_skinny_gemm_scaled")(
        _ptr(weight), _ptr(x), c_int(x.stride(0)), c_float(rows.eps), _ptr(rows.partials),
        c_int(rows.partials.stride(0)), c_int(rows.blocks), _ptr(out), c_int(out.shape[1]),
        c_int(1 if silu_mul else 0), c_int(M), c_int(N), c_int(K), _stream()), "skinny_gemm_scaled")
    return out


def rope_pair_order(d: int) -> torch.Tensor:
    """The "paired8" order of a head's features (d % 16 == 0): storage index ->
    original feature, such that rotation pair i = (i, i + d/2) sits at storage
    indices (16 (i // 8) + i % 8, + 8): every 16 consecutive features hold 8
    whole pairs.  q . k does not notice a reordering that q and k share."""
    if d % 16:
        raise KernelError(f"the paired8 order needs a head size that is a multiple of 16, not {d}")
    s = torch.arange(d)
    blk, r = s // 16, s % 16
    return torch.where(r < 8, 8 * blk + r, d // 2 + 8 * blk + (r - 8))


def reorder_rope_rows(weight: torch.Tensor, n_heads: int, d: int) -> torch.Tensor:
    """Rows of a q or k projection [n_heads * d, K] in the paired8 order."""
    order = rope_pair_order(d).to(weight.device)
    return weight.view(n_heads, d, -1)[:, order, :].reshape(n_heads * d, -1).contiguous()


def rope_cache_write(qkv: torch.Tensor, table, positions: torch.Tensor, slots, kv_cache,
                     nh: int, nkv: int, d: int, page_size: int, err_flag=None, paired8: bool = False) -> None:
    """Rotate the q and k heads of qkv [T, (nh+2nkv)d] in place by ``table``
    [max_pos, d] (None: no rotation) and write k, v to the paged cache
    [NP, 2, nkv, page_size, d] at ``slots`` (None: no write).  ``paired8``: the
    heads' features are in ``rope_pair_order``."""
    _check(qkv, "qkv")
    _check(positions, "positions", torch.int32)
    T = qkv.shape[0]
    if qkv.shape[1] != (nh + 2 * nkv) * d:
        raise KernelError(f"qkv row has {qkv.shape[1]} elements, expected {(nh + 2 * nkv) * d}")
    max_pos = 1 << 30
    if table is not None:
        _check(table, "rope table", torch.float32)
        if table.shape[1] != d:
            raise KernelError(f"rope table is for head size {table.shape[1]}, heads have {d}")
        max_pos = table.shape[0]
    if slots is not None:
        _check(slots, "slots", torch.int32)
        _check(kv_cache, "kv_cache", qkv.dtype)
        if tuple(kv_cache.shape[1:]) != (2, nkv, page_size, d):
            raise KernelError(f"kv cache shape {tuple(kv_cache.shape)} does not match "
                              f"[pages, 2, {nkv}, {page_size}, {d}]")
    _ok(_fn("rope_cache", "rg_rope_cache")(
        _ptr(qkv), c_int(_dtype_code(qkv)), _ptr(table), _ptr(positions), _ptr(slots),
        _ptr(kv_cache if slots is not None else None), c_int(T), c_int(nh), c_int(nkv), c_int(d),
        c_int(page_size), c_int(max_pos), _ptr(err_flag), c_int(1 if paired8 else 0), _stream()), "rope_cache_write")


def skinny_gemm_rope_cache(x, weight: torch.Tensor, table: torch.Tensor, positions: torch.Tensor, slots, kv_cache,
                           nh: int, nkv: int, d: int, err_flag=None) -> torch.Tensor:
    """The q|k|v projection of up to 8 single tokens with the rotary encoding
    and the cache write inside the product's kernel: returns [M, (nh+2nkv)d]
    whose q heads are rotated (its k and v columns are not written); k
    (rotated) and v go to ``kv_cache`` at ``slots`` (None: no write).  ``x``:
    bfloat16 rows or a ``NormedRows``; ``weight``'s q and k rows are in
    ``rope_pair_order``."""
    rows = x if isinstance(x, NormedRows) else None
    xin = rows.scaled if rows is not None else x
    if not skinny_rope_ok(x, weight, d):
        raise KernelError(f"skinny_gemm_rope_cache refuses rows {tuple(xin.shape)}, W {tuple(weight.shape)}, head size {d}")
    M, K = xin.shape
    N = weight.shape[0]
    if weight.shape[1] != K or N != (nh + 2 * nkv) * d:
        raise KernelError(f"skinny_gemm_rope_cache: W {tuple(weight.shape)} is not [({nh} + 2 x {nkv}) x {d}, {K}]")
    _check(table, "rope table", torch.float32)
    _check(positions, "positions", torch.int32)
    if table.shape[1] != d or positions.numel() < M:
        raise KernelError("skinny_gemm_rope_cache: the table's head size or the number of positions does not match")
    page_size = 0
    if slots is not None:
        _check(slots, "slots", torch.int32)
        _check(kv_cache, "kv_cache", torch.bfloat16)
        page_size = kv_cache.shape[3]
        if tuple(kv_cache.shape[1:]) != (2, nkv, page_size, d) or slots.numel() < M:
            raise KernelError(f"kv cache shape {tuple(kv_cache.shape)} does not match [pages, 2, {nkv}, page, {d}]")
    out = torch.empty((M, N), dtype=torch.bfloat16, device=xin.device)
    _ok(_fn("gemm_skinny_fused", "rg_skinny_gemm_rope_cache")(
        _ptr(weight), _ptr(xin), c_int(xin.stride(0)), c_float(rows.eps if rows is not None else 0.0),
        _ptr(rows.partials if rows is not None else None), c_int(rows.partials.stride(0) if rows is not None else 0),
        c_int(rows.blocks if rows is not None else 0), _ptr(out), c_int(N), c_int(M), c_int(N), c_int(K), _ptr(table),
        _ptr(positions), _ptr(slots), _ptr(kv_cache if slots is not None else None), c_int(nh), c_int(nkv), c_int(d),
        c_int(page_size), c_int(table.shape[0]), _ptr(err_flag), _stream()), "skinny_gemm_rope_cache")
    return out


def skinny_rope_ok(x, weight: torch.Tensor, d: int) -> bool:
    """Can the q|k|v projection of these rows rotate and write the cache in its own kernel?"""
    if d % 16:
        return False
    if isinstance(x, NormedRows):
        return skinny_scaled_ok(x, weight)
    return x.shape[0] <= min(SKINNY_AUTO_ROWS, SKINNY_FUSED_MAX_ROWS) and skinny_gemm_ok(x, weight)


def paged_attention_general(q: torch.Tensor, q_stride: int, kv_cache: torch.Tensor, block_table: torch.Tensor,
                            req_of_token: torch.Tensor, positions: torch.Tensor, nh: int, nkv: int, d: int,
                            window: int, scale: float, keep_first: int = 0, sink=None, gate=None) -> torch.Tensor:
    """The general attention kernel: out [T, nh*d].  ``q`` may be a view whose
    rows are ``q_stride`` elements apart (the q part of a fused qkv buffer).
    ``keep_first``: with a window, the first positions of a request that every
    later query still sees.  ``sink``, ``gate``: see ``_sink_and_gate``."""
    if not q.is_cuda:
        raise KernelError("q must be a CUDA tensor (there is no CPU path)")
    _check(kv_cache, "kv_cache", q.dtype)
    _check(block_table, "block_table", torch.int32)
    _check(req_of_token, "req_of_token", torch.int32)
    _check(positions, "positions", torch.int32)
    T = positions.numel()
    page_size = kv_cache.shape[3]
    if tuple(kv_cache.shape[1:]) != (2, nkv, page_size, d):
        raise KernelError(f"kv cache shape {tuple(kv_cache.shape)} does not match heads {nkv} x {d}")
    if d > 256:
        raise KernelError(f"head size {d} is above the kernels' limit of 256")
    out = torch.empty((T, nh * d), dtype=q.dtype, device=q.device)
    gate_ld = _sink_and_gate(sink, gate, nh, T, q.dtype)
    _ok(_fn("attention_general", "rg_paged_attention_general")(
        _ptr(q), c_int(q_stride), _ptr(out), _ptr(kv_cache), c_int(_dtype_code(q)), _ptr(block_table),
        c_int(block_table.shape[1]), _ptr(req_of_token), _ptr(positions), c_int(T), c_int(nh), c_int(nkv),
        c_int(d), c_int(page_size), c_int(window or 0), c_float(scale), c_int(keep_first if window else 0),
        _ptr(sink), _ptr(gate), c_int(gate_ld), _stream()),
        "paged_attention_general")
    return out


def _check_paged(q, kv_cache, block_table, nkv, d):
    if not q.is_cuda:
        raise KernelError("q must be a CUDA tensor (there is no CPU path)")
    if q.dtype != torch.bfloat16:
        raise KernelError(f"the tensor-core attention kernels take bfloat16, got {q.dtype}")
    _check(kv_cache, "kv_cache", q.dtype)
    _check(block_table, "block_table", torch.int32)
    page_size = kv_cache.shape[3]
    if tuple(kv_cache.shape[1:]) != (2, nkv, page_size, d):
        raise KernelError(f"kv cache shape {tuple(kv_cache.shape)} does not match heads {nkv} x {d}")
    if d % 16 or not 16 <= d <= 256:
        raise KernelError(f"the tensor-core attention kernels take head sizes 16, 32, ..., 256; got {d}")
    return page_size


def prefill_attention(q, q_stride: int, out, kv_cache, block_table, tiles, positions, nh: int, nkv: int, d: int,
                      window: int, scale: float, keep_first: int = 0, sink=None, gate=None) -> None:
    """Flash-style attention for requests that bring several tokens: ``tiles``
    [n, 3] = (first row, rows <= 64, request index).  Writes the tiles' rows of
    ``out`` [T, nh*d].  ``keep_first``: with a window, the first positions of a
    request that every later query still sees.  ``sink``, ``gate``: see
    ``_sink_and_gate``."""
    page_size = _check_paged(q, kv_cache, block_table, nkv, d)
    _check(tiles, "tiles", torch.int32)
    _check(positions, "positions", torch.int32)
    _check(out, "out", q.dtype)
    gate_ld = _sink_and_gate(sink, gate, nh, out.shape[0], q.dtype)
    _ok(_fn("attention_mma", "rg_prefill_attention_sink")(
        _ptr(q), c_int(q_stride), _ptr(out), _ptr(kv_cache), _ptr(block_table), c_int(block_table.shape[1]),
        _ptr(tiles), c_int(tiles.shape[0]), _ptr(positions), c_int(nh), c_int(nkv), c_int(d), c_int(page_size),
        c_int(window or 0), c_int(keep_first if window else 0), c_float(scale), _ptr(sink), _ptr(gate), c_int(gate_ld),
        _stream()), "prefill_attention")


def decode_splits(n_tokens: int, kv_tiles: int, max_context: int) -> int:
    """How many parts each context is cut into.  Measured on B200: the split
    kernel runs best when all its thread blocks are resident at once (4 per SM,
    592 in all) and each part has at least 256 keys; more parts only add
    partial results to reduce."""
    by_residency = 592 // max(1, n_tokens * kv_tiles)
    by_length = -(-max_context // 256)
    return max(1, min(by_residency, by_length, 256))


_decode_counters: dict = {}


def decode_attention(q, q_stride: int, out, kv_cache, block_table, rows, n_tokens: int, req_of_token, positions,
                     nh: int, nkv: int, d: int, window: int, scale: float, num_splits: int,
                     scratch=None, fused_reduce=None, cluster: bool = False, keep_first: int = 0, sink=None,
                     gate=None) -> None:
    """Split attention for single tokens: token rows ``rows`` (None: rows
    0..n_tokens-1) each attend their request's context.  Partial results go
    through scratch memory (allocated here unless given) and are reduced into
    ``out`` [T, nh*d] by the block that finishes last for each token and head
    tile (``fused_reduce``) or by a second kernel (the default: measured
    faster, the last block would reduce alone at the end of the launch); a
    single split writes the result itself.  ``cluster`` (2 to 8 splits): the
    splits of a (token, head tile) are one thread-block cluster and add their
    partial results through distributed shared memory; the fastest way for the
    kernel alone, not inside a decode step (see attention_mma.cu), so the
    engine leaves it off.  Every way adds the splits in split order.
    ``keep_first``: with a window, the first positions of a request that every
    later query still sees (not with ``cluster``).  ``sink``, ``gate``: see
    ``_sink_and_gate``; they enter where the splits are added up (not with
    ``cluster``)."""
    if fused_reduce is None:
        fused_reduce = num_splits == 1
    page_size = _check_paged(q, kv_cache, block_table, nkv, d)
    _check(req_of_token, "req_of_token", torch.int32)
    _check(positions, "positions", torch.int32)
    _check(out, "out", q.dtype)
    if rows is not None:
        _check(rows, "rows", torch.int32)
    gate_ld = _sink_and_gate(sink, gate, nh, out.shape[0], q.dtype)
    if cluster:
        if keep_first and window:
            raise KernelError("decode_attention: the cluster form does not keep first tokens")
        if sink is not None or gate is not None:
            raise KernelError("decode_attention: the cluster form has neither sink nor gate")
        if not 2 <= num_splits <= 8:
            raise KernelError("decode_attention: a cluster takes 2 to 8 splits")
        _ok(_fn("attention_mma", "rg_decode_attention_cluster")(
            _ptr(q), c_int(q_stride), _ptr(out), _ptr(kv_cache), _ptr(block_table), c_int(block_table.shape[1]),
            _ptr(rows), c_int(n_tokens), _ptr(req_of_token), _ptr(positions), c_int(nh), c_int(nkv), c_int(d),
            c_int(page_size), c_int(window or 0), c_float(scale), c_int(num_splits), _stream()), "decode_attention")
        return
    if scratch is None:
        part_o = torch.empty((n_tokens, nh, num_splits, d), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((n_tokens, nh, num_splits, 2), dtype=torch.float32, device=q.device)
    else:
        part_o, part_ml = scratch
        if part_o.numel() < n_tokens * nh * num_splits * d or part_ml.numel() < n_tokens * nh * num_splits * 2:
            raise KernelError("decode_attention: the scratch buffers are too small")
    counters = None
    if fused_reduce:
        # one counter per (token, kv head, tile of 8 query heads): zero on entry, left zero by the kernel
        need = n_tokens * nkv * (-(-(nh // nkv) // 8))
        counters = _decode_counters.get(q.device)
        if counters is None or counters.numel() < need:
            counters = _decode_counters[q.device] = torch.zeros(max(need, 4096), dtype=torch.int32, device=q.device)
    else:
        _COUNTER.value += 1                  # the launcher runs two kernels: partial results, then the reduction
    _ok(_fn("attention_mma", "rg_decode_attention_sink")(
        _ptr(q), c_int(q_stride), _ptr(out), _ptr(kv_cache), _ptr(block_table), c_int(block_table.shape[1]),
        _ptr(rows), c_int(n_tokens), _ptr(req_of_token), _ptr(positions), _ptr(part_o), _ptr(part_ml),
        _ptr(counters), c_int(nh), c_int(nkv), c_int(d), c_int(page_size), c_int(window or 0),
        c_int(keep_first if window else 0), c_float(scale), c_int(num_splits), _ptr(sink), _ptr(gate), c_int(gate_ld),
        _stream()), "decode_attention")


_tc_err: dict = {}
TC_GEMM_MIN_ROWS = 1024        # from here the fused tcgen05 gate|up product beats cuBLAS + SiLU-mul (measured)


def tc_gemm_ok(x: torch.Tensor, weight: torch.Tensor) -> bool:
    """Can the tcgen05 product take these operands?"""
    return (x.is_cuda and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.dim() == 2
            and x.shape[1] % 8 == 0 and x.stride(1) == 1 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0
            and weight.is_contiguous() and weight.data_ptr() % 16 == 0)


TC_TILES = {"128x128": 0, "128x256": 1, "256x256": 2, "256x128": 3}


def tc_gemm(x: torch.Tensor, weight: torch.Tensor, out_dtype=None, silu_mul: bool = False, wide: bool = True,
            check: bool = False, tile: str | None = None) -> torch.Tensor:
    """y = x W^T on the tcgen05 tensor cores (TMA-fed, accumulators in tensor
    memory).  ``silu_mul``: W is interleaved gate|up storage and y = silu(gate)
    * up.  ``tile`` (rows of x by rows of W): "128x128" or "128x256", one CTA
    per tile, or "256x256" / "256x128", a pair of CTAs on two SMs per tile
    (cta_group::2); without it ``wide`` picks between the first two.  The
    kernel's waits are bounded; ``tc_gemm_check()`` (or ``check=True``, which
    synchronises) raises if one gave up."""
    if tile is None:
        tile = "128x256" if wide else "128x128"
    if tile not in TC_TILES:
        raise KernelError(f"tc_gemm: tile {tile!r} is not one of {sorted(TC_TILES)}")
    if not tc_gemm_ok(x, weight):
        raise KernelError(f"tc_gemm refuses x {tuple(x.shape)} {x.dtype} stride {x.stride()}, "
                          f"W {tuple(weight.shape)} {weight.dtype}: bfloat16, K a multiple of 8, 16-byte aligned")
    M, K = x.shape
    N = weight.shape[0]
    if weight.shape[1] != K:
        raise KernelError(f"tc_gemm: x has {K} columns, W has {weight.shape[1]}")
    out_dtype = out_dtype or torch.bfloat16
    if silu_mul and (N % 16 or out_dtype != torch.bfloat16):
        raise KernelError("tc_gemm: the SiLU-mul epilogue needs N % 16 == 0 and bfloat16 output")
    err = _tc_err.get(x.device)
    if err is None:
        err = _tc_err[x.device] = torch.zeros(1, dtype=torch.int32, device=x.device)
    global _tc_unchecked
    _tc_unchecked = True
    out = torch.empty((M, N // 2 if silu_mul else N), dtype=out_dtype, device=x.device)
    _ok(_fn("gemm_tcgen05", "rg_tc_gemm")(
        _ptr(x), c_int(x.stride(0)), _ptr(weight), _ptr(out), c_int(out.shape[1]), c_int(_dtype_code(out)),
        c_int(1 if silu_mul else 0), c_int(M), c_int(N), c_int(K), c_int(TC_TILES[tile]), _ptr(err), _stream()),
        "tc_gemm")
    if check:
        tc_gemm_check(x.device)
    return out


TC_STREAM_MAX_ROWS = 64
# From 17 rows up to here a decode batch's layer products go through the streaming tcgen05 product with the
# neighbouring operations in its epilogues (residual addition, RMSNorm, rotation and cache write, SiLU-mul).  Alone
# the product is level with the library's; the step gains what the separate small kernels cost (measured at
# 1,024-token contexts: 10 % at batch 24, 6 % at 48, 3 % at 64).  RAILGUN_B200_TC_STREAM_ROWS overrides (16: off).
TC_STREAM_AUTO_ROWS = int(os.environ.get("RAILGUN_B200_TC_STREAM_ROWS", "64"))


def tc_stream_ok(x: torch.Tensor, weight: torch.Tensor) -> bool:
    """Can the weight-streaming tcgen05 product (up to 64 rows of x) take these operands?"""
    return 0 < x.shape[0] <= TC_STREAM_MAX_ROWS and tc_gemm_ok(x, weight)


def tc_stream_gemm(x, weight: torch.Tensor, out_dtype=None, silu_mul: bool = False, splits: int = 0,
                   check: bool = False) -> torch.Tensor:
    """y = x W^T for up to 64 rows of x on the tcgen05 tensor cores with the operands swapped: 128 rows of W per
    tile stream through once, the rows of x are the narrow side.  ``silu_mul``: W is interleaved gate|up storage
    and y = silu(gate) * up.  ``splits``: 1, 2, 4 or 8 CTAs of a cluster share a tile's K and add their partial
    sums in rank order (0: as many as keep the product in one wave).  A row's result does not depend on the other
    rows.  ``x`` may be a ``NormedRows`` (an RMSNorm not finished yet): the product runs over its scaled rows and
    multiplies the 32-bit sums by 1 / rms.  The kernel's waits are bounded; ``tc_gemm_check()`` (or ``check=True``)
    raises if one gave up."""
    rows = x if isinstance(x, NormedRows) else None
    if rows is not None:
        x = rows.scaled
    if not tc_stream_ok(x, weight):
        raise KernelError(f"tc_stream_gemm refuses x {tuple(x.shape)} {x.dtype} stride {x.stride()}, "
                          f"W {tuple(weight.shape)} {weight.dtype}: bfloat16, at most 64 rows, K a multiple of 8")
    M, K = x.shape
    N = weight.shape[0]
    if weight.shape[1] != K:
        raise KernelError(f"tc_stream_gemm: x has {K} columns, W has {weight.shape[1]}")
    out_dtype = out_dtype or torch.bfloat16
    if silu_mul and (N % 16 or out_dtype != torch.bfloat16):
        raise KernelError("tc_stream_gemm: the SiLU-mul epilogue needs N % 16 == 0 and bfloat16 output")
    if splits not in (0, 1, 2, 4, 8) or (splits and -(-K // 64) < splits):
        raise KernelError(f"tc_stream_gemm: {splits} splits of K = {K}")
    err = _tc_err.get(x.device)
    if err is None:
        err = _tc_err[x.device] = torch.zeros(1, dtype=torch.int32, device=x.device)
    global _tc_unchecked
    _tc_unchecked = True
    out = torch.empty((M, N // 2 if silu_mul else N), dtype=out_dtype, device=x.device)
    _ok(_fn("gemm_stream_tcgen05", "rg_tc_stream_gemm")(
        _ptr(x), c_int(x.stride(0)), _ptr(weight), _ptr(out), c_int(out.shape[1]), c_int(_dtype_code(out)),
        c_int(1 if silu_mul else 0), c_int(M), c_int(N), c_int(K), c_int(splits),
        _ptr(rows.partials if rows is not None else None), c_int(rows.blocks if rows is not None else 0),
        c_int(rows.partials.stride(0) if rows is not None else 0), c_float(rows.eps if rows is not None else 0.0),
        _ptr(err), _stream()), "tc_stream_gemm")
    if check:
        tc_gemm_check(x.device)
    return out


def tc_stream_rope_ok(x, weight: torch.Tensor, d: int) -> bool:
    """Can the q|k|v projection of these rows (17 to 64 of them) rotate and write the cache in the streaming
    tcgen05 product's own kernel?"""
    if d % 16:
        return False
    if isinstance(x, NormedRows):
        return tc_stream_scaled_ok(x, weight)
    return SKINNY_AUTO_ROWS < x.shape[0] <= TC_STREAM_AUTO_ROWS and tc_stream_ok(x, weight)


def tc_stream_gemm_rope_cache(x, weight: torch.Tensor, table: torch.Tensor, positions: torch.Tensor, slots, kv_cache,
                              nh: int, nkv: int, d: int, err_flag=None, splits: int = 0) -> torch.Tensor:
    """``skinny_gemm_rope_cache`` for up to 64 rows: the q|k|v projection with the rotary encoding and the cache
    write in the product's epilogue.  Returns [M, (nh+2nkv)d] whose q heads are rotated (its k and v columns are
    not written); k (rotated) and v go to ``kv_cache`` at ``slots`` (None: no write).  ``x``: bfloat16 rows or a
    ``NormedRows``; ``weight``'s q and k rows are in ``rope_pair_order``."""
    rows = x if isinstance(x, NormedRows) else None
    xin = rows.scaled if rows is not None else x
    if d % 16 or not tc_stream_ok(xin, weight):
        raise KernelError(f"tc_stream_gemm_rope_cache refuses rows {tuple(xin.shape)}, W {tuple(weight.shape)}, head size {d}")
    M, K = xin.shape
    N = weight.shape[0]
    if weight.shape[1] != K or N != (nh + 2 * nkv) * d:
        raise KernelError(f"tc_stream_gemm_rope_cache: W {tuple(weight.shape)} is not [({nh} + 2 x {nkv}) x {d}, {K}]")
    _check(table, "rope table", torch.float32)
    _check(positions, "positions", torch.int32)
    if table.shape[1] != d or positions.numel() < M:
        raise KernelError("tc_stream_gemm_rope_cache: the table's head size or the number of positions does not match")
    page_size = 0
    if slots is not None:
        _check(slots, "slots", torch.int32)
        _check(kv_cache, "kv_cache", torch.bfloat16)
        page_size = kv_cache.shape[3]
        if tuple(kv_cache.shape[1:]) != (2, nkv, page_size, d) or slots.numel() < M:
            raise KernelError(f"kv cache shape {tuple(kv_cache.shape)} does not match [pages, 2, {nkv}, page, {d}]")
    err = _tc_err.get(xin.device)
    if err is None:
        err = _tc_err[xin.device] = torch.zeros(1, dtype=torch.int32, device=xin.device)
    global _tc_unchecked
    _tc_unchecked = True
    out = torch.empty((M, N), dtype=torch.bfloat16, device=xin.device)
    _ok(_fn("gemm_stream_tcgen05", "rg_tc_stream_gemm_rope_cache")(
        _ptr(xin), c_int(xin.stride(0)), _ptr(weight), _ptr(out), c_int(N), c_int(M), c_int(N), c_int(K), c_int(splits),
        _ptr(rows.partials if rows is not None else None), c_int(rows.blocks if rows is not None else 0),
        c_int(rows.partials.stride(0) if rows is not None else 0), c_float(rows.eps if rows is not None else 0.0),
        _ptr(table), _ptr(positions), _ptr(slots), _ptr(kv_cache if slots is not None else None), c_int(nh), c_int(nkv),
        c_int(d), c_int(page_size), c_int(table.shape[0]), _ptr(err_flag), _ptr(err), _stream()),
        "tc_stream_gemm_rope_cache")
    return out


def tc_stream_fused_ok(x: torch.Tensor, weight: torch.Tensor, resid: torch.Tensor) -> bool:
    """Can x W^T be added to ``resid`` inside the streaming tcgen05 product (which then also prepares the next
    norm)?  Decode batches above the skinny product's and up to ``TC_STREAM_AUTO_ROWS`` rows."""
    return (SKINNY_AUTO_ROWS < x.shape[0] <= TC_STREAM_AUTO_ROWS and tc_stream_ok(x, weight)
            and resid.dtype == torch.float32 and resid.is_contiguous() and resid.shape == (x.shape[0], weight.shape[0])
            and resid.shape[1] % 8 == 0)


def tc_stream_gemm_residual(x: torch.Tensor, weight: torch.Tensor, resid: torch.Tensor, norm_weight: torch.Tensor,
                            eps: float, splits: int = 0) -> NormedRows:
    """resid += x W^T (32-bit, in place), and the RMSNorm (``norm_weight``, ``eps``) of the new rows but for the
    factor 1 / rms, which the product that reads the result applies (``skinny_gemm_residual`` for 17 to 64 rows)."""
    if not tc_stream_ok(x, weight):
        raise KernelError(f"tc_stream_gemm_residual refuses x {tuple(x.shape)} {x.dtype}, W {tuple(weight.shape)}")
    _check(resid, "resid", torch.float32)
    _check(norm_weight, "norm_weight", torch.float32)
    M, K = x.shape
    N = weight.shape[0]
    if weight.shape[1] != K or resid.shape != (M, N) or norm_weight.numel() != N:
        raise KernelError(f"tc_stream_gemm_residual: x {tuple(x.shape)}, W {tuple(weight.shape)}, residual "
                          f"{tuple(resid.shape)}, norm weight {norm_weight.numel()}")
    partials = torch.empty((-(-N // 128), TC_STREAM_MAX_ROWS), dtype=torch.float32, device=x.device)
    scaled = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    err = _tc_err.get(x.device)
    if err is None:
        err = _tc_err[x.device] = torch.zeros(1, dtype=torch.int32, device=x.device)
    global _tc_unchecked
    _tc_unchecked = True
    tiles = c_int(0)
    _ok(_fn("gemm_stream_tcgen05", "rg_tc_stream_gemm_residual")(
        _ptr(x), c_int(x.stride(0)), _ptr(weight), _ptr(resid), c_int(resid.stride(0)), _ptr(norm_weight), _ptr(scaled),
        _ptr(partials), c_int(partials.stride(0)), c_int(M), c_int(N), c_int(K), c_int(splits), ctypes.byref(tiles),
        _ptr(err), _stream()), "tc_stream_gemm_residual")
    return NormedRows(resid, scaled, partials, tiles.value, norm_weight, eps, torch.bfloat16)


def tc_stream_scaled_ok(rows: NormedRows, weight: torch.Tensor) -> bool:
    return (rows.dtype == torch.bfloat16 and SKINNY_AUTO_ROWS < rows.shape[0] <= TC_STREAM_AUTO_ROWS
            and tc_stream_ok(rows.scaled, weight) and rows.shape[1] == weight.shape[1])


_tc_unchecked = False


def mark_tc_unchecked() -> None:
    """A replayed graph may have run tcgen05 kernels: the next ``tc_gemm_check`` looks at their error flag."""
    global _tc_unchecked
    _tc_unchecked = True


def prefill_attention_tc_ok(q, kv_cache, d: int, page_size: int) -> bool:
    """Can the tcgen05 flash kernel take this?  bfloat16, head size 64, pages of 8, 16, 32, 64 or 128 tokens."""
    return (q.is_cuda and q.dtype == torch.bfloat16 and d == 64 and page_size in (8, 16, 32, 64, 128)
            and q.dim() == 2 and q.stride(1) == 1 and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0
            and kv_cache.is_contiguous())


def prefill_attention_tc(q, out, kv_cache, block_table, tiles, positions, nh: int, nkv: int, d: int,
                         window: int, scale: float) -> None:
    """Flash attention on the tcgen05 tensor cores for requests that bring
    several tokens: ``q`` is the fused qkv buffer [T, (nh + 2 nkv) d], ``tiles``
    [n, 3] = (first row, rows <= 128, request index).  Writes the tiles' rows
    of ``out`` [T, nh*d].  Its waits are bounded; ``tc_gemm_check()`` raises if
    one gave up."""
    page_size = kv_cache.shape[3]
    if not prefill_attention_tc_ok(q, kv_cache, d, page_size):
        raise KernelError("prefill_attention_tc: bfloat16, head size 64, page size 8..128 dividing 128")
    _check(kv_cache, "kv_cache", q.dtype)
    _check(block_table, "block_table", torch.int32)
    _check(tiles, "tiles", torch.int32)
    _check(positions, "positions", torch.int32)
    _check(out, "out", q.dtype)
    if tuple(kv_cache.shape[1:]) != (2, nkv, page_size, d):
        raise KernelError(f"kv cache shape {tuple(kv_cache.shape)} does not match heads {nkv} x {d}")
    err = _tc_err.get(q.device)
    if err is None:
        err = _tc_err[q.device] = torch.zeros(1, dtype=torch.int32, device=q.device)
    global _tc_unchecked
    _tc_unchecked = True
    _ok(_fn("attention_tcgen05", "rg_prefill_attention_tc")(
        _ptr(q), c_int(q.stride(0)), c_int(q.shape[0]), _ptr(out), _ptr(kv_cache), c_int(kv_cache.shape[0]),
        _ptr(block_table), c_int(block_table.shape[1]), _ptr(tiles), c_int(tiles.shape[0]), _ptr(positions),
        c_int(nh), c_int(nkv), c_int(d), c_int(page_size), c_int(window or 0), c_float(scale), _ptr(err),
        _stream()), "prefill_attention_tc")


def probe_sm100(device="cuda:0") -> dict:
    """Cycle counts of the building blocks of the tcgen05 kernels on this GPU
    (csrc/kernels/probe_sm100.cu): a diagnostic, on no product path."""
    from ctypes import c_double
    names = ["ex2.approx.ftz.f32", "cvt.rn.bf16x2.f32", "fma.rn.f32x2", "fma.rn.f32", "max.f32",
             "tcgen05.mma M128 N64 K16", "tcgen05.mma M128 N128 K16", "tcgen05.mma M128 N256 K16",
             "four N64 MMAs + two commits", "mbarrier wait (done), every lane", "mbarrier wait (done), lane 0 + shuffle",
             "fence.proxy.async", "mbarrier.arrive", "tcgen05.st x8 + wait::st",
             "softmax pass of 64 columns, 2 warps per scheduler", "softmax pass of 64 columns, 1 warp per scheduler"]
    dev = torch.device(device)
    scratch = torch.randn(148 * 512 * 64, device=dev)
    cyc = torch.zeros(16, dtype=torch.int64, device=dev)
    err = torch.zeros(1, dtype=torch.int32, device=dev)
    out = (c_double * len(names))()
    with torch.cuda.device(dev):
        _ok(_fn("probe_sm100", "rg_probe_sm100")(out, _ptr(scratch), _ptr(cyc), _ptr(err), _stream()), "probe_sm100")
    if int(err.item()) != 0 or any(v < 0 for v in out):
        raise KernelError(f"probe_sm100: a bounded wait gave up (code {int(err.item())})")
    return {n: round(float(v), 1) for n, v in zip(names, out)}


def tc_gemm_check(device=None) -> None:
    """Raise if a wait inside a tcgen05 product gave up since the last check
    (synchronises; free when no such product ran since)."""
    global _tc_unchecked
    if not _tc_unchecked:
        return
    _tc_unchecked = False
    for dev, err in _tc_err.items():
        if device is not None and dev != device:
            continue
        code = int(err.item())
        if code:
            err.zero_()
            who = {1: "the TMA producer", 2: "the MMA issuer", 3: "the epilogue", 4: "the MMA issuer"}.get(
                code, f"role {code} of the attention kernel")
            raise KernelError(f"a tcgen05 kernel: {who} gave up waiting on a barrier; the result is invalid")


def argmax(logits: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """Index of the largest logit of every row, ties to the lowest index
    (into ``out``, int32 [rows], if given)."""
    _check(logits, "logits", torch.float32)
    rows, V = logits.shape
    if out is None:
        out = torch.empty((rows,), dtype=torch.int32, device=logits.device)
    else:
        _check(out, "out", torch.int32)
        if out.shape != (rows,):
            raise KernelError(f"argmax: out has shape {tuple(out.shape)}, the logits have {rows} rows")
    pieces = min(64, -(-V // 2048))            # wide rows are cut into pieces so that many blocks share a row
    pv = pi = None
    if pieces > 1:
        pv = torch.empty((rows, pieces), dtype=torch.float32, device=logits.device)
        pi = torch.empty((rows, pieces), dtype=torch.int32, device=logits.device)
        _COUNTER.value += 1
    _ok(_fn("sampling", "rg_argmax")(_ptr(logits), c_int(rows), c_int(V), _ptr(out), _ptr(pv), _ptr(pi),
                                     c_int(pieces), _stream()), "argmax")
    return out


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k, top_p, seed: torch.Tensor,
           counter: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """One token per row; rows with temperature <= 0 are greedy.  ``seed`` and
    ``counter`` are int64 tensors read as unsigned 64-bit."""
    _check(logits, "logits", torch.float32)
    rows, V = logits.shape
    _check(temperature, "temperature", torch.float32)
    _check(seed, "seed", torch.int64)
    _check(counter, "counter", torch.int64)
    if top_k is not None:
        _check(top_k, "top_k", torch.int32)
    if top_p is not None:
        _check(top_p, "top_p", torch.float32)
    for name, t in (("temperature", temperature), ("seed", seed), ("counter", counter),
                    ("top_k", top_k), ("top_p", top_p)):
        if t is not None and t.numel() != rows:
            raise KernelError(f"{name} has {t.numel()} entries for {rows} rows")
    if out is None:
        out = torch.empty((rows,), dtype=torch.int32, device=logits.device)
    else:
        _check(out, "out", torch.int32)
        if out.shape != (rows,):
            raise KernelError(f"sample: out has shape {tuple(out.shape)}, the logits have {rows} rows")
    _ok(_fn("sampling", "rg_sample")(_ptr(logits), c_int(rows), c_int(V), _ptr(temperature), _ptr(top_k),
                                     _ptr(top_p), _ptr(seed), _ptr(counter), _ptr(out), _stream()), "sample")
    return out


def linear(x: torch.Tensor, weight: torch.Tensor, out_dtype=None, bias: torch.Tensor | None = None) -> torch.Tensor:
    """y = x W^T (+ ``bias``, added inside the library product), W stored [out, in].  Up to 64 bfloat16 rows go through the
    weight-streaming kernel of this package; everything else through the
    library matrix product (cuBLAS), as in the reference, whose projections
    are library GEMMs (crates/vllm-models/src/llama/attention.rs:94-96,133).
    32-bit inputs run in true 32-bit: the reduced-precision matrix mode is
    refused."""
    if isinstance(x, NormedRows):
        if (out_dtype is None or out_dtype == torch.bfloat16) and skinny_scaled_ok(x, weight):
            return skinny_gemm_scaled(x, weight)              # the norm is finished inside the product
        if tc_stream_scaled_ok(x, weight):
            return tc_stream_gemm(x, weight, out_dtype)      # likewise, for 17 to 64 rows
        x = x.materialize()
    if not x.is_cuda:
        raise KernelError("linear: CUDA tensors only (there is no CPU path)")
    if x.dtype == torch.float32 and torch.backends.cuda.matmul.allow_tf32:
        raise KernelError("linear: TF32 is enabled; the 32-bit path must be true 32-bit")
    if bias is not None:
        if out_dtype is not None and out_dtype != x.dtype:
            raise KernelError("linear: a product with a bias comes out in its input's type")
        return torch.addmm(bias, x, weight.t())
    if x.shape[0] <= SKINNY_AUTO_ROWS and skinny_gemm_ok(x, weight):
        return skinny_gemm(x, weight, out_dtype)             # small decode batches: stream the weights once
    if out_dtype is not None and out_dtype != x.dtype:
        return torch.mm(x, weight.t(), out_dtype=out_dtype)
    return torch.mm(x, weight.t())

